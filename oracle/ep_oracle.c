/*
 * CPU oracle for the Mooncake EP dispatch/combine arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY. Nothing in the product path links or calls this
 * file; it exists so that the GPU kernels can be checked against a plain-C
 * restatement of what the reference kernels compute.
 *
 * Every function names the reference lines it restates (paths are relative to
 * the Mooncake source tree).
 *
 * Parity status: pinned. The FP8 bytes are checked against the reference's own
 * torch path (mooncake-wheel/mooncake/mooncake_ep_buffer.py:693-703) through
 * the committed golden vectors, and the scale formula against the kernel text
 * (mooncake-ep/src/mooncake_ep_kernel.cu:184,252).
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

static inline float bf16_to_f32(uint16_t h) {
    uint32_t u = ((uint32_t)h) << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* Round-to-nearest-even fp32 -> bf16, as `__float2bfloat16` does
 * (mooncake-ep/src/mooncake_ep_kernel.cu:750). NaN keeps a quiet payload. */
static inline uint16_t f32_to_bf16_rn(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}

/*
 * fp32 -> FP8 E4M3 (the "fn" flavour: no infinities, 0x7f/0xff are NaN,
 * largest finite 448), round-to-nearest-even, saturating to +-448.
 * This is what `__nv_cvt_float2_to_fp8x2(x, __NV_SATFINITE, __NV_E4M3)` does
 * per element (mooncake-ep/include/mooncake_ep_device.h:98-100).
 *
 * Format: 1 sign, 4 exponent (bias 7), 3 mantissa. Normal numbers
 * 2^(e-7) * (1 + m/8) for e in 1..15 (e=15,m=7 excluded: NaN); subnormals
 * m/8 * 2^-6.
 */
uint8_t ora_e4m3_from_f32(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
    uint32_t au = u & 0x7fffffffu;
    if (au > 0x7f800000u) return (uint8_t)(sign | 0x7fu); /* NaN */
    float a;
    memcpy(&a, &au, 4);
    if (a >= 448.0f) {
        /* satfinite: everything at or beyond the largest finite value clamps.
         * (Values in [448, 464) would round to 448 anyway.) */
        return (uint8_t)(sign | 0x7eu);
    }
    /* Quantum: spacing of representable values around `a`. */
    int e;
    (void)frexpf(a, &e); /* a = m * 2^e, m in [0.5, 1) -> unbiased exp e-1 */
    int ue = e - 1;
    if (a == 0.0f) return sign;
    if (ue < -6) ue = -6;                   /* subnormal range shares 2^-6 */
    float quantum = ldexpf(1.0f, ue - 3);   /* 3 mantissa bits */
    /* a / quantum is exact (power of two); rintf is RNE by default. */
    float q = rintf(a / quantum);
    int iq = (int)q;                        /* 0..16 */
    if (iq == 16) {                         /* carried into the next binade */
        ue += 1;
        iq = 8;
    }
    uint8_t bits;
    if (iq < 8) {
        /* only reachable in the subnormal binade (ue == -6) */
        bits = (uint8_t)iq;
    } else {
        bits = (uint8_t)(((ue + 7) << 3) | (iq - 8));
    }
    if (bits > 0x7eu) bits = 0x7eu;
    return (uint8_t)(sign | bits);
}

/*
 * Per-token, per-128-channel quantisation of `rows` bf16 rows of `hidden`
 * channels. Restates the dispatch send loop,
 * mooncake-ep/src/mooncake_ep_kernel.cu:239-264 with the constants of :184:
 *   amax      = max(1e-4f, max|x|)        (fp32 of the bf16 inputs)
 *   scale     = 448.0f / amax             (IEEE fp32 division)
 *   scale_inv = amax * (1.0f / 448.0f)    (fp32 multiply by the rounded
 *                                          reciprocal - NOT amax / 448)
 *   q         = e4m3_rn_satfinite(x * scale)
 * `q` is rows*hidden bytes, `scale_inv` is rows*(hidden/128) floats, row-major.
 */
void ora_fp8_quant_rows(const uint16_t* x, int64_t rows, int hidden,
                        uint8_t* q, float* scale_inv) {
    const float k_margin = 1e-4f, k_amax = 448.0f;
    const float k_amax_inv = 1.0f / 448.0f;
    const int groups = hidden / 128;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const uint16_t* xr = x + r * (int64_t)hidden;
        for (int g = 0; g < groups; ++g) {
            float amax = k_margin;
            for (int j = 0; j < 128; ++j) {
                float v = fabsf(bf16_to_f32(xr[g * 128 + j]));
                amax = fmaxf(amax, v);
            }
            volatile float scale = k_amax / amax;
            volatile float sinv = amax * k_amax_inv;
            scale_inv[r * groups + g] = sinv;
            for (int j = 0; j < 128; ++j) {
                volatile float p = bf16_to_f32(xr[g * 128 + j]) * scale;
                q[r * (int64_t)hidden + g * 128 + j] = ora_e4m3_from_f32(p);
            }
        }
    }
}

/*
 * Weighted top-k reduction of the combine receive side,
 * mooncake-ep/src/mooncake_ep_kernel.cu:715-752: for each token, for k in
 * ascending order, skipping entries whose row index is negative (masked
 * top-k entry `:728`, or an expert whose owner rank is inactive `:730-732`),
 *   acc = fma(float(row[c]), w[t][k], acc)      (`:742`, contracted by nvcc)
 * then one RNE rounding to bf16 (`:750`).
 *
 * `rows` is a flat [n_rows][hidden] bf16 array, `row_index` is [tokens][topk]
 * (negative = skip).
 */
void ora_combine_reduce(const uint16_t* rows, const int64_t* row_index,
                        const float* weights, int64_t tokens, int topk,
                        int hidden, uint16_t* out) {
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < tokens; ++t) {
        for (int c = 0; c < hidden; ++c) {
            float acc = 0.0f;
            for (int k = 0; k < topk; ++k) {
                int64_t ri = row_index[t * topk + k];
                if (ri < 0) continue;
                float v = bf16_to_f32(rows[ri * (int64_t)hidden + c]);
                acc = fmaf(v, weights[t * topk + k], acc);
            }
            out[t * (int64_t)hidden + c] = f32_to_bf16_rn(acc);
        }
    }
}

/* fp32 reference of the same reduction (double accumulation, rounded once to
 * fp32): the yardstick for the 1e-2 relative tolerance of the combine output. */
void ora_combine_reduce_f32(const uint16_t* rows, const int64_t* row_index,
                            const float* weights, int64_t tokens, int topk,
                            int hidden, float* out) {
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < tokens; ++t) {
        for (int c = 0; c < hidden; ++c) {
            double acc = 0.0;
            for (int k = 0; k < topk; ++k) {
                int64_t ri = row_index[t * topk + k];
                if (ri < 0) continue;
                acc += (double)bf16_to_f32(rows[ri * (int64_t)hidden + c]) *
                       (double)weights[t * topk + k];
            }
            out[t * (int64_t)hidden + c] = (float)acc;
        }
    }
}
