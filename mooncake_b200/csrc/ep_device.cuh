// Device-side primitives for the EP kernels (sm_100a only).
//
// Counterparts in the reference: the memory-order helpers of
// mooncake-transfer-engine/include/transport/device/cuda/cuda_ops.cuh:14-139
// and the warp utilities of mooncake-ep/include/mooncake_ep_utils.cuh:141-209.
// Differences that matter here: 32-byte (256-bit) vector loads and stores,
// 64-bit flags that carry an epoch, and wall-clock (%globaltimer) timeouts.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mcep {

struct alignas(32) V32 {  // 32 bytes = 16 bf16 = 8 x b32
    uint32_t w[8];
};

__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ---- flags ------------------------------------------------------------------
__device__ __forceinline__ uint64_t ld_acquire_sys(const uint64_t* p) {
    uint64_t v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint64_t ld_acquire_gpu(const uint64_t* p) {
    uint64_t v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint64_t* p, uint64_t v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// Flag store without a fence of its own: used where the writer has already
// fenced everything the flag announces (or announces nothing but a count).
__device__ __forceinline__ void st_relaxed_sys(uint64_t* p, uint64_t v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ int ld_volatile_s32(const int* p) {
    int v;
    asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_volatile_s32(int* p, int v) {
    asm volatile("st.volatile.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// ---- 32-byte vector memory ops ----------------------------------------------
// Read-only inputs that no kernel writes while this one runs (x, expert outputs).
__device__ __forceinline__ V32 ld32_readonly(const void* p) {
    V32 r;
    asm volatile(
        "ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
        : "=r"(r.w[0]), "=r"(r.w[1]), "=r"(r.w[2]), "=r"(r.w[3]), "=r"(r.w[4]),
          "=r"(r.w[5]), "=r"(r.w[6]), "=r"(r.w[7])
        : "l"(p));
    return r;
}
// Staging memory that peers wrote before the flag this kernel acquired: coherent
// path, never through the read-only cache and never allocated in L1.
__device__ __forceinline__ V32 ld32_coherent(const void* p) {
    V32 r;
    asm volatile(
        "ld.global.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
        : "=r"(r.w[0]), "=r"(r.w[1]), "=r"(r.w[2]), "=r"(r.w[3]), "=r"(r.w[4]),
          "=r"(r.w[5]), "=r"(r.w[6]), "=r"(r.w[7])
        : "l"(p)
        : "memory");
    return r;
}
__device__ __forceinline__ void st32(void* p, const V32& r) {
    asm volatile(
        "st.global.L1::no_allocate.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p),
        "r"(r.w[0]), "r"(r.w[1]), "r"(r.w[2]), "r"(r.w[3]), "r"(r.w[4]), "r"(r.w[5]),
        "r"(r.w[6]), "r"(r.w[7])
        : "memory");
}
__device__ __forceinline__ uint4 ld16_coherent(const void* p) {
    uint4 r;
    asm volatile("ld.global.L1::no_allocate.v4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p)
                 : "memory");
    return r;
}
__device__ __forceinline__ void st16(void* p, const uint4& r) {
    asm volatile("st.global.L1::no_allocate.v4.b32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(r.x),
                 "r"(r.y), "r"(r.z), "r"(r.w)
                 : "memory");
}
__device__ __forceinline__ float ld_f32_coherent(const void* p) {
    float r;
    asm volatile("ld.global.L1::no_allocate.f32 %0, [%1];" : "=f"(r) : "l"(p) : "memory");
    return r;
}
__device__ __forceinline__ int ld_s32_coherent(const void* p) {
    int r;
    asm volatile("ld.global.L1::no_allocate.s32 %0, [%1];" : "=r"(r) : "l"(p) : "memory");
    return r;
}

// ---- programmatic dependent launch ---------------------------------------------
// No-ops unless the kernel was launched with the programmatic-serialisation
// attribute; then `pdl_wait` blocks until the previous kernel in the stream has
// completed and its writes are visible, and `pdl_launch_dependents` lets the
// next kernel's blocks start their prologue early.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---- bf16 / fp8 ------------------------------------------------------------------
__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// Two fp32 -> two e4m3 bytes, round-to-nearest-even, saturating to +-448:
// the conversion of mooncake-ep/include/mooncake_ep_device.h:98-100.
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi) {
    return (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3);
}

// 16 bf16 (one V32) -> 16 e4m3 bytes with a per-128-channel scale shared by the
// 8 lanes that hold one group. Arithmetic of
// mooncake-ep/src/mooncake_ep_kernel.cu:184,239-264:
//   amax = max(1e-4f, max|x|); scale = 448.0f / amax (IEEE division);
//   scale_inv = amax * (1.0f / 448.0f); q = e4m3(x * scale).
// All 32 lanes must call it (shuffles); lanes without data pass zeros.
__device__ __forceinline__ uint4 quantize16(const V32& v, float& scale_inv) {
    float f[16];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        f[2 * i] = bf16lo(v.w[i]);
        f[2 * i + 1] = bf16hi(v.w[i]);
    }
    float amax = 1e-4f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(f[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    const float scale = __fdiv_rn(448.0f, amax);
    scale_inv = __fmul_rn(amax, 1.0f / 448.0f);
    uint32_t q[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t a = cvt_e4m3x2(__fmul_rn(f[4 * i], scale), __fmul_rn(f[4 * i + 1], scale));
        uint32_t b = cvt_e4m3x2(__fmul_rn(f[4 * i + 2], scale), __fmul_rn(f[4 * i + 3], scale));
        q[i] = a | (b << 16);
    }
    return make_uint4(q[0], q[1], q[2], q[3]);
}

// 16 fp32 -> 16 bf16, round-to-nearest-even (`__float2bfloat16`,
// mooncake-ep/src/mooncake_ep_kernel.cu:750).
__device__ __forceinline__ V32 pack_bf16x16(const float (&a)[16]) {
    V32 r;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a[2 * i], a[2 * i + 1]);
        r.w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return r;
}

}  // namespace mcep
