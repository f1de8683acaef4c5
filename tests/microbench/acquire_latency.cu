// Microbenchmark behind a design decision, not part of the product or the tests.
//
// Dependent-load latency of acquire / relaxed / volatile loads, of a
// compare-and-swap, and of a load followed by a device- or system-scope fence
// (one warp, pointer chase in L2).
//   nvcc -O3 -gencode arch=compute_100a,code=sm_100a -o acq tests/microbench/acquire_latency.cu && ./acq
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdint>
__device__ __forceinline__ uint64_t ld_acq_sys(const uint64_t* p){uint64_t v; asm volatile("ld.acquire.sys.global.u64 %0, [%1];":"=l"(v):"l"(p):"memory"); return v;}
__device__ __forceinline__ uint64_t ld_acq_gpu(const uint64_t* p){uint64_t v; asm volatile("ld.acquire.gpu.global.u64 %0, [%1];":"=l"(v):"l"(p):"memory"); return v;}
__device__ __forceinline__ uint64_t ld_rlx_sys(const uint64_t* p){uint64_t v; asm volatile("ld.relaxed.sys.global.u64 %0, [%1];":"=l"(v):"l"(p):"memory"); return v;}
__device__ __forceinline__ uint64_t ld_vol(const uint64_t* p){uint64_t v; asm volatile("ld.volatile.global.u64 %0, [%1];":"=l"(v):"l"(p):"memory"); return v;}
__device__ __forceinline__ uint64_t ld_cg(const uint64_t* p){uint64_t v; asm volatile("ld.global.cg.u64 %0, [%1];":"=l"(v):"l"(p):"memory"); return v;}
template<int MODE> __global__ void k(uint64_t* buf, long long* out, int n) {
  // pointer chase: buf[i] holds index of next
  uint64_t idx = threadIdx.x == 0 ? 0 : 1;
  long long t0 = clock64();
  for (int i = 0; i < n; ++i) {
    const uint64_t* p = buf + idx * 32;
    if (MODE==0) idx = ld_acq_sys(p); else if (MODE==1) idx = ld_acq_gpu(p); else if (MODE==2) idx = ld_rlx_sys(p); else if (MODE==3) idx = ld_vol(p); else if (MODE==4) idx = ld_cg(p);
    else if (MODE==5) { idx = atomicCAS((unsigned long long*)p, 0xffffffffffffull, 1ull); }
    else if (MODE==6) { idx = ld_vol(p); __threadfence(); }
    else if (MODE==7) { idx = ld_vol(p); __threadfence_system(); }
  }
  long long t1 = clock64();
  if (threadIdx.x == 0) { out[0] = t1 - t0; out[1] = (long long)idx; }
}
int main() {
  const int N = 4096, n = 2000;
  uint64_t* h = new uint64_t[N*32]; for (int i=0;i<N;i++) h[i*32] = (uint64_t)((i*1237+1) % N);
  uint64_t* d; cudaMalloc(&d, N*32*8); cudaMemcpy(d, h, N*32*8, cudaMemcpyHostToDevice);
  long long* o; cudaMalloc(&o, 16); long long ho[2];
  int clk; cudaDeviceGetAttribute(&clk, cudaDevAttrClockRate, 0);
  const char* names[8] = {"ld.acquire.sys","ld.acquire.gpu","ld.relaxed.sys","ld.volatile","ld.cg","atomicCAS","ld.volatile+fence.gpu","ld.volatile+fence.sys"};
#define RUN(M) k<M><<<1,32>>>(d,o,n); k<M><<<1,32>>>(d,o,n); cudaDeviceSynchronize(); cudaMemcpy(ho,o,16,cudaMemcpyDeviceToHost); printf("%-26s %.0f cycles/op (~%.0f ns at max clock)\n", names[M], (double)ho[0]/n, (double)ho[0]/n/(clk/1e6));
  RUN(0) RUN(1) RUN(2) RUN(3) RUN(4) RUN(5) RUN(6) RUN(7)
  return 0;
}
