// Microbenchmark behind a design decision, not part of the product or the tests.
//
// What a system-scope fence, a device-scope fence, a release store and an
// acquire-release atomic cost at the end of (or inside) a store-heavy kernel,
// with local and with peer destinations. Run with an argument to include the
// peer (2-GPU) part.
//   nvcc -O3 -gencode arch=compute_100a,code=sm_100a -o fence tests/microbench/fence_cost.cu && ./fence peer
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdint>
#include <vector>
#define CK(x) do{cudaError_t e=(x); if(e!=cudaSuccess){printf("ERR %s line %d\n", cudaGetErrorString(e), __LINE__); return 1;}}while(0)
// mode: 0 none, 1 fence.gpu by t0, 2 fence.sys by t0, 3 st.release.sys by t0, 4 two fence.sys, 5 atom.acq_rel.sys per warp, 6 fence.sys per warp lane0
template<int MODE>
__global__ void k(char* dst, int* ctr, uint64_t* flag, int rows_per_cta, int row_bytes) {
  const int tid = threadIdx.x;
  for (int r = 0; r < rows_per_cta; ++r) {
    char* d = dst + ((size_t)(blockIdx.x * rows_per_cta + r)) * row_bytes + tid * 32;
    uint4 v = make_uint4(tid, r, 1, 2);
    if (tid * 32 < row_bytes) { *(uint4*)d = v; *(uint4*)(d+16) = v; }
    if (MODE == 5) { __syncwarp(); if ((tid&31)==0) { int old; asm volatile("atom.add.acq_rel.sys.global.s32 %0, [%1], 1;" : "=r"(old) : "l"(ctr + (blockIdx.x&255)) : "memory"); } }
    if (MODE == 6) { __syncwarp(); if ((tid&31)==0) { __threadfence_system(); atomicAdd(ctr + (blockIdx.x&255), 1);} }
  }
  __syncthreads();
  if (tid == 0) {
    if (MODE == 1) __threadfence();
    if (MODE == 2) __threadfence_system();
    if (MODE == 4) { __threadfence_system(); atomicAdd(ctr + (blockIdx.x&255), 1); __threadfence_system(); }
    if (MODE == 3) asm volatile("st.release.sys.global.u64 [%0], %1;" :: "l"(flag + blockIdx.x), "l"((uint64_t)7) : "memory");
    if (MODE == 1 || MODE == 2) atomicAdd(ctr + (blockIdx.x&255), 1);
  }
}
template<int MODE> float run(char* dst, int* ctr, uint64_t* flag, int grid, int threads, int rows, int row_bytes, char* flushbuf, size_t flushbytes) {
  cudaEvent_t a,b; cudaEventCreate(&a); cudaEventCreate(&b);
  float best = 1e9, sum=0; int n=10;
  for (int i=0;i<n+3;i++){ if (flushbuf) cudaMemsetAsync(flushbuf, i, flushbytes); cudaEventRecord(a); k<MODE><<<grid,threads>>>(dst,ctr,flag,rows,row_bytes); cudaEventRecord(b); cudaEventSynchronize(b); float ms; cudaEventElapsedTime(&ms,a,b); if(i>=3){ if(ms<best)best=ms; sum+=ms;} }
  return sum/n*1000.f;
}
int main(int argc, char** argv) {
  int ndev=0; cudaGetDeviceCount(&ndev);
  int peer = (argc>1 && ndev>1) ? 1 : 0;
  CK(cudaSetDevice(0));
  char* local; CK(cudaMalloc(&local, 1<<28));
  char* remote = nullptr;
  if (peer) { CK(cudaSetDevice(1)); CK(cudaMalloc(&remote, 1<<28)); CK(cudaSetDevice(0)); CK(cudaDeviceEnablePeerAccess(1,0)); }
  int* ctr; CK(cudaMalloc(&ctr, 4096)); CK(cudaMemset(ctr,0,4096));
  uint64_t* flag; CK(cudaMalloc(&flag, 1<<20));
  char* fl; size_t flb = 512u<<20; CK(cudaMalloc(&fl, flb));
  const int threads=448, row_bytes=14336;
  for (int pass=0; pass<(peer?2:1); ++pass) {
    char* dst = pass? remote: local;
    for (int cfg=0; cfg<3; ++cfg) {
      int grid = cfg==0? 128 : (cfg==1? 592 : 592); int rows = cfg==2? 8 : (cfg==1?2:1);
      for (int flush=0; flush<2; ++flush) {
        char* f = flush? fl: nullptr;
        printf("%s grid %d rows %d flush %d: none %.1f | fence.gpu %.1f | fence.sys %.1f | st.rel.sys %.1f | 2x fence.sys %.1f | atom.acq_rel.sys/warp %.1f | fence.sys/warp %.1f us\n", pass?"PEER ":"LOCAL", grid, rows, flush,
          run<0>(dst,ctr,flag,grid,threads,rows,row_bytes,f,flb), run<1>(dst,ctr,flag,grid,threads,rows,row_bytes,f,flb), run<2>(dst,ctr,flag,grid,threads,rows,row_bytes,f,flb),
          run<3>(dst,ctr,flag,grid,threads,rows,row_bytes,f,flb), run<4>(dst,ctr,flag,grid,threads,rows,row_bytes,f,flb), run<5>(dst,ctr,flag,grid,threads,rows,row_bytes,f,flb), run<6>(dst,ctr,flag,grid,threads,rows,row_bytes,f,flb));
      }
    }
  }
  return 0;
}
