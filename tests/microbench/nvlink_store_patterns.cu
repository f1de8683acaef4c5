// Microbenchmark behind a design decision, not part of the product or the tests.
//
// Pushes rows of 7168 / 14336 bytes from GPU 0 into GPU 1's memory over NVLink
// with (a) 32-byte stores per lane, (b) 16-byte stores per lane, (c) a
// shared-memory copy followed by one bulk (TMA) store per row, and pulls the
// same rows with 32-byte loads; prints time and GB/s next to a local copy and
// cudaMemcpyPeer. Needs two GPUs with peer access.
//   nvcc -O3 -gencode arch=compute_100a,code=sm_100a -o nvl tests/microbench/nvlink_store_patterns.cu && ./nvl
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdint>
#define CK(x) do{cudaError_t e=(x); if(e!=cudaSuccess){printf("ERR %s line %d\n", cudaGetErrorString(e), __LINE__); return 1;}}while(0)
struct alignas(32) V32 { uint32_t w[8]; };
__device__ __forceinline__ V32 ld32(const void* p){ V32 r; asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];" : "=r"(r.w[0]),"=r"(r.w[1]),"=r"(r.w[2]),"=r"(r.w[3]),"=r"(r.w[4]),"=r"(r.w[5]),"=r"(r.w[6]),"=r"(r.w[7]) : "l"(p)); return r; }
__device__ __forceinline__ void st32(void* p, const V32& r){ asm volatile("st.global.L1::no_allocate.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" :: "l"(p),"r"(r.w[0]),"r"(r.w[1]),"r"(r.w[2]),"r"(r.w[3]),"r"(r.w[4]),"r"(r.w[5]),"r"(r.w[6]),"r"(r.w[7]) : "memory"); }
__device__ __forceinline__ void st16(void* p, const uint4& r){ asm volatile("st.global.L1::no_allocate.v4.b32 [%0], {%1,%2,%3,%4};" :: "l"(p),"r"(r.x),"r"(r.y),"r"(r.z),"r"(r.w) : "memory"); }
// MODE 0: ld32 + st32 (32B/lane), 1: ld32 + 2x st16 lane-contiguous 16B (two 512B segments), 2: smem + bulk store, 3: ld from peer (pull) st local 32B
template<int MODE>
__global__ void __launch_bounds__(512) copyk(const char* src, char* dst, int rows, int row_bytes) {
  extern __shared__ __align__(128) char sm[];
  const int tid = threadIdx.x, nthr = blockDim.x;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const char* s = src + (size_t)r * row_bytes; char* d = dst + (size_t)r * row_bytes;
    if (MODE == 0 || MODE == 3) { for (int o = tid*32; o < row_bytes; o += nthr*32) st32(d+o, ld32(s+o)); }
    else if (MODE == 1) { for (int o = tid*32; o < row_bytes; o += nthr*32) { V32 v = ld32(s+o); int w = (o/1024)*1024; int l = (o%1024)/32; st16(d+w+l*16, make_uint4(v.w[0],v.w[1],v.w[2],v.w[3])); st16(d+w+512+l*16, make_uint4(v.w[4],v.w[5],v.w[6],v.w[7])); } }
    else if (MODE == 2) {
      for (int o = tid*32; o < row_bytes; o += nthr*32) *(V32*)(sm+o) = ld32(s+o);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncthreads();
      if (tid == 0) {
        uint32_t sa = (uint32_t)__cvta_generic_to_shared(sm);
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" :: "l"(d), "r"(sa), "r"(row_bytes) : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      }
      __syncthreads();
    }
  }
  if (MODE == 2 && tid == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}
template<int MODE> float run(const char* src, char* dst, int grid, int threads, int rows, int row_bytes) {
  cudaEvent_t a,b; cudaEventCreate(&a); cudaEventCreate(&b);
  float sum=0; int n=8;
  for (int i=0;i<n+2;i++){ cudaEventRecord(a); copyk<MODE><<<grid,threads,MODE==2?row_bytes:0>>>(src,dst,rows,row_bytes); cudaEventRecord(b); cudaEventSynchronize(b); float ms; cudaEventElapsedTime(&ms,a,b); if(i>=2) sum+=ms; }
  cudaError_t e = cudaGetLastError(); if (e != cudaSuccess) printf("kernel err %s\n", cudaGetErrorString(e));
  return sum/n*1000.f;
}
int main() {
  int ndev=0; cudaGetDeviceCount(&ndev); if (ndev<2) { printf("need 2 gpus\n"); return 0; }
  CK(cudaSetDevice(1)); char* remote; CK(cudaMalloc(&remote, 1u<<30)); CK(cudaMemset(remote,1,1u<<30));
  CK(cudaSetDevice(0)); CK(cudaDeviceEnablePeerAccess(1,0));
  char* local; CK(cudaMalloc(&local, 1u<<30)); CK(cudaMemset(local,2,1u<<30));
  char* local2; CK(cudaMalloc(&local2, 1u<<30));
  CK(cudaFuncSetAttribute(copyk<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64*1024));
  int rbs[2] = {7168, 14336};
  for (int ri=0; ri<2; ++ri) { int rb = rbs[ri]; int threads = rb/32 > 448 ? 448 : rb/32;
    int rowsv[3] = {1024, 8192, 32768};
    for (int rv=0; rv<3; ++rv) { int rows = rowsv[rv]; double mb = (double)rows*rb/1e6;
      int grids[3] = {148, 592, 1184};
      for (int gi=0; gi<3; ++gi) { int grid = grids[gi];
        float t0 = run<0>(local, remote, grid, threads, rows, rb);
        float t1 = run<1>(local, remote, grid, threads, rows, rb);
        float t2 = run<2>(local, remote, grid, threads, rows, rb);
        float t3 = run<3>(remote, local2, grid, threads, rows, rb);
        float tl = run<0>(local, local2, grid, threads, rows, rb);
        printf("row %5d B rows %5d (%.0f MB) grid %4d: push st32 %.1f us %.0f GB/s | push st16 %.1f us %.0f GB/s | push TMA %.1f us %.0f GB/s | pull ld32 %.1f us %.0f GB/s | local %.1f us %.0f GB/s\n",
          rb, rows, mb, grid, t0, mb/t0*1e3, t1, mb/t1*1e3, t2, mb/t2*1e3, t3, mb/t3*1e3, tl, mb/tl*1e3);
      } } }
  // cudaMemcpyPeer reference
  cudaEvent_t a,b; cudaEventCreate(&a); cudaEventCreate(&b);
  for (int i=0;i<3;i++){ cudaEventRecord(a); cudaMemcpyPeerAsync(remote,1,local,0,1u<<29); cudaEventRecord(b); cudaEventSynchronize(b); float ms; cudaEventElapsedTime(&ms,a,b); printf("memcpyPeer 512MB %.1f us %.0f GB/s\n", ms*1e3, (1u<<29)/1e6/ms); }
  return 0;
}
