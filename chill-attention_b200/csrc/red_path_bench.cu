// Microbenchmark: how fast can 148 CTAs (one per SM, 128 threads) add fp32 tiles into global memory?
// Compares red.global (scalar / v2 / v4), plain vector stores and bulk reductions of the copy engine
// (cp.reduce.async.bulk ... add.f32 from shared memory), for L2-resident and larger-than-L2 targets.
// Stand-alone program, not part of the library:
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o red_path_bench red_path_bench.cu && ./red_path_bench
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
#define CK(x) do{cudaError_t e=(x); if(e!=cudaSuccess){printf("err %s line %d\n", cudaGetErrorString(e), __LINE__); return 1;}}while(0)

__device__ __forceinline__ uint32_t smem_u32(const void* p){ return (uint32_t)__cvta_generic_to_shared(p);}  

// mode 0: red.v4.f32 ; 1: red.f32 x4 ; 2: st.v4 ; 3: red.v2.f32 x2
template <int MODE>
__global__ void __launch_bounds__(128) k_red(float* buf, size_t n_tiles, int iters, int stride_tiles) {
  // each CTA: per iteration reduces one 64 KB tile laid out [32 c4][128 rows][4]
  const int row = threadIdx.x;
  size_t tile = (size_t)blockIdx.x * stride_tiles;
  for (int it = 0; it < iters; ++it) {
    float* dst = buf + (tile % n_tiles) * 16384 + row * 4;
#pragma unroll 8
    for (int c4 = 0; c4 < 32; ++c4) {
      float* p = dst + c4 * 512;
      float a = 1.0f;
      if (MODE == 0) asm volatile("red.global.add.v4.f32 [%0], {%1,%1,%1,%1};" ::"l"(p), "f"(a) : "memory");
      else if (MODE == 1) { for (int e = 0; e < 4; ++e) asm volatile("red.global.add.f32 [%0], %1;" ::"l"(p + e), "f"(a) : "memory"); }
      else if (MODE == 2) *reinterpret_cast<float4*>(p) = make_float4(a, a, a, a);
      else { asm volatile("red.global.add.v2.f32 [%0], {%1,%1};" ::"l"(p), "f"(a) : "memory"); asm volatile("red.global.add.v2.f32 [%0], {%1,%1};" ::"l"(p + 2), "f"(a) : "memory"); }
    }
    tile += 1;
  }
}

// TMA bulk reduce from shared memory: chunk bytes per instruction
template <int CHUNK>
__global__ void __launch_bounds__(128) k_bulk(float* buf, size_t n_tiles, int iters, int stride_tiles) {
  extern __shared__ __align__(128) uint8_t sm[];
  for (int i = threadIdx.x; i < CHUNK / 4; i += 128) reinterpret_cast<float*>(sm)[i] = 1.0f;
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();
  size_t tile = (size_t)blockIdx.x * stride_tiles;
  if (threadIdx.x == 0) {
    for (int it = 0; it < iters; ++it) {
      float* dst = buf + (tile % n_tiles) * 16384;
      for (int c = 0; c < 65536 / CHUNK; ++c) {
        asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(dst + c * (CHUNK / 4)), "r"(smem_u32(sm)), "r"(CHUNK) : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 4;" ::: "memory");
      }
      tile += 1;
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }
}

int main() {
  const size_t n_tiles_big = 4096;  // 268 MB
  float* buf; CK(cudaMalloc(&buf, n_tiles_big * 65536));
  CK(cudaMemset(buf, 0, n_tiles_big * 65536));
  cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
  const int iters = 256; const int grid = 148;
  auto report = [&](const char* name, size_t nt, float ms) {
    double bytes = (double)grid * iters * 65536.0;
    printf("%-28s tiles=%5zu  %.3f ms  %.2f TB/s\n", name, nt, ms, bytes / ms / 1e9);
  };
  for (size_t nt : {(size_t)4096, (size_t)512, (size_t)148}) {
    for (int stride : {27, 1}) {
      printf("-- working set %zu MB, cta start stride %d tiles\n", nt * 65536 / 1000000, stride);
#define RUN(NAME, LAUNCH) { LAUNCH; CK(cudaDeviceSynchronize()); cudaEventRecord(e0); LAUNCH; cudaEventRecord(e1); CK(cudaDeviceSynchronize()); float ms; cudaEventElapsedTime(&ms, e0, e1); report(NAME, nt, ms); }
      RUN("red.v4.f32", (k_red<0><<<grid, 128>>>(buf, nt, iters, stride)));
      RUN("red.f32 x4", (k_red<1><<<grid, 128>>>(buf, nt, iters, stride)));
      RUN("red.v2.f32 x2", (k_red<3><<<grid, 128>>>(buf, nt, iters, stride)));
      RUN("st.v4 (plain store)", (k_red<2><<<grid, 128>>>(buf, nt, iters, stride)));
      RUN("bulk reduce 16 KB", (k_bulk<16384><<<grid, 128, 16384>>>(buf, nt, iters, stride)));
      RUN("bulk reduce 4 KB", (k_bulk<4096><<<grid, 128, 4096>>>(buf, nt, iters, stride)));
    }
  }
  // two CTAs per SM issuing reds
  {
    size_t nt = 4096; 
    cudaEventRecord(e0); k_red<0><<<296, 128>>>(buf, nt, iters, 13); cudaEventRecord(e1); CK(cudaDeviceSynchronize());
    float ms; cudaEventElapsedTime(&ms, e0, e1); printf("red.v4.f32 296 CTAs: %.3f ms %.2f TB/s\n", ms, 296.0 * iters * 65536 / ms / 1e9);
    cudaEventRecord(e0); k_red<0><<<148 * 8, 128>>>(buf, nt, iters / 4, 13); cudaEventRecord(e1); CK(cudaDeviceSynchronize());
    cudaEventElapsedTime(&ms, e0, e1); printf("red.v4.f32 1184 CTAs: %.3f ms %.2f TB/s\n", ms, 1184.0 * (iters / 4) * 65536 / ms / 1e9);
  }
  printf("done\n");
  return 0;
}
