// Microbenchmark: cycles per tcgen05.mma for several shapes (one CTA per SM, one issuing thread).
// Stand-alone program, not part of the library:
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o mma_shape_bench mma_shape_bench.cu && ./mma_shape_bench
#include <cstdio>
#include <cuda_runtime.h>
#include "tc_common.cuh"
using namespace chill::tc;

template <int N, bool TS, bool BMN, int REPS>
__global__ void __launch_bounds__(128, 1) bench(unsigned long long* out, int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t sA = base, sB = base + 32768, bar = base + 32768 + 65536;
  volatile uint32_t* slot = reinterpret_cast<volatile uint32_t*>(gen + 32768 + 65536 + 16);
  volatile int* abortf = reinterpret_cast<volatile int*>(gen + 32768 + 65536 + 24);
  for (int i = threadIdx.x; i < (32768 + 65536) / 4; i += 128) reinterpret_cast<uint32_t*>(gen)[i] = 0x3c003c00u;
  if (threadIdx.x == 0) { *abortf = 0; mbar_init(bar, 1); fence_barrier_init(); fence_proxy_async_smem(); }
  if (threadIdx.x < 32) { tmem_alloc(smem_u32(const_cast<uint32_t*>(slot)), 512); tmem_relinquish(); }
  fence_proxy_async_smem();
  tc_fence_before(); __syncthreads(); tc_fence_after();
  const uint32_t tmem = *slot;
  Guard g{status, abortf};
  if (threadIdx.x == 0) {
    const uint32_t idesc = make_idesc<__half>(128, N, false, BMN);
    unsigned long long t0 = clock64();
    for (int r = 0; r < REPS; ++r) {
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const uint64_t bd = BMN ? smem_desc_sw128(sB + kk * 2048, 16384, 1024) : smem_desc_sw128(sB + kk * 32, 16, 1024);
        if (TS) mma_ts(tmem, tmem + 256 + kk * 8, bd, idesc, 1u);
        else mma_ss(tmem, smem_desc_sw128(sA + kk * 32, 16, 1024), bd, idesc, 1u);
      }
    }
    unsigned long long t1 = clock64();
    mma_commit(bar);
    mbar_wait(bar, 0, g, 900);
    unsigned long long t2 = clock64();
    if (blockIdx.x == 0) { out[0] = t1 - t0; out[1] = t2 - t0; }
  }
  tc_fence_before(); __syncthreads();
  if (threadIdx.x < 32) tmem_dealloc(tmem, 512);
}

template <int N, bool TS, bool BMN>
void run(const char* name, unsigned long long* d_out, int* d_status) {
  constexpr int REPS = 64;
  auto k = bench<N, TS, BMN, REPS>;
  const int smem = 32768 + 65536 + 64 + 1024;
  cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  for (int it = 0; it < 2; ++it) k<<<148, 128, smem>>>(d_out, d_status);
  cudaError_t e = cudaDeviceSynchronize();
  unsigned long long h[2]; int st;
  cudaMemcpy(h, d_out, sizeof(h), cudaMemcpyDeviceToHost); cudaMemcpy(&st, d_status, 4, cudaMemcpyDeviceToHost);
  printf("%-28s issue %7.1f clk/MMA  done %7.1f clk/MMA  (err %d status %d)  -> %.0f FLOP/clk/SM\n", name,
         (double)h[0] / (REPS * 4), (double)h[1] / (REPS * 4), (int)e, st, 2.0 * 128 * N * 16 / ((double)h[1] / (REPS * 4)));
}

int main() {
  unsigned long long* d_out; int* d_status;
  cudaMalloc(&d_out, 64); cudaMalloc(&d_status, 4); cudaMemset(d_status, 0, 4);
  run<64, false, false>("SS M128 N64  K-major B", d_out, d_status);
  run<128, false, false>("SS M128 N128 K-major B", d_out, d_status);
  run<256, false, false>("SS M128 N256 K-major B", d_out, d_status);
  run<128, false, true>("SS M128 N128 MN-major B", d_out, d_status);
  run<64, true, true>("TS M128 N64  MN-major B", d_out, d_status);
  run<128, true, true>("TS M128 N128 MN-major B", d_out, d_status);
  run<256, true, true>("TS M128 N256 MN-major B", d_out, d_status);
  run<128, true, false>("TS M128 N128 K-major B", d_out, d_status);
  return 0;
}
