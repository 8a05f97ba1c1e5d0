// Instantiates the tensor-core kernels for ONE mask functor: compile with
//   -DCHILL_INST_MASK=<functor struct>   (e.g. CausalMask)
#include "bwd_fused.cuh"
#include "bwd_tc.cuh"
#include "fwd_tc.cuh"
#include "fwd_tf32.cuh"
#include "tc_launch.h"

#ifndef CHILL_INST_MASK
#error "define CHILL_INST_MASK"
#endif

namespace chill {

using InstMask = CHILL_INST_MASK;

template <typename T, int D, int NSTAGE>
static int launch_fwd_one(const CUtensorMap* maps, const tc::FwdTcParams& p, dim3 grid, cudaStream_t st) {
  auto kern = tc::fwd_tc_kernel<T, D, InstMask, NSTAGE>;
  constexpr int smem = tc::FwdSmem<D, NSTAGE>::kDynamic;
  static bool configured = false;  // attribute is per device; set it on every device we meet
  static int configured_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured || configured_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    configured = true;
    configured_dev = dev;
  }
  kern<<<grid, tc::kFwdThreads, smem, st>>>(maps[0], maps[1], maps[2], maps[3], p);
  return (int)cudaGetLastError();
}

}  // namespace chill

// Evaluated alternative (off by default, build with -DCHILL_FWD_PINGPONG=1): one CTA per pair of query tiles
// with a fixed MMA interleave (fwd_pp.cuh).  It passes the same parity suite; on B200 it measured level with
// the two-CTAs-per-SM kernel on causal / full masks (0.61 vs 0.57-0.60 ms on C2) and slower on short key
// ranges (chunkwise: 0.68 vs 0.53 ms), so the simpler kernel stays the default.
#ifndef CHILL_FWD_PINGPONG
#define CHILL_FWD_PINGPONG 0
#endif
#if CHILL_FWD_PINGPONG
#include "fwd_pp.cuh"
namespace chill {
template <typename T, int D>
static int launch_fwd_pp(const CUtensorMap* maps, const tc::FwdTcParams& p, cudaStream_t st) {
  auto kern = tc::fwd_pp_kernel<T, D, InstMask>;
  constexpr int smem = tc::PpSmem<D>::kDynamic;
  static int configured_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured_dev = dev;
  }
  const int n_qt = (p.g.Lq + tc::kTile - 1) / tc::kTile;
  dim3 grid((unsigned)(((n_qt + 1) / 2) * p.g.H * p.g.B), 1, 1);
  kern<<<grid, tc::kPpThreads, smem, st>>>(maps[0], maps[1], maps[2], maps[3], p);
  return (int)cudaGetLastError();
}

}  // namespace chill
#endif

namespace chill {
template <>
int tc_launch_fwd<InstMask>(int dtype, int D, const CUtensorMap* maps, const tc::FwdTcParams& p, dim3 grid,
                            cudaStream_t st) {
#if CHILL_FWD_PINGPONG
  if (dtype == 2) {
    if (D == 128) return launch_fwd_pp<__nv_bfloat16, 128>(maps, p, st);
    if (D == 64) return launch_fwd_pp<__nv_bfloat16, 64>(maps, p, st);
  } else if (dtype == 1) {
    if (D == 128) return launch_fwd_pp<__half, 128>(maps, p, st);
    if (D == 64) return launch_fwd_pp<__half, 64>(maps, p, st);
  }
#endif
  if (dtype == 2) {
    if (D == 128) return launch_fwd_one<__nv_bfloat16, 128, 1>(maps, p, grid, st);
    if (D == 64) return launch_fwd_one<__nv_bfloat16, 64, 2>(maps, p, grid, st);
  } else if (dtype == 1) {
    if (D == 128) return launch_fwd_one<__half, 128, 1>(maps, p, grid, st);
    if (D == 64) return launch_fwd_one<__half, 64, 2>(maps, p, grid, st);
  }
  return (int)cudaErrorInvalidValue;
}

template <int D>
static int launch_fwd_tf32_one(const CUtensorMap* maps, const tc::FwdTcParams& p, dim3 grid, cudaStream_t st) {
  auto kern = tc::fwd_tf32_kernel<D, InstMask>;
  constexpr int smem = tc::FwdTf32Smem<D>::kDynamic;
  static_assert(smem <= 232448, "exceeds the 227 KB of shared memory a CTA can opt in to");
  static int configured_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    configured_dev = dev;
  }
  kern<<<grid, tc::kFwdThreads, smem, st>>>(maps[0], maps[1], maps[2], maps[3], p);
  return (int)cudaGetLastError();
}

template <>
int tc_launch_fwd_tf32<InstMask>(int D, const CUtensorMap* maps, const tc::FwdTcParams& p, dim3 grid, cudaStream_t st) {
  if (D == 64) return launch_fwd_tf32_one<64>(maps, p, grid, st);
  if (D == 128) return launch_fwd_tf32_one<128>(maps, p, grid, st);
  return (int)cudaErrorInvalidValue;
}

template <>
int tc_launch_bwd<InstMask>(int dtype, int D, const CUtensorMap* maps, const tc::BwdTcParams& p, cudaStream_t st) {
  if (p.dq_accum != nullptr) return tc::launch_bwd_fused_all<InstMask>(dtype, D, maps, p, st);
  return tc::launch_bwd_all<InstMask>(dtype, D, maps, p, st);
}

}  // namespace chill
