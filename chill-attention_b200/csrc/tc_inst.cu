// Instantiates the tensor-core kernels for ONE mask functor: compile with
//   -DCHILL_INST_MASK=<functor struct>   (e.g. CausalMask)
#include "bwd_fused.cuh"
#include "bwd_tc.cuh"
#include "bwd_tf32.cuh"
#include "bwd_wide.cuh"
#include "fwd_tc.cuh"
#include "fwd_tf32.cuh"
#include "tc_launch.h"

#ifndef CHILL_INST_MASK
#error "define CHILL_INST_MASK"
#endif

namespace chill {

using InstMask = CHILL_INST_MASK;

template <typename T, int D>
static int launch_fwd_one(const CUtensorMap* maps, const tc::FwdTcParams& p, dim3 grid, cudaStream_t st) {
  auto kern = tc::fwd_tc_kernel<T, D, InstMask>;
  using SH = tc::FwdShape<D>;
  constexpr int smem = tc::FwdSmem<D, SH::kStages, SH::kKeys>::kDynamic;
  static_assert(SH::kCtasPerSm * smem <= 232448, "the CTAs that are to share an SM must fit its shared memory");
  struct Tag {};
  cudaError_t e = ensure_dynamic_smem<Tag>(kern, smem, /*prefer_max_carveout=*/true);
  if (e != cudaSuccess) return (int)e;
  kern<<<grid, tc::kFwdThreads, smem, st>>>(maps[0], maps[1], maps[2], maps[3], p);
  return (int)cudaGetLastError();
}

template <>
int tc_launch_fwd<InstMask>(int dtype, int D, const CUtensorMap* maps, const tc::FwdTcParams& p, dim3 grid,
                            cudaStream_t st) {
  if (dtype == 2) {
    if (D == 128) return launch_fwd_one<__nv_bfloat16, 128>(maps, p, grid, st);
    if (D == 64) return launch_fwd_one<__nv_bfloat16, 64>(maps, p, grid, st);
    if (D == 256) return launch_fwd_one<__nv_bfloat16, 256>(maps, p, grid, st);
  } else if (dtype == 1) {
    if (D == 128) return launch_fwd_one<__half, 128>(maps, p, grid, st);
    if (D == 64) return launch_fwd_one<__half, 64>(maps, p, grid, st);
    if (D == 256) return launch_fwd_one<__half, 256>(maps, p, grid, st);
  }
  return (int)cudaErrorInvalidValue;
}

template <int D>
static int launch_fwd_tf32_one(const CUtensorMap* maps, const tc::FwdTcParams& p, dim3 grid, cudaStream_t st) {
  auto kern = tc::fwd_tf32_kernel<D, InstMask>;
  constexpr int smem = tc::FwdTf32Smem<D>::kDynamic;
  static_assert(smem <= 232448, "exceeds the 227 KB of shared memory a CTA can opt in to");
  struct Tag {};
  cudaError_t e = ensure_dynamic_smem<Tag>(kern, smem, /*prefer_max_carveout=*/true);
  if (e != cudaSuccess) return (int)e;
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
int tc_launch_bwd_tf32<InstMask>(int D, const CUtensorMap* maps, const tc::BwdTcParams& p, cudaStream_t st) {
  return tc::launch_bwd_tf32<InstMask>(D, maps, p, st);
}

template <>
int tc_launch_bwd<InstMask>(int dtype, int D, const CUtensorMap* maps, const tc::BwdTcParams& p, cudaStream_t st) {
  if (p.dq_accum != nullptr) return tc::launch_bwd_fused_all<InstMask>(dtype, D, maps, p, st);
  return tc::launch_bwd_all<InstMask>(dtype, D, maps, p, st);
}

template <>
int tc_launch_bwd_wide<InstMask>(int dtype, const CUtensorMap* maps, const tc::BwdTcParams& p, cudaStream_t st) {
  return tc::launch_bwd_wide_all<InstMask>(dtype, maps, p, st);
}

}  // namespace chill
