// Instantiates the tensor-core kernels for ONE mask functor: compile with
//   -DCHILL_INST_MASK=<functor struct>   (e.g. CausalMask)
#include "bwd_tc.cuh"
#include "fwd_tc.cuh"
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

template <>
int tc_launch_fwd<InstMask>(int dtype, int D, const CUtensorMap* maps, const tc::FwdTcParams& p, dim3 grid,
                            cudaStream_t st) {
  if (dtype == 2) {
    if (D == 128) return launch_fwd_one<__nv_bfloat16, 128, 1>(maps, p, grid, st);
    if (D == 64) return launch_fwd_one<__nv_bfloat16, 64, 2>(maps, p, grid, st);
  } else if (dtype == 1) {
    if (D == 128) return launch_fwd_one<__half, 128, 1>(maps, p, grid, st);
    if (D == 64) return launch_fwd_one<__half, 64, 2>(maps, p, grid, st);
  }
  return (int)cudaErrorInvalidValue;
}

template <>
int tc_launch_bwd<InstMask>(int dtype, int D, const CUtensorMap* maps, const tc::BwdTcParams& p, cudaStream_t st) {
  return tc::launch_bwd_all<InstMask>(dtype, D, maps, p, st);
}

}  // namespace chill
