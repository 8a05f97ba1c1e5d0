// Backward attention on tcgen05 tensor cores (placeholder until the kernels land).
#pragma once
#include "generic.cuh"
#include "tc_common.cuh"

namespace chill {
namespace tc {

struct BwdTcParams {
  Geo g;
  const float* lse;
  long long lse_sb, lse_sh, lse_sl;
  const float* delta;
  int* status;
};

template <class M>
int launch_bwd_all(int, int, const CUtensorMap*, const BwdTcParams&, cudaStream_t) {
  return -1;  // not built yet: callers use the generic kernels
}

constexpr bool kHaveBwdTc = false;

}  // namespace tc
}  // namespace chill
