// Host-side launchers of the tensor-core kernels.  Each mask functor's kernels are compiled
// in a translation unit of their own (tc_inst.cu with -DCHILL_INST_MASK=<functor>), which
// defines the explicit specialisations declared here.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "generic.cuh"

namespace chill {
namespace tc {
struct FwdTcParams;
struct BwdTcParams;
}  // namespace tc

// maps: Q, K, V, O.  Returns a cudaError_t cast to int.
template <class M>
int tc_launch_fwd(int dtype, int D, const CUtensorMap* maps, const tc::FwdTcParams& p, dim3 grid, cudaStream_t st);

// fp32 tensors in TF32 (fwd_tf32.cuh); maps: Q, K, V (128B swizzle with 32-byte atoms), O.
template <class M>
int tc_launch_fwd_tf32(int D, const CUtensorMap* maps, const tc::FwdTcParams& p, dim3 grid, cudaStream_t st);

// maps: Q, K, V, dO, dQ, dK, dV.
template <class M>
int tc_launch_bwd(int dtype, int D, const CUtensorMap* maps, const tc::BwdTcParams& p, cudaStream_t st);

}  // namespace chill
