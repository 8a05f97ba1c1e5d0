// Host-side launchers of the tensor-core kernels.  Each mask functor's kernels are compiled
// in a translation unit of their own (tc_inst.cu with -DCHILL_INST_MASK=<functor>), which
// defines the explicit specialisations declared here.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>

#include "generic.cuh"

namespace chill {
namespace tc {
struct FwdTcParams;
struct BwdTcParams;
}  // namespace tc

// Raises a kernel's dynamic shared-memory limit the first time the kernel is launched on a device.  The attribute
// is per (kernel, device); the record of where it has been set is per call site (pass a distinct `Tag` per kernel)
// and guarded by a mutex, so host threads driving different devices do not race on it.
// `static`: the record must stay private to one copy of the library.  As an inline function its local statics become
// process-wide unique symbols, and a second library built from the same sources (a custom-mask build) loaded into
// the same process would find "already set" for kernels of its own that never had their limit raised.
template <class Tag, class Kern>
static cudaError_t ensure_dynamic_smem(Kern kern, int smem_bytes, bool prefer_max_carveout = false) {
  constexpr int kMaxDevices = 64;
  static bool done[kMaxDevices] = {};
  static std::mutex mu;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(mu);
  if (done[dev]) return cudaSuccess;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
  if (e != cudaSuccess) return e;
  if (prefer_max_carveout)
    cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  done[dev] = true;
  return cudaSuccess;
}

// maps: Q, K, V, O.  Returns a cudaError_t cast to int.
template <class M>
int tc_launch_fwd(int dtype, int D, const CUtensorMap* maps, const tc::FwdTcParams& p, dim3 grid, cudaStream_t st);

// fp32 tensors in TF32 (fwd_tf32.cuh); maps: Q, K, V (128B swizzle with 32-byte atoms), O.
template <class M>
int tc_launch_fwd_tf32(int D, const CUtensorMap* maps, const tc::FwdTcParams& p, dim3 grid, cudaStream_t st);

// maps: Q, K, V, dO, dQ, dK, dV.
template <class M>
int tc_launch_bwd(int dtype, int D, const CUtensorMap* maps, const tc::BwdTcParams& p, cudaStream_t st);

// 16-bit head dim 256 (bwd_wide.cuh, three launches); maps: Q, K, V, dO with 128-row boxes, the same four with 64-row
// boxes, dQ, dK, dV.
template <class M>
int tc_launch_bwd_wide(int dtype, const CUtensorMap* maps, const tc::BwdTcParams& p, cudaStream_t st);

// fp32 tensors in TF32, head dim 64 / 128 (bwd_tf32.cuh, which lists the eleven maps).
template <class M>
int tc_launch_bwd_tf32(int D, const CUtensorMap* maps, const tc::BwdTcParams& p, cudaStream_t st);

}  // namespace chill
