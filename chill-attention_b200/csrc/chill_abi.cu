// C ABI of the library (declared in include/chill_b200.h): argument validation, choice between
// the tensor-core and the generic kernels, TMA descriptor encoding, launches.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdio.h>
#include <string.h>

#include <atomic>
#include <mutex>

#include "bwd_tc.cuh"
#include "chill_b200.h"
#include "fwd_tc.cuh"
#include "generic.cuh"
#include "tc_launch.h"

namespace chill {

static thread_local char g_cuda_err[256] = "";
__device__ int g_device_status = 0;
static std::atomic<unsigned long long> g_launches{0};  // kernels launched by this library (chill_launch_count)

static int cuda_fail(cudaError_t e, const char* what) {
  snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: %s", what, cudaGetErrorString(e));
  return CHILL_E_CUDA;
}

int record_cuda_failure(cudaError_t e, const char* what) { return cuda_fail(e, what); }  // for host_pipeline.cu

static int* device_status_ptr() {
  // one word per device (the symbol is instantiated in every device's module image)
  int* p = nullptr;
  if (cudaGetSymbolAddress((void**)&p, g_device_status) != cudaSuccess) return nullptr;
  return p;
}

// ------------------------------------------------------------------------- validation
static size_t esize(int dtype) { return dtype == CHILL_F32 ? 4 : 2; }

static int check_shape(const chill_shape& s) {
  if (s.B <= 0 || s.H <= 0 || s.H_kv <= 0 || s.Lq <= 0 || s.Lk <= 0 || s.D <= 0) return CHILL_E_INVALID;
  if (s.H % s.H_kv != 0) return CHILL_E_INVALID;
  if (s.dtype != CHILL_F32 && s.dtype != CHILL_F16 && s.dtype != CHILL_BF16) return CHILL_E_UNSUPPORTED;
  if (s.D > kMaxD) return CHILL_E_UNSUPPORTED;
  if (s.seq_len <= 0 || s.q_offset < 0 || s.k_offset < 0) return CHILL_E_INVALID;
  if (s.B > 65535 || s.H > 65535) return CHILL_E_TOO_LARGE;
  if (s.mask.n_args < 0 || s.mask.n_args > CHILL_MAX_MASK_ARGS) return CHILL_E_INVALID;
#ifdef CHILL_CUSTOM_MASK
  if (s.mask.id < 0 || s.mask.id > CHILL_MASK_CUSTOM) return CHILL_E_UNSUPPORTED;
#else
  if (s.mask.id < 0 || s.mask.id >= CHILL_MASK_CUSTOM) return CHILL_E_UNSUPPORTED;
#endif
  if (s.mask.id == CHILL_MASK_CHUNKWISE && (s.mask.n_args < 2 || s.mask.i[0] <= 0)) return CHILL_E_INVALID;
  if (s.mask.id == CHILL_MASK_SLIDING && s.mask.n_args < 2) return CHILL_E_INVALID;
  if (s.mask.id == CHILL_MASK_PREFIXLM && s.mask.n_args < 1) return CHILL_E_INVALID;
  return CHILL_OK;
}

// The functors do their index arithmetic in 32 bits (position + constant), so the 64-bit constants of the ABI are
// saturated first.  For the built-in masks every constant is a distance or a size measured in positions, and any value
// beyond +-seq_len selects the same pairs as +-seq_len itself, so they are clamped there ("unbounded" written as
// 2**31 - 1 or 2**40 stays unbounded).  Constants of a custom functor are saturated to +-2^30, which still leaves
// room for adding a position.
static MaskArgs to_mask_args(const chill_mask_desc& m, long long seq_len) {
  MaskArgs a;
  const long long lim = (m.id >= 0 && m.id < CHILL_MASK_CUSTOM && seq_len > 0) ? seq_len : (1ll << 30);
  for (int i = 0; i < 8; ++i) {
    long long v = i < m.n_args ? (long long)m.i[i] : 0;
    v = v > lim ? lim : (v < -lim ? -lim : v);
    a.i[i] = (int)v;
    a.f[i] = i < m.n_args ? (float)m.f[i] : 0.f;
  }
  if (m.id == CHILL_MASK_CHUNKWISE && a.i[0] > 0 && seq_len > 0) {
    // back_contexts counts chunks: more chunks than the sequence has changes nothing, and (chunk + back + 1) * size
    // then stays far below 2^31
    const int n_chunks = (int)((seq_len + a.i[0] - 1) / a.i[0]);
    a.i[1] = a.i[1] > n_chunks ? n_chunks : (a.i[1] < -n_chunks ? -n_chunks : a.i[1]);
  }
  return a;
}

static Geo to_geo(const chill_shape& s) {
  Geo g;
  g.B = s.B; g.H = s.H; g.Hkv = s.H_kv; g.Lq = s.Lq; g.Lk = s.Lk; g.D = s.D;
  g.q_off = s.q_offset; g.k_off = s.k_offset; g.seq_len = s.seq_len;
  g.scale = s.sm_scale; g.lens = s.lens; g.margs = to_mask_args(s.mask, s.seq_len);
  return g;
}

static TRef to_ref(const void* p, const int64_t* st) {
  TRef r;
  r.p = const_cast<void*>(p);
  r.sb = st[0]; r.sh = st[1]; r.sl = st[2]; r.sd = st[3];
  return r;
}

// A [B][H][L][D] tensor can be described to TMA when channels are contiguous and everything
// else is 16-byte aligned.
static bool tma_ok(const void* p, const int64_t* st, int B, int H, int L, size_t es) {
  if (st[3] != 1) return false;
  if (((uintptr_t)p) % 16 != 0) return false;
  if ((st[2] * (int64_t)es) % 16 != 0 || st[2] <= 0) return false;
  if (H > 1 && ((st[1] * (int64_t)es) % 16 != 0 || st[1] <= 0)) return false;
  if (B > 1 && ((st[0] * (int64_t)es) % 16 != 0 || st[0] <= 0)) return false;
  (void)L;
  return true;
}

static bool shape_tc_ok(const chill_shape& s) {
  if (s.flags & CHILL_FLAG_FORCE_GENERIC) return false;
  if (s.dtype != CHILL_F16 && s.dtype != CHILL_BF16) return false;
  if (s.D != 64 && s.D != 128) return false;
  if (!(s.sm_scale > 0.f)) return false;
  return true;
}

// ------------------------------------------------------------------------ TMA encoding
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

// Box = 64 channels x `box_rows` positions of one (batch, head), 128B swizzle.
static int make_map(CUtensorMap* m, const void* p, const int64_t* st, int B, int H, int L, int D, int dtype,
                    int box_rows, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "cuTensorMapEncodeTiled entry point not available");
    return CHILL_E_CUDA;
  }
  const cuuint64_t es = esize(dtype);
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)L, (cuuint64_t)H, (cuuint64_t)B};
  const cuuint64_t row = (cuuint64_t)st[2] * es;
  cuuint64_t strides[3] = {row, H > 1 ? (cuuint64_t)st[1] * es : row * (cuuint64_t)L,
                           B > 1 ? (cuuint64_t)st[0] * es : row * (cuuint64_t)L * (cuuint64_t)H};
  cuuint32_t box[4] = {(cuuint32_t)(128 / es), (cuuint32_t)box_rows, 1, 1};  // 128-byte rows
  cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUtensorMapDataType dt = dtype == CHILL_BF16   ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                 : dtype == CHILL_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                      : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = fn(m, dt, 4, const_cast<void*>(p), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return CHILL_E_CUDA;
  }
  return CHILL_OK;
}

// --------------------------------------------------------------------------- dispatch
#ifdef CHILL_CUSTOM_MASK
#define CHILL_CUSTOM_CASE(CALL) \
  case CHILL_MASK_CUSTOM: { using MaskT = CHILL_CUSTOM_MASK; CALL; break; }
#else
#define CHILL_CUSTOM_CASE(CALL)
#endif

#define CHILL_MASK_SWITCH(ID, CALL)                                        \
  switch (ID) {                                                            \
    case CHILL_MASK_FULL: { using MaskT = FullMask; CALL; break; }         \
    case CHILL_MASK_CAUSAL: { using MaskT = CausalMask; CALL; break; }     \
    case CHILL_MASK_SLIDING: { using MaskT = SlidingWindowMask; CALL; break; } \
    case CHILL_MASK_CHUNKWISE: { using MaskT = ChunkwiseMask; CALL; break; } \
    case CHILL_MASK_PREFIXLM: { using MaskT = PrefixLMMask; CALL; break; } \
    CHILL_CUSTOM_CASE(CALL)                                                \
    default: return CHILL_E_UNSUPPORTED;                                   \
  }

#define CHILL_DTYPE_SWITCH(DT, CALL)                                  \
  switch (DT) {                                                       \
    case CHILL_F32: { using ElemT = float; CALL; break; }             \
    case CHILL_F16: { using ElemT = __half; CALL; break; }            \
    case CHILL_BF16: { using ElemT = __nv_bfloat16; CALL; break; }    \
    default: return CHILL_E_UNSUPPORTED;                              \
  }

// fp32 tensors whose caller allowed TF32: forward on the tensor cores (fwd_tf32.cuh)
static bool shape_tf32_ok(const chill_shape& s) {
  if (s.flags & CHILL_FLAG_FORCE_GENERIC) return false;
  return s.dtype == CHILL_F32 && (s.flags & CHILL_FLAG_ALLOW_TF32) && (s.D == 64 || s.D == 128) && s.sm_scale > 0.f;
}

// the forward also has a tensor-core kernel for 16-bit head dim 256 (one CTA per SM); the backward does not
static bool shape_tc_fwd_only_ok(const chill_shape& s) {
  if (s.flags & CHILL_FLAG_FORCE_GENERIC) return false;
  return (s.dtype == CHILL_F16 || s.dtype == CHILL_BF16) && s.D == 256 && s.sm_scale > 0.f;
}

static bool fwd_tc_eligible(const chill_fwd_args& a) {
  const chill_shape& s = a.s;
  if (!shape_tc_ok(s) && !shape_tf32_ok(s) && !shape_tc_fwd_only_ok(s)) return false;
  const size_t es = esize(s.dtype);
  return tma_ok(a.q, a.q_strides, s.B, s.H, s.Lq, es) && tma_ok(a.k, a.k_strides, s.B, s.H_kv, s.Lk, es) &&
         tma_ok(a.v, a.v_strides, s.B, s.H_kv, s.Lk, es) && tma_ok(a.o, a.o_strides, s.B, s.H, s.Lq, es);
}

static int check_fwd(const chill_fwd_args* a) {
  if (a == nullptr) return CHILL_E_INVALID;
  int st = check_shape(a->s);
  if (st != CHILL_OK) return st;
  if (!a->q || !a->k || !a->v || !a->o) return CHILL_E_INVALID;
  return CHILL_OK;
}

static int fwd_generic(const chill_fwd_args& a, cudaStream_t st) {
  FwdP p;
  p.g = to_geo(a.s);
  p.q = to_ref(a.q, a.q_strides); p.k = to_ref(a.k, a.k_strides);
  p.v = to_ref(a.v, a.v_strides); p.o = to_ref(a.o, a.o_strides);
  p.lse = a.lse;
  p.lse_sb = a.lse_strides[0]; p.lse_sh = a.lse_strides[1]; p.lse_sl = a.lse_strides[2];
  dim3 grid((a.s.Lq + kGenericWarps - 1) / kGenericWarps, a.s.H, a.s.B);
  CHILL_MASK_SWITCH(a.s.mask.id,
                    CHILL_DTYPE_SWITCH(a.s.dtype, (fwd_generic_kernel<ElemT, MaskT><<<grid, kGenericWarps * 32, 0, st>>>(p))))
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) g_launches += 1;
  return e == cudaSuccess ? CHILL_OK : cuda_fail(e, "fwd_generic launch");
}

static int fwd_tc(const chill_fwd_args& a, cudaStream_t st) {
  const chill_shape& s = a.s;
  CUtensorMap maps[4];
  int rc;
  if ((rc = make_map(&maps[0], a.q, a.q_strides, s.B, s.H, s.Lq, s.D, s.dtype, tc::kTile)) != CHILL_OK) return rc;
  // V is the MN-major operand of O += P V; with 32-bit elements that takes the 128B swizzle with 32-byte atoms
  const bool tf32 = s.dtype == CHILL_F32;
  // keys per K / V tile of the kernel that will run (see FwdShape)
  const int kv_rows = tf32 ? tc::kTile
                           : (s.D == 64 ? tc::FwdShape<64>::kKeys
                                        : (s.D == 128 ? tc::FwdShape<128>::kKeys : tc::FwdShape<256>::kKeys));
  if ((rc = make_map(&maps[1], a.k, a.k_strides, s.B, s.H_kv, s.Lk, s.D, s.dtype, kv_rows)) != CHILL_OK) return rc;
  if ((rc = make_map(&maps[2], a.v, a.v_strides, s.B, s.H_kv, s.Lk, s.D, s.dtype, kv_rows,
                     tf32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B)) != CHILL_OK)
    return rc;
  if ((rc = make_map(&maps[3], a.o, a.o_strides, s.B, s.H, s.Lq, s.D, s.dtype, tc::kTile)) != CHILL_OK) return rc;
  tc::FwdTcParams p;
  p.g = to_geo(s);
  p.lse = a.lse;
  p.lse_sb = a.lse_strides[0]; p.lse_sh = a.lse_strides[1]; p.lse_sl = a.lse_strides[2];
  p.o = a.o;
  p.o_sb = a.o_strides[0]; p.o_sh = a.o_strides[1]; p.o_sl = a.o_strides[2];
  p.status = device_status_ptr();
  if (p.status == nullptr) return cuda_fail(cudaGetLastError(), "status symbol");
  dim3 grid((unsigned)(((s.Lq + tc::kTile - 1) / tc::kTile) * s.H * s.B), 1, 1);
  int e = 0;
  if (tf32) {
    CHILL_MASK_SWITCH(s.mask.id, (e = tc_launch_fwd_tf32<MaskT>(s.D, maps, p, grid, st)))
  } else {
    CHILL_MASK_SWITCH(s.mask.id, (e = tc_launch_fwd<MaskT>(s.dtype, s.D, maps, p, grid, st)))
  }
  if (e == 0) g_launches += 1;
  return e == 0 ? CHILL_OK : cuda_fail((cudaError_t)e, "fwd_tc launch");
}

// ------------------------------------------------------------------------------ backward
static int check_bwd(const chill_bwd_args* a, bool need_all) {
  if (a == nullptr) return CHILL_E_INVALID;
  int st = check_shape(a->s);
  if (st != CHILL_OK) return st;
  if (!a->o || !a->d_o || !a->delta) return CHILL_E_INVALID;
  if (need_all && (!a->q || !a->k || !a->v || !a->lse || !a->dq || !a->dk || !a->dv)) return CHILL_E_INVALID;
  if ((a->dk_part == nullptr) != (a->dv_part == nullptr)) return CHILL_E_INVALID;
  if (a->dk_part != nullptr) {
    if (a->part_head < 0 || a->part_tail < 0 || (long long)a->part_head + a->part_tail > a->s.Lk) return CHILL_E_INVALID;
    // rows are written 16 bytes at a time
    if (((uintptr_t)a->dk_part | (uintptr_t)a->dv_part) % 16 != 0 || a->s.D % 4 != 0) return CHILL_E_INVALID;
    for (int i = 0; i < 3; ++i)
      if (a->part_strides[i] % 4 != 0 || a->part_strides[i] < 0) return CHILL_E_INVALID;
  }
  return CHILL_OK;
}

static bool bwd_tc_eligible(const chill_bwd_args& a) {
  if (!tc::kHaveBwdTc) return false;
  const chill_shape& s = a.s;
  if (!shape_tc_ok(s)) return false;
  const size_t es = esize(s.dtype);
  return tma_ok(a.q, a.q_strides, s.B, s.H, s.Lq, es) && tma_ok(a.k, a.k_strides, s.B, s.H_kv, s.Lk, es) &&
         tma_ok(a.v, a.v_strides, s.B, s.H_kv, s.Lk, es) && tma_ok(a.d_o, a.do_strides, s.B, s.H, s.Lq, es) &&
         tma_ok(a.dq, a.dq_strides, s.B, s.H, s.Lq, es) && tma_ok(a.dk, a.dk_strides, s.B, s.H_kv, s.Lk, es) &&
         tma_ok(a.dv, a.dv_strides, s.B, s.H_kv, s.Lk, es) && a.lse_strides[2] == 1;
}

// 16-bit head dim 256: three tensor-core launches (bwd_wide.cuh); no per-kernel selection
static bool bwd_wide_eligible(const chill_bwd_args& a) {
  const chill_shape& s = a.s;
  if (!shape_tc_fwd_only_ok(s)) return false;
  if (s.flags & (CHILL_FLAG_BWD_ONLY_DKDV | CHILL_FLAG_BWD_ONLY_DQ)) return false;
  const size_t es = esize(s.dtype);
  return tma_ok(a.q, a.q_strides, s.B, s.H, s.Lq, es) && tma_ok(a.k, a.k_strides, s.B, s.H_kv, s.Lk, es) &&
         tma_ok(a.v, a.v_strides, s.B, s.H_kv, s.Lk, es) && tma_ok(a.d_o, a.do_strides, s.B, s.H, s.Lq, es) &&
         tma_ok(a.dq, a.dq_strides, s.B, s.H, s.Lq, es) && tma_ok(a.dk, a.dk_strides, s.B, s.H_kv, s.Lk, es) &&
         tma_ok(a.dv, a.dv_strides, s.B, s.H_kv, s.Lk, es) && a.lse_strides[2] == 1;
}

static PartOut to_part(const chill_bwd_args& a) {
  PartOut o;
  if (a.dk_part != nullptr && a.dv_part != nullptr && a.part_head + a.part_tail > 0) {
    o.dk = a.dk_part; o.dv = a.dv_part;
    o.sb = a.part_strides[0]; o.sh = a.part_strides[1]; o.sl = a.part_strides[2];
    o.head = a.part_head; o.tail = a.part_tail;
  }
  return o;
}

// fp32 tensors whose caller allowed TF32, head dim 64 / 128: backward on the tensor cores (bwd_tf32.cuh).  dQ / dK / dV
// are written by the threads themselves, 16 bytes at a time.
static bool bwd_tf32_eligible(const chill_bwd_args& a) {
  const chill_shape& s = a.s;
  if (s.flags & CHILL_FLAG_FORCE_GENERIC) return false;
  if (s.dtype != CHILL_F32 || !(s.flags & CHILL_FLAG_ALLOW_TF32) || (s.D != 64 && s.D != 128) || !(s.sm_scale > 0.f)) return false;
  if (a.dk_part != nullptr) return false;
  return tma_ok(a.q, a.q_strides, s.B, s.H, s.Lq, 4) && tma_ok(a.k, a.k_strides, s.B, s.H_kv, s.Lk, 4) &&
         tma_ok(a.v, a.v_strides, s.B, s.H_kv, s.Lk, 4) && tma_ok(a.d_o, a.do_strides, s.B, s.H, s.Lq, 4) &&
         tma_ok(a.dq, a.dq_strides, s.B, s.H, s.Lq, 4) && tma_ok(a.dk, a.dk_strides, s.B, s.H_kv, s.Lk, 4) &&
         tma_ok(a.dv, a.dv_strides, s.B, s.H_kv, s.Lk, 4) && a.lse_strides[2] == 1;
}

static BwdP to_bwdp(const chill_bwd_args& a) {
  BwdP p;
  p.g = to_geo(a.s);
  p.q = to_ref(a.q, a.q_strides); p.k = to_ref(a.k, a.k_strides); p.v = to_ref(a.v, a.v_strides);
  p.o = to_ref(a.o, a.o_strides); p.d_o = to_ref(a.d_o, a.do_strides);
  p.dq = to_ref(a.dq, a.dq_strides); p.dk = to_ref(a.dk, a.dk_strides); p.dv = to_ref(a.dv, a.dv_strides);
  p.lse = a.lse;
  p.lse_sb = a.lse_strides[0]; p.lse_sh = a.lse_strides[1]; p.lse_sl = a.lse_strides[2];
  p.delta = a.delta;
  p.part = to_part(a);
  return p;
}

static int delta_launch(const chill_bwd_args& a, cudaStream_t st) {
  const chill_shape& s = a.s;
  const size_t es = esize(s.dtype);
  const long long dl[3] = {a.d_lse ? a.dlse_strides[0] : 0, a.d_lse ? a.dlse_strides[1] : 0, a.d_lse ? a.dlse_strides[2] : 0};
  const bool fast = (s.dtype != CHILL_F32) && (s.D == 64 || s.D == 128) &&
                    tma_ok(a.o, a.o_strides, s.B, s.H, s.Lq, es) && tma_ok(a.d_o, a.do_strides, s.B, s.H, s.Lq, es);
  if (fast) {
    const int rows_per_block = 8 * (32 / (s.D / 8));
    dim3 grid((s.Lq + rows_per_block - 1) / rows_per_block, s.H, s.B);
#define CHILL_DELTA16(T, DD)                                                                                     \
  delta_rows16_kernel<T, DD><<<grid, 256, 0, st>>>((const T*)a.o, (const T*)a.d_o, a.delta, a.o_strides[0],        \
                                                   a.o_strides[1], a.o_strides[2], a.do_strides[0], a.do_strides[1], \
                                                   a.do_strides[2], s.H, s.Lq, a.d_lse, dl[0], dl[1], dl[2])
    if (s.dtype == CHILL_BF16) {
      if (s.D == 64) CHILL_DELTA16(__nv_bfloat16, 64); else CHILL_DELTA16(__nv_bfloat16, 128);
    } else {
      if (s.D == 64) CHILL_DELTA16(__half, 64); else CHILL_DELTA16(__half, 128);
    }
#undef CHILL_DELTA16
  } else {
    dim3 grid((s.Lq + kGenericWarps - 1) / kGenericWarps, s.H, s.B);
    TRef o = to_ref(a.o, a.o_strides), d_o = to_ref(a.d_o, a.do_strides);
    CHILL_DTYPE_SWITCH(s.dtype, (delta_kernel<ElemT><<<grid, kGenericWarps * 32, 0, st>>>(o, d_o, a.delta, s.H, s.Lq, s.D, a.d_lse, dl[0], dl[1], dl[2])))
  }
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) g_launches += 1;
  return e == cudaSuccess ? CHILL_OK : cuda_fail(e, "delta launch");
}

static int bwd_which(uint32_t flags) {
  if (flags & CHILL_FLAG_BWD_ONLY_DKDV) return 1;
  if (flags & CHILL_FLAG_BWD_ONLY_DQ) return 2;
  return 3;
}

static int bwd_generic(const chill_bwd_args& a, cudaStream_t st) {
  BwdP p = to_bwdp(a);
  const chill_shape& s = a.s;
  const int which = bwd_which(s.flags);
  dim3 gq((s.Lq + kGenericWarps - 1) / kGenericWarps, s.H, s.B);
  dim3 gk((s.Lk + kGenericWarps - 1) / kGenericWarps, s.H_kv, s.B);
  CHILL_MASK_SWITCH(s.mask.id, CHILL_DTYPE_SWITCH(s.dtype, {
                      if (which & 2) (bwd_dq_generic_kernel<ElemT, MaskT><<<gq, kGenericWarps * 32, 0, st>>>(p));
                      if (which & 1) (bwd_dkdv_generic_kernel<ElemT, MaskT><<<gk, kGenericWarps * 32, 0, st>>>(p));
                    }))
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) g_launches += (which == 3 ? 2 : 1);
  return e == cudaSuccess ? CHILL_OK : cuda_fail(e, "bwd_generic launch");
}

// Side stream + fork/join events per device, created on first use: the dK/dV and the dQ kernel are
// independent, so the second one starts filling SMs as the first one's last wave drains.
struct SideStream {
  cudaStream_t stream = nullptr;
  cudaEvent_t fork = nullptr, join = nullptr;
  std::mutex mu;  // held across one fork / launch / join sequence
};

static SideStream* side_stream() {
  constexpr int kMaxDevices = 64;
  static SideStream cache[kMaxDevices];
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  SideStream& s = cache[dev];
  if (s.stream == nullptr) {
    if (cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
    if (cudaEventCreateWithFlags(&s.fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&s.join, cudaEventDisableTiming) != cudaSuccess) {
      s.stream = nullptr;
      return nullptr;
    }
  }
  return &s;
}

static void fill_bwd_tc_params(const chill_bwd_args& a, tc::BwdTcParams& p) {
  const chill_shape& s = a.s;
  p.g = to_geo(s);
  p.lse = a.lse;
  p.lse_sb = a.lse_strides[0]; p.lse_sh = a.lse_strides[1]; p.lse_sl = a.lse_strides[2];
  p.delta = a.delta;
  p.dq = a.dq; p.dk = a.dk; p.dv = a.dv;
  p.dq_sb = a.dq_strides[0]; p.dq_sh = a.dq_strides[1]; p.dq_sl = a.dq_strides[2];
  p.dk_sb = a.dk_strides[0]; p.dk_sh = a.dk_strides[1]; p.dk_sl = a.dk_strides[2];
  p.dv_sb = a.dv_strides[0]; p.dv_sh = a.dv_strides[1]; p.dv_sl = a.dv_strides[2];
  p.which = bwd_which(s.flags);
  p.dq_accum = nullptr;
  p.part = to_part(a);
}

static int bwd_tf32(const chill_bwd_args& a, cudaStream_t st) {
  const chill_shape& s = a.s;
  // streamed tiles have TO rows (128 at head dim 64, 32 at head dim 128), resident ones 128; "mn" copies (read
  // MN-major by the tensor core) take the 128-byte swizzle with 32-byte atoms
  const int to = s.D == 64 ? 128 : 32;
  struct MapSpec { const void* p; const int64_t* st; bool kv; int rows; bool mn; };
  const MapSpec spec[11] = {
      {a.q, a.q_strides, false, to, false},   {a.q, a.q_strides, false, to, true},
      {a.d_o, a.do_strides, false, to, false}, {a.d_o, a.do_strides, false, to, true},
      {a.k, a.k_strides, true, tc::kTile, false}, {a.v, a.v_strides, true, tc::kTile, false},
      {a.q, a.q_strides, false, tc::kTile, false}, {a.d_o, a.do_strides, false, tc::kTile, false},
      {a.k, a.k_strides, true, to, false},    {a.k, a.k_strides, true, to, true},
      {a.v, a.v_strides, true, to, false}};
  CUtensorMap maps[11];
  for (int i = 0; i < 11; ++i) {
    int rc = make_map(&maps[i], spec[i].p, spec[i].st, s.B, spec[i].kv ? s.H_kv : s.H, spec[i].kv ? s.Lk : s.Lq, s.D, s.dtype,
                      spec[i].rows, spec[i].mn ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != CHILL_OK) return rc;
  }
  tc::BwdTcParams p;
  fill_bwd_tc_params(a, p);
  p.status = device_status_ptr();
  if (p.status == nullptr) return cuda_fail(cudaGetLastError(), "status symbol");
  int e = 0;
  CHILL_MASK_SWITCH(s.mask.id, (e = tc_launch_bwd_tf32<MaskT>(s.D, maps, p, st)))
  if (e == 0) g_launches += (p.which == 3 ? 2 : 1);
  return e == 0 ? CHILL_OK : cuda_fail((cudaError_t)e, "bwd_tf32 launch");
}

static int bwd_tc(const chill_bwd_args& a, cudaStream_t st, bool concurrent = true, bool fused = true) {
  const chill_shape& s = a.s;
  CUtensorMap maps[7];
  const void* ptrs[7] = {a.q, a.k, a.v, a.d_o, a.dq, a.dk, a.dv};
  const int64_t* strs[7] = {a.q_strides, a.k_strides, a.v_strides, a.do_strides, a.dq_strides, a.dk_strides, a.dv_strides};
  const bool is_kv[7] = {false, true, true, false, false, true, true};
  for (int i = 0; i < 7; ++i) {
    int rc = make_map(&maps[i], ptrs[i], strs[i], s.B, is_kv[i] ? s.H_kv : s.H, is_kv[i] ? s.Lk : s.Lq, s.D, s.dtype,
                      tc::kTile);
    if (rc != CHILL_OK) return rc;
  }
  tc::BwdTcParams p;
  fill_bwd_tc_params(a, p);
  p.status = device_status_ptr();
  if (p.status == nullptr) return cuda_fail(cudaGetLastError(), "status symbol");
  int e = 0;
  if (fused && p.which == 3 && a.dq_accum != nullptr) {
    if ((reinterpret_cast<uintptr_t>(a.dq_accum) & 15u) != 0) return CHILL_E_INVALID;
    p.dq_accum = a.dq_accum;  // single-kernel backward + conversion of the fp32 dQ sums
    CHILL_MASK_SWITCH(s.mask.id, (e = tc_launch_bwd<MaskT>(s.dtype, s.D, maps, p, st)))
    if (e == 0) g_launches += 2;
    return e == 0 ? CHILL_OK : cuda_fail((cudaError_t)e, "bwd_fused launch");
  }
  SideStream* side = (concurrent && p.which == 3) ? side_stream() : nullptr;
  if (side != nullptr) {
    // fork: dK/dV on the caller's stream, dQ on the side stream; join back before returning.  The helper stream and
    // its two events are shared by every caller on this device, so the whole record / wait / launch / record / wait
    // sequence is one critical section: a second host thread must not re-record `fork` or `join` in between.
    std::lock_guard<std::mutex> lock(side->mu);
    cudaError_t ce = cudaEventRecord(side->fork, st);
    if (ce == cudaSuccess) ce = cudaStreamWaitEvent(side->stream, side->fork, 0);
    if (ce != cudaSuccess) return cuda_fail(ce, "bwd fork");
    p.which = 1;
    CHILL_MASK_SWITCH(s.mask.id, (e = tc_launch_bwd<MaskT>(s.dtype, s.D, maps, p, st)))
    if (e == 0) {
      p.which = 2;
      CHILL_MASK_SWITCH(s.mask.id, (e = tc_launch_bwd<MaskT>(s.dtype, s.D, maps, p, side->stream)))
    }
    ce = cudaEventRecord(side->join, side->stream);
    if (ce == cudaSuccess) ce = cudaStreamWaitEvent(st, side->join, 0);
    if (ce != cudaSuccess) return cuda_fail(ce, "bwd join");
    if (e == 0) g_launches += 2;
    return e == 0 ? CHILL_OK : cuda_fail((cudaError_t)e, "bwd_tc launch");
  }
  CHILL_MASK_SWITCH(s.mask.id, (e = tc_launch_bwd<MaskT>(s.dtype, s.D, maps, p, st)))
  if (e == 0) g_launches += (p.which == 3 ? 2 : 1);
  return e == 0 ? CHILL_OK : cuda_fail((cudaError_t)e, "bwd_tc launch");
}

static int bwd_wide(const chill_bwd_args& a, cudaStream_t st) {
  const chill_shape& s = a.s;
  CUtensorMap maps[11];
  const void* in[4] = {a.q, a.k, a.v, a.d_o};
  const int64_t* in_st[4] = {a.q_strides, a.k_strides, a.v_strides, a.do_strides};
  const bool in_kv[4] = {false, true, true, false};
  int rc;
  for (int i = 0; i < 4; ++i) {
    const int H = in_kv[i] ? s.H_kv : s.H, L = in_kv[i] ? s.Lk : s.Lq;
    if ((rc = make_map(&maps[i], in[i], in_st[i], s.B, H, L, s.D, s.dtype, tc::kTile)) != CHILL_OK) return rc;
    if ((rc = make_map(&maps[4 + i], in[i], in_st[i], s.B, H, L, s.D, s.dtype, tc::kWideCols)) != CHILL_OK) return rc;
  }
  if ((rc = make_map(&maps[8], a.dq, a.dq_strides, s.B, s.H, s.Lq, s.D, s.dtype, tc::kTile)) != CHILL_OK) return rc;
  if ((rc = make_map(&maps[9], a.dk, a.dk_strides, s.B, s.H_kv, s.Lk, s.D, s.dtype, tc::kTile)) != CHILL_OK) return rc;
  if ((rc = make_map(&maps[10], a.dv, a.dv_strides, s.B, s.H_kv, s.Lk, s.D, s.dtype, tc::kTile)) != CHILL_OK) return rc;
  tc::BwdTcParams p;
  fill_bwd_tc_params(a, p);
  p.status = device_status_ptr();
  if (p.status == nullptr) return cuda_fail(cudaGetLastError(), "status symbol");
  int e = 0;
  CHILL_MASK_SWITCH(s.mask.id, (e = tc_launch_bwd_wide<MaskT>(s.dtype, maps, p, st)))
  if (e == 0) g_launches += 3;
  return e == 0 ? CHILL_OK : cuda_fail((cudaError_t)e, "bwd_wide launch");
}

// ------------------------------------------------------------- backward without a scratch argument
// Library-owned scratch for chill_bwd_noalloc: lives in the device image of this file, one copy per
// GPU that loads the library.  In host code the name below is only a handle for the runtime; the
// address the kernels need comes from cudaGetSymbolAddress, once per device.
static __device__ __align__(256) float g_noalloc_delta[CHILL_NOALLOC_MAX_ROWS];

static int noalloc_scratch(float** out) {
  constexpr int kMaxDevices = 64;
  static float* ptrs[kMaxDevices] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices) return CHILL_E_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(mu);
  if (ptrs[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_delta);  // resolves against the CURRENT device
    if (e != cudaSuccess || p == nullptr) return cuda_fail(e, "cudaGetSymbolAddress(noalloc scratch)");
    ptrs[dev] = p;
  }
  *out = ptrs[dev];
  return CHILL_OK;
}

// Self-test of the give-up path (chill_selftest_bounded_wait): the role structure of the tensor-core kernels in
// miniature.  Warp 0 owns a TMEM allocation and plays the producer, every other warp a consumer; all of them wait on
// an mbarrier that is initialised but never arrived at.  The first waiter whose limit runs out records the code and
// raises the CTA's abort flag, the others see the flag and leave, TMEM is released and the kernel returns.
__global__ void __launch_bounds__(128) selftest_bounded_wait_kernel(int* status, unsigned long long limit_ns) {
  __shared__ __align__(8) unsigned long long bar_storage;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t bar = tc::smem_u32(&bar_storage);
  if (threadIdx.x == 0) {
    abort_flag = 0;
    tc::mbar_init(bar, 1);
    tc::fence_barrier_init();
  }
  if (warp == 0) {
    tc::tmem_alloc(tc::smem_u32(&tmem_slot), 32);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const tc::Guard guard{status, &abort_flag};
  bool ok = true;
  if (lane == 0) ok = tc::mbar_wait(bar, 0, guard, tc::kStSelfTest, limit_ns + (unsigned long long)warp * 1000ull);
  ok = __all_sync(0xffffffffu, ok);  // the warp leaves together, as the kernels' roles do
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem_slot, 32);
  (void)ok;
}

template <class M>
static int traits_of() {
  return (M::kHasKFullRange ? 1 : 0) | (M::kHasQFullRange ? 2 : 0) | (M::kKLimsContinuous ? 4 : 0) |
         (M::kQLimsContinuous ? 8 : 0) | (M::kGuaranteedSafe ? 16 : 0);
}

}  // namespace chill

using namespace chill;

extern "C" {

int chill_abi_version(void) { return CHILL_ABI_VERSION; }

const char* chill_status_string(int status) {
  switch (status) {
    case CHILL_OK: return "ok";
    case CHILL_E_INVALID: return "invalid argument";
    case CHILL_E_UNSUPPORTED: return "unsupported dtype, head dim or mask for this build";
    case CHILL_E_CUDA: return "CUDA call failed";
    case CHILL_E_TOO_LARGE: return "size exceeds the supported maximum";
    default: return "unknown status";
  }
}

const char* chill_last_cuda_error(void) { return g_cuda_err; }

int chill_fwd_uses_tensor_cores(const chill_fwd_args* a) {
  int st = check_fwd(a);
  if (st != CHILL_OK) return st;
  return fwd_tc_eligible(*a) ? 1 : 0;
}

int chill_bwd_uses_tensor_cores(const chill_bwd_args* a) {
  int st = check_bwd(a, true);
  if (st != CHILL_OK) return st;
  return (bwd_tc_eligible(*a) || bwd_wide_eligible(*a) || bwd_tf32_eligible(*a)) ? 1 : 0;
}

int chill_fwd(const chill_fwd_args* a, void* stream) {
  int st = check_fwd(a);
  if (st != CHILL_OK) return st;
  if (fwd_tc_eligible(*a)) return fwd_tc(*a, (cudaStream_t)stream);
  if (a->s.flags & CHILL_FLAG_REQUIRE_TC) return CHILL_E_UNSUPPORTED;
  return fwd_generic(*a, (cudaStream_t)stream);
}

size_t chill_bwd_scratch_bytes(const chill_shape* s) {
  if (s == nullptr || s->B <= 0 || s->H <= 0 || s->Lq <= 0) return 0;
  return (size_t)s->B * (size_t)s->H * (size_t)s->Lq * sizeof(float);
}

size_t chill_bwd_dq_accum_bytes(const chill_shape* s) {
  if (s == nullptr || s->B <= 0 || s->H <= 0 || s->Lq <= 0) return 0;
  if (s->dtype == CHILL_F32 || (s->D != 64 && s->D != 128)) return 0;
  return tc::dq_accum_bytes(s->B, s->H, s->Lq, s->D);
}

int chill_bwd_delta(const chill_bwd_args* a, void* stream) {
  int st = check_bwd(a, false);
  if (st != CHILL_OK) return st;
  return delta_launch(*a, (cudaStream_t)stream);
}

int chill_bwd(const chill_bwd_args* a, void* stream) {
  int st = check_bwd(a, true);
  if (st != CHILL_OK) return st;
  if (bwd_tc_eligible(*a)) return bwd_tc(*a, (cudaStream_t)stream);
  if (bwd_wide_eligible(*a)) return bwd_wide(*a, (cudaStream_t)stream);
  if (bwd_tf32_eligible(*a)) return bwd_tf32(*a, (cudaStream_t)stream);
  if (a->s.flags & CHILL_FLAG_REQUIRE_TC) return CHILL_E_UNSUPPORTED;
  return bwd_generic(*a, (cudaStream_t)stream);
}

int chill_bwd_noalloc(const chill_bwd_args* a, void* stream) {
  if (a == nullptr) return CHILL_E_INVALID;
  chill_bwd_args b = *a;  // private copy: the caller's struct is not modified
  float* scratch = reinterpret_cast<float*>(16);  // placeholder so the pointer check below passes
  b.delta = scratch;
  int st = check_bwd(&b, true);
  if (st != CHILL_OK) return st;
  const unsigned long long rows = (unsigned long long)b.s.B * (unsigned long long)b.s.H * (unsigned long long)b.s.Lq;
  if (rows > (unsigned long long)CHILL_NOALLOC_MAX_ROWS) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "chill_bwd_noalloc: B*H*Lq = %llu exceeds CHILL_NOALLOC_MAX_ROWS = %u",
             rows, (unsigned)CHILL_NOALLOC_MAX_ROWS);
    return CHILL_E_TOO_LARGE;
  }
  st = noalloc_scratch(&scratch);
  if (st != CHILL_OK) return st;
  b.delta = scratch;
  st = delta_launch(b, (cudaStream_t)stream);
  if (st != CHILL_OK) return st;
  if (bwd_tc_eligible(b)) return bwd_tc(b, (cudaStream_t)stream, /*concurrent=*/false, /*fused=*/false);  // one stream, no helper objects
  if (bwd_wide_eligible(b)) return bwd_wide(b, (cudaStream_t)stream);
  if (bwd_tf32_eligible(b)) return bwd_tf32(b, (cudaStream_t)stream);
  if (b.s.flags & CHILL_FLAG_REQUIRE_TC) return CHILL_E_UNSUPPORTED;
  return bwd_generic(b, (cudaStream_t)stream);
}

int chill_mask_tabulate(const chill_mask_desc* m, int32_t n, int32_t tile, uint8_t* dense, int32_t* k_lims,
                        int32_t* q_lims, int32_t* k_full, int32_t* q_full, void* stream) {
  if (m == nullptr || n <= 0 || tile <= 0 || n > 32768) return CHILL_E_INVALID;
  MaskArgs a = to_mask_args(*m, n);
  const long long total = dense != nullptr ? (long long)n * n : (long long)n;
  const int threads = 256;
  const unsigned blocks = (unsigned)((total + threads - 1) / threads);
  cudaStream_t st = (cudaStream_t)stream;
  CHILL_MASK_SWITCH(m->id, (mask_tabulate_kernel<MaskT><<<blocks, threads, 0, st>>>(a, n, tile, dense, k_lims, q_lims, k_full, q_full)))
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) g_launches += 1;
  return e == cudaSuccess ? CHILL_OK : cuda_fail(e, "mask_tabulate launch");
}

int chill_mask_tabulate_blocks(const chill_mask_desc* m, int32_t n, int32_t q_tile, int32_t k_tile, uint8_t* full,
                               void* stream) {
  if (m == nullptr || full == nullptr || n <= 0 || q_tile <= 0 || k_tile <= 0 || n > 32768) return CHILL_E_INVALID;
  MaskArgs a = to_mask_args(*m, n);
  const long long total = (long long)((n + q_tile - 1) / q_tile) * ((n + k_tile - 1) / k_tile);
  const int threads = 256;
  const unsigned blocks = (unsigned)((total + threads - 1) / threads);
  cudaStream_t st = (cudaStream_t)stream;
  CHILL_MASK_SWITCH(m->id, (mask_tabulate_blocks_kernel<MaskT><<<blocks, threads, 0, st>>>(a, n, q_tile, k_tile, full)))
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) g_launches += 1;
  return e == cudaSuccess ? CHILL_OK : cuda_fail(e, "mask_tabulate_blocks launch");
}

int chill_selftest_bounded_wait(int32_t limit_us, void* stream) {
  int* status = device_status_ptr();
  if (status == nullptr) return cuda_fail(cudaGetLastError(), "status symbol");
  const long long us = limit_us < 10 ? 10 : (limit_us > 100000 ? 100000 : limit_us);
  selftest_bounded_wait_kernel<<<1, 128, 0, (cudaStream_t)stream>>>(status, (unsigned long long)us * 1000ull);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) g_launches += 1;
  return e == cudaSuccess ? CHILL_OK : cuda_fail(e, "selftest launch");
}

int chill_mask_traits(int32_t mask_id) {
  CHILL_MASK_SWITCH(mask_id, return traits_of<MaskT>())
  return CHILL_E_UNSUPPORTED;
}

unsigned long long chill_launch_count(void) { return g_launches.load(); }

int chill_read_device_status(void) {
  int* p = device_status_ptr();
  if (p == nullptr) return CHILL_E_CUDA;
  int v = 0;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return cuda_fail(e, "synchronize");
  e = cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return cuda_fail(e, "status read");
  if (v != 0) {
    int zero = 0;
    cudaMemcpy(p, &zero, sizeof(int), cudaMemcpyHostToDevice);
  }
  return v;
}

}  // extern "C"
