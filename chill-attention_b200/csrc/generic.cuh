// Generic (CUDA-core, fp32 arithmetic) kernels: any dtype, any head dim <= 256, any strides.
//
// They serve every call the tensor-core kernels cannot take (fp32 inputs with IEEE
// precision, head dims other than 64/128, channel stride != 1, misaligned strides) so the
// operator has no host fallback.  One warp owns one output row; the other axis is walked in
// chunks of 32 positions, one per lane, clipped by the mask functor's range function.
//
//   fwd_generic_kernel     O, LSE          (reference math: chill_attention/chill_fwd.py:188-359)
//   delta_kernel           delta           (chill_attention/utils.py:93-217)
//   bwd_dq_generic_kernel  dQ              (chill_attention/chill_bwd_dq.py:15-229)
//   bwd_dkdv_generic_kernel dK, dV         (chill_attention/chill_bwd_dkdv.py:15-277)
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math_constants.h>

#include "masks.cuh"

namespace chill {

struct TRef {
  void* p;
  long long sb, sh, sl, sd;  // element strides of [batch][head][position][channel]
};

struct Geo {
  int B, H, Hkv, Lq, Lk, D;
  int q_off, k_off, seq_len;
  float scale;
  const int* lens;
  MaskArgs margs;
};

struct FwdP {
  Geo g;
  TRef q, k, v, o;
  float* lse;
  long long lse_sb, lse_sh, lse_sl;
};

// Optional fp32 copies of the un-rounded dK (times sm_scale) and dV for the first `head` and the last `tail` key
// rows of a call: key row j < head is part row j, key row j >= Lk - tail is part row head + j - (Lk - tail).
struct PartOut {
  float *dk = nullptr, *dv = nullptr;
  long long sb = 0, sh = 0, sl = 0;  // element strides of [batch][kv head][part row]; channels are contiguous
  int head = 0, tail = 0;
  // address of the part row of key row j in tensor `t` (dk or dv), or nullptr if the row is outside both windows
  __device__ __forceinline__ float* row(float* t, int b, int hk, int j, int Lk) const {
    if (t == nullptr || j >= Lk) return nullptr;
    int pr;
    if (j < head) pr = j;
    else if (j >= Lk - tail) pr = head + j - (Lk - tail);
    else return nullptr;
    return t + b * sb + hk * sh + pr * sl;
  }
};

struct BwdP {
  Geo g;
  TRef q, k, v, o, d_o, dq, dk, dv;
  const float* lse;
  long long lse_sb, lse_sh, lse_sl;
  float* delta;  // contiguous [B][H][Lq]
  PartOut part;
};

constexpr float kLog2e = 1.4426950408889634f;
constexpr int kGenericWarps = 4;
constexpr int kMaxD = 256;

__device__ __forceinline__ float to_f(float x) { return x; }
__device__ __forceinline__ float to_f(__half x) { return __half2float(x); }
__device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T>
__device__ __forceinline__ T from_f(float x);
template <>
__device__ __forceinline__ float from_f<float>(float x) { return x; }
template <>
__device__ __forceinline__ __half from_f<__half>(float x) { return __float2half_rn(x); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

template <typename T>
__device__ __forceinline__ const T* row_ptr(const TRef& t, int b, int h, int l) {
  return reinterpret_cast<const T*>(t.p) + b * t.sb + h * t.sh + l * t.sl;
}
template <typename T>
__device__ __forceinline__ T* row_ptr_w(const TRef& t, int b, int h, int l) {
  return reinterpret_cast<T*>(t.p) + b * t.sb + h * t.sh + l * t.sl;
}

__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

__device__ __forceinline__ int valid_len(const Geo& g, int b) {
  int n = g.seq_len;
  if (g.lens != nullptr) n = imin(n, g.lens[b]);
  return n;
}

template <typename T>
__device__ __forceinline__ float dot_row(const float* s, const T* x, long long sd, int D) {
  float acc = 0.f;
  for (int d = 0; d < D; ++d) acc = fmaf(s[d], to_f(x[d * sd]), acc);
  return acc;
}

// ------------------------------------------------------------------------------- forward
template <typename T, class M>
__global__ void __launch_bounds__(kGenericWarps * 32) fwd_generic_kernel(FwdP p) {
  __shared__ float qs[kGenericWarps][kMaxD];
  const Geo& g = p.g;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * kGenericWarps + warp;
  const int h = blockIdx.y, b = blockIdx.z;
  if (row >= g.Lq) return;
  const int hk = h / (g.H / g.Hkv);
  const int n = valid_len(g, b);
  const int qg = row + g.q_off;
  const int D = g.D;
  T* orow = row_ptr_w<T>(p.o, b, h, row);
  if (qg >= n) {  // padded query row
    for (int d = lane; d < D; d += 32) orow[d * p.o.sd] = from_f<T>(0.f);
    if (p.lse != nullptr && lane == 0) p.lse[b * p.lse_sb + h * p.lse_sh + row * p.lse_sl] = 0.f;
    return;
  }
  const T* qrow = row_ptr<T>(p.q, b, h, row);
  for (int d = lane; d < D; d += 32) qs[warp][d] = to_f(qrow[d * p.q.sd]);
  __syncwarp();

  int lo, hi;
  M::k_range_for_q(qg, n, g.margs, lo, hi);
  const int jlo = imax(lo - g.k_off, 0);
  const int jhi = imin(imin(hi, n - 1) - g.k_off, g.Lk - 1);
  const float c = g.scale * kLog2e;

  float m = -CUDART_INF_F, l = 0.f;
  float acc[kMaxD / 32];
#pragma unroll
  for (int t = 0; t < kMaxD / 32; ++t) acc[t] = 0.f;

  for (int j0 = jlo; j0 <= jhi; j0 += 32) {
    const int j = j0 + lane;
    const bool ok = (j <= jhi) && M::mask(qg, j + g.k_off, n, g.margs);
    float s = -CUDART_INF_F;
    if (ok) s = dot_row<T>(qs[warp], row_ptr<T>(p.k, b, hk, j), p.k.sd, D) * c;
    const float m_new = fmaxf(m, warp_max(s));
    const float m_safe = (m_new == -CUDART_INF_F) ? 0.f : m_new;
    const float alpha = exp2f(m - m_safe);
    const float pj = ok ? exp2f(s - m_safe) : 0.f;
    l = l * alpha + warp_sum(pj);
#pragma unroll
    for (int t = 0; t < kMaxD / 32; ++t) acc[t] *= alpha;
    const int cnt = imin(32, jhi - j0 + 1);
    for (int jj = 0; jj < cnt; ++jj) {
      const float pb = __shfl_sync(0xffffffffu, pj, jj);
      if (pb != 0.f) {
        const T* vrow = row_ptr<T>(p.v, b, hk, j0 + jj);
#pragma unroll
        for (int t = 0; t < kMaxD / 32; ++t) {
          const int d = lane + 32 * t;
          if (d < D) acc[t] = fmaf(pb, to_f(vrow[d * p.v.sd]), acc[t]);
        }
      }
    }
    m = m_new;
  }
  const float l_safe = (l == 0.f) ? 1.f : l;
  const float inv = 1.f / l_safe;
#pragma unroll
  for (int t = 0; t < kMaxD / 32; ++t) {
    const int d = lane + 32 * t;
    if (d < D) orow[d * p.o.sd] = from_f<T>(acc[t] * inv);
  }
  if (p.lse != nullptr && lane == 0) p.lse[b * p.lse_sb + h * p.lse_sh + row * p.lse_sl] = m + log2f(l_safe);
}

// --------------------------------------------------------------------------------- delta
// delta[b,h,t] = sum_d O*dO in fp32; one warp per row, every row (no `lens`), like the reference.
template <typename T>
__global__ void __launch_bounds__(kGenericWarps * 32) delta_kernel(TRef o, TRef d_o, float* delta, int H, int Lq, int D,
                                                                   const float* dlse, long long dl_sb, long long dl_sh, long long dl_sl) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * kGenericWarps + warp;
  const int h = blockIdx.y, b = blockIdx.z;
  if (row >= Lq) return;
  const T* orow = row_ptr<T>(o, b, h, row);
  const T* drow = row_ptr<T>(d_o, b, h, row);
  float acc = 0.f;
  for (int d = lane; d < D; d += 32) acc = fmaf(to_f(orow[d * o.sd]), to_f(drow[d * d_o.sd]), acc);
  acc = warp_sum(acc);
  if (dlse != nullptr) acc -= kLog2e * dlse[b * dl_sb + h * dl_sh + row * dl_sl];  // gradient through the returned LSE
  if (lane == 0) delta[((long long)b * H + h) * Lq + row] = acc;
}

// Contiguous 16-bit rows of 64 or 128 channels: 8 lanes x 16 B (D=64) or 16 lanes x 16 B cover one
// row, so a warp streams 4 or 2 rows per step.  Bandwidth-bound: 2 reads of B*H*L*D elements.
template <typename T, int D>
__global__ void __launch_bounds__(256) delta_rows16_kernel(const T* __restrict__ o, const T* __restrict__ d_o,
                                                           float* __restrict__ delta, long long o_sb, long long o_sh,
                                                           long long o_sl, long long do_sb, long long do_sh,
                                                           long long do_sl, int H, int Lq, const float* __restrict__ dlse,
                                                           long long dl_sb, long long dl_sh, long long dl_sl) {
  constexpr int LPR = D / 8;  // lanes per row
  constexpr int RPW = 32 / LPR;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane / LPR, li = lane % LPR;
  const int h = blockIdx.y, b = blockIdx.z;
  const int row = (blockIdx.x * 8 + warp) * RPW + sub;
  float acc = 0.f;
  if (row < Lq) {
    const uint4 a = *reinterpret_cast<const uint4*>(o + b * o_sb + h * o_sh + row * o_sl + li * 8);
    const uint4 c = *reinterpret_cast<const uint4*>(d_o + b * do_sb + h * do_sh + row * do_sl + li * 8);
    const T* pa = reinterpret_cast<const T*>(&a);
    const T* pc = reinterpret_cast<const T*>(&c);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc = fmaf(to_f(pa[i]), to_f(pc[i]), acc);
  }
#pragma unroll
  for (int ofs = LPR / 2; ofs > 0; ofs >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, ofs);
  if (row < Lq && li == 0) {
    if (dlse != nullptr) acc -= kLog2e * dlse[b * dl_sb + h * dl_sh + row * dl_sl];  // gradient through the returned LSE
    delta[((long long)b * H + h) * Lq + row] = acc;
  }
}

// ------------------------------------------------------------------------------ backward
template <typename T, class M>
__global__ void __launch_bounds__(kGenericWarps * 32) bwd_dq_generic_kernel(BwdP p) {
  __shared__ float qs[kGenericWarps][kMaxD];
  __shared__ float ds_[kGenericWarps][kMaxD];
  const Geo& g = p.g;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * kGenericWarps + warp;
  const int h = blockIdx.y, b = blockIdx.z;
  if (row >= g.Lq) return;
  const int hk = h / (g.H / g.Hkv);
  const int n = valid_len(g, b);
  const int qg = row + g.q_off;
  const int D = g.D;
  T* dqrow = row_ptr_w<T>(p.dq, b, h, row);
  if (qg >= n) {
    for (int d = lane; d < D; d += 32) dqrow[d * p.dq.sd] = from_f<T>(0.f);
    return;
  }
  const T* qrow = row_ptr<T>(p.q, b, h, row);
  const T* dorow = row_ptr<T>(p.d_o, b, h, row);
  for (int d = lane; d < D; d += 32) {
    qs[warp][d] = to_f(qrow[d * p.q.sd]);
    ds_[warp][d] = to_f(dorow[d * p.d_o.sd]);
  }
  __syncwarp();
  float lse = p.lse[b * p.lse_sb + h * p.lse_sh + row * p.lse_sl];
  if (lse == -CUDART_INF_F) lse = 0.f;
  const float delta = p.delta[((long long)b * g.H + h) * g.Lq + row];

  int lo, hi;
  M::k_range_for_q(qg, n, g.margs, lo, hi);
  const int jlo = imax(lo - g.k_off, 0);
  const int jhi = imin(imin(hi, n - 1) - g.k_off, g.Lk - 1);
  const float c = g.scale * kLog2e;
  float acc[kMaxD / 32];
#pragma unroll
  for (int t = 0; t < kMaxD / 32; ++t) acc[t] = 0.f;

  for (int j0 = jlo; j0 <= jhi; j0 += 32) {
    const int j = j0 + lane;
    const bool ok = (j <= jhi) && M::mask(qg, j + g.k_off, n, g.margs);
    float ds = 0.f;
    if (ok) {
      const float s = dot_row<T>(qs[warp], row_ptr<T>(p.k, b, hk, j), p.k.sd, D) * c;
      const float pj = exp2f(s - lse);
      const float dp = dot_row<T>(ds_[warp], row_ptr<T>(p.v, b, hk, j), p.v.sd, D);
      ds = pj * (dp - delta);
    }
    const int cnt = imin(32, jhi - j0 + 1);
    for (int jj = 0; jj < cnt; ++jj) {
      const float dsb = __shfl_sync(0xffffffffu, ds, jj);
      if (dsb != 0.f) {
        const T* krow = row_ptr<T>(p.k, b, hk, j0 + jj);
#pragma unroll
        for (int t = 0; t < kMaxD / 32; ++t) {
          const int d = lane + 32 * t;
          if (d < D) acc[t] = fmaf(dsb, to_f(krow[d * p.k.sd]), acc[t]);
        }
      }
    }
  }
#pragma unroll
  for (int t = 0; t < kMaxD / 32; ++t) {
    const int d = lane + 32 * t;
    if (d < D) dqrow[d * p.dq.sd] = from_f<T>(acc[t] * g.scale);
  }
}

template <typename T, class M>
__global__ void __launch_bounds__(kGenericWarps * 32) bwd_dkdv_generic_kernel(BwdP p) {
  __shared__ float ks[kGenericWarps][kMaxD];
  __shared__ float vs[kGenericWarps][kMaxD];
  const Geo& g = p.g;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j = blockIdx.x * kGenericWarps + warp;
  const int hk = blockIdx.y, b = blockIdx.z;
  if (j >= g.Lk) return;
  const int G = g.H / g.Hkv;
  const int n = valid_len(g, b);
  const int kg = j + g.k_off;
  const int D = g.D;
  T* dkrow = row_ptr_w<T>(p.dk, b, hk, j);
  T* dvrow = row_ptr_w<T>(p.dv, b, hk, j);
  float* dkpart = p.part.row(p.part.dk, b, hk, j, g.Lk);
  float* dvpart = p.part.row(p.part.dv, b, hk, j, g.Lk);
  if (kg >= n) {
    for (int d = lane; d < D; d += 32) {
      dkrow[d * p.dk.sd] = from_f<T>(0.f);
      dvrow[d * p.dv.sd] = from_f<T>(0.f);
      if (dkpart != nullptr) dkpart[d] = dvpart[d] = 0.f;
    }
    return;
  }
  const T* krow = row_ptr<T>(p.k, b, hk, j);
  const T* vrow = row_ptr<T>(p.v, b, hk, j);
  for (int d = lane; d < D; d += 32) {
    ks[warp][d] = to_f(krow[d * p.k.sd]);
    vs[warp][d] = to_f(vrow[d * p.v.sd]);
  }
  __syncwarp();
  int lo, hi;
  M::q_range_for_k(kg, n, g.margs, lo, hi);
  const int ilo = imax(lo - g.q_off, 0);
  const int ihi = imin(imin(hi, n - 1) - g.q_off, g.Lq - 1);
  const float c = g.scale * kLog2e;
  float acck[kMaxD / 32], accv[kMaxD / 32];
#pragma unroll
  for (int t = 0; t < kMaxD / 32; ++t) acck[t] = accv[t] = 0.f;

  for (int gi = 0; gi < G; ++gi) {
    const int h = hk * G + gi;
    for (int i0 = ilo; i0 <= ihi; i0 += 32) {
      const int i = i0 + lane;
      const bool ok = (i <= ihi) && M::mask(i + g.q_off, kg, n, g.margs);
      float pi = 0.f, ds = 0.f;
      if (ok) {
        float lse = p.lse[b * p.lse_sb + h * p.lse_sh + i * p.lse_sl];
        if (lse == -CUDART_INF_F) lse = 0.f;
        const float s = dot_row<T>(ks[warp], row_ptr<T>(p.q, b, h, i), p.q.sd, D) * c;
        pi = exp2f(s - lse);
        const float dp = dot_row<T>(vs[warp], row_ptr<T>(p.d_o, b, h, i), p.d_o.sd, D);
        ds = pi * (dp - p.delta[((long long)b * g.H + h) * g.Lq + i]);
      }
      const int cnt = imin(32, ihi - i0 + 1);
      for (int ii = 0; ii < cnt; ++ii) {
        const float pb = __shfl_sync(0xffffffffu, pi, ii);
        const float dsb = __shfl_sync(0xffffffffu, ds, ii);
        if (pb != 0.f || dsb != 0.f) {
          const T* qrow = row_ptr<T>(p.q, b, h, i0 + ii);
          const T* dorow = row_ptr<T>(p.d_o, b, h, i0 + ii);
#pragma unroll
          for (int t = 0; t < kMaxD / 32; ++t) {
            const int d = lane + 32 * t;
            if (d < D) {
              accv[t] = fmaf(pb, to_f(dorow[d * p.d_o.sd]), accv[t]);
              acck[t] = fmaf(dsb, to_f(qrow[d * p.q.sd]), acck[t]);
            }
          }
        }
      }
    }
  }
#pragma unroll
  for (int t = 0; t < kMaxD / 32; ++t) {
    const int d = lane + 32 * t;
    if (d < D) {
      dkrow[d * p.dk.sd] = from_f<T>(acck[t] * g.scale);
      dvrow[d * p.dv.sd] = from_f<T>(accv[t]);
      if (dkpart != nullptr) {
        dkpart[d] = acck[t] * g.scale;
        dvpart[d] = accv[t];
      }
    }
  }
}

// ----------------------------------------------------------------------- mask tabulation
template <class M>
__global__ void mask_tabulate_kernel(MaskArgs a, int n, int tile, uint8_t* dense, int* k_lims, int* q_lims,
                                     int* k_full, int* q_full) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (dense != nullptr && idx < (long long)n * n) {
    const int q = (int)(idx / n), k = (int)(idx % n);
    dense[idx] = M::mask(q, k, n, a) ? 1 : 0;
  }
  if (idx < n) {
    int lo, hi;
    if (k_lims != nullptr) {
      M::k_range_for_q((int)idx, n, a, lo, hi);
      k_lims[2 * idx] = lo;
      k_lims[2 * idx + 1] = hi;
    }
    if (q_lims != nullptr) {
      M::q_range_for_k((int)idx, n, a, lo, hi);
      q_lims[2 * idx] = lo;
      q_lims[2 * idx + 1] = hi;
    }
  }
  const int ntiles = (n + tile - 1) / tile;
  if (idx < ntiles) {
    int lo, hi;
    if (k_full != nullptr) {
      M::k_full_range_for_q((int)idx * tile, tile, n, a, lo, hi);
      k_full[2 * idx] = lo;
      k_full[2 * idx + 1] = hi;
    }
    if (q_full != nullptr) {
      M::q_full_range_for_k((int)idx * tile, tile, n, a, lo, hi);
      q_full[2 * idx] = lo;
      q_full[2 * idx + 1] = hi;
    }
  }
}

template <class M>
__global__ void mask_tabulate_blocks_kernel(MaskArgs a, int n, int q_tile, int k_tile, uint8_t* full) {
  const int nq = (n + q_tile - 1) / q_tile, nk = (n + k_tile - 1) / k_tile;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx < (long long)nq * nk) {
    const int qi = (int)(idx / nk), ki = (int)(idx % nk);
    full[idx] = M::is_full_block(qi * q_tile, ki * k_tile, q_tile, k_tile, n, a) ? 1 : 0;
  }
}

}  // namespace chill
