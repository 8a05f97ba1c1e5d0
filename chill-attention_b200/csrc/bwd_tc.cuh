// Backward attention on tcgen05 tensor cores (sm_100a), 16-bit inputs, head dim 64 or 128.
//
// Two kernels, both with every MMA operand that the softmax math produces kept in TMEM
// (no shared-memory round trip for P or dS) and no atomics, so results are deterministic:
//
//   bwd_dkdv_tc_kernel  one CTA per (batch, kv head, tile of 128 keys).  K and V stay in shared
//       memory; Q / dO tiles of every query tile that can see the key tile (functor's
//       q_range_for_k) and of every head of the GQA group stream through a 2-stage TMA ring.
//       Per query tile:  S^T = K Q^T, dP^T = V dO^T  (TMEM, fp32)
//                        P^T = 2^(S^T c - LSE),  dS^T = P^T (dP^T - delta)   (registers -> TMEM, 16-bit)
//                        dV += P^T dO,  dK += dS^T Q   (A from TMEM, B = dO / Q MN-major)
//       Reference math: chill_attention/chill_bwd_dkdv.py:347-508.
//
//   bwd_dq_tc_kernel    one CTA per (batch, head, tile of 128 queries).  Q and dO stay in shared
//       memory; K / V tiles from the functor's k_range_for_q stream through the ring.
//       Per key tile:    S = Q K^T, dP = dO V^T;  dS = 2^(S c - LSE) (dP - delta);  dQ += dS K.
//       Reference math: chill_attention/chill_bwd_dq.py:300-394.
//
// Roles in both (320 threads): warps 0-7 do the exponentials (thread (w % 4) * 32 + lane owns
// TMEM lane = tile row; warps 0-3 and warps 4-7 split the columns), warp 8 is the TMA producer
// and owns the TMEM allocation, warp 9 issues the MMAs.  Every MMA runs at full width (N = 128 or D):
// tcgen05.mma at N = 64 takes as long as at N = 128 on this part.
#pragma once
#include <type_traits>

#include "fwd_tc.cuh"
#include "generic.cuh"
#include "tc_common.cuh"
#include "tc_launch.h"

namespace chill {
namespace tc {

constexpr int kBwdThreads = 320;
constexpr int kBwdComputeThreads = 256;
constexpr int kTmemColsBwd = 512;
constexpr bool kHaveBwdTc = true;
constexpr int kWideCols = 64;  // head dim 256 (bwd_wide.cuh): positions of the streamed axis per step = rows of its TMA boxes

struct BwdTcParams {
  Geo g;
  const float* lse;
  long long lse_sb, lse_sh, lse_sl;
  const float* delta;  // [B][H][Lq]
  void *dq, *dk, *dv;  // for zero-filling tiles that are entirely padding
  long long dq_sb, dq_sh, dq_sl, dk_sb, dk_sh, dk_sl, dv_sb, dv_sh, dv_sl;
  int* status;
  int which;  // bit0: launch the dK/dV kernel, bit1: launch the dQ kernel
  float* dq_accum;  // fp32 accumulator of the single-kernel backward (bwd_fused.cuh), else nullptr
  PartOut part;     // optional un-rounded fp32 copies of dK / dV rows
};

// fp32 dQ accumulator of the single-kernel backward (bwd_fused.cuh): one block of 128 rows x D channels per
// (batch, head, query tile), stored as [4 row groups][D / 4][32 rows][4 channels]: the part a drain warp owns
// (32 rows) is contiguous, and so is every run of channel groups inside it, so it leaves the SM as bulk reductions.
__host__ __device__ inline size_t dq_accum_bytes(int B, int H, int Lq, int D) {
  return (size_t)B * H * ((Lq + kTile - 1) / kTile) * kTile * D * sizeof(float);
}

template <int D>
struct BwdSmem {
  static constexpr int kTileBytes = kTile * D * 2;
  static constexpr int kStages = 2;
  static constexpr int kFixA = 0;                      // K (dkdv) or Q (dq)
  static constexpr int kFixB = kFixA + kTileBytes;     // V (dkdv) or dO (dq)
  static constexpr int kRing = kFixB + kTileBytes;     // per stage: [Q | dO] (dkdv) or [K | V] (dq)
  static constexpr int kRows = kRing + kStages * 2 * kTileBytes;  // per compute warp: lse[64], delta[64] floats
  static constexpr int kBars = kRows + 8 * 2 * 64 * 4;
  static constexpr int kNumBars = 6 + 2 * kStages;
  static constexpr int kMisc = kBars + 8 * kNumBars;
  static constexpr int kTotal = kMisc + 16;
  static constexpr int kDynamic = kTotal + 1024;
};

enum : int {
  kStBwdProducer = 201, kStBwdMma = 202, kStBwdCompute = 203, kStBwdEpilogue = 204,
  kStDqProducer = 301, kStDqMma = 302, kStDqCompute = 303, kStDqEpilogue = 304
};

// Zero `rows` rows of D 16-bit channels starting at `base` (row stride `sl` elements).
template <typename T, int D>
__device__ __forceinline__ void zero_rows(T* base, long long sl, int rows, int nthreads) {
  for (int idx = threadIdx.x; idx < rows * (D / 8); idx += nthreads) {
    const int r = idx / (D / 8), c = idx % (D / 8);
    *reinterpret_cast<uint4*>(base + r * sl + c * 8) = make_uint4(0, 0, 0, 0);
  }
}

// Convert 32 fp32 accumulator columns [col0, col0+32) of this thread's row to 16-bit and put them
// into the row's 128-byte lines of a 128B-swizzled staging tile (layout of a TMA box).
template <typename T>
__device__ __forceinline__ void stage_row32(uint8_t* tile, int r, int q4, const uint32_t* acc, float mul, bool keep) {
  uint32_t packed[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float a = keep ? __uint_as_float(acc[2 * i]) * mul : 0.f;
    const float b = keep ? __uint_as_float(acc[2 * i + 1]) * mul : 0.f;
    packed[i] = pack2<T>(a, b);
  }
  uint8_t* line = tile + (q4 / 2) * (kTile * 128) + r * 128;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int unit = ((q4 % 2) * 4 + u) ^ (r & 7);
    *reinterpret_cast<uint4*>(line + unit * 16) =
        make_uint4(packed[4 * u], packed[4 * u + 1], packed[4 * u + 2], packed[4 * u + 3]);
  }
}

// 32 un-rounded fp32 values (accumulator * mul, or zeros) of this thread's key row to the partial-output tensor.
__device__ __forceinline__ void store_part32(float* dst, const uint32_t* acc, float mul, bool keep) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (keep)
      v = make_float4(__uint_as_float(acc[4 * i]) * mul, __uint_as_float(acc[4 * i + 1]) * mul,
                      __uint_as_float(acc[4 * i + 2]) * mul, __uint_as_float(acc[4 * i + 3]) * mul);
    *reinterpret_cast<float4*>(dst + 4 * i) = v;
  }
}

// Zero the partial-output rows that belong to key rows [kb, kb + rows) of (b, hk).
template <int D>
__device__ __forceinline__ void zero_part_rows(const PartOut& part, int b, int hk, int kb, int rows, int Lk, int nthreads) {
  if (part.dk == nullptr) return;
  for (int idx = threadIdx.x; idx < rows * (D / 4); idx += nthreads) {
    const int r = idx / (D / 4), c = idx % (D / 4);
    float* a = part.row(part.dk, b, hk, kb + r, Lk);
    float* bb = part.row(part.dv, b, hk, kb + r, Lk);
    if (a != nullptr) {
      *reinterpret_cast<float4*>(a + 4 * c) = make_float4(0.f, 0.f, 0.f, 0.f);
      *reinterpret_cast<float4*>(bb + 4 * c) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
}

// =========================================================================== dK / dV
// TMEM: S^T (128 columns, overlaid by the 16-bit P^T), dP^T (128, overlaid by dS^T), dV, dK: 512 columns,
// every MMA at N = 128.  Tensor-core order in steady state (u = query tile):
//     dV += P^T(u) dO(u)      needs P^T(u)
//     S^T(u+1) = K Q(u+1)^T
//     dK += dS^T(u) Q(u)      needs dS^T(u)
//     dP^T(u+1) = V dO(u+1)^T
// The compute warps work in two steps per tile: the exponentials P^T = 2^(S^T c - LSE) as soon as S^T is
// there (while the tensor cores run dK(u-1) and dP^T(u)), then dS^T = P^T (dP^T - delta) once dP^T has
// landed (while dV(u) and S^T(u+1) run).  The MUFU-heavy step is thereby off the tensor cores' critical path.
template <typename T, int D, class M>
__global__ void __launch_bounds__(kBwdThreads, 1)
bwd_dkdv_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                   const __grid_constant__ CUtensorMap tmdK, const __grid_constant__ CUtensorMap tmdV, BwdTcParams p) {
  using L = BwdSmem<D>;
  constexpr int kChunks = D / 64;
  constexpr int kChunkBytes = kTile * 128;
  const Geo& g = p.g;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int hb, kt;
  cta_order((int)blockIdx.x, g.B * g.Hkv, (g.Lk + kTile - 1) / kTile, hb, kt);  // first key tile = most query tiles (causal)
  const int hk = hb % g.Hkv, b = hb / g.Hkv;
  const int G = g.H / g.Hkv;
  const int kb = kt * kTile;
  const int kg0 = kb + g.k_off;
  int n = g.seq_len;
  if (g.lens != nullptr) n = imin(n, g.lens[b]);

  // query-tile range that can see this key tile
  int qt_lo = 0, qt_hi = 0, full_lo = 0, full_hi = 0;
  if (kg0 < n) {
    int lo, hi;
    tile_range<M, false>(kg0, imin(kTile, g.Lk - kb), n, g.margs, lo, hi);
    const int lo_l = imax(lo - g.q_off, 0);
    const int hi_l = imin(imin(hi, n - 1) - g.q_off, g.Lq - 1);
    if (hi_l >= lo_l) {
      qt_lo = lo_l / kTile;
      qt_hi = hi_l / kTile + 1;
    }
    if (M::kHasQFullRange) M::q_full_range_for_k(kg0, kTile, n, g.margs, full_lo, full_hi);
  }
  const int n_qt = qt_hi - qt_lo;
  const int n_it = n_qt * G;
  if (n_it == 0) {
    // nobody attends these keys (padding, or outside every query's range on this shard)
    const int rows = imin(kTile, g.Lk - kb);
    zero_rows<T, D>(reinterpret_cast<T*>(p.dk) + b * p.dk_sb + hk * p.dk_sh + kb * p.dk_sl, p.dk_sl, rows, kBwdThreads);
    zero_rows<T, D>(reinterpret_cast<T*>(p.dv) + b * p.dv_sb + hk * p.dv_sh + kb * p.dv_sl, p.dv_sl, rows, kBwdThreads);
    zero_part_rows<D>(p.part, b, hk, kb, rows, g.Lk, kBwdThreads);
    return;
  }

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t sK = base + L::kFixA, sV = base + L::kFixB, sRing = base + L::kRing;
  float* rows_s = reinterpret_cast<float*>(gen_base + L::kRows);  // [warp][0: -lse, 1: -delta][64]
  const uint32_t bars = base + L::kBars;
  const uint32_t bar_kv_full = bars, bar_acc_full = bars + 8, bar_s_full = bars + 16, bar_dp_full = bars + 24,
                 bar_p_full = bars + 32, bar_ds_full = bars + 40;
  const uint32_t bar_ring_full = bars + 48, bar_ring_empty = bar_ring_full + 8 * L::kStages;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen_base + L::kMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + L::kMisc + 4);
  const Guard guard{p.status, abort_flag};

  if (warp == 8) {
    // The producer thread initialises the barriers itself and puts K, V and the first Q/dO tile in flight
    // before the CTA-wide set-up (TMEM allocation, __syncthreads) completes.
    if (lane == 0) {
      *abort_flag = 0;
      mbar_init(bar_kv_full, 1);
      mbar_init(bar_acc_full, 1);
      mbar_init(bar_s_full, 1);
      mbar_init(bar_dp_full, 1);
      mbar_init(bar_p_full, kBwdComputeThreads / 32);
      mbar_init(bar_ds_full, kBwdComputeThreads / 32);
      for (int s = 0; s < L::kStages; ++s) {
        mbar_init(bar_ring_full + 8 * s, 1);
        mbar_init(bar_ring_empty + 8 * s, 1);
      }
      fence_barrier_init();
      fence_proxy_async_smem();
      mbar_arrive_expect_tx(bar_kv_full, 2 * L::kTileBytes);
      for (int c = 0; c < kChunks; ++c) {
        tma_load_4d(sK + c * kChunkBytes, &tmK, bar_kv_full, c * 64, kb, hk, b);
        tma_load_4d(sV + c * kChunkBytes, &tmV, bar_kv_full, c * 64, kb, hk, b);
      }
      mbar_arrive_expect_tx(bar_ring_full, 2 * L::kTileBytes);
      for (int c = 0; c < kChunks; ++c) {
        tma_load_4d(sRing + c * kChunkBytes, &tmQ, bar_ring_full, c * 64, qt_lo * kTile, hk * G, b);
        tma_load_4d(sRing + L::kTileBytes + c * kChunkBytes, &tmdO, bar_ring_full, c * 64, qt_lo * kTile, hk * G, b);
      }
    }
    __syncwarp();
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemColsBwd);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tSt = tmem, tdPt = tmem + 128, tdV = tmem + 256, tdK = tmem + 384;

  if (warp == 8) {
    // --------------------------------------------------------------------- TMA producer
    if (lane == 0) {
      bool ok = true;
      for (int it = 1; it < n_it; ++it) {  // tile 0 was issued during set-up
        const int s = it % L::kStages;
        const uint32_t ph = (uint32_t)(it / L::kStages) & 1u;
        const int h = hk * G + it / n_qt;
        const int qrow = (qt_lo + it % n_qt) * kTile;
        ok = mbar_wait(bar_ring_empty + 8 * s, ph ^ 1u, guard, kStBwdProducer);
        if (!ok) break;
        mbar_arrive_expect_tx(bar_ring_full + 8 * s, 2 * L::kTileBytes);
        const uint32_t dst = sRing + s * 2 * L::kTileBytes;
        for (int c = 0; c < kChunks; ++c) {
          tma_load_4d(dst + c * kChunkBytes, &tmQ, bar_ring_full + 8 * s, c * 64, qrow, h, b);
          tma_load_4d(dst + L::kTileBytes + c * kChunkBytes, &tmdO, bar_ring_full + 8 * s, c * 64, qrow, h, b);
        }
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 9) {
    // ----------------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc<T>(kTile, kTile, false, false);
      constexpr uint32_t idesc_acc = make_idesc<T>(kTile, D, false, true);
      constexpr uint32_t hi_k = desc_hi_sw128(1024);
      const uint32_t k_lo = desc_lo_sw128(sK, 16), v_lo = desc_lo_sw128(sV, 16);
      bool ok = mbar_wait(bar_kv_full, 0, guard, kStBwdMma);
      auto stage_q = [&](int it) { return sRing + (it % L::kStages) * 2 * L::kTileBytes; };
      auto issue_s = [&](int it) -> bool {  // S^T(it) = K Q^T; first user of ring stage `it`
        const int s = it % L::kStages;
        if (!mbar_wait(bar_ring_full + 8 * s, (uint32_t)(it / L::kStages) & 1u, guard, kStBwdMma)) return false;
        tc_fence_after();
        const uint32_t q_lo = desc_lo_sw128(stage_q(it), 16);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_ss_lh(tSt, k_lo + kmajor_step(kk), q_lo + kmajor_step(kk), hi_k, idesc_s, kk > 0);
        mma_commit(bar_s_full);
        return true;
      };
      auto issue_dp = [&](int it) {  // dP^T(it) = V dO^T
        const uint32_t do_lo = desc_lo_sw128(stage_q(it) + L::kTileBytes, 16);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_ss_lh(tdPt, v_lo + kmajor_step(kk), do_lo + kmajor_step(kk), hi_k, idesc_s, kk > 0);
        mma_commit(bar_dp_full);
      };
      if (ok) ok = issue_s(0);
      if (ok) issue_dp(0);
      for (int it = 0; it < n_it && ok; ++it) {
        const uint32_t par = (uint32_t)it & 1u;
        const uint32_t qmn_lo = desc_lo_sw128(stage_q(it), kChunkBytes);
        const uint32_t domn_lo = desc_lo_sw128(stage_q(it) + L::kTileBytes, kChunkBytes);
        ok = mbar_wait(bar_p_full, par, guard, kStBwdMma);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk)  // dV += P^T dO   (16 queries per step)
          mma_ts_lh(tdV, tSt + (kk / 4) * 64 + (kk % 4) * 8, domn_lo + kk * 128, hi_k, idesc_acc, (it > 0 || kk > 0));
        if (it + 1 < n_it) {
          ok = issue_s(it + 1);  // overwrites P^T(it) only after dV(it) has read it (MMAs complete in order)
          if (!ok) break;
        }
        ok = mbar_wait(bar_ds_full, par, guard, kStBwdMma);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk)  // dK += dS^T Q
          mma_ts_lh(tdK, tdPt + (kk / 4) * 64 + (kk % 4) * 8, qmn_lo + kk * 128, hi_k, idesc_acc, (it > 0 || kk > 0));
        mma_commit(bar_ring_empty + 8 * (it % L::kStages));
        if (it + 1 < n_it) issue_dp(it + 1);
      }
      if (ok) mma_commit(bar_acc_full);
    }
  } else {
    // ------------------------------------------------------------------- compute warps
    const int wg = warp >> 2;                       // column half: query columns [64 wg, 64 wg + 64)
    const int r = (warp & 3) * 32 + lane;           // key row inside the tile == TMEM lane
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
    const int c0 = wg * 64;
    const int kg = kg0 + r;
    const bool key_ok = kg < n && kb + r < g.Lk;
    const float c = g.scale * kLog2e;
    const uint64_t c2 = pk2(c, c);
    const int t = threadIdx.x;  // 0..255
    float* slot = rows_s + warp * 128;  // warp-private: [0,64) -LSE, [64,128) -delta of this warp's columns
    bool ok = true;
    // LSE / delta of this lane's two query columns of tile `it`, fetched one tile ahead.  The loaded values are
    // not touched until the next iteration (any dependent instruction here would stall on the global load).
    auto fetch_rows = [&](int it, float* lv, float* dl) {
      const int h = hk * G + it / n_qt;
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int qrow = (qt_lo + it % n_qt) * kTile + c0 + e * 32 + lane;
        const bool in = qrow < g.Lq;
        const float* pl = p.lse + b * p.lse_sb + h * p.lse_sh + (in ? qrow : 0) * p.lse_sl;
        const float* pd = p.delta + ((long long)b * g.H + h) * g.Lq + (in ? qrow : 0);
        lv[e] = __ldg(pl);  // row 0 stands in for rows beyond Lq: those columns are masked out anyway
        dl[e] = __ldg(pd);
      }
    };
    float nl_next[2], nd_next[2];
    fetch_rows(0, nl_next, nd_next);
    for (int it = 0; it < n_it; ++it) {
      const uint32_t par = (uint32_t)it & 1u;
      const int qi = qt_lo + it % n_qt;
      const int qg0 = qi * kTile + g.q_off;
      __syncwarp();
#pragma unroll
      for (int e = 0; e < 2; ++e) {  // negated: they enter the packed FMA / ADD as addends
        slot[e * 32 + lane] = (nl_next[e] == -CUDART_INF_F) ? 0.f : -nl_next[e];
        slot[64 + e * 32 + lane] = -nd_next[e];
      }
      __syncwarp();
      if (it + 1 < n_it) fetch_rows(it + 1, nl_next, nd_next);
      const bool full = M::kHasQFullRange && qg0 >= full_lo && qg0 + kTile <= full_hi && qg0 + kTile <= n &&
                        qi * kTile + kTile <= g.Lq && kg0 + kTile <= n && kb + kTile <= g.Lk;
      const int qlim = imin(n - qg0, g.Lq - qi * kTile);
      int w_lo = 0, w_hi = -1;  // visible query columns of this key row inside the tile (interval functors)
      if (interval_rows<M>::value && !full && key_ok) row_window<M, false>(kg, qg0, qlim, n, g.margs, w_lo, w_hi);

      // ---- step 1: P^T = 2^(S^T c - LSE), masked; 16-bit copy to TMEM for the dV GEMM, kept packed in registers
      ok = mbar_wait(bar_s_full, par, guard, kStBwdCompute);
      ok = __all_sync(0xffffffffu, ok);  // keep the warp converged for the .sync.aligned TMEM accesses
      if (!ok) break;
      tc_fence_after();
      uint32_t preg[32];
      {
        uint32_t sreg[64];
        tmem_ld32(tSt + lane_sel + c0, sreg);
        tmem_ld32(tSt + lane_sel + c0 + 32, sreg + 32);
        tmem_wait_ld();
        auto body = [&](auto masked_tag) {  // two copies: full tiles run without any mask arithmetic
          constexpr bool kMasked = decltype(masked_tag)::value;
#pragma unroll
          for (int j = 0; j < 16; ++j) {  // four query columns per step
            const float4 nl4 = reinterpret_cast<const float4*>(slot)[j];
            float p0, p1, p2, p3;
            upk2(ex2_pair(ffma2(pk2u(sreg[4 * j], sreg[4 * j + 1]), c2, pk2(nl4.x, nl4.y)),
                          ((2 * j) % CHILL_BWD_POLY_DEN) < CHILL_BWD_POLY_NUM), p0, p1);
            upk2(ex2_pair(ffma2(pk2u(sreg[4 * j + 2], sreg[4 * j + 3]), c2, pk2(nl4.z, nl4.w)),
                          ((2 * j + 1) % CHILL_BWD_POLY_DEN) < CHILL_BWD_POLY_NUM), p2, p3);
            if (kMasked) {
              const int cq = c0 + 4 * j;
              if (interval_rows<M>::value) {
                p0 = (cq >= w_lo && cq <= w_hi) ? p0 : 0.f;
                p1 = (cq + 1 >= w_lo && cq + 1 <= w_hi) ? p1 : 0.f;
                p2 = (cq + 2 >= w_lo && cq + 2 <= w_hi) ? p2 : 0.f;
                p3 = (cq + 3 >= w_lo && cq + 3 <= w_hi) ? p3 : 0.f;
              } else {
                p0 = (key_ok && cq < qlim && M::mask(qg0 + cq, kg, n, g.margs)) ? p0 : 0.f;
                p1 = (key_ok && cq + 1 < qlim && M::mask(qg0 + cq + 1, kg, n, g.margs)) ? p1 : 0.f;
                p2 = (key_ok && cq + 2 < qlim && M::mask(qg0 + cq + 2, kg, n, g.margs)) ? p2 : 0.f;
                p3 = (key_ok && cq + 3 < qlim && M::mask(qg0 + cq + 3, kg, n, g.margs)) ? p3 : 0.f;
              }
            }
            preg[2 * j] = pack2<T>(p0, p1);
            preg[2 * j + 1] = pack2<T>(p2, p3);
          }
        };
        if (full) body(std::false_type{});
        else body(std::true_type{});
      }
      tmem_st32(tSt + lane_sel + c0, preg);  // over the first half of the fp32 columns this warp just consumed
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p_full);

      // ---- step 2: dS^T = P^T (dP^T - delta) with the rounded P^T the dV GEMM uses
      ok = mbar_wait(bar_dp_full, par, guard, kStBwdCompute);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      {
        uint32_t dpreg[64];
        tmem_ld32(tdPt + lane_sel + c0, dpreg);
        tmem_ld32(tdPt + lane_sel + c0 + 32, dpreg + 32);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float4 nd4 = reinterpret_cast<const float4*>(slot + 64)[j];
          float p0, p1, p2, p3, d0, d1, d2, d3;
          unpack2<T>(preg[2 * j], p0, p1);
          unpack2<T>(preg[2 * j + 1], p2, p3);
          upk2(fmul2(pk2(p0, p1), fadd2(pk2u(dpreg[4 * j], dpreg[4 * j + 1]), pk2(nd4.x, nd4.y))), d0, d1);
          upk2(fmul2(pk2(p2, p3), fadd2(pk2u(dpreg[4 * j + 2], dpreg[4 * j + 3]), pk2(nd4.z, nd4.w))), d2, d3);
          preg[2 * j] = pack2<T>(d0, d1);
          preg[2 * j + 1] = pack2<T>(d2, d3);
        }
      }
      tmem_st32(tdPt + lane_sel + c0, preg);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_ds_full);
    }

    // ---- epilogue: warps 0-3 store dV, warps 4-7 store dK * sm_scale (staging = ring stage 0)
    if (ok) ok = mbar_wait(bar_acc_full, 0, guard, kStBwdEpilogue);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    uint8_t* stage = gen_base + L::kRing + wg * L::kTileBytes;
    const uint32_t tacc = wg == 0 ? tdV : tdK;
    const float mul = wg == 0 ? 1.f : g.scale;
    float* part_row = p.part.row(wg == 0 ? p.part.dv : p.part.dk, b, hk, kb + r, g.Lk);
#pragma unroll
    for (int q4 = 0; q4 < D / 32; ++q4) {
      uint32_t acc[32];
      if (ok) {
        tmem_ld32(tacc + lane_sel + q4 * 32, acc);
        tmem_wait_ld();
      }
      stage_row32<T>(stage, r, q4, acc, mul, ok && key_ok);
      if (part_row != nullptr) store_part32(part_row + q4 * 32, acc, mul, ok && key_ok);
    }
    fence_proxy_async_smem();
    named_bar_sync(1, kBwdComputeThreads);
    if (t == 0 || t == 128) {
      const CUtensorMap* map = (t == 0) ? &tmdV : &tmdK;
      for (int cc = 0; cc < kChunks; ++cc)
        tma_store_4d(map, sRing + wg * L::kTileBytes + cc * kChunkBytes, cc * 64, kb, hk, b);
      tma_store_commit();
      tma_store_wait_read();  // shared memory may be released; the global writes complete by kernel end
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 8) tmem_dealloc(tmem, kTmemColsBwd);
}

// ================================================================================ dQ
// TMEM: two full-width score buffers S[2] (fp32, 128 columns each), dP (128, overlaid by the
// 16-bit dS) and the dQ accumulator.  Every MMA runs at N = 128.  Tensor-core order per key tile u:
//   dQ += dS(u) K(u)   (in two halves, each as soon as its 64 columns of dS are in TMEM)
//   dP(u+1) = dO V(u+1)^T,   S(u+2) = Q K(u+2)^T
// The compute warps take two steps per tile, like the dK/dV kernel: P = 2^(S c - LSE) as soon as S(u+1) is
// there (it is issued a whole tile ahead, so this overlaps dQ(u) and dP(u+1)), then dS = P (dP - delta) when
// dP(u+1) has landed.  K needs three ring stages (S(u+2) is issued while K(u) is still read by the dQ GEMM),
// V two.
template <int D>
struct DqSmem {
  static constexpr int kTileBytes = kTile * D * 2;
  static constexpr int kKStages = 3, kVStages = 2;
  static constexpr int kQ = 0;
  static constexpr int kdO = kQ + kTileBytes;
  static constexpr int kK = kdO + kTileBytes;
  static constexpr int kV = kK + kKStages * kTileBytes;
  static constexpr int kBars = kV + kVStages * kTileBytes;
  static constexpr int kNumBars = 7 + 2 * kKStages + 2 * kVStages;
  static constexpr int kMisc = kBars + 8 * kNumBars;
  static constexpr int kTotal = kMisc + 16;
  static constexpr int kDynamic = kTotal + 1024;
};

template <typename T, int D, class M>
__global__ void __launch_bounds__(kBwdThreads, 1)
bwd_dq_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                 const __grid_constant__ CUtensorMap tmdQ, BwdTcParams p) {
  using L = DqSmem<D>;
  constexpr int kChunks = D / 64;
  constexpr int kChunkBytes = kTile * 128;
  const Geo& g = p.g;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt_total = (g.Lq + kTile - 1) / kTile;
  int hb, rank;
  cta_order((int)blockIdx.x, g.B * g.H, n_qt_total, hb, rank);
  const int qt = n_qt_total - 1 - rank;
  const int h = hb % g.H, b = hb / g.H;
  const int hk = h / (g.H / g.Hkv);
  const int qb = qt * kTile;
  const int qg0 = qb + g.q_off;
  int n = g.seq_len;
  if (g.lens != nullptr) n = imin(n, g.lens[b]);

  int kt_lo = 0, kt_hi = 0, full_lo = 0, full_hi = 0;
  if (qg0 < n) {
    int lo, hi;
    tile_range<M, true>(qg0, imin(kTile, g.Lq - qb), n, g.margs, lo, hi);
    const int lo_l = imax(lo - g.k_off, 0);
    const int hi_l = imin(imin(hi, n - 1) - g.k_off, g.Lk - 1);
    if (hi_l >= lo_l) {
      kt_lo = lo_l / kTile;
      kt_hi = hi_l / kTile + 1;
    }
    if (M::kHasKFullRange) M::k_full_range_for_q(qg0, kTile, n, g.margs, full_lo, full_hi);
  }
  const int n_it = kt_hi - kt_lo;
  if (n_it == 0) {
    zero_rows<T, D>(reinterpret_cast<T*>(p.dq) + b * p.dq_sb + h * p.dq_sh + qb * p.dq_sl, p.dq_sl,
                    imin(kTile, g.Lq - qb), kBwdThreads);
    return;
  }

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t sQ = base + L::kQ, sdO = base + L::kdO, sKr = base + L::kK, sVr = base + L::kV;
  const uint32_t bars = base + L::kBars;
  const uint32_t bar_q_full = bars, bar_acc_full = bars + 8, bar_s_full = bars + 16 /* [2], per S buffer */,
                 bar_p_full = bars + 32 /* [2], per column half */, bar_dp_full = bars + 48;
  const uint32_t bar_k_full = bars + 56, bar_k_empty = bar_k_full + 8 * L::kKStages;
  const uint32_t bar_v_full = bar_k_empty + 8 * L::kKStages, bar_v_empty = bar_v_full + 8 * L::kVStages;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen_base + L::kMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + L::kMisc + 4);
  const Guard guard{p.status, abort_flag};

  if (warp == 8) {
    // The producer thread initialises the barriers itself and puts Q, dO and the first K/V tile in flight
    // before the CTA-wide set-up (TMEM allocation, __syncthreads) completes.
    if (lane == 0) {
      *abort_flag = 0;
      mbar_init(bar_q_full, 1);
      mbar_init(bar_acc_full, 1);
      mbar_init(bar_s_full, 1);
      mbar_init(bar_s_full + 8, 1);
      mbar_init(bar_dp_full, 1);
      mbar_init(bar_p_full, kBwdComputeThreads / 32);
      mbar_init(bar_p_full + 8, kBwdComputeThreads / 32);
      for (int s = 0; s < L::kKStages; ++s) {
        mbar_init(bar_k_full + 8 * s, 1);
        mbar_init(bar_k_empty + 8 * s, 1);
      }
      for (int s = 0; s < L::kVStages; ++s) {
        mbar_init(bar_v_full + 8 * s, 1);
        mbar_init(bar_v_empty + 8 * s, 1);
      }
      fence_barrier_init();
      fence_proxy_async_smem();
      mbar_arrive_expect_tx(bar_q_full, 2 * L::kTileBytes);
      for (int c = 0; c < kChunks; ++c) {
        tma_load_4d(sQ + c * kChunkBytes, &tmQ, bar_q_full, c * 64, qb, h, b);
        tma_load_4d(sdO + c * kChunkBytes, &tmdO, bar_q_full, c * 64, qb, h, b);
      }
      mbar_arrive_expect_tx(bar_k_full, L::kTileBytes);
      for (int c = 0; c < kChunks; ++c) tma_load_4d(sKr + c * kChunkBytes, &tmK, bar_k_full, c * 64, kt_lo * kTile, hk, b);
      mbar_arrive_expect_tx(bar_v_full, L::kTileBytes);
      for (int c = 0; c < kChunks; ++c) tma_load_4d(sVr + c * kChunkBytes, &tmV, bar_v_full, c * 64, kt_lo * kTile, hk, b);
    }
    __syncwarp();
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemColsBwd);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem, tdP = tmem + 256, tdQ = tmem + 384;  // S buffer i at tS + 128 i

  if (warp == 8) {
    // --------------------------------------------------------------------- TMA producer
    if (lane == 0) {
      bool ok = true;
      for (int it = 1; it < n_it; ++it) {  // tile 0 was issued during set-up
        const int ks = it % L::kKStages, vs = it % L::kVStages;
        const int krow = (kt_lo + it) * kTile;
        ok = mbar_wait(bar_k_empty + 8 * ks, ((uint32_t)(it / L::kKStages) & 1u) ^ 1u, guard, kStDqProducer);
        if (!ok) break;
        mbar_arrive_expect_tx(bar_k_full + 8 * ks, L::kTileBytes);
        for (int c = 0; c < kChunks; ++c)
          tma_load_4d(sKr + ks * L::kTileBytes + c * kChunkBytes, &tmK, bar_k_full + 8 * ks, c * 64, krow, hk, b);
        ok = mbar_wait(bar_v_empty + 8 * vs, ((uint32_t)(it / L::kVStages) & 1u) ^ 1u, guard, kStDqProducer);
        if (!ok) break;
        mbar_arrive_expect_tx(bar_v_full + 8 * vs, L::kTileBytes);
        for (int c = 0; c < kChunks; ++c)
          tma_load_4d(sVr + vs * L::kTileBytes + c * kChunkBytes, &tmV, bar_v_full + 8 * vs, c * 64, krow, hk, b);
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 9) {
    // ----------------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc<T>(kTile, kTile, false, false);
      constexpr uint32_t idesc_acc = make_idesc<T>(kTile, D, false, true);
      constexpr uint32_t hi_k = desc_hi_sw128(1024);
      const uint32_t q_lo = desc_lo_sw128(sQ, 16), do_lo = desc_lo_sw128(sdO, 16);
      bool ok = mbar_wait(bar_q_full, 0, guard, kStDqMma);
      auto issue_s = [&](int it) -> bool {  // S(it) = Q K(it)^T into score buffer it & 1
        const int ks = it % L::kKStages;
        if (!mbar_wait(bar_k_full + 8 * ks, (uint32_t)(it / L::kKStages) & 1u, guard, kStDqMma)) return false;
        tc_fence_after();
        const uint32_t k_lo = desc_lo_sw128(sKr + ks * L::kTileBytes, 16);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_ss_lh(tS + (it & 1) * 128, q_lo + kmajor_step(kk), k_lo + kmajor_step(kk), hi_k, idesc_s, kk > 0);
        mma_commit(bar_s_full + 8 * (it & 1));
        return true;
      };
      auto issue_dp = [&](int it) -> bool {  // dP(it) = dO V(it)^T
        const int vs = it % L::kVStages;
        if (!mbar_wait(bar_v_full + 8 * vs, (uint32_t)(it / L::kVStages) & 1u, guard, kStDqMma)) return false;
        tc_fence_after();
        const uint32_t v_lo = desc_lo_sw128(sVr + vs * L::kTileBytes, 16);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_ss_lh(tdP, do_lo + kmajor_step(kk), v_lo + kmajor_step(kk), hi_k, idesc_s, kk > 0);
        mma_commit(bar_v_empty + 8 * vs);
        mma_commit(bar_dp_full);
        return true;
      };
      if (ok) ok = issue_s(0);
      if (ok) ok = issue_dp(0);
      if (ok && n_it > 1) ok = issue_s(1);
      for (int it = 0; it < n_it && ok; ++it) {
        const int ks = it % L::kKStages;
        const uint32_t kmn_lo = desc_lo_sw128(sKr + ks * L::kTileBytes, kChunkBytes);
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {  // dQ += dS K, 64 keys at a time as their dS lands in TMEM
          ok = mbar_wait(bar_p_full + 8 * hf, (uint32_t)it & 1u, guard, kStDqMma);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int kk = hf * 4 + j;
            const uint32_t acol = hf * 64 + (j / 2) * 32 + (j % 2) * 8;
            mma_ts_lh(tdQ, tdP + acol, kmn_lo + kk * 128, hi_k, idesc_acc, (it > 0 || kk > 0));
          }
        }
        if (!ok) break;
        mma_commit(bar_k_empty + 8 * ks);
        if (it + 1 < n_it) ok = issue_dp(it + 1);
        if (ok && it + 2 < n_it) ok = issue_s(it + 2);
      }
      if (ok) mma_commit(bar_acc_full);
    }
  } else {
    // ------------------------------------------------------------------- compute warps
    const int wg = warp >> 2;
    const int r = (warp & 3) * 32 + lane;  // query row inside the tile
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
    const int qg = qg0 + r;
    const bool row_ok = qg < n && qb + r < g.Lq;
    const float c = g.scale * kLog2e;
    float lse = 0.f, delta = 0.f;
    if (qb + r < g.Lq) {
      lse = p.lse[b * p.lse_sb + h * p.lse_sh + (qb + r) * p.lse_sl];
      if (lse == -CUDART_INF_F) lse = 0.f;
      delta = p.delta[((long long)b * g.H + h) * g.Lq + qb + r];
    }
    if (!row_ok) lse = CUDART_INF_F;  // padded query rows: 2^(x - inf) = 0, so they contribute nothing and stay finite
    const uint64_t c2 = pk2(c, c), nl2 = pk2(-lse, -lse), nd2 = pk2(-delta, -delta);
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const int kt = kt_lo + it;
      const int kg0 = kt * kTile + g.k_off;
      const bool full = M::kHasKFullRange && kg0 >= full_lo && kg0 + kTile <= full_hi && kg0 + kTile <= n &&
                        kt * kTile + kTile <= g.Lk;
      const int klim = imin(n - kg0, g.Lk - kt * kTile);
      const uint32_t tSb = tS + (it & 1) * 128;
      int w_lo = 0, w_hi = -1;  // visible key columns of this query row inside the tile (interval functors)
      if (interval_rows<M>::value && !full) row_window<M, true>(qg, kg0, klim, n, g.margs, w_lo, w_hi);
      // ---- step 1: P = 2^(S c - LSE) as soon as S(it) is there (it was issued a tile ahead); kept packed
      ok = mbar_wait(bar_s_full + 8 * (it & 1), (uint32_t)(it >> 1) & 1u, guard, kStDqCompute);
      ok = __all_sync(0xffffffffu, ok);  // keep the warp converged for the .sync.aligned TMEM accesses
      if (!ok) break;
      tc_fence_after();
      uint32_t preg[2][16];
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int cbase = hf * 64 + wg * 32;  // this warp's 32 key columns of the half
        uint32_t sreg[32];
        tmem_ld32(tSb + lane_sel + cbase, sreg);
        tmem_wait_ld();
        auto body = [&](auto masked_tag) {  // two copies: full tiles run without any mask arithmetic
          constexpr bool kMasked = decltype(masked_tag)::value;
#pragma unroll
          for (int i = 0; i < 16; ++i) {  // packed fp32 pairs; lse = +inf on padded rows gives p = 0
            float p0, p1;
            upk2(ex2_pair(ffma2(pk2u(sreg[2 * i], sreg[2 * i + 1]), c2, nl2), (i % CHILL_BWD_POLY_DEN) < CHILL_BWD_POLY_NUM),
                 p0, p1);
            if (kMasked) {
              const int col = cbase + 2 * i;
              if (interval_rows<M>::value) {
                p0 = (col >= w_lo && col <= w_hi) ? p0 : 0.f;
                p1 = (col + 1 >= w_lo && col + 1 <= w_hi) ? p1 : 0.f;
              } else {
                p0 = (col < klim && M::mask(qg, kg0 + col, n, g.margs)) ? p0 : 0.f;
                p1 = (col + 1 < klim && M::mask(qg, kg0 + col + 1, n, g.margs)) ? p1 : 0.f;
              }
            }
            preg[hf][i] = pack2<T>(p0, p1);
          }
        };
        if (full) body(std::false_type{});
        else body(std::true_type{});
      }
      // ---- step 2: dS = P (dP - delta) once dP(it) has landed; each half goes to the dQ GEMM as soon as it is stored
      ok = mbar_wait(bar_dp_full, (uint32_t)it & 1u, guard, kStDqCompute);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int cbase = hf * 64 + wg * 32;
        uint32_t dpreg[32], dsreg[16];
        tmem_ld32(tdP + lane_sel + cbase, dpreg);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float p0, p1, d0, d1;
          unpack2<T>(preg[hf][i], p0, p1);
          upk2(fmul2(pk2(p0, p1), fadd2(pk2u(dpreg[2 * i], dpreg[2 * i + 1]), nd2)), d0, d1);
          dsreg[i] = pack2<T>(d0, d1);
        }
        tmem_st16(tdP + lane_sel + cbase, dsreg);  // 16-bit dS over the dP columns this warp just consumed
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_p_full + 8 * hf);  // one arrival per compute warp
      }
    }

    // ---- epilogue: dQ * sm_scale; warps 0-3 take channels [0, D/2), warps 4-7 the rest
    if (ok) ok = mbar_wait(bar_acc_full, 0, guard, kStDqEpilogue);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    uint8_t* stage = gen_base + L::kK;
#pragma unroll
    for (int qq = 0; qq < D / 64; ++qq) {
      const int q4 = wg * (D / 64) + qq;
      uint32_t acc[32];
      if (ok) {
        tmem_ld32(tdQ + lane_sel + q4 * 32, acc);
        tmem_wait_ld();
      }
      stage_row32<T>(stage, r, q4, acc, g.scale, ok && row_ok);
    }
    fence_proxy_async_smem();
    named_bar_sync(1, kBwdComputeThreads);
    if (threadIdx.x == 0) {
      for (int cc = 0; cc < kChunks; ++cc) tma_store_4d(&tmdQ, sKr + cc * kChunkBytes, cc * 64, qb, h, b);
      tma_store_commit();
      tma_store_wait_read();  // shared memory may be released; the global writes complete by kernel end
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 8) tmem_dealloc(tmem, kTmemColsBwd);
}

// ---------------------------------------------------------------------------- launchers
template <typename T, int D, class M>
int launch_bwd_one(const CUtensorMap* maps, const BwdTcParams& p, cudaStream_t st) {
  auto kdkdv = bwd_dkdv_tc_kernel<T, D, M>;
  auto kdq = bwd_dq_tc_kernel<T, D, M>;
  constexpr int smem = BwdSmem<D>::kDynamic;
  constexpr int smem_dq = DqSmem<D>::kDynamic;
  static_assert(smem_dq <= 232448 && smem <= 232448, "exceeds the 227 KB of shared memory a CTA can opt in to");
  struct TagDkdv {};
  struct TagDq {};
  cudaError_t ea = ensure_dynamic_smem<TagDkdv>(kdkdv, smem);
  if (ea != cudaSuccess) return (int)ea;
  ea = ensure_dynamic_smem<TagDq>(kdq, smem_dq);
  if (ea != cudaSuccess) return (int)ea;
  const Geo& g = p.g;
  // maps: 0 Q, 1 K, 2 V, 3 dO, 4 dQ, 5 dK, 6 dV
  if (p.which & 1) {
    dim3 gk((unsigned)(((g.Lk + kTile - 1) / kTile) * g.Hkv * g.B), 1, 1);
    kdkdv<<<gk, kBwdThreads, smem, st>>>(maps[0], maps[1], maps[2], maps[3], maps[5], maps[6], p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
  }
  if (p.which & 2) {
    dim3 gq((unsigned)(((g.Lq + kTile - 1) / kTile) * g.H * g.B), 1, 1);
    kdq<<<gq, kBwdThreads, smem_dq, st>>>(maps[0], maps[1], maps[2], maps[3], maps[4], p);
  }
  return (int)cudaGetLastError();
}

template <class M>
int launch_bwd_all(int dtype, int D, const CUtensorMap* maps, const BwdTcParams& p, cudaStream_t st) {
  if (dtype == 2) {
    if (D == 128) return launch_bwd_one<__nv_bfloat16, 128, M>(maps, p, st);
    if (D == 64) return launch_bwd_one<__nv_bfloat16, 64, M>(maps, p, st);
  } else if (dtype == 1) {
    if (D == 128) return launch_bwd_one<__half, 128, M>(maps, p, st);
    if (D == 64) return launch_bwd_one<__half, 64, M>(maps, p, st);
  }
  return (int)cudaErrorInvalidValue;
}

}  // namespace tc
}  // namespace chill
