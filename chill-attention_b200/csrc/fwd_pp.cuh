// Forward attention, "ping-pong" variant: one CTA per SM owns TWO consecutive 128-row query tiles of a
// head and one shared K/V ring.  Each query tile has its own softmax warpgroup, score buffer and output
// accumulator in TMEM (S0 S1 O0 O1 = 512 columns), and a single MMA-issuing thread interleaves the two
// tiles in a fixed order
//        PV0(j)  QK0(j+1)  PV1(j)  QK1(j+1)  PV0(j+1) ...
// so that tile 0's exponentials run while the tensor cores work for tile 1 and vice versa: the two
// softmax phases are held in anti-phase by construction instead of by chance (two independent CTAs
// per SM drift into phase and then fight over the MUFU unit), and K/V tiles are fetched once for both.
// Math and conventions are those of fwd_tc.cuh (softmax_tile / stage_output_row are shared).
#pragma once
#include "fwd_tc.cuh"

namespace chill {
namespace tc {

constexpr int kPpThreads = 384;      // warps 0-3: softmax of tile 0, 4-7: tile 1, 8: TMA, 9: MMA, 10-11 idle
constexpr int kPpSoftmaxRegs = 208;  // 2 * 128 * 208 + 128 * 56 = 60416 <= 65536
constexpr int kPpOtherRegs = 56;

template <int D>
struct PpSmem {
  static constexpr int kTileBytes = kTile * D * 2;
  static constexpr int kStages = 2;
  static constexpr int kQ = 0;                                  // two query tiles
  static constexpr int kK = kQ + 2 * kTileBytes;
  static constexpr int kV = kK + kStages * kTileBytes;
  static constexpr int kBars = kV + kStages * kTileBytes;
  static constexpr int kNumBars = 1 + 4 * kStages + 6;
  static constexpr int kMisc = kBars + 8 * kNumBars;
  static constexpr int kTotal = kMisc + 16;
  static constexpr int kDynamic = kTotal + 1024;
};

enum : int { kStPpProducer = 111, kStPpMma = 112, kStPpSoftmax = 113, kStPpEpilogue = 114 };

template <typename T, int D, class M>
__global__ void __launch_bounds__(kPpThreads, 1)
fwd_pp_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
              const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO, FwdTcParams p) {
  using L = PpSmem<D>;
  constexpr int kChunks = D / 64;
  constexpr int kChunkBytes = kTile * 128;
  const Geo& g = p.g;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = (g.Lq + kTile - 1) / kTile;
  const int n_pairs = (n_qt + 1) / 2;
  int hb, rank;
  cta_order((int)blockIdx.x, g.B * g.H, n_pairs, hb, rank);
  const int pair = n_pairs - 1 - rank;  // late (long) causal tiles first
  const int h = hb % g.H, b = hb / g.H;
  const int hk = h / (g.H / g.Hkv);
  int n = g.seq_len;
  if (g.lens != nullptr) n = imin(n, g.lens[b]);

  // ---- per query tile: does it exist, its key-tile range [lo, hi) and its full range
  int qb_[2], lo_[2], hi_[2], flo_[2], fhi_[2];
  bool exists_[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    qb_[t] = (2 * pair + t) * kTile;
    exists_[t] = qb_[t] < g.Lq;
    lo_[t] = hi_[t] = 0;
    flo_[t] = fhi_[t] = 0;
    const int qg0 = qb_[t] + g.q_off;
    if (exists_[t] && qg0 < n) {
      int lo, hi;
      tile_range<M, true>(qg0, imin(kTile, g.Lq - qb_[t]), n, g.margs, lo, hi);
      const int lo_l = imax(lo - g.k_off, 0);
      const int hi_l = imin(imin(hi, n - 1) - g.k_off, g.Lk - 1);
      if (hi_l >= lo_l) {
        lo_[t] = lo_l / kTile;
        hi_[t] = hi_l / kTile + 1;
      }
      if (M::kHasKFullRange) M::k_full_range_for_q(qg0, kTile, n, g.margs, flo_[t], fhi_[t]);
    }
  }
  const bool any0 = hi_[0] > lo_[0], any1 = hi_[1] > lo_[1];
  int j_lo = 0, j_hi = 0;
  if (any0 && any1) {
    j_lo = imin(lo_[0], lo_[1]);
    j_hi = imax(hi_[0], hi_[1]);
  } else if (any0) {
    j_lo = lo_[0];
    j_hi = hi_[0];
  } else if (any1) {
    j_lo = lo_[1];
    j_hi = hi_[1];
  }

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t sQ = base + L::kQ, sK = base + L::kK, sV = base + L::kV;
  const uint32_t bars = base + L::kBars;
  const uint32_t bar_q_full = bars;
  const uint32_t bar_k_full = bars + 8, bar_k_empty = bar_k_full + 16, bar_v_full = bar_k_empty + 16,
                 bar_v_empty = bar_v_full + 16;
  const uint32_t bar_s_full = bar_v_empty + 16, bar_p_full = bar_s_full + 16, bar_o_full = bar_p_full + 16;  // [2] each
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen_base + L::kMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + L::kMisc + 4);
  const Guard guard{p.status, abort_flag};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(bar_q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_k_full + 8 * s, 1);
      mbar_init(bar_k_empty + 8 * s, 1);
      mbar_init(bar_v_full + 8 * s, 1);
      mbar_init(bar_v_empty + 8 * s, 1);
      mbar_init(bar_s_full + 8 * s, 1);
      mbar_init(bar_p_full + 8 * s, 4);
      mbar_init(bar_o_full + 8 * s, 1);
    }
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 8) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 8) {
    reg_dealloc<kPpOtherRegs>();
    // ------------------------------------------------------------------- TMA producer
    if (lane == 0 && j_hi > j_lo) {
      prefetch_tmap(&tmQ);
      prefetch_tmap(&tmK);
      prefetch_tmap(&tmV);
      mbar_arrive_expect_tx(bar_q_full, (uint32_t)((any0 ? 1 : 0) + (any1 ? 1 : 0)) * L::kTileBytes);
#pragma unroll
      for (int t = 0; t < 2; ++t)
        if (hi_[t] > lo_[t])
          for (int c = 0; c < kChunks; ++c)
            tma_load_4d(sQ + t * L::kTileBytes + c * kChunkBytes, &tmQ, bar_q_full, c * 64, qb_[t], h, b);
      bool ok = true;
      for (int j = j_lo; j < j_hi && ok; ++j) {
        const int i = j - j_lo, s = i & 1;
        const uint32_t ph = (uint32_t)(i >> 1) & 1u;
        const int krow = j * kTile;
        ok = mbar_wait(bar_k_empty + 8 * s, ph ^ 1u, guard, kStPpProducer);
        if (!ok) break;
        mbar_arrive_expect_tx(bar_k_full + 8 * s, L::kTileBytes);
        for (int c = 0; c < kChunks; ++c)
          tma_load_4d(sK + s * L::kTileBytes + c * kChunkBytes, &tmK, bar_k_full + 8 * s, c * 64, krow, hk, b);
        ok = mbar_wait(bar_v_empty + 8 * s, ph ^ 1u, guard, kStPpProducer);
        if (!ok) break;
        mbar_arrive_expect_tx(bar_v_full + 8 * s, L::kTileBytes);
        for (int c = 0; c < kChunks; ++c)
          tma_load_4d(sV + s * L::kTileBytes + c * kChunkBytes, &tmV, bar_v_full + 8 * s, c * 64, krow, hk, b);
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 9) {
    reg_dealloc<kPpOtherRegs>();
    // --------------------------------------------------------------------- MMA issuer
    if (lane == 0 && j_hi > j_lo) {
      constexpr uint32_t idesc_s = make_idesc<T>(kTile, kTile, false, false);
      constexpr uint32_t idesc_o = make_idesc<T>(kTile, D, false, true);
      constexpr uint32_t hi_k = desc_hi_sw128(1024);
      const uint32_t q_lo[2] = {desc_lo_sw128(sQ, 16), desc_lo_sw128(sQ + L::kTileBytes, 16)};
      auto active = [&](int t, int j) { return j >= lo_[t] && j < hi_[t]; };
      auto issue_qk = [&](int t, int s) {
        const uint32_t k_lo = desc_lo_sw128(sK + s * L::kTileBytes, 16);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_ss_lh(tmem + t * 128, q_lo[t] + kmajor_step(kk), k_lo + kmajor_step(kk), hi_k, idesc_s, kk > 0 ? 1u : 0u);
        mma_commit(bar_s_full + 8 * t);
      };
      int cnt[2] = {0, 0};  // key tiles already accumulated per query tile
      bool ok = mbar_wait(bar_q_full, 0, guard, kStPpMma);
      if (ok) ok = mbar_wait(bar_k_full, 0, guard, kStPpMma);
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int t = 0; t < 2; ++t)
          if (active(t, j_lo)) issue_qk(t, 0);
        mma_commit(bar_k_empty);
      }
      for (int j = j_lo; j < j_hi && ok; ++j) {
        const int i = j - j_lo, s = i & 1;
        const uint32_t ph = (uint32_t)(i >> 1) & 1u, ph_next = (uint32_t)((i + 1) >> 1) & 1u;
        const bool next = j + 1 < j_hi;
        const uint32_t v_lo = desc_lo_sw128(sV + s * L::kTileBytes, kChunkBytes);
        bool have_v = false, have_k = false;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (active(t, j)) {
            ok = mbar_wait(bar_p_full + 8 * t, (uint32_t)cnt[t] & 1u, guard, kStPpMma);
            if (!ok) break;
            if (!have_v) {
              ok = mbar_wait(bar_v_full + 8 * s, ph, guard, kStPpMma);
              if (!ok) break;
              have_v = true;
            }
            tc_fence_after();
#pragma unroll
            for (int kk = 0; kk < kTile / 16; ++kk)
              mma_ts_lh(tmem + 256 + t * 128, tmem + t * 128 + kk * 8, v_lo + kk * 128, hi_k, idesc_o,
                        (cnt[t] > 0 || kk > 0) ? 1u : 0u);
            ++cnt[t];
            if (j == hi_[t] - 1) mma_commit(bar_o_full + 8 * t);
          }
          if (t == 1) {
            if (!have_v) {  // no tile used this V tile (gap between the two ranges): still consume its load
              ok = mbar_wait(bar_v_full + 8 * s, ph, guard, kStPpMma);
              if (!ok) break;
            }
            mma_commit(bar_v_empty + 8 * s);
          }
          if (next && active(t, j + 1)) {
            if (!have_k) {
              ok = mbar_wait(bar_k_full + 8 * (s ^ 1), ph_next, guard, kStPpMma);
              if (!ok) break;
              have_k = true;
              tc_fence_after();
            }
            issue_qk(t, s ^ 1);
          }
          if (t == 1 && next) {
            if (!have_k) {
              ok = mbar_wait(bar_k_full + 8 * (s ^ 1), ph_next, guard, kStPpMma);
              if (!ok) break;
            }
            mma_commit(bar_k_empty + 8 * (s ^ 1));
          }
        }
      }
    }
  } else if (warp >= 10) {
    reg_dealloc<kPpOtherRegs>();
  } else {
    reg_alloc<kPpSoftmaxRegs>();
    // --------------------------------------------------------- softmax + epilogue warpgroups
    const int t = warp >> 2;                     // which query tile
    const int r = (warp & 3) * 32 + lane;        // row inside the tile == TMEM lane
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + t * 128, tO = tmem + 256 + t * 128;
    const int qb = t ? qb_[1] : qb_[0];  // static indices keep the per-tile scalars in registers
    const int qg = qb + g.q_off + r;
    const int my_lo = t ? lo_[1] : lo_[0], my_hi = t ? hi_[1] : hi_[0];
    const int full_lo = t ? flo_[1] : flo_[0], full_hi = t ? fhi_[1] : fhi_[0];
    const bool exists = t ? exists_[1] : exists_[0];
    const float c = g.scale * kLog2e;
    float m_used = -CUDART_INF_F, l = 0.f;
    bool ok = true;
    for (int j = my_lo; j < my_hi; ++j) {
      const int kg0 = j * kTile + g.k_off;
      ok = mbar_wait(bar_s_full + 8 * t, (uint32_t)(j - my_lo) & 1u, guard, kStPpSoftmax);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const bool full = M::kHasKFullRange && kg0 >= full_lo && kg0 + kTile <= full_hi && kg0 + kTile <= n &&
                        j * kTile + kTile <= g.Lk;
      const int klim = imin(n - kg0, g.Lk - j * kTile);
      softmax_tile<T, D, M>(tS, tO, lane_sel, j == my_lo, full, klim, qg, kg0, n, g.margs, c, m_used, l);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p_full + 8 * t);
    }
    // ---- epilogue of this warpgroup's tile (staging = its own Q buffer)
    const bool have = my_hi > my_lo;
    if (ok && have) ok = mbar_wait(bar_o_full + 8 * t, 0, guard, kStPpEpilogue);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    if (exists) {
      stage_output_row<T, D>(gen_base + L::kQ + t * L::kTileBytes, tO, lane_sel, r, have && ok, qg < n, l, m_used,
                             (p.lse != nullptr && qb + r < g.Lq) ? p.lse + b * p.lse_sb + h * p.lse_sh + (qb + r) * p.lse_sl
                                                                  : nullptr);
      fence_proxy_async_smem();
      named_bar_sync(1 + t, 128);
      if ((threadIdx.x & 127) == 0) {
        for (int cc = 0; cc < kChunks; ++cc)
          tma_store_4d(&tmO, sQ + t * L::kTileBytes + cc * kChunkBytes, cc * 64, qb, h, b);
        tma_store_commit();
        tma_store_wait_read();  // shared memory may be released; the global writes complete by kernel end
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 8) tmem_dealloc(tmem, 512);
}

}  // namespace tc
}  // namespace chill
