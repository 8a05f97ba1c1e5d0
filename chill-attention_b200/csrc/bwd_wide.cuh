// Backward attention for head dim 256 on tcgen05 tensor cores (sm_100a, 16-bit inputs).
//
// At D = 256 the accumulators of dK and dV alone would fill TMEM (2 x 256 of 512 columns), so the gradients are
// computed by THREE launches of one kernel template, each with a single 128 x 256 accumulator and the scores
// recomputed (eight GEMMs per tile pair instead of the five of the single-kernel backward for D <= 128):
//
//   kWideDV  one CTA per (batch, kv head, 128 keys):   S^T = K Q^T,                  W = P^T,                dV += W dO
//   kWideDK  same rows:                                S^T = K Q^T, dP^T = V dO^T,   W = P^T (dP^T - delta), dK += W Q
//   kWideDQ  one CTA per (batch, head, 128 queries):   S = Q K^T,   dP = dO V^T,     W = P (dP - delta),     dQ += W K
//
// with P = 2^(S c - LSE) from the stored LSE (no running maximum).  The "row" operands (K / V, resp. Q / dO: 64 KB
// each) stay in shared memory, the other axis streams through in tiles of 64 positions (one stage: 2 x 32 KB; the
// tile that only a score GEMM reads is refilled while the step is still running), clipped by the mask functor's
// range function.  Roles as in fwd_tc.cuh: warps 0-3 own one tile row each per thread and turn the fp32 scores in
// TMEM into the 16-bit W (written over the scores, A operand of the accumulating GEMM), warp 4 is the TMA producer,
// warp 5 owns TMEM and issues the MMAs.
// TMEM columns: [0,64) S (W over its first 32), [64,128) dP, [128,384) accumulator.
// Reference math: chill_attention/chill_bwd_dkdv.py:347-508, chill_bwd_dq.py:300-394.
#pragma once
#include "bwd_tc.cuh"

namespace chill {
namespace tc {

enum : int { kWideDV = 0, kWideDK = 1, kWideDQ = 2 };
constexpr int kWideThreads = 256;  // warps 0-3 elementwise + epilogue, 4 TMA producer, 5 MMA issuer, 6-7 idle
constexpr int kWideComputeRegs = 200, kWideOtherRegs = 56;  // 128 * 200 + 128 * 56 = 256 * 128

template <int D>
struct WideSmem {
  static constexpr int kRowBytes = kTile * D * 2;      // a 128-row operand
  static constexpr int kColBytes = kWideCols * D * 2;  // a 64-row streamed tile
  static constexpr int kR1 = 0;
  static constexpr int kR2 = kR1 + kRowBytes;
  static constexpr int kC1 = kR2 + kRowBytes;
  static constexpr int kC2 = kC1 + kColBytes;
  static constexpr int kVec = kC2 + kColBytes;         // per warp: -LSE and -delta of the 64 streamed columns
  static constexpr int kBars = kVec + 4 * 2 * kWideCols * 4;
  static constexpr int kNumBars = 8;
  static constexpr int kMisc = kBars + 8 * kNumBars;
  static constexpr int kTotal = kMisc + 16;
  static constexpr int kDynamic = kTotal + 1024;
};

enum : int { kStWideProducer = 501, kStWideMma = 502, kStWideCompute = 503, kStWideEpilogue = 504 };

// maps: R1, R2 = 128-row boxes of the row operands; C1, C2 = 64-row boxes of the streamed operands; OUT = 128-row
// box of the gradient written.  kWideDV: R1 = K, (R2 unused), C1 = Q, C2 = dO, OUT = dV.  kWideDK: R1 = K, R2 = V,
// C1 = Q, C2 = dO, OUT = dK.  kWideDQ: R1 = Q, R2 = dO, C1 = K, C2 = V, OUT = dQ.
template <typename T, int D, class M, int MODE>
__global__ void __launch_bounds__(kWideThreads, 2)  // 2: 128 registers at launch, the pool setmaxnreg redistributes
bwd_wide_kernel(const __grid_constant__ CUtensorMap tmR1, const __grid_constant__ CUtensorMap tmR2,
                const __grid_constant__ CUtensorMap tmC1, const __grid_constant__ CUtensorMap tmC2,
                const __grid_constant__ CUtensorMap tmOut, BwdTcParams p) {
  using L = WideSmem<D>;
  constexpr bool kKeyRows = MODE != kWideDQ;   // tile rows are keys (dV, dK) or queries (dQ)
  constexpr bool kTwoScores = MODE != kWideDV;  // dP is needed as well
  constexpr int CT = kWideCols;
  constexpr int kChunks = D / 64;
  constexpr int kChunkBytes = kTile * 128;  // one 64-channel column block of a 128-row tile
  constexpr int kColChunkBytes = CT * 128;  // the same of a streamed tile
  const Geo& g = p.g;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = g.H / g.Hkv;
  const int n_rt = ((kKeyRows ? g.Lk : g.Lq) + kTile - 1) / kTile;
  const int n_units = kKeyRows ? g.B * g.Hkv : g.B * g.H;
  int unit, rank;
  cta_order((int)blockIdx.x, n_units, n_rt, unit, rank);
  const int rt = kKeyRows ? rank : n_rt - 1 - rank;  // longest tiles first under a causal mask
  const int hr = kKeyRows ? unit % g.Hkv : unit % g.H;  // head index of the row operands
  const int b = kKeyRows ? unit / g.Hkv : unit / g.H;
  const int hk = kKeyRows ? hr : hr / G;
  const int rb = rt * kTile;                                   // first local row
  const int rg0 = rb + (kKeyRows ? g.k_off : g.q_off);         // its global position
  const int rows_here = imin(kTile, (kKeyRows ? g.Lk : g.Lq) - rb);
  int n = g.seq_len;
  if (g.lens != nullptr) n = imin(n, g.lens[b]);

  // ---- range of the streamed axis, in tiles of CT local positions
  int ct_lo = 0, ct_hi = 0;
  if (rg0 < n) {
    int lo, hi;
    tile_range<M, !kKeyRows>(rg0, rows_here, n, g.margs, lo, hi);
    const int off = kKeyRows ? g.q_off : g.k_off, len = kKeyRows ? g.Lq : g.Lk;
    const int lo_l = imax(lo - off, 0);
    const int hi_l = imin(imin(hi, n - 1) - off, len - 1);
    if (hi_l >= lo_l) {
      ct_lo = lo_l / CT;
      ct_hi = hi_l / CT + 1;
    }
  }
  const int n_ct = ct_hi - ct_lo;
  const int n_it = n_ct * (kKeyRows ? G : 1);  // key rows: every head of the GQA group contributes
  T* out_base = reinterpret_cast<T*>(MODE == kWideDV ? p.dv : (MODE == kWideDK ? p.dk : p.dq));
  const long long o_sb = MODE == kWideDV ? p.dv_sb : (MODE == kWideDK ? p.dk_sb : p.dq_sb);
  const long long o_sh = MODE == kWideDV ? p.dv_sh : (MODE == kWideDK ? p.dk_sh : p.dq_sh);
  const long long o_sl = MODE == kWideDV ? p.dv_sl : (MODE == kWideDK ? p.dk_sl : p.dq_sl);
  if (n_it == 0) {  // padding rows, or rows nothing on this shard can see: zero gradient
    zero_rows<T, D>(out_base + b * o_sb + hr * o_sh + rb * o_sl, o_sl, rows_here, kWideThreads);
    if (MODE == kWideDV) zero_part_rows<D>(p.part, b, hr, rb, rows_here, g.Lk, kWideThreads);  // dK and dV partials
    return;
  }

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t sR1 = base + L::kR1, sR2 = base + L::kR2, sC1 = base + L::kC1, sC2 = base + L::kC2;
  float* vec_s = reinterpret_cast<float*>(gen_base + L::kVec);  // [warp][0: -lse, 1: -delta][64]
  const uint32_t bars = base + L::kBars;
  // The two streamed tiles have different lifetimes: the "early" one (Q for dV, dO / V for dK / dQ) is only read by
  // a score GEMM and can be refilled while the step is still running; the "late" one is the B operand of the
  // accumulating GEMM.  e_done = the early tile's GEMM has finished (for dV that is also "scores ready").
  const uint32_t bar_r_full = bars, bar_ce_full = bars + 8, bar_cl_full = bars + 16, bar_e_done = bars + 24,
                 bar_cl_empty = bars + 32, bar_t_full = bars + 40, bar_w_full = bars + 48, bar_acc_full = bars + 56;
  const uint32_t sEarly = MODE == kWideDV ? sC1 : sC2, sLate = MODE == kWideDV ? sC2 : sC1;
  const CUtensorMap* tmEarly = MODE == kWideDV ? &tmC1 : &tmC2;
  const CUtensorMap* tmLate = MODE == kWideDV ? &tmC2 : &tmC1;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen_base + L::kMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + L::kMisc + 4);
  const Guard guard{p.status, abort_flag};
  // streamed tile `it`: head and first local position
  auto col_head = [&](int it) { return kKeyRows ? hk * G + it / n_ct : hk; };
  auto col_pos = [&](int it) { return (ct_lo + it % n_ct) * CT; };

  if (warp == 4) {
    if (lane == 0) {
      *abort_flag = 0;
      mbar_init(bar_r_full, 1);
      mbar_init(bar_ce_full, 1);
      mbar_init(bar_cl_full, 1);
      mbar_init(bar_e_done, 1);
      mbar_init(bar_cl_empty, 1);
      mbar_init(bar_t_full, 1);
      mbar_init(bar_w_full, 4);
      mbar_init(bar_acc_full, 1);
      fence_barrier_init();
      fence_proxy_async_smem();
      mbar_arrive_expect_tx(bar_r_full, (kTwoScores ? 2 : 1) * L::kRowBytes);
      for (int c = 0; c < kChunks; ++c) {
        tma_load_4d(sR1 + c * kChunkBytes, &tmR1, bar_r_full, c * 64, rb, hr, b);
        if (kTwoScores) tma_load_4d(sR2 + c * kChunkBytes, &tmR2, bar_r_full, c * 64, rb, hr, b);
      }
      mbar_arrive_expect_tx(bar_ce_full, L::kColBytes);
      for (int c = 0; c < kChunks; ++c)
        tma_load_4d(sEarly + c * kColChunkBytes, tmEarly, bar_ce_full, c * 64, col_pos(0), col_head(0), b);
      mbar_arrive_expect_tx(bar_cl_full, L::kColBytes);
      for (int c = 0; c < kChunks; ++c)
        tma_load_4d(sLate + c * kColChunkBytes, tmLate, bar_cl_full, c * 64, col_pos(0), col_head(0), b);
    }
  } else if (warp == 5) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem, tdP = tmem + CT, tAcc = tmem + 2 * CT;

  if (warp == 4) {
    reg_dealloc<kWideOtherRegs>();
    // ------------------------------------------------------------------- TMA producer
    if (lane == 0) {
      bool ok = true;
      for (int it = 1; it < n_it && ok; ++it) {  // tile 0 was issued during set-up
        const uint32_t prev = (uint32_t)(it - 1) & 1u;
        ok = mbar_wait(bar_e_done, prev, guard, kStWideProducer);
        if (!ok) break;
        mbar_arrive_expect_tx(bar_ce_full, L::kColBytes);
        for (int c = 0; c < kChunks; ++c)
          tma_load_4d(sEarly + c * kColChunkBytes, tmEarly, bar_ce_full, c * 64, col_pos(it), col_head(it), b);
        ok = mbar_wait(bar_cl_empty, prev, guard, kStWideProducer);
        if (!ok) break;
        mbar_arrive_expect_tx(bar_cl_full, L::kColBytes);
        for (int c = 0; c < kChunks; ++c)
          tma_load_4d(sLate + c * kColChunkBytes, tmLate, bar_cl_full, c * 64, col_pos(it), col_head(it), b);
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 5) {
    reg_dealloc<kWideOtherRegs>();
    // --------------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc<T>(kTile, CT, false, false);
      constexpr uint32_t idesc_acc = make_idesc<T>(kTile, D, false, true);  // A from TMEM, B MN-major
      constexpr uint32_t hi_k = desc_hi_sw128(1024);
      const uint32_t r1_lo = desc_lo_sw128(sR1, 16), r2_lo = desc_lo_sw128(sR2, 16);
      const uint32_t c1_lo = desc_lo_sw128(sC1, 16), c2_lo = desc_lo_sw128(sC2, 16);
      // the streamed tile that multiplies W: dO for dV, Q for dK, K for dQ; MN-major, channel blocks one chunk apart
      const uint32_t x_lo = desc_lo_sw128(MODE == kWideDV ? sC2 : sC1, kColChunkBytes);
      bool ok = mbar_wait(bar_r_full, 0, guard, kStWideMma);
      auto score = [&](uint32_t t_dst, uint32_t r_lo, uint32_t c_lo) {  // rows x 64 positions, contraction over D
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_ss_lh(t_dst, r_lo + kmajor_step(kk), c_lo + (uint32_t)((kk / 4) * (kColChunkBytes / 16) + (kk % 4) * 2), hi_k,
                    idesc_s, kk > 0 ? 1u : 0u);
      };
      for (int it = 0; it < n_it && ok; ++it) {
        const uint32_t par = (uint32_t)it & 1u;
        // the GEMM that reads the early tile: S for dV, dP for dK / dQ
        ok = mbar_wait(bar_ce_full, par, guard, kStWideMma);
        if (!ok) break;
        tc_fence_after();
        if (MODE == kWideDV) score(tS, r1_lo, c1_lo);
        else score(tdP, r2_lo, c2_lo);
        mma_commit(bar_e_done);
        ok = mbar_wait(bar_cl_full, par, guard, kStWideMma);
        if (!ok) break;
        tc_fence_after();
        if (kTwoScores) {
          score(tS, r1_lo, c1_lo);
          mma_commit(bar_t_full);
        }
        ok = mbar_wait(bar_w_full, par, guard, kStWideMma);
        if (!ok) break;
        tc_fence_after();
        // accumulator += W X: W (16-bit) from TMEM, 16 streamed positions = 8 columns of W and 2 KB of X per MMA
#pragma unroll
        for (int kk = 0; kk < CT / 16; ++kk)
          mma_ts_lh(tAcc, tS + kk * 8, x_lo + kk * 128, hi_k, idesc_acc, (it > 0 || kk > 0) ? 1u : 0u);
        mma_commit(bar_cl_empty);  // the late tile, S and dP may be overwritten
      }
      if (ok) mma_commit(bar_acc_full);
    }
  } else if (warp >= 6) {
    reg_dealloc<kWideOtherRegs>();
  } else {
    reg_alloc<kWideComputeRegs>();
    // --------------------------------------------------------- elementwise + epilogue warps
    const int r = warp * 32 + lane;  // row inside the tile == TMEM lane
    const uint32_t lane_sel = (uint32_t)(warp * 32) << 16;
    const int rg = rg0 + r;  // global position of this thread's row (a key, or a query for kWideDQ)
    const bool row_ok = rg < n && r < rows_here;
    const float c = g.scale * kLog2e;
    float row_nl = 0.f, row_nd = 0.f;  // kWideDQ: -LSE and -delta of this thread's query row
    if (!kKeyRows && r < rows_here) {
      const float lv = p.lse[b * p.lse_sb + hr * p.lse_sh + (rb + r) * p.lse_sl];
      row_nl = (lv == -CUDART_INF_F) ? 0.f : -lv;
      row_nd = -p.delta[((long long)b * g.H + hr) * g.Lq + rb + r];
    }
    // streamed positions that EVERY row of this tile sees (half-open, global): tiles inside skip the mask arithmetic
    int full_lo = 0, full_hi = 0;
    constexpr bool kHasFull = kKeyRows ? M::kHasQFullRange : M::kHasKFullRange;
    if (kHasFull && rg0 + kTile <= n && rows_here == kTile) {
      if (kKeyRows) M::q_full_range_for_k(rg0, kTile, n, g.margs, full_lo, full_hi);
      else M::k_full_range_for_q(rg0, kTile, n, g.margs, full_lo, full_hi);
    }
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const uint32_t par = (uint32_t)it & 1u;
      const int cpos = col_pos(it);  // first local position of the streamed tile
      const int cg0 = cpos + (kKeyRows ? g.q_off : g.k_off);
      const int clim = imin(n - cg0, (kKeyRows ? g.Lq : g.Lk) - cpos);  // streamed positions >= clim do not exist
      float* vb = vec_s + warp * (2 * CT);  // warp-private copy: no barrier across warps inside the loop
      if (kKeyRows) {
        // -LSE and -delta of the 64 query columns: two of each per lane
        const int h = col_head(it);
        __syncwarp();  // the previous step's reads of vb are done
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int cc = lane + 32 * e;
          const int q = imin(cpos + cc, g.Lq - 1);
          const float lv = p.lse[b * p.lse_sb + h * p.lse_sh + q * p.lse_sl];
          vb[cc] = (lv == -CUDART_INF_F) ? 0.f : -lv;
          vb[CT + cc] = -p.delta[((long long)b * g.H + h) * g.Lq + q];
        }
        __syncwarp();
      }
      ok = mbar_wait(kTwoScores ? bar_t_full : bar_e_done, par, guard, kStWideCompute);
      ok = __all_sync(0xffffffffu, ok);  // keep the warp converged for the .sync.aligned TMEM accesses
      if (!ok) break;
      tc_fence_after();
      const bool full = kHasFull && cg0 >= full_lo && cg0 + CT <= full_hi && clim >= CT;
      uint32_t w[CT / 2];
      auto body = [&](auto masked_tag) {  // two copies: full tiles run without any mask arithmetic
        constexpr bool kMasked = decltype(masked_tag)::value;
#pragma unroll
        for (int half = 0; half < 2; ++half) {  // 32 streamed positions at a time
          uint32_t sreg[32], dreg[32];
          tmem_ld32(tS + lane_sel + half * 32, sreg);
          if (kTwoScores) tmem_ld32(tdP + lane_sel + half * 32, dreg);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float wv[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int cc = half * 32 + i + e;
              const float nl = kKeyRows ? vb[cc] : row_nl;
              const float nd = kKeyRows ? vb[CT + cc] : row_nd;
              float pv = ex2(fmaf(__uint_as_float(sreg[i + e]), c, nl));
              if (kMasked) {
                const int qg = kKeyRows ? cg0 + cc : rg, kg = kKeyRows ? rg : cg0 + cc;
                pv = (row_ok && cc < clim && M::mask(qg, kg, n, g.margs)) ? pv : 0.f;
              }
              if (kTwoScores) pv *= __uint_as_float(dreg[i + e]) + nd;
              wv[e] = pv;
            }
            w[half * 16 + i / 2] = pack2<T>(wv[0], wv[1]);
          }
        }
      };
      if (full) body(std::false_type{});
      else body(std::true_type{});
      tmem_st32(tS + lane_sel, w);  // CT / 2 = 32 columns of 16-bit pairs over the scores just consumed
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_w_full);
    }

    // ---- epilogue: accumulator (x sm_scale for dK, dQ) -> 16-bit -> swizzled shared memory (R1's buffer) -> TMA store
    if (ok) ok = mbar_wait(bar_acc_full, 0, guard, kStWideEpilogue);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    const float mul = MODE == kWideDV ? 1.f : g.scale;
    // optional un-rounded fp32 copy of this key row's dV / dK (first / last key rows of the call, see PartOut)
    float* part_row = kKeyRows ? p.part.row(MODE == kWideDV ? p.part.dv : p.part.dk, b, hr, rb + r, g.Lk) : nullptr;
#pragma unroll 1
    for (int q4 = 0; q4 < D / 32; ++q4) {
      uint32_t acc[32];
      if (ok) {
        tmem_ld32(tAcc + lane_sel + q4 * 32, acc);
        tmem_wait_ld();
      }
      stage_row32<T>(gen_base + L::kR1, r, q4, acc, mul, ok && row_ok);
      if (part_row != nullptr) store_part32(part_row + q4 * 32, acc, mul, ok && row_ok);
    }
    fence_proxy_async_smem();
    named_bar_sync(1, 128);
    if (threadIdx.x == 0) {
      for (int cc = 0; cc < kChunks; ++cc) tma_store_4d(&tmOut, sR1 + cc * kChunkBytes, cc * 64, rb, hr, b);
      tma_store_commit();
      tma_store_wait_read();  // shared memory may be released; the global writes complete by kernel end
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem, 512);
}

// maps: 0 Q128, 1 K128, 2 V128, 3 dO128 (128-row boxes), 4 Q64, 5 K64, 6 V64, 7 dO64 (64-row boxes), 8 dQ, 9 dK, 10 dV
template <typename T, class M>
int launch_bwd_wide(const CUtensorMap* maps, const BwdTcParams& p, cudaStream_t st) {
  constexpr int D = 256;
  constexpr int smem = WideSmem<D>::kDynamic;
  static_assert(smem <= 232448, "exceeds the 227 KB of shared memory a CTA can opt in to");
  const Geo& g = p.g;
  const unsigned key_ctas = (unsigned)(((g.Lk + kTile - 1) / kTile) * g.Hkv * g.B);
  const unsigned query_ctas = (unsigned)(((g.Lq + kTile - 1) / kTile) * g.H * g.B);
  cudaError_t e;
  {
    auto kern = bwd_wide_kernel<T, D, M, kWideDV>;
    struct Tag {};
    if ((e = ensure_dynamic_smem<Tag>(kern, smem)) != cudaSuccess) return (int)e;
    kern<<<key_ctas, kWideThreads, smem, st>>>(maps[1], maps[2], maps[4], maps[7], maps[10], p);
    if ((e = cudaGetLastError()) != cudaSuccess) return (int)e;
  }
  {
    auto kern = bwd_wide_kernel<T, D, M, kWideDK>;
    struct Tag {};
    if ((e = ensure_dynamic_smem<Tag>(kern, smem)) != cudaSuccess) return (int)e;
    kern<<<key_ctas, kWideThreads, smem, st>>>(maps[1], maps[2], maps[4], maps[7], maps[9], p);
    if ((e = cudaGetLastError()) != cudaSuccess) return (int)e;
  }
  {
    auto kern = bwd_wide_kernel<T, D, M, kWideDQ>;
    struct Tag {};
    if ((e = ensure_dynamic_smem<Tag>(kern, smem)) != cudaSuccess) return (int)e;
    kern<<<query_ctas, kWideThreads, smem, st>>>(maps[0], maps[3], maps[5], maps[6], maps[8], p);
    if ((e = cudaGetLastError()) != cudaSuccess) return (int)e;
  }
  return 0;
}

template <class M>
int launch_bwd_wide_all(int dtype, const CUtensorMap* maps, const BwdTcParams& p, cudaStream_t st) {
  if (dtype == 2) return launch_bwd_wide<__nv_bfloat16, M>(maps, p, st);
  if (dtype == 1) return launch_bwd_wide<__half, M>(maps, p, st);
  return (int)cudaErrorInvalidValue;
}

}  // namespace tc
}  // namespace chill
