// Forward attention on tcgen05 tensor cores (sm_100a), 16-bit inputs, head dim 64, 128 or 256.
//
// One CTA owns a tile of 128 query rows of one (batch, head) and walks the key tiles (64 or 128 keys
// each, see FwdShape) that the mask functor's range function leaves for it.  Several CTAs share an SM, so
// one CTA's softmax overlaps the others' MMAs.  Roles inside a CTA:
//
//   warps 0-3  softmax: thread r owns query row r.  Per key tile: read the S row from TMEM,
//              mask (boundary tiles only), online softmax in base 2, write P (16-bit) back
//              into the TMEM columns S occupied, rescale the O accumulator in TMEM when the
//              running max grew by more than 2^8, and finally normalise and store O / LSE.
//   warp 4     TMA producer: Q once, then K and V tiles into shared-memory rings
//              (128B-swizzled boxes of 64 channels x KT rows); owns the TMEM allocation.
//   warp 5     MMA issuer (one thread): S = Q K^T (both operands from shared memory) and
//              O += P V (P from TMEM, V from shared memory, MN-major), completion signalled to
//              mbarriers with tcgen05.commit.
//
// TMEM columns: kSBufs buffers of KT fp32 columns for S, each overlaid by its P (16-bit, first KT / 2
// columns); then D columns of O.
// Reference math: chill_attention/chill_fwd.py:188-359 (three-segment key loop, base-2
// online softmax, LSE = m + log2 l); the segment split is replaced by a per-tile "full tile"
// test derived from the functor's k_full_range_for_q.
#pragma once
#include <type_traits>

#include "generic.cuh"
#include "tc_common.cuh"

namespace chill {
namespace tc {

constexpr int kTile = 128;          // query rows per CTA and keys per tile
#ifndef CHILL_HEAD_GROUP
#define CHILL_HEAD_GROUP 4
#endif
#ifndef CHILL_HEAD_GROUP_FWD
#define CHILL_HEAD_GROUP_FWD 8
#endif
constexpr int kHeadGroup = CHILL_HEAD_GROUP;         // (batch, head) pairs scheduled together, see cta_order
constexpr int kHeadGroupFwd = CHILL_HEAD_GROUP_FWD;  // the same for the forward kernel

// CTA order of the 1-D grids: (batch, head) pairs are taken in groups of `group`; inside a group the
// tile rank is the slow index and the head the fast one.  With rank 0 = the longest tile (last query tile /
// first key tile of a causal mask) the SMs drain from long to short work items, so the tail of a launch
// consists of the shortest ones, while only `group` heads' K/V (or Q/dO) are live at a time, so the tiles
// of one head still run close together and share their operands through L2.  Measured on one B200 (causal bf16
// B8 H16 L4096 D128), three alternating runs each: forward 0.577-0.587 ms with groups of 4, 0.562-0.567 ms with 8
// or 16; single-kernel backward 1.456-1.466 ms with 4, 1.472-1.479 ms with 8 or 16; groups of 32 cost both 3-5 %.
__device__ __forceinline__ void cta_order(int idx, int n_hb, int n_tiles, int& hb, int& rank, int group = kHeadGroup) {
  const int per_group = group * n_tiles;
  const int grp = idx / per_group, rem = idx - grp * per_group;
  const int heads_here = imin(group, n_hb - grp * group);
  rank = rem / heads_here;
  hb = grp * group + (rem - rank * heads_here);
}
constexpr int kFwdThreads = 256;      // warps 0-3 softmax, 4 TMA producer, 5 MMA issuer, 6-7 idle
constexpr int kFwdSoftmaxRegs = 200;  // TF32 forward (fwd_tf32.cuh): per-thread register budget after setmaxnreg
constexpr int kFwdOtherRegs = 56;     //   (2 CTAs/SM: 2 * 128 * (200 + 56) = 65536)
constexpr int kTmemColsFwd = 256;     // TF32 forward: S 128 + O 128 columns

// Shape of the 16-bit forward kernel for one head dimension.  With one S buffer per CTA the steps of a tile form
// a chain S = Q K^T -> softmax -> O += P V -> next S (the next S overwrites P), measured at ~4100 clocks per 128-key
// tile against 1024 clocks of tensor work; what counts then is how many such chains an SM runs side by side, which
// TMEM (512 columns: S + O per CTA) limits.
// D = 64: key tiles of 64 keys need S 64 + O 64 = 128 columns, four CTAs per SM; the narrower MMAs (N = 64) run at
// 2/3 of the rate, which the kernel does not feel.
// D = 128: two CTAs per SM, 256 columns each, spent on O and TWO 64-key S buffers: S(j+1) = Q K(j+1)^T is issued
// before O += P(j) V(j), so it runs while the softmax warps work on tile j and the chain of a CTA shrinks to
// softmax -> PV (measured ~1850 clocks per 64-key step per CTA).
// D = 256: S 128 + O 256 columns and 192 KB of Q / K / V tiles leave room for one CTA per SM only.
// A CTA's register pool is threads x launch registers, and the softmax warpgroup's setmaxnreg.inc is only ever
// granted if softmax + other <= 2 x launch.
template <int D>
struct FwdShape {
  static constexpr int kKeys = (D <= 128) ? 64 : 128;      // keys per tile
  static constexpr int kSBufs = (D == 128) ? 2 : 1;        // S / P buffers in TMEM
  static constexpr int kCtasPerSm = (D == 64) ? 4 : (D == 128 ? 2 : 1);
  static constexpr int kStages = (D <= 128) ? 2 : 1;       // K / V ring depth
  static constexpr int kSO = kSBufs * kKeys + D;           // columns in use: S buffers, then O
  static constexpr int kTmemCols = (kSO <= 128) ? 128 : (kSO <= 256 ? 256 : 512);
  static constexpr int kLaunchRegs = (65536 / (kCtasPerSm * kFwdThreads) > 128) ? 128 : 65536 / (kCtasPerSm * kFwdThreads);
  static constexpr int kSoftmaxRegs = (D == 64) ? 96 : 200;
  static constexpr int kOtherRegs = (D == 64) ? 32 : 56;
  static_assert(kSoftmaxRegs + kOtherRegs <= 2 * kLaunchRegs, "setmaxnreg.inc would never be granted");
  static_assert(kCtasPerSm * kTmemCols <= 512, "TMEM columns of an SM");
};
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct FwdTcParams {
  Geo g;
  float* lse;
  long long lse_sb, lse_sh, lse_sl;
  void* o;  // for zero-filling tiles that are entirely padding
  long long o_sb, o_sh, o_sl;
  int* status;
};

template <int D, int NSTAGE, int KT = kTile>
struct FwdSmem {
  static constexpr int kTileBytes = kTile * D * 2;  // one 128 x D tile of 16-bit elements (Q)
  static constexpr int kKvBytes = KT * D * 2;       // one K or V tile: KT keys
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + kTileBytes;
  static constexpr int kV = kK + NSTAGE * kKvBytes;
  static constexpr int kBars = kV + NSTAGE * kKvBytes;
  static constexpr int kNumBars = 8 + 4 * NSTAGE;
  static constexpr int kMisc = kBars + 8 * kNumBars;
  static constexpr int kTotal = kMisc + 16;
  static constexpr int kDynamic = kTotal + 1024;  // slack for manual 1024-byte alignment
};

// Status codes recorded by bounded waits (1xx = forward).
enum : int { kStProducer = 101, kStMma = 102, kStSoftmax = 103, kStEpilogue = 104 };

// Online-softmax step of one thread (= one query row) for one 128-key tile: reads the row of S from
// TMEM, updates the running maximum / sum, rescales the O accumulator in TMEM when needed and writes the
// 16-bit P row back over S.  `first` = first key tile of this row (no O to rescale yet).
template <typename T, int D, class M, int KT = kTile>
__device__ __forceinline__ void softmax_tile(uint32_t tS, uint32_t tO, uint32_t lane_sel, bool first, bool full, int klim,
                                             int qg, int kg0, int n, const MaskArgs& margs, float c, float& m_used,
                                             float& l, uint32_t bar_pv = 0, uint32_t pv_parity = 0,
                                             const Guard* guard = nullptr) {
  // One pass over the row: all 128 scores of this thread's row come into registers, the maximum
  // is taken with 3-input max on four independent chains, and exponentials, row sum and the
  // 16-bit packing run on pairs (packed fp32 FMA / ADD).  Full tiles skip the mask arithmetic
  // (separate copy of the body, so nothing is if-converted into the fast path).
  uint32_t sreg[KT];
#pragma unroll
  for (int q4 = 0; q4 < KT / 32; ++q4) tmem_ld32(tS + lane_sel + q4 * 32, sreg + q4 * 32);
  tmem_wait_ld();
  if (!full) {
    if (interval_rows<M>::value) {  // two per-row bounds instead of a mask() call per element
      int c_lo, c_hi;
      row_window<M, true>(qg, kg0, klim, n, margs, c_lo, c_hi);
#pragma unroll
      for (int cidx = 0; cidx < KT; ++cidx) sreg[cidx] = (cidx >= c_lo && cidx <= c_hi) ? sreg[cidx] : 0xff800000u;
    } else {
#pragma unroll
      for (int cidx = 0; cidx < KT; ++cidx) {
        const bool vis = cidx < klim && M::mask(qg, kg0 + cidx, n, margs);
        sreg[cidx] = vis ? sreg[cidx] : 0xff800000u;  // -inf
      }
    }
  }
  float mx0 = -CUDART_INF_F, mx1 = -CUDART_INF_F, mx2 = -CUDART_INF_F, mx3 = -CUDART_INF_F;
#pragma unroll
  for (int i = 0; i < KT; i += 8) {
    mx0 = fmax3(mx0, __uint_as_float(sreg[i]), __uint_as_float(sreg[i + 1]));
    mx1 = fmax3(mx1, __uint_as_float(sreg[i + 2]), __uint_as_float(sreg[i + 3]));
    mx2 = fmax3(mx2, __uint_as_float(sreg[i + 4]), __uint_as_float(sreg[i + 5]));
    mx3 = fmax3(mx3, __uint_as_float(sreg[i + 6]), __uint_as_float(sreg[i + 7]));
  }
  const float m_tile = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * c;  // c > 0 (checked by the host)
  const float m_cand = fmaxf(m_used, m_tile);
  if (first) {
    m_used = m_cand;
  } else {
    const bool need = (m_cand - m_used) > kRescaleThreshold;  // false when both are -inf
    if (__any_sync(0xffffffffu, need)) {
      // With two S buffers the previous tile's O += P V may still be running: wait for it before touching O.
      if (bar_pv != 0) {
        mbar_wait(bar_pv, pv_parity, *guard, kStSoftmax);
        tc_fence_after();
      }
      const float alpha = (m_cand == -CUDART_INF_F) ? 1.f : ex2(m_used - m_cand);
      l *= alpha;
      m_used = m_cand;
#pragma unroll 1
      for (int q4 = 0; q4 < D / 16; ++q4) {
        uint32_t oreg[16];
        tmem_ld16(tO + lane_sel + q4 * 16, oreg);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 16; ++i) oreg[i] = __float_as_uint(__uint_as_float(oreg[i]) * alpha);
        tmem_st16(tO + lane_sel + q4 * 16, oreg);
      }
    }
  }
  const float m_safe = (m_used == -CUDART_INF_F) ? 0.f : m_used;
  const uint64_t c2 = pk2(c, c), nm2 = pk2(-m_safe, -m_safe);
  uint64_t l0 = 0ull, l1 = 0ull;  // two packed partial row sums (+0.0f, +0.0f)
  // Share of the pairs whose 2^x is the polynomial on the FMA pipe instead of MUFU.  Head dim 256 runs one CTA per
  // SM, i.e. one softmax warp per scheduler with nothing to hide its MUFU latency behind: a quarter there measured
  // 1.155 vs 1.211 ms (causal L = 4096); every share made head dims 64 / 128 slower (see tc_common.cuh).
  constexpr int kPolyNum = (D == 256 && CHILL_FWD_POLY_NUM == 0) ? 1 : CHILL_FWD_POLY_NUM;
  constexpr int kPolyDen = (D == 256 && CHILL_FWD_POLY_NUM == 0) ? 4 : CHILL_FWD_POLY_DEN;
#pragma unroll
  for (int i = 0; i < KT / 2; i += 2) {
    // two pairs per step
    const uint64_t e0 = ex2_pair(ffma2(pk2u(sreg[2 * i], sreg[2 * i + 1]), c2, nm2), (i % kPolyDen) < kPolyNum);
    const uint64_t e1 = ex2_pair(ffma2(pk2u(sreg[2 * i + 2], sreg[2 * i + 3]), c2, nm2), ((i + 1) % kPolyDen) < kPolyNum);
    l0 = fadd2(l0, e0);
    l1 = fadd2(l1, e1);
    float p0, p1, p2, p3;
    upk2(e0, p0, p1);
    upk2(e1, p2, p3);
    sreg[i] = pack2<T>(p0, p1);      // 16-bit P pair i overwrites a slot already consumed (i <= 2i)
    sreg[i + 1] = pack2<T>(p2, p3);
  }
  {
    float a0, a1, a2, a3;
    upk2(l0, a0, a1);
    upk2(l1, a2, a3);
    l += (a0 + a1) + (a2 + a3);
  }
#pragma unroll
  for (int q4 = 0; q4 < KT / 64; ++q4) tmem_st32(tS + lane_sel + q4 * 32, sreg + q4 * 32);  // KT / 2 columns of 16-bit pairs
}

// Normalise this thread's O row, convert to 16 bits and stage it in the 128B-swizzled TMA box layout;
// also writes the row's LSE.  `have` = the accumulator holds data (at least one key tile was processed).
template <typename T, int D>
__device__ __forceinline__ void stage_output_row(uint8_t* sO, uint32_t tO, uint32_t lane_sel, int r, bool have,
                                                 bool row_valid, float l, float m_used, float* lse_ptr) {
  const float l_safe = (l == 0.f) ? 1.f : l;
  const float inv = 1.f / l_safe;
#pragma unroll
  for (int q4 = 0; q4 < D / 32; ++q4) {
    uint32_t oreg[32];
    if (have) {
      tmem_ld32(tO + lane_sel + q4 * 32, oreg);
      tmem_wait_ld();
    }
    uint32_t packed[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float a = 0.f, bb = 0.f;
      if (have && row_valid && l != 0.f) {
        a = __uint_as_float(oreg[2 * i]) * inv;
        bb = __uint_as_float(oreg[2 * i + 1]) * inv;
      }
      packed[i] = pack2<T>(a, bb);
    }
    // 32 channels = 64 bytes = four 16-byte units of the row's 128-byte line in chunk (q4 / 2)
    uint8_t* line = sO + (q4 / 2) * (kTile * 128) + r * 128;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int unit = ((q4 % 2) * 4 + u) ^ (r & 7);
      *reinterpret_cast<uint4*>(line + unit * 16) =
          make_uint4(packed[4 * u], packed[4 * u + 1], packed[4 * u + 2], packed[4 * u + 3]);
    }
  }
  if (lse_ptr != nullptr) {
    float v = 0.f;
    if (row_valid) v = (l == 0.f) ? -CUDART_INF_F : m_used + lg2(l);
    *lse_ptr = v;
  }
}

template <typename T, int D, class M>
__global__ void __launch_bounds__(kFwdThreads, (FwdShape<D>::kCtasPerSm > 1 ? FwdShape<D>::kCtasPerSm : 2))
fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
              const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO, FwdTcParams p) {
  using SH = FwdShape<D>;
  constexpr int NSTAGE = SH::kStages;
  constexpr int KT = SH::kKeys;                // keys per tile
  using L = FwdSmem<D, NSTAGE, KT>;
  constexpr int kChunks = D / 64;              // 64-channel (128-byte) column blocks per tile
  constexpr int kChunkBytes = kTile * 128;     // one column block of Q / O: 128 rows x 128 bytes
  constexpr int kKvChunkBytes = KT * 128;      // one column block of a K / V tile: KT rows x 128 bytes
  const Geo& g = p.g;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = (g.Lq + kTile - 1) / kTile;
  int hb, rank;
  cta_order((int)blockIdx.x, g.B * g.H, n_qt, hb, rank, kHeadGroupFwd);
  const int qt = n_qt - 1 - rank;  // late (long) causal tiles first
  const int h = hb % g.H, b = hb / g.H;
  const int hk = h / (g.H / g.Hkv);
  const int qb = qt * kTile;
  const int qg0 = qb + g.q_off;
  int n = g.seq_len;
  if (g.lens != nullptr) n = imin(n, g.lens[b]);

  if (qg0 >= n) {
    // Every row of this tile is padding: O = 0, LSE = 0 (the reference returns early and leaves
    // its zero-initialised outputs, chill_fwd.py:70-71).
    T* obase = reinterpret_cast<T*>(p.o) + b * p.o_sb + h * p.o_sh;
    const int rows = imin(kTile, g.Lq - qb);
    for (int idx = threadIdx.x; idx < rows * (D / 8); idx += kFwdThreads) {
      const int r = idx / (D / 8), c = idx % (D / 8);
      *reinterpret_cast<uint4*>(obase + (qb + r) * p.o_sl + c * 8) = make_uint4(0, 0, 0, 0);
    }
    if (p.lse != nullptr)
      for (int r = threadIdx.x; r < rows; r += kFwdThreads) p.lse[b * p.lse_sb + h * p.lse_sh + (qb + r) * p.lse_sl] = 0.f;
    return;
  }

  // ---- key-tile range of this query tile (same arithmetic in every role)
  int kt_lo = 0, kt_hi = 0;  // [kt_lo, kt_hi) in units of KT local key rows
  int full_lo = 0, full_hi = 0;  // global, half-open: keys visible to every row of the tile
  {
    int lo, hi;
    tile_range<M, true>(qg0, imin(kTile, g.Lq - qb), n, g.margs, lo, hi);
    const int lo_l = imax(lo - g.k_off, 0);
    const int hi_l = imin(imin(hi, n - 1) - g.k_off, g.Lk - 1);
    if (hi_l >= lo_l) {
      kt_lo = lo_l / KT;
      kt_hi = hi_l / KT + 1;
    }
    if (M::kHasKFullRange) M::k_full_range_for_q(qg0, kTile, n, g.margs, full_lo, full_hi);
  }
  const int n_tiles = kt_hi - kt_lo;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t sQ = base + L::kQ, sK = base + L::kK, sV = base + L::kV;
  const uint32_t bars = base + L::kBars;
  constexpr int NSB = SH::kSBufs;
  // One tcgen05.commit per MMA batch is free, a second one costs the issuing thread ~48 clocks (measured), so a
  // batch signals ONE barrier with several waiters: s_full[j % NSTAGE] tells the softmax warps that S(j) is there
  // and the producer that K stage j % NSTAGE is free; v_empty[j % NSTAGE] tells the producer that V stage is free
  // and a softmax warp that has to rescale O that O += P(j) V(j) has finished.  Per barrier at most one phase can
  // be ahead of any waiter (the next commit on it needs that waiter's own progress), so the parity tests hold.
  // p_full: one barrier per S buffer.
  const uint32_t bar_q_full = bars, bar_s_full = bars + 8, bar_p_full = bars + 24, bar_o_full = bars + 40;
  const uint32_t bar_k_full = bars + 64, bar_v_full = bar_k_full + 8 * NSTAGE, bar_v_empty = bar_v_full + 8 * NSTAGE;
  const uint32_t bar_k_empty = bar_s_full;  // same barriers: S(j) complete == K stage j % NSTAGE consumed
  static_assert(NSTAGE <= 2 && NSB <= 2, "barrier layout");
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen_base + L::kMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + L::kMisc + 4);
  const Guard guard{p.status, abort_flag};

  if (warp == 4) {
    // The producer thread initialises the barriers itself, so it can put Q and the first K/V tile in flight
    // before the CTA-wide set-up (TMEM allocation, __syncthreads) completes instead of after it.
    if (lane == 0) {
      *abort_flag = 0;
      mbar_init(bar_q_full, 1);
      for (int i = 0; i < NSB; ++i) mbar_init(bar_p_full + 8 * i, 4);
      mbar_init(bar_o_full, 1);
      for (int s = 0; s < NSTAGE; ++s) {
        mbar_init(bar_s_full + 8 * s, 1);
        mbar_init(bar_k_full + 8 * s, 1);
        mbar_init(bar_v_full + 8 * s, 1);
        mbar_init(bar_v_empty + 8 * s, 1);
      }
      fence_barrier_init();
      fence_proxy_async_smem();
      if (n_tiles > 0) {
        mbar_arrive_expect_tx(bar_q_full, L::kTileBytes);
        for (int c = 0; c < kChunks; ++c) tma_load_4d(sQ + c * kChunkBytes, &tmQ, bar_q_full, c * 64, qb, h, b);
        mbar_arrive_expect_tx(bar_k_full, L::kKvBytes);
        for (int c = 0; c < kChunks; ++c) tma_load_4d(sK + c * kKvChunkBytes, &tmK, bar_k_full, c * 64, kt_lo * KT, hk, b);
        mbar_arrive_expect_tx(bar_v_full, L::kKvBytes);
        for (int c = 0; c < kChunks; ++c) tma_load_4d(sV + c * kKvChunkBytes, &tmV, bar_v_full, c * 64, kt_lo * KT, hk, b);
      }
    }
    __syncwarp();
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), SH::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem;            // S / P columns: NSB buffers of KT columns
  const uint32_t tO = tmem + NSB * KT; // O columns

  if (warp == 4) {
    reg_dealloc<SH::kOtherRegs>();
    // ------------------------------------------------------------------- TMA producer
    if (lane == 0 && n_tiles > 0) {
      bool ok = true;
      for (int j = 1; j < n_tiles && ok; ++j) {  // tile 0 was issued during set-up
        const int s = j % NSTAGE;
        const uint32_t ph = (uint32_t)(j / NSTAGE) & 1u;
        const int krow = (kt_lo + j) * KT;
        ok = mbar_wait(bar_k_empty + 8 * s, ph ^ 1u, guard, kStProducer);
        if (!ok) break;
        mbar_arrive_expect_tx(bar_k_full + 8 * s, L::kKvBytes);
        for (int c = 0; c < kChunks; ++c)
          tma_load_4d(sK + s * L::kKvBytes + c * kKvChunkBytes, &tmK, bar_k_full + 8 * s, c * 64, krow, hk, b);
        ok = mbar_wait(bar_v_empty + 8 * s, ph ^ 1u, guard, kStProducer);
        if (!ok) break;
        mbar_arrive_expect_tx(bar_v_full + 8 * s, L::kKvBytes);
        for (int c = 0; c < kChunks; ++c)
          tma_load_4d(sV + s * L::kKvBytes + c * kKvChunkBytes, &tmV, bar_v_full + 8 * s, c * 64, krow, hk, b);
      }
      if (!ok) {
        // give copies already in flight time to land before the CTA's shared memory goes away
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 5) {
    reg_dealloc<SH::kOtherRegs>();
    // --------------------------------------------------------------------- MMA issuer
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_s = make_idesc<T>(kTile, KT, false, false);
      constexpr uint32_t idesc_o = make_idesc<T>(kTile, D, false, true);
      constexpr uint32_t hi_k = desc_hi_sw128(1024);  // both operand kinds: 8-row groups 1 KB apart
      const uint32_t q_lo = desc_lo_sw128(sQ, 16);
      bool ok = mbar_wait(bar_q_full, 0, guard, kStMma);
      auto issue_s = [&](int j) -> bool {  // S(j) = Q K(j)^T into S buffer j % NSB: both K-major, 16 channels per MMA
        const int s = j % NSTAGE;
        const uint32_t k_lo = desc_lo_sw128(sK + s * L::kKvBytes, 16);
        if (!mbar_wait(bar_k_full + 8 * s, (uint32_t)(j / NSTAGE) & 1u, guard, kStMma)) return false;
        tc_fence_after();
        const uint32_t ts = tS + (uint32_t)((j % NSB) * KT);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)  // Q chunks are 128 rows apart, K chunks KT rows
          mma_ss_lh(ts, q_lo + kmajor_step(kk), k_lo + (uint32_t)((kk / 4) * (kKvChunkBytes / 16) + (kk % 4) * 2), hi_k, idesc_s,
                    kk > 0 ? 1u : 0u);
        mma_commit(bar_s_full + 8 * s);
        return true;
      };
      auto issue_pv = [&](int j) -> bool {  // O += P(j) V(j): P (16-bit) from TMEM, 16 keys = 8 columns per MMA
        const int s = j % NSTAGE;
        const uint32_t v_lo = desc_lo_sw128(sV + s * L::kKvBytes, kKvChunkBytes);  // MN-major: channel blocks one chunk apart
        if (!mbar_wait(bar_p_full + 8 * (j % NSB), (uint32_t)(j / NSB) & 1u, guard, kStMma)) return false;
        if (!mbar_wait(bar_v_full + 8 * s, (uint32_t)(j / NSTAGE) & 1u, guard, kStMma)) return false;
        tc_fence_after();
        const uint32_t tp = tS + (uint32_t)((j % NSB) * KT);
#pragma unroll
        for (int kk = 0; kk < KT / 16; ++kk)
          mma_ts_lh(tO, tp + kk * 8, v_lo + kk * 128, hi_k, idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
        mma_commit(bar_v_empty + 8 * s);
        return true;
      };
      if (NSB == 1) {
        // one S buffer: S(j+1) overwrites P(j), so the two GEMMs of a tile alternate
        for (int j = 0; j < n_tiles && ok; ++j) {
          ok = issue_s(j);
          if (ok) ok = issue_pv(j);
        }
      } else {
        // S(j+1) goes to the other buffer and is issued ahead of O += P(j) V(j): it runs during softmax(j).
        // MMAs execute in issue order, so S(j+2) cannot overtake the P V(j) that still reads its buffer.
        if (ok) ok = issue_s(0);
        for (int j = 0; j < n_tiles && ok; ++j) {
          if (j + 1 < n_tiles) ok = issue_s(j + 1);
          if (ok) ok = issue_pv(j);
        }
      }
      if (ok) mma_commit(bar_o_full);
    }
  } else if (warp >= 6) {
    reg_dealloc<SH::kOtherRegs>();  // idle warps of the second warpgroup only give their registers back
  } else {
    reg_alloc<SH::kSoftmaxRegs>();
    // --------------------------------------------------------- softmax + epilogue warps
    const int r = warp * 32 + lane;  // row inside the tile == TMEM lane
    const uint32_t lane_sel = (uint32_t)(warp * 32) << 16;
    const int qg = qg0 + r;
    const float c = g.scale * kLog2e;
    float m_used = -CUDART_INF_F, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int kt = kt_lo + j;
      const int kg0 = kt * KT + g.k_off;
      ok = mbar_wait(bar_s_full + 8 * (j % NSTAGE), (uint32_t)(j / NSTAGE) & 1u, guard, kStSoftmax);
      ok = __all_sync(0xffffffffu, ok);  // keep the warp converged for the .sync.aligned TMEM accesses
      if (!ok) break;
      tc_fence_after();
      const bool full = M::kHasKFullRange && kg0 >= full_lo && kg0 + KT <= full_hi && kg0 + KT <= n &&
                        kt * KT + KT <= g.Lk;
      const int klim = imin(n - kg0, g.Lk - kt * KT);  // columns >= klim do not exist
      softmax_tile<T, D, M, KT>(tS + (uint32_t)((j % NSB) * KT), tO, lane_sel, j == 0, full, klim, qg, kg0, n, g.margs, c,
                                m_used, l, NSB > 1 ? bar_v_empty + 8 * (uint32_t)((j - 1) % NSTAGE) : 0u,
                                (uint32_t)((j - 1) / NSTAGE) & 1u, &guard);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p_full + 8 * (j % NSB));  // one arrival per softmax warp
    }

    // ---- epilogue: O / l -> 16-bit -> swizzled shared memory (Q's buffer) -> TMA store
    if (ok && n_tiles > 0) ok = mbar_wait(bar_o_full, 0, guard, kStEpilogue);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    const bool row_valid = qg < n;
    stage_output_row<T, D>(gen_base + L::kQ, tO, lane_sel, r, n_tiles > 0 && ok, row_valid, l, m_used,
                           (p.lse != nullptr && qb + r < g.Lq) ? p.lse + b * p.lse_sb + h * p.lse_sh + (qb + r) * p.lse_sl
                                                                : nullptr);
    fence_proxy_async_smem();
    named_bar_sync(1, 128);
    if (threadIdx.x == 0) {
      for (int cc = 0; cc < kChunks; ++cc) tma_store_4d(&tmO, base + L::kQ + cc * kChunkBytes, cc * 64, qb, h, b);
      tma_store_commit();
      tma_store_wait_read();  // shared memory may be released; the global writes complete by kernel end
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem, SH::kTmemCols);
}

}  // namespace tc
}  // namespace chill
