// Mask functors: the device half of a ChillMask.
//
// The reference inlines a mask's static Triton functions into its kernels
// (chill_attention/mask.py:54-250); here a mask is a struct of static
// __host__ __device__ functions and the kernels are templates over it.
// Contract of a functor `M` (positions are GLOBAL token indices, `a` holds the
// constants the Python mask object was constructed with):
//
//   bool M::mask(q, k, seq_len, a)                    true = q may attend k
//   void M::k_range_for_q(q, seq_len, a, lo, hi)      inclusive key range of one query
//   void M::q_range_for_k(k, seq_len, a, lo, hi)      inclusive query range of one key
//   void M::k_full_range_for_q(qb, tq, seq_len, a, lo, hi)   half-open: keys seen by EVERY query of [qb, qb+tq)
//   void M::q_full_range_for_k(kb, tk, seq_len, a, lo, hi)   half-open: queries seeing EVERY key of [kb, kb+tk)
//   bool M::is_full_block(q, k, qt, kt, seq_len, a)   tile needs no mask evaluation
//   constexpr bool kHasKFullRange, kHasQFullRange     the two full-range functions are meaningful
//   constexpr bool kKLimsContinuous, kQLimsContinuous a tile's range = [range(first).lo, range(last).hi]
//   constexpr bool kGuaranteedSafe                    every query sees at least one key
//   constexpr bool kIntervalRows (optional, default false)   mask(q, k) == (k_range_for_q(q).lo <= k <= .hi) and
//                                                      == (q_range_for_k(k).lo <= q <= .hi): visible sets are intervals,
//                                                      so boundary tiles compare column indices against two per-row
//                                                      bounds instead of evaluating mask() per element
//
// The key-length bound (k < lens[b]) is applied by the kernels, not by the functor.
#pragma once
#include <stdint.h>

#include <type_traits>

#ifndef __CUDACC__
#define __host__
#define __device__
#endif
#define CHILL_HD __host__ __device__ __forceinline__

namespace chill {

struct MaskArgs {
  int i[8];
  float f[8];
};

CHILL_HD int imax(int a, int b) { return a > b ? a : b; }
CHILL_HD int imin(int a, int b) { return a < b ? a : b; }

// chill_attention/mask.py:806-889
struct FullMask {
  static constexpr bool kHasKFullRange = true, kHasQFullRange = true;
  static constexpr bool kIntervalRows = true;
  static constexpr bool kKLimsContinuous = true, kQLimsContinuous = true, kGuaranteedSafe = true;
  CHILL_HD static bool mask(int, int, int, const MaskArgs&) { return true; }
  CHILL_HD static void k_range_for_q(int, int n, const MaskArgs&, int& lo, int& hi) { lo = 0; hi = n - 1; }
  CHILL_HD static void q_range_for_k(int, int n, const MaskArgs&, int& lo, int& hi) { lo = 0; hi = n - 1; }
  CHILL_HD static void k_full_range_for_q(int, int, int n, const MaskArgs&, int& lo, int& hi) { lo = 0; hi = n; }
  CHILL_HD static void q_full_range_for_k(int, int, int n, const MaskArgs&, int& lo, int& hi) { lo = 0; hi = n; }
  CHILL_HD static bool is_full_block(int, int, int, int, int, const MaskArgs&) { return true; }
};

// chill_attention/mask.py:892-976
struct CausalMask {
  static constexpr bool kHasKFullRange = true, kHasQFullRange = true;
  static constexpr bool kIntervalRows = true;
  static constexpr bool kKLimsContinuous = true, kQLimsContinuous = true, kGuaranteedSafe = true;
  CHILL_HD static bool mask(int q, int k, int, const MaskArgs&) { return q >= k; }
  CHILL_HD static void k_range_for_q(int q, int, const MaskArgs&, int& lo, int& hi) { lo = 0; hi = q; }
  CHILL_HD static void q_range_for_k(int k, int n, const MaskArgs&, int& lo, int& hi) { lo = k; hi = n - 1; }
  CHILL_HD static void k_full_range_for_q(int qb, int, int, const MaskArgs&, int& lo, int& hi) { lo = 0; hi = qb + 1; }
  CHILL_HD static void q_full_range_for_k(int kb, int tk, int n, const MaskArgs&, int& lo, int& hi) {
    lo = imax(0, kb + tk - 1);
    hi = n;
  }
  CHILL_HD static bool is_full_block(int q, int k, int, int kt, int, const MaskArgs&) { return k + kt - 1 <= q; }
};

// chill_attention/mask.py:979-1108; args: left_context, right_context
struct SlidingWindowMask {
  static constexpr bool kHasKFullRange = true, kHasQFullRange = true;
  static constexpr bool kIntervalRows = true;
  static constexpr bool kKLimsContinuous = true, kQLimsContinuous = true, kGuaranteedSafe = false;
  CHILL_HD static bool mask(int q, int k, int, const MaskArgs& a) { return (k <= q + a.i[1]) && (k >= q - a.i[0]); }
  CHILL_HD static void k_range_for_q(int q, int n, const MaskArgs& a, int& lo, int& hi) {
    lo = imax(0, q - a.i[0]);
    hi = imin(q + a.i[1], n - 1);
  }
  CHILL_HD static void q_range_for_k(int k, int n, const MaskArgs& a, int& lo, int& hi) {
    lo = imax(0, k - a.i[1]);
    hi = imin(k + a.i[0], n - 1);
  }
  CHILL_HD static void k_full_range_for_q(int qb, int tq, int n, const MaskArgs& a, int& lo, int& hi) {
    lo = imax(0, qb + tq - 1 - a.i[0]);
    hi = imax(lo, imin(n, qb + a.i[1] + 1));
  }
  // The reference leaves this one at the empty default (mask.py:131-151); it is the same
  // derivation as k_full_range_for_q with the two contexts swapped.
  CHILL_HD static void q_full_range_for_k(int kb, int tk, int n, const MaskArgs& a, int& lo, int& hi) {
    lo = imax(0, kb + tk - 1 - a.i[1]);
    hi = imax(lo, imin(n, kb + a.i[0] + 1));
  }
  CHILL_HD static bool inside(int diff, const MaskArgs& a) {
    return (diff >= 0 && diff <= a.i[0]) || (diff <= 0 && diff >= -a.i[1]);
  }
  CHILL_HD static bool is_full_block(int q, int k, int qt, int kt, int, const MaskArgs& a) {
    return inside(q + qt - 1 - k, a) && inside(q - (k + kt - 1), a);
  }
};

// chill_attention/mask.py:1111-1266; args: context_size, back_contexts
struct ChunkwiseMask {
  static constexpr bool kHasKFullRange = true, kHasQFullRange = true;
  static constexpr bool kIntervalRows = true;
  static constexpr bool kKLimsContinuous = true, kQLimsContinuous = true, kGuaranteedSafe = false;
  CHILL_HD static bool mask(int q, int k, int, const MaskArgs& a) {
    const int d = q / a.i[0] - k / a.i[0];
    return d >= 0 && d <= a.i[1];
  }
  CHILL_HD static void k_range_for_q(int q, int n, const MaskArgs& a, int& lo, int& hi) {
    const int c = q / a.i[0];
    lo = imax(0, (c - a.i[1]) * a.i[0]);
    hi = imin((c + 1) * a.i[0] - 1, n - 1);
  }
  CHILL_HD static void q_range_for_k(int k, int n, const MaskArgs& a, int& lo, int& hi) {
    const int c = k / a.i[0];
    lo = c * a.i[0];
    hi = imin((c + a.i[1] + 1) * a.i[0] - 1, n - 1);
  }
  CHILL_HD static void k_full_range_for_q(int qb, int tq, int n, const MaskArgs& a, int& lo, int& hi) {
    lo = imax(0, ((qb + tq - 1) / a.i[0] - a.i[1]) * a.i[0]);
    hi = imax(lo, imin(n, (qb / a.i[0] + 1) * a.i[0]));
  }
  // Not in the reference (empty default): queries whose chunk is within back_contexts of
  // every chunk the key tile touches.
  CHILL_HD static void q_full_range_for_k(int kb, int tk, int n, const MaskArgs& a, int& lo, int& hi) {
    lo = ((kb + tk - 1) / a.i[0]) * a.i[0];
    hi = imax(lo, imin(n, (kb / a.i[0] + a.i[1] + 1) * a.i[0]));
  }
  CHILL_HD static bool is_full_block(int q, int k, int qt, int kt, int, const MaskArgs& a) {
    const int d1 = q / a.i[0] - (k + kt - 1) / a.i[0];
    const int d2 = (q + qt - 1) / a.i[0] - k / a.i[0];
    return d1 >= 0 && d1 <= a.i[1] && d2 >= 0 && d2 <= a.i[1];
  }
};

// chill_attention/mask.py:1269-1394; args: prefix_size
struct PrefixLMMask {
  static constexpr bool kHasKFullRange = true, kHasQFullRange = true;
  static constexpr bool kIntervalRows = true;
  static constexpr bool kKLimsContinuous = true, kQLimsContinuous = true, kGuaranteedSafe = true;
  CHILL_HD static bool mask(int q, int k, int, const MaskArgs& a) { return k < a.i[0] || q >= k; }
  CHILL_HD static void k_range_for_q(int q, int n, const MaskArgs& a, int& lo, int& hi) {
    lo = 0;
    hi = imin(imax(q, a.i[0] - 1), n - 1);
  }
  CHILL_HD static void q_range_for_k(int k, int n, const MaskArgs& a, int& lo, int& hi) {
    lo = k < a.i[0] ? 0 : k;
    hi = n - 1;
  }
  CHILL_HD static void k_full_range_for_q(int qb, int, int n, const MaskArgs& a, int& lo, int& hi) {
    lo = 0;
    hi = imin(imax(a.i[0], qb + 1), n);
  }
  // Not in the reference (empty default): a key tile inside the prefix is seen by every
  // query, otherwise the causal rule applies.
  CHILL_HD static void q_full_range_for_k(int kb, int tk, int n, const MaskArgs& a, int& lo, int& hi) {
    if (kb + tk <= a.i[0]) {
      lo = 0;
      hi = n;
    } else {
      lo = imax(0, kb + tk - 1);
      hi = imax(lo, n);
    }
  }
  CHILL_HD static bool is_full_block(int q, int k, int qt, int kt, int, const MaskArgs& a) {
    return (k + kt - 1 <= q) || (q + qt <= a.i[0] && k + kt <= a.i[0]);
  }
};

// kIntervalRows of a functor, false when it does not declare it.
template <class M, class = void>
struct interval_rows : std::false_type {};
template <class M>
struct interval_rows<M, std::void_t<decltype(M::kIntervalRows)>> : std::bool_constant<M::kIntervalRows> {};

// Visible column window [c_lo, c_hi] (inclusive, tile-local, empty when c_hi < c_lo) of one row of a boundary
// tile for interval functors.  KForQ: the row is query `pos`, columns are keys starting at global `col0`;
// otherwise the row is key `pos`, columns are queries.  `ncols` = number of existing columns in the tile.
template <class M, bool KForQ>
CHILL_HD void row_window(int pos, int col0, int ncols, int n, const MaskArgs& a, int& c_lo, int& c_hi) {
  int lo, hi;
  if (KForQ) M::k_range_for_q(pos, n, a, lo, hi);
  else M::q_range_for_k(pos, n, a, lo, hi);
  c_lo = imax(lo - col0, 0);
  c_hi = imin(imin(hi, n - 1) - col0, ncols - 1);
  if (pos >= n || pos < 0) c_hi = -1;
}

// ----------------------------------------------------------------------------------------
// Tile-loop clipping, shared by every kernel (reference: chill_attention/utils.py:221-272).
//
// For the tile of `tile_in` positions starting at global position `i` on one axis, returns
// the inclusive global range [lo, hi] of the OTHER axis that any valid position of the tile
// can see.  `n` is the sequence length (positions >= n are ignored).  Empty when hi < lo.
template <class M, bool KForQ>
CHILL_HD void tile_range(int i, int tile_in, int n, const MaskArgs& a, int& lo, int& hi) {
  const int last = imin(i + tile_in, n) - 1;
  if (last < i) {
    lo = 0;
    hi = -1;
    return;
  }
  constexpr bool cont = KForQ ? M::kKLimsContinuous : M::kQLimsContinuous;
  if (cont) {
    int t;
    if (KForQ) {
      M::k_range_for_q(i, n, a, lo, t);
      M::k_range_for_q(last, n, a, t, hi);
    } else {
      M::q_range_for_k(i, n, a, lo, t);
      M::q_range_for_k(last, n, a, t, hi);
    }
  } else {
    lo = n;
    hi = -1;
    for (int p = i; p <= last; ++p) {
      int l, h;
      if (KForQ) M::k_range_for_q(p, n, a, l, h);
      else M::q_range_for_k(p, n, a, l, h);
      lo = imin(lo, l);
      hi = imax(hi, h);
    }
  }
}

}  // namespace chill

#ifdef CHILL_CUSTOM_MASK_HEADER
#include CHILL_CUSTOM_MASK_HEADER
#endif
