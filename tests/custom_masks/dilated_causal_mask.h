// Example user functor for the custom-mask extension point: causal attention restricted to keys at the
// same residue as the query modulo `stride` (args[0]), i.e. a dilated causal pattern.  Rows are not
// contiguous intervals and the per-row limits are not monotone in the position, so the functor declares
// its limits non-continuous (a tile's range is then the min/max over all its rows), has no full ranges,
// and every tile goes through mask evaluation.
#pragma once

namespace chill {

struct DilatedCausalMask {
  static constexpr bool kHasKFullRange = false, kHasQFullRange = false;
  static constexpr bool kKLimsContinuous = false, kQLimsContinuous = false, kGuaranteedSafe = true;
  CHILL_HD static bool mask(int q, int k, int, const MaskArgs& a) { return k <= q && (q - k) % a.i[0] == 0; }
  CHILL_HD static void k_range_for_q(int q, int, const MaskArgs& a, int& lo, int& hi) {
    lo = q % a.i[0];
    hi = q;
  }
  CHILL_HD static void q_range_for_k(int k, int n, const MaskArgs& a, int& lo, int& hi) {
    lo = k;
    hi = k + ((n - 1 - k) / a.i[0]) * a.i[0];
  }
  CHILL_HD static void k_full_range_for_q(int, int, int, const MaskArgs&, int& lo, int& hi) { lo = hi = 0; }
  CHILL_HD static void q_full_range_for_k(int, int, int, const MaskArgs&, int& lo, int& hi) { lo = hi = 0; }
  CHILL_HD static bool is_full_block(int, int, int, int, int, const MaskArgs&) { return false; }
};

}  // namespace chill
