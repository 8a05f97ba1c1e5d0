// A DELIBERATELY WRONG functor, used only by the test of ChillMask.verify(device=True): a sliding window over the
// previous args[0] keys whose k_range_for_q starts one key too late.  mask() itself is right, so the Python twin
// verifies, but kernels built with this functor would clip the first visible key of every row out of their tile loop.
#pragma once

namespace chill {

struct OffByOneWindowMask {
  static constexpr bool kHasKFullRange = false, kHasQFullRange = false;
  static constexpr bool kKLimsContinuous = true, kQLimsContinuous = true, kGuaranteedSafe = true;
  CHILL_HD static bool mask(int q, int k, int, const MaskArgs& a) { return k <= q && k >= q - a.i[0]; }
  CHILL_HD static void k_range_for_q(int q, int, const MaskArgs& a, int& lo, int& hi) {
    lo = imax(0, q - a.i[0] + 1);  // wrong: the window starts at q - args[0]
    hi = q;
  }
  CHILL_HD static void q_range_for_k(int k, int n, const MaskArgs& a, int& lo, int& hi) {
    lo = k;
    hi = imin(k + a.i[0], n - 1);
  }
  CHILL_HD static void k_full_range_for_q(int, int, int, const MaskArgs&, int& lo, int& hi) { lo = hi = 0; }
  CHILL_HD static void q_full_range_for_k(int, int, int, const MaskArgs&, int& lo, int& hi) { lo = hi = 0; }
  CHILL_HD static bool is_full_block(int, int, int, int, int, const MaskArgs&) { return false; }
};

}  // namespace chill
