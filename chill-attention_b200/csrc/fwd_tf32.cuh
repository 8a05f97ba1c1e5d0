// Forward attention for fp32 tensors on the tensor cores in TF32 (tcgen05.mma.kind::tf32, sm_100a), head dim 64 or
// 128.  Same structure as fwd_tc_kernel (fwd_tc.cuh): one CTA per (batch, head, tile of 128 queries), a TMA
// producer warp, one MMA-issuing thread, four softmax warps that own one query row per thread; what differs is the
// element size:
//   * a tile row is D * 4 bytes = D / 32 column blocks of 128 bytes; Q and K are K-major 128B-swizzled tiles as
//     before (an MMA step covers 8 channels = 32 bytes);
//   * P stays fp32: the softmax warps write it back over S in TMEM unchanged in width (the tensor core reads the
//     upper 19 bits of every value), and an MMA step of O += P V takes 8 keys = 8 TMEM columns;
//   * V is the MN-major operand.  For 32-bit elements that operand kind needs the "128-byte swizzle with 32-byte
//     atoms" layout (descriptor layout type 1, groups of 4 rows, 512 bytes apart), which TMA produces with
//     CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B;
//   * O is stored as fp32.
// Q, K and V are used as they are: the tensor core drops all but 10 mantissa bits (truncation); P is rounded to
// nearest by the softmax warps.  Against the fp64 oracle the output error on N(0,1) inputs is 2e-3 .. 4e-3 (the
// tests state 5e-3), three orders above the generic IEEE kernels that serve precision="ieee".
// Reference: chill_attention/chill_fwd.py:13-359 with input_precision="tf32".
#pragma once
#include <type_traits>

#include "fwd_tc.cuh"

namespace chill {
namespace tc {

template <>
__host__ __device__ constexpr uint32_t mma_fmt<float>() {
  return 2u;  // TF32
}

// descriptor high word: stride byte offset, version 1, layout type 1 (128B swizzle, 32-byte atoms)
__host__ __device__ constexpr uint32_t desc_hi_sw128_base32(uint32_t sbo_bytes) {
  return ((sbo_bytes >> 4) & 0x3FFFu) | (1u << 14) | (1u << 29);
}

__device__ __forceinline__ void mma_ss_tf32(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 da, {%1, %3};\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], da, db, %4, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_ts_tf32(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t hi, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 db;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], db, %4, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ uint32_t to_tf32(float x) {
  uint32_t y;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(y) : "f"(x));
  return y;
}

template <int D>
struct FwdTf32Smem {
  static constexpr int kTileBytes = kTile * D * 4;  // one 128 x D tile of fp32 elements
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + kTileBytes;
  static constexpr int kV = kK + kTileBytes;
  static constexpr int kBars = kV + kTileBytes;
  static constexpr int kNumBars = 8;
  static constexpr int kMisc = kBars + 8 * kNumBars;
  static constexpr int kTotal = kMisc + 16;
  static constexpr int kDynamic = kTotal + 1024;  // slack for manual 1024-byte alignment
};

// Online-softmax step of one thread (= one query row) for one 128-key tile; like softmax_tile of fwd_tc.cuh, but
// P goes back to TMEM as fp32 over the S columns it came from.
template <int D, class M>
__device__ __forceinline__ void softmax_tile_f32(uint32_t tS, uint32_t tO, uint32_t lane_sel, bool first, bool full,
                                                 int klim, int qg, int kg0, int n, const MaskArgs& margs, float c,
                                                 float& m_used, float& l) {
  uint32_t sreg[kTile];
#pragma unroll
  for (int q4 = 0; q4 < 4; ++q4) tmem_ld32(tS + lane_sel + q4 * 32, sreg + q4 * 32);
  tmem_wait_ld();
  if (!full) {
    if (interval_rows<M>::value) {  // two per-row bounds instead of a mask() call per element
      int c_lo, c_hi;
      row_window<M, true>(qg, kg0, klim, n, margs, c_lo, c_hi);
#pragma unroll
      for (int cidx = 0; cidx < kTile; ++cidx) sreg[cidx] = (cidx >= c_lo && cidx <= c_hi) ? sreg[cidx] : 0xff800000u;
    } else {
#pragma unroll
      for (int cidx = 0; cidx < kTile; ++cidx) {
        const bool vis = cidx < klim && M::mask(qg, kg0 + cidx, n, margs);
        sreg[cidx] = vis ? sreg[cidx] : 0xff800000u;  // -inf
      }
    }
  }
  float mx0 = -CUDART_INF_F, mx1 = -CUDART_INF_F, mx2 = -CUDART_INF_F, mx3 = -CUDART_INF_F;
#pragma unroll
  for (int i = 0; i < kTile; i += 8) {
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
#pragma unroll
  for (int i = 0; i < kTile; i += 4) {
    const uint64_t e0 = ex2_pair(ffma2(pk2u(sreg[i], sreg[i + 1]), c2, nm2), false);
    const uint64_t e1 = ex2_pair(ffma2(pk2u(sreg[i + 2], sreg[i + 3]), c2, nm2), false);
    l0 = fadd2(l0, e0);
    l1 = fadd2(l1, e1);
    float p0, p1, p2, p3;
    upk2(e0, p0, p1);
    upk2(e1, p2, p3);
    sreg[i] = to_tf32(p0);  // rounded to nearest: the tensor core would truncate
    sreg[i + 1] = to_tf32(p1);
    sreg[i + 2] = to_tf32(p2);
    sreg[i + 3] = to_tf32(p3);
  }
  {
    float a0, a1, a2, a3;
    upk2(l0, a0, a1);
    upk2(l1, a2, a3);
    l += (a0 + a1) + (a2 + a3);
  }
#pragma unroll
  for (int q4 = 0; q4 < 4; ++q4) tmem_st32(tS + lane_sel + q4 * 32, sreg + q4 * 32);
}

// Normalise this thread's O row and stage it as fp32 in the 128B-swizzled TMA box layout (one 128-byte line of 32
// channels per column block); also writes the row's LSE.
template <int D>
__device__ __forceinline__ void stage_output_row_f32(uint8_t* sO, uint32_t tO, uint32_t lane_sel, int r, bool have,
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
    const bool keep = have && row_valid && l != 0.f;
    uint8_t* line = sO + q4 * (kTile * 128) + r * 128;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (keep)
        v = make_float4(__uint_as_float(oreg[4 * u]) * inv, __uint_as_float(oreg[4 * u + 1]) * inv,
                        __uint_as_float(oreg[4 * u + 2]) * inv, __uint_as_float(oreg[4 * u + 3]) * inv);
      *reinterpret_cast<float4*>(line + ((u ^ (r & 7)) * 16)) = v;
    }
  }
  if (lse_ptr != nullptr) {
    float v = 0.f;
    if (row_valid) v = (l == 0.f) ? -CUDART_INF_F : m_used + lg2(l);
    *lse_ptr = v;
  }
}

template <int D, class M>
__global__ void __launch_bounds__(kFwdThreads, (D == 64 ? 2 : 1))
fwd_tf32_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO, FwdTcParams p) {
  using L = FwdTf32Smem<D>;
  constexpr int kChunks = D / 32;              // 32-channel (128-byte) column blocks per tile
  constexpr int kChunkBytes = kTile * 128;     // one column block: 128 rows x 128 bytes
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
    // Every row of this tile is padding: O = 0, LSE = 0 (chill_fwd.py:70-71).
    float* obase = reinterpret_cast<float*>(p.o) + b * p.o_sb + h * p.o_sh;
    const int rows = imin(kTile, g.Lq - qb);
    for (int idx = threadIdx.x; idx < rows * (D / 4); idx += kFwdThreads) {
      const int r = idx / (D / 4), c = idx % (D / 4);
      *reinterpret_cast<float4*>(obase + (qb + r) * p.o_sl + c * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (p.lse != nullptr)
      for (int r = threadIdx.x; r < rows; r += kFwdThreads) p.lse[b * p.lse_sb + h * p.lse_sh + (qb + r) * p.lse_sl] = 0.f;
    return;
  }

  int kt_lo = 0, kt_hi = 0;      // [kt_lo, kt_hi) in units of 128 local key rows
  int full_lo = 0, full_hi = 0;  // global, half-open: keys visible to every row of the tile
  {
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
  const int n_tiles = kt_hi - kt_lo;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t sQ = base + L::kQ, sK = base + L::kK, sV = base + L::kV;
  const uint32_t bars = base + L::kBars;
  const uint32_t bar_q_full = bars, bar_s_full = bars + 8, bar_p_full = bars + 16, bar_o_full = bars + 24,
                 bar_k_full = bars + 32, bar_k_empty = bars + 40, bar_v_full = bars + 48, bar_v_empty = bars + 56;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen_base + L::kMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + L::kMisc + 4);
  const Guard guard{p.status, abort_flag};

  if (warp == 4) {
    if (lane == 0) {
      *abort_flag = 0;
      mbar_init(bar_q_full, 1);
      mbar_init(bar_s_full, 1);
      mbar_init(bar_p_full, 4);
      mbar_init(bar_o_full, 1);
      mbar_init(bar_k_full, 1);
      mbar_init(bar_k_empty, 1);
      mbar_init(bar_v_full, 1);
      mbar_init(bar_v_empty, 1);
      fence_barrier_init();
      fence_proxy_async_smem();
      if (n_tiles > 0) {
        mbar_arrive_expect_tx(bar_q_full, L::kTileBytes);
        for (int c = 0; c < kChunks; ++c) tma_load_4d(sQ + c * kChunkBytes, &tmQ, bar_q_full, c * 32, qb, h, b);
        mbar_arrive_expect_tx(bar_k_full, L::kTileBytes);
        for (int c = 0; c < kChunks; ++c) tma_load_4d(sK + c * kChunkBytes, &tmK, bar_k_full, c * 32, kt_lo * kTile, hk, b);
        mbar_arrive_expect_tx(bar_v_full, L::kTileBytes);
        for (int c = 0; c < kChunks; ++c) tma_load_4d(sV + c * kChunkBytes, &tmV, bar_v_full, c * 32, kt_lo * kTile, hk, b);
      }
    }
    __syncwarp();
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemColsFwd);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem;          // S / P columns (fp32 both)
  const uint32_t tO = tmem + kTile;  // O columns

  if (warp == 4) {
    reg_dealloc<kFwdOtherRegs>();
    // ------------------------------------------------------------------- TMA producer (single-stage K and V)
    if (lane == 0 && n_tiles > 0) {
      bool ok = true;
      for (int j = 1; j < n_tiles && ok; ++j) {  // tile 0 was issued during set-up
        const uint32_t ph = (uint32_t)j & 1u;
        const int krow = (kt_lo + j) * kTile;
        ok = mbar_wait(bar_k_empty, ph ^ 1u, guard, kStProducer);
        if (!ok) break;
        mbar_arrive_expect_tx(bar_k_full, L::kTileBytes);
        for (int c = 0; c < kChunks; ++c) tma_load_4d(sK + c * kChunkBytes, &tmK, bar_k_full, c * 32, krow, hk, b);
        ok = mbar_wait(bar_v_empty, ph ^ 1u, guard, kStProducer);
        if (!ok) break;
        mbar_arrive_expect_tx(bar_v_full, L::kTileBytes);
        for (int c = 0; c < kChunks; ++c) tma_load_4d(sV + c * kChunkBytes, &tmV, bar_v_full, c * 32, krow, hk, b);
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 5) {
    reg_dealloc<kFwdOtherRegs>();
    // --------------------------------------------------------------------- MMA issuer
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_s = make_idesc<float>(kTile, kTile, false, false);
      constexpr uint32_t idesc_o = make_idesc<float>(kTile, D, false, true);
      constexpr uint32_t hi_k = desc_hi_sw128(1024);        // K-major tiles: 8-row groups 1 KB apart
      constexpr uint32_t hi_v = desc_hi_sw128_base32(512);  // MN-major fp32 tile: 4-row groups 512 B apart
      const uint32_t q_lo = desc_lo_sw128(sQ, 16), k_lo = desc_lo_sw128(sK, 16);
      const uint32_t v_lo = desc_lo_sw128(sV, kChunkBytes);  // channel blocks 16 KB apart
      bool ok = mbar_wait(bar_q_full, 0, guard, kStMma);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const uint32_t ph = (uint32_t)j & 1u;
        ok = mbar_wait(bar_k_full, ph, guard, kStMma);
        if (!ok) break;
        tc_fence_after();
        // S = Q K^T: both K-major; 8 channels (32 bytes) per instruction
#pragma unroll
        for (int kk = 0; kk < D / 8; ++kk)
          mma_ss_tf32(tS, q_lo + kmajor_step(kk), k_lo + kmajor_step(kk), hi_k, idesc_s, kk > 0 ? 1u : 0u);
        mma_commit(bar_k_empty);
        mma_commit(bar_s_full);
        ok = mbar_wait(bar_p_full, ph, guard, kStMma);
        if (!ok) break;
        ok = mbar_wait(bar_v_full, ph, guard, kStMma);
        if (!ok) break;
        tc_fence_after();
        // O += P V: P (128 x 128, fp32) from TMEM, 8 keys = 8 columns and 1 KB of V per instruction
#pragma unroll
        for (int kk = 0; kk < kTile / 8; ++kk)
          mma_ts_tf32(tO, tS + kk * 8, v_lo + kk * 64, hi_v, idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
        mma_commit(bar_v_empty);
      }
      if (ok) mma_commit(bar_o_full);
    }
  } else if (warp >= 6) {
    reg_dealloc<kFwdOtherRegs>();  // idle warps of the second warpgroup only give their registers back
  } else {
    reg_alloc<kFwdSoftmaxRegs>();
    // --------------------------------------------------------- softmax + epilogue warps
    const int r = warp * 32 + lane;  // row inside the tile == TMEM lane
    const uint32_t lane_sel = (uint32_t)(warp * 32) << 16;
    const int qg = qg0 + r;
    const float c = g.scale * kLog2e;
    float m_used = -CUDART_INF_F, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int kt = kt_lo + j;
      const int kg0 = kt * kTile + g.k_off;
      ok = mbar_wait(bar_s_full, (uint32_t)j & 1u, guard, kStSoftmax);
      ok = __all_sync(0xffffffffu, ok);  // keep the warp converged for the .sync.aligned TMEM accesses
      if (!ok) break;
      tc_fence_after();
      const bool full = M::kHasKFullRange && kg0 >= full_lo && kg0 + kTile <= full_hi && kg0 + kTile <= n &&
                        kt * kTile + kTile <= g.Lk;
      const int klim = imin(n - kg0, g.Lk - kt * kTile);  // columns >= klim do not exist
      softmax_tile_f32<D, M>(tS, tO, lane_sel, j == 0, full, klim, qg, kg0, n, g.margs, c, m_used, l);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p_full);  // one arrival per softmax warp
    }

    // ---- epilogue: O / l -> fp32 -> swizzled shared memory (Q's buffer) -> TMA store
    if (ok && n_tiles > 0) ok = mbar_wait(bar_o_full, 0, guard, kStEpilogue);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    const bool row_valid = qg < n;
    stage_output_row_f32<D>(gen_base + L::kQ, tO, lane_sel, r, n_tiles > 0 && ok, row_valid, l, m_used,
                            (p.lse != nullptr && qb + r < g.Lq) ? p.lse + b * p.lse_sb + h * p.lse_sh + (qb + r) * p.lse_sl
                                                                 : nullptr);
    fence_proxy_async_smem();
    named_bar_sync(1, 128);
    if (threadIdx.x == 0) {
      for (int cc = 0; cc < kChunks; ++cc) tma_store_4d(&tmO, base + L::kQ + cc * kChunkBytes, cc * 32, qb, h, b);
      tma_store_commit();
      tma_store_wait_read();  // shared memory may be released; the global writes complete by kernel end
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem, kTmemColsFwd);
}

}  // namespace tc
}  // namespace chill
