// Backward attention for fp32 tensors on the tensor cores in TF32 (tcgen05.mma.kind::tf32, sm_100a), head dim 64 / 128.
// What precision="tf32" asks for in the reference's backward kernels (chill_bwd_dq.py:312,330 and
// chill_bwd_dkdv.py:347-508 take input_precision like the forward does).
//
// Two kernels with the partition of bwd_tc.cuh (no accumulation crosses CTAs, results are bitwise reproducible):
//   bwd_dkdv_tf32_kernel  one CTA per (batch, kv head, tile of 128 keys); per tile of TO queries of every head of the group
//                         S^T = K Q^T, dP^T = V dO^T, P^T = 2^(S^T c - LSE), dS^T = P^T (dP^T - delta),
//                         dV += P^T dO, dK += dS^T Q
//   bwd_dq_tf32_kernel    one CTA per (batch, head, tile of 128 queries); per tile of TO keys
//                         S = Q K^T, dP = dO V^T, dS = 2^(S c - LSE) (dP - delta), dQ += dS K
// What differs from the 16-bit kernels is the element size:
//   * a tile row is D * 4 bytes = D / 32 column blocks of 128 bytes; an MMA step covers 8 elements;
//   * P^T / dS^T stay fp32: the compute warps round them to TF32 and write them back over the TMEM columns the
//     scores came from, from where they are the A operands of the accumulate GEMMs (8 columns per MMA step);
//   * an fp32 operand read MN-major (dO and Q as B of the dV / dK GEMMs, K as B of the dQ GEMM) needs the
//     "128-byte swizzle with 32-byte atoms" layout, a K-major one the plain 128-byte swizzle (a K-major descriptor
//     does not take the 32-byte-atom layout), so those tiles are loaded twice, once per layout.  Shared memory
//     then decides the size TO of the streamed tiles: 128 positions at head dim 64 (64 KB resident + 128 KB
//     streamed), 32 at head dim 128 (128 KB resident + 64 KB streamed).
// The kernels are deliberately plain: one ring stage, the tensor cores and the compute warps alternate.  They run
// at a few hundred TFLOP/s where the IEEE kernels (generic.cuh) that otherwise serve fp32 reach about one.
// Inputs are used as they are (the tensor core drops all but 10 mantissa bits); gradients match the fp64 oracle
// to about 1e-3 relative on N(0,1) inputs (the tests state 5e-3).
#pragma once
#include <type_traits>

#include "bwd_tc.cuh"
#include "fwd_tf32.cuh"

namespace chill {
namespace tc {

enum : int { kStTfProducer = 501, kStTfMma = 502, kStTfCompute = 503, kStTfEpilogue = 504 };

// D: head dim; TO: positions per streamed tile (queries in the dK/dV kernel, keys in the dQ kernel).
template <int D>
struct Tf32Shape {
  static constexpr int TO = (D == 64) ? 128 : 32;
  static constexpr int kChunks = D / 32;                       // 128-byte column blocks per row
  static constexpr int kFixBytes = kTile * D * 4;              // a resident tile: 128 positions
  static constexpr int kFixChunkBytes = kTile * 128;
  static constexpr int kRingBytes = TO * D * 4;                // a streamed tile: TO positions
  static constexpr int kRingChunkBytes = TO * 128;
  static constexpr int kFixA = 0;                              // K (dkdv) or Q (dq), K-major
  static constexpr int kFixB = kFixA + kFixBytes;              // V (dkdv) or dO (dq), K-major
  static constexpr int kRing = kFixB + kFixBytes;              // up to four streamed tiles
  static constexpr int kRows = kRing + 4 * kRingBytes;         // per compute warp: -lse[TO/2], -delta[TO/2] (dkdv)
  static constexpr int kBars = kRows + 8 * 2 * 64 * 4;
  static constexpr int kNumBars = 6;
  static constexpr int kMisc = kBars + 8 * kNumBars;
  static constexpr int kTotal = kMisc + 16;
  static constexpr int kDynamic = kTotal + 1024;
  static_assert(kDynamic <= 232448, "exceeds the 227 KB of shared memory a CTA can opt in to");
  static_assert(256 + 2 * D <= 512, "TMEM columns");
  // 16-byte units to add to a K-major descriptor for MMA step kk (8 channels = 32 bytes) of a tile whose column
  // blocks are `chunk_bytes` apart
  __host__ __device__ static constexpr uint32_t kstep(int kk, int chunk_bytes) {
    return (uint32_t)((kk / 4) * (chunk_bytes / 16) + (kk % 4) * 2);
  }
};

template <int D, int ROWS>
__device__ __forceinline__ void tma_tile_f32(uint32_t dst, const CUtensorMap* map, uint32_t bar, int row, int h, int b) {
#pragma unroll
  for (int c = 0; c < D / 32; ++c) tma_load_4d(dst + c * (ROWS * 128), map, bar, c * 32, row, h, b);
}

// Write `rows` rows of D fp32 zeros starting at `base` (row stride `sl` elements).
template <int D>
__device__ __forceinline__ void zero_rows_f32(float* base, long long sl, int rows, int nthreads) {
  for (int idx = threadIdx.x; idx < rows * (D / 4); idx += nthreads) {
    const int r = idx / (D / 4), c = idx % (D / 4);
    *reinterpret_cast<float4*>(base + r * sl + c * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

// One chunk of CC (32 or 16) consecutive fp32 TMEM columns of this thread's lane.
template <int CC>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t* r) {
  if constexpr (CC == 32) tmem_ld32(taddr, r);
  else tmem_ld16(taddr, r);
}
template <int CC>
__device__ __forceinline__ void tmem_st_cols(uint32_t taddr, const uint32_t* r) {
  if constexpr (CC == 32) tmem_st32(taddr, r);
  else tmem_st16(taddr, r);
}

// ============================================================================ dK / dV
// TMEM: S^T / P^T at column 0 (TO columns), dP^T / dS^T at 128 (TO), dV at 256 (D), dK at 256 + D (D).
template <int D, class M>
__global__ void __launch_bounds__(kBwdThreads, 1)
bwd_dkdv_tf32_kernel(const __grid_constant__ CUtensorMap tmQk, const __grid_constant__ CUtensorMap tmQm,
                     const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                     const __grid_constant__ CUtensorMap tmdOk, const __grid_constant__ CUtensorMap tmdOm, BwdTcParams p) {
  using L = Tf32Shape<D>;
  constexpr int TO = L::TO;     // queries per streamed tile
  constexpr int CW = TO / 2;    // query columns per compute warp
  constexpr int CC = CW < 32 ? CW : 32;  // columns per TMEM access
  const Geo& g = p.g;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int hb, kt;
  cta_order((int)blockIdx.x, g.B * g.Hkv, (g.Lk + kTile - 1) / kTile, hb, kt);
  const int hk = hb % g.Hkv, b = hb / g.Hkv;
  const int G = g.H / g.Hkv;
  const int kb = kt * kTile;
  const int kg0 = kb + g.k_off;
  int n = g.seq_len;
  if (g.lens != nullptr) n = imin(n, g.lens[b]);

  int qt_lo = 0, qt_hi = 0, full_lo = 0, full_hi = 0;  // query tiles of TO rows
  if (kg0 < n) {
    int lo, hi;
    tile_range<M, false>(kg0, imin(kTile, g.Lk - kb), n, g.margs, lo, hi);
    const int lo_l = imax(lo - g.q_off, 0);
    const int hi_l = imin(imin(hi, n - 1) - g.q_off, g.Lq - 1);
    if (hi_l >= lo_l) {
      qt_lo = lo_l / TO;
      qt_hi = hi_l / TO + 1;
    }
    if (M::kHasQFullRange) M::q_full_range_for_k(kg0, kTile, n, g.margs, full_lo, full_hi);
  }
  const int n_qt = qt_hi - qt_lo;
  const int n_it = n_qt * G;
  float* dk_base = reinterpret_cast<float*>(p.dk) + b * p.dk_sb + hk * p.dk_sh + (long long)kb * p.dk_sl;
  float* dv_base = reinterpret_cast<float*>(p.dv) + b * p.dv_sb + hk * p.dv_sh + (long long)kb * p.dv_sl;
  if (n_it == 0) {  // nobody attends these keys
    const int rows = imin(kTile, g.Lk - kb);
    zero_rows_f32<D>(dk_base, p.dk_sl, rows, kBwdThreads);
    zero_rows_f32<D>(dv_base, p.dv_sl, rows, kBwdThreads);
    return;
  }

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t sK = base + L::kFixA, sV = base + L::kFixB;
  const uint32_t sQk = base + L::kRing, sQm = sQk + L::kRingBytes, sdOk = sQm + L::kRingBytes, sdOm = sdOk + L::kRingBytes;
  float* rows_s = reinterpret_cast<float*>(gen_base + L::kRows);
  const uint32_t bars = base + L::kBars;
  const uint32_t bar_kv_full = bars, bar_ring_full = bars + 8, bar_ring_empty = bars + 16, bar_sdp_full = bars + 24,
                 bar_ds_full = bars + 32, bar_acc_full = bars + 40;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen_base + L::kMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + L::kMisc + 4);
  const Guard guard{p.status, abort_flag};

  if (warp == 8) {
    if (lane == 0) {
      *abort_flag = 0;
      mbar_init(bar_kv_full, 1);
      mbar_init(bar_ring_full, 1);
      mbar_init(bar_ring_empty, 1);
      mbar_init(bar_sdp_full, 1);
      mbar_init(bar_ds_full, kBwdComputeThreads / 32);
      mbar_init(bar_acc_full, 1);
      fence_barrier_init();
      fence_proxy_async_smem();
      mbar_arrive_expect_tx(bar_kv_full, 2 * L::kFixBytes);
      tma_tile_f32<D, kTile>(sK, &tmK, bar_kv_full, kb, hk, b);
      tma_tile_f32<D, kTile>(sV, &tmV, bar_kv_full, kb, hk, b);
    }
    __syncwarp();
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemColsBwd);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tSt = tmem, tdPt = tmem + 128, tdV = tmem + 256, tdK = tmem + 256 + D;

  if (warp == 8) {
    // --------------------------------------------------------------------- TMA producer (one ring stage)
    if (lane == 0) {
      bool ok = true;
      for (int it = 0; it < n_it && ok; ++it) {
        const int h = hk * G + it / n_qt;
        const int qrow = (qt_lo + it % n_qt) * TO;
        ok = mbar_wait(bar_ring_empty, ((uint32_t)it & 1u) ^ 1u, guard, kStTfProducer);
        if (!ok) break;
        mbar_arrive_expect_tx(bar_ring_full, 4 * L::kRingBytes);
        tma_tile_f32<D, TO>(sQk, &tmQk, bar_ring_full, qrow, h, b);
        tma_tile_f32<D, TO>(sQm, &tmQm, bar_ring_full, qrow, h, b);
        tma_tile_f32<D, TO>(sdOk, &tmdOk, bar_ring_full, qrow, h, b);
        tma_tile_f32<D, TO>(sdOm, &tmdOm, bar_ring_full, qrow, h, b);
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 9) {
    // ----------------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc<float>(kTile, TO, false, false);
      constexpr uint32_t idesc_acc = make_idesc<float>(kTile, D, false, true);
      constexpr uint32_t hi_k = desc_hi_sw128(1024);         // K-major tiles: 8-row groups 1 KB apart
      constexpr uint32_t hi_m = desc_hi_sw128_base32(512);   // MN-major fp32 tiles: 4-row groups 512 B apart
      const uint32_t k_lo = desc_lo_sw128(sK, 16), v_lo = desc_lo_sw128(sV, 16);
      const uint32_t qk_lo = desc_lo_sw128(sQk, 16), dok_lo = desc_lo_sw128(sdOk, 16);
      const uint32_t qm_lo = desc_lo_sw128(sQm, L::kRingChunkBytes), dom_lo = desc_lo_sw128(sdOm, L::kRingChunkBytes);
      bool ok = mbar_wait(bar_kv_full, 0, guard, kStTfMma);
      for (int it = 0; it < n_it && ok; ++it) {
        const uint32_t par = (uint32_t)it & 1u;
        ok = mbar_wait(bar_ring_full, par, guard, kStTfMma);
        if (!ok) break;
        tc_fence_after();
        // S^T = K Q^T and dP^T = V dO^T: 8 channels (32 bytes) per instruction.  They overwrite P^T / dS^T of the
        // previous query tile, which the accumulate GEMMs issued before them have consumed (issue order).
#pragma unroll
        for (int kk = 0; kk < D / 8; ++kk)
          mma_ss_tf32(tSt, k_lo + L::kstep(kk, L::kFixChunkBytes), qk_lo + L::kstep(kk, L::kRingChunkBytes), hi_k, idesc_s,
                      kk > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < D / 8; ++kk)
          mma_ss_tf32(tdPt, v_lo + L::kstep(kk, L::kFixChunkBytes), dok_lo + L::kstep(kk, L::kRingChunkBytes), hi_k, idesc_s,
                      kk > 0 ? 1u : 0u);
        mma_commit(bar_sdp_full);
        ok = mbar_wait(bar_ds_full, par, guard, kStTfMma);
        if (!ok) break;
        tc_fence_after();
        // dV += P^T dO, dK += dS^T Q: A from TMEM (8 queries = 8 columns per step), B = 8 rows (1 KB) of dO / Q
#pragma unroll
        for (int kk = 0; kk < TO / 8; ++kk)
          mma_ts_tf32(tdV, tSt + kk * 8, dom_lo + kk * 64, hi_m, idesc_acc, (it > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < TO / 8; ++kk)
          mma_ts_tf32(tdK, tdPt + kk * 8, qm_lo + kk * 64, hi_m, idesc_acc, (it > 0 || kk > 0) ? 1u : 0u);
        mma_commit(bar_ring_empty);
      }
      if (ok) mma_commit(bar_acc_full);
    }
  } else {
    // ------------------------------------------------------------------- compute warps
    const int wg = warp >> 2;                       // column half: query columns [CW wg, CW wg + CW)
    const int r = (warp & 3) * 32 + lane;           // key row inside the tile == TMEM lane
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
    const int c0 = wg * CW;
    const int kg = kg0 + r;
    const bool key_ok = kg < n && kb + r < g.Lk;
    const float c = g.scale * kLog2e;
    float* slot = rows_s + warp * 128;  // warp-private: [0, CW) -LSE, [64, 64 + CW) -delta of this warp's columns
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const uint32_t par = (uint32_t)it & 1u;
      const int h = hk * G + it / n_qt;
      const int qi = qt_lo + it % n_qt;
      const int qg0 = qi * TO + g.q_off;
      __syncwarp();
      for (int e = lane; e < CW; e += 32) {
        const int qrow = qi * TO + c0 + e;
        const bool in = qrow < g.Lq;
        const float lv = p.lse[b * p.lse_sb + h * p.lse_sh + (in ? qrow : 0) * p.lse_sl];
        const float dl = p.delta[((long long)b * g.H + h) * g.Lq + (in ? qrow : 0)];
        slot[e] = (lv == -CUDART_INF_F) ? 0.f : -lv;
        slot[64 + e] = -dl;
      }
      __syncwarp();
      const bool full = M::kHasQFullRange && qg0 >= full_lo && qg0 + TO <= full_hi && qg0 + TO <= n &&
                        qi * TO + TO <= g.Lq && kg0 + kTile <= n && kb + kTile <= g.Lk;
      const int qlim = imin(n - qg0, g.Lq - qi * TO);
      int w_lo = 0, w_hi = -1;  // visible query columns of this key row inside the tile (interval functors)
      if (interval_rows<M>::value && !full && key_ok) row_window<M, false>(kg, qg0, qlim, n, g.margs, w_lo, w_hi);
      ok = mbar_wait(bar_sdp_full, par, guard, kStTfCompute);
      ok = __all_sync(0xffffffffu, ok);  // keep the warp converged for the .sync.aligned TMEM accesses
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int part = 0; part < CW / CC; ++part) {
        const int cb = c0 + part * CC;
        uint32_t sreg[CC], dpreg[CC];
        tmem_ld_cols<CC>(tSt + lane_sel + cb, sreg);
        tmem_ld_cols<CC>(tdPt + lane_sel + cb, dpreg);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < CC; ++j) {
          const int cq = cb + j;
          float pv = ex2(fmaf(__uint_as_float(sreg[j]), c, slot[part * CC + j]));
          bool vis = full;
          if (!full) {
            if (interval_rows<M>::value) vis = cq >= w_lo && cq <= w_hi;
            else vis = key_ok && cq < qlim && M::mask(qg0 + cq, kg, n, g.margs);
          }
          pv = vis ? pv : 0.f;
          const float ds = pv * (__uint_as_float(dpreg[j]) + slot[64 + part * CC + j]);
          sreg[j] = to_tf32(pv);
          dpreg[j] = to_tf32(ds);
        }
        tmem_st_cols<CC>(tSt + lane_sel + cb, sreg);    // P^T over the scores it came from
        tmem_st_cols<CC>(tdPt + lane_sel + cb, dpreg);  // dS^T over dP^T
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_ds_full);
    }

    // ---- epilogue: warps 0-3 store dV, warps 4-7 store dK * sm_scale, one fp32 row per thread
    if (ok) ok = mbar_wait(bar_acc_full, 0, guard, kStTfEpilogue);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    const uint32_t tacc = wg == 0 ? tdV : tdK;
    const float mul = wg == 0 ? 1.f : g.scale;
    float* out = (wg == 0 ? dv_base : dk_base) + (long long)r * (wg == 0 ? p.dv_sl : p.dk_sl);
#pragma unroll
    for (int q4 = 0; q4 < D / 32; ++q4) {
      uint32_t acc[32];
      if (ok) {
        tmem_ld32(tacc + lane_sel + q4 * 32, acc);
        tmem_wait_ld();
      }
      if (kb + r < g.Lk) {
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          float4 v4 = make_float4(0.f, 0.f, 0.f, 0.f);
          if (ok && key_ok)
            v4 = make_float4(__uint_as_float(acc[4 * u]) * mul, __uint_as_float(acc[4 * u + 1]) * mul,
                             __uint_as_float(acc[4 * u + 2]) * mul, __uint_as_float(acc[4 * u + 3]) * mul);
          *reinterpret_cast<float4*>(out + q4 * 32 + u * 4) = v4;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 8) tmem_dealloc(tmem, kTmemColsBwd);
}

// ================================================================================ dQ
// TMEM: S at column 0 (TO columns), dP / dS at 128 (TO), dQ at 256 (D).
template <int D, class M>
__global__ void __launch_bounds__(kBwdThreads, 1)
bwd_dq_tf32_kernel(const __grid_constant__ CUtensorMap tmQk, const __grid_constant__ CUtensorMap tmKk,
                   const __grid_constant__ CUtensorMap tmKm, const __grid_constant__ CUtensorMap tmV,
                   const __grid_constant__ CUtensorMap tmdOk, BwdTcParams p) {
  using L = Tf32Shape<D>;
  constexpr int TO = L::TO;     // keys per streamed tile
  constexpr int CW = TO / 2;
  constexpr int CC = CW < 32 ? CW : 32;
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

  int kt_lo = 0, kt_hi = 0, full_lo = 0, full_hi = 0;  // key tiles of TO rows
  if (qg0 < n) {
    int lo, hi;
    tile_range<M, true>(qg0, imin(kTile, g.Lq - qb), n, g.margs, lo, hi);
    const int lo_l = imax(lo - g.k_off, 0);
    const int hi_l = imin(imin(hi, n - 1) - g.k_off, g.Lk - 1);
    if (hi_l >= lo_l) {
      kt_lo = lo_l / TO;
      kt_hi = hi_l / TO + 1;
    }
    if (M::kHasKFullRange) M::k_full_range_for_q(qg0, kTile, n, g.margs, full_lo, full_hi);
  }
  const int n_it = kt_hi - kt_lo;
  float* dq_base = reinterpret_cast<float*>(p.dq) + b * p.dq_sb + h * p.dq_sh + (long long)qb * p.dq_sl;
  if (n_it == 0) {
    zero_rows_f32<D>(dq_base, p.dq_sl, imin(kTile, g.Lq - qb), kBwdThreads);
    return;
  }

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t sQ = base + L::kFixA, sdO = base + L::kFixB;
  const uint32_t sKk = base + L::kRing, sKm = sKk + L::kRingBytes, sVk = sKm + L::kRingBytes;
  const uint32_t bars = base + L::kBars;
  const uint32_t bar_q_full = bars, bar_ring_full = bars + 8, bar_ring_empty = bars + 16, bar_sdp_full = bars + 24,
                 bar_ds_full = bars + 32, bar_acc_full = bars + 40;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen_base + L::kMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + L::kMisc + 4);
  const Guard guard{p.status, abort_flag};

  if (warp == 8) {
    if (lane == 0) {
      *abort_flag = 0;
      mbar_init(bar_q_full, 1);
      mbar_init(bar_ring_full, 1);
      mbar_init(bar_ring_empty, 1);
      mbar_init(bar_sdp_full, 1);
      mbar_init(bar_ds_full, kBwdComputeThreads / 32);
      mbar_init(bar_acc_full, 1);
      fence_barrier_init();
      fence_proxy_async_smem();
      mbar_arrive_expect_tx(bar_q_full, 2 * L::kFixBytes);
      tma_tile_f32<D, kTile>(sQ, &tmQk, bar_q_full, qb, h, b);
      tma_tile_f32<D, kTile>(sdO, &tmdOk, bar_q_full, qb, h, b);
    }
    __syncwarp();
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemColsBwd);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem, tdP = tmem + 128, tdQ = tmem + 256;

  if (warp == 8) {
    if (lane == 0) {
      bool ok = true;
      for (int it = 0; it < n_it && ok; ++it) {
        const int krow = (kt_lo + it) * TO;
        ok = mbar_wait(bar_ring_empty, ((uint32_t)it & 1u) ^ 1u, guard, kStTfProducer);
        if (!ok) break;
        mbar_arrive_expect_tx(bar_ring_full, 3 * L::kRingBytes);
        tma_tile_f32<D, TO>(sKk, &tmKk, bar_ring_full, krow, hk, b);
        tma_tile_f32<D, TO>(sKm, &tmKm, bar_ring_full, krow, hk, b);
        tma_tile_f32<D, TO>(sVk, &tmV, bar_ring_full, krow, hk, b);
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 9) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc<float>(kTile, TO, false, false);
      constexpr uint32_t idesc_acc = make_idesc<float>(kTile, D, false, true);
      constexpr uint32_t hi_k = desc_hi_sw128(1024);
      constexpr uint32_t hi_m = desc_hi_sw128_base32(512);
      const uint32_t q_lo = desc_lo_sw128(sQ, 16), do_lo = desc_lo_sw128(sdO, 16);
      const uint32_t kk_lo = desc_lo_sw128(sKk, 16), vk_lo = desc_lo_sw128(sVk, 16);
      const uint32_t km_lo = desc_lo_sw128(sKm, L::kRingChunkBytes);
      bool ok = mbar_wait(bar_q_full, 0, guard, kStTfMma);
      for (int it = 0; it < n_it && ok; ++it) {
        const uint32_t par = (uint32_t)it & 1u;
        ok = mbar_wait(bar_ring_full, par, guard, kStTfMma);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 8; ++kk)  // S = Q K^T
          mma_ss_tf32(tS, q_lo + L::kstep(kk, L::kFixChunkBytes), kk_lo + L::kstep(kk, L::kRingChunkBytes), hi_k, idesc_s,
                      kk > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < D / 8; ++kk)  // dP = dO V^T
          mma_ss_tf32(tdP, do_lo + L::kstep(kk, L::kFixChunkBytes), vk_lo + L::kstep(kk, L::kRingChunkBytes), hi_k, idesc_s,
                      kk > 0 ? 1u : 0u);
        mma_commit(bar_sdp_full);
        ok = mbar_wait(bar_ds_full, par, guard, kStTfMma);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < TO / 8; ++kk)  // dQ += dS K: 8 keys = 8 columns of dS, 8 rows of K per step
          mma_ts_tf32(tdQ, tdP + kk * 8, km_lo + kk * 64, hi_m, idesc_acc, (it > 0 || kk > 0) ? 1u : 0u);
        mma_commit(bar_ring_empty);
      }
      if (ok) mma_commit(bar_acc_full);
    }
  } else {
    const int wg = warp >> 2;                       // column half: key columns [CW wg, CW wg + CW)
    const int r = (warp & 3) * 32 + lane;           // query row inside the tile == TMEM lane
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
    const int c0 = wg * CW;
    const int qg = qg0 + r;
    const bool row_ok = qg < n && qb + r < g.Lq;
    const float c = g.scale * kLog2e;
    float nlse = 0.f, ndelta = 0.f;
    if (qb + r < g.Lq) {
      const float lv = p.lse[b * p.lse_sb + h * p.lse_sh + (qb + r) * p.lse_sl];
      nlse = (lv == -CUDART_INF_F) ? 0.f : -lv;
      ndelta = -p.delta[((long long)b * g.H + h) * g.Lq + qb + r];
    }
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const uint32_t par = (uint32_t)it & 1u;
      const int kt = kt_lo + it;
      const int kg0 = kt * TO + g.k_off;
      const bool full = M::kHasKFullRange && kg0 >= full_lo && kg0 + TO <= full_hi && kg0 + TO <= n &&
                        kt * TO + TO <= g.Lk && qg0 + kTile <= n && qb + kTile <= g.Lq;
      const int klim = imin(n - kg0, g.Lk - kt * TO);
      int w_lo = 0, w_hi = -1;
      if (interval_rows<M>::value && !full && row_ok) row_window<M, true>(qg, kg0, klim, n, g.margs, w_lo, w_hi);
      ok = mbar_wait(bar_sdp_full, par, guard, kStTfCompute);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int part = 0; part < CW / CC; ++part) {
        const int cb = c0 + part * CC;
        uint32_t sreg[CC], dpreg[CC];
        tmem_ld_cols<CC>(tS + lane_sel + cb, sreg);
        tmem_ld_cols<CC>(tdP + lane_sel + cb, dpreg);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < CC; ++j) {
          const int col = cb + j;
          float pv = ex2(fmaf(__uint_as_float(sreg[j]), c, nlse));
          bool vis = full;
          if (!full) {
            if (interval_rows<M>::value) vis = col >= w_lo && col <= w_hi;
            else vis = row_ok && col < klim && M::mask(qg, kg0 + col, n, g.margs);
          }
          pv = vis ? pv : 0.f;
          dpreg[j] = to_tf32(pv * (__uint_as_float(dpreg[j]) + ndelta));
        }
        tmem_st_cols<CC>(tdP + lane_sel + cb, dpreg);  // dS over dP
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_ds_full);
    }

    // ---- epilogue: dQ * sm_scale; warps 0-3 take channels [0, D/2), warps 4-7 the rest
    if (ok) ok = mbar_wait(bar_acc_full, 0, guard, kStTfEpilogue);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
#pragma unroll
    for (int qq = 0; qq < D / 64; ++qq) {
      const int q4 = wg * (D / 64) + qq;  // group of 32 channels
      uint32_t acc[32];
      if (ok) {
        tmem_ld32(tdQ + lane_sel + q4 * 32, acc);
        tmem_wait_ld();
      }
      if (qb + r < g.Lq) {
        float* out = dq_base + (long long)r * p.dq_sl + q4 * 32;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          float4 v4 = make_float4(0.f, 0.f, 0.f, 0.f);
          if (ok && row_ok)
            v4 = make_float4(__uint_as_float(acc[4 * u]) * g.scale, __uint_as_float(acc[4 * u + 1]) * g.scale,
                             __uint_as_float(acc[4 * u + 2]) * g.scale, __uint_as_float(acc[4 * u + 3]) * g.scale);
          *reinterpret_cast<float4*>(out + u * 4) = v4;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 8) tmem_dealloc(tmem, kTmemColsBwd);
}

// ---------------------------------------------------------------------------- launcher
// maps (fp32; "ring" maps have boxes of Tf32Shape<D>::TO rows, the others of 128; mn = 32-byte-atom swizzle):
//   0 Q km ring, 1 Q mn ring, 2 dO km ring, 3 dO mn ring, 4 K km, 5 V km                (dK/dV kernel)
//   6 Q km, 7 dO km, 8 K km ring, 9 K mn ring, 10 V km ring                              (dQ kernel)
constexpr int kBwdTf32Maps = 11;

template <int D, class M>
int launch_bwd_tf32_one(const CUtensorMap* maps, const BwdTcParams& p, cudaStream_t st) {
  auto kdkdv = bwd_dkdv_tf32_kernel<D, M>;
  auto kdq = bwd_dq_tf32_kernel<D, M>;
  constexpr int smem = Tf32Shape<D>::kDynamic;
  struct TagA {};
  struct TagB {};
  cudaError_t e = ensure_dynamic_smem<TagA>(kdkdv, smem);
  if (e != cudaSuccess) return (int)e;
  e = ensure_dynamic_smem<TagB>(kdq, smem);
  if (e != cudaSuccess) return (int)e;
  const Geo& g = p.g;
  if (p.which & 1) {
    dim3 gk((unsigned)(((g.Lk + kTile - 1) / kTile) * g.Hkv * g.B), 1, 1);
    kdkdv<<<gk, kBwdThreads, smem, st>>>(maps[0], maps[1], maps[4], maps[5], maps[2], maps[3], p);
    e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
  }
  if (p.which & 2) {
    dim3 gq((unsigned)(((g.Lq + kTile - 1) / kTile) * g.H * g.B), 1, 1);
    kdq<<<gq, kBwdThreads, smem, st>>>(maps[6], maps[8], maps[9], maps[10], maps[7], p);
  }
  return (int)cudaGetLastError();
}

template <class M>
int launch_bwd_tf32(int D, const CUtensorMap* maps, const BwdTcParams& p, cudaStream_t st) {
  if (D == 64) return launch_bwd_tf32_one<64, M>(maps, p, st);
  if (D == 128) return launch_bwd_tf32_one<128, M>(maps, p, st);
  return (int)cudaErrorInvalidValue;
}

}  // namespace tc
}  // namespace chill
