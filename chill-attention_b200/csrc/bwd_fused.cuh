// Backward attention in ONE kernel with five GEMMs per (query tile, key tile) pair (sm_100a, 16-bit inputs,
// head dim 64 or 128).  The two-kernel backward in bwd_tc.cuh computes S and dP twice (seven GEMMs) so that
// no accumulation crosses CTAs; here a CTA owns a tile of 128 keys, keeps dK and dV in TMEM as that kernel
// does, and additionally forms the partial product dQ_tile = dS K for every query tile it visits.  The partial
// products of the CTAs that share a query tile are summed in an fp32 accumulator in global memory with bulk
// reductions of the copy engine (cp.reduce.async.bulk ... add.f32), and a small second kernel scales and rounds
// the sums to the output type.
// fp32 additions commute only up to rounding, so dQ can differ in the last bits between two runs; dK and dV
// stay deterministic.  Reference math: chill_attention/chill_bwd_dkdv.py:347-508 and chill_bwd_dq.py:300-394.
//
// Per query tile u (all MMAs 128 x 128 x 16 steps):
//     S^T = K Q^T, dP^T = V dO^T                                  (fp32 in TMEM)
//     P^T = 2^(S^T c - LSE)             -> 16-bit over S^T in TMEM, A operand of  dV += P^T dO
//     dS^T = P^T (dP^T - delta)         -> 16-bit tile in shared memory [key][query]; read K-major it is the
//                                          A operand of dK += dS^T Q, read MN-major the A operand of dQ = dS K
// TMEM (512 columns): S^T | dP^T (re-used for the dQ tile once the compute warps have read dP^T) | dV | dK.
// Shared memory (D = 128): K, V, two stages of [Q | dO]; the dS^T tile overlays the dO slot of its own stage
// once dV(u) has consumed dO(u) (no 32 KB are left for a buffer of its own; D = 64 has one).
//
// Tensor-core order in steady state, chosen so that every wait of the issuing thread has been satisfied long
// before it is reached:
//     dQ(u), dK(u)        need dS^T(u)           | compute warps: exponentials of S^T(u+1)
//     dP^T(u+1)           needs dQ(u) drained    | drain warps read dQ(u) while dK(u) runs
//     dV(u+1)             needs P^T(u+1)         | compute warps: dS^T(u+1)
//     S^T(u+2)
//
// Roles (512 threads, register budgets re-balanced per warpgroup with setmaxnreg): warps 0-7 compute (thread
// (w % 4) * 32 + lane owns key row = TMEM lane; warps 0-3 / 4-7 split the query columns), warps 8-11 drain the
// dQ tiles (TMEM -> registers -> shared memory -> bulk reductions into global memory), warp 12 is the TMA producer and owns the TMEM allocation,
// warp 13 issues the MMAs.
#pragma once
#include <type_traits>

#include "bwd_tc.cuh"

namespace chill {
namespace tc {

constexpr int kFusedThreads = 512;
constexpr int kFusedComputeRegs = 160;  // 256 * 160 + 128 * 136 + 128 * 56 = 65536
constexpr int kFusedDrainRegs = 136;    // a drain thread holds one fp32 row of the dQ tile (D registers)
constexpr int kFusedOtherRegs = 56;

enum : int { kStFusProducer = 401, kStFusMma = 402, kStFusCompute = 403, kStFusDrain = 404, kStFusEpilogue = 405 };

// Adds `bytes` of fp32 data in shared memory to global memory (both 16-byte aligned, bytes a multiple of 16); the
// copy engine reads the shared memory asynchronously: see bulk_wait_read.
__device__ __forceinline__ void bulk_reduce_add_f32(float* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(dst), "r"(src_smem),
               "r"(bytes)
               : "memory");
}
// Waits until all but the N most recent bulk groups of this thread have finished reading shared memory.
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

template <int D>
struct FusedSmem {
  static constexpr int kTileBytes = kTile * D * 2;
  static constexpr int kStages = 2;
  static constexpr int kDsBytes = kTile * kTile * 2;
  static constexpr bool kDsOverlay = (kTileBytes >= kDsBytes);  // dS^T lives in the dO slot of its stage
  static constexpr int kK = 0;
  static constexpr int kV = kK + kTileBytes;
  static constexpr int kRing = kV + kTileBytes;  // per stage: [Q | dO]
  static constexpr int kDs = kRing + kStages * 2 * kTileBytes;
  static constexpr int kRows = kDs + (kDsOverlay ? 0 : kDsBytes);  // per compute warp: -lse[64], -delta[64]
  static constexpr int kDrainChunkBytes = 16 * 32 * 4;  // 16 channels of a drain warp's 32 rows, fp32
  static constexpr int kDrainBufs = 3;
  static constexpr int kDrain = kRows + 8 * 2 * 64 * 4;  // per drain warp: kDrainBufs staging chunks
  static constexpr int kBars = kDrain + 4 * kDrainBufs * kDrainChunkBytes;
  static constexpr int kNumBars = 9 + 2 * kStages;
  static constexpr int kMisc = kBars + 8 * kNumBars;
  static constexpr int kTotal = kMisc + 16;
  static constexpr int kDynamic = kTotal + 1024;
};

template <typename T, int D, class M>
__global__ void __launch_bounds__(kFusedThreads, 1)
bwd_fused_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                    const __grid_constant__ CUtensorMap tmdK, const __grid_constant__ CUtensorMap tmdV, BwdTcParams p) {
  using L = FusedSmem<D>;
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
  const int n_qt_total = (g.Lq + kTile - 1) / kTile;
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
    zero_rows<T, D>(reinterpret_cast<T*>(p.dk) + b * p.dk_sb + hk * p.dk_sh + kb * p.dk_sl, p.dk_sl, rows, kFusedThreads);
    zero_rows<T, D>(reinterpret_cast<T*>(p.dv) + b * p.dv_sb + hk * p.dv_sh + kb * p.dv_sl, p.dv_sl, rows, kFusedThreads);
    zero_part_rows<D>(p.part, b, hk, kb, rows, g.Lk, kFusedThreads);
    return;
  }

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t sK = base + L::kK, sV = base + L::kV, sRing = base + L::kRing;
  float* rows_s = reinterpret_cast<float*>(gen_base + L::kRows);  // [warp][0: -lse, 1: -delta][64]
  const uint32_t bars = base + L::kBars;
  const uint32_t bar_kv_full = bars, bar_acc_full = bars + 8, bar_s_full = bars + 16, bar_dp_full = bars + 24,
                 bar_p_full = bars + 32, bar_ds_full = bars + 40, bar_dv_done = bars + 48, bar_dq_full = bars + 56,
                 bar_dq_drained = bars + 64;
  const uint32_t bar_ring_full = bars + 72, bar_ring_empty = bar_ring_full + 8 * L::kStages;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen_base + L::kMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + L::kMisc + 4);
  const Guard guard{p.status, abort_flag};
  // byte offset (from the aligned base) of the dS^T tile that belongs to iteration `it`
  auto ds_offset = [&](int it) -> int {
    return L::kDsOverlay ? L::kRing + (it % L::kStages) * 2 * L::kTileBytes + L::kTileBytes : L::kDs;
  };

  if (warp == 12) {
    // The producer thread initialises the barriers itself and puts K, V and the first Q/dO tile in flight
    // before the CTA-wide set-up (TMEM allocation, __syncthreads) completes.
    if (lane == 0) {
      *abort_flag = 0;
      mbar_init(bar_kv_full, 1);
      mbar_init(bar_acc_full, 1);
      mbar_init(bar_s_full, 1);
      mbar_init(bar_dp_full, 1);
      mbar_init(bar_p_full, 8);
      mbar_init(bar_ds_full, 8);
      mbar_init(bar_dv_done, 1);
      mbar_init(bar_dq_full, 1);
      mbar_init(bar_dq_drained, 4);
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
  const uint32_t tSt = tmem, tdPt = tmem + 128, tdQ = tmem + 128, tdV = tmem + 256, tdK = tmem + 384;

  if (warp >= 12) {
    reg_dealloc<kFusedOtherRegs>();
    if (warp == 12) {
      // ------------------------------------------------------------------- TMA producer
      if (lane == 0) {
        bool ok = true;
        for (int it = 1; it < n_it; ++it) {  // tile 0 was issued during set-up
          const int s = it % L::kStages;
          const uint32_t ph = (uint32_t)(it / L::kStages) & 1u;
          const int h = hk * G + it / n_qt;
          const int qrow = (qt_lo + it % n_qt) * kTile;
          ok = mbar_wait(bar_ring_empty + 8 * s, ph ^ 1u, guard, kStFusProducer);
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
    } else if (warp == 13) {
      // --------------------------------------------------------------------- MMA issuer
      if (lane == 0) {
        constexpr uint32_t idesc_s = make_idesc<T>(kTile, kTile, false, false);
        constexpr uint32_t idesc_acc = make_idesc<T>(kTile, D, false, true);  // A K-major (or TMEM), B MN-major
        constexpr uint32_t idesc_dq = make_idesc<T>(kTile, D, true, true);    // A and B MN-major
        constexpr uint32_t hi_k = desc_hi_sw128(1024);
        const uint32_t k_lo = desc_lo_sw128(sK, 16), v_lo = desc_lo_sw128(sV, 16);
        const uint32_t kmn_lo = desc_lo_sw128(sK, kChunkBytes);
        bool ok = mbar_wait(bar_kv_full, 0, guard, kStFusMma);
        auto stage_q = [&](int it) { return sRing + (it % L::kStages) * 2 * L::kTileBytes; };
        auto issue_s = [&](int it) -> bool {  // S^T(it) = K Q^T; first user of ring stage `it`
          const int s = it % L::kStages;
          if (!mbar_wait(bar_ring_full + 8 * s, (uint32_t)(it / L::kStages) & 1u, guard, kStFusMma)) return false;
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
        auto issue_dv = [&](int it) -> bool {  // dV += P^T(it) dO(it)   (16 queries per step)
          if (!mbar_wait(bar_p_full, (uint32_t)it & 1u, guard, kStFusMma)) return false;
          tc_fence_after();
          const uint32_t domn_lo = desc_lo_sw128(stage_q(it) + L::kTileBytes, kChunkBytes);
#pragma unroll
          for (int kk = 0; kk < kTile / 16; ++kk)
            mma_ts_lh(tdV, tSt + (kk / 4) * 64 + (kk % 4) * 8, domn_lo + kk * 128, hi_k, idesc_acc, (it > 0 || kk > 0));
          mma_commit(bar_dv_done);
          return true;
        };
        if (ok) ok = issue_s(0);
        if (ok) issue_dp(0);
        if (ok) ok = issue_dv(0);
        if (ok && n_it > 1) ok = issue_s(1);  // overwrites P^T(0) only after dV(0) has read it (MMAs complete in order)
        for (int it = 0; it < n_it && ok; ++it) {
          const uint32_t par = (uint32_t)it & 1u;
          const uint32_t qmn_lo = desc_lo_sw128(stage_q(it), kChunkBytes);
          const uint32_t ds_addr = base + ds_offset(it);
          const uint32_t dsmn_lo = desc_lo_sw128(ds_addr, kChunkBytes), dsk_lo = desc_lo_sw128(ds_addr, 16);
          ok = mbar_wait(bar_ds_full, par, guard, kStFusMma);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < kTile / 16; ++kk)  // dQ tile = dS K   (16 keys per step; overwrites dP^T(it))
            mma_ss_lh(tdQ, dsmn_lo + kk * 128, kmn_lo + kk * 128, hi_k, idesc_dq, kk > 0);
          mma_commit(bar_dq_full);
#pragma unroll
          for (int kk = 0; kk < kTile / 16; ++kk)  // dK += dS^T Q   (16 queries per step)
            mma_ss_lh(tdK, dsk_lo + kmajor_step(kk), qmn_lo + kk * 128, hi_k, idesc_acc, (it > 0 || kk > 0));
          mma_commit(bar_ring_empty + 8 * (it % L::kStages));
          if (it + 1 < n_it) {
            ok = mbar_wait(bar_dq_drained, par, guard, kStFusMma);  // the drain warps hold dQ(it) in registers
            if (!ok) break;
            tc_fence_after();
            issue_dp(it + 1);
            ok = issue_dv(it + 1);
            if (ok && it + 2 < n_it) ok = issue_s(it + 2);
          }
        }
        if (ok) mma_commit(bar_acc_full);
      }
    }
  } else if (warp >= 8) {
    // --------------------------------------------------------------------- dQ drain warps
    reg_alloc<kFusedDrainRegs>();
    const int rg = warp & 3;  // query rows [32 rg, 32 rg + 32) of the tile == this warp's TMEM lanes
    const uint32_t lane_sel = (uint32_t)(rg * 32) << 16;
    // Per warp a ring of kDrainBufs staging buffers, each one chunk of 16 channels: [4 channel groups][32 rows][4],
    // which is also the order of the warp's part of the accumulator block, so a chunk is one contiguous bulk reduce.
    uint8_t* stage_gen = gen_base + L::kDrain + rg * (L::kDrainBufs * L::kDrainChunkBytes);
    const uint32_t stage_sh = base + L::kDrain + rg * (L::kDrainBufs * L::kDrainChunkBytes);
    int chunk_no = 0;
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const int h = hk * G + it / n_qt;
      const int qi = qt_lo + it % n_qt;
      float* dst = p.dq_accum + (((size_t)b * g.H + h) * n_qt_total + qi) * (size_t)(kTile * D) + rg * (32 * D);
      ok = mbar_wait(bar_dq_full, (uint32_t)it & 1u, guard, kStFusDrain);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      // The whole row goes to registers first and frees the TMEM columns at once: an SM hands reductions to the
      // L2 at about 32 bytes per clock, so the 64 KB of a tile take ~2000 clocks to leave, far longer than
      // dP^T(it+1) can wait.  From the registers the tile leaves through shared memory and bulk reductions of
      // the copy engine; reductions issued by the threads themselves (red.global) queue up in the load/store
      // pipeline and hold back the shared-memory traffic of the compute warps (measured: 20 % longer steps).
      uint32_t acc[D];
#pragma unroll
      for (int q4 = 0; q4 < D / 32; ++q4) tmem_ld32(tdQ + lane_sel + q4 * 32, acc + q4 * 32);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_dq_drained);  // the tile has left TMEM: dP^T(it+1) may overwrite it
#pragma unroll
      for (int ch = 0; ch < D / 16; ++ch, ++chunk_no) {
        const int buf = chunk_no % L::kDrainBufs;
        if (lane == 0) bulk_wait_read<L::kDrainBufs - 1>();  // the reduction that last used this buffer has read it
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 4; ++j)
          *reinterpret_cast<uint4*>(stage_gen + buf * L::kDrainChunkBytes + (j * 32 + lane) * 16) =
              make_uint4(acc[16 * ch + 4 * j], acc[16 * ch + 4 * j + 1], acc[16 * ch + 4 * j + 2], acc[16 * ch + 4 * j + 3]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          bulk_reduce_add_f32(dst + ch * (L::kDrainChunkBytes / 4), stage_sh + buf * L::kDrainChunkBytes, L::kDrainChunkBytes);
          tma_store_commit();
        }
      }
    }
    if (lane == 0) bulk_wait_read<0>();  // the staging buffers have been read; the sums land in global memory by kernel end
  } else {
    // ------------------------------------------------------------------- compute warps
    reg_alloc<kFusedComputeRegs>();
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
      ok = mbar_wait(bar_s_full, par, guard, kStFusCompute);
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
      ok = mbar_wait(bar_dp_full, par, guard, kStFusCompute);
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
      tc_fence_before();  // orders this warp's dP^T reads before the dQ GEMM that re-uses the columns
      if (L::kDsOverlay) {
        // dS^T goes where dO(it) sits: wait until the dV GEMM has read it
        ok = mbar_wait(bar_dv_done, par, guard, kStFusCompute);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      {
        // row r of the [key][query] tile: this warp's 64 query columns are one 128-byte line of chunk `wg`
        uint8_t* line = gen_base + ds_offset(it) + wg * kChunkBytes + r * 128;
#pragma unroll
        for (int u = 0; u < 8; ++u)
          *reinterpret_cast<uint4*>(line + ((u ^ (r & 7)) * 16)) =
              make_uint4(preg[4 * u], preg[4 * u + 1], preg[4 * u + 2], preg[4 * u + 3]);
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_ds_full);
    }

    // ---- epilogue: warps 0-3 store dV, warps 4-7 store dK * sm_scale (staging = ring stage 0)
    if (ok) ok = mbar_wait(bar_acc_full, 0, guard, kStFusEpilogue);
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
  if (warp == 12) tmem_dealloc(tmem, kTmemColsBwd);
}

// dQ = sm_scale * accumulator, rounded to the output type.  One block per (query tile, head, batch); a thread
// takes two consecutive rows of one group of four channels, i.e. one 32-byte sector of the accumulator.
template <typename T, int D>
__global__ void __launch_bounds__(256)
dq_convert_kernel(const float* __restrict__ accum, T* __restrict__ dq, long long sb, long long sh, long long sl, int H,
                  int Lq, float scale) {
  const int qi = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int n_qt_total = gridDim.x;
  const float* src = accum + (((size_t)b * H + h) * n_qt_total + qi) * (size_t)(kTile * D);
  T* dst = dq + b * sb + h * sh + (long long)qi * kTile * sl;
  const int rows = imin(kTile, Lq - qi * kTile);
  for (int idx = threadIdx.x; idx < (kTile / 2) * (D / 4); idx += 256) {
    const int c4 = idx % (D / 4), r0 = (idx / (D / 4)) * 2;
    const float4* s4 = reinterpret_cast<const float4*>(src + (size_t)(r0 / 32) * (32 * D) + c4 * 128 + (r0 % 32) * 4);
    const float4 a = s4[0], bb = s4[1];
    if (r0 < rows)
      *reinterpret_cast<uint2*>(dst + r0 * sl + c4 * 4) =
          make_uint2(pack2<T>(a.x * scale, a.y * scale), pack2<T>(a.z * scale, a.w * scale));
    if (r0 + 1 < rows)
      *reinterpret_cast<uint2*>(dst + (r0 + 1) * sl + c4 * 4) =
          make_uint2(pack2<T>(bb.x * scale, bb.y * scale), pack2<T>(bb.z * scale, bb.w * scale));
  }
}

// ---------------------------------------------------------------------------- launcher
template <typename T, int D, class M>
int launch_bwd_fused_one(const CUtensorMap* maps, const BwdTcParams& p, cudaStream_t st) {
  auto kern = bwd_fused_tc_kernel<T, D, M>;
  constexpr int smem = FusedSmem<D>::kDynamic;
  static_assert(smem <= 232448, "exceeds the 227 KB of shared memory a CTA can opt in to");
  struct Tag {};
  cudaError_t e = ensure_dynamic_smem<Tag>(kern, smem);
  if (e != cudaSuccess) return (int)e;
  const Geo& g = p.g;
  e = cudaMemsetAsync(p.dq_accum, 0, dq_accum_bytes(g.B, g.H, g.Lq, D), st);
  if (e != cudaSuccess) return (int)e;
  // maps: 0 Q, 1 K, 2 V, 3 dO, 4 dQ, 5 dK, 6 dV
  dim3 gk((unsigned)(((g.Lk + kTile - 1) / kTile) * g.Hkv * g.B), 1, 1);
  kern<<<gk, kFusedThreads, smem, st>>>(maps[0], maps[1], maps[2], maps[3], maps[5], maps[6], p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  dim3 gc((unsigned)((g.Lq + kTile - 1) / kTile), (unsigned)g.H, (unsigned)g.B);
  dq_convert_kernel<T, D><<<gc, 256, 0, st>>>(p.dq_accum, reinterpret_cast<T*>(p.dq), p.dq_sb, p.dq_sh, p.dq_sl, g.H,
                                               g.Lq, g.scale);
  return (int)cudaGetLastError();
}

template <class M>
int launch_bwd_fused_all(int dtype, int D, const CUtensorMap* maps, const BwdTcParams& p, cudaStream_t st) {
  if (dtype == 2) {
    if (D == 128) return launch_bwd_fused_one<__nv_bfloat16, 128, M>(maps, p, st);
    if (D == 64) return launch_bwd_fused_one<__nv_bfloat16, 64, M>(maps, p, st);
  } else if (dtype == 1) {
    if (D == 128) return launch_bwd_fused_one<__half, 128, M>(maps, p, st);
    if (D == 64) return launch_bwd_fused_one<__half, 64, M>(maps, p, st);
  }
  return (int)cudaErrorInvalidValue;
}

}  // namespace tc
}  // namespace chill
