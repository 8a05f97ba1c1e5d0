/*
 * chill_b200.h - C ABI of the B200 (sm_100a) masked flash-attention kernels.
 *
 * Every entry point takes plain device pointers, element strides and sizes; none
 * allocates device memory, synchronises, or keeps state between calls, apart from:
 *  - a per-process cache of the driver entry point used to encode TMA descriptors and
 *    a per-device record of which kernels had their shared-memory limit raised;
 *  - for the two-kernel form of chill_bwd, one helper stream + two events per device
 *    (created on the first call) on which the dQ kernel runs beside the dK/dV kernel;
 *    chill_bwd joins that stream back into the caller's stream before it returns, so
 *    stream ordering as seen by the caller is unchanged.  The fork / launch / join
 *    sequence holds a per-device lock, so host threads may call chill_bwd on the same
 *    device from different streams;
 *  - for chill_bwd_noalloc, a 16 MiB array in device global memory per GPU (part of
 *    the library image) and a per-device cache of its address;
 *  - for chill_fwd_bwd_host, three streams and a handful of events per device (created on the
 *    first call) that carry its upload / compute / download pipeline; a per-device lock
 *    serialises the host side of concurrent calls;
 *  - a process-wide count of launched kernels (chill_launch_count).
 * All work is enqueued on the CUDA stream passed in (a cudaStream_t cast to
 * void*; NULL = the default stream) of the CURRENT device.  Return value: 0 on
 * success, a negative CHILL_E_* code otherwise; nothing aborts the process.
 *
 * Tensors are indexed [batch][head][position][channel]; `*_strides[4]` are in
 * ELEMENTS.  The tensor-core path needs channel stride 1 and 16-byte aligned
 * base / batch / head / position strides for a 16-bit dtype with D in {64,128,256}
 * (or fp32 with CHILL_FLAG_ALLOW_TF32 and D in {64,128}); anything else (fp32 in
 * IEEE arithmetic, other D, odd strides) is served by the generic kernels of the
 * same library - there is no host fallback.
 *
 * Reference counterparts (alexdremov/chill-attention, paths inside that project):
 *   chill_fwd            replaces the launch of _chill_attn_fwd
 *                        chill_attention/chill.py:64-211, kernel chill_fwd.py:13-359
 *   chill_bwd_delta      replaces _chill_attn_bwd_precompute
 *                        chill_attention/chill.py:261-290, kernel utils.py:93-217
 *   chill_bwd            replaces the fused launch of _chill_attn_bwd
 *                        chill_attention/chill.py:292-444, kernels chill_bwd.py:14-168,
 *                        chill_bwd_dq.py:233-397, chill_bwd_dkdv.py:281-509
 *   chill_mask_tabulate  replaces ChillMask._mask_infer / _limits_infer /
 *                        _full_ranges_infer, chill_attention/mask.py:284-377, :487-534
 */
#ifndef CHILL_B200_H_
#define CHILL_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CHILL_ABI_VERSION 5

/* status codes */
#define CHILL_OK 0
#define CHILL_E_INVALID (-1)      /* null pointer, bad size, H % H_kv != 0, ... */
#define CHILL_E_UNSUPPORTED (-2)  /* dtype / head dim / mask id this build has no kernel for */
#define CHILL_E_CUDA (-3)         /* a CUDA runtime/driver call failed; see chill_last_cuda_error */
#define CHILL_E_TOO_LARGE (-4)    /* a size exceeds what the entry point supports */

/* element types */
#define CHILL_F32 0
#define CHILL_F16 1
#define CHILL_BF16 2

/* built-in mask functors (csrc/masks.cuh); CHILL_MASK_CUSTOM is only present in a
 * library built with a user functor header */
#define CHILL_MASK_FULL 0     /* FullChillMask            mask.py:806-889   */
#define CHILL_MASK_CAUSAL 1   /* CausalChillMask          mask.py:892-976   */
#define CHILL_MASK_SLIDING 2  /* SlidingWindowChillMask   mask.py:979-1108  args: left, right */
#define CHILL_MASK_CHUNKWISE 3/* ChunkwiseChillMask       mask.py:1111-1266 args: context_size, back_contexts */
#define CHILL_MASK_PREFIXLM 4 /* PrefixLMChillMask        mask.py:1269-1394 args: prefix_size */
#define CHILL_MASK_CUSTOM 5

#define CHILL_MAX_MASK_ARGS 8

/* flags */
#define CHILL_FLAG_FORCE_GENERIC 1u /* never take the tensor-core path */
#define CHILL_FLAG_REQUIRE_TC 2u    /* fail with CHILL_E_UNSUPPORTED instead of using the generic path */
#define CHILL_FLAG_BWD_ONLY_DKDV 4u /* chill_bwd launches only the dK/dV kernel (per-kernel timing) */
#define CHILL_FLAG_BWD_ONLY_DQ 8u   /* chill_bwd launches only the dQ kernel */
#define CHILL_FLAG_ALLOW_TF32 16u   /* fp32 tensors may go through the tensor cores in TF32 (10-bit mantissa):
                                     * chill_fwd then runs its tcgen05 kernel for head dim 64 / 128 and chill_bwd its
                                     * TF32 kernels for head dim 64 / 128; the reference's precision="tf32"
                                     * (chill_fwd.py:13-359, chill_bwd_dq.py:312, chill_bwd_dkdv.py:347:
                                     * input_precision).  Without the flag, and for other head dims, fp32 is
                                     * computed in IEEE fp32 by the generic kernels. */

/* The mask constants a ChillMask instance was built with (ChillMask.constargs,
 * mask.py:31-49).  Each is passed both ways: `i[n]` = the value truncated to an
 * integer, `f[n]` = the value as a double; a functor reads the one it means. */
typedef struct chill_mask_desc {
  int32_t id;  /* CHILL_MASK_* */
  int32_t n_args;
  int64_t i[CHILL_MAX_MASK_ARGS];
  double f[CHILL_MAX_MASK_ARGS];
} chill_mask_desc;

/* Problem geometry shared by forward and backward.
 *
 * Query rows are local positions [0, Lq), key rows [0, Lk); the mask functor and
 * the `lens` bound see GLOBAL positions q + q_offset and k + k_offset, and
 * `seq_len` is the global sequence length (the value the reference passes to
 * its mask functions).  A single-device call has Lq == Lk == seq_len and both
 * offsets 0; a sequence-sharded call passes its shard of the queries, its shard
 * plus halo of the keys, and the offsets of both.  The reference has no
 * offsets (chill_fwd.py:141-142 uses local indices).
 *
 * `lens` (optional, int32[B], device): valid length of each batch row, clamped
 * to seq_len.  Keys at global position >= lens[b] are never attended; query rows
 * at global position >= lens[b] produce O = 0, LSE = 0 and zero gradients. */
typedef struct chill_shape {
  int32_t B, H, H_kv, Lq, Lk, D;
  int32_t dtype; /* CHILL_F32 / CHILL_F16 / CHILL_BF16: q, k, v, o, do, dq, dk, dv */
  int32_t q_offset, k_offset, seq_len;
  float sm_scale;
  uint32_t flags;
  const int32_t* lens;
  chill_mask_desc mask;
} chill_shape;

typedef struct chill_fwd_args {
  chill_shape s;
  const void *q, *k, *v;
  void* o;    /* written for every row of every (b, h) */
  float* lse; /* optional (may be NULL): log2-domain log-sum-exp, m + log2(l) */
  int64_t q_strides[4], k_strides[4], v_strides[4], o_strides[4];
  int64_t lse_strides[3];
} chill_fwd_args;

typedef struct chill_bwd_args {
  chill_shape s;
  const void *q, *k, *v, *o, *d_o;
  const float* lse; /* from chill_fwd, log2 domain */
  float* delta;     /* scratch, B*H*Lq floats, contiguous [B][H][Lq]; filled by chill_bwd_delta */
  void *dq, *dk, *dv; /* written for every row; dk/dv are summed over the GQA group */
  int64_t q_strides[4], k_strides[4], v_strides[4], o_strides[4], do_strides[4];
  int64_t dq_strides[4], dk_strides[4], dv_strides[4];
  int64_t lse_strides[3];
  /* Optional (may be NULL): fp32 scratch of chill_bwd_dq_accum_bytes() bytes, 16-byte aligned, contents
   * irrelevant on entry.  With it, and when the tensor-core kernels serve the call, chill_bwd runs its
   * single-kernel backward: S and dP are computed once per tile pair (five GEMMs instead of seven) and the
   * per-key-tile contributions to dQ are summed in this buffer with fp32 reductions, whose order is not
   * fixed, so dQ may differ in its last bits from run to run (dK and dV do not).  Without it chill_bwd runs
   * the deterministic two-kernel backward, which is also what the reference's accumulation order
   * (chill_bwd_dq.py:300-394: one program owns a query tile) corresponds to.  The call zero-fills the buffer on
   * the given stream before use; two calls that can overlap on the GPU need a buffer each. */
  float* dq_accum;
  /* Optional (may be NULL): gradient of the loss with respect to the LSE that chill_fwd returned (log2 units,
   * same layout rules as lse).  chill_bwd_delta folds it into delta (delta -= log2(e) * d_lse), which is all the
   * backward kernels need to propagate it to dQ and dK.  The reference drops this gradient (chill.py:466-490);
   * with NULL the behaviour is the reference's. */
  const float* d_lse;
  int64_t dlse_strides[3];
  /* Optional (may be NULL, both or neither): un-rounded fp32 copies of dK (already multiplied by sm_scale) and dV
   * for the first `part_head` and the last `part_tail` key rows of the call (part_head + part_tail <= Lk).  Key row
   * j < part_head goes to part row j, key row j >= Lk - part_tail to part row part_head + j - (Lk - part_tail);
   * element (b, h_kv, part row, channel) sits at b * part_strides[0] + h_kv * part_strides[1] + row * part_strides[2]
   * + channel.  The 16-bit dk / dv are written as usual.  For callers that add several partial dK / dV of the same
   * key rows (a sequence-sharded backward sums the contribution of its own queries and of a neighbour's) and
   * want to round once, after the sum.  No counterpart in the reference, which is single-device. */
  float *dk_part, *dv_part;
  int64_t part_strides[3];
  int32_t part_head, part_tail;
} chill_bwd_args;

/* O = softmax(mask(Q K^T * sm_scale)) V and LSE.  See chill_shape for conventions. */
int chill_fwd(const chill_fwd_args* a, void* stream);

/* delta[b,h,t] = sum_d float(O[b,h,t,d]) * float(dO[b,h,t,d]) (- log2(e) * d_lse[b,h,t] if a->d_lse is given).
 * Uses a->o, a->d_o, a->delta, a->d_lse. */
int chill_bwd_delta(const chill_bwd_args* a, void* stream);

/* dQ, dK, dV.  a->delta must hold the result of chill_bwd_delta for the same a->o / a->d_o
 * (enqueue both on the same stream). */
int chill_bwd(const chill_bwd_args* a, void* stream);

/* chill_bwd_delta + chill_bwd for callers that cannot hand over a scratch buffer.
 * (No counterpart in the reference: its adapter allocates `delta` with torch.empty on every call.)
 *
 * Who needs it: code that runs where device allocation is off limits - a host callback or a
 * plugin hook invoked while the framework's allocator is locked, a real-time / serving loop with
 * a frozen memory plan, an embedder that received all its buffers up front and has no allocator
 * handle to pass down.  Such a caller still owns q, k, v, o, d_o, lse and the three outputs, but
 * has nowhere to put the B*H*Lq floats of `delta` that the backward kernels exchange.
 *
 * This entry point keeps that scratch inside the library: a fixed array in device global memory
 * (part of the library image, so every GPU that loads the library holds its
 * CHILL_NOALLOC_MAX_ROWS * 4 bytes = 16 MiB until the process exits).  `a->delta` is ignored and
 * may be NULL.  The call allocates nothing: no cudaMalloc / cudaFree / stream-ordered allocation
 * and no allocating library routine.
 *
 * Limits and rules:
 *  - B * H * Lq must not exceed CHILL_NOALLOC_MAX_ROWS, otherwise CHILL_E_TOO_LARGE is returned
 *    and nothing is launched.
 *  - The first call on each device looks up the array's device address (one-time set-up with
 *    that device current).  Make that first call outside any stream capture.
 *  - All calls on a device share the one array and it keeps the previous call's contents.
 *    Nothing in it needs clearing (every row the kernels read is rewritten first by the same
 *    call), but two calls whose kernels can overlap on the GPU - different streams, no
 *    dependency between them - race on it.  Serialise them (same stream, or an event). */
#define CHILL_NOALLOC_MAX_ROWS (1u << 22)
int chill_bwd_noalloc(const chill_bwd_args* a, void* stream);

/* Forward + backward for a caller whose tensors live in HOST memory (no counterpart in the reference, whose
 * tensors are torch CUDA tensors; this is the call an embedder with host-resident activations makes, and what
 * the end-to-end figure of the benchmark times).
 *
 * q, d_o, o, dq: contiguous [B][H][L][D]; k, v, dk, dv: contiguous [B][H_kv][L][D]; L = s.Lq = s.Lk = s.seq_len,
 * offsets 0, s.lens NULL (CHILL_E_INVALID otherwise).  Host memory should be page-locked: pageable memory works
 * but its copies do not overlap anything.
 *
 * The batch goes through the GPU in chunks of `chunk_groups` whole kv-head groups of one batch row, on three
 * streams (uploads, kernels, downloads) over two sets of device staging buffers carved from `workspace`, so
 * transfers in both directions overlap each other and the kernels.  Per chunk it calls chill_fwd, chill_bwd_delta
 * and chill_bwd (single-kernel backward with the fp32 dQ scratch unless CHILL_FLAG_BWD_DETERMINISTIC is set in
 * s.flags).
 *
 * The work is ordered after everything already enqueued on `stream`, and `stream` is made to wait for all of it;
 * the call itself does not synchronise: synchronise `stream` before reading the outputs or reusing `workspace`. */
#define CHILL_FLAG_BWD_DETERMINISTIC 32u /* chill_fwd_bwd_host: two-kernel backward (no fp32 dQ scratch) */
typedef struct chill_host_args {
  chill_shape s;
  const void *q, *k, *v, *d_o; /* host */
  void *o, *dq, *dk, *dv;      /* host */
  void* workspace;             /* device, 256-byte aligned, chill_host_workspace_bytes() bytes */
  size_t workspace_bytes;
  int32_t chunk_groups;        /* kv-head groups per full-size chunk; 0 = about 40 MB of input per chunk */
  int32_t reserved;
} chill_host_args;
size_t chill_host_workspace_bytes(const chill_host_args* a);
int chill_fwd_bwd_host(const chill_host_args* a, void* stream);
/* The chunk schedule chill_fwd_bwd_host would run for these arguments (host-only, pointers in `a` are not
 * looked at): up to `capacity` triples (batch row, first kv-head group, groups) are written to `out` (may be
 * NULL); returns the number of chunks or a negative status. */
int chill_host_chunk_schedule(const chill_host_args* a, int32_t* out, int32_t capacity);

/* Bytes of the `delta` scratch buffer chill_bwd_delta / chill_bwd need. */
size_t chill_bwd_scratch_bytes(const chill_shape* s);

/* Bytes of the optional `dq_accum` scratch buffer (0 if the shape can never use it: fp32 data or a head
 * dimension other than 64 / 128).  No counterpart in the reference. */
size_t chill_bwd_dq_accum_bytes(const chill_shape* s);

/* 1 if chill_fwd / chill_bwd would run the tcgen05 tensor-core kernels for these
 * arguments, 0 if the generic kernels, negative status if the arguments are invalid. */
int chill_fwd_uses_tensor_cores(const chill_fwd_args* a);
int chill_bwd_uses_tensor_cores(const chill_bwd_args* a);

/* Tabulate a mask functor on the device (all outputs optional, device pointers):
 *   dense   uint8[n*n]   mask(q, k) for q, k in [0, n)            (row = query)
 *   k_lims  int32[n*2]   k_range_for_q(q), inclusive
 *   q_lims  int32[n*2]   q_range_for_k(k), inclusive
 *   k_full  int32[ceil(n/tile)*2]  k_full_range_for_q(tile start, tile), half-open
 *   q_full  int32[ceil(n/tile)*2]  q_full_range_for_k(tile start, tile), half-open
 * with seq_len = n. */
int chill_mask_tabulate(const chill_mask_desc* m, int32_t n, int32_t tile, uint8_t* dense, int32_t* k_lims,
                        int32_t* q_lims, int32_t* k_full, int32_t* q_full, void* stream);

/* is_full_block of a functor on the tile grid of [0, n)^2 with seq_len = n (device pointer, optional stream):
 *   full  uint8[ceil(n/q_tile) * ceil(n/k_tile)]   is_full_block(qi*q_tile, ki*k_tile, q_tile, k_tile, n), row = query tile
 * Together with chill_mask_tabulate this is what ChillMask.verify(n, device=True) checks a CUDA functor with; the
 * reference verifies the very functions its kernels inline the same way (mask.py:700-803, :487-534). */
int chill_mask_tabulate_blocks(const chill_mask_desc* m, int32_t n, int32_t q_tile, int32_t k_tile, uint8_t* full,
                               void* stream);

/* Host-side properties of a functor: bit0 has_k_full_range, bit1 has_q_full_range,
 * bit2 k_lims_continious, bit3 q_lims_continious, bit4 is_guaranteed_safe. */
int chill_mask_traits(int32_t mask_id);

/* Device-side error word.  Kernels with bounded waits record a non-zero code here instead
 * of hanging; reading it synchronises the device. Returns the code (0 = none) and clears it. */
int chill_read_device_status(void);

/* Number of kernels this library has launched in the calling process so far (all devices, all streams;
 * memsets and copies are not counted).  A benchmark reads it before and after a timed region. */
unsigned long long chill_launch_count(void);

/* Self-test of the give-up path of the kernels' bounded waits.  Launches one small kernel in which every role waits,
 * with a limit of `limit_us` microseconds (clamped to [10, 100000]), on an mbarrier that nothing ever arrives at; the
 * waits run out, the kernel records CHILL_SELFTEST_STATUS in the device status word, releases its TMEM and returns.
 * Nothing faults or hangs and the context stays usable; afterwards chill_read_device_status() returns
 * CHILL_SELFTEST_STATUS once.  Returns 0 if the kernel was launched.  No counterpart in the reference. */
#define CHILL_SELFTEST_STATUS 901
int chill_selftest_bounded_wait(int32_t limit_us, void* stream);

int chill_abi_version(void);
const char* chill_status_string(int status);
const char* chill_last_cuda_error(void);

#ifdef __cplusplus
}
#endif
#endif /* CHILL_B200_H_ */
