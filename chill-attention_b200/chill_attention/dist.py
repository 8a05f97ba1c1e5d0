"""Multi-GPU use of the attention kernels (one process per GPU, torch.distributed).

Two ways the path shards (the reference has neither, it is single-device):

* ``shard_units``: (batch x kv-head-group) units are independent in forward and backward
  (a GQA group stays together because dK/dV sum over it), so N ranks each take a contiguous
  slice - no communication at all.

* sequence sharding for masks with a bounded window (SlidingWindowChillMask,
  ChunkwiseChillMask): rank r owns positions [r*L/N, (r+1)*L/N) of q, k, v.  Forward needs the
  ``halo_left`` key/value rows before the shard from rank r-1 (and ``halo_right`` rows after it
  from rank r+1); backward returns the dK/dV rows computed for those halo keys to their owner,
  which adds them.  The exchange is NCCL send/recv (torch.distributed.batch_isend_irecv); halos
  land in this GPU's own memory and the kernels read them with ordinary per-CTA TMA loads.
  The kernels see global positions through q_offset / k_offset / seq_len of the C ABI.

``local_forward`` / ``local_backward`` are injectable so the partition and halo logic can be
exercised on CPU ranks (gloo) with any dense implementation.
"""
from __future__ import annotations

import json
import os
import time

import torch
import torch.distributed as dist

from . import _cabi
from .mask import ChillMask


def shard_units(n_units: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous [lo, hi) slice of ``n_units`` independent units for ``rank`` (sizes differ by at most 1)."""
    base, rem = divmod(n_units, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def shard_batch_heads(t: torch.Tensor, h_kv: int, world: int, rank: int) -> torch.Tensor:
    """Slice [B, H, L, D] by (batch, kv-head group) units; returns a [units, H/h_kv, L, D] view-compatible tensor."""
    B, H, L, D = t.shape
    g = H // h_kv
    lo, hi = shard_units(B * h_kv, world, rank)
    return t.reshape(B * h_kv, g, L, D)[lo:hi]


def halo_sizes(mask: ChillMask, shard_len: int) -> tuple[int, int]:
    """(left, right) number of neighbour key rows a shard needs.  Only masks whose window is bounded
    and fits one neighbour are supported."""
    name, args = mask.name, mask.constargs
    if name == "SlidingWindowChillMask":
        left, right = int(args[0]), int(args[1])
    elif name == "ChunkwiseChillMask":
        cs, bc = int(args[0]), int(args[1])
        # a query's oldest visible key is the start of the chunk `bc` chunks back: at most
        # (bc + 1) * cs - 1 positions before it; nothing after its own chunk end (< cs ahead)
        left, right = (bc + 1) * cs - 1, cs - 1
    else:
        raise NotImplementedError(f"sequence sharding needs a bounded window; {name} has none")
    if left > shard_len or right > shard_len:
        raise ValueError(f"window ({left}, {right}) exceeds the shard length {shard_len}: more than one neighbour involved")
    return left, right


def _peer(group):
    return (lambda r: dist.get_global_rank(group, r)) if group is not None else (lambda r: r)


def start_halo_exchange(k_local, v_local, left: int, right: int, group=None):
    """Post the K/V halo sends and receives (asynchronous).  Returns (works, recv_left, recv_right, hl, hr):
    ``recv_left`` = [2, B, H, hl, D] buffer for the last ``left`` rows of rank-1 (K then V), ``recv_right`` the
    first ``right`` rows of rank+1; hl / hr are 0 at the ends of the sequence.  Wait on ``works`` before
    reading the buffers."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    hl = left if rank > 0 else 0
    hr = right if rank < world - 1 else 0
    B, H, Ls, D = k_local.shape
    ops, recv_l, recv_r = [], None, None
    peer = _peer(group)
    if rank < world - 1 and left > 0:  # my tail is the right neighbour's left halo
        tail = torch.stack([k_local[:, :, Ls - left:], v_local[:, :, Ls - left:]]).contiguous()
        ops.append(dist.P2POp(dist.isend, tail, peer(rank + 1), group))
    if rank > 0 and right > 0:
        head = torch.stack([k_local[:, :, :right], v_local[:, :, :right]]).contiguous()
        ops.append(dist.P2POp(dist.isend, head, peer(rank - 1), group))
    if hl > 0:
        recv_l = torch.empty((2, B, H, hl, D), dtype=k_local.dtype, device=k_local.device)
        ops.append(dist.P2POp(dist.irecv, recv_l, peer(rank - 1), group))
    if hr > 0:
        recv_r = torch.empty((2, B, H, hr, D), dtype=k_local.dtype, device=k_local.device)
        ops.append(dist.P2POp(dist.irecv, recv_r, peer(rank + 1), group))
    works = dist.batch_isend_irecv(ops) if ops else []
    return works, recv_l, recv_r, hl, hr


def exchange_halo_grads(dk_halo_left, dk_halo_right, left: int, right: int, like, group=None):
    """Send the dK/dV rows computed for halo keys back to their owners; receive what the neighbours
    computed for this rank's boundary rows.  ``dk_halo_left`` / ``dk_halo_right``: [2, B, H, hl|hr, D] or None.
    Returns (from_right, from_left): [2, B, H, left, D] to add to the last ``left`` local rows, and
    [2, B, H, right, D] to add to the first ``right`` rows (None where there is no neighbour)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    B, H, _, D = like.shape
    ops, from_right, from_left = [], None, None
    peer = _peer(group)
    if dk_halo_left is not None:
        ops.append(dist.P2POp(dist.isend, dk_halo_left.contiguous(), peer(rank - 1), group))
    if dk_halo_right is not None:
        ops.append(dist.P2POp(dist.isend, dk_halo_right.contiguous(), peer(rank + 1), group))
    if rank < world - 1 and left > 0:  # the right neighbour used my last `left` rows as its left halo
        from_right = torch.empty((2, B, H, left, D), dtype=like.dtype, device=like.device)
        ops.append(dist.P2POp(dist.irecv, from_right, peer(rank + 1), group))
    if rank > 0 and right > 0:
        from_left = torch.empty((2, B, H, right, D), dtype=like.dtype, device=like.device)
        ops.append(dist.P2POp(dist.irecv, from_left, peer(rank - 1), group))
    for w in (dist.batch_isend_irecv(ops) if ops else []):
        w.wait()
    return from_right, from_left


# ------------------------------------------------------------------ local kernels (C ABI)
def cabi_local_forward(mask, q, k_ext, v_ext, q_offset, k_offset, seq_len, sm_scale, o=None, lse=None):
    """O, LSE of local query rows against local key rows with global offsets.  ``o`` / ``lse`` may be views
    of larger buffers (row slices); they are written in place."""
    lib, functor = _library_for(mask)
    if o is None:
        o = torch.empty_like(q, memory_format=torch.contiguous_format)
    if lse is None:
        lse = torch.empty(q.shape[:3], dtype=torch.float32, device=q.device)
    shape = _cabi.make_shape(q, k_ext, functor, mask.constargs, None, sm_scale, q_offset, k_offset, seq_len)
    _cabi.forward(lib, q, k_ext, v_ext, o, lse, shape)
    return o, lse


def cabi_local_backward(mask, q, k_ext, v_ext, o, lse, do, q_offset, k_offset, seq_len, sm_scale, dq=None):
    lib, functor = _library_for(mask)
    if dq is None:
        dq = torch.empty_like(q, memory_format=torch.contiguous_format)
    dk = torch.empty_like(k_ext, memory_format=torch.contiguous_format)
    dv = torch.empty_like(v_ext, memory_format=torch.contiguous_format)
    delta = torch.empty(q.shape[:3], dtype=torch.float32, device=q.device)
    shape = _cabi.make_shape(q, k_ext, functor, mask.constargs, None, sm_scale, q_offset, k_offset, seq_len)
    _cabi.backward(lib, q, k_ext, v_ext, o, do, lse, delta, dq, dk, dv, shape)
    return dq, dk, dv


def _library_for(mask):
    functor = _cabi.BUILTIN_FUNCTOR_IDS.get(getattr(mask, "cuda_functor", None))
    if functor is None:
        raise NotImplementedError("sequence sharding supports the built-in masks")
    return _cabi.load_library(), functor


# -------------------------------------------------------------------- sharded operator
def _regions(Ls, hl, hr, left, right):
    """Row ranges of a shard: boundary rows that need the left halo, interior rows that only see local keys,
    boundary rows that need the right halo; and the local key rows each boundary part can see."""
    bl = left if hl > 0 else 0
    br = right if hr > 0 else 0
    if bl + br > Ls:  # tiny shard: treat every row as boundary-left (keys = halo_left + local + halo_right)
        return None
    return {"bl": bl, "br": br, "kl_hi": min(Ls, bl + right), "kr_lo": max(0, Ls - br - left)}


def _call_fwd(fn, o, lse, mask, q, k, v, q_off, k_off, seq_len, sm_scale):
    """Run a local forward into the views ``o`` / ``lse`` (callbacks without out-parameters are copied)."""
    try:
        ro, rl = fn(mask, q, k, v, q_off, k_off, seq_len, sm_scale, o=o, lse=lse)
    except TypeError:
        ro, rl = fn(mask, q, k, v, q_off, k_off, seq_len, sm_scale)
    if ro.data_ptr() != o.data_ptr():
        o.copy_(ro)
        lse.copy_(rl)


class _SequenceShardedAttention(torch.autograd.Function):
    """Forward: post the halo exchange, run the interior rows (which see local keys only) while it is in
    flight, then the boundary rows against [halo | the few local rows they can see].  Backward mirrors it and
    returns the halo keys' dK/dV to their owners.  No full-size copy of K/V is ever made."""

    @staticmethod
    def forward(ctx, q, k, v, mask, seq_len, sm_scale, group, local_forward, local_backward):
        rank = dist.get_rank(group)
        B, H, Ls, D = q.shape
        left, right = halo_sizes(mask, Ls)
        works, recv_l, recv_r, hl, hr = start_halo_exchange(k, v, left, right, group)
        reg = _regions(Ls, hl, hr, left, right)
        base = rank * Ls
        o = torch.empty((B, H, Ls, D), dtype=q.dtype, device=q.device)
        lse = torch.empty((B, H, Ls), dtype=torch.float32, device=q.device)
        parts = []  # (row slice, k tensor, v tensor, k_offset, halo rows in front, halo rows behind)
        if reg is not None:
            bl, br = reg["bl"], reg["br"]
            if Ls - br > bl:  # interior first: independent of the exchange
                sl = slice(bl, Ls - br)
                _call_fwd(local_forward, o[:, :, sl], lse[:, :, sl], mask, q[:, :, sl], k, v, base + bl, base, seq_len, sm_scale)
                parts.append((sl, None, None, base, 0, 0))
        for w in works:
            w.wait()
        if reg is None:
            pieces_k = ([recv_l[0]] if hl else []) + [k] + ([recv_r[0]] if hr else [])
            pieces_v = ([recv_l[1]] if hl else []) + [v] + ([recv_r[1]] if hr else [])
            k_ext, v_ext = torch.cat(pieces_k, dim=2), torch.cat(pieces_v, dim=2)
            _call_fwd(local_forward, o, lse, mask, q, k_ext, v_ext, base, base - hl, seq_len, sm_scale)
            parts.append((slice(0, Ls), k_ext, v_ext, base - hl, hl, hr))
        else:
            if reg["bl"] > 0:
                k_b = torch.cat([recv_l[0], k[:, :, :reg["kl_hi"]]], dim=2)
                v_b = torch.cat([recv_l[1], v[:, :, :reg["kl_hi"]]], dim=2)
                sl = slice(0, reg["bl"])
                _call_fwd(local_forward, o[:, :, sl], lse[:, :, sl], mask, q[:, :, sl], k_b, v_b, base, base - hl, seq_len, sm_scale)
                parts.append((sl, k_b, v_b, base - hl, hl, 0))
            if reg["br"] > 0:
                k_b = torch.cat([k[:, :, reg["kr_lo"]:], recv_r[0]], dim=2)
                v_b = torch.cat([v[:, :, reg["kr_lo"]:], recv_r[1]], dim=2)
                sl = slice(Ls - reg["br"], Ls)
                _call_fwd(local_forward, o[:, :, sl], lse[:, :, sl], mask, q[:, :, sl], k_b, v_b, base + Ls - reg["br"],
                          base + reg["kr_lo"], seq_len, sm_scale)
                parts.append((sl, k_b, v_b, base + reg["kr_lo"], 0, hr))
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.parts = parts
        ctx.cfg = (mask, seq_len, sm_scale, group, local_backward, hl, hr, left, right, base, reg)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        mask, seq_len, sm_scale, group, local_backward, hl, hr, left, right, base, reg = ctx.cfg
        B, H, Ls, D = q.shape
        do = do.contiguous()
        dq = torch.empty_like(q, memory_format=torch.contiguous_format)
        dk = dv = None
        small = []  # (dk_part, dv_part, first local key row, halo rows in front, halo rows behind)
        for sl, k_b, v_b, k_off, h_front, h_back in ctx.parts:
            qs, os_, ls, dos = q[:, :, sl], o[:, :, sl], lse[:, :, sl], do[:, :, sl]
            kk, vv = (k, v) if k_b is None else (k_b, v_b)
            q_off = base + sl.start
            try:
                rdq, rdk, rdv = local_backward(mask, qs, kk, vv, os_, ls, dos, q_off, k_off, seq_len, sm_scale, dq=dq[:, :, sl])
            except TypeError:
                rdq, rdk, rdv = local_backward(mask, qs, kk, vv, os_, ls, dos, q_off, k_off, seq_len, sm_scale)
            if rdq.data_ptr() != dq[:, :, sl].data_ptr():
                dq[:, :, sl].copy_(rdq)
            if k_b is None:  # interior: its dK/dV cover every local key row and become the result buffers
                dk, dv = rdk, rdv
            else:
                small.append((rdk, rdv, k_off + h_front - base, h_front, h_back))
        if dk is None:
            dk, dv = torch.zeros_like(k, memory_format=torch.contiguous_format), torch.zeros_like(v, memory_format=torch.contiguous_format)
        send_l = send_r = None
        for rdk, rdv, row0, h_front, h_back in small:
            n_local = rdk.shape[2] - h_front - h_back
            dk[:, :, row0:row0 + n_local] += rdk[:, :, h_front:h_front + n_local]
            dv[:, :, row0:row0 + n_local] += rdv[:, :, h_front:h_front + n_local]
            if h_front:
                send_l = torch.stack([rdk[:, :, :h_front], rdv[:, :, :h_front]])
            if h_back:
                send_r = torch.stack([rdk[:, :, h_front + n_local:], rdv[:, :, h_front + n_local:]])
        from_right, from_left = exchange_halo_grads(send_l, send_r, left, right, dk, group)
        if from_right is not None:
            dk[:, :, Ls - left:] += from_right[0]
            dv[:, :, Ls - left:] += from_right[1]
        if from_left is not None:
            dk[:, :, :right] += from_left[0]
            dv[:, :, :right] += from_left[1]
        return dq, dk, dv, None, None, None, None, None, None


def sequence_sharded_attention(q, k, v, mask: ChillMask, seq_len: int, sm_scale=None, group=None,
                               local_forward=cabi_local_forward, local_backward=cabi_local_backward):
    """Attention over a sequence split evenly across the ranks of ``group``.

    q, k, v: this rank's [B, H(_kv), L/N, D] shard (rank r holds positions [r*L/N, (r+1)*L/N));
    ``seq_len`` is the global length L.  Differentiable; returns this rank's shard of O."""
    if sm_scale is None:
        sm_scale = q.shape[-1] ** -0.5
    return _SequenceShardedAttention.apply(q, k, v, mask, seq_len, sm_scale, group, local_forward, local_backward)


# --------------------------------------------------------------------------- benchmark
def bench_sequence_sharded(args, workload, metric):
    """bench.py leg for the long sliding-window workload on N > 1 GPUs (already initialised NCCL)."""
    from . import SlidingWindowChillMask

    world, rank = dist.get_world_size(), dist.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    mname, margs, dt, B, H, L, D = workload
    assert mname == "SlidingWindowChillMask" and L % world == 0
    mask = SlidingWindowChillMask(*margs)
    dtype = getattr(torch, dt)
    Ls = L // world
    g = torch.Generator(device=dev).manual_seed(20 + rank)
    q, k, v, do = (torch.randn(B, H, Ls, D, generator=g, device=dev, dtype=torch.float32).to(dtype) for _ in range(4))
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)

    def step():
        q.grad = k.grad = v.grad = None
        o = sequence_sharded_attention(q, k, v, mask, L)
        o.backward(do)

    for _ in range(args.warmup):
        step()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    dist.barrier()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / args.steps], dtype=torch.float64, device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    pos = torch.arange(L, dtype=torch.int64)
    lo, hi = type(mask).k_range_for_q(pos, L, mask.constargs)
    pairs = int((hi - lo + 1).sum())
    if rank == 0:
        value = 14.0 * B * H * D * pairs / (ms.item() * 1e-3) / 1e12
        halo = 2 * B * H * int(margs[0]) * D * q.element_size()
        print(json.dumps({
            "metric": metric, "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms.item(), 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic: seeded N(0,1)",
            "config": {"workload": f"c5: {mname}{margs} fwd+bwd {dt} (B={B},H={H},L={L},D={D}) sequence-sharded",
                       "global_batch": B, "seq_len": L,
                       "parallelism": f"sequence sharded over {world} GPUs, {halo} B K/V halo per boundary via NCCL send/recv, "
                                      "dK/dV halo returned the same way"},
            "gpu_launches": 4 * args.steps,
        }), flush=True)
    dist.barrier()
    dist.destroy_process_group()
