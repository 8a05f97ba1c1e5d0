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


def exchange_halos(k_local, v_local, left: int, right: int, group=None):
    """Receive the last ``left`` rows of rank-1 and the first ``right`` rows of rank+1.

    Returns (k_ext, v_ext, hl, hr): local rows with the received halos attached along the
    position axis; hl/hr are the halo lengths actually present (0 at the sequence ends)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    hl = left if rank > 0 else 0
    hr = right if rank < world - 1 else 0
    B, H, Ls, D = k_local.shape
    ops, recv_l, recv_r = [], None, None
    peer = (lambda r: dist.get_global_rank(group, r)) if group is not None else (lambda r: r)
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
    if ops:
        for w in dist.batch_isend_irecv(ops):
            w.wait()
    k_ext = torch.empty((B, H, hl + Ls + hr, D), dtype=k_local.dtype, device=k_local.device)
    v_ext = torch.empty_like(k_ext)
    k_ext[:, :, hl:hl + Ls] = k_local
    v_ext[:, :, hl:hl + Ls] = v_local
    if hl > 0:
        k_ext[:, :, :hl], v_ext[:, :, :hl] = recv_l[0], recv_l[1]
    if hr > 0:
        k_ext[:, :, hl + Ls:], v_ext[:, :, hl + Ls:] = recv_r[0], recv_r[1]
    return k_ext, v_ext, hl, hr


def return_halo_grads(dk_ext, dv_ext, hl: int, hr: int, left: int, right: int, group=None):
    """Send the gradient rows of the halo keys back to their owners and add what the neighbours
    computed for this rank's own boundary rows.  Returns (dk_local, dv_local)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    Ls = dk_ext.shape[2] - hl - hr
    dk = dk_ext[:, :, hl:hl + Ls].contiguous()
    dv = dv_ext[:, :, hl:hl + Ls].contiguous()
    ops, recv_from_right, recv_from_left = [], None, None
    peer = (lambda r: dist.get_global_rank(group, r)) if group is not None else (lambda r: r)
    B, H, _, D = dk.shape
    if hl > 0:  # gradients of the left neighbour's tail
        ops.append(dist.P2POp(dist.isend, torch.stack([dk_ext[:, :, :hl], dv_ext[:, :, :hl]]).contiguous(), peer(rank - 1), group))
    if hr > 0:
        ops.append(dist.P2POp(dist.isend, torch.stack([dk_ext[:, :, hl + Ls:], dv_ext[:, :, hl + Ls:]]).contiguous(), peer(rank + 1), group))
    if rank < world - 1 and left > 0:  # the right neighbour used my last `left` rows as its left halo
        recv_from_right = torch.empty((2, B, H, left, D), dtype=dk.dtype, device=dk.device)
        ops.append(dist.P2POp(dist.irecv, recv_from_right, peer(rank + 1), group))
    if rank > 0 and right > 0:
        recv_from_left = torch.empty((2, B, H, right, D), dtype=dk.dtype, device=dk.device)
        ops.append(dist.P2POp(dist.irecv, recv_from_left, peer(rank - 1), group))
    if ops:
        for w in dist.batch_isend_irecv(ops):
            w.wait()
    if recv_from_right is not None:
        dk[:, :, Ls - left:] += recv_from_right[0]
        dv[:, :, Ls - left:] += recv_from_right[1]
    if recv_from_left is not None:
        dk[:, :, :right] += recv_from_left[0]
        dv[:, :, :right] += recv_from_left[1]
    return dk, dv


# ------------------------------------------------------------------ local kernels (C ABI)
def cabi_local_forward(mask, q, k_ext, v_ext, q_offset, k_offset, seq_len, sm_scale):
    lib, functor = _library_for(mask)
    o = torch.empty_like(q, memory_format=torch.contiguous_format)
    lse = torch.empty(q.shape[:3], dtype=torch.float32, device=q.device)
    shape = _cabi.make_shape(q, k_ext, functor, mask.constargs, None, sm_scale, q_offset, k_offset, seq_len)
    _cabi.forward(lib, q, k_ext, v_ext, o, lse, shape)
    return o, lse


def cabi_local_backward(mask, q, k_ext, v_ext, o, lse, do, q_offset, k_offset, seq_len, sm_scale):
    lib, functor = _library_for(mask)
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
class _SequenceShardedAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, mask, seq_len, sm_scale, group, local_forward, local_backward):
        rank = dist.get_rank(group)
        Ls = q.shape[2]
        left, right = halo_sizes(mask, Ls)
        k_ext, v_ext, hl, hr = exchange_halos(k, v, left, right, group)
        q_off, k_off = rank * Ls, rank * Ls - hl
        o, lse = local_forward(mask, q, k_ext, v_ext, q_off, k_off, seq_len, sm_scale)
        ctx.save_for_backward(q, k_ext, v_ext, o, lse)
        ctx.cfg = (mask, seq_len, sm_scale, group, local_backward, hl, hr, left, right, q_off, k_off)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k_ext, v_ext, o, lse = ctx.saved_tensors
        mask, seq_len, sm_scale, group, local_backward, hl, hr, left, right, q_off, k_off = ctx.cfg
        dq, dk_ext, dv_ext = local_backward(mask, q, k_ext, v_ext, o, lse, do.contiguous(), q_off, k_off, seq_len, sm_scale)
        dk, dv = return_halo_grads(dk_ext, dv_ext, hl, hr, left, right, group)
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
