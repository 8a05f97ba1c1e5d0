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


class HaloBuffer:
    """A rank's shard of K or V with spare rows in front of and behind it for the neighbours' halo rows.

    Memory order is [batch][position][head][channel], so the halo rows of all heads of one batch row are one
    contiguous block: the NCCL receive writes them straight into place and the send reads the shard's own
    first / last rows in place - no staging copy on either side.  ``local`` is the [B, H, Ls, D] view the
    attention call takes as k or v (fill it, or have the projection write into it); ``rows(lo, hi)`` is the
    same kind of view over positions lo..hi relative to the shard's first row (negative = left halo).
    The kernels read such views through their strides (TMA descriptors), no copy is made.
    """

    def __init__(self, B, H, Ls, D, left, right, dtype, device):
        self.B, self.H, self.Ls, self.D, self.left, self.right = B, H, Ls, D, int(left), int(right)
        self.storage = torch.empty((B, self.left + Ls + self.right, H, D), dtype=dtype, device=device)

    @classmethod
    def like(cls, t, left, right):
        """A buffer for a [B, H, Ls, D] tensor ``t`` with the tensor copied into ``local``."""
        B, H, Ls, D = t.shape
        buf = cls(B, H, Ls, D, left, right, t.dtype, t.device)
        buf.local.copy_(t.detach())
        return buf

    def seq_rows(self, lo, hi):
        """[B, hi - lo, H, D] in memory order (contiguous per batch row)."""
        return self.storage[:, self.left + lo:self.left + hi]

    def rows(self, lo, hi):
        return self.seq_rows(lo, hi).permute(0, 2, 1, 3)

    @property
    def local(self):
        return self.rows(0, self.Ls)


def _per_batch(t):
    """Contiguous pieces of a [B, rows, H, D] view whose batch rows are each contiguous."""
    return [t] if t.is_contiguous() else [t[b] for b in range(t.shape[0])]


def start_halo_exchange(kbuf: HaloBuffer, vbuf: HaloBuffer, left: int, right: int, group=None):
    """Post the K/V halo sends and receives (asynchronous) between neighbouring ranks: the last ``left`` rows of
    every shard go to rank+1's left spare rows, the first ``right`` rows to rank-1's right spare rows.  Returns
    (works, hl, hr): the number of halo rows this rank receives on each side (0 at the ends of the sequence).
    Wait on ``works`` before reading the spare rows."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    hl = left if rank > 0 else 0
    hr = right if rank < world - 1 else 0
    Ls = kbuf.Ls
    ops = []
    peer = _peer(group)
    for buf in (kbuf, vbuf):  # the same order on both sides of every pair: K pieces, then V pieces
        if rank < world - 1 and left > 0:  # my tail is the right neighbour's left halo
            ops += [dist.P2POp(dist.isend, t, peer(rank + 1), group) for t in _per_batch(buf.seq_rows(Ls - left, Ls))]
        if rank > 0 and right > 0:
            ops += [dist.P2POp(dist.isend, t, peer(rank - 1), group) for t in _per_batch(buf.seq_rows(0, right))]
        if hl > 0:
            ops += [dist.P2POp(dist.irecv, t, peer(rank - 1), group) for t in _per_batch(buf.seq_rows(-hl, 0))]
        if hr > 0:
            ops += [dist.P2POp(dist.irecv, t, peer(rank + 1), group) for t in _per_batch(buf.seq_rows(Ls, Ls + hr))]
    works = dist.batch_isend_irecv(ops) if ops else []
    return works, hl, hr


def start_halo_grad_exchange(part_left, hl, part_right, hr, left, right, like, group=None, dtype=torch.float32):
    """Post the return of the dK/dV rows computed for halo keys to their owners, in fp32 (asynchronous).
    ``part_left`` / ``part_right``: [2 (dK, dV), B, rows, H_kv, D] fp32 partial results of the boundary calls,
    whose first ``hl`` / last ``hr`` rows belong to the neighbours.  Returns (works, from_right, from_left):
    [2, B, left, H_kv, D] to add to this rank's last ``left`` key rows and [2, B, right, H_kv, D] for its first
    ``right`` rows (None where there is no neighbour)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    B, Hkv, _, D = like.shape
    ops, from_right, from_left = [], None, None
    peer = _peer(group)
    if rank < world - 1 and left > 0:  # the right neighbour used my last `left` rows as its left halo
        from_right = torch.empty((2, B, left, Hkv, D), dtype=dtype, device=like.device)
    if rank > 0 and right > 0:
        from_left = torch.empty((2, B, right, Hkv, D), dtype=dtype, device=like.device)
    for t in range(2):
        if hl > 0:
            ops += [dist.P2POp(dist.isend, part_left[t, b, :hl], peer(rank - 1), group) for b in range(B)]
        if hr > 0:
            n = part_right.shape[2]
            ops += [dist.P2POp(dist.isend, part_right[t, b, n - hr:], peer(rank + 1), group) for b in range(B)]
        if from_right is not None:
            ops += [dist.P2POp(dist.irecv, from_right[t, b], peer(rank + 1), group) for b in range(B)]
        if from_left is not None:
            ops += [dist.P2POp(dist.irecv, from_left[t, b], peer(rank - 1), group) for b in range(B)]
    works = dist.batch_isend_irecv(ops) if ops else []
    return works, from_right, from_left


# ------------------------------------------------------------------ local kernels (C ABI)
def cabi_local_forward(mask, q, k_ext, v_ext, q_offset, k_offset, seq_len, sm_scale, o, lse):
    """O, LSE of local query rows against local key rows with global offsets, written into ``o`` / ``lse``
    (which may be row slices of larger buffers)."""
    lib, functor = _library_for(mask)
    shape = _cabi.make_shape(q, k_ext, functor, mask.constargs, None, sm_scale, q_offset, k_offset, seq_len)
    _cabi.forward(lib, q, k_ext, v_ext, o, lse, shape)


def cabi_local_backward(mask, q, k_ext, v_ext, o, lse, do, q_offset, k_offset, seq_len, sm_scale, dq, dk, dv, part):
    """dQ (into ``dq``), 16-bit dK / dV (into ``dk`` / ``dv``) and, when ``part`` = (dk_part, dv_part, head, tail)
    is given, the un-rounded fp32 dK / dV of the first ``head`` and last ``tail`` key rows."""
    lib, functor = _library_for(mask)
    delta = torch.empty(q.shape[:3], dtype=torch.float32, device=q.device)
    shape = _cabi.make_shape(q, k_ext, functor, mask.constargs, None, sm_scale, q_offset, k_offset, seq_len)
    _cabi.backward(lib, q, k_ext, v_ext, o, do, lse, delta, dq, dk, dv, shape, part=part)


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
    if bl + br > Ls:  # tiny shard: treat every row as boundary (keys = halo_left + local + halo_right)
        return None
    return {"bl": bl, "br": br, "kl_hi": min(Ls, bl + right), "kr_lo": max(0, Ls - br - left)}


def _calls(Ls, hl, hr, left, right):
    """The local attention calls of one shard as (kind, first query row, end query row, first key row, end key
    row), rows relative to the shard's first position (key rows < 0 or >= Ls are halo rows)."""
    reg = _regions(Ls, hl, hr, left, right)
    if reg is None:
        return [("boundary", 0, Ls, -hl, Ls + hr)]
    calls = []
    if reg["bl"] > 0:
        calls.append(("boundary", 0, reg["bl"], -hl, reg["kl_hi"]))
    if reg["br"] > 0:
        calls.append(("boundary", Ls - reg["br"], Ls, reg["kr_lo"], Ls + hr))
    if Ls - reg["br"] > reg["bl"]:
        calls.append(("interior", reg["bl"], Ls - reg["br"], 0, Ls))
    return calls


class _SequenceShardedAttention(torch.autograd.Function):
    """Forward: post the halo exchange, run the interior rows (which see local keys only) while it is in
    flight, then the boundary rows against views of [halo | the local rows they can see].  Backward: the
    boundary rows first, so that the dK/dV they produce for halo keys travel back to their owners (in fp32)
    while the interior rows run; every key row that receives more than one contribution is summed in fp32 and
    rounded once.  No copy of K or V is made when they live in HaloBuffers."""

    @staticmethod
    def forward(ctx, q, k, v, mask, seq_len, sm_scale, group, local_forward, local_backward, halo_buffers):
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        B, H, Ls, D = q.shape
        left, right = halo_sizes(mask, Ls)
        cap_l = left if rank > 0 else 0
        cap_r = right if rank < world - 1 else 0
        if halo_buffers is None:
            kbuf, vbuf = HaloBuffer.like(k, cap_l, cap_r), HaloBuffer.like(v, cap_l, cap_r)
        else:
            kbuf, vbuf = halo_buffers
            for buf, t in ((kbuf, k), (vbuf, v)):
                if buf.local.data_ptr() != t.data_ptr() or buf.local.shape != t.shape or buf.local.stride() != t.stride():
                    raise ValueError("halo_buffers must be the HaloBuffers whose .local views were passed as k and v")
                if buf.left < cap_l or buf.right < cap_r:
                    raise ValueError(f"HaloBuffer has ({buf.left}, {buf.right}) spare rows, the mask needs ({cap_l}, {cap_r})")
        works, hl, hr = start_halo_exchange(kbuf, vbuf, left, right, group)
        base = rank * Ls
        o = torch.empty((B, H, Ls, D), dtype=q.dtype, device=q.device)
        lse = torch.empty((B, H, Ls), dtype=torch.float32, device=q.device)
        calls = _calls(Ls, hl, hr, left, right)
        waited = False
        for kind, q0, q1, k0, k1 in sorted(calls, key=lambda c: c[0] != "interior"):  # interior first
            if kind != "interior" and not waited:
                for w in works:
                    w.wait()
                waited = True
            local_forward(mask, q[:, :, q0:q1], kbuf.rows(k0, k1), vbuf.rows(k0, k1), base + q0, base + k0, seq_len,
                          sm_scale, o=o[:, :, q0:q1], lse=lse[:, :, q0:q1])
        if not waited:
            for w in works:
                w.wait()
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.bufs = (kbuf, vbuf)
        ctx.cfg = (mask, seq_len, sm_scale, group, local_backward, hl, hr, left, right, base, calls)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        kbuf, vbuf = ctx.bufs
        mask, seq_len, sm_scale, group, local_backward, hl, hr, left, right, base, calls = ctx.cfg
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        B, H, Ls, D = q.shape
        Hkv = k.shape[1]
        dev = q.device
        acc_dtype = torch.float64 if k.dtype == torch.float64 else torch.float32
        do = do.contiguous()
        # Gradients in the memory order of their tensors (a dense K / V view of a HaloBuffer is position-major):
        # autograd then accumulates them as they are instead of re-laying them out with a strided copy.
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        interior = [c for c in calls if c[0] == "interior"]
        boundary = [c for c in calls if c[0] != "interior"]
        # Key rows that get more than one contribution (this rank's boundary and interior calls, the neighbours'
        # boundary calls) are summed in fp32: the first `hd` and the last `tl` rows of the shard.
        hd = max([c[4] for c in boundary if c[3] <= 0] + [right if rank > 0 else 0] + [0])
        tl = max([Ls - max(c[3], 0) for c in boundary if c[4] >= Ls and c[3] > 0] + [left if rank < world - 1 else 0] + [0])
        hd, tl = min(hd, Ls), min(tl, Ls)
        if not interior or hd + tl > Ls:
            hd, tl = Ls, 0
        acc = None

        def run(call, part_buf, head, tail):
            _, q0, q1, k0, k1 = call
            part = (part_buf[0].permute(0, 2, 1, 3), part_buf[1].permute(0, 2, 1, 3), head, tail)
            if call[0] == "interior":
                dkc, dvc = dk, dv  # the 16-bit results of the rows in between are final
            else:
                dkc = torch.empty((B, Hkv, k1 - k0, D), dtype=k.dtype, device=dev)
                dvc = torch.empty_like(dkc)
            local_backward(mask, q[:, :, q0:q1], kbuf.rows(k0, k1), vbuf.rows(k0, k1), o[:, :, q0:q1], lse[:, :, q0:q1],
                           do[:, :, q0:q1], base + q0, base + k0, seq_len, sm_scale, dq=dq[:, :, q0:q1], dk=dkc, dv=dvc,
                           part=part)

        parts = []  # (fp32 [2, B, rows, Hkv, D], first key row relative to the shard)
        part_left = part_right = None
        for call in boundary:
            _, q0, q1, k0, k1 = call
            buf = torch.empty((2, B, k1 - k0, Hkv, D), dtype=acc_dtype, device=dev)
            run(call, buf, k1 - k0, 0)
            parts.append((buf, k0))
            if k0 < 0:
                part_left = buf
            if k1 > Ls:
                part_right = buf
        works, from_right, from_left = start_halo_grad_exchange(part_left, hl, part_right, hr, left, right, k, group, acc_dtype)
        if hd + tl > 0:
            if interior:
                acc = torch.empty((2, B, hd + tl, Hkv, D), dtype=acc_dtype, device=dev)
                run(interior[0], acc, hd, tl)
            else:
                acc = torch.zeros((2, B, hd + tl, Hkv, D), dtype=acc_dtype, device=dev)
        elif interior:
            run(interior[0], torch.empty((2, B, 0, Hkv, D), dtype=acc_dtype, device=dev), 0, 0)

        def add_rows(t, row0):
            """acc += t for the shard's key rows [row0, row0 + rows of t) that lie inside it."""
            n = t.shape[2]
            lo, hi = max(row0, 0), min(row0 + n, Ls)
            done = 0
            a, b = lo, min(hi, hd)  # part in the head region
            if b > a:
                acc[:, :, a:b] += t[:, :, a - row0:b - row0]
                done += b - a
            a, b = max(lo, Ls - tl), hi  # part in the tail region
            if b > a:
                acc[:, :, hd + a - (Ls - tl):hd + b - (Ls - tl)] += t[:, :, a - row0:b - row0]
                done += b - a
            assert done == max(hi - lo, 0), "a partial dK/dV row has no fp32 accumulator"

        for buf, k0 in parts:
            add_rows(buf, k0)
        for w in works:
            w.wait()
        if from_right is not None:
            add_rows(from_right, Ls - left)
        if from_left is not None:
            add_rows(from_left, 0)
        if acc is not None:
            for dst, src in ((dk, acc[0]), (dv, acc[1])):
                if hd > 0:
                    dst[:, :, :hd].copy_(src[:, :hd].permute(0, 2, 1, 3))
                if tl > 0:
                    dst[:, :, Ls - tl:].copy_(src[:, hd:].permute(0, 2, 1, 3))
        return dq, dk, dv, None, None, None, None, None, None, None


def sequence_sharded_attention(q, k, v, mask: ChillMask, seq_len: int, sm_scale=None, group=None,
                               local_forward=cabi_local_forward, local_backward=cabi_local_backward,
                               halo_buffers=None):
    """Attention over a sequence split evenly across the ranks of ``group``.

    q, k, v: this rank's [B, H(_kv), L/N, D] shard (rank r holds positions [r*L/N, (r+1)*L/N));
    ``seq_len`` is the global length L.  Differentiable; returns this rank's shard of O.

    ``halo_buffers=(kbuf, vbuf)``: the HaloBuffers whose ``.local`` views are ``k`` and ``v``.  The neighbours'
    halo rows are then received straight into the buffers' spare rows and K / V are never copied; the spare
    rows must stay untouched until the backward pass has run.  Without it the call makes its own buffers and
    copies k and v into them once."""
    if sm_scale is None:
        sm_scale = q.shape[-1] ** -0.5
    return _SequenceShardedAttention.apply(q, k, v, mask, seq_len, sm_scale, group, local_forward, local_backward,
                                           halo_buffers)
