"""Forward + backward for callers whose tensors live in HOST memory.

``attention_fwd_bwd_host`` hands host pointers to ``chill_fwd_bwd_host`` of the C ABI (csrc/host_pipeline.cu), which
streams the batch through the GPU in chunks on three CUDA streams (uploads, kernels, downloads) over two sets of
device staging buffers, so the PCIe transfers in both directions overlap each other and the kernels.  No autograd
graph.  Host tensors should be pinned (``tensor.pin_memory()``); pageable memory works but serialises the copies.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from . import _cabi
from .chill import _resolve_functor
from .mask import ChillMask


def _host_args(q, k, v, do, out, functor, mask, sm_scale, chunk_groups):
    a = _cabi.HostArgs()
    a.s = _cabi.make_shape(q, k, functor, mask.constargs, None, sm_scale,
                           flags=_cabi.FLAG_BWD_DETERMINISTIC if _cabi.is_deterministic() else 0)
    a.q, a.k, a.v, a.d_o = (t.data_ptr() for t in (q, k, v, do))
    a.o, a.dq, a.dk, a.dv = (t.data_ptr() for t in out)
    a.chunk_groups = chunk_groups
    return a


def chunk_schedule(q, k, mask: ChillMask, chunk_heads: int | None = None):
    """[(batch row, first kv-head group, groups)] of the chunks a call with these tensors is cut into (host only)."""
    lib, functor = _resolve_functor(mask)
    G = q.shape[1] // k.shape[1]
    a = _host_args(q, k, k, q, (q, q, k, k), functor, mask, 1.0, 0 if chunk_heads is None else max(1, chunk_heads // G))
    n = lib.chill_host_chunk_schedule(C.byref(a), None, 0)
    _cabi.check(lib, min(n, 0), "chill_host_chunk_schedule")
    buf = (C.c_int32 * (3 * n))()
    lib.chill_host_chunk_schedule(C.byref(a), buf, n)
    return [tuple(buf[3 * i:3 * i + 3]) for i in range(n)]


def attention_fwd_bwd_host(q, k, v, do, mask: ChillMask, sm_scale=None, out=None, chunk_batches: int = 1,
                           device=None, chunk_heads: int | None = None):
    """q, do: [B, H, L, D]; k, v: [B, H_kv, L, D] on the host.  Returns host tensors (o, dq, dk, dv)
    (pinned; pass ``out=(o, dq, dk, dv)`` to reuse buffers).  Synchronises before returning.

    The batch goes through the GPU in chunks of whole GQA groups of one batch row: at most `chunk_heads` heads
    (default: about CHILL_HOST_CHUNK_MB = 40 MB of input per chunk; measured on C2, 4.2 MB per head: 16 chunks of
    34 MB reach 155 TFLOP/s, 8 chunks of 67 MB 144).  `chunk_batches` is accepted for compatibility with earlier
    versions and has no effect."""
    device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    B, H, L, D = q.shape
    Hkv = k.shape[1]
    assert H % Hkv == 0 and k.shape == v.shape and do.shape == q.shape and q.dtype == k.dtype == v.dtype == do.dtype
    for t in (q, k, v, do):
        assert not t.is_cuda, "attention_fwd_bwd_host takes host tensors"
    if sm_scale is None:
        sm_scale = D ** -0.5
    lib, functor = _resolve_functor(mask)
    q, k, v, do = (t if t.is_contiguous() else t.contiguous() for t in (q, k, v, do))
    if out is None:
        out = tuple(torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in (q, q, k, v))
    for t, like in zip(out, (q, q, k, v)):
        assert t.shape == like.shape and t.dtype == like.dtype and t.is_contiguous() and not t.is_cuda
    G = H // Hkv
    if chunk_heads is None:
        per_group = L * D * q.element_size() * (2 * G + 2)
        target = float(os.environ.get("CHILL_HOST_CHUNK_MB", "40")) * 1e6
        big = max(1, min(Hkv, int(target // per_group)))
        n_chunks = -(-Hkv // big)
        chunk_groups = -(-Hkv // n_chunks)  # even split of a batch row
    else:
        chunk_groups = max(1, min(Hkv, chunk_heads // G))
    a = _host_args(q, k, v, do, out, functor, mask, float(sm_scale), chunk_groups)
    with torch.cuda.device(device):
        nbytes = lib.chill_host_workspace_bytes(C.byref(a))
        if nbytes == 0:
            raise ValueError("chill_fwd_bwd_host: unsupported arguments")
        work = torch.empty(nbytes + 256, dtype=torch.uint8, device=device)
        base = (work.data_ptr() + 255) // 256 * 256
        a.workspace, a.workspace_bytes = base, nbytes
        stream = torch.cuda.current_stream()
        _cabi.check(lib, lib.chill_fwd_bwd_host(C.byref(a), C.c_void_p(stream.cuda_stream)), "chill_fwd_bwd_host")
        stream.synchronize()  # outputs are in host memory; `work` may go back to the allocator
    return out
