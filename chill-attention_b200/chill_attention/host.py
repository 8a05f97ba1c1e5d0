"""Forward + backward for callers whose tensors live in HOST memory.

``attention_fwd_bwd_host`` streams the batch through the GPU in chunks on three CUDA streams
(host->device copies, kernels, device->host copies) with double-buffered device staging, so the
PCIe transfers in both directions overlap each other and the kernels.  It drives the C ABI
directly (forward, delta, backward), no autograd graph.  Host tensors should be pinned
(``tensor.pin_memory()``); pageable memory works but serialises the copies.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from . import _cabi
from .chill import _resolve_functor
from .mask import ChillMask


def _heads_per_chunk(H, G, bytes_per_head, target_bytes):
    """Largest divisor of H that is a multiple of the GQA group size G and keeps a chunk under target_bytes
    (at least one group)."""
    best = G
    for ch in range(G, H + 1, G):
        if H % ch == 0 and ch * bytes_per_head <= target_bytes:
            best = ch
    return best


def attention_fwd_bwd_host(q, k, v, do, mask: ChillMask, sm_scale=None, out=None, chunk_batches: int = 1,
                           device=None, chunk_heads: int | None = None):
    """q, do: [B, H, L, D]; k, v: [B, H_kv, L, D] on the host.  Returns host tensors (o, dq, dk, dv)
    (pinned; pass ``out=(o, dq, dk, dv)`` to reuse buffers).  Synchronises before returning.

    The batch goes through the GPU in chunks of `chunk_batches` batch rows x `chunk_heads` heads (default: up to
    40 MB of input per chunk, whole GQA groups).  The first chunk's upload and the last chunk's download are the
    only transfers that nothing overlaps, which favours small chunks, but every chunk costs ~0.3 ms of host time
    (copies, events, launches): measured on C2 (67 MB per batch row) in one session, 8 chunks of 67 MB reach
    144 TFLOP/s, 16 chunks of 34 MB 153, 32 chunks of 17 MB 141."""
    device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    B, H, L, D = q.shape
    Hkv = k.shape[1]
    if sm_scale is None:
        sm_scale = D ** -0.5
    lib, functor = _resolve_functor(mask)
    if out is None:
        out = tuple(torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in (q, q, k, v))
    o_h, dq_h, dk_h, dv_h = out
    cb = max(1, min(chunk_batches, B))
    G = H // Hkv
    if chunk_heads is None:
        target = float(os.environ.get("CHILL_HOST_CHUNK_MB", "40")) * 1e6
        bytes_per_head = cb * L * D * q.element_size() * (2 + 2.0 / G)
        chunk_heads = _heads_per_chunk(H, G, bytes_per_head, target)
    ch = max(G, min(H, (chunk_heads // G) * G))
    if ch < H:
        cb = 1  # [b, h0:h1] of a contiguous [B, H, L, D] host tensor is one contiguous block only for a single b
    chk = ch // G
    with torch.cuda.device(device):
        s_in, s_cmp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        start = torch.cuda.Event()
        start.record()  # everything below is ordered after work already queued on the caller's stream
        for s in (s_in, s_cmp, s_out):
            s.wait_event(start)

        def dev(shape, dtype):
            return torch.empty(shape, dtype=dtype, device=device)

        slots = []
        for _ in range(2):
            slots.append({
                "in": [dev((cb, ch, L, D), q.dtype), dev((cb, chk, L, D), q.dtype), dev((cb, chk, L, D), q.dtype),
                       dev((cb, ch, L, D), q.dtype)],
                "out": [dev((cb, ch, L, D), q.dtype), dev((cb, ch, L, D), q.dtype), dev((cb, chk, L, D), q.dtype),
                        dev((cb, chk, L, D), q.dtype)],
                "lse": dev((cb, ch, L), torch.float32), "delta": dev((cb, ch, L), torch.float32),
                "in_free": None, "out_free": None,
            })
        # fp32 dQ scratch of the single-kernel backward, one per slot like the other staging buffers (allocated
        # here, on the caller's stream, so that the caching allocator can hand the same blocks out on the next call)
        shape0 = _cabi.make_shape(slots[0]["in"][0], slots[0]["in"][1], functor, mask.constargs, None, sm_scale)
        nacc = 0 if _cabi.is_deterministic() else lib.chill_bwd_dq_accum_bytes(C.byref(shape0))
        for sl in slots:
            sl["accum"] = dev((nacc // 4,), torch.float32) if nacc else None
        chunks = [(b0, h0) for b0 in range(0, B, cb) for h0 in range(0, H, ch)]
        for i, (b0, h0) in enumerate(chunks):
            b1 = min(B, b0 + cb)
            n = b1 - b0
            hs, ks = slice(h0, h0 + ch), slice(h0 // G, h0 // G + chk)
            sl = slots[i % 2]
            qd, kd, vd, dod = (t[:n] for t in sl["in"])
            od, dqd, dkd, dvd = (t[:n] for t in sl["out"])
            with torch.cuda.stream(s_in):
                if sl["in_free"] is not None:
                    s_in.wait_event(sl["in_free"])
                for dst, src, hsel in zip((qd, kd, vd, dod), (q, k, v, do), (hs, ks, ks, hs)):
                    dst.copy_(src[b0:b1, hsel], non_blocking=True)
                ev_in = torch.cuda.Event()
                ev_in.record(s_in)
            with torch.cuda.stream(s_cmp):
                s_cmp.wait_event(ev_in)
                if sl["out_free"] is not None:
                    s_cmp.wait_event(sl["out_free"])
                shape = _cabi.make_shape(qd, kd, functor, mask.constargs, None, sm_scale)
                _cabi.forward(lib, qd, kd, vd, od, sl["lse"][:n], shape)
                if sl["accum"] is not None:
                    _cabi.backward(lib, qd, kd, vd, od, dod, sl["lse"][:n], sl["delta"][:n], dqd, dkd, dvd, shape, sl["accum"])
                else:
                    _cabi.backward(lib, qd, kd, vd, od, dod, sl["lse"][:n], sl["delta"][:n], dqd, dkd, dvd, shape,
                                   deterministic=True)
                ev_cmp = torch.cuda.Event()
                ev_cmp.record(s_cmp)
                sl["in_free"] = ev_cmp
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_cmp)
                for dst, src, hsel in zip((o_h, dq_h, dk_h, dv_h), (od, dqd, dkd, dvd), (hs, hs, ks, ks)):
                    dst[b0:b1, hsel].copy_(src, non_blocking=True)
                ev_out = torch.cuda.Event()
                ev_out.record(s_out)
                sl["out_free"] = ev_out
        cur = torch.cuda.current_stream()
        for s in (s_in, s_cmp, s_out):
            ev = torch.cuda.Event()
            ev.record(s)
            cur.wait_event(ev)
        cur.synchronize()
    return o_h, dq_h, dk_h, dv_h
