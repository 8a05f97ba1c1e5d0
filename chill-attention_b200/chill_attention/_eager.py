"""Eager-mode call path of ``chill_attention``: same kernels, less host time per call.

Under ``torch.compile`` the operator is reached through its dispatcher ops
(``chill_attention::forward<Name>`` / ``backward<Name>``, chill.py).  In plain eager mode that route costs
more host time than a short sequence needs on the GPU (a Python custom op is entered through the dispatcher
twice, its autograd rule is another Python layer, and every call rebuilds the C-ABI argument structs field by
field): about 115 us per forward and 180 us per backward call, whatever the problem size.  Here an eager call
goes straight from ``chill_attention()`` to a ``torch.autograd.Function`` whose two halves keep their C-ABI
structs (geometry, strides, mask constants) in a per-thread cache keyed by everything but the data pointers,
so a call only allocates its outputs, stores the pointers and enqueues the kernels.

The path is taken only for plain CUDA tensors outside of tracing / dispatch modes / functorch transforms
(``usable``); everything else, and every ``torch.compile`` graph, uses the dispatcher ops.  Set
``CHILL_ATTENTION_EAGER_FAST=0`` to switch it off.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

import torch

from . import _cabi

ENABLED = os.environ.get("CHILL_ATTENTION_EAGER_FAST", "1") not in ("", "0")
_tls = threading.local()  # the cached structs are rewritten by every call: one set per host thread


_dispatch_depth = getattr(torch._C, "_len_torch_dispatch_stack", None)
_function_depth = getattr(torch._C, "_len_torch_function_stack", None)
_functorch_top = getattr(getattr(torch._C, "_functorch", None), "peek_interpreter_stack", None)
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_PROBES_OK = None not in (_dispatch_depth, _function_depth, _functorch_top)
_Tensor = torch.Tensor


def usable(q, k, v, lens) -> bool:
    """True when nothing is watching the dispatcher: plain tensors, no tracing, no modes, no transforms.
    (A torch without the probes used here stays on the dispatcher path.)"""
    if not (ENABLED and _PROBES_OK) or type(q) is not _Tensor or type(k) is not _Tensor or type(v) is not _Tensor:
        return False
    if not q.is_cuda or (lens is not None and type(lens) is not _Tensor):
        return False
    return _dispatch_depth() == 0 and _function_depth() == 0 and _functorch_top() is None


def _stream(device_index):
    if _raw_stream is not None:
        return C.c_void_p(_raw_stream(device_index))
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _cache():
    c = getattr(_tls, "cache", None)
    if c is None:
        c = _tls.cache = {}
    return c


def _pack(q, k, v):
    """See chill._tensor_core_operands: 16-bit operands TMA cannot describe are packed once."""
    if q.dtype == torch.float32 or q.shape[-1] not in (64, 128, 256):
        return q, k, v
    ok = _cabi.tma_compatible
    if ok(q) and ok(k) and ok(v):
        return q, k, v
    return tuple(t if ok(t) else t.contiguous() for t in (q, k, v))


def _forward(entry, q, k, v, lens, mask_args, sm_scale, want_lse, flags):
    lib, functor_id = entry
    # everything the argument checks look at is part of the key, so a hit has passed them before
    key = ("f", id(lib), functor_id, mask_args, q.shape, q.stride(), k.shape, k.stride(), v.shape, v.stride(), q.dtype,
           k.dtype, v.dtype, k.device, v.device, sm_scale, flags, want_lse)
    cache = _cache()
    a = cache.get(key)
    if lens is not None:
        assert lens.dtype == torch.int32 and lens.ndim == 1 and lens.shape[0] == q.shape[0] and lens.device == q.device
    o = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    lse = torch.empty(q.shape[:3], dtype=torch.float32, device=q.device) if want_lse else None
    if a is None:
        from .chill import _check_inputs

        _check_inputs(q, k, v, lens, sm_scale)
        a = _cabi.FwdArgs()
        a.s = _cabi.make_shape(q, k, functor_id, mask_args, None, sm_scale, flags=flags)
        a.q_strides, a.k_strides, a.v_strides, a.o_strides = (_cabi._strides(t, 4) for t in (q, k, v, o))
        if lse is not None:
            a.lse_strides = _cabi._strides(lse, 3)
        if len(cache) > 256:
            cache.clear()
        cache[key] = a
    a.q, a.k, a.v, a.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
    a.lse = lse.data_ptr() if lse is not None else None
    a.s.lens = lens.data_ptr() if lens is not None else None
    st = lib.chill_fwd(C.byref(a), _stream(q.device.index))
    if st != 0:
        _cabi.check(lib, st, "chill_fwd")
    return o, lse


def _backward(entry, q, k, v, lens, o, lse, do, mask_args, sm_scale, d_lse, flags=0):
    from .chill import _BWD_PATHS, _backward_operand

    lib, functor_id = entry
    do = _backward_operand(do)
    deterministic = _cabi.is_deterministic()
    key = ("b", id(lib), functor_id, mask_args, q.shape, q.stride(), k.shape, k.stride(), v.stride(), o.stride(),
           do.stride(), lse.stride(), q.dtype, sm_scale, lens is None, deterministic, flags,
           None if d_lse is None else d_lse.stride())
    cache = _cache()
    ent = cache.get(key)
    dev = q.device
    delta = torch.empty(q.shape[:3], dtype=torch.float32, device=dev)
    dq = torch.empty(q.shape, dtype=q.dtype, device=dev)
    dk = torch.empty(k.shape, dtype=k.dtype, device=dev)
    dv = torch.empty(v.shape, dtype=v.dtype, device=dev)
    if ent is None:
        shape = _cabi.make_shape(q, k, functor_id, mask_args, None, sm_scale, flags=flags)
        a = _cabi.backward_args(q, k, v, o, do, lse, delta, dq, dk, dv, shape, None, d_lse)
        tc = lib.chill_bwd_uses_tensor_cores(C.byref(a)) == 1
        nacc = lib.chill_bwd_dq_accum_bytes(C.byref(a.s)) if (tc and not deterministic) else 0
        ent = (a, tc, nacc // 4)
        if len(cache) > 256:
            cache.clear()
        cache[key] = ent
    a, tc, nacc = ent
    _BWD_PATHS["tensor_core" if tc else "generic"] += 1
    accum = torch.empty(nacc, dtype=torch.float32, device=dev) if nacc else None
    a.q, a.k, a.v, a.o, a.d_o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr()
    a.lse, a.delta = lse.data_ptr(), delta.data_ptr()
    a.dq, a.dk, a.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    a.dq_accum = accum.data_ptr() if accum is not None else None
    a.d_lse = d_lse.data_ptr() if d_lse is not None else None
    a.s.lens = lens.data_ptr() if lens is not None else None
    stream = _stream(dev.index)
    st = lib.chill_bwd_delta(C.byref(a), stream)
    if st == 0:
        st = lib.chill_bwd(C.byref(a), stream)
    if st != 0:
        _cabi.check(lib, st, "chill_bwd")
    return dq, dk, dv


class _ChillAttentionEager(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, lens, entry, mask_args, sm_scale, return_lse, flags):
        q, k, v = _pack(q, k, v)  # the packed copies are what the backward reads again
        o, lse = _forward(entry, q, k, v, lens, mask_args, sm_scale, True, flags)
        ctx.save_for_backward(q, k, v, o, lse, lens)
        ctx.entry, ctx.mask_args, ctx.sm_scale, ctx.flags = entry, mask_args, sm_scale, flags
        ctx.set_materialize_grads(False)
        if not return_lse:
            ctx.mark_non_differentiable(lse)
        return o, lse

    @staticmethod
    def backward(ctx, do, dlse):
        q, k, v, o, lse, lens = ctx.saved_tensors
        if do is None:
            do = torch.zeros_like(o)
        d_lse = dlse.float() if dlse is not None else None  # a gradient that reached the returned LSE is propagated
        if q.device.index != torch._C._cuda_getDevice():
            with torch.cuda.device(q.device):
                dq, dk, dv = _backward(ctx.entry, q, k, v, lens, o, lse, do, ctx.mask_args, ctx.sm_scale, d_lse, ctx.flags)
        else:
            dq, dk, dv = _backward(ctx.entry, q, k, v, lens, o, lse, do, ctx.mask_args, ctx.sm_scale, d_lse, ctx.flags)
        return dq, dk, dv, None, None, None, None, None, None


def attention(entry, q, k, v, lens, mask_args, sm_scale, return_lse, flags):
    """O, or (O, LSE): the eager counterpart of chill._chill_attention."""
    if lens is not None and not lens.is_contiguous():
        lens = lens.contiguous()
    needs_grad = torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad)
    if q.device.index != torch._C._cuda_getDevice():
        with torch.cuda.device(q.device):
            return _attention(entry, q, k, v, lens, mask_args, sm_scale, return_lse, flags, needs_grad)
    return _attention(entry, q, k, v, lens, mask_args, sm_scale, return_lse, flags, needs_grad)


def _attention(entry, q, k, v, lens, mask_args, sm_scale, return_lse, flags, needs_grad):
    if needs_grad:
        o, lse = _ChillAttentionEager.apply(q, k, v, lens, entry, mask_args, sm_scale, return_lse, flags)
    else:
        q, k, v = _pack(q, k, v)
        o, lse = _forward(entry, q, k, v, lens, mask_args, sm_scale, return_lse, flags)
    return (o, lse) if return_lse else o
