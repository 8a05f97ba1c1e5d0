"""Public API: ``chill_attention`` and ``register_chill_mask``.

Same call surface as the reference (chill_attention/chill.py:579-645 and :30-495):
one pair of dispatcher ops per mask CLASS NAME,

    chill_attention::forward<Name>(q, k, v, lens, mask_args, sm_scale, return_lse,
                                   prescale_qk, precision, autotune) -> (O, LSE)
    chill_attention::backward<Name>(q, k, v, lens, o, lse, do, mask_args, sm_scale,
                                    prescale_qk, precision, autotune) -> (dQ, dK, dV)

registered as ``torch.library.custom_op`` with fake (meta) implementations and an
autograd rule, so the call is opaque to and safe under ``torch.compile``.  The op
bodies hand raw device pointers to the C ABI (include/chill_b200.h); kernels run on
the current CUDA stream.  ``autotune`` and ``prescale_qk`` are accepted for
compatibility and have no effect: there is nothing to tune at run time and the
softmax scale is always applied in fp32 inside the exponent.
``precision`` only matters for fp32 inputs: "ieee" (default) computes them with IEEE fp32 FMAs, "tf32" lets the
forward and the backward (head dim 64 / 128) run on the tensor cores in TF32.
"""
from __future__ import annotations

import logging
import typing

import torch

from . import _cabi, _eager
from .mask import ChillMask

logger = logging.getLogger(__name__)

_HEAD_DIMS = {16, 32, 64, 128, 256}
#: how many backward calls each kernel family served (read by tests; see backward_path_counts)
_BWD_PATHS = {"tensor_core": 0, "generic": 0}


def backward_path_counts() -> dict:
    """Copy of the per-process counters of backward calls served by the tensor-core and by the generic kernels."""
    return dict(_BWD_PATHS)


def _backward_operand(do: torch.Tensor) -> torch.Tensor:
    """The incoming gradient as the kernels want it.  Autograd often hands over an expanded tensor (all strides 0
    after ``o.sum().backward()``) or a transposed view; the tensor-core kernels cannot describe those to TMA and
    the call would otherwise be served by the ~1000x slower generic kernels.  One L x D copy fixes that (the
    reference asserts ``do.stride(-1) == 1`` at this point, chill.py:270)."""
    return do if _cabi.tma_compatible(do) else do.contiguous()


#: 16-bit head dims that chill_attention() zero-pads to _PADDED_TO channels (tensor-core kernels instead of generic)
_PADDED_HEAD_DIMS = (16, 32)
_PADDED_TO = 64


def _tensor_core_operands(q, k, v):
    """16-bit q, k, v with a head dimension the tensor-core kernels serve, but in a memory layout TMA cannot describe
    (channel stride != 1, a broadcast dimension, rows not 16-byte aligned): one packing copy each puts them on the
    tensor-core path, ~1000x faster than the generic kernels that would otherwise take the call.  The reference reads
    such tensors through block pointers at full speed (chill_fwd.py:74-98); results are identical either way."""
    if q.dtype == torch.float32 or q.shape[-1] not in (64, 128, 256):
        return q, k, v
    return tuple(t if _cabi.tma_compatible(t) else t.contiguous() for t in (q, k, v))


def _precision_flags(precision, dtype) -> int:
    """precision="tf32" (the reference's tl.dot input_precision) lets fp32 tensors use the TF32 tensor cores."""
    return _cabi.FLAG_ALLOW_TF32 if (precision == "tf32" and dtype == torch.float32) else 0


def _run_backward(lib, functor_id, q, k, v, lens, o, lse, do, mask_args, sm_scale, d_lse=None, flags=0):
    import ctypes as C

    q, k, v = _tensor_core_operands(q, k, v)
    with torch.cuda.device(q.device):
        do = _backward_operand(do)
        delta = torch.empty(o.shape[:-1], dtype=torch.float32, device=o.device)
        DQ = torch.empty_like(q, memory_format=torch.contiguous_format)
        DK = torch.empty_like(k, memory_format=torch.contiguous_format)
        DV = torch.empty_like(v, memory_format=torch.contiguous_format)
        lens_c = lens.contiguous() if lens is not None else None
        shape = _cabi.make_shape(q, k, functor_id, mask_args, lens_c, sm_scale, flags=flags)
        a = _cabi.backward_args(q, k, v, o, do, lse, delta, DQ, DK, DV, shape, None, d_lse)
        tc = lib.chill_bwd_uses_tensor_cores(C.byref(a)) == 1
        _BWD_PATHS["tensor_core" if tc else "generic"] += 1
        accum = _cabi.dq_accum_for(lib, a, q.device) if tc else None
        a.dq_accum = accum.data_ptr() if accum is not None else None
        st = _cabi._stream()
        _cabi.check(lib, lib.chill_bwd_delta(C.byref(a), st), "chill_bwd_delta")
        _cabi.check(lib, lib.chill_bwd(C.byref(a), st), "chill_bwd")
    return DQ, DK, DV
#: mask class name -> (library, functor id); filled by register_chill_mask
_REGISTRY: dict[str, tuple] = {}


def _resolve_functor(mask: ChillMask):
    """Library + functor id serving this mask class (builds a custom library if needed)."""
    functor = getattr(mask, "cuda_functor", None)
    header = getattr(mask, "cuda_functor_header", None)
    if header is not None:
        from .custom import build_custom_library

        if not functor:
            raise ValueError(f"{mask.name}: cuda_functor_header is set but cuda_functor (struct name) is not")
        return _cabi.load_library(build_custom_library(header, functor)), _cabi.MASK_CUSTOM
    if functor in _cabi.BUILTIN_FUNCTOR_IDS:
        return _cabi.load_library(), _cabi.BUILTIN_FUNCTOR_IDS[functor]
    raise NotImplementedError(
        f"{mask.name} has no CUDA functor: set `cuda_functor` to a built-in functor name or provide "
        "`cuda_functor_header` + `cuda_functor` (see chill_attention/custom.py)"
    )


def _check_inputs(q, k, v, lens, sm_scale):
    batch, heads, T, D = q.shape
    assert heads % k.shape[1] == 0
    assert D in _HEAD_DIMS
    assert D == k.shape[-1] and D == v.shape[-1]
    assert T == k.shape[-2] and T == v.shape[-2]
    assert k.shape[1] == v.shape[1] and k.shape[0] == batch and v.shape[0] == batch
    assert q.dtype == k.dtype == v.dtype and q.dtype in (torch.float32, torch.float16, torch.bfloat16)
    assert sm_scale is not None
    assert lens is None or (lens.dtype == torch.int32 and batch == len(lens) and lens.ndim == 1)
    assert q.is_cuda and k.is_cuda and v.is_cuda, "chill_attention runs on CUDA tensors only"


def register_chill_mask(mask: ChillMask):
    """Create and register the forward/backward ops of ``type(mask)`` (idempotent per class name)."""
    mask_name = mask.name
    if hasattr(torch.ops.chill_attention, f"forward{mask_name}"):
        return
    lib, functor_id = _resolve_functor(mask)
    _REGISTRY[mask_name] = (lib, functor_id)  # also what the eager call path (_eager.py) looks up

    @torch.library.custom_op(f"chill_attention::forward{mask_name}", mutates_args=(), device_types=("cuda",))
    def attention_forward_adapter(
        q: torch.Tensor,
        k: torch.Tensor,
        v: torch.Tensor,
        lens: typing.Optional[torch.Tensor],
        mask_args: typing.List[typing.Union[int, float, bool]],
        sm_scale: float,
        return_lse: bool,
        prescale_qk: bool,
        precision: str,
        autotune: bool,
    ) -> tuple[torch.Tensor, torch.Tensor]:
        _check_inputs(q, k, v, lens, sm_scale)
        q, k, v = _tensor_core_operands(q, k, v)
        with torch.cuda.device(q.device):
            O = torch.empty_like(q, memory_format=torch.contiguous_format)
            LSE = torch.empty(q.shape[:3], dtype=torch.float32, device=q.device) if return_lse else None
            lens_c = lens.contiguous() if lens is not None else None
            flags = _precision_flags(precision, q.dtype)
            shape = _cabi.make_shape(q, k, functor_id, mask_args, lens_c, sm_scale, flags=flags)
            _cabi.forward(lib, q, k, v, O, LSE, shape)
        if LSE is None:
            LSE = torch.empty(0, dtype=torch.float32, device=q.device)
        return O, LSE

    @torch.library.register_fake(f"chill_attention::forward{mask_name}")
    def attention_forward_adapter_abstract(q, k, v, lens, mask_args, sm_scale, return_lse, prescale_qk, precision,
                                           autotune):
        return (
            torch.empty_like(q, memory_format=torch.contiguous_format),
            torch.empty(q.shape[:3] if return_lse else (0,), dtype=torch.float32, device=q.device),
        )

    @torch.library.custom_op(f"chill_attention::backward{mask_name}", mutates_args=(), device_types=("cuda",))
    def attention_backward_adapter(
        q: torch.Tensor,
        k: torch.Tensor,
        v: torch.Tensor,
        lens: typing.Optional[torch.Tensor],
        o: torch.Tensor,
        lse: torch.Tensor,
        do: torch.Tensor,
        mask_args: typing.List[typing.Union[int, float, bool]],
        sm_scale: float,
        prescale_qk: bool,
        precision: str,
        autotune: bool,
    ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        return _run_backward(lib, functor_id, q, k, v, lens, o, lse, do, mask_args, sm_scale,
                             flags=_precision_flags(precision, q.dtype))

    @torch.library.register_fake(f"chill_attention::backward{mask_name}")
    def attention_backward_adapter_abstract(q, k, v, lens, o, lse, do, mask_args, sm_scale, prescale_qk, precision,
                                            autotune):
        return (
            torch.empty_like(q, memory_format=torch.contiguous_format),
            torch.empty_like(k, memory_format=torch.contiguous_format),
            torch.empty_like(v, memory_format=torch.contiguous_format),
        )

    # Same computation with one more input, the gradient that reached the returned LSE.  The reference has no
    # such op: its backward drops that gradient (chill.py:466-490), so differentiating through `return_lse=True`
    # silently gives wrong gradients there.  backward<Name> above keeps the reference's schema; this op is used
    # only when a gradient for the LSE actually arrives.
    @torch.library.custom_op(f"chill_attention::backward_with_dlse{mask_name}", mutates_args=(), device_types=("cuda",))
    def attention_backward_dlse_adapter(
        q: torch.Tensor,
        k: torch.Tensor,
        v: torch.Tensor,
        lens: typing.Optional[torch.Tensor],
        o: torch.Tensor,
        lse: torch.Tensor,
        do: torch.Tensor,
        dlse: torch.Tensor,
        mask_args: typing.List[typing.Union[int, float, bool]],
        sm_scale: float,
    ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        return _run_backward(lib, functor_id, q, k, v, lens, o, lse, do, mask_args, sm_scale, d_lse=dlse.float())

    @torch.library.register_fake(f"chill_attention::backward_with_dlse{mask_name}")
    def attention_backward_dlse_adapter_abstract(q, k, v, lens, o, lse, do, dlse, mask_args, sm_scale):
        return (
            torch.empty_like(q, memory_format=torch.contiguous_format),
            torch.empty_like(k, memory_format=torch.contiguous_format),
            torch.empty_like(v, memory_format=torch.contiguous_format),
        )

    def setup_context(ctx, inputs, output):
        O, LSE = output
        q, k, v, lens, mask_args, sm_scale, return_lse, prescale_qk, precision, autotune = inputs
        ctx.save_for_backward(q, k, v, O, LSE, lens)
        ctx.set_materialize_grads(False)  # an unused output arrives as None instead of a tensor of zeros
        ctx.mask_args = mask_args
        ctx.sm_scale = sm_scale
        ctx.prescale_qk = prescale_qk
        ctx.precision = precision
        ctx.autotune = autotune

    def backward(ctx, do, dlse):
        q, k, v, o, lse, lens = ctx.saved_tensors
        if do is None:
            do = torch.zeros_like(o)
        if dlse is not None and dlse.numel() == lse.numel() and lse.numel() > 0:
            # a gradient reached the returned LSE: propagate it (the reference drops it, chill.py:466-490)
            DQ, DK, DV = attention_backward_dlse_adapter(
                q=q, k=k, v=v, lens=lens, o=o, lse=lse, do=do, dlse=dlse, mask_args=ctx.mask_args, sm_scale=ctx.sm_scale,
            )
        else:
            DQ, DK, DV = attention_backward_adapter(
                q=q, k=k, v=v, lens=lens, o=o, lse=lse, do=do, mask_args=ctx.mask_args, sm_scale=ctx.sm_scale,
                prescale_qk=ctx.prescale_qk, precision=ctx.precision, autotune=ctx.autotune,
            )
        return DQ, DK, DV, None, None, None, None, None, None, None

    attention_forward_adapter.register_autograd(backward, setup_context=setup_context)


def _chill_reference_naive(mask: ChillMask, q, k, v, lens):
    """Dense-mask attention in plain PyTorch, for tests (same contract as the reference's helper of this name,
    chill.py:498-544): returns ``(output * row_mask, row_mask)`` where ``row_mask`` zeroes query rows at or beyond
    ``lens[b]`` (a 0-dim 1 when ``lens`` is None).  Keys at or beyond ``lens[b]`` are never attended.
    Scores are scaled by head_dim ** -0.5; a row that sees no key yields zeros."""
    B, H, T, D = q.shape
    assert k.shape[2] == T and v.shape[2] == T
    groups = H // k.shape[1]
    if groups > 1:  # grouped-query attention: every kv head serves `groups` consecutive query heads
        k, v = (t[:, :, None].expand(B, t.shape[1], groups, T, D).reshape(B, H, T, D) for t in (k, v))
    visible = mask.make_mask(T, device=q.device)[None, None]  # [1, 1, T, T]
    row_mask = torch.ones((), dtype=torch.bool, device=q.device)
    if lens is not None:
        inside = torch.arange(T, device=q.device)[None, :] < lens[:, None]  # [B, T]
        visible = visible & inside[:, None, None, :] & inside[:, None, :, None]
        row_mask = inside[:, None, :, None]
    scores = torch.matmul(q, k.transpose(-1, -2)) * (D ** -0.5)
    scores = scores.masked_fill(~visible, float("-inf"))
    probs = torch.softmax(scores.float(), dim=-1).nan_to_num(0.0).to(q.dtype)  # all -inf row -> zeros
    return torch.matmul(probs, v) * row_mask, row_mask


def _chill_attention(q, k, v, lens, mask_name, mask_args, sm_scale, return_lse, prescale_qk, precision, autotune):
    requires_grad = any(i.requires_grad for i in (q, k, v))
    attention_forward = getattr(torch.ops.chill_attention, f"forward{mask_name}")
    O, LSE = attention_forward(
        q=q, k=k, v=v, lens=lens, mask_args=mask_args, sm_scale=sm_scale, prescale_qk=prescale_qk,
        return_lse=return_lse or requires_grad, precision=precision, autotune=autotune,
    )
    if return_lse:
        return O, LSE
    return O


def chill_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    mask: ChillMask,
    lens: torch.Tensor | None = None,
    sm_scale: float | None = None,
    return_lse=False,
    prescale_qk=False,
    precision="ieee",
    autotune=False,
):
    """Exact softmax attention restricted to the pairs ``mask`` allows.

    Args:
        q: [batch, heads, seq_len, head_dim]; k, v: [batch, kv_heads, seq_len, head_dim]
           (kv_heads divides heads: grouped-query attention).  fp16 / bf16 / fp32, any strides.
        mask: a ChillMask instance.
        lens: optional int32 [batch] valid lengths.
        sm_scale: softmax scale, default head_dim ** -0.5.
        return_lse: also return the log-sum-exp of every row in log2 units, shape [batch, heads, seq_len].
        prescale_qk, autotune: accepted for compatibility with the reference, no effect.
        precision: "ieee" or "tf32"; for fp32 inputs "tf32" runs forward and backward (head dim 64 / 128) on the
            tensor cores in TF32 (~1e-3 error instead of ~1e-6), everything else is IEEE fp32.

    fp16 / bf16 tensors with head dim 16 or 32 are zero-padded to 64 channels here, so that they run the tensor-core
    kernels (zero channels change neither Q K^T nor the first head_dim columns of P V; autograd slices the gradients
    back).  The reference serves these head dims with tl.dot directly (chill.py:81-92).

    Returns: O, or (O, LSE) when ``return_lse``.
    """
    entry = _REGISTRY.get(mask.name)
    if entry is None:
        register_chill_mask(mask)
        entry = _REGISTRY.get(mask.name)
    if sm_scale is None:
        sm_scale = 1.0 / (q.shape[-1] ** 0.5)
    head_dim = q.shape[-1]
    if head_dim in _PADDED_HEAD_DIMS and q.dtype in (torch.float16, torch.bfloat16) and q.is_cuda \
            and k.shape[-1] == head_dim and v.shape[-1] == head_dim and k.dtype == q.dtype and v.dtype == q.dtype:
        pad = (0, _PADDED_TO - head_dim)
        out = chill_attention(
            torch.nn.functional.pad(q, pad), torch.nn.functional.pad(k, pad), torch.nn.functional.pad(v, pad), mask,
            lens=lens, sm_scale=sm_scale, return_lse=return_lse, prescale_qk=prescale_qk, precision=precision,
            autotune=autotune,
        )
        if return_lse:
            return out[0][..., :head_dim].contiguous(), out[1]
        return out[..., :head_dim].contiguous()
    compiling = torch.compiler.is_compiling()
    if not compiling and entry is not None and _eager.usable(q, k, v, lens):
        # plain eager call: same kernels through the short host path (see _eager.py), which validates the arguments
        flags = _precision_flags(precision, q.dtype)
        return _eager.attention(entry, q, k, v, lens, mask.constargs, float(sm_scale), bool(return_lse), flags)
    if not compiling:
        for i in (q, k, v):
            if getattr(i, "_dynamo_static_indices", None) != {1, 3}:
                torch._dynamo.mark_static(i, 1)
                torch._dynamo.mark_static(i, 3)
    return _chill_attention(
        q=q, k=k, v=v, lens=lens, mask_name=mask.name, mask_args=mask.constargs, sm_scale=sm_scale,
        return_lse=return_lse, prescale_qk=prescale_qk, precision=precision, autotune=autotune,
    )
