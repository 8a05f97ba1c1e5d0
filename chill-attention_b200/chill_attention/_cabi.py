"""ctypes binding of the C ABI declared in include/chill_b200.h.

The shared library is built in-tree (``python chill-attention_b200/build.py``) as
``chill_attention/_lib/libchill_b200.so``.  There is no other implementation behind
this module: if the library is missing, or a call returns a non-zero status, the
caller gets an exception.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_DIR = os.path.join(_HERE, "_lib")
DEFAULT_LIB = os.path.join(LIB_DIR, "libchill_b200.so")

CHILL_F32, CHILL_F16, CHILL_BF16 = 0, 1, 2
MASK_FULL, MASK_CAUSAL, MASK_SLIDING, MASK_CHUNKWISE, MASK_PREFIXLM, MASK_CUSTOM = range(6)
FLAG_FORCE_GENERIC, FLAG_REQUIRE_TC, FLAG_BWD_ONLY_DKDV, FLAG_BWD_ONLY_DQ, FLAG_ALLOW_TF32 = 1, 2, 4, 8, 16
MAX_MASK_ARGS = 8

BUILTIN_FUNCTOR_IDS = {
    "FullMask": MASK_FULL,
    "CausalMask": MASK_CAUSAL,
    "SlidingWindowMask": MASK_SLIDING,
    "ChunkwiseMask": MASK_CHUNKWISE,
    "PrefixLMMask": MASK_PREFIXLM,
}

_DTYPES = {torch.float32: CHILL_F32, torch.float16: CHILL_F16, torch.bfloat16: CHILL_BF16}

ABI_VERSION = 5
FLAG_BWD_DETERMINISTIC = 32
SELFTEST_STATUS = 901

EXPORTS = (
    "chill_fwd", "chill_bwd_delta", "chill_bwd", "chill_bwd_noalloc", "chill_bwd_scratch_bytes", "chill_bwd_dq_accum_bytes",
    "chill_fwd_uses_tensor_cores",
    "chill_bwd_uses_tensor_cores", "chill_mask_tabulate", "chill_mask_tabulate_blocks", "chill_mask_traits",
    "chill_read_device_status", "chill_selftest_bounded_wait",
    "chill_launch_count", "chill_abi_version", "chill_status_string", "chill_last_cuda_error",
    "chill_host_workspace_bytes", "chill_fwd_bwd_host", "chill_host_chunk_schedule",
)


class MaskDesc(C.Structure):
    _fields_ = [("id", C.c_int32), ("n_args", C.c_int32), ("i", C.c_int64 * MAX_MASK_ARGS),
                ("f", C.c_double * MAX_MASK_ARGS)]


class Shape(C.Structure):
    _fields_ = [("B", C.c_int32), ("H", C.c_int32), ("H_kv", C.c_int32), ("Lq", C.c_int32), ("Lk", C.c_int32),
                ("D", C.c_int32), ("dtype", C.c_int32), ("q_offset", C.c_int32), ("k_offset", C.c_int32),
                ("seq_len", C.c_int32), ("sm_scale", C.c_float), ("flags", C.c_uint32), ("lens", C.c_void_p),
                ("mask", MaskDesc)]


_S4 = C.c_int64 * 4
_S3 = C.c_int64 * 3


class FwdArgs(C.Structure):
    _fields_ = [("s", Shape), ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p),
                ("lse", C.c_void_p), ("q_strides", _S4), ("k_strides", _S4), ("v_strides", _S4), ("o_strides", _S4),
                ("lse_strides", _S3)]


class BwdArgs(C.Structure):
    _fields_ = [("s", Shape), ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p),
                ("d_o", C.c_void_p), ("lse", C.c_void_p), ("delta", C.c_void_p), ("dq", C.c_void_p),
                ("dk", C.c_void_p), ("dv", C.c_void_p), ("q_strides", _S4), ("k_strides", _S4), ("v_strides", _S4),
                ("o_strides", _S4), ("do_strides", _S4), ("dq_strides", _S4), ("dk_strides", _S4),
                ("dv_strides", _S4), ("lse_strides", _S3), ("dq_accum", C.c_void_p), ("d_lse", C.c_void_p),
                ("dlse_strides", _S3), ("dk_part", C.c_void_p), ("dv_part", C.c_void_p), ("part_strides", _S3),
                ("part_head", C.c_int32), ("part_tail", C.c_int32)]


class HostArgs(C.Structure):
    _fields_ = [("s", Shape), ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("d_o", C.c_void_p),
                ("o", C.c_void_p), ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("chunk_groups", C.c_int32),
                ("reserved", C.c_int32)]


class ChillLibraryError(RuntimeError):
    pass


_libs: dict[str, C.CDLL] = {}
_lock = threading.Lock()


def load_library(path: str | None = None) -> C.CDLL:
    """dlopen the kernel library (cached per path) and declare its prototypes."""
    path = os.path.abspath(path or os.environ.get("CHILL_B200_LIB", DEFAULT_LIB))
    with _lock:
        lib = _libs.get(path)
        if lib is not None:
            return lib
        if not os.path.exists(path):
            raise ChillLibraryError(
                f"{path} not found: build the CUDA library first (python chill-attention_b200/build.py). "
                "chill_attention has no other backend."
            )
        lib = C.CDLL(path)
        lib.chill_fwd.argtypes = [C.POINTER(FwdArgs), C.c_void_p]
        lib.chill_bwd_delta.argtypes = [C.POINTER(BwdArgs), C.c_void_p]
        lib.chill_bwd.argtypes = [C.POINTER(BwdArgs), C.c_void_p]
        lib.chill_bwd_noalloc.argtypes = [C.POINTER(BwdArgs), C.c_void_p]
        lib.chill_bwd_scratch_bytes.argtypes = [C.POINTER(Shape)]
        lib.chill_bwd_scratch_bytes.restype = C.c_size_t
        lib.chill_bwd_dq_accum_bytes.argtypes = [C.POINTER(Shape)]
        lib.chill_bwd_dq_accum_bytes.restype = C.c_size_t
        lib.chill_fwd_uses_tensor_cores.argtypes = [C.POINTER(FwdArgs)]
        lib.chill_bwd_uses_tensor_cores.argtypes = [C.POINTER(BwdArgs)]
        lib.chill_mask_tabulate.argtypes = [C.POINTER(MaskDesc), C.c_int32, C.c_int32] + [C.c_void_p] * 6
        lib.chill_mask_tabulate_blocks.argtypes = [C.POINTER(MaskDesc), C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]
        lib.chill_selftest_bounded_wait.argtypes = [C.c_int32, C.c_void_p]
        lib.chill_mask_traits.argtypes = [C.c_int32]
        lib.chill_status_string.argtypes = [C.c_int]
        lib.chill_status_string.restype = C.c_char_p
        lib.chill_last_cuda_error.restype = C.c_char_p
        lib.chill_launch_count.restype = C.c_ulonglong
        lib.chill_host_workspace_bytes.argtypes = [C.POINTER(HostArgs)]
        lib.chill_host_workspace_bytes.restype = C.c_size_t
        lib.chill_fwd_bwd_host.argtypes = [C.POINTER(HostArgs), C.c_void_p]
        lib.chill_fwd_bwd_host.restype = C.c_int
        lib.chill_host_chunk_schedule.argtypes = [C.POINTER(HostArgs), C.POINTER(C.c_int32), C.c_int32]
        lib.chill_host_chunk_schedule.restype = C.c_int
        for name in ("chill_fwd", "chill_bwd_delta", "chill_bwd", "chill_bwd_noalloc", "chill_fwd_uses_tensor_cores",
                     "chill_bwd_uses_tensor_cores", "chill_mask_tabulate", "chill_mask_tabulate_blocks", "chill_mask_traits",
                     "chill_selftest_bounded_wait",
                     "chill_read_device_status", "chill_abi_version"):
            getattr(lib, name).restype = C.c_int
        if lib.chill_abi_version() != ABI_VERSION:
            raise ChillLibraryError(f"{path}: ABI version {lib.chill_abi_version()} != {ABI_VERSION}")
        _libs[path] = lib
        return lib


def check(lib, status: int, what: str):
    if status != 0:
        msg = lib.chill_status_string(status).decode()
        extra = lib.chill_last_cuda_error().decode() if status == -3 else ""
        raise ChillLibraryError(f"{what} failed: {msg} (status {status}) {extra}".strip())


def mask_desc(mask_id: int, args) -> MaskDesc:
    d = MaskDesc()
    d.id = mask_id
    args = tuple(args)
    if len(args) > MAX_MASK_ARGS:
        raise ValueError(f"a mask takes at most {MAX_MASK_ARGS} constants")
    d.n_args = len(args)
    for n, a in enumerate(args):
        d.i[n] = int(a)
        d.f[n] = float(a)
    return d


def make_shape(q, k, mask_id, mask_args, lens, sm_scale, q_offset=0, k_offset=0, seq_len=None, flags=0) -> Shape:
    s = Shape()
    s.B, s.H, s.Lq, s.D = q.shape
    s.H_kv, s.Lk = k.shape[1], k.shape[2]
    s.dtype = _DTYPES[q.dtype]
    s.q_offset, s.k_offset = q_offset, k_offset
    s.seq_len = s.Lq if seq_len is None else seq_len
    s.sm_scale = sm_scale
    s.flags = flags
    s.lens = lens.data_ptr() if lens is not None else None
    s.mask = mask_desc(mask_id, mask_args)
    return s


def _strides(t, n):
    return (C.c_int64 * n)(*t.stride())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def forward(lib, q, k, v, o, lse, shape: Shape):
    a = FwdArgs()
    a.s = shape
    a.q, a.k, a.v, a.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
    a.lse = lse.data_ptr() if lse is not None else None
    a.q_strides, a.k_strides, a.v_strides, a.o_strides = (_strides(t, 4) for t in (q, k, v, o))
    if lse is not None:
        a.lse_strides = _strides(lse, 3)
    check(lib, lib.chill_fwd(C.byref(a), _stream()), "chill_fwd")


def backward_args(q, k, v, o, do, lse, delta, dq, dk, dv, shape: Shape, dq_accum=None, d_lse=None, part=None) -> BwdArgs:
    a = BwdArgs()
    a.s = shape
    a.q, a.k, a.v, a.o, a.d_o = (t.data_ptr() for t in (q, k, v, o, do))
    a.lse, a.delta = lse.data_ptr(), (delta.data_ptr() if delta is not None else None)
    a.dq, a.dk, a.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    (a.q_strides, a.k_strides, a.v_strides, a.o_strides, a.do_strides, a.dq_strides, a.dk_strides,
     a.dv_strides) = (_strides(t, 4) for t in (q, k, v, o, do, dq, dk, dv))
    a.lse_strides = _strides(lse, 3)
    a.dq_accum = dq_accum.data_ptr() if dq_accum is not None else None
    if d_lse is not None:  # gradient of the loss w.r.t. the returned LSE (log2 units), fp32 [B, H, L]
        a.d_lse = d_lse.data_ptr()
        a.dlse_strides = _strides(d_lse, 3)
    if part is not None:
        # (dk_part, dv_part, head, tail): fp32 [B, H_kv, head + tail, D] views (any batch / head / row strides,
        # contiguous channels) that receive the un-rounded dK / dV of the first `head` and last `tail` key rows
        dk_part, dv_part, head, tail = part
        if dk_part.dtype != torch.float32 or dk_part.stride() != dv_part.stride() or dk_part.stride(3) != 1:
            raise ValueError("partial dK / dV outputs must be fp32 with equal strides and contiguous channels")
        a.dk_part, a.dv_part = dk_part.data_ptr(), dv_part.data_ptr()
        a.part_strides = (C.c_int64 * 3)(*dk_part.stride()[:3])
        a.part_head, a.part_tail = head, tail
    return a


_deterministic = os.environ.get("CHILL_ATTENTION_DETERMINISTIC", "0") not in ("", "0")


def set_deterministic(flag: bool) -> None:
    """True: the backward never sums dQ with floating-point reductions (two-kernel backward, bitwise
    reproducible); False (default): the single-kernel backward is used where it applies.  Also on when
    ``torch.use_deterministic_algorithms(True)`` is set or CHILL_ATTENTION_DETERMINISTIC=1."""
    global _deterministic
    _deterministic = bool(flag)


def is_deterministic() -> bool:
    return _deterministic or torch.are_deterministic_algorithms_enabled()


def dq_accum_for(lib, a: BwdArgs, device):
    """The fp32 scratch tensor that switches chill_bwd to its single-kernel form, or None if the call
    would not use it (generic kernels, deterministic mode)."""
    if is_deterministic() or (a.s.flags & (FLAG_BWD_ONLY_DKDV | FLAG_BWD_ONLY_DQ)):
        return None
    nbytes = lib.chill_bwd_dq_accum_bytes(C.byref(a.s))
    if nbytes == 0 or lib.chill_bwd_uses_tensor_cores(C.byref(a)) != 1:
        return None
    return torch.empty(nbytes // 4, dtype=torch.float32, device=device)


def tma_compatible(t) -> bool:
    """What the tensor-core kernels need of a [B, H, L, D] operand: contiguous channels, no broadcast
    (zero-stride) dimension, 16-byte aligned base and batch / head / row strides."""
    es = t.element_size()
    if t.stride(-1) != 1 or t.data_ptr() % 16:
        return False
    return all(st > 0 and (st * es) % 16 == 0 for st, n in zip(t.stride()[:-1], t.shape[:-1]) if n > 1)


def backward(lib, q, k, v, o, do, lse, delta, dq, dk, dv, shape: Shape, dq_accum=None, deterministic=False,
             d_lse=None, part=None):
    """chill_bwd_delta + chill_bwd.  Without `dq_accum` the fp32 dQ scratch of the single-kernel backward is
    allocated here when the call can use it; `deterministic=True` forces the two-kernel form."""
    a = backward_args(q, k, v, o, do, lse, delta, dq, dk, dv, shape, dq_accum, d_lse, part)
    if dq_accum is None and not deterministic:
        dq_accum = dq_accum_for(lib, a, q.device)  # stays referenced until the launches are enqueued
        a.dq_accum = dq_accum.data_ptr() if dq_accum is not None else None
    st = _stream()
    check(lib, lib.chill_bwd_delta(C.byref(a), st), "chill_bwd_delta")
    check(lib, lib.chill_bwd(C.byref(a), st), "chill_bwd")


NOALLOC_MAX_ROWS = 1 << 22


def backward_noalloc(lib, q, k, v, o, do, lse, dq, dk, dv, shape: Shape):
    """Backward through ``chill_bwd_noalloc``: the delta scratch lives inside the library
    (at most NOALLOC_MAX_ROWS = B*H*Lq rows); calls sharing a device must not overlap."""
    a = backward_args(q, k, v, o, do, lse, None, dq, dk, dv, shape)
    check(lib, lib.chill_bwd_noalloc(C.byref(a), _stream()), "chill_bwd_noalloc")
