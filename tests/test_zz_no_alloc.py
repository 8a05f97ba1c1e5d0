"""chill_bwd_noalloc: the backward for callers that cannot allocate device memory.

Some users of the C ABI run where cudaMalloc is not an option - inside a host callback or a
plugin hook while the framework's allocator is locked, in a serving loop whose memory plan is
frozen, or as an embedded component that was handed all its buffers up front.  For them the
library keeps the `delta` scratch of the backward pass in a fixed device array of its own
(4 Mi rows = 16 MiB per GPU).  This test drives that entry point through ctypes, twice in a row
with different problems (the array keeps the first call's contents), and compares dQ/dK/dV with
the regular chill_bwd_delta + chill_bwd path that takes a caller-provided scratch buffer.

The file sorts last on purpose, so a run that stops at the first failure has already run
everything else.
"""
import ctypes

import pytest
import torch

from helpers import G_RTOL, ensure_built, make_inputs

pytestmark = pytest.mark.gpu


def _problem(lib, mask, B, H, Hkv, L, D, dtype, seed, lens=None):
    from chill_attention import _cabi

    q, k, v, do = (t.cuda() for t in make_inputs(B, H, Hkv, L, D, dtype, seed=seed))
    lens_d = lens.cuda() if lens is not None else None
    functor = _cabi.BUILTIN_FUNCTOR_IDS[mask.cuda_functor]
    shape = _cabi.make_shape(q, k, functor, mask.constargs, lens_d, D ** -0.5)
    o = torch.empty_like(q)
    lse = torch.empty(B, H, L, dtype=torch.float32, device="cuda")
    _cabi.forward(lib, q, k, v, o, lse, shape)
    return q, k, v, do, o, lse, shape, lens_d


def _both_paths(lib, prob):
    from chill_attention import _cabi

    q, k, v, do, o, lse, shape, _ = prob
    ref = [torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)]
    delta = torch.empty(q.shape[:3], dtype=torch.float32, device="cuda")
    _cabi.backward(lib, q, k, v, o, do, lse, delta, *ref, shape)
    out = [torch.full_like(q, float("nan")), torch.full_like(k, float("nan")), torch.full_like(v, float("nan"))]
    _cabi.backward_noalloc(lib, q, k, v, o, do, lse, *out, shape)
    torch.cuda.synchronize()
    return out, ref


def _compare(out, ref, dtype):
    for name, a, b in zip(("dq", "dk", "dv"), out, ref):
        a, b = a.double(), b.double()
        assert torch.isfinite(a).all(), name
        rel = ((a - b).norm() / b.norm().clamp(min=1e-30)).item()
        assert rel <= G_RTOL[dtype], f"{name}: {rel}"


def test_noalloc_matches_regular_backward_twice_in_a_row():
    import chill_attention as ca
    from chill_attention import _cabi

    ensure_built()
    lib = _cabi.load_library()
    # call 1: tensor-core kernels, bf16, causal
    p1 = _problem(lib, ca.CausalChillMask(), 2, 4, 2, 700, 128, torch.bfloat16, seed=5)
    out1, ref1 = _both_paths(lib, p1)
    _compare(out1, ref1, torch.bfloat16)
    # call 2 right after, other shape / dtype / mask / lens: generic kernels, scratch holds call 1's rows
    lens = torch.tensor([300, 77, 1], dtype=torch.int32)
    p2 = _problem(lib, ca.SlidingWindowChillMask(40, 3), 3, 2, 2, 300, 32, torch.float32, seed=6, lens=lens)
    out2, ref2 = _both_paths(lib, p2)
    _compare(out2, ref2, torch.float32)
    # and the first problem again: identical answer to the first time (nothing stale leaks in)
    out3, _ = _both_paths(lib, p1)
    for a, b in zip(out3, out1):
        assert torch.equal(a, b)
    assert lib.chill_read_device_status() == 0


def test_noalloc_rejects_oversize_and_bad_arguments():
    import chill_attention as ca
    from chill_attention import _cabi

    ensure_built()
    lib = _cabi.load_library()
    assert lib.chill_bwd_noalloc(None, None) == -1
    # B*H*Lq one tile over the limit: refused before anything is launched (buffers are never touched)
    a = _cabi.BwdArgs()
    s = a.s
    s.B, s.H, s.H_kv, s.Lq, s.Lk, s.D, s.seq_len = 1, 33, 33, 131072, 131072, 64, 131072
    s.dtype, s.sm_scale = _cabi.CHILL_BF16, 0.125
    s.mask = _cabi.mask_desc(_cabi.MASK_CAUSAL, ())
    for f in ("q", "k", "v", "o", "d_o", "lse", "dq", "dk", "dv"):
        setattr(a, f, 256)  # non-null placeholders
    assert 33 * 131072 > _cabi.NOALLOC_MAX_ROWS
    assert lib.chill_bwd_noalloc(ctypes.byref(a), None) == -4
    assert b"CHILL_NOALLOC_MAX_ROWS" in lib.chill_last_cuda_error()
    s.H = s.H_kv = 32  # exactly at the limit passes the size check (and would launch), so stop here
    assert 32 * 131072 == _cabi.NOALLOC_MAX_ROWS
