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

from helpers import G_RTOL, check_grads, ensure_built, make_inputs, oracle_all

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
    # call 4: head dim 256 (the three-launch tensor-core backward; bitwise reproducible, so equal to the regular path)
    p4 = _problem(lib, ca.PrefixLMChillMask(100), 1, 4, 2, 520, 256, torch.float16, seed=7)
    out4, ref4 = _both_paths(lib, p4)
    for a, b in zip(out4, ref4):
        assert torch.equal(a, b)
    # not only equal to the regular path: right, against the fp64 dense-mask oracle
    for prob, out, mask, dtype, ln in ((p1, out1, ca.CausalChillMask(), torch.bfloat16, None),
                                       (p2, out2, ca.SlidingWindowChillMask(40, 3), torch.float32, lens),
                                       (p4, out4, ca.PrefixLMChillMask(100), torch.float16, None)):
        q, k, v, do = (t.cpu() for t in prob[:4])
        check_grads(out, oracle_all(mask, q, k, v, do, ln)[2:], dtype, ln)


def test_noalloc_allocates_nothing_and_honours_flags_and_dlse():
    """After the one-time address look-up of the first call on the device, a call must leave both the driver's
    free-memory figure and torch's allocator untouched; CHILL_FLAG_REQUIRE_TC and the optional d_lse input behave
    as in chill_bwd."""
    import chill_attention as ca
    from chill_attention import _cabi

    ensure_built()
    lib = _cabi.load_library()
    mask = ca.CausalChillMask()
    q, k, v, do, o, lse, shape, _ = _problem(lib, mask, 1, 4, 4, 512, 128, torch.bfloat16, seed=8)
    out = [torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)]
    _cabi.backward_noalloc(lib, q, k, v, o, do, lse, *out, shape)  # first call: resolves the array's address
    torch.cuda.synchronize()
    a = _cabi.backward_args(q, k, v, o, do, lse, None, *out, shape)
    free0, alloc0, reserved0 = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    for _ in range(3):
        _cabi.check(lib, lib.chill_bwd_noalloc(ctypes.byref(a), _cabi._stream()), "chill_bwd_noalloc")
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0
    assert torch.cuda.memory_allocated() == alloc0 and torch.cuda.memory_reserved() == reserved0
    # REQUIRE_TC: served by the tensor-core kernels here, refused for a shape only the generic kernels take
    shape_tc = _cabi.make_shape(q, k, _cabi.BUILTIN_FUNCTOR_IDS[mask.cuda_functor], (), None, 128 ** -0.5, flags=_cabi.FLAG_REQUIRE_TC)
    _cabi.backward_noalloc(lib, q, k, v, o, do, lse, *out, shape_tc)
    q32 = q.float()
    shape32 = _cabi.make_shape(q32, q32, _cabi.BUILTIN_FUNCTOR_IDS[mask.cuda_functor], (), None, 128 ** -0.5, flags=_cabi.FLAG_REQUIRE_TC)
    a32 = _cabi.backward_args(q32, q32, q32, q32, q32, lse, None, q32.clone(), q32.clone(), q32.clone(), shape32)
    assert lib.chill_bwd_noalloc(ctypes.byref(a32), _cabi._stream()) == -2
    # d_lse is folded into delta exactly as by chill_bwd_delta
    d_lse = torch.randn(lse.shape, device="cuda", dtype=torch.float32)
    ref = [torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)]
    delta = torch.empty_like(lse)
    _cabi.backward(lib, q, k, v, o, do, lse, delta, *ref, shape, deterministic=True, d_lse=d_lse)
    ad = _cabi.backward_args(q, k, v, o, do, lse, None, *out, shape, d_lse=d_lse)
    _cabi.check(lib, lib.chill_bwd_noalloc(ctypes.byref(ad), _cabi._stream()), "chill_bwd_noalloc")
    torch.cuda.synchronize()
    for x, y in zip(out, ref):
        assert torch.equal(x, y)  # both ran the two-kernel backward on the same delta
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
