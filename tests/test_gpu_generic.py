"""Generic CUDA kernels (fp32 / odd head dims / strided inputs) against the oracle and the
reference's own outputs.  Runs through the public API, i.e. custom op -> ctypes -> C ABI."""
import ctypes

import pytest
import torch

from helpers import (all_masks, check_forward, check_grads, ensure_built, load_golden, make_inputs, oracle_all)

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _lib():
    ensure_built()
    from chill_attention import _cabi

    lib = _cabi.load_library()
    yield lib
    assert lib.chill_read_device_status() == 0


def run(mask, q, k, v, do, lens=None, sm_scale=None):
    from chill_attention import chill_attention

    dev = "cuda"
    qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    lens_d = lens.to(dev) if lens is not None else None
    o, lse = chill_attention(qd, kd, vd, mask=mask, lens=lens_d, sm_scale=sm_scale, return_lse=True)
    o.backward(do.to(dev))
    return o, lse, (qd.grad, kd.grad, vd.grad)


@pytest.mark.parametrize("name", ["c1_causal", "full", "causal_small", "sliding", "chunkwise", "prefixlm", "sliding_rows"])
def test_golden_reference_outputs(name):
    """Bit-for-bit the same inputs the reference ran on; its outputs are the expectation."""
    import chill_attention as ca

    mname, margs, lens, t = load_golden(name)
    mask = getattr(ca, mname)(*margs)
    o, lse, grads = run(mask, t["q"], t["k"], t["v"], t["do"], lens)
    B, H, L, D = t["q"].shape
    valid = torch.ones(B, 1, L, dtype=torch.bool) if lens is None else (torch.arange(L)[None, None] < lens[:, None, None])
    vm = valid[..., None]
    torch.testing.assert_close(o.detach().cpu() * vm, t["o"] * vm, atol=2e-6, rtol=1e-4)  # the reference's own fp32 bar
    fin = torch.isfinite(t["lse"]) & valid
    torch.testing.assert_close(lse.cpu()[fin.expand_as(lse)], t["lse"][fin.expand_as(lse)], atol=1e-5, rtol=1e-5)
    inf_rows = torch.isinf(t["lse"]) & valid
    assert torch.equal(torch.isinf(lse.cpu()) & valid, inf_rows)
    for g, key in zip(grads, ("dq", "dk", "dv")):
        torch.testing.assert_close(g.cpu(), t[key], atol=5e-5, rtol=1e-3)  # test/test_chill_attention.py:299-321


@pytest.mark.parametrize("mask", all_masks(), ids=str)
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16], ids=str)
@pytest.mark.parametrize("D", [16, 32, 256])
def test_odd_head_dims(mask, dtype, D):
    q, k, v, do = make_inputs(2, 4, 2, 70, D, dtype)
    lens = torch.tensor([70, 0], dtype=torch.int32)
    o_ref, lse_ref, *g_ref = oracle_all(mask, q, k, v, do, lens)
    o, lse, grads = run(mask, q, k, v, do, lens)
    check_forward(o, lse, o_ref, lse_ref, lens, dtype)
    check_grads(grads, g_ref, dtype, lens)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=str)
@pytest.mark.parametrize("D", [16, 32])
def test_small_head_dims_take_the_tensor_cores(dtype, D):
    """16-bit head dim 16 / 32 is zero-padded to 64 channels by chill_attention(): the tensor-core backward serves it,
    the outputs have the caller's head dim and are contiguous, and a default sm_scale still means head_dim ** -0.5."""
    import chill_attention as ca
    from chill_attention.chill import backward_path_counts

    mask = ca.SlidingWindowChillMask(40, 3)
    q, k, v, do = make_inputs(2, 4, 2, 300, D, dtype)
    o_ref, lse_ref, *g_ref = oracle_all(mask, q, k, v, do)
    before = backward_path_counts()
    o, lse, grads = run(mask, q, k, v, do)
    after = backward_path_counts()
    assert after["tensor_core"] == before["tensor_core"] + 1 and after["generic"] == before["generic"]
    assert o.shape == q.shape and o.is_contiguous() and all(g.shape == q.shape or g.shape == k.shape for g in grads)
    check_forward(o, lse, o_ref, lse_ref, None, dtype)
    check_grads(grads, g_ref, dtype)


@pytest.mark.parametrize("D", [16, 32])
def test_small_head_dims_through_the_c_abi(D, _lib):
    """A C-ABI caller that hands over 16-bit head dim 16 / 32 as it is gets the generic kernels: same results."""
    import chill_attention as ca
    from chill_attention import _cabi

    mask = ca.ChunkwiseChillMask(16, 2)
    dtype = torch.bfloat16
    q, k, v, do = make_inputs(1, 4, 2, 150, D, dtype)
    o_ref, lse_ref, *g_ref = oracle_all(mask, q, k, v, do)
    qd, kd, vd, dod = (t.cuda() for t in (q, k, v, do))
    o = torch.empty_like(qd)
    lse = torch.empty(qd.shape[:3], dtype=torch.float32, device="cuda")
    shape = _cabi.make_shape(qd, kd, _cabi.BUILTIN_FUNCTOR_IDS[mask.cuda_functor], mask.constargs, None, D ** -0.5)
    _cabi.forward(_lib, qd, kd, vd, o, lse, shape)
    delta = torch.empty_like(lse)
    dq, dk, dv = torch.empty_like(qd), torch.empty_like(kd), torch.empty_like(vd)
    a = _cabi.backward_args(qd, kd, vd, o, dod, lse, delta, dq, dk, dv, shape)
    assert _lib.chill_bwd_uses_tensor_cores(ctypes.byref(a)) == 0
    _cabi.backward(_lib, qd, kd, vd, o, dod, lse, delta, dq, dk, dv, shape)
    torch.cuda.synchronize()
    check_forward(o, lse, o_ref, lse_ref, None, dtype)
    check_grads((dq, dk, dv), g_ref, dtype)


@pytest.mark.parametrize("mask", all_masks(), ids=str)
@pytest.mark.parametrize("T", [1, 10, 16, 129])
@pytest.mark.parametrize("heads", [(1, 1), (6, 1), (6, 3)])
def test_fp32_shapes_of_the_reference_suite(mask, T, heads):
    H, Hkv = heads
    q, k, v, do = make_inputs(3, H, Hkv, T, 64, torch.float32)
    lens = torch.tensor([T, max(T // 2, 1), T + 1], dtype=torch.int32)  # T + 1 is legal and clamped
    o_ref, lse_ref, *g_ref = oracle_all(mask, q, k, v, do, lens)
    o, lse, grads = run(mask, q, k, v, do, lens)
    check_forward(o, lse, o_ref, lse_ref, lens, torch.float32)
    check_grads(grads, g_ref, torch.float32, lens)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=str)
def test_noncontiguous_inputs(dtype):
    import chill_attention as ca

    mask = ca.SlidingWindowChillMask(10, 4)
    q, k, v, do = make_inputs(2, 4, 4, 50, 128, dtype)
    o_ref, lse_ref, *g_ref = oracle_all(mask, q, k, v, do)

    def strided(t):  # channel stride 2, like torch.testing.make_tensor(noncontiguous=True)
        buf = torch.zeros(*t.shape[:-1], t.shape[-1] * 2, dtype=t.dtype)
        buf[..., ::2] = t
        return buf.cuda()[..., ::2]

    from chill_attention import chill_attention

    from chill_attention import chill as chill_mod

    qd, kd, vd = (strided(t).requires_grad_(True) for t in (q, k, v))
    assert qd.stride(-1) == 2
    before = chill_mod.backward_path_counts()
    o, lse = chill_attention(qd, kd, vd, mask=mask, return_lse=True)
    o.backward(do.cuda())
    assert o.is_contiguous()
    check_forward(o, lse, o_ref, lse_ref, None, dtype)
    check_grads((qd.grad, kd.grad, vd.grad), g_ref, dtype)
    # 16-bit operands with a head dimension the tensor-core kernels serve are packed once and stay on that path;
    # fp32 is read in place through its strides by the generic kernels
    after = chill_mod.backward_path_counts()
    which = "generic" if dtype == torch.float32 else "tensor_core"
    assert after[which] == before[which] + 1


def test_sm_scale_and_no_lse():
    import chill_attention as ca
    from chill_attention import chill_attention

    mask = ca.CausalChillMask()
    q, k, v, do = make_inputs(1, 2, 2, 40, 32, torch.float32)
    o_ref, *_ = oracle_all(mask, q, k, v, do, None, 0.3)
    o = chill_attention(q.cuda(), k.cuda(), v.cuda(), mask=mask, sm_scale=0.3)
    assert isinstance(o, torch.Tensor)
    assert (o.cpu().double() - o_ref).abs().max() <= 5e-6


@pytest.mark.parametrize("mask", all_masks(), ids=str)
def test_device_functors_equal_host_functions(mask, _lib):
    """Integer parity of the CUDA functors with the Python mask functions (bit-exact)."""
    from chill_attention import _cabi

    n, tile = 200, 32
    dense = torch.empty(n * n, dtype=torch.uint8, device="cuda")
    k_lims = torch.empty(n, 2, dtype=torch.int32, device="cuda")
    q_lims = torch.empty(n, 2, dtype=torch.int32, device="cuda")
    nt = (n + tile - 1) // tile
    k_full = torch.empty(nt, 2, dtype=torch.int32, device="cuda")
    q_full = torch.empty(nt, 2, dtype=torch.int32, device="cuda")
    desc = _cabi.mask_desc(_cabi.BUILTIN_FUNCTOR_IDS[mask.cuda_functor], mask.constargs)
    st = _lib.chill_mask_tabulate(ctypes.byref(desc), n, tile, dense.data_ptr(), k_lims.data_ptr(), q_lims.data_ptr(),
                                  k_full.data_ptr(), q_full.data_ptr(), None)
    assert st == 0
    torch.cuda.synchronize()
    cls = type(mask)
    assert torch.equal(dense.cpu().reshape(n, n).bool(), mask.make_mask(n, device="cpu"))
    pos = torch.arange(n)
    for table, fn in ((k_lims, cls.k_range_for_q), (q_lims, cls.q_range_for_k)):
        lo, hi = fn(pos, n, mask.constargs)
        exp = torch.stack([torch.as_tensor(lo).expand(n), torch.as_tensor(hi).expand(n)], 1).int()
        assert torch.equal(table.cpu(), exp)
    # the built-in functors declare kIntervalRows: every row and every column of the mask is exactly its range
    d, kl, ql = dense.cpu().reshape(n, n).bool(), k_lims.cpu().long(), q_lims.cpu().long()
    assert torch.equal(d, (pos[None, :] >= kl[:, :1]) & (pos[None, :] <= kl[:, 1:]))
    assert torch.equal(d, (pos[:, None] >= ql[:, 0][None, :]) & (pos[:, None] <= ql[:, 1][None, :]))
    assert torch.equal(k_full.cpu(), mask._calc_full_ranges(n, tile, cls.k_full_range_for_q))
    assert torch.equal(q_full.cpu(), mask._calc_full_ranges(n, tile, cls.q_full_range_for_k))
