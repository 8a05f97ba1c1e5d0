"""The two forms of the tensor-core backward against each other and against the fp64 oracle:
single kernel (five GEMMs per tile pair, dQ summed in an fp32 scratch buffer) and two kernels
(seven GEMMs, bitwise reproducible).  Called through the C ABI."""
import pytest
import torch

from helpers import G_RTOL, all_masks, big_masks, check_grads, ensure_built, make_inputs, oracle_all

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib():
    ensure_built()
    from chill_attention import _cabi

    lib = _cabi.load_library()
    yield lib
    assert lib.chill_read_device_status() == 0, "a bounded wait gave up inside a kernel"


def _run_both(lib, mask, q, k, v, do, lens=None):
    import ctypes as C

    from chill_attention import _cabi

    qd, kd, vd, dod = (t.cuda() for t in (q, k, v, do))
    lens_d = lens.cuda() if lens is not None else None
    B, H, L, D = q.shape
    shape = _cabi.make_shape(qd, kd, _cabi.BUILTIN_FUNCTOR_IDS[mask.cuda_functor], mask.constargs, lens_d, D ** -0.5)
    o = torch.empty_like(qd)
    lse = torch.empty(B, H, L, dtype=torch.float32, device="cuda")
    _cabi.forward(lib, qd, kd, vd, o, lse, shape)
    delta = torch.empty(B, H, L, dtype=torch.float32, device="cuda")
    nbytes = lib.chill_bwd_dq_accum_bytes(C.byref(shape))
    assert nbytes >= B * H * L * D * 4
    accum = torch.full((nbytes // 4,), float("nan"), dtype=torch.float32, device="cuda")  # contents must not matter
    outs = []
    for scratch in (accum, None):
        g = [torch.full_like(qd, float("nan")), torch.full_like(kd, float("nan")), torch.full_like(vd, float("nan"))]
        a = _cabi.backward_args(qd, kd, vd, o, dod, lse, delta, *g, shape, scratch)
        assert lib.chill_bwd_uses_tensor_cores(C.byref(a)) == 1
        st = _cabi._stream()
        _cabi.check(lib, lib.chill_bwd_delta(C.byref(a), st), "chill_bwd_delta")
        _cabi.check(lib, lib.chill_bwd(C.byref(a), st), "chill_bwd")
        torch.cuda.synchronize()
        outs.append(g)
    return outs


def _check_pair(fused, split, dtype):
    assert torch.equal(fused[1], split[1]), "dK: both forms run the same GEMMs in the same order"
    assert torch.equal(fused[2], split[2]), "dV: both forms run the same GEMMs in the same order"
    a, b = fused[0].double(), split[0].double()
    assert torch.isfinite(a).all()
    rel = ((a - b).norm() / b.norm().clamp(min=1e-30)).item()
    assert rel <= G_RTOL[dtype], f"dQ single-kernel vs two-kernel: {rel}"


@pytest.mark.parametrize("mask", big_masks(), ids=str)
@pytest.mark.parametrize("dtype,D", [(torch.bfloat16, 128), (torch.float16, 64), (torch.float16, 128), (torch.bfloat16, 64)])
@pytest.mark.parametrize("L", [128, 700, 1024])
def test_single_kernel_matches_two_kernel_and_oracle(lib, mask, dtype, D, L):
    q, k, v, do = make_inputs(2, 2, 2, L, D, dtype, seed=31)
    fused, split = _run_both(lib, mask, q, k, v, do)
    _check_pair(fused, split, dtype)
    g_ref = oracle_all(mask, q, k, v, do)[2:]
    check_grads(fused, g_ref, dtype)
    check_grads(split, g_ref, dtype)


@pytest.mark.parametrize("mask", all_masks() + big_masks()[2:5], ids=str)
@pytest.mark.parametrize("heads", [(6, 1), (6, 3)])
def test_lens_and_gqa(lib, mask, heads):
    H, Hkv = heads
    L, dtype = 520, torch.bfloat16
    q, k, v, do = make_inputs(4, H, Hkv, L, 128, dtype, seed=32)
    lens = torch.tensor([L, 1, 130, L + 1], dtype=torch.int32)
    fused, split = _run_both(lib, mask, q, k, v, do, lens)
    _check_pair(fused, split, dtype)
    g_ref = oracle_all(mask, q, k, v, do, lens)[2:]
    check_grads(fused, g_ref, dtype, lens)


def test_deterministic_switch_gives_bitwise_repeatable_gradients(lib):
    import chill_attention as ca

    mask = ca.CausalChillMask()
    q, k, v, do = make_inputs(2, 4, 2, 900, 128, torch.bfloat16, seed=33)

    def grads():
        qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
        ca.chill_attention(qd, kd, vd, mask=mask).backward(do.cuda())
        return qd.grad, kd.grad, vd.grad

    from chill_attention import _cabi

    before = _cabi._deterministic  # the switch may have been set through CHILL_ATTENTION_DETERMINISTIC
    try:
        ca.set_deterministic(False)
        assert not ca.is_deterministic()
        loose = grads()
        ca.set_deterministic(True)
        a, b = grads(), grads()
    finally:
        ca.set_deterministic(before)
    for x, y in zip(a, b):
        assert torch.equal(x, y)
    for x, y in zip(loose, a):
        rel = ((x.double() - y.double()).norm() / y.double().norm()).item()
        assert rel <= G_RTOL[torch.bfloat16]


@pytest.mark.parametrize("q0,k0", [(512, 256), (500, 300)])
def test_shard_with_global_offsets_matches_the_full_problem(lib, q0, k0):
    """Queries [q0, L) against keys [k0, L) of a sliding-window problem, with q_offset / k_offset / seq_len:
    the rows a shard owns must equal the same rows of the unsharded result (what the sequence-sharded
    multi-GPU path relies on), for both forms of the backward."""
    import ctypes as C

    import chill_attention as ca
    from chill_attention import _cabi

    L, D, W, dtype = 1024, 128, 200, torch.bfloat16
    mask = ca.SlidingWindowChillMask(W, 0)
    assert q0 - k0 >= W  # the key shard holds the whole window of its first query
    q, k, v, do = make_inputs(1, 2, 2, L, D, dtype, seed=34)
    o_ref, _, dq_ref, dk_ref, dv_ref = oracle_all(mask, q, k, v, do)
    qs, dos = (t[:, :, q0:].contiguous().cuda() for t in (q, do))
    ks, vs = (t[:, :, k0:].contiguous().cuda() for t in (k, v))
    shape = _cabi.make_shape(qs, ks, _cabi.BUILTIN_FUNCTOR_IDS[mask.cuda_functor], mask.constargs, None, D ** -0.5,
                             q_offset=q0, k_offset=k0, seq_len=L)
    o = torch.empty_like(qs)
    lse = torch.empty(1, 2, L - q0, dtype=torch.float32, device="cuda")
    _cabi.forward(lib, qs, ks, vs, o, lse, shape)
    assert (o.cpu().double() - o_ref[:, :, q0:]).abs().max().item() <= 2e-2
    delta = torch.empty_like(lse)
    accum = torch.empty(lib.chill_bwd_dq_accum_bytes(C.byref(shape)) // 4, dtype=torch.float32, device="cuda")
    for scratch in (accum, None):
        g = [torch.full_like(qs, float("nan")), torch.full_like(ks, float("nan")), torch.full_like(vs, float("nan"))]
        a = _cabi.backward_args(qs, ks, vs, o, dos, lse, delta, *g, shape, scratch)
        assert lib.chill_bwd_uses_tensor_cores(C.byref(a)) == 1
        st = _cabi._stream()
        _cabi.check(lib, lib.chill_bwd_delta(C.byref(a), st), "chill_bwd_delta")
        _cabi.check(lib, lib.chill_bwd(C.byref(a), st), "chill_bwd")
        torch.cuda.synchronize()
        dq, dk, dv = (t.cpu().double() for t in g)
        assert torch.isfinite(dq).all() and torch.isfinite(dk).all() and torch.isfinite(dv).all()
        for name, got, ref in (("dq", dq, dq_ref[:, :, q0:]), ("dk", dk[:, :, q0 - k0:], dk_ref[:, :, q0:]),
                               ("dv", dv[:, :, q0 - k0:], dv_ref[:, :, q0:])):
            rel = ((got - ref).norm() / ref.norm()).item()
            assert rel <= G_RTOL[dtype], f"{name}: {rel}"


def test_misaligned_dq_scratch_is_rejected(lib):
    import ctypes as C

    import chill_attention as ca
    from chill_attention import _cabi

    mask = ca.CausalChillMask()
    q, k, v, do = (t.cuda() for t in make_inputs(1, 1, 1, 256, 64, torch.float16, seed=35))
    shape = _cabi.make_shape(q, k, _cabi.BUILTIN_FUNCTOR_IDS[mask.cuda_functor], mask.constargs, None, 0.125)
    o, lse = torch.empty_like(q), torch.empty(1, 1, 256, dtype=torch.float32, device="cuda")
    _cabi.forward(lib, q, k, v, o, lse, shape)
    delta = torch.empty_like(lse)
    accum = torch.empty(lib.chill_bwd_dq_accum_bytes(C.byref(shape)) // 4 + 4, dtype=torch.float32, device="cuda")
    g = [torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)]
    a = _cabi.backward_args(q, k, v, o, do, lse, delta, *g, shape, accum[1:])  # 4 bytes off a 16-byte boundary
    st = _cabi._stream()
    _cabi.check(lib, lib.chill_bwd_delta(C.byref(a), st), "chill_bwd_delta")
    assert lib.chill_bwd(C.byref(a), st) == -1
    torch.cuda.synchronize()
