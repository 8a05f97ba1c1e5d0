"""tcgen05 tensor-core kernels (fp16/bf16, head dim 64/128) against the fp64 dense-mask oracle."""
import ctypes

import pytest
import torch

from helpers import O_ATOL, all_masks, big_masks, check_forward, check_grads, ensure_built, make_inputs, oracle_all

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _lib():
    ensure_built()
    from chill_attention import _cabi

    lib = _cabi.load_library()
    yield lib
    assert lib.chill_read_device_status() == 0


@pytest.fixture(autouse=True)
def _status_clean(_lib):
    yield
    assert _lib.chill_read_device_status() == 0, "a bounded wait gave up inside a kernel"


def uses_tc(lib, q, k, v, mask):
    from chill_attention import _cabi

    a = _cabi.FwdArgs()
    a.s = _cabi.make_shape(q, k, _cabi.BUILTIN_FUNCTOR_IDS[mask.cuda_functor], mask.constargs, None, q.shape[-1] ** -0.5)
    o = torch.empty_like(q)
    a.q, a.k, a.v, a.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
    for name, t in (("q_strides", q), ("k_strides", k), ("v_strides", v), ("o_strides", o)):
        setattr(a, name, (ctypes.c_int64 * 4)(*t.stride()))
    return lib.chill_fwd_uses_tensor_cores(ctypes.byref(a))


def run(mask, q, k, v, do, lens=None, backward=True):
    from chill_attention import chill_attention

    qd, kd, vd = (t.cuda().requires_grad_(backward) for t in (q, k, v))
    lens_d = lens.cuda() if lens is not None else None
    o, lse = chill_attention(qd, kd, vd, mask=mask, lens=lens_d, return_lse=True)
    grads = None
    if backward:
        o.backward(do.cuda())
        grads = (qd.grad, kd.grad, vd.grad)
    return o, lse, grads


def test_dispatch_takes_the_tensor_core_path(_lib):
    import chill_attention as ca

    q = torch.zeros(1, 2, 256, 128, dtype=torch.bfloat16, device="cuda")
    assert uses_tc(_lib, q, q, q, ca.CausalChillMask()) == 1
    q32 = torch.zeros(1, 2, 256, 128, dtype=torch.float32, device="cuda")
    assert uses_tc(_lib, q32, q32, q32, ca.CausalChillMask()) == 0
    q16 = torch.zeros(1, 2, 256, 16, dtype=torch.bfloat16, device="cuda")
    assert uses_tc(_lib, q16, q16, q16, ca.CausalChillMask()) == 0
    q256 = torch.zeros(1, 2, 256, 256, dtype=torch.float16, device="cuda")
    assert uses_tc(_lib, q256, q256, q256, ca.CausalChillMask()) == 1  # one CTA per SM


@pytest.mark.parametrize("mask", big_masks(), ids=str)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=str)
@pytest.mark.parametrize("L", [128, 700])
def test_head_dim_256_on_the_tensor_cores(mask, dtype, L, _lib):
    """Head dim 256: the forward runs the tcgen05 kernel with S 128 + O 256 TMEM columns (one CTA per SM), the backward
    three launches of the score-and-accumulate kernel of bwd_wide.cuh (dV, dK, dQ).  GQA, per-row lengths with a row
    that ends inside a tile, a sequence that is not a multiple of the tile."""
    from chill_attention.chill import backward_path_counts

    q, k, v, do = make_inputs(2, 4, 2, L, 256, dtype, seed=79)
    lens = torch.tensor([L, max(1, L // 3)], dtype=torch.int32)
    assert uses_tc(_lib, q.cuda(), k.cuda(), v.cuda(), mask) == 1
    o_ref, lse_ref, *g_ref = oracle_all(mask, q, k, v, do, lens)
    before = backward_path_counts()
    o, lse, grads = run(mask, q, k, v, do, lens)
    after = backward_path_counts()
    assert after["tensor_core"] == before["tensor_core"] + 1 and after["generic"] == before["generic"]
    check_forward(o, lse, o_ref, lse_ref, lens, dtype)
    check_grads(grads, g_ref, dtype, lens)


def test_head_dim_256_backward_is_reproducible_and_packs_strided_inputs():
    """No atomics in the head-dim-256 backward: two runs agree bit for bit; operands TMA cannot describe (a
    transposed view) are packed once and still take the tensor-core kernels."""
    import chill_attention as ca
    from chill_attention.chill import backward_path_counts

    mask = ca.SlidingWindowChillMask(150, 20)
    q, k, v, do = make_inputs(1, 4, 4, 520, 256, torch.bfloat16, seed=80)
    o_ref, lse_ref, *g_ref = oracle_all(mask, q, k, v, do)
    a = run(mask, q, k, v, do)
    b = run(mask, q, k, v, do)
    for x, y in zip(a[2], b[2]):
        assert torch.equal(x, y)
    # [B, L, H, D] storage viewed as [B, H, L, D]: position-major, which TMA can describe; [B, H, D, L] cannot
    qd, kd, vd = (t.cuda().transpose(2, 3).contiguous().transpose(2, 3).requires_grad_(True) for t in (q, k, v))
    before = backward_path_counts()
    o = ca.chill_attention(qd, kd, vd, mask=mask)
    o.backward(do.cuda())
    after = backward_path_counts()
    assert after["tensor_core"] == before["tensor_core"] + 1
    check_grads((qd.grad, kd.grad, vd.grad), g_ref, torch.bfloat16)


@pytest.mark.parametrize("mask", big_masks(), ids=str)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=str)
@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("L", [128, 640, 1000])
def test_forward_backward(mask, dtype, D, L):
    q, k, v, do = make_inputs(2, 2, 2, L, D, dtype)
    o_ref, lse_ref, *g_ref = oracle_all(mask, q, k, v, do)
    o, lse, grads = run(mask, q, k, v, do)
    check_forward(o, lse, o_ref, lse_ref, None, dtype)
    check_grads(grads, g_ref, dtype)


@pytest.mark.parametrize("mask", all_masks() + big_masks()[2:5], ids=str)
@pytest.mark.parametrize("heads", [(6, 1), (6, 3), (4, 4)])
def test_lens_and_gqa(mask, heads):
    H, Hkv = heads
    L, dtype = 520, torch.bfloat16
    q, k, v, do = make_inputs(4, H, Hkv, L, 128, dtype)
    lens = torch.tensor([L, 1, 130, L + 1], dtype=torch.int32)
    o_ref, lse_ref, *g_ref = oracle_all(mask, q, k, v, do, lens)
    o, lse, grads = run(mask, q, k, v, do, lens)
    check_forward(o, lse, o_ref, lse_ref, lens, dtype)
    check_grads(grads, g_ref, dtype, lens)


@pytest.mark.parametrize("L", [1, 10, 16, 127, 129])
def test_tiny_sequences(L):
    import chill_attention as ca

    for mask in (ca.CausalChillMask(), ca.SlidingWindowChillMask(3, 1)):
        q, k, v, do = make_inputs(2, 2, 1, L, 64, torch.float16)
        o_ref, lse_ref, *g_ref = oracle_all(mask, q, k, v, do)
        o, lse, grads = run(mask, q, k, v, do)
        check_forward(o, lse, o_ref, lse_ref, None, torch.float16)
        check_grads(grads, g_ref, torch.float16)


def test_permuted_layout_blhd():
    """q/k/v stored [B, L, H, D] and viewed as [B, H, L, D]: still TMA-describable."""
    import chill_attention as ca
    from chill_attention import chill_attention

    mask = ca.CausalChillMask()
    q, k, v, do = make_inputs(2, 4, 4, 300, 128, torch.bfloat16)
    o_ref, lse_ref, *g_ref = oracle_all(mask, q, k, v, do)
    qd, kd, vd = (t.transpose(1, 2).contiguous().cuda().transpose(1, 2).requires_grad_(True) for t in (q, k, v))
    assert not qd.is_contiguous()
    o, lse = chill_attention(qd, kd, vd, mask=mask, return_lse=True)
    o.backward(do.cuda())
    check_forward(o, lse, o_ref, lse_ref, None, torch.bfloat16)
    check_grads((qd.grad, kd.grad, vd.grad), g_ref, torch.bfloat16)


def test_deterministic():
    import chill_attention as ca

    mask = ca.PrefixLMChillMask(100)
    q, k, v, do = make_inputs(1, 4, 4, 700, 128, torch.bfloat16)
    a = run(mask, q, k, v, do)
    b = run(mask, q, k, v, do)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


def test_large_magnitude_scores_rescale_path():
    """Scores whose running maximum keeps growing by more than the lazy-rescale threshold."""
    import chill_attention as ca

    mask = ca.FullChillMask()
    q, k, v, do = make_inputs(1, 1, 1, 1024, 128, torch.bfloat16)
    ramp = torch.linspace(0.2, 6.0, 1024).reshape(1, 1, 1024, 1)
    k = (k.float() * ramp).to(torch.bfloat16)  # later keys have larger norms -> the max moves tile after tile
    o_ref, lse_ref, *g_ref = oracle_all(mask, q, k, v, do)
    o, lse, grads = run(mask, q, k, v, do)
    check_forward(o, lse, o_ref, lse_ref, None, torch.bfloat16)
    check_grads(grads, g_ref, torch.bfloat16)


def test_torch_compile_traces_the_op():
    import chill_attention as ca
    from chill_attention import chill_attention

    mask = ca.CausalChillMask()
    q, k, v, do = make_inputs(1, 2, 2, 256, 64, torch.bfloat16)

    def f(q, k, v):
        return chill_attention(q, k, v, mask=mask) * 2.0

    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    eager = f(qd, kd, vd)
    compiled = torch.compile(f, fullgraph=True)(qd, kd, vd)
    assert torch.equal(eager, compiled)
    compiled.backward(do.cuda())
    assert qd.grad is not None and torch.isfinite(qd.grad).all()
    torch.library.opcheck(torch.ops.chill_attention.forwardCausalChillMask.default,
                          (qd.detach(), kd.detach(), vd.detach(), None, [], 0.125, True, False, "ieee", False),
                          test_utils=("test_schema", "test_faketensor"))


def test_host_buffer_pipeline_matches_device_path():
    import chill_attention as ca
    from chill_attention.host import attention_fwd_bwd_host

    mask = ca.CausalChillMask()
    q, k, v, do = make_inputs(5, 4, 2, 384, 128, torch.bfloat16)
    host = [t.pin_memory() for t in (q, k, v, do)]
    ca.set_deterministic(True)  # two-kernel backward: chunking must not change a single bit
    o_ref, lse_ref, *g_ref = oracle_all(mask, q, k, v, do)
    try:
        o, lse, grads = run(mask, q, k, v, do)
        for chunk, heads in ((1, None), (2, 4), (8, 4), (1, 2)):
            oh, dqh, dkh, dvh = attention_fwd_bwd_host(*host, mask, chunk_batches=chunk, chunk_heads=heads)
            assert torch.equal(oh, o.detach().cpu())
            for a, b in zip((dqh, dkh, dvh), grads):
                assert torch.equal(a, b.cpu())
        # and against the oracle directly, not only against the device-resident path
        assert (oh.double() - o_ref).abs().max() <= O_ATOL[torch.bfloat16]
        check_grads((dqh, dkh, dvh), g_ref, torch.bfloat16)
    finally:
        ca.set_deterministic(False)
    # default (single-kernel backward, dQ summed with fp32 reductions): equal up to the order of those sums
    oh, dqh, dkh, dvh = attention_fwd_bwd_host(*host, mask, chunk_heads=2)
    assert torch.equal(oh, o.detach().cpu())
    assert torch.equal(dkh, grads[1].cpu()) and torch.equal(dvh, grads[2].cpu())
    rel = ((dqh.double() - grads[0].cpu().double()).norm() / grads[0].cpu().double().norm()).item()
    assert rel <= 1e-2
    # many head groups per batch row, a chunk size that does not divide them: still bit for bit
    mask = ca.SlidingWindowChillMask(100, 0)
    for B in (1, 3):
        q, k, v, do = make_inputs(B, 16, 8, 256, 64, torch.float16, seed=5)
        host = [t.pin_memory() for t in (q, k, v, do)]
        ca.set_deterministic(True)
        try:
            o, lse, grads = run(mask, q, k, v, do)
            oh, dqh, dkh, dvh = attention_fwd_bwd_host(*host, mask, chunk_heads=6)
            assert torch.equal(oh, o.detach().cpu())
            for a, b in zip((dqh, dkh, dvh), grads):
                assert torch.equal(a, b.cpu())
        finally:
            ca.set_deterministic(False)


@pytest.mark.parametrize("dtype,D", [(torch.bfloat16, 128), (torch.float16, 64), (torch.float32, 32)], ids=str)
def test_gradient_through_the_returned_lse(dtype, D):
    """loss = <O, dO> + <LSE, dLSE>: the second term's gradient reaches dQ and dK (the reference drops it,
    chill.py:466-490).  Expected values: autograd through a dense fp64 restatement."""
    import math

    import chill_attention as ca
    from helpers import G_RTOL

    B, H, Hkv, L = 2, 4, 2, 300
    for mask in (ca.CausalChillMask(), ca.SlidingWindowChillMask(40, 10)):
        q, k, v, do = make_inputs(B, H, Hkv, L, D, dtype, seed=41)
        dlse = torch.randn(B, H, L, generator=torch.Generator().manual_seed(42))
        qr, kr, vr = (t.double().requires_grad_(True) for t in (q, k, v))
        ke, ve = (t.repeat_interleave(H // Hkv, dim=1) for t in (kr, vr))
        s = (qr @ ke.transpose(-1, -2)) * D ** -0.5
        s = s.masked_fill(~mask.make_mask(L, device="cpu"), float("-inf"))
        lse2 = torch.logsumexp(s, dim=-1) * math.log2(math.e)
        o_ref = torch.softmax(s, dim=-1) @ ve
        ((o_ref * do.double()).sum() + (lse2 * dlse.double()).sum()).backward()
        qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
        o, lse = ca.chill_attention(qd, kd, vd, mask=mask, return_lse=True)
        assert (lse.cpu().double() - lse2.detach()).abs().max().item() <= 2e-2
        ((o.float() * do.cuda().float()).sum() + (lse * dlse.cuda()).sum()).backward()
        for name, got, ref in (("dq", qd.grad, qr.grad), ("dk", kd.grad, kr.grad), ("dv", vd.grad, vr.grad)):
            rel = ((got.cpu().double() - ref).norm() / ref.norm()).item()
            assert rel <= 2 * G_RTOL[dtype], f"{mask} {name}: {rel}"
        # only the LSE is used: dO arrives as None
        qd2, kd2, vd2 = (t.cuda().requires_grad_(True) for t in (q, k, v))
        _, lse_only = ca.chill_attention(qd2, kd2, vd2, mask=mask, return_lse=True)
        (lse_only * dlse.cuda()).sum().backward()
        assert torch.isfinite(qd2.grad).all() and vd2.grad.abs().max().item() == 0.0


@pytest.mark.parametrize("mask", big_masks(), ids=str)
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("L", [128, 700])
def test_fp32_forward_in_tf32(mask, D, L, _lib):
    """precision="tf32": fp32 tensors through tcgen05.mma.kind::tf32.  Stated bars: O max-abs <= 5e-3 against the
    fp64 oracle (Q, K, V truncated to 10 mantissa bits by the tensor core, P rounded; measured 2e-3 .. 4e-3),
    LSE <= 3e-3 * max(1, |LSE|) (measured up to 1.7e-3), gradients 5e-3 relative; the backward stays IEEE fp32."""
    import ctypes as C

    from chill_attention import _cabi, chill_attention

    q, k, v, do = make_inputs(2, 4, 2, L, D, torch.float32, seed=51)
    o_ref, lse_ref, *g_ref = oracle_all(mask, q, k, v, do)
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    # the dispatch really takes the tensor-core kernel
    a = _cabi.FwdArgs()
    a.s = _cabi.make_shape(qd, kd, _cabi.BUILTIN_FUNCTOR_IDS[mask.cuda_functor], mask.constargs, None, D ** -0.5,
                           flags=_cabi.FLAG_ALLOW_TF32)
    o_tmp = torch.empty_like(qd)
    a.q, a.k, a.v, a.o = qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o_tmp.data_ptr()
    for name, t in (("q_strides", qd), ("k_strides", kd), ("v_strides", vd), ("o_strides", o_tmp)):
        setattr(a, name, (C.c_int64 * 4)(*t.stride()))
    assert _lib.chill_fwd_uses_tensor_cores(C.byref(a)) == 1
    o, lse = chill_attention(qd, kd, vd, mask=mask, return_lse=True, precision="tf32")
    err = (o.detach().cpu().double() - o_ref).abs().max().item()
    assert err <= 5e-3, f"O max-abs {err}"
    fin = torch.isfinite(lse_ref)
    assert torch.equal(torch.isfinite(lse.cpu()), fin)
    lerr = ((lse.cpu().double() - lse_ref)[fin].abs() / lse_ref[fin].abs().clamp(min=1.0)).max().item()
    assert lerr <= 3e-3, f"LSE {lerr}"
    o.backward(do.cuda())
    for name, got, ref in zip(("dq", "dk", "dv"), (qd.grad, kd.grad, vd.grad), g_ref):
        rel = ((got.cpu().double() - ref).norm() / ref.norm()).item()
        assert rel <= 5e-3, f"{name}: {rel}"  # O and LSE carry the TF32 error into the (IEEE) backward


def test_fp32_forward_in_tf32_with_lens_and_ragged_length(_lib):
    """The TF32 forward with per-row valid lengths, a sequence length that is not a multiple of the tile and
    more query heads than key heads: padded rows are exactly zero, the rest within the TF32 bars."""
    import chill_attention as ca
    from chill_attention import chill_attention

    L, D = 333, 64
    lens = torch.tensor([L, 0, 130, 200], dtype=torch.int32)
    for mask in (ca.CausalChillMask(), ca.SlidingWindowChillMask(50, 7)):
        q, k, v, do = make_inputs(4, 6, 2, L, D, torch.float32, seed=52)
        o_ref, lse_ref, *_ = oracle_all(mask, q, k, v, do, lens)
        o, lse = chill_attention(q.cuda(), k.cuda(), v.cuda(), mask=mask, lens=lens.cuda(), return_lse=True,
                                 precision="tf32")
        valid = torch.arange(L)[None, None, :] < lens.long()[:, None, None]
        oc = o.cpu().double()
        assert (oc[(~valid).expand(4, 6, L)] == 0).all(), "padded rows must be exactly zero"
        assert (oc - o_ref).abs().max().item() <= 5e-3
        fin = torch.isfinite(lse_ref)
        assert torch.equal(torch.isfinite(lse.cpu()), fin)
        assert ((lse.cpu().double() - lse_ref)[fin].abs() / lse_ref[fin].abs().clamp(min=1.0)).max().item() <= 3e-3


@pytest.mark.parametrize("mask", big_masks(), ids=str)
@pytest.mark.parametrize("L", [128, 700])
@pytest.mark.parametrize("D", [64, 128])
def test_fp32_backward_in_tf32(mask, L, D, _lib):
    """precision="tf32" also puts the backward of fp32 tensors on the tensor cores (csrc/bwd_tf32.cuh; head dim
    64 streams tiles of 128 positions, head dim 128 tiles of 32).  Stated bars against the fp64 oracle on N(0,1)
    inputs: gradients 5e-3 relative (Frobenius), padded rows exactly zero; GQA and per-row lengths included."""
    import chill_attention as ca
    from chill_attention import chill as chill_mod
    from chill_attention import chill_attention

    q, k, v, do = make_inputs(3, 4, 2, L, D, torch.float32, seed=53)
    lens = torch.tensor([L, max(1, L // 3), L + 1], dtype=torch.int32)
    g_ref = oracle_all(mask, q, k, v, do, lens)[2:]
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    before = chill_mod.backward_path_counts()
    o = chill_attention(qd, kd, vd, mask=mask, lens=lens.cuda(), precision="tf32")
    o.backward(do.cuda())
    after = chill_mod.backward_path_counts()
    assert after["tensor_core"] == before["tensor_core"] + 1 and after["generic"] == before["generic"]
    valid = torch.arange(L)[None, None, :] < lens.long()[:, None, None]
    for name, got, ref in zip(("dq", "dk", "dv"), (qd.grad, kd.grad, vd.grad), g_ref):
        got = got.cpu().double()
        assert torch.isfinite(got).all(), name
        rel = ((got - ref).norm() / ref.norm()).item()
        assert rel <= 5e-3, f"{name}: {rel}"
        pad = (~valid).expand(3, got.shape[1], L)
        assert (got[pad] == 0).all(), f"{name}: rows at or beyond lens[b] carry exactly zero gradient"
    # the same call twice: bitwise equal (no atomics in these kernels)
    q2, k2, v2 = (t.cuda().requires_grad_(True) for t in (q, k, v))
    chill_attention(q2, k2, v2, mask=mask, lens=lens.cuda(), precision="tf32").backward(do.cuda())
    for a, b in zip((qd.grad, kd.grad, vd.grad), (q2.grad, k2.grad, v2.grad)):
        assert torch.equal(a, b)


def test_fp32_without_the_tf32_flag_stays_ieee(_lib):
    """precision="ieee" (the default) never touches the TF32 kernels: fp32 bars of the generic kernels."""
    import chill_attention as ca
    from chill_attention import chill as chill_mod
    from chill_attention import chill_attention

    mask = ca.CausalChillMask()
    q, k, v, do = make_inputs(1, 2, 2, 200, 64, torch.float32, seed=54)
    g_ref = oracle_all(mask, q, k, v, do)[2:]
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    before = chill_mod.backward_path_counts()
    chill_attention(qd, kd, vd, mask=mask).backward(do.cuda())
    assert chill_mod.backward_path_counts()["generic"] == before["generic"] + 1
    check_grads((qd.grad, kd.grad, vd.grad), g_ref, torch.float32)


def test_a_bounded_wait_that_runs_out_ends_as_a_status_code(_lib):
    """The give-up path of the kernels' bounded mbarrier waits, exercised without faulting or hanging anything:
    a small kernel whose roles all wait (1 ms limit) on a barrier nobody arrives at must return, release its
    TMEM, leave its code in the device status word, and leave the context fully usable."""
    import time

    import chill_attention as ca
    from chill_attention import _cabi

    assert _lib.chill_read_device_status() == 0
    t0 = time.perf_counter()
    assert _lib.chill_selftest_bounded_wait(1000, None) == 0
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.0, "the waits are bounded by their limit, not by the 2 s default"
    assert _lib.chill_read_device_status() == _cabi.SELFTEST_STATUS
    assert _lib.chill_read_device_status() == 0, "reading the status clears it"
    # the context, the TMEM allocator and the kernels are unaffected
    q, k, v, do = make_inputs(1, 2, 2, 256, 128, torch.bfloat16, seed=77)
    o, lse, grads = run(ca.CausalChillMask(), q, k, v, do)
    o_ref, lse_ref, *g_ref = oracle_all(ca.CausalChillMask(), q, k, v, do)
    check_forward(o, lse, o_ref, lse_ref, None, torch.bfloat16)
    check_grads(grads, g_ref, torch.bfloat16)


def test_eager_call_path_equals_the_dispatcher_ops(_lib):
    """chill_attention() in plain eager mode takes the short host path (_eager.py); the dispatcher ops that
    torch.compile graphs use must give the same bits (same kernels, same arguments), forward and backward,
    with and without lens / return_lse, and with a gradient arriving at the LSE."""
    import chill_attention as ca
    from chill_attention import _cabi, _eager, chill

    mask = ca.SlidingWindowChillMask(100, 7)
    q, k, v, do = make_inputs(2, 4, 2, 333, 128, torch.bfloat16, seed=78)
    lens = torch.tensor([333, 150], dtype=torch.int32).cuda()
    before = _cabi._deterministic
    ca.set_deterministic(True)  # bitwise comparable dQ
    try:
        for ln in (None, lens):
            outs = []
            for fast in (True, False):
                qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
                assert _eager.usable(qd, kd, vd, ln)
                if fast:
                    o, lse = ca.chill_attention(qd, kd, vd, mask=mask, lens=ln, return_lse=True)
                else:
                    o, lse = chill._chill_attention(q=qd, k=kd, v=vd, lens=ln, mask_name=mask.name, mask_args=mask.constargs,
                                                    sm_scale=128 ** -0.5, return_lse=True, prescale_qk=False,
                                                    precision="ieee", autotune=False)
                (o.float() * do.cuda().float()).sum().add(lse.sum() * 0.01).backward()
                outs.append((o.detach(), lse.detach(), qd.grad, kd.grad, vd.grad))
            for x, y in zip(*outs):
                assert torch.equal(x, y)
    finally:
        ca.set_deterministic(before)
    # no-grad call: a single tensor comes back, nothing is recorded
    with torch.no_grad():
        o = ca.chill_attention(q.cuda(), k.cuda(), v.cuda(), mask=mask)
    assert isinstance(o, torch.Tensor) and not o.requires_grad


def test_forward_and_backward_replay_from_a_cuda_graph():
    """chill_attention() and its backward enqueue on the current stream without synchronising or allocating outside
    torch's allocator, so a caller can capture them in a CUDA graph (how the reference's benchmark script times its
    kernels, benchmark/benchmark.py:263-264).  Replays with new input values must give what eager calls give."""
    import chill_attention as ca

    mask = ca.SlidingWindowChillMask(16, 16)
    q, k, v, do = (t.cuda() for t in make_inputs(2, 4, 2, 520, 128, torch.float16, seed=51))
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)

    def step():
        o = ca.chill_attention(q, k, v, mask=mask)
        gq, gk, gv = torch.autograd.grad(o, (q, k, v), do)
        return o, gq, gk, gv

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            step()  # one-time set-up of the kernels happens outside the capture
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = step()
    with torch.no_grad():  # new values in the captured input buffers
        for t, s_ in zip((q, k, v, do), make_inputs(2, 4, 2, 520, 128, torch.float16, seed=52)):
            t.copy_(s_.cuda())
    graph.replay()
    torch.cuda.synchronize()
    eager = step()
    assert torch.equal(outs[0], eager[0])
    assert torch.equal(outs[2], eager[2]) and torch.equal(outs[3], eager[3])  # dK, dV are deterministic
    rel = ((outs[1].double() - eager[1].double()).norm() / eager[1].double().norm()).item()
    assert rel <= 1e-2  # dQ: fp32 reductions in an order that is not fixed
