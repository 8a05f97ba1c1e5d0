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
    lens = torch.tensor([L, 0, 130, L + 1], dtype=torch.int32)
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


@pytest.mark.parametrize("D", [128, 256])
@pytest.mark.parametrize("q0,k0", [(512, 256), (500, 300)])
def test_shard_with_global_offsets_matches_the_full_problem(lib, q0, k0, D):
    """Queries [q0, L) against keys [k0, L) of a sliding-window problem, with q_offset / k_offset / seq_len:
    the rows a shard owns must equal the same rows of the unsharded result (what the sequence-sharded
    multi-GPU path relies on), for both forms of the backward."""
    import ctypes as C

    import chill_attention as ca
    from chill_attention import _cabi

    L, W, dtype = 1024, 200, torch.bfloat16
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
    nacc = lib.chill_bwd_dq_accum_bytes(C.byref(shape)) // 4  # 0 for head dim 256 (three-launch backward, no scratch)
    accum = torch.empty(nacc, dtype=torch.float32, device="cuda") if nacc else None
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


@pytest.mark.parametrize("form", ["single_kernel", "two_kernel", "generic", "head_dim_256"])
@pytest.mark.parametrize("layout", ["rows_major", "heads_major"])
def test_fp32_partial_copies_of_dk_dv(lib, form, layout):
    """chill_bwd_args.dk_part / dv_part: un-rounded fp32 dK / dV of the first `head` and last `tail` key rows.
    They must round to exactly the 16-bit outputs of the same call, be closer to the fp64 oracle than those, and
    rows outside the two windows must stay untouched."""
    import ctypes as C

    import chill_attention as ca
    from chill_attention import _cabi

    mask = ca.SlidingWindowChillMask(300, 40)
    B, H, Hkv, L, D, dtype = 2, 4, 2, 700, (256 if form == "head_dim_256" else 128), torch.bfloat16
    q, k, v, do = make_inputs(B, H, Hkv, L, D, dtype, seed=36)
    lens = torch.tensor([L, 650], dtype=torch.int32)  # the last key tile of batch row 1 is partly padding
    _, _, _, dk_ref, dv_ref = oracle_all(mask, q, k, v, do, lens)
    qd, kd, vd, dod, lens_d = (t.cuda() for t in (q, k, v, do, lens))
    flags = _cabi.FLAG_FORCE_GENERIC if form == "generic" else 0
    shape = _cabi.make_shape(qd, kd, _cabi.BUILTIN_FUNCTOR_IDS[mask.cuda_functor], mask.constargs, lens_d, D ** -0.5, flags=flags)
    o, lse = torch.empty_like(qd), torch.empty(B, H, L, dtype=torch.float32, device="cuda")
    _cabi.forward(lib, qd, kd, vd, o, lse, shape)
    delta = torch.empty_like(lse)
    accum = None
    if form == "single_kernel":
        accum = torch.empty(lib.chill_bwd_dq_accum_bytes(C.byref(shape)) // 4, dtype=torch.float32, device="cuda")
    head, tail = 200, 130
    if layout == "rows_major":   # [2, B, rows, H_kv, D] in memory, as the sequence-sharded path uses it
        buf = torch.full((2, B, head + tail + 3, Hkv, D), float("nan"), dtype=torch.float32, device="cuda")
        views = [buf[t].permute(0, 2, 1, 3) for t in range(2)]
    else:
        buf = torch.full((2, B, Hkv, head + tail + 3, D), float("nan"), dtype=torch.float32, device="cuda")
        views = [buf[t] for t in range(2)]
    g = [torch.empty_like(qd), torch.empty_like(kd), torch.empty_like(vd)]
    a = _cabi.backward_args(qd, kd, vd, o, dod, lse, delta, *g, shape, accum, part=(views[0], views[1], head, tail))
    assert lib.chill_bwd_uses_tensor_cores(C.byref(a)) == (0 if form == "generic" else 1)
    st = _cabi._stream()
    _cabi.check(lib, lib.chill_bwd_delta(C.byref(a), st), "chill_bwd_delta")
    _cabi.check(lib, lib.chill_bwd(C.byref(a), st), "chill_bwd")
    torch.cuda.synchronize()
    for part, out16, ref in ((views[0], g[1], dk_ref), (views[1], g[2], dv_ref)):
        part = part.cpu()
        assert torch.isnan(part[:, :, head + tail:]).all(), "rows beyond head + tail must not be written"
        got = torch.cat([part[:, :, :head], part[:, :, head:head + tail]], dim=2)
        want16 = torch.cat([out16[:, :, :head], out16[:, :, L - tail:]], dim=2).cpu()
        assert torch.equal(got.to(dtype), want16), "the 16-bit output is the rounded partial"
        want = torch.cat([ref[:, :, :head], ref[:, :, L - tail:]], dim=2)
        err32 = (got.double() - want).norm().item()
        err16 = (want16.double() - want).norm().item()
        assert err32 <= err16 and err32 <= G_RTOL[dtype] * want.norm().item()
        assert (got[1, :, head + (650 - (L - tail)):] == 0).all(), "key rows at or beyond lens[b] have zero gradient"
    # invalid windows are refused before any launch
    a.part_head, a.part_tail = L, 1
    assert lib.chill_bwd(C.byref(a), st) == -1


def test_huge_mask_constants_mean_unbounded(lib):
    """Mask constants beyond the 32-bit range (a common way to write 'unbounded') must not wrap."""
    import chill_attention as ca

    q, k, v, do = make_inputs(1, 2, 2, 300, 64, torch.float16, seed=37)
    outs = []
    for mask in (ca.CausalChillMask(), ca.SlidingWindowChillMask(2 ** 31 - 1, 0), ca.SlidingWindowChillMask(2 ** 40, 0),
                 ca.ChunkwiseChillMask(2 ** 33, 2 ** 35)):
        qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
        o = ca.chill_attention(qd, kd, vd, mask=mask)
        o.backward(do.cuda())
        outs.append((o.detach(), qd.grad, kd.grad, vd.grad))
    for other in outs[1:3]:
        # Equal up to rounding, not bit for bit: the two functors mark different tiles as "full", padding rows of
        # the last query tile then carry different running maxima, and the forward's lazy rescale (decided per warp)
        # may fire at different tiles for the real rows that share a warp with them; dQ is summed in an order that
        # is not fixed.
        for x, y in zip(outs[0], other):
            assert ((x.double() - y.double()).norm() / y.double().norm()).item() <= 1e-3
            assert (x.double() - y.double()).abs().max().item() <= 2e-3 * max(1.0, y.double().abs().max().item())
    full = oracle_all(ca.FullChillMask(), q, k, v, do)  # one chunk that spans everything = full attention
    assert (outs[3][0].cpu().double() - full[0]).abs().max().item() <= 1e-2
    check_grads(outs[3][1:], full[2:], torch.float16)


def test_expanded_grad_output_stays_on_the_tensor_cores(lib):
    """o.sum().backward() hands the backward an expanded (stride-0) dO; it is made contiguous instead of
    dropping to the generic kernels."""
    import chill_attention as ca
    from chill_attention import chill as chill_mod

    q, k, v, _ = make_inputs(1, 2, 2, 384, 128, torch.bfloat16, seed=38)
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    before = chill_mod.backward_path_counts()
    ca.chill_attention(qd, kd, vd, mask=ca.CausalChillMask()).sum().backward()
    after = chill_mod.backward_path_counts()
    assert after["tensor_core"] == before["tensor_core"] + 1 and after["generic"] == before["generic"]
    ref = oracle_all(ca.CausalChillMask(), q, k, v, torch.ones_like(q))[2:]
    check_grads((qd.grad, kd.grad, vd.grad), ref, torch.bfloat16)


def test_two_host_threads_run_the_two_kernel_backward_on_one_device(lib):
    """The two-kernel backward forks onto a helper stream shared per device; two host threads on two streams
    must still get the serial result bit for bit."""
    import ctypes as C
    import threading

    import chill_attention as ca
    from chill_attention import _cabi

    mask = ca.CausalChillMask()
    fid = _cabi.BUILTIN_FUNCTOR_IDS[mask.cuda_functor]
    cases = []
    for seed in (41, 42):
        q, k, v, do = (t.cuda() for t in make_inputs(2, 4, 4, 1024, 128, torch.bfloat16, seed=seed))
        shape = _cabi.make_shape(q, k, fid, (), None, 128 ** -0.5)
        o, lse = torch.empty_like(q), torch.empty(2, 4, 1024, dtype=torch.float32, device="cuda")
        _cabi.forward(lib, q, k, v, o, lse, shape)
        cases.append((q, k, v, do, o, lse, shape))
    torch.cuda.synchronize()

    def run(case, stream, reps):
        q, k, v, do, o, lse, shape = case
        delta = torch.empty_like(lse)
        g = [torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)]
        a = _cabi.backward_args(q, k, v, o, do, lse, delta, *g, shape, None)
        st = C.c_void_p(stream.cuda_stream)
        for _ in range(reps):
            _cabi.check(lib, lib.chill_bwd_delta(C.byref(a), st), "chill_bwd_delta")
            _cabi.check(lib, lib.chill_bwd(C.byref(a), st), "chill_bwd")
        stream.synchronize()
        return g

    serial = [run(c, torch.cuda.Stream(), 1) for c in cases]
    results = [None, None]

    def worker(i):
        torch.cuda.set_device(0)
        results[i] = run(cases[i], torch.cuda.Stream(), 20)

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    torch.cuda.synchronize()
    for want, got in zip(serial, results):
        for x, y in zip(want, got):
            assert torch.equal(x, y)


def test_two_copies_of_the_library_in_one_process(tmp_path):
    """A custom-mask build is a second library made from the same sources.  Each copy keeps its own record of which
    kernels had their shared-memory limit raised: if the copies shared it, the second one would launch kernels whose
    limit was never set ("invalid argument")."""
    import shutil

    import chill_attention as ca
    from chill_attention import _cabi

    second = str(tmp_path / "libchill_b200_copy.so")
    shutil.copy(_cabi.DEFAULT_LIB, second)
    libs = [_cabi.load_library(), _cabi.load_library(second)]
    assert libs[0] is not libs[1]
    mask = ca.CausalChillMask()
    q, k, v, do = (t.cuda() for t in make_inputs(1, 2, 2, 300, 128, torch.bfloat16))
    shape = _cabi.make_shape(q, k, _cabi.BUILTIN_FUNCTOR_IDS[mask.cuda_functor], mask.constargs, None, 128 ** -0.5)
    outs = []
    for lib in libs:
        o = torch.empty_like(q)
        lse = torch.empty(q.shape[:3], dtype=torch.float32, device="cuda")
        _cabi.forward(lib, q, k, v, o, lse, shape)
        delta = torch.empty_like(lse)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        for deterministic in (False, True):  # single-kernel and two-kernel backward: different kernels, each set up once
            _cabi.backward(lib, q, k, v, o, do, lse, delta, dq, dk, dv, shape, deterministic=deterministic)
        torch.cuda.synchronize()
        assert lib.chill_read_device_status() == 0
        outs.append((o, dq, dk, dv))
    for a, b in zip(*outs):
        assert torch.equal(a, b)
