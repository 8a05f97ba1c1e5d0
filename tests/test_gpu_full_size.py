"""Parity at the full sizes of the benchmark configurations, through properties that do not need an
L x L oracle:

* sampled rows: O and LSE of 64 random query rows per case against the fp64 oracle evaluated on
  exactly those rows (the key range of a row is small or at most L);
* V = 1 gives O = 1 on every row that sees a key (softmax normalisation over the whole masked row);
* column-sum identities of the gradients, valid for any mask because every P row sums to 1:
      sum_k dV[k, :] = sum_q dO[q, :]         (per batch and kv head, summed over its GQA group)
      sum_k dS[q, k] = 0  =>  with K = const rows, dQ = 0
* sampled rows of dQ and sampled key rows of dK, dV against the oracle restricted to the rows/keys
  that can interact with them.
"""
import pytest
import torch

from helpers import G_RTOL, O_ATOL, ensure_built

pytestmark = pytest.mark.gpu

CASES = {
    "c2": ("CausalChillMask", (), torch.bfloat16, 8, 16, 4096, 128),
    "c3": ("ChunkwiseChillMask", (128, 2), torch.float16, 4, 32, 16384, 64),
    "c4": ("PrefixLMChillMask", (1024,), torch.bfloat16, 4, 16, 8192, 128),
    "c5": ("SlidingWindowChillMask", (1024, 0), torch.bfloat16, 1, 32, 131072, 128),
}


@pytest.fixture(scope="module", autouse=True)
def _lib():
    ensure_built()
    from chill_attention import _cabi

    lib = _cabi.load_library()
    yield lib
    assert lib.chill_read_device_status() == 0


def _run(name, ones_v=False, const_k=False):
    import chill_attention as ca

    mname, margs, dtype, B, H, L, D = CASES[name]
    mask = getattr(ca, mname)(*margs)
    g = torch.Generator(device="cuda").manual_seed(20)
    q, k, v, do = (torch.randn(B, H, L, D, generator=g, device="cuda", dtype=torch.float32).to(dtype) for _ in range(4))
    if ones_v:
        v = torch.ones_like(v)
    if const_k:
        k = k[:, :, :1].expand(B, H, L, D).contiguous()
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    o, lse = ca.chill_attention(q, k, v, mask=mask, return_lse=True)
    o.backward(do)
    return mask, q, k, v, do, o, lse


@pytest.mark.parametrize("name", sorted(CASES))
def test_sampled_rows_and_identities(name):
    from oracle import attention_oracle as orc

    mask, q, k, v, do, o, lse = _run(name)
    mname, margs, dtype, B, H, L, D = CASES[name]
    cls = type(mask)
    gen = torch.Generator().manual_seed(1)
    # ---- forward + dQ on sampled query rows (including first/last rows and tile edges)
    rows = torch.cat([torch.tensor([0, 1, 127, 128, 129, L - 129, L - 128, L - 1]), torch.randint(0, L, (56,), generator=gen)]).unique()
    # the corner (batch, head) units plus two drawn at random: a wrong tile in any head must be able to show
    units = {(0, 0), (B - 1, H - 1)}
    while len(units) < 4:
        units.add((int(torch.randint(0, B, (1,), generator=gen)), int(torch.randint(0, H, (1,), generator=gen))))
    for bi, hi in sorted(units):
        for r in rows.tolist():
            lo, hi_k = (int(x) for x in cls.k_range_for_q(r, L, margs))
            kp = torch.arange(lo, hi_k + 1)
            md = orc.builtin_mask_dense(mname, margs, torch.tensor([r]), kp)
            qs = q[bi:bi + 1, hi:hi + 1, r:r + 1].detach().cpu().double()
            ks = k[bi:bi + 1, hi:hi + 1, lo:hi_k + 1].detach().cpu().double()
            vs = v[bi:bi + 1, hi:hi + 1, lo:hi_k + 1].detach().cpu().double()
            dos = do[bi:bi + 1, hi:hi + 1, r:r + 1].cpu().double()
            o_ref, lse_ref = orc.attention_forward(md, qs, ks, vs, None, None, torch.float64, torch.tensor([r]), kp, L)
            dq_ref, _, _ = orc.attention_backward(md, qs, ks, vs, dos, None, None, torch.float64, torch.tensor([r]), kp, L)
            assert (o[bi, hi, r].cpu().double() - o_ref[0, 0, 0]).abs().max() <= O_ATOL[dtype], (name, r)
            assert abs(lse[bi, hi, r].item() - lse_ref[0, 0, 0].item()) <= 1e-3 * max(1.0, abs(lse_ref[0, 0, 0].item()))
            err = (q.grad[bi, hi, r].cpu().double() - dq_ref[0, 0, 0]).norm().item()
            # one row: less averaging than a whole tensor; the absolute term covers rows whose exact gradient is 0
            assert err <= 2 * G_RTOL[dtype] * dq_ref.norm().item() + 2e-2, (name, "dq", r, err)
    # ---- dK / dV on sampled key rows
    keys = torch.cat([torch.tensor([0, 127, 128, L - 1]), torch.randint(0, L, (12,), generator=gen)]).unique()
    key_units = [(B - 1, 0), (int(torch.randint(0, B, (1,), generator=gen)), int(torch.randint(0, H, (1,), generator=gen)))]
    for bi, hi in key_units:
        for kk in keys.tolist():
            lo, hi_q = (int(x) for x in cls.q_range_for_k(kk, L, margs))
            qp = torch.arange(lo, hi_q + 1)
            # P needs the full softmax row of every query that sees this key: use the stored LSE instead
            qs = q[bi, hi, lo:hi_q + 1].detach().cpu().double()
            dos = do[bi, hi, lo:hi_q + 1].cpu().double()
            os_ = o[bi, hi, lo:hi_q + 1].detach().cpu().double()
            lses = lse[bi, hi, lo:hi_q + 1].cpu().double()
            kv, vv = k[bi, hi, kk].detach().cpu().double(), v[bi, hi, kk].detach().cpu().double()
            vis = orc.builtin_mask_dense(mname, margs, qp, torch.tensor([kk]))[:, 0]
            s2 = (qs @ kv) * (D ** -0.5) * orc.LOG2E
            p = torch.where(vis, torch.exp2(s2 - lses), torch.zeros_like(s2))
            dv_ref = p @ dos
            ds = p * (dos @ vv - (os_ * dos).sum(-1))
            dk_ref = (ds @ qs) * (D ** -0.5)
            for nm, mine, ref in (("dv", v.grad[bi, hi, kk], dv_ref), ("dk", k.grad[bi, hi, kk], dk_ref)):
                err = (mine.cpu().double() - ref).norm().item()
                assert err <= 3 * G_RTOL[dtype] * ref.norm().item() + 2e-2, (name, nm, kk, err)
    # ---- checksum identity: sum over keys of dV equals sum over queries of dO
    lhs = v.grad.double().sum(dim=2)
    rhs = do.double().sum(dim=2)
    assert ((lhs - rhs).norm() / rhs.norm()).item() <= G_RTOL[dtype]


@pytest.mark.parametrize("name", ["c2", "c5"])
def test_unit_values_give_unit_output(name):
    mask, q, k, v, do, o, lse = _run(name, ones_v=True)
    assert (o.float() - 1.0).abs().max().item() <= 4e-3   # one 16-bit rounding of the normalised sum


@pytest.mark.parametrize("name", ["c2", "c3"])
def test_constant_keys_give_zero_dq(name):
    mask, q, k, v, do, o, lse = _run(name, const_k=True)
    # dS rows sum to zero, so with identical key rows dQ = (sum_k dS) k = 0 up to rounding of P and dS
    scale = do.float().abs().mean().item() * k.float().abs().mean().item()
    assert q.grad.float().abs().max().item() <= 0.05 * scale * 16
