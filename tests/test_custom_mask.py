"""Custom-mask extension point: a user CUDA functor header compiled into a private library
(counterpart of the reference inlining a subclass's Triton functions, chill_attention/chill.py:45-52)."""
import os

import pytest
import torch

import chill_attention as ca
from helpers import ROOT, check_forward, check_grads, make_inputs

HEADER = os.path.join(ROOT, "tests", "custom_masks", "dilated_causal_mask.h")


class DilatedCausalChillMask(ca.ChillMask):
    cuda_functor_header = HEADER
    cuda_functor = "DilatedCausalMask"

    def __init__(self, stride):
        super().__init__((stride,))

    @staticmethod
    def mask(q, k, seq_len, args):
        d = q[:, None] - k[None, :]
        return (d >= 0) & (d % args[0] == 0)

    @staticmethod
    def k_range_for_q(q, seq_len, args):
        return q % args[0], q

    @staticmethod
    def q_range_for_k(k, seq_len, args):
        return k, k + ((seq_len - 1 - k) // args[0]) * args[0]

    @staticmethod
    def is_guaranteed_safe():
        return True

    @staticmethod
    def q_lims_continious():
        return False

    @staticmethod
    def k_lims_continious():
        return False


def test_python_side_verifies():
    DilatedCausalChillMask(3).verify(200)


def test_custom_library_builds_and_exports(tmp_path):
    """nvcc cross-compiles the private library without a GPU; it must export the ABI with the custom id enabled."""
    from chill_attention import _cabi
    from chill_attention.custom import build_custom_library

    path = build_custom_library(HEADER, "DilatedCausalMask")
    lib = _cabi.load_library(path)
    assert lib.chill_mask_traits(_cabi.MASK_CUSTOM) == 16   # guaranteed safe; no full ranges, limits not continuous
    assert _cabi.load_library().chill_mask_traits(_cabi.MASK_CUSTOM) == -2  # the stock library has no custom functor


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,D", [(torch.bfloat16, 128), (torch.float32, 32), (torch.float16, 256), (torch.bfloat16, 32)], ids=str)
def test_custom_mask_on_gpu(dtype, D):
    from chill_attention import chill_attention
    from oracle import attention_oracle as orc

    mask = DilatedCausalChillMask(3)
    L = 300
    q, k, v, do = make_inputs(2, 4, 2, L, D, dtype)
    pos = torch.arange(L)
    md = DilatedCausalChillMask.mask(pos, pos, L, mask.constargs)
    o_ref, lse_ref = orc.attention_forward(md, q.double(), k.double(), v.double())
    g_ref = orc.attention_backward(md, q.double(), k.double(), v.double(), do.double())
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    o, lse = chill_attention(qd, kd, vd, mask=mask, return_lse=True)
    o.backward(do.cuda())
    check_forward(o, lse, o_ref, lse_ref, None, dtype)
    check_grads((qd.grad, kd.grad, vd.grad), g_ref, dtype)
    assert hasattr(torch.ops.chill_attention, "forwardDilatedCausalChillMask")


class OffByOneWindowChillMask(ca.ChillMask):
    """Python twin of tests/custom_masks/off_by_one_window_mask.h - the Python side is right, the header is not."""
    cuda_functor_header = os.path.join(ROOT, "tests", "custom_masks", "off_by_one_window_mask.h")
    cuda_functor = "OffByOneWindowMask"

    def __init__(self, window):
        super().__init__((window,))

    @staticmethod
    def mask(q, k, seq_len, args):
        d = q[:, None] - k[None, :]
        return (d >= 0) & (d <= args[0])

    @staticmethod
    def k_range_for_q(q, seq_len, args):
        return torch.clamp(q - args[0], min=0) if isinstance(q, torch.Tensor) else max(q - args[0], 0), q

    @staticmethod
    def q_range_for_k(k, seq_len, args):
        hi = k + args[0]
        return k, (torch.clamp(hi, max=seq_len - 1) if isinstance(hi, torch.Tensor) else min(hi, seq_len - 1))

    @staticmethod
    def is_guaranteed_safe():
        return True


@pytest.mark.gpu
def test_verify_checks_the_cuda_functor_not_only_its_python_twin():
    """verify(device=True) tabulates the functor the kernels are compiled with.  The built-in functors and the
    dilated example pass; a header whose k_range_for_q is off by one passes the Python-only check and must
    raise on the device check."""
    for mask in (ca.FullChillMask(), ca.CausalChillMask(), ca.SlidingWindowChillMask(37, 5), ca.ChunkwiseChillMask(24, 2),
                 ca.PrefixLMChillMask(50), DilatedCausalChillMask(3)):
        mask.verify(300, device=True)
    wrong = OffByOneWindowChillMask(20)
    wrong.verify(300)  # the Python functions are consistent
    with pytest.raises(AssertionError, match="k_range_for_q differs"):
        wrong.verify(300, device=True)


@pytest.mark.gpu
def test_flex_mask_equals_dense_mask_on_gpu():
    """make_flex_mask (FlexAttention BlockMask, reference mask.py:456-466 and test_chill_attention.py:332-345)
    describes the same pattern as make_mask."""
    n = 300
    for mask in (ca.FullChillMask(), ca.CausalChillMask(), ca.SlidingWindowChillMask(37, 5), ca.ChunkwiseChillMask(24, 2),
                 ca.PrefixLMChillMask(50)):
        bm = mask.make_flex_mask(n)
        assert bm is not None
        dense = mask.make_mask(n, device="cuda")
        mod = mask.mask_mod()
        qi, ki = torch.meshgrid(torch.arange(n, device="cuda"), torch.arange(n, device="cuda"), indexing="ij")
        assert torch.equal(mod(0, 0, qi, ki), dense)
        # every tile the block mask keeps contains a visible pair, every visible pair lies in a kept tile
        kept = bm.to_dense()[0, 0].bool()  # (n_q_blocks, n_k_blocks)
        bs_q, bs_k = bm.BLOCK_SIZE
        nq, nk = kept.shape
        pad = torch.zeros(nq * bs_q, nk * bs_k, dtype=torch.bool, device="cuda")
        pad[:n, :n] = dense
        has_pair = pad.reshape(nq, bs_q, nk, bs_k).any(dim=3).any(dim=1)
        assert torch.equal(kept, has_pair)
