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
@pytest.mark.parametrize("dtype,D", [(torch.bfloat16, 128), (torch.float32, 32)], ids=str)
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
