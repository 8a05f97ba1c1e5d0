"""Host half of the mask contract: same API as the reference, same tables as the reference."""
import os

import numpy as np
import pytest
import torch

import chill_attention as ca
from conftest import GOLDEN
from helpers import all_masks, big_masks


def test_export_list():
    for name in ("chill_attention", "register_chill_mask", "_chill_reference_naive", "ChillMask", "FullChillMask",
                 "CausalChillMask", "SlidingWindowChillMask", "ChunkwiseChillMask", "PrefixLMChillMask"):
        assert hasattr(ca, name)


def test_names_and_constargs():
    m = ca.SlidingWindowChillMask(10, 4)
    assert m.name == "SlidingWindowChillMask" and m.constargs == (10, 4) and str(m) == "SlidingWindowChillMask(10, 4)"
    assert str(ca.CausalChillMask()) == "CausalChillMask()" and ca.CausalChillMask().constargs == ()
    assert str(ca.PrefixLMChillMask(7)) == "PrefixLMChillMask(7)"
    with pytest.raises(AssertionError):
        ca.ChillMask(constargs=[1, 2])
    with pytest.raises(AssertionError):
        ca.ChillMask(constargs=("a",))


def test_host_predicates():
    assert ca.CausalChillMask.is_guaranteed_safe() and not ca.SlidingWindowChillMask.is_guaranteed_safe()
    assert not ca.ChillMask.has_k_full_range() and ca.ChunkwiseChillMask.has_k_full_range()
    assert ca.ChillMask.q_lims_continious() and ca.ChillMask.k_lims_continious()
    assert ca.CausalChillMask.has_full_blocks(64, 64, seq_len=128, args=())
    assert not ca.CausalChillMask.has_full_blocks(128, 64, seq_len=128, args=())
    assert ca.SlidingWindowChillMask.has_full_blocks(32, 32, 1024, (64, 0))
    assert not ca.SlidingWindowChillMask.has_full_blocks(64, 64, 1024, (64, 0))
    assert ca.ChunkwiseChillMask.has_full_blocks(128, 128, 4096, (128, 2))
    assert ca.ChillMask.k_full_range_for_q(0, 16, 64, ()) == (0, 0)


@pytest.mark.parametrize("mask", all_masks() + big_masks(), ids=str)
def test_masks_verify(mask):
    mask.verify(512)


def test_verify_catches_a_wrong_range():
    class Broken(ca.CausalChillMask):
        @staticmethod
        def k_range_for_q(q, seq_len, args):
            return q * 0, q + 1

    with pytest.raises(AssertionError):
        Broken().verify(64)


def test_tables_equal_reference():
    z = np.load(os.path.join(GOLDEN, "masks.npz"))
    for key in sorted({k.split("/")[0] for k in z.files}):
        name, rest = key.split("(")
        args = tuple(int(a) for a in rest.rstrip(")").split(",") if a)
        m = getattr(ca, name)(*args)
        ref_mask = torch.from_numpy(np.unpackbits(z[key + "/mask"])[: 96 * 96].reshape(96, 96).astype(bool))
        assert torch.equal(m.make_mask(96, device="cpu"), ref_mask), key
        assert torch.equal(m._calc_limits(96, type(m).k_range_for_q, device="cpu"), torch.from_numpy(z[key + "/k_lims"])), key
        assert torch.equal(m._calc_limits(96, type(m).q_range_for_k, device="cpu"), torch.from_numpy(z[key + "/q_lims"])), key


@pytest.mark.parametrize("mask", all_masks(), ids=str)
def test_flex_mask_mod_consistent(mask):
    # the reference compares make_mask with FlexAttention's create_mask (test/test_chill_attention.py:332-345)
    from torch.nn.attention.flex_attention import create_mask

    n = 200
    flex = create_mask(mask.mask_mod(), None, None, n, n, device="cpu")[0, 0]
    assert torch.equal(flex, mask.make_mask(n, device="cpu"))
