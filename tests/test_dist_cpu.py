"""Partition and halo-exchange logic on CPU ranks (gloo, world_size 2 and 3).

The local attention is the dense oracle here (the CUDA kernels need a GPU); what is under test
is chill_attention.dist: who sends which rows to whom, the global offsets handed to the local
kernel, and the accumulation of returned dK/dV halos.  Expectation = single-process oracle."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import ROOT


def _oracle_local_forward(mask, q, k_ext, v_ext, q_off, k_off, seq_len, sm_scale, o, lse):
    from oracle import attention_oracle as orc

    qp = torch.arange(q_off, q_off + q.shape[2])
    kp = torch.arange(k_off, k_off + k_ext.shape[2])
    md = orc.builtin_mask_dense(mask.name, mask.constargs, qp, kp)
    o_ref, lse_ref = orc.attention_forward(md, q, k_ext, v_ext, None, sm_scale, torch.float64, qp, kp, seq_len)
    o.copy_(o_ref)
    lse.copy_(lse_ref)


def _oracle_local_backward(mask, q, k_ext, v_ext, o, lse, do, q_off, k_off, seq_len, sm_scale, dq, dk, dv, part):
    from oracle import attention_oracle as orc

    qp = torch.arange(q_off, q_off + q.shape[2])
    kp = torch.arange(k_off, k_off + k_ext.shape[2])
    md = orc.builtin_mask_dense(mask.name, mask.constargs, qp, kp)
    rdq, rdk, rdv = orc.attention_backward(md, q, k_ext, v_ext, do, None, sm_scale, torch.float64, qp, kp, seq_len)
    dq.copy_(rdq)
    # the 16-bit results of a real kernel are rounded; mimic that here so that a wrong use of them shows
    dk.copy_(rdk.to(torch.bfloat16))
    dv.copy_(rdv.to(torch.bfloat16))
    if part is not None:
        dkp, dvp, head, tail = part
        Lk = k_ext.shape[2]
        for dst, src in ((dkp, rdk), (dvp, rdv)):
            dst[:, :, :head] = src[:, :, :head]
            dst[:, :, head:head + tail] = src[:, :, Lk - tail:]


def _worker(rank, world, port, mask_name, mask_args, L, fail_rank, use_buffers=False):
    for p in (os.path.join(ROOT, "chill-attention_b200"), ROOT, os.path.join(ROOT, "tests")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import chill_attention as ca
        from chill_attention import dist as cdist
        from oracle import attention_oracle as orc

        mask = getattr(ca, mask_name)(*mask_args)
        g = torch.Generator().manual_seed(7)
        B, H, Hkv, D = 2, 4, 2, 8
        q, do = (torch.randn(B, H, L, D, generator=g, dtype=torch.float64) for _ in range(2))
        k, v = (torch.randn(B, Hkv, L, D, generator=g, dtype=torch.float64) for _ in range(2))
        Ls = L // world
        sl = slice(rank * Ls, (rank + 1) * Ls)
        if fail_rank is not None:
            # a window wider than the shard must be refused on every rank before any message is sent
            with pytest.raises(ValueError):
                cdist.halo_sizes(mask, Ls)
            return
        left, right = cdist.halo_sizes(mask, Ls)
        ql = q[:, :, sl].clone().requires_grad_(True)
        if use_buffers:
            # K and V live in HaloBuffers: the halo rows are received straight into their spare rows
            kbuf = cdist.HaloBuffer(B, Hkv, Ls, D, left, right, torch.float64, "cpu")
            vbuf = cdist.HaloBuffer(B, Hkv, Ls, D, left, right, torch.float64, "cpu")
            kbuf.storage.fill_(float("nan")), vbuf.storage.fill_(float("nan"))  # unreceived rows must never be read
            kbuf.local.copy_(k[:, :, sl]), vbuf.local.copy_(v[:, :, sl])
            kl, vl = kbuf.local.requires_grad_(True), vbuf.local.requires_grad_(True)
            buffers = (kbuf, vbuf)
        else:
            kl, vl = (t[:, :, sl].clone().requires_grad_(True) for t in (k, v))
            buffers = None
        o = cdist.sequence_sharded_attention(ql, kl, vl, mask, L, group=None, halo_buffers=buffers,
                                             local_forward=_oracle_local_forward, local_backward=_oracle_local_backward)
        o.backward(do[:, :, sl])
        pos = torch.arange(L)
        md = orc.builtin_mask_dense(mask.name, mask.constargs, pos, pos)
        o_ref, _ = orc.attention_forward(md, q, k, v)
        dq, dk, dv = orc.attention_backward(md, q, k, v, do)
        torch.testing.assert_close(o.detach(), o_ref[:, :, sl], atol=1e-10, rtol=1e-10)
        torch.testing.assert_close(ql.grad, dq[:, :, sl], atol=1e-10, rtol=1e-10)
        # Key rows that receive contributions from more than one call (this rank's boundary + interior calls, a
        # neighbour's boundary call) must be summed before any rounding: exact here.  The rows in between come
        # from the interior call's 16-bit output alone, which the stand-in kernel above rounds to bf16.
        must_be_exact = torch.zeros(Ls, dtype=torch.bool)
        if rank > 0:
            must_be_exact[:min(Ls, left + right)] = True
        if rank < world - 1:
            must_be_exact[max(0, Ls - left - right):] = True
        for mine, ref in ((kl.grad, dk[:, :, sl]), (vl.grad, dv[:, :, sl])):
            torch.testing.assert_close(mine[:, :, must_be_exact], ref[:, :, must_be_exact], atol=1e-10, rtol=1e-10)
            torch.testing.assert_close(mine, ref, atol=2e-2, rtol=1e-2)
    finally:
        dist.destroy_process_group()


def _spawn(world, *a):
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port) + a, nprocs=world, join=True)


@pytest.mark.parametrize("world", [2, 3])
@pytest.mark.parametrize("mask", [("SlidingWindowChillMask", (10, 0)), ("SlidingWindowChillMask", (7, 5)),
                                  ("SlidingWindowChillMask", (9, 8)),  # both boundaries overlap on a 16-row shard
                                  ("ChunkwiseChillMask", (6, 1))], ids=str)
@pytest.mark.parametrize("use_buffers", [False, True], ids=["copied", "halo_buffers"])
def test_sequence_sharded_equals_single_process(world, mask, use_buffers):
    _spawn(world, mask[0], mask[1], 48, None, use_buffers)


def test_window_wider_than_shard_is_refused():
    _spawn(2, "SlidingWindowChillMask", (30, 0), 48, 0)


def test_shard_units_partition():
    from chill_attention.dist import shard_batch_heads, shard_units

    for n, w in ((128, 8), (64, 3), (5, 8), (7, 2)):
        spans = [shard_units(n, w, r) for r in range(w)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert max(h - l for l, h in spans) - min(h - l for l, h in spans) <= 1
    t = torch.arange(2 * 6 * 3 * 2).reshape(2, 6, 3, 2)
    parts = [shard_batch_heads(t, 3, 2, r) for r in range(2)]       # GQA: 3 kv heads, groups of 2 query heads stay together
    assert torch.equal(torch.cat(parts).reshape(2, 6, 3, 2), t) and parts[0].shape == (3, 2, 3, 2)


def test_unbounded_masks_are_refused():
    import chill_attention as ca
    from chill_attention.dist import halo_sizes

    with pytest.raises(NotImplementedError):
        halo_sizes(ca.CausalChillMask(), 1024)
    assert halo_sizes(ca.SlidingWindowChillMask(1024, 0), 16384) == (1024, 0)
    assert halo_sizes(ca.ChunkwiseChillMask(128, 2), 4096) == (383, 127)
