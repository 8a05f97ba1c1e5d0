"""Sequence-sharded attention on 2 GPUs (NCCL halo exchange + the CUDA kernels with global offsets).
Skipped on a single-GPU box; the partition logic itself is covered on CPU ranks in test_dist_cpu.py."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import ROOT, ensure_built

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, mask_name, mask_args, L, dtype_name, use_buffers):
    for p in (os.path.join(ROOT, "chill-attention_b200"), ROOT, os.path.join(ROOT, "tests")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import chill_attention as ca
        from chill_attention import _cabi
        from chill_attention import dist as cdist
        from helpers import G_RTOL, O_ATOL
        from oracle import attention_oracle as orc

        dtype = getattr(torch, dtype_name)
        mask = getattr(ca, mask_name)(*mask_args)
        g = torch.Generator().manual_seed(11)
        B, H, Hkv, D = 1, 4, 2, 128
        q, do = (torch.randn(B, H, L, D, generator=g).to(dtype) for _ in range(2))
        k, v = (torch.randn(B, Hkv, L, D, generator=g).to(dtype) for _ in range(2))
        Ls = L // world
        sl = slice(rank * Ls, (rank + 1) * Ls)
        ql = q[:, :, sl].cuda().requires_grad_(True)
        if use_buffers:
            left, right = cdist.halo_sizes(mask, Ls)
            kbuf = cdist.HaloBuffer(B, Hkv, Ls, D, left, right, dtype, "cuda")
            vbuf = cdist.HaloBuffer(B, Hkv, Ls, D, left, right, dtype, "cuda")
            kbuf.storage.fill_(float("nan")), vbuf.storage.fill_(float("nan"))  # rows nobody sends must never be read
            kbuf.local.copy_(k[:, :, sl]), vbuf.local.copy_(v[:, :, sl])
            kl, vl = kbuf.local.requires_grad_(True), vbuf.local.requires_grad_(True)
            buffers = (kbuf, vbuf)
        else:
            kl, vl = (t[:, :, sl].cuda().requires_grad_(True) for t in (k, v))
            buffers = None
        o = cdist.sequence_sharded_attention(ql, kl, vl, mask, L, halo_buffers=buffers)
        o.backward(do[:, :, sl].cuda())
        torch.cuda.synchronize()
        assert _cabi.load_library().chill_read_device_status() == 0
        pos = torch.arange(L)
        md = orc.builtin_mask_dense(mask.name, mask.constargs, pos, pos)
        o_ref, _ = orc.attention_forward(md, q.double(), k.double(), v.double())
        grads = orc.attention_backward(md, q.double(), k.double(), v.double(), do.double())
        assert (o.detach().cpu().double() - o_ref[:, :, sl]).abs().max() <= O_ATOL[dtype]
        for mine, ref in zip((ql.grad, kl.grad, vl.grad), grads):
            ref = ref[:, :, sl]
            rel = ((mine.cpu().double() - ref).norm() / ref.norm()).item()
            assert rel <= G_RTOL[dtype], rel  # partial dK/dV of boundary rows are summed in fp32 and rounded once
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mask", [("SlidingWindowChillMask", (300, 0)), ("SlidingWindowChillMask", (200, 70)),
                                  ("ChunkwiseChillMask", (128, 2))], ids=str)
@pytest.mark.parametrize("use_buffers", [False, True], ids=["copied", "halo_buffers"])
def test_sequence_sharded_on_two_gpus(mask, use_buffers):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ensure_built()
    port = 29600 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, mask[0], mask[1], 2048, "bfloat16", use_buffers), nprocs=2, join=True)


def test_tensors_on_a_device_that_is_not_current():
    """One process, two GPUs: calls for tensors on cuda:1 while cuda:0 is the current device (and the other way
    round afterwards).  The library keeps its per-kernel set-up, status word and helper streams per device."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ensure_built()
    import chill_attention as ca
    from chill_attention import _cabi
    from helpers import check_forward, check_grads, make_inputs, oracle_all

    lib = _cabi.load_library()
    mask = ca.SlidingWindowChillMask(200, 0)
    for dtype, D in ((torch.bfloat16, 128), (torch.float32, 32)):
        q, k, v, do = make_inputs(2, 4, 2, 520, D, dtype, seed=61)
        o_ref, lse_ref, *g_ref = oracle_all(mask, q, k, v, do)
        for current, other in ((0, 1), (1, 0)):
            torch.cuda.set_device(current)
            dev = torch.device("cuda", other)
            qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
            for deterministic in (False, True):
                ca.set_deterministic(deterministic)
                try:
                    o, lse = ca.chill_attention(qd, kd, vd, mask=mask, return_lse=True)
                    grads = torch.autograd.grad(o, (qd, kd, vd), do.to(dev))
                finally:
                    ca.set_deterministic(False)
                assert o.device == dev and all(g.device == dev for g in grads)
                check_forward(o, lse, o_ref, lse_ref, None, dtype)
                check_grads(grads, g_ref, dtype)
            for d in (0, 1):
                with torch.cuda.device(d):
                    torch.cuda.synchronize()
                    assert lib.chill_read_device_status() == 0
    torch.cuda.set_device(0)
