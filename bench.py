#!/usr/bin/env python
"""Benchmark of the masked-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl reference]

One "step" is one forward + backward pass (chill_fwd, chill_bwd_delta, chill_bwd) over one
synthetic batch of the workload; --bwd fused (default) gives chill_bwd the fp32 dQ scratch so that it runs
its single-kernel form, --bwd split times the bitwise-reproducible two-kernel form.  The default workload is the configuration the headline
metric is quoted on: CausalChillMask, bf16, (B, H, L, D) = (8, 16, 4096, 128), inputs ~N(0,1)
seeded, sm_scale = D**-0.5.  Other workloads (c3, c4, c5 ...) are for kernel work, not for the
reported line.

Reported (one JSON line on rank 0):
  value        effective TFLOP/s of forward+backward counting only unmasked (q, k) pairs:
               14 * B * H * D * pairs FLOPs per step (4 fwd + 10 bwd), inputs resident in HBM,
               timed with CUDA events on the launching stream, max over ranks.  The timed step is
               chill_fwd, chill_bwd_delta, chill_bwd exactly as a caller issues them; `kernel_ms`
               comes from a second pass in which the kernels are launched one at a time.
  fwd / fwd_bwd / pct_of_peak   the forward-only number and both as a share of the measured
               dense bf16 peak (MEASURED_PEAKS.json) and of the nominal 2250 TFLOP/s.
  roofline     dominant kernel (largest share of the step): algorithmic FLOPs / its mean
               CUDA-event duration, against the measured cuBLAS bf16 peak.
  e2e          the same metric through the public host-buffer API
               (chill_attention.host.attention_fwd_bwd_host): per step q, k, v, dO are copied from
               pinned host memory and O, dQ, dK, dV are copied back, all inside the timed region
               (batch chunks on three streams so the PCIe copies overlap the kernels).
  cpu_baseline the CPU oracle (dense-mask fp32 attention, fwd + closed-form bwd) timed on the
               host cores on a bounded sample of the same workload.

  op_ms_per_step  one forward and one backward call through chill_attention() + autograd, allocations inside.
  triton_baseline the reference's own Triton kernels on the same GPU (subprocess), when a copy of its package is
               importable from baseline/_ref or $CHILL_REFERENCE_DIR; otherwise the reason it is not.

Multi-GPU (torchrun, one rank per GPU): the B x H (batch, head) units of the workload are split evenly over
the ranks - no data-path collective; the problem size is fixed ("strong" scaling), `value` = the whole
problem's FLOPs / the slowest rank's time.  After that leg the run also times workload c5 sequence-sharded
over the same ranks (K/V halo over NCCL send/recv, dK/dV halo returned in fp32) and checks rows next to
every shard boundary against the fp64 CPU oracle: block `c5_seq_sharded`.  `--workload c5 --gpus N` runs only
that leg.

`--impl reference` times the reference's CPU path (dense boolean mask + fp32 attention, the
oracle port of its `_chill_reference_naive` with closed-form gradients) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (os.path.join(ROOT, "chill-attention_b200"), ROOT):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

METRIC = "effective TFLOP/s (unmasked FLOPs) fwd & fwd+bwd, % of B200 dense BF16 peak"
NOMINAL_BF16_TFLOPS = 2250.0
FALLBACK_BF16_TFLOPS = 1590.0
# dram__bytes_read.sum + dram__bytes_write.sum per (batch, head) unit from an ncu capture of the causal bf16
# L=4096 D=128 kernels on 32 units per launch; traffic grows in proportion to the units a launch processes,
# so a full launch = per-unit figure x units.
NCU_DRAM_BYTES_PER_UNIT = {("c2", "fwd"): 120.3e6 / 32, ("c2", "dkdv"): 176.5e6 / 32, ("c2", "dq"): 156.1e6 / 32,
                           # single-kernel backward: bwd_fused_tc_kernel 290.2 MB + dq_convert_kernel 74.3 MB
                           ("c2", "bwd"): (290.2e6 + 74.3e6) / 32}

WORKLOADS = {
    # name: (mask class, mask args, dtype, B, H, L, D)
    "c1": ("CausalChillMask", (), "float32", 1, 2, 128, 64),
    "c2": ("CausalChillMask", (), "bfloat16", 8, 16, 4096, 128),
    "c3": ("ChunkwiseChillMask", (128, 2), "float16", 4, 32, 16384, 64),
    "c4": ("PrefixLMChillMask", (1024,), "bfloat16", 4, 16, 8192, 128),
    "c5": ("SlidingWindowChillMask", (1024, 0), "bfloat16", 1, 32, 131072, 128),
    "full": ("FullChillMask", (), "bfloat16", 8, 16, 4096, 128),
    # c2 with a quarter of the batch: same kernels and tile counts per CTA, small enough for an ncu capture
    "c2s": ("CausalChillMask", (), "bfloat16", 2, 16, 4096, 128),
    # c3 with a quarter of the batch, for the same purpose (head dim 64: 64-key tiles, four CTAs per SM)
    "c3s": ("ChunkwiseChillMask", (128, 2), "float16", 1, 32, 16384, 64),
    # fp32 tensors with precision="tf32": forward and backward on the TF32 tensor cores (two-kernel backward)
    "c2f32": ("CausalChillMask", (), "float32", 2, 16, 4096, 128),
    "c2f32d64": ("CausalChillMask", (), "float32", 2, 32, 4096, 64),
    # head dim 256: tensor-core forward (one CTA per SM) and the three-launch backward; "s" = a quarter of the batch
    "c2d256": ("CausalChillMask", (), "bfloat16", 8, 16, 4096, 256),
    "c2d256s": ("CausalChillMask", (), "bfloat16", 2, 16, 4096, 256),
}


def describe(name):
    m, a, dt, B, H, L, D = WORKLOADS[name]
    return f"{name}: {m}{a} fwd+bwd {dt} (B={B},H={H},L={L},D={D}), N(0,1) inputs, sm_scale=D^-0.5"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    return FALLBACK_BF16_TFLOPS, 1400.0, "fallback"


def unmasked_pairs(mask, L):
    """Visible (q, k) pairs per head: every built-in mask row is one contiguous key interval."""
    pos = torch.arange(L, dtype=torch.int64)
    lo, hi = type(mask).k_range_for_q(pos, L, mask.constargs)
    lo = torch.as_tensor(lo).expand(L)
    hi = torch.as_tensor(hi).expand(L)
    return int((hi - lo + 1).clamp(min=0).sum())


class ClockSampler:
    """nvidia-smi sampling of SM clock and throttle reasons (one sampler process per run, 20 ms period, started
    before the warm-up because it needs ~0.2 s to come up).  `window(tag)` is a context manager around a timed
    region; `summary(tag)` uses only the samples stamped inside the windows of that tag - if they are shorter
    than the sampling period, the samples taken under load during the whole run are used instead and the result
    says so."""

    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.idx = device_index
        self.proc = None
        self.windows = {}
        self.rows = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def window(self, tag):
        sampler = self

        class _W:
            def __enter__(self):
                self.t0 = time.time()

            def __exit__(self, *exc):
                sampler.windows.setdefault(tag, []).append((self.t0, time.time()))

        return _W()

    def stop(self):
        if self.proc is None or self.rows is not None:
            return
        time.sleep(0.1)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        import datetime

        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        self.rows = []
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                self.rows.append((ts, float(f[1]), float(f[2]), float(f[3]),
                                  [nm for nm, val in zip(names, f[5:9]) if val.lower().startswith("active")]))
            except ValueError:
                continue

    def summary(self, tag):
        self.stop()
        res = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        rows = self.rows or []
        wins = self.windows.get(tag, [])
        inside = [r for r in rows if any(t0 - 0.005 <= r[0] <= t1 + 0.005 for t0, t1 in wins)]
        where = f"{len(wins)} timed region(s)"
        if not inside:
            mx = max((r[3] for r in rows), default=0.0)
            inside = [r for r in rows if r[3] > 0.6 * mx]
            where = "all samples under load of the run (timed regions shorter than the 20 ms sampling period)"
        if inside:
            res = {"sm_mhz": statistics.median(r[1] for r in inside), "sm_min_mhz": min(r[1] for r in inside),
                   "sm_max_mhz": inside[-1][2], "power_w_max": max(r[3] for r in inside),
                   "reasons": sorted({nm for r in inside for nm in r[4]}), "samples": len(inside), "window": where}
        return res


def make_host_inputs(name, B, seed):
    _, _, dt, _, H, L, D = WORKLOADS[name]
    dtype = getattr(torch, dt)
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(B, H, L, D, generator=g, dtype=torch.float32).to(dtype) for _ in range(4)]


def config_dict(name, world):
    """The `config` object of the JSON line.  Both arms (this repository's kernels and the CPU reference) print
    exactly this for the same command line, so that the two lines can be matched on it."""
    _, _, _, B, H, L, _ = WORKLOADS[name]
    return {"workload": describe(name), "global_batch": B, "seq_len": L,
            "parallelism": f"{B * H} (batch, head) units split evenly over {world} GPU(s), no collective on the data path"}


def median_ms(block_ms, steps):
    return statistics.median(block_ms) / steps


def copy_bandwidth(dev, nbytes=256 << 20, reps=4):
    """Pinned-host <-> device copy rates with both directions running at once (two streams), GB/s per direction.
    Every rank calls it at the same time, so ranks that share a host show the contention they have in the
    end-to-end step."""
    h_in, h_out = torch.empty(nbytes, dtype=torch.uint8).pin_memory(), torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    d_in, d_out = torch.empty(nbytes, dtype=torch.uint8, device=dev), torch.empty(nbytes, dtype=torch.uint8, device=dev)
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(2)] for _ in range(2)]
    d_in.copy_(h_in, non_blocking=True), h_out.copy_(d_out, non_blocking=True)
    torch.cuda.synchronize()
    with torch.cuda.stream(s1):
        ev[0][0].record()
        for _ in range(reps):
            d_in.copy_(h_in, non_blocking=True)
        ev[0][1].record()
    with torch.cuda.stream(s2):
        ev[1][0].record()
        for _ in range(reps):
            h_out.copy_(d_out, non_blocking=True)
        ev[1][1].record()
    torch.cuda.synchronize()
    h2d = reps * nbytes / (ev[0][0].elapsed_time(ev[0][1]) * 1e-3) / 1e9
    d2h = reps * nbytes / (ev[1][0].elapsed_time(ev[1][1]) * 1e-3) / 1e9
    return h2d, d2h


def time_public_op(ca, mask, shape, dtype, dev, steps):
    """Milliseconds of one forward call and of one backward call through chill_attention() + autograd, with every
    allocation (outputs, delta, dQ scratch) inside the call - what a user of the operator pays."""
    g = torch.Generator(device=dev).manual_seed(5)
    q, k, v, do = (torch.randn(shape, generator=g, device=dev, dtype=torch.float32).to(dtype) for _ in range(4))
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    out = {}

    def fwd():
        return ca.chill_attention(q, k, v, mask=mask)

    o = fwd()

    def bwd():
        o.backward(do, retain_graph=True)

    for name, fn in (("fwd", fwd), ("bwd", bwd)):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        out[name] = e0.elapsed_time(e1) / steps
    return out


# --------------------------------------------------------------------------------- our arm
def run_ours(args):
    import ctypes as C

    import torch.distributed as dist

    import chill_attention as ca
    from chill_attention import _cabi
    from chill_attention import dist as cdist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.workload == "c5" and world > 1:
        block = run_c5_sharded(args, dev, world, rank, barrier)
        if rank == 0:
            line = {"metric": METRIC, "value": block["value"], "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
                    "warmup": args.warmup, "ms_per_step": block["ms_per_step"], "higher_is_better": True,
                    "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic: seeded N(0,1)",
                    "config": {"workload": describe("c5"), "global_batch": 1, "seq_len": WORKLOADS["c5"][5],
                               "parallelism": block["parallelism"]},
                    "c5_seq_sharded": block, "gpu_launches": block["gpu_launches"]}
            print(json.dumps(line), flush=True)
        barrier()
        dist.destroy_process_group()
        return

    mname, margs, dt, B, H, L, D = WORKLOADS[args.workload]
    dtype = getattr(torch, dt)
    mask = getattr(ca, mname)(*margs)
    lib = _cabi.load_library()
    functor = _cabi.BUILTIN_FUNCTOR_IDS[mask.cuda_functor]
    scale = D ** -0.5
    pairs = unmasked_pairs(mask, L)
    # The B x H (batch, head) units are independent; rank r takes a contiguous 1/world slice of them (strong
    # scaling: the problem stays (B, H, L, D) whatever the number of GPUs).  A rank's slice is laid out as
    # [units, 1, L, D]; with one GPU the tensors keep their (B, H, L, D) shape.
    u_lo, u_hi = cdist.shard_units(B * H, world, rank)
    units = u_hi - u_lo
    lshape = (B, H, L, D) if world == 1 else (units, 1, L, D)
    flops_fwd_job = 4.0 * B * H * D * pairs
    flops_step_job = 14.0 * B * H * D * pairs
    esz = torch.empty((), dtype=dtype).element_size()

    # ---- device-resident inputs (generated on the device: throughput run)
    g = torch.Generator(device=dev).manual_seed(20 + rank)
    q, k, v, do = (torch.randn(lshape, generator=g, device=dev, dtype=torch.float32).to(dtype) for _ in range(4))
    o = torch.empty_like(q)
    lse = torch.empty(lshape[:3], dtype=torch.float32, device=dev)
    delta = torch.empty(lshape[:3], dtype=torch.float32, device=dev)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    tf32 = _cabi.FLAG_ALLOW_TF32 if dtype == torch.float32 else 0  # what precision="tf32" sets for fp32 tensors
    shape = _cabi.make_shape(q, k, functor, margs, None, scale, flags=tf32)
    shape_dkdv = _cabi.make_shape(q, k, functor, margs, None, scale, flags=_cabi.FLAG_BWD_ONLY_DKDV | tf32)
    shape_dq = _cabi.make_shape(q, k, functor, margs, None, scale, flags=_cabi.FLAG_BWD_ONLY_DQ | tf32)
    bargs_dkdv = _cabi.backward_args(q, k, v, o, do, lse, delta, dq, dk, dv, shape_dkdv)
    bargs_dq = _cabi.backward_args(q, k, v, o, do, lse, delta, dq, dk, dv, shape_dq)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    # --bwd fused: chill_bwd gets the fp32 dQ scratch and runs its single-kernel form (what chill_attention()
    # does by default); --bwd split: the bitwise-reproducible two-kernel form (chill_attention.set_deterministic)
    dq_accum = None
    if args.bwd == "fused":
        nacc = lib.chill_bwd_dq_accum_bytes(C.byref(shape))
        if nacc:
            dq_accum = torch.empty(nacc // 4, dtype=torch.float32, device=dev)
    bargs_all = _cabi.backward_args(q, k, v, o, do, lse, delta, dq, dk, dv, shape, dq_accum)

    def run_fwd():
        _cabi.forward(lib, q, k, v, o, lse, shape)

    def run_delta():
        _cabi.check(lib, lib.chill_bwd_delta(C.byref(bargs_all), stream), "chill_bwd_delta")

    def run_bwd():
        _cabi.check(lib, lib.chill_bwd(C.byref(bargs_all), stream), "chill_bwd")

    def run_dkdv():
        _cabi.check(lib, lib.chill_bwd(C.byref(bargs_dkdv), stream), "chill_bwd(dkdv)")

    def run_dq():
        _cabi.check(lib, lib.chill_bwd(C.byref(bargs_dq), stream), "chill_bwd(dq)")

    wide = D == 256 and dtype in (torch.float16, torch.bfloat16)  # three launches behind one chill_bwd call
    if dq_accum is not None or wide:
        # "bwd" = zero-fill of the scratch + the fused kernel + the fp32 -> 16-bit conversion of dQ
        # (head dim 256: the dV, dK and dQ launches)
        parts = (("fwd", run_fwd), ("delta", run_delta), ("bwd", run_bwd))
        kflops = {"fwd": 4.0, "bwd": 10.0}
    else:
        parts = (("fwd", run_fwd), ("delta", run_delta), ("dkdv", run_dkdv), ("dq", run_dq))
        kflops = {"fwd": 4.0, "dkdv": 8.0, "dq": 6.0}
    kernels = tuple(name for name, _ in parts)

    def step_plain():
        # the path a caller runs: forward, delta, then chill_bwd
        run_fwd()
        run_delta()
        run_bwd()

    clk = ClockSampler(local)
    for _ in range(args.warmup):
        step_plain()
    barrier()

    def idle_gap():
        # A B200 under its 1000 W cap holds the maximum SM clock for the first ~50 ms of a dense kernel sequence and
        # then settles 15-20 % lower.  The contract's timed region (K = 20 steps of ~2 ms) is of the first kind; the
        # gap lets every repetition of it start from the same state.  The settled figure is reported beside it
        # (`sustained`).
        # Two untimed steps after the gap bring the clocks back up from idle before anything is timed.
        if args.block_gap_ms > 0:
            time.sleep(args.block_gap_ms * 1e-3)
            for _ in range(2):
                step_plain()
            torch.cuda.current_stream().synchronize()

    # The timed region: `blocks` repetitions of exactly `steps` steps, each bracketed by a barrier + synchronize and
    # timed with CUDA events on the launching stream; the reported step time is the median block (max over ranks).
    block_ms = []
    launches = 0
    t_host = 0.0
    for _ in range(args.blocks):
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        idle_gap()
        barrier()
        launches0 = lib.chill_launch_count()
        with clk.window("timed"):
            th0 = time.perf_counter()
            ev0.record()
            for i in range(args.steps):
                step_plain()
            ev1.record()
            barrier()
            t_host += time.perf_counter() - th0
        block_ms.append(ev0.elapsed_time(ev1))
        launches += lib.chill_launch_count() - launches0  # kernels launched inside the timed regions only
    # per-kernel durations: a second pass with the kernels launched one by one and an event between them
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(len(parts) + 1)] for _ in range(args.steps)]
    idle_gap()
    for i in range(args.steps):
        for j, (_, fn) in enumerate(parts):
            evs[i][j].record()
            fn()
        evs[i][len(parts)].record()
    barrier()
    per_kernel = {kn: sum(e[i].elapsed_time(e[i + 1]) for e in evs) / args.steps for i, kn in enumerate(kernels)}
    # the same step back to back for >= 0.8 s: the second half runs at the clocks the power cap settles on
    sustained_ms = 0.0
    if not args.no_sustained:
        n_half = max(args.steps, int(400.0 / max(statistics.median(block_ms) / args.steps, 1e-3)))
        es = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        idle_gap()
        barrier()
        for i in range(n_half):
            step_plain()
        es[0].record()
        torch.cuda.current_stream().synchronize()
        with clk.window("sustained"):
            for i in range(n_half):
                step_plain()
            es[1].record()
            barrier()
        sustained_ms = es[0].elapsed_time(es[1]) / n_half
    status = lib.chill_read_device_status()
    if status != 0:
        raise SystemExit(f"device status {status}: a kernel gave up on a bounded wait")
    uses_tc = lib.chill_bwd_uses_tensor_cores(C.byref(bargs_dq))

    # ---- the public operator (chill_attention + autograd, allocations inside) on this rank's shard and on a tiny shape
    op_ms = None
    if not args.no_op:
        big = time_public_op(ca, mask, lshape, dtype, dev, max(3, min(args.steps, 10)))
        tiny = time_public_op(ca, mask, (8, 4, 128, 128), torch.float16, dev, 50)
        op_ms = {"fwd": round(big["fwd"], 4), "bwd": round(big["bwd"], 4), "fwd_bwd": round(big["fwd"] + big["bwd"], 4),
                 "t128_fwd_us": round(tiny["fwd"] * 1e3, 1), "t128_bwd_us": round(tiny["bwd"] * 1e3, 1),
                 "note": "chill_attention() and .backward() as a user calls them in eager mode, outputs and scratch "
                         "allocated inside the call; t128 = (8, 4, 128, 128) fp16, one call each (the backward figure "
                         "includes autograd's engine and the accumulation into three .grad tensors)"}

    # ---- end to end through the public API with host buffers
    e2e = None
    if not args.no_e2e:
        hg = torch.Generator().manual_seed(20 + rank)
        host = [torch.randn(lshape, generator=hg, dtype=torch.float32).to(dtype).pin_memory() for _ in range(4)]
        out_host = [torch.empty(lshape, dtype=dtype).pin_memory() for _ in range(4)]

        from chill_attention.host import attention_fwd_bwd_host

        def e2e_step():
            # public host-buffer entry point: batch chunks stream through the GPU, copies in both
            # directions overlap the kernels (chill_attention/host.py)
            attention_fwd_bwd_host(host[0], host[1], host[2], host[3], mask, out=tuple(out_host))

        for _ in range(max(1, min(args.warmup, 3))):
            e2e_step()
        barrier()
        n_e2e = max(2, min(args.steps, 10))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n_e2e):
            e2e_step()
        e1.record()
        barrier()
        e2e_ms = e0.elapsed_time(e1) / n_e2e
        barrier()
        h2d_gbs, d2h_gbs = copy_bandwidth(dev)
        e2e = {"ms_per_step": e2e_ms, "bytes": 4 * units * L * D * esz, "h2d_gbs": h2d_gbs, "d2h_gbs": d2h_gbs}
        del host, out_host

    # ---- max over ranks (min for the copy rates)
    vec = block_ms + [per_kernel[k_] for k_ in kernels] + [sustained_ms, e2e["ms_per_step"] if e2e else 0.0]
    times = torch.tensor(vec, dtype=torch.float64, device=dev)
    rates = torch.tensor([e2e["h2d_gbs"], e2e["d2h_gbs"]] if e2e else [0.0, 0.0], dtype=torch.float64, device=dev)
    counts = torch.tensor([float(launches)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(rates, op=dist.ReduceOp.MIN)
        dist.all_reduce(counts, op=dist.ReduceOp.SUM)
    times = times.tolist()
    block_ms = times[:args.blocks]
    per_kernel = {kn: times[args.blocks + i] for i, kn in enumerate(kernels)}
    sustained_ms, e2e_ms = times[-2], times[-1]

    c5_block = None
    if world > 1 and args.workload == "c2" and not args.no_c5:
        c5_block = run_c5_sharded(args, dev, world, rank, barrier)

    if rank == 0:
        peak, peak_sustained, peak_src = measured_peaks()
        ms_per_step = median_ms(block_ms, args.steps)
        fwd_ms = per_kernel["fwd"]
        value = flops_step_job / (ms_per_step * 1e-3) / 1e12
        fwd_tflops = flops_fwd_job / (fwd_ms * 1e-3) / 1e12
        dom = max(kflops, key=lambda kn: per_kernel[kn])
        # the slowest rank's launch processes ceil(B*H / world) units
        units_max = -(-B * H // world)
        flops_launch = kflops[dom] * units_max * D * pairs
        achieved = flops_launch / (per_kernel[dom] * 1e-3) / 1e12
        wl = args.workload.rstrip("s")
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16" if dt == "bfloat16" else ("f16" if dt == "float16" else "f32"),
            "data": "synthetic: seeded N(0,1) q,k,v,dO of the workload's shape; no dataset is involved",
            "config": config_dict(args.workload, world),
            "details": {
                "units_per_gpu": units_max,
                "timing": f"{args.blocks} repetitions of {args.steps} steps, {args.block_gap_ms:.0f} ms idle before each, median "
                          "repetition; ms per repetition (max over ranks): " + ", ".join(f"{b:.3f}" for b in block_ms),
                "l2": "inputs+outputs per step and GPU (%.0f MB) exceed the 126 MB L2; no explicit flush"
                      % (8 * units_max * L * D * esz / 1e6),
                "tensor_core_path": bool(uses_tc == 1),
                "backward": ("three launches (dV, dK, dQ), 8 GEMMs per tile pair, bitwise reproducible" if wide
                             else "single kernel, 5 GEMMs per tile pair, dQ summed in fp32 scratch" if args.bwd == "fused"
                             else "two kernels (dK/dV, dQ), 7 GEMMs per tile pair, bitwise reproducible")},
            "fwd": {"tflops": round(fwd_tflops, 2), "ms": round(fwd_ms, 4),
                    "pct_of_measured_peak": round(100 * fwd_tflops / world / peak, 2),
                    "pct_of_nominal_peak": round(100 * fwd_tflops / world / NOMINAL_BF16_TFLOPS, 2)},
            "fwd_bwd": {"tflops": round(value, 2), "pct_of_measured_peak": round(100 * value / world / peak, 2),
                        "pct_of_nominal_peak": round(100 * value / world / NOMINAL_BF16_TFLOPS, 2)},
            "kernel_ms": {kn: round(per_kernel[kn], 4) for kn in kernels},
            "roofline": {"bound": "tensor", "kernel": dom, "achieved": round(achieved, 2), "peak": peak,
                         "unit": "TFLOP/s", "frac": round(achieved / peak, 4),
                         "traffic": (round(NCU_DRAM_BYTES_PER_UNIT[(wl, dom)] * units_max)
                                     if (wl, dom) in NCU_DRAM_BYTES_PER_UNIT else None),
                         "peak_source": f"{peak_src} cuBLAS bf16 burst (sustained {peak_sustained})",
                         "flops_per_launch": flops_launch},
            "gpu_launches": int(counts.item()),
            "clocks": clk.summary("timed"),
            "host_wall_ms_per_step": round(t_host * 1e3 / (args.steps * args.blocks), 4),
        }
        if sustained_ms > 0:
            sv = flops_step_job / (sustained_ms * 1e-3) / 1e12
            line["sustained"] = {"value": round(sv, 2), "unit": "TFLOP/s", "ms_per_step": round(sustained_ms, 4),
                                 "pct_of_measured_sustained_peak": round(100 * sv / world / peak_sustained, 2),
                                 "clocks": clk.summary("sustained"),
                                 "note": "the same step back to back for >= 0.8 s, second half timed: what the 1000 W "
                                         "power cap leaves; compared with the cuBLAS figure taken the same way"}
        if op_ms:
            line["op_ms_per_step"] = op_ms
        if e2e:
            moved = 2 * e2e["bytes"]  # this rank's bytes per step, both directions
            both = rates[0].item() + rates[1].item()
            line["e2e"] = {"value": round(flops_step_job / (e2e_ms * 1e-3) / 1e12, 3), "unit": "TFLOP/s",
                           "h2d_bytes_per_step": 4 * B * H * L * D * esz, "d2h_bytes_per_step": 4 * B * H * L * D * esz,
                           "ms_per_step": round(e2e_ms, 3),
                           "copy_roofline": {
                               "h2d_gbs": round(rates[0].item(), 1), "d2h_gbs": round(rates[1].item(), 1),
                               "achieved_gbs": round(moved / (e2e_ms * 1e-3) / 1e9, 1),
                               "frac": round(moved / (e2e_ms * 1e-3) / 1e9 / both, 3) if both > 0 else None,
                               "note": "pinned-host copies of 256 MB in both directions at once, measured on every rank "
                                       "at the same time (slowest rank shown); achieved = bytes one rank moves per "
                                       "step / step time"}}
        if c5_block is not None:
            line["c5_seq_sharded"] = c5_block
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(args.workload, budget_s=args.cpu_budget)
        line["triton_baseline"] = triton_baseline(args, world)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def triton_baseline(args, world):
    """The reference's own Triton kernels on this GPU, run in a subprocess (its package has this package's
    import name), when an unmodified copy of it is importable from baseline/_ref or $CHILL_REFERENCE_DIR."""
    if world != 1:
        return {"unavailable": "measured with one GPU only"}
    if args.no_triton:
        return {"unavailable": "skipped (--no-triton)"}
    ref_dir = reference_dir()
    if ref_dir is None:
        return {"unavailable": "no chill_attention package under baseline/_ref or $CHILL_REFERENCE_DIR (the reference's "
                               "pip install yields an empty package: its pyproject lists a py-module for a package directory)"}
    cmd = [sys.executable, os.path.abspath(__file__), "--impl", "triton", "--workload", args.workload, "--steps", "5", "--warmup", "2"]
    if args.triton_autotune:
        cmd.append("--triton-autotune")
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=args.triton_timeout)
    except subprocess.TimeoutExpired:
        return {"unavailable": f"reference Triton run exceeded {args.triton_timeout} s"}
    for ln in reversed(r.stdout.strip().splitlines()):
        try:
            d = json.loads(ln)
        except ValueError:
            continue
        if "results" in d:
            res = d["results"].get("default_tables", {})
            out = {"fwd": res.get("fwd"), "fwd_bwd": res.get("fwd_bwd"), "autotune": d["results"].get("autotune"),
                   "note": d.get("note")}
            return out
        if "unavailable" in d:
            return {"unavailable": d["unavailable"]}
    return {"unavailable": "reference Triton run failed: " + (r.stderr.strip().splitlines() or ["no output"])[-1][:300]}


def reference_dir():
    for cand in (os.environ.get("CHILL_REFERENCE_DIR"), os.path.join(ROOT, "baseline", "_ref")):
        if cand and os.path.isfile(os.path.join(cand, "chill_attention", "chill.py")):
            return cand
    return None


# ------------------------------------------------------------------- sequence-sharded leg
def run_c5_sharded(args, dev, world, rank, barrier):
    """The long sliding-window workload split by sequence position over the ranks (K/V halo over NCCL send/recv,
    dK/dV halo returned in fp32), timed like the main leg, followed by a parity check of this rank's rows on both
    sides of its shard boundaries against the fp64 CPU oracle.  Returns the block for the JSON line (rank 0) ."""
    import torch.distributed as dist

    import chill_attention as ca
    from chill_attention import _cabi
    from chill_attention import dist as cdist
    from oracle import attention_oracle as orc

    mname, margs, dt, B, H, L, D = WORKLOADS["c5"]
    assert L % world == 0
    mask = getattr(ca, mname)(*margs)
    dtype = getattr(torch, dt)
    lib = _cabi.load_library()
    Ls = L // world
    base = rank * Ls
    left, right = cdist.halo_sizes(mask, Ls)
    # every rank generates the whole sequence from the same seed (so that the oracle below can see the neighbours'
    # rows) and keeps its own slice for the timed part
    g = torch.Generator(device=dev).manual_seed(25)
    full = [torch.randn(B, H, L, D, generator=g, device=dev, dtype=torch.float32).to(dtype) for _ in range(4)]
    sl = slice(base, base + Ls)
    q = full[0][:, :, sl].contiguous().requires_grad_(True)
    kbuf = cdist.HaloBuffer(B, H, Ls, D, left, right, dtype, dev)
    vbuf = cdist.HaloBuffer(B, H, Ls, D, left, right, dtype, dev)
    kbuf.local.copy_(full[1][:, :, sl]), vbuf.local.copy_(full[2][:, :, sl])
    k, v = kbuf.local.requires_grad_(True), vbuf.local.requires_grad_(True)
    do = full[3][:, :, sl].contiguous()
    out = {}

    def step():
        q.grad = k.grad = v.grad = None
        o = cdist.sequence_sharded_attention(q, k, v, mask, L, halo_buffers=(kbuf, vbuf))
        o.backward(do)
        out["o"] = o

    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    block_ms = []
    launches0 = lib.chill_launch_count()
    steps = max(2, min(args.steps, 10))
    for _ in range(args.blocks):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if args.block_gap_ms > 0:
            time.sleep(args.block_gap_ms * 1e-3)  # every repetition starts from the same power state
        barrier()
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        barrier()
        block_ms.append(e0.elapsed_time(e1))
    launches = lib.chill_launch_count() - launches0
    status = lib.chill_read_device_status()
    if status != 0:
        raise SystemExit(f"device status {status}: a kernel gave up on a bounded wait")

    # ---- parity: 32-row windows at the shard's first rows (need the left halo), where boundary rows hand over to
    # interior rows, where the fp32-summed tail of dK/dV begins, and at the shard's last rows (dK/dV get the right
    # neighbour's contribution), two heads each
    torch.set_num_threads(max(1, (os.cpu_count() or 1) // world))
    o = out["o"].detach()
    lse = None  # the sharded operator returns O only; LSE is checked through dQ/dK/dV, which depend on it
    W = 32
    starts = sorted({base, base + left - W // 2, base + Ls - left - W // 2, base + Ls - W} if Ls >= 2 * left + W else {base, base + Ls - W})
    errs = {"o": 0.0, "dq": 0.0, "dk": 0.0, "dv": 0.0}
    for a in starts:
        a = max(base, min(a, base + Ls - W))
        b = a + W
        q1, k0, k1 = min(L, b + left), max(0, a - left), min(L, b + left + right)
        qp, kp = torch.arange(a, q1), torch.arange(k0, k1)
        md = orc.builtin_mask_dense(mname, margs, qp, kp)
        for h in (0, H - 1):
            qs, dos = (t[:, h:h + 1, a:q1].cpu().double() for t in (full[0], full[3]))
            ks, vs = (t[:, h:h + 1, k0:k1].cpu().double() for t in (full[1], full[2]))
            o_ref, _ = orc.attention_forward(md, qs, ks, vs, None, None, torch.float64, qp, kp, L)
            dq_ref, dk_ref, dv_ref = orc.attention_backward(md, qs, ks, vs, dos, None, None, torch.float64, qp, kp, L)
            la, lb = a - base, b - base
            errs["o"] = max(errs["o"], (o[:, h:h + 1, la:lb].cpu().double() - o_ref[:, :, :W]).abs().max().item())
            for nm, mine, ref in (("dq", q.grad[:, h:h + 1, la:lb], dq_ref[:, :, :W]),
                                  ("dk", k.grad[:, h:h + 1, la:lb], dk_ref[:, :, a - k0:b - k0]),
                                  ("dv", v.grad[:, h:h + 1, la:lb], dv_ref[:, :, a - k0:b - k0])):
                rel = ((mine.cpu().double() - ref).norm() / ref.norm().clamp(min=1e-30)).item()
                errs[nm] = max(errs[nm], rel)
    ev = torch.tensor(block_ms + [errs["o"], errs["dq"], errs["dk"], errs["dv"], float(launches)], dtype=torch.float64, device=dev)
    dist.all_reduce(ev, op=dist.ReduceOp.MAX)
    ev = ev.tolist()
    block_ms, (eo, edq, edk, edv, launches_max) = ev[:args.blocks], ev[args.blocks:]
    pairs = unmasked_pairs(mask, L)
    ms = median_ms(block_ms, steps)
    halo = 2 * B * H * left * D * q.element_size()
    # bars: O max-abs 2e-2 (bf16); gradients of a 32-row window relative Frobenius 2e-2 (twice the whole-tensor bar)
    ok = eo <= 2e-2 and max(edq, edk, edv) <= 2e-2
    del full
    return {
        "workload": describe("c5"), "scaling": "strong", "n_gpus": world, "steps": steps, "ms_per_step": round(ms, 4),
        "value": round(14.0 * B * H * D * pairs / (ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
        "halo_bytes": halo, "halo_grad_bytes": 2 * halo,
        "parallelism": f"sequence sharded over {world} GPUs ({Ls} positions each), {halo} B K/V halo per boundary via NCCL "
                       f"send/recv into the spare rows of the K/V buffers, dK/dV halo returned in fp32",
        "gpu_launches": int(launches_max) * world,
        "parity": {"o_max_abs": eo, "dq_rel": edq, "dk_boundary_rel": edk, "dv_boundary_rel": edv, "ok": bool(ok),
                   "checked": f"{len(starts)} windows of {W} rows x 2 heads per rank at shard start / boundary-interior "
                              f"hand-over / start of the fp32-summed tail / shard end, against the fp64 CPU oracle; LSE "
                              f"enters through the gradients"},
    }


# ------------------------------------------------------------------------------ CPU arm
def cpu_pass(name, n_units, seed=20):
    """fwd + bwd of `n_units` (batch, head) units of the workload with the CPU oracle. Returns seconds."""
    from oracle import attention_oracle as orc

    mname, margs, dt, B, H, L, D = WORKLOADS[name]
    g = torch.Generator().manual_seed(seed)
    dtype = getattr(torch, dt)
    q, k, v, do = (torch.randn(1, n_units, L, D, generator=g).to(dtype).float() for _ in range(4))
    t0 = time.perf_counter()
    if L <= 8192:
        pos = torch.arange(L)
        md = orc.builtin_mask_dense(mname, margs, pos, pos)
        for u in range(n_units):
            sl = slice(u, u + 1)
            orc.attention_forward(md, q[:, sl], k[:, sl], v[:, sl], dtype=torch.float32)
            orc.attention_backward(md, q[:, sl], k[:, sl], v[:, sl], do[:, sl], dtype=torch.float32)
    else:
        orc.banded_forward(mname, margs, q, k, v, dtype=torch.float32)
        orc.banded_backward(mname, margs, q, k, v, do, dtype=torch.float32)
    return time.perf_counter() - t0


def cpu_baseline(name, budget_s=15.0):
    import chill_attention as ca

    mname, margs, dt, B, H, L, D = WORKLOADS[name]
    mask = getattr(ca, mname)(*margs)
    pairs = unmasked_pairs(mask, L)
    t1 = cpu_pass(name, 1)
    units = max(1, min(B * H, int(budget_s / max(t1, 1e-3))))
    t = cpu_pass(name, units) if units > 1 else t1
    tflops = 14.0 * units * D * pairs / t / 1e12
    return {"value": round(tflops, 5), "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{units} of {B * H} (batch, head) units of the workload, fp32 dense-mask attention fwd + "
                      f"closed-form bwd (oracle/attention_oracle.py), {t:.2f} s",
            "seconds": round(t, 3), "units": units}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # torchrun exports OMP_NUM_THREADS=1 to its workers; the CPU arm is meant to use the host's cores
    torch.set_num_threads(os.cpu_count() or 1)
    import chill_attention as ca

    mname, margs, dt, B, H, L, D = WORKLOADS[args.workload]
    mask = getattr(ca, mname)(*margs)
    pairs = unmasked_pairs(mask, L)
    t1 = cpu_pass(args.workload, 1)
    # size a step so that warmup + steps stay within a few minutes
    units = max(1, min(B * H, int(args.cpu_budget / max(t1, 1e-3))))
    for _ in range(args.warmup):
        cpu_pass(args.workload, units)
    ts = [cpu_pass(args.workload, units) for _ in range(args.steps)]
    t = sum(ts) / len(ts)
    value = 14.0 * units * D * pairs / t / 1e12
    world = int(os.environ.get("WORLD_SIZE", "1"))
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 5), "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(t * 1e3, 2), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic: seeded N(0,1)",
        "config": config_dict(args.workload, world),
        "cpu_baseline": {"value": round(value, 5), "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"each step = {units} of {B * H} (batch, head) units, fp32 dense-mask attention "
                                   f"fwd + closed-form bwd on the host (the reference's CPU path restated in "
                                   f"oracle/attention_oracle.py; its Triton kernels have no timed CPU mode)"},
        "e2e": {"value": round(value, 5), "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_triton_reference(args):
    """Extra arm (not the driver's reference arm): the reference's own Triton kernels on this GPU,
    through its public API, if an unmodified copy of its package sits in baseline/_ref (git-ignored;
    its pip install produces an empty package because of `py-modules` in its pyproject.toml)."""
    ref_dir = reference_dir()
    if int(os.environ.get("RANK", "0")) != 0:
        return
    if ref_dir is None or not torch.cuda.is_available():
        print(json.dumps({"impl": "triton", "unavailable": "no chill_attention package under baseline/_ref or "
                                                           "$CHILL_REFERENCE_DIR, or no CUDA device"}))
        return
    sys.path.insert(0, ref_dir)
    import chill_attention as ref  # the reference, not this repository's package

    assert os.path.realpath(ref.__file__).startswith(os.path.realpath(ref_dir)), ref.__file__
    mname, margs, dt, B, H, L, D = WORKLOADS[args.workload]
    dtype = getattr(torch, dt)
    mask = getattr(ref, mname)(*margs)
    pos = torch.arange(L, dtype=torch.int64)
    pairs = {"FullChillMask": L * L, "CausalChillMask": L * (L + 1) // 2}.get(mname)
    if pairs is None:
        import importlib.util

        spec = importlib.util.spec_from_file_location("own_mask", os.path.join(ROOT, "chill-attention_b200", "chill_attention", "mask.py"))
        own = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(own)
        pairs = unmasked_pairs(getattr(own, mname)(*margs), L)
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(20)
    q, k, v, do = (torch.randn(B, H, L, D, generator=g, device=dev, dtype=torch.float32).to(dtype) for _ in range(4))
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    out = {}
    for autotune in ((False, True) if args.triton_autotune else (False,)):
        def fwd():
            with torch.no_grad():
                return ref.chill_attention(q, k, v, mask=mask, autotune=autotune)

        def fwd_bwd():
            q.grad = k.grad = v.grad = None
            ref.chill_attention(q, k, v, mask=mask, autotune=autotune).backward(do)

        res = {}
        for name, fn, flops in (("fwd", fwd, 4.0), ("fwd_bwd", fwd_bwd, 14.0)):
            for _ in range(max(args.warmup, 3)):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.steps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / args.steps
            res[name] = {"ms": round(ms, 4), "tflops": round(flops * B * H * D * pairs / (ms * 1e-3) / 1e12, 2)}
        out["autotune" if autotune else "default_tables"] = res
    print(json.dumps({"impl": "triton", "metric": METRIC, "unit": "TFLOP/s", "config": {"workload": describe(args.workload)},
                      "results": out, "note": "reference Triton kernels (triton %s) through chill_attention(), outputs allocated "
                      "and zero-filled by the reference inside the timed region" % __import__("triton").__version__}), flush=True)


def run_reference_shapes(args):
    """The shapes of the reference's own benchmark (benchmark/benchmark.py:25-35, 38-55, 73): five masks x
    {B8 H12 D64, B8 H4 D128} x T in linspace(128, 6000, 4), fp16, inputs N(0, 0.01); forward and backward
    milliseconds through the public op, one JSON line per case.  An aid for like-for-like comparison with the
    reference's published curves, not the reported metric."""
    sys.path.insert(0, os.path.join(ROOT, "chill-attention_b200"))
    import chill_attention as ca

    torch.cuda.set_device(0)
    masks = [ca.SlidingWindowChillMask(16, 16), ca.CausalChillMask(), ca.ChunkwiseChillMask(16, 8),
             ca.PrefixLMChillMask(128), ca.FullChillMask()]
    times = sorted({int(t) for t in torch.linspace(128, 6000, 4).tolist()})
    for mask in masks:
        for name, heads, dim in (("small", 12, 64), ("medium", 4, 128)):
            for T in times:
                g = torch.Generator(device="cuda").manual_seed(20)
                q, k, v = (torch.empty(8, heads, T, dim, device="cuda", dtype=torch.float16).normal_(0.0, 0.01, generator=g)
                           .requires_grad_() for _ in range(3))
                do = torch.randn(8, heads, T, dim, device="cuda", dtype=torch.float16, generator=g)

                def fwd():
                    return ca.chill_attention(q, k, v, mask=mask)

                o = fwd()

                def bwd():
                    o.backward(do, retain_graph=True)

                res = {}
                for what, fn in (("fwd", fwd), ("bwd", bwd)):
                    for _ in range(max(3, args.warmup)):
                        fn()
                    torch.cuda.synchronize()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for _ in range(args.steps):
                        fn()
                    e1.record()
                    torch.cuda.synchronize()
                    res[what] = e0.elapsed_time(e1) / args.steps
                    # the same call replayed from a CUDA graph (no host time per call), which is how the reference's
                    # script measures (benchmark/benchmark.py:263-264, triton.testing.do_bench_cudagraph)
                    res[what + "_graph"] = None
                    for attempt in range(0 if args.no_cuda_graph else 2):  # a process's first capture of a path can
                        try:                                                # meet one-time set-up: one more try
                            side = torch.cuda.Stream()
                            side.wait_stream(torch.cuda.current_stream())
                            with torch.cuda.stream(side):
                                fn()
                            torch.cuda.current_stream().wait_stream(side)
                            graph = torch.cuda.CUDAGraph()
                            n_in_graph = 10
                            with torch.cuda.graph(graph):
                                for _ in range(n_in_graph):
                                    fn()
                            graph.replay()
                            torch.cuda.synchronize()
                            e0.record()
                            for _ in range(max(1, args.steps // 2)):
                                graph.replay()
                            e1.record()
                            torch.cuda.synchronize()
                            res[what + "_graph"] = e0.elapsed_time(e1) / (max(1, args.steps // 2) * n_in_graph)
                            res.pop(what + "_graph_error", None)
                            del graph
                            break
                        except Exception as exc:  # noqa: BLE001 - reported in the line, the eager figures stand
                            res[what + "_graph_error"] = repr(exc)[:200]
                            torch.cuda.synchronize()
                pairs = unmasked_pairs(mask, T)
                print(json.dumps({"mask": str(mask), "shape": name, "batch": 8, "heads": heads, "dim": dim, "time": T,
                                  "dtype": "f16", "fwd_ms": round(res["fwd"], 4), "bwd_ms": round(res["bwd"], 4),
                                  "fwd_graph_ms": None if res["fwd_graph"] is None else round(res["fwd_graph"], 4),
                                  "bwd_graph_ms": None if res["bwd_graph"] is None else round(res["bwd_graph"], 4),
                                  **{k_: v_ for k_, v_ in res.items() if k_.endswith("_error")},
                                  "fwd_tflops": round(4.0 * 8 * heads * dim * pairs / res["fwd"] / 1e9, 1),
                                  "bwd_tflops": round(10.0 * 8 * heads * dim * pairs / res["bwd"] / 1e9, 1)}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=("ours", "reference", "triton"))
    ap.add_argument("--triton-autotune", action="store_true", help="--impl triton: also time autotune=True")
    ap.add_argument("--bwd", default="fused", choices=("fused", "split"), help="form of the backward pass")
    ap.add_argument("--reference-shapes", action="store_true",
                    help="time the shapes of the reference's own benchmark script instead of a workload")
    ap.add_argument("--no-cuda-graph", action="store_true", help="--reference-shapes: skip the CUDA-graph replay timings")
    ap.add_argument("--blocks", type=int, default=5, help="the K-step block is timed this many times; the median is reported")
    ap.add_argument("--block-gap-ms", type=float, default=300.0,
                    help="idle time before each timed repetition, so that each starts from the same power state")
    ap.add_argument("--no-sustained", action="store_true", help="skip the >= 0.8 s back-to-back region")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-op", action="store_true", help="skip the timing of the public operator (op_ms_per_step)")
    ap.add_argument("--no-c5", action="store_true", help="with --gpus > 1: skip the sequence-sharded c5 leg")
    ap.add_argument("--no-triton", action="store_true", help="skip the reference-Triton subprocess")
    ap.add_argument("--triton-timeout", type=float, default=300.0)
    ap.add_argument("--cpu-budget", type=float, default=12.0, help="seconds of CPU work per baseline sample")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.reference_shapes:
        run_reference_shapes(args)
    elif args.impl == "triton":
        run_triton_reference(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
