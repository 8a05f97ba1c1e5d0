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

Multi-GPU (torchrun, one rank per GPU): every rank runs the workload on its own shard of the
batch x head units - no data-path collective; per-GPU work is fixed ("weak").  Workload c5
with --gpus > 1 is sequence-sharded instead (K/V halo over NCCL send/recv).

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
# dram__bytes_read.sum + dram__bytes_write.sum per (batch, head) unit from the ncu capture summarised in
# profiles/c2s_causal_bf16_kernels_ncu.md (causal bf16 L=4096 D=128, 32 units per launch); traffic grows in
# proportion to the units a launch processes, so a full launch = per-unit figure x B x H.
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
    # fp32 tensors with precision="tf32": forward on the TF32 tensor cores, backward in IEEE fp32 on the generic
    # kernels (seconds per step: use --steps 2); the forward figure is the one of interest
    "c2f32": ("CausalChillMask", (), "float32", 2, 16, 4096, 128),
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
    """nvidia-smi sampling of SM clock and throttle reasons.  The sampler process is started before the
    warm-up (it needs ~0.2 s to come up); `begin()` / `end()` bracket the timed region and only samples
    stamped inside it are used - if the region is shorter than the sampling period, the samples taken under
    load since the warm-up started are used instead and the result says so."""

    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.idx = device_index
        self.proc = None
        self.t0 = self.t1 = None
        self.result = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def begin(self):
        self.t0 = time.time()

    def end(self):
        self.t1 = time.time()

    def __enter__(self):
        self.begin()
        return self

    def __exit__(self, *exc):
        self.end()
        if self.proc is None:
            return
        time.sleep(0.12)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        import datetime

        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        rows = []
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                rows.append((ts, float(f[1]), float(f[2]), [nm for nm, val in zip(names, f[5:9]) if val.lower().startswith("active")]))
            except ValueError:
                continue
        inside = [r for r in rows if self.t0 - 0.02 <= r[0] <= self.t1 + 0.02]
        window = "timed region"
        if not inside:
            mx = max((r[1] for r in rows), default=0.0)
            inside = [r for r in rows if r[1] > 0.5 * mx]
            window = "warm-up + timed region (timed region shorter than the 50 ms sampling period)"
        if inside:
            self.result = {"sm_mhz": statistics.median(r[1] for r in inside), "sm_max_mhz": inside[-1][2],
                           "reasons": sorted({nm for r in inside for nm in r[3]}), "samples": len(inside), "window": window}


def make_host_inputs(name, B, seed):
    _, _, dt, _, H, L, D = WORKLOADS[name]
    dtype = getattr(torch, dt)
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(B, H, L, D, generator=g, dtype=torch.float32).to(dtype) for _ in range(4)]


# --------------------------------------------------------------------------------- our arm
def run_ours(args):
    import torch.distributed as dist

    import chill_attention as ca
    from chill_attention import _cabi

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if args.workload == "c5" and world > 1:
        from chill_attention import dist as cdist  # sequence-sharded path

        return cdist.bench_sequence_sharded(args, WORKLOADS["c5"], METRIC)

    mname, margs, dt, B, H, L, D = WORKLOADS[args.workload]
    dtype = getattr(torch, dt)
    mask = getattr(ca, mname)(*margs)
    lib = _cabi.load_library()
    functor = _cabi.BUILTIN_FUNCTOR_IDS[mask.cuda_functor]
    scale = D ** -0.5
    pairs = unmasked_pairs(mask, L)
    flops_fwd = 4.0 * B * H * D * pairs
    flops_step = 14.0 * B * H * D * pairs

    # ---- device-resident inputs (generated on the device: throughput run)
    g = torch.Generator(device=dev).manual_seed(20 + rank)
    q, k, v, do = (torch.randn(B, H, L, D, generator=g, device=dev, dtype=torch.float32).to(dtype) for _ in range(4))
    o = torch.empty_like(q)
    lse = torch.empty(B, H, L, dtype=torch.float32, device=dev)
    delta = torch.empty(B, H, L, dtype=torch.float32, device=dev)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    tf32 = _cabi.FLAG_ALLOW_TF32 if dtype == torch.float32 else 0  # what precision="tf32" sets for fp32 tensors
    shape = _cabi.make_shape(q, k, functor, margs, None, scale, flags=tf32)
    shape_dkdv = _cabi.make_shape(q, k, functor, margs, None, scale, flags=_cabi.FLAG_BWD_ONLY_DKDV | tf32)
    shape_dq = _cabi.make_shape(q, k, functor, margs, None, scale, flags=_cabi.FLAG_BWD_ONLY_DQ | tf32)
    import ctypes as C

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

    if dq_accum is not None:
        # "bwd" = zero-fill of the scratch + the fused kernel + the fp32 -> 16-bit conversion of dQ
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

    def step(events):
        for i, (_, fn) in enumerate(parts):
            events[i].record()
            fn()
        events[len(parts)].record()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    clk = ClockSampler(local)
    for _ in range(args.warmup):
        step_plain()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with clk:
        barrier()
        t_host0 = time.perf_counter()
        ev0.record()
        for i in range(args.steps):
            step_plain()
        ev1.record()
        barrier()
        t_host1 = time.perf_counter()
    total_ms = ev0.elapsed_time(ev1)
    # per-kernel durations: a second pass with the kernels launched one by one and an event between them
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(len(parts) + 1)] for _ in range(args.steps)]
    for i in range(args.steps):
        step(evs[i])
    barrier()
    per_kernel = {kn: sum(e[i].elapsed_time(e[i + 1]) for e in evs) / args.steps for i, kn in enumerate(kernels)}
    fwd_ms = per_kernel["fwd"]
    status = lib.chill_read_device_status()
    if status != 0:
        raise SystemExit(f"device status {status}: a kernel gave up on a bounded wait")
    uses_tc = lib.chill_bwd_uses_tensor_cores(C.byref(bargs_dq))

    # ---- end to end through the public API with host buffers
    e2e = None
    if not args.no_e2e:
        host = [t.pin_memory() for t in make_host_inputs(args.workload, B, 20 + rank)]
        out_host = [torch.empty(B, H, L, D, dtype=dtype).pin_memory() for _ in range(4)]
        dq_, dk_, dv_ = None, None, None

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
        esz = q.element_size()
        e2e = {"ms_per_step": e2e_ms, "h2d": 4 * B * H * L * D * esz, "d2h": 4 * B * H * L * D * esz}

    # ---- max over ranks
    times = torch.tensor([total_ms, fwd_ms, e2e["ms_per_step"] if e2e else 0.0] + [per_kernel[k_] for k_ in kernels],
                         dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    total_ms, fwd_ms, e2e_ms = times[0].item(), times[1].item(), times[2].item()
    per_kernel = {kn: times[3 + i].item() for i, kn in enumerate(kernels)}

    if rank == 0:
        peak, peak_sustained, peak_src = measured_peaks()
        ms_per_step = total_ms / args.steps
        value = world * flops_step / (ms_per_step * 1e-3) / 1e12
        fwd_tflops = world * flops_fwd / (fwd_ms * 1e-3) / 1e12
        dom = max(kflops, key=lambda kn: per_kernel[kn])
        achieved = kflops[dom] * B * H * D * pairs / (per_kernel[dom] * 1e-3) / 1e12
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if dt == "bfloat16" else ("f16" if dt == "float16" else "f32"),
            "data": "synthetic: seeded N(0,1) q,k,v,dO of the workload's shape; no dataset is involved",
            "config": {"workload": describe(args.workload), "global_batch": B * world, "seq_len": L,
                       "parallelism": f"batch x head units sharded over {world} GPU(s), no collective",
                       "l2": "inputs+outputs per step (%.0f MB) exceed the 126 MB L2; no explicit flush"
                             % (8 * B * H * L * D * q.element_size() / 1e6),
                       "tensor_core_path": bool(uses_tc == 1),
                       "backward": "single kernel, 5 GEMMs per tile pair, dQ summed in fp32 scratch" if dq_accum is not None
                                   else "two kernels (dK/dV, dQ), 7 GEMMs per tile pair, bitwise reproducible"},
            "fwd": {"tflops": round(fwd_tflops, 2), "ms": round(fwd_ms, 4),
                    "pct_of_measured_peak": round(100 * fwd_tflops / world / peak, 2),
                    "pct_of_nominal_peak": round(100 * fwd_tflops / world / NOMINAL_BF16_TFLOPS, 2)},
            "fwd_bwd": {"tflops": round(value, 2), "pct_of_measured_peak": round(100 * value / world / peak, 2),
                        "pct_of_nominal_peak": round(100 * value / world / NOMINAL_BF16_TFLOPS, 2)},
            "kernel_ms": {kn: round(per_kernel[kn], 4) for kn in kernels},
            "roofline": {"bound": "tensor", "kernel": dom, "achieved": round(achieved, 2), "peak": peak,
                         "unit": "TFLOP/s", "frac": round(achieved / peak, 4),
                         "traffic": (round(NCU_DRAM_BYTES_PER_UNIT[(args.workload.rstrip("s"), dom)] * B * H)
                                     if (args.workload.rstrip("s"), dom) in NCU_DRAM_BYTES_PER_UNIT else None),
                         "peak_source": f"{peak_src} cuBLAS bf16 burst (sustained {peak_sustained})",
                         "flops_per_launch": kflops[dom] * B * H * D * pairs},
            "gpu_launches": 4 * args.steps,
            "clocks": clk.result,
            "host_wall_ms_per_step": round((t_host1 - t_host0) * 1e3 / args.steps, 4),
        }
        if e2e:
            line["e2e"] = {"value": round(world * flops_step / (e2e_ms * 1e-3) / 1e12, 3), "unit": "TFLOP/s",
                           "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"],
                           "ms_per_step": round(e2e_ms, 3)}
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(args.workload, budget_s=args.cpu_budget)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


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
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic: seeded N(0,1)",
        "config": {"workload": describe(args.workload), "global_batch": B, "seq_len": L,
                   "parallelism": "host cores only (rank 0)"},
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
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if int(os.environ.get("RANK", "0")) != 0:
        return
    if not os.path.isdir(os.path.join(ref_dir, "chill_attention")) or not torch.cuda.is_available():
        print(json.dumps({"impl": "triton", "unavailable": "baseline/_ref/chill_attention or CUDA device not present"}))
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
                pairs = unmasked_pairs(mask, T)
                print(json.dumps({"mask": str(mask), "shape": name, "batch": 8, "heads": heads, "dim": dim, "time": T,
                                  "dtype": "f16", "fwd_ms": round(res["fwd"], 4), "bwd_ms": round(res["bwd"], 4),
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
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
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
