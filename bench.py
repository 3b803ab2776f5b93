#!/usr/bin/env python
"""Benchmark of the MoE expert-FFN path.

One "step" is one pass of one MoE layer over a batch of tokens, all experts resident in HBM:
router -> top-k -> batch union -> int4 x int8 gate/up + SwiGLU -> down -> routing-weighted combine.

    python bench.py --gpus 1 --steps K --warmup W            # this backend, configs[1]: M = 1 decode
    torchrun ... bench.py --gpus N --steps K --warmup W      # N > 1: configs[4] layer, batch 32, expert-parallel
    python bench.py --impl reference --steps K --warmup W    # the reference's CPU int4 path (oracle port)

Prints ONE JSON line (rank 0).  Timing: CUDA events on the stream the kernels are launched on, L2
flushed before every step (256 MiB written, then 256 MiB read so that the flush leaves no dirty
lines to write back; untimed), max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

# headline config: single decode layer, all experts resident
CFG = dict(hidden=6144, inter=2048, n_experts=256, k=8, n_shared=1, gs=32, norm_topk=True, routed_scale=2.5)
METRIC = "moe_expert_ffn_decode_tok_s"
UNIT = "tok/s"
N_TOKENS = 64            # distinct synthetic batches cycled through the steps
FLUSH_BYTES = 256 << 20  # > 126 MB L2
EP_BATCH = 32            # configs[4]: decode batch of the expert-parallel runs
ROUTER_SEED, SHARED_SEED, EXPERT_SEED0 = 1234, 4999, 5000
# DRAM traffic of one single-launch decode step from a profiler capture of that kernel
# (dram__bytes_read.sum + dram__bytes_write.sum): a recorded constant, not measured by this run.
RECORDED_STEP_TRAFFIC = {"bytes": 225.1e6, "source": "profiles/decode_step_kernel_m1.md (captured at 64 resident "
                         "experts: 220.4 MB; + 4.72 MB of router rows at 256)"}


def ep_workload_text(m_total: int, world: int) -> str:
    return (f"configs[4] MoE layer, expert-parallel: decode batch {m_total} fixed, hidden 6144, 256 routed experts "
            f"top-8 split {CFG['n_experts'] // world} per GPU + replicated shared expert, moe_inter 2048, int4 "
            "group-32, Zipf(1.1) selection bias")


def workload_text(m: int) -> str:
    return ("configs[1]: one MoE decode layer, hidden 6144, 256 experts top-8 + 1 shared, moe_inter 2048, "
            f"int4 group-32, M={m}, Zipf(1.1) selection bias, all experts resident")


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def algorithmic_bytes(n_union: float, m: int):
    """Bytes one step must move: (|U| + shared) experts, router weights, x in and out."""
    from peregrine_b200.synth import expert_bytes

    c = CFG
    we = expert_bytes(c["hidden"], c["inter"], c["gs"])
    ne = n_union + c["n_shared"]
    return ne * we + c["n_experts"] * c["hidden"] * 4 + 2 * m * c["hidden"] * 4, we


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int):
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
            "hw_power_brake": getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                try:
                    mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                except Exception:
                    mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            self._stop.wait(0.01)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unsampled"]}
        return {"sm_mhz": int(np.median(self.samples)), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# ----------------------------------------------------------------------------- CPU leg (oracle port)
def cpu_model_name() -> str:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("model name"):
                    return line.split(":", 1)[1].strip()
    except Exception:
        pass
    return "unknown"


def host_layer(seed: int, distinct: int):
    from peregrine_b200.synth import synth_layer

    c = CFG
    return synth_layer(seed, c["hidden"], c["inter"], c["n_experts"], c["k"], c["gs"], shared=True,
                       norm_topk=c["norm_topk"], routed_scale=c["routed_scale"], zipf=True,
                       distinct_experts=distinct)


def cpu_pass(layer, xs, m: int, threads: int, budget_s: float, max_steps: int = 4096):
    """Times the oracle's layer forward (the reference's CPU int4 path restated in C) on batches of m
    tokens until `budget_s` of CPU work has been spent.  Returns per-step seconds (list) and steps."""
    import oracle as po

    def ow(w):
        return po.Weight(w.q, w.scale, 4, w.gs, w.i_n, w.o_n)

    experts = [(ow(e.gate), ow(e.up), ow(e.down)) for e in layer.experts]
    shared = (ow(layer.shared.gate), ow(layer.shared.up), ow(layer.shared.down))
    c = CFG

    def one(x):
        return po.moe_forward(x, layer.router_w, layer.router_bias, experts, shared, x.shape[0], c["hidden"], c["k"],
                              c["norm_topk"], c["routed_scale"], threads=threads)

    nb = max(1, len(xs) // m)
    one(xs[0:m])  # warm-up (page in the weights touched, spin up the pool)
    n, spent, times = 0, 0.0, []
    while spent < budget_s and n < max_steps:
        x = xs[(n % nb) * m:(n % nb) * m + m]
        t0 = time.perf_counter()
        one(x)
        dt = time.perf_counter() - t0
        times.append(dt)
        spent += dt
        n += 1
    return times, n


def cpu_leg(m: int, threads: int, budget_s: float, max_steps: int):
    import oracle as po
    from peregrine_b200.synth import synth_tokens

    po.build()
    layer = host_layer(seed=1, distinct=32)
    xs = synth_tokens(2, max(N_TOKENS, 4 * m), CFG["hidden"])
    times, n = cpu_pass(layer, xs, m, threads, budget_s, max_steps)
    med = float(np.median(times))
    return {"value": m / med, "unit": UNIT, "cores": threads, "kind": "port",
            "simd": "avx2" if po.simd_tier() == 1 else "scalar", "cpu": cpu_model_name(),
            "host_cores": os.cpu_count(),
            "step_ms": {"min": min(times) * 1e3, "median": med * 1e3, "max": max(times) * 1e3},
            "sample": f"{n} steps of {m} decode token(s) of the same layer shape, median per-step time, "
                      "32 distinct expert blobs on the host"}, med, n


def run_reference(args, rank: int, world: int):
    """The reference's own CPU implementation of the path (oracle port), all host threads."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    # the same configuration as this backend's arm at this --gpus: M = 1 decode on one GPU, the
    # batch-32 layer of the expert-parallel runs otherwise (the CPU has no ranks: one host does it all)
    ep = args.gpus > 1
    m = (args.m if args.m > 1 else EP_BATCH) if ep else args.m
    base, med, n = cpu_leg(m, threads, budget_s=60.0, max_steps=args.steps)
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": n,
        "warmup": 1, "ms_per_step": med * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int4 x int8 -> int32 -> f32", "data": "synthetic",
        "config": {"workload": ep_workload_text(m, args.gpus) if ep else workload_text(m), "m": m},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- resident layer
def expert_of(e: int):
    """Expert e of the benchmark layer (e == n_experts: the shared expert): seeded per expert, so
    every rank and every world size sees the same weights."""
    from peregrine_b200.synth import synth_expert

    c = CFG
    seed = SHARED_SEED if e == c["n_experts"] else EXPERT_SEED0 + e
    return synth_expert(np.random.default_rng(seed), c["hidden"], c["inter"], c["gs"])


def router_of():
    from peregrine_b200.synth import zipf_bias

    c = CFG
    rng = np.random.default_rng(ROUTER_SEED)
    router_w = (rng.standard_normal((c["n_experts"], c["hidden"])).astype(np.float32) * np.float32(0.02))
    return router_w, zipf_bias(rng, c["n_experts"])


def resident_layer(dev: int, owned=None, rank: int = 0, world: int = 1):
    from peregrine_b200 import cuda
    from peregrine_b200.resident import upload_expert

    c = CFG
    router_w, bias = router_of()
    ml = cuda.MoeLayer(dev, c["hidden"], c["inter"], c["n_experts"], c["k"], c["norm_topk"], c["routed_scale"],
                       router_w, bias)
    if world > 1:
        ml.set_ep(rank, world)
    t0 = time.time()
    for e in (range(c["n_experts"]) if owned is None else owned):
        ml.set_expert(e, upload_expert(dev, expert_of(e), c["hidden"], c["inter"]))
    ml.set_shared(upload_expert(dev, expert_of(c["n_experts"]), c["hidden"], c["inter"]))
    return ml, bias, time.time() - t0


class Flusher:
    def __init__(self, torch, dev, stream):
        with torch.cuda.stream(stream):
            self.flush = torch.empty(FLUSH_BYTES, dtype=torch.uint8, device=dev)
            self.drain = torch.zeros(FLUSH_BYTES // 4, dtype=torch.float32, device=dev)

    def __call__(self):
        # 1. write 256 MiB: every line of the 126 MB L2 now belongs to the flush buffer;
        # 2. read another 256 MiB: the dirty lines left by the write are written back and replaced by
        #    clean lines, so the timed step starts with a cold L2 and pays for no write-backs of the flush.
        self.flush.zero_()
        self.drain.sum()


def timed_steps(torch, stream, flush, fn, steps, warmup):
    """fn(i) enqueues step i on `stream`.  Returns per-step ms (CUDA events on that stream)."""
    for i in range(warmup):
        with torch.cuda.stream(stream):
            flush()
            fn(i)
    stream.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for i in range(steps):
        with torch.cuda.stream(stream):
            flush()
            evs[i][0].record(stream)
            fn(i)
            evs[i][1].record(stream)
    stream.synchronize()
    return np.array([a.elapsed_time(b) for a, b in evs])


def overlapping_tokens(rng, n_batches: int, m: int, hidden: int, mix: float):
    """Batches whose tokens share a common direction: x = sqrt(mix) * c + sqrt(1 - mix) * n, c drawn per
    batch, n per token, both N(0, 1) — still N(0, 1) per element, but the tokens of a batch now agree
    on part of their top-k."""
    c = rng.standard_normal((n_batches, 1, hidden)).astype(np.float32)
    n = rng.standard_normal((n_batches, m, hidden)).astype(np.float32)
    return (np.float32(np.sqrt(mix)) * c + np.float32(np.sqrt(1.0 - mix)) * n).astype(np.float32)


def pair_overlap(idx: np.ndarray) -> float:
    """Mean over token pairs of |top-k(i) & top-k(j)| / k."""
    m, k = idx.shape
    if m < 2:
        return 1.0
    tot, cnt = 0.0, 0
    for i in range(m):
        for j in range(i + 1, m):
            tot += len(set(idx[i]) & set(idx[j])) / k
            cnt += 1
    return tot / cnt


def run_ours(args, rank: int, local_rank: int, world: int):
    import torch

    from peregrine_b200 import cuda
    from peregrine_b200.synth import expert_bytes, synth_tokens

    c = CFG
    m = args.m
    dev = local_rank
    torch.cuda.set_device(dev)
    if cuda.init([dev]) < 1:
        raise RuntimeError("bench: the CUDA backend could not initialise its device (no CPU fallback exists)")
    if args.experts != c["n_experts"]:
        c["n_experts"] = args.experts
    ml, zbias, t_up = resident_layer(dev)
    stream = torch.cuda.ExternalStream(cuda.lib().coli_cuda_stream(dev), device=dev)
    n_batches = N_TOKENS if m <= 64 else max(2, 4096 // m)  # large batches: a few distinct ones are enough
    xs_host = synth_tokens(99, n_batches * m, c["hidden"]).reshape(n_batches, m, c["hidden"])
    with torch.cuda.stream(stream):
        xs = torch.from_numpy(xs_host).cuda(dev)
        out = torch.empty((m, c["hidden"]), dtype=torch.float32, device=dev)
    flush = Flusher(torch, dev, stream)
    stream.synchronize()

    def step(i):
        ml.forward_dev(out.data_ptr(), xs[i % n_batches].data_ptr(), m)

    if args.profile_case:
        # a short run for profiler captures: a few steps of the chosen batch, nothing else
        ms = timed_steps(torch, stream, flush, step, max(args.steps, 1), max(args.warmup, 1))
        print(json.dumps({"profile_case": True, "m": m, "experts": c["n_experts"], "ms_per_step": float(ms.mean())}),
              flush=True)
        ml.free()
        cuda.shutdown()
        return

    n0 = cuda.kernel_launches()
    with ClockSampler(dev) as clocks:
        step_ms = timed_steps(torch, stream, flush, step, args.steps, args.warmup)
    launches = int(round((cuda.kernel_launches() - n0) * args.steps / (args.steps + args.warmup)))
    if cuda.last_device_error(dev) != 0:
        raise RuntimeError("bench: a kernel reported a device-side error")
    ms_step = float(step_ms.mean())
    value = m * 1e3 / ms_step
    unions = []
    for i in range(min(args.steps, 64)):
        with torch.cuda.stream(stream):
            step(i)
        unions.append(len(ml.last_routing(m)[3]))
    n_union = float(np.mean(unions))
    total_b, we = algorithmic_bytes(n_union, m)
    peak, peak_kind = measured_peaks()

    # ---- roofline of the dominant kernel.  One token: the whole step is ONE launch
    # (decode_step_kernel), timed by the events above (an empty pair of event records on this stream
    # costs ~2.5 us and is part of the figure).  Batches: per-launch events of a separate pass.
    if m == 1:
        empty = timed_steps(torch, stream, lambda: None, lambda i: None, 50, 3)
        achieved = total_b / (ms_step * 1e-3) / 1e9
        roofline = {
            "bound": "hbm", "kernel": "decode_step_kernel (routing, gate/up, down, combine of one token in one launch)",
            "achieved": achieved, "peak": peak, "peak_kind": f"{peak_kind} copy bandwidth", "unit": "GB/s",
            "frac": achieved / peak, "frac_of_8000": achieved / 8000.0,
            "launch_ms": ms_step, "empty_event_bracket_ms": float(np.median(empty)),
            "traffic": RECORDED_STEP_TRAFFIC["bytes"], "traffic_source": RECORDED_STEP_TRAFFIC["source"],
            "traffic_is_recorded_constant": True, "algorithmic_bytes": total_b,
            "kernel_timing": "CUDA events on the launching stream around the single launch of every timed step",
        }
    else:
        ml.set_profile(True)
        for i in range(min(args.steps, 200)):
            with torch.cuda.stream(stream):
                flush()
                step(i)
        stage_ms, ncalls = ml.profile()
        ml.set_profile(False)
        gemv_ms = (stage_ms["gemv_gateup"] + stage_ms["gemv_down"]) / max(ncalls, 1)
        gemv_b = (n_union + c["n_shared"]) * we
        achieved = gemv_b / (gemv_ms * 1e-3) / 1e9 if gemv_ms > 0 else 0.0
        roofline = {
            "bound": "hbm", "kernel": "gate/up + down launches of one step (tensor-core small-batch kernel)",
            "achieved": achieved, "peak": peak, "peak_kind": f"{peak_kind} copy bandwidth", "unit": "GB/s",
            "frac": achieved / peak, "frac_of_8000": achieved / 8000.0, "traffic": None, "algorithmic_bytes": gemv_b,
            "stage_ms": {k: v / max(ncalls, 1) for k, v in stage_ms.items()},
            "kernel_timing": "separate pass with CUDA events around every launch (brackets included)",
        }

    # ---- end to end through the host-pointer call (H2D of x and D2H of the result inside)
    e2e_steps = min(args.steps, 300)
    out_host = np.empty((m, c["hidden"]), np.float32)
    for i in range(3):
        ml.forward(xs_host[i % n_batches], out_host)
    ml.host_times(reset=True)
    e2e_t = 0.0
    for i in range(e2e_steps):
        with torch.cuda.stream(stream):
            flush()
        stream.synchronize()
        t0 = time.perf_counter()
        ml.forward(xs_host[i % n_batches], out_host)
        e2e_t += time.perf_counter() - t0
    host_us, _ = ml.host_times(reset=True)
    e2e = {"value": m * e2e_steps / e2e_t, "unit": UNIT, "h2d_bytes_per_step": m * c["hidden"] * 4,
           "d2h_bytes_per_step": m * c["hidden"] * 4, "steps": e2e_steps,
           "us_per_call": e2e_t / e2e_steps * 1e6,
           "host_us_inside_call": {k: round(v, 2) for k, v in host_us.items()},
           "call": "coli_cuda_moe_layer_forward (host x in, host out back, blocking)"}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int4 x int8 -> int32 -> f32", "data": "synthetic",
        "config": {"workload": workload_text(m), "m": m,
                   "l2": "flushed before every step, untimed: 256 MiB written, then 256 MiB read so no dirty lines remain",
                   "parallelism": "1 GPU", "mean_union": n_union, "upload_s": round(t_up, 1)},
        "hbm_gbs_whole_step": total_b / (ms_step * 1e-3) / 1e9,
        "hbm_frac_of_8000_whole_step": total_b / (ms_step * 1e-3) / 1e9 / 8000.0,
        "roofline": roofline, "e2e": e2e, "gpu_launches": launches, "clocks": clocks.summary(),
    }
    if m == 1 and not args.no_extras:
        line.update(extras_one_gpu(torch, cuda, ml, stream, flush, zbias, dev))
    if rank == 0 and not args.no_cpu:
        widths = sorted({min(os.cpu_count() or 1, 16), os.cpu_count() or 1})
        legs = [cpu_leg(m, t, budget_s=10.0, max_steps=4096)[0] for t in widths]
        line["cpu_baseline"] = legs[0]          # the reference's default worker count, min(cores, 16)
        line["cpu_baseline_all_cores"] = legs[-1]
    if rank == 0:
        print(json.dumps(line), flush=True)
    torch.cuda.synchronize()
    ml.free()
    cuda.shutdown()


def extras_one_gpu(torch, cuda, ml, stream, flush, zbias, dev):
    """The other single-GPU configurations on the same resident layer: configs[2] (M = 4, 8, 16 with
    overlapping picks), the batch-32 layer of configs[4] on one GPU, configs[3] (4096-token prefill
    with Dirichlet(0.5) expert popularity), and the measured int8 tensor peak."""
    from peregrine_b200.synth import expert_bytes, synth_tokens

    c = CFG
    peak, _ = measured_peaks()
    we = expert_bytes(c["hidden"], c["inter"], c["gs"])
    extra = {}
    rng = np.random.default_rng(31)

    def time_batches(xb_host, mm, steps, warm):
        with torch.cuda.stream(stream):
            xb = torch.from_numpy(xb_host).cuda(dev)
            ob = torch.empty((mm, c["hidden"]), dtype=torch.float32, device=dev)
        nb = xb_host.shape[0]
        ms = timed_steps(torch, stream, flush, lambda i: ml.forward_dev(ob.data_ptr(), xb[i % nb].data_ptr(), mm),
                         steps, warm)
        return float(ms.mean()), xb, ob

    # configs[2]: tokens of a step share 30-60 % of their top-8 (a common direction mixed into the tokens;
    # the mix is chosen per M from a few candidates by the overlap the router actually produces)
    small = []
    for mm in (4, 8, 16):
        best = None
        for mix in (0.0, 0.1, 0.2, 0.3, 0.45):
            xb_host = overlapping_tokens(rng, 16, mm, c["hidden"], mix)
            ov = []
            for b in range(4):
                ml.forward(xb_host[b])
                ov.append(pair_overlap(ml.last_routing(mm)[0]))
            ov = float(np.mean(ov))
            if best is None or abs(ov - 0.45) < abs(best[1] - 0.45):
                best = (mix, ov, xb_host)
        mix, ov, xb_host = best
        ms, xb, ob = time_batches(xb_host, mm, 60, 5)
        un = []
        for b in range(16):
            with torch.cuda.stream(stream):
                ml.forward_dev(ob.data_ptr(), xb[b].data_ptr(), mm)
            un.append(len(ml.last_routing(mm)[3]))
        u = float(np.mean(un))
        tb, _ = algorithmic_bytes(u, mm)
        small.append({"m": mm, "ms": ms, "tok_s": mm * 1e3 / ms, "union": u, "pair_overlap": ov, "mix": mix,
                      "gbs_whole_step": tb / (ms * 1e-3) / 1e9, "frac": tb / (ms * 1e-3) / 1e9 / peak,
                      "bytes_reused": (mm * c["k"] - u) * we})
        del xb, ob
    extra["small_batch"] = small
    # configs[4] layer at its decode batch on this one GPU: the base of the expert-parallel lines
    xb_host = synth_tokens(7, 8 * EP_BATCH, c["hidden"]).reshape(8, EP_BATCH, c["hidden"])
    ms32, xb, ob = time_batches(xb_host, EP_BATCH, 40, 5)
    extra["ep_batch32"] = {"value": EP_BATCH * 1e3 / ms32, "unit": UNIT, "ms_per_step": ms32, "m": EP_BATCH, "steps": 40}
    del xb, ob
    # configs[3]: one prefill chunk of 4096 tokens, expert popularity ~ Dirichlet(0.5) through the selection bias
    pm = 4096
    p = np.random.default_rng(17).dirichlet(np.full(c["n_experts"], 0.5))
    dbias = np.maximum(0.35 * (np.log(np.maximum(p, 1e-30)) - np.log(p.max())), -4.0).astype(np.float32)
    ml.set_bias(dbias)
    xp_host = synth_tokens(11, pm, c["hidden"]).reshape(1, pm, c["hidden"])
    pms, xp, op = time_batches(xp_host, pm, 5, 2)
    idx = ml.last_routing(pm)[0]
    counts = np.bincount(idx.reshape(-1), minlength=c["n_experts"]).astype(np.float64)
    ml.set_bias(zbias)
    pops = 2.0 * 3 * c["hidden"] * c["inter"] * pm * (c["k"] + 1)
    tops = pops / (pms * 1e-3) / 1e12
    probe = cuda.int8_peak_probe(dev, 8192, 20)
    extra["prefill_4096"] = {
        "value": pm * 1e3 / pms, "unit": UNIT, "ms_per_step": pms, "m": pm, "steps": 5, "int8_tops": tops,
        "int8_peak_measured_tops": probe, "frac_of_measured": tops / probe if probe > 0 else None,
        "frac_of_nominal": tops / 4500.0,
        "int8_peak_how": "bare tcgen05.mma kind::i8 128x256x32 loop, one CTA per SM, operands resident in shared memory",
        "expert_counts": {"max": float(counts.max()), "mean": float(counts.mean()), "zero": int((counts == 0).sum()),
                          "target": "Dirichlet(0.5) popularity through the selection bias"},
        "note": "group-32 format: every 32-element block dot is folded into fp32 on the CUDA cores in reference "
                "order, which bounds this kernel, not the tensor pipe"}
    del xp, op
    # configs[4], one-GPU point: the 8-layer subset of the stack, batch 32, 256 greedy steps
    st = stack_model()
    ids, secs, ds = stack_decode(torch, cuda, dev, st, stack_ids0())
    extra["stack_8layer"] = {
        "value": STACK["batch"] * STACK["steps"] / secs, "unit": UNIT, "seconds": secs, "batch": STACK["batch"],
        "steps": STACK["steps"], "layers": "3 dense (width 12288) + 5 MoE (256 experts top-8 + shared), hidden 6144, "
                                           "embedding, final norm, int4 lm_head (vocab 4096), greedy argmax",
        "distinct_ids": int(len(np.unique(ids))), "step_graphs": bool(ds.graphs),
        "timing": "CUDA events around the 256 steps (each a replay of the recorded step graph when step_graphs is "
                  "true); every step streams several GB of expert weights, far more than the L2 holds"}
    ds.free()
    return extra


STACK = dict(n_layers=8, first_dense=3, dense_inter=12288, vocab=4096, batch=EP_BATCH, steps=256, distinct=16)


def stack_model():
    """The 8-layer subset of the synthetic stack of configs[4] (3 dense layers of width 12288, 5 MoE
    layers as configs[1]); every MoE layer cycles 16 distinct expert blobs on the host, the device
    holds 256 separate copies per layer."""
    from peregrine_b200.stack import synth_stack

    c, s = CFG, STACK
    return synth_stack(seed=9, hidden=c["hidden"], inter=c["inter"], dense_inter=s["dense_inter"],
                       n_experts=c["n_experts"], k=c["k"], n_layers=s["n_layers"], first_dense=s["first_dense"],
                       vocab=s["vocab"], gs=c["gs"], distinct_experts=s["distinct"], scale_std=0.02 / 64)


def stack_decode(torch, cuda, dev, st, ids0, ep=None, meet=None):
    """256 greedy steps of the stack for the tokens `ids0`; returns (ids [steps, batch], seconds, stack).
    `meet` (expert parallel): a host barrier of the ranks; building the stack takes a different time
    on every rank and the ranks must enter a step within the device-side wait limit of each other."""
    from peregrine_b200.stack import DeviceStack

    s = STACK
    ds = DeviceStack(dev, st, len(ids0), s["steps"], ep=ep, repeats="clone")
    stream = torch.cuda.ExternalStream(cuda.lib().coli_cuda_stream(dev), device=dev)
    if meet:
        meet()
    ds.start(ids0)
    ds.run(4)  # warm-up steps (overwritten by the timed run); on one GPU this also records the step graphs
    stream.synchronize()
    if meet:
        meet()
    ds.start(ids0)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e0.record(stream)
        ds.run(s["steps"])
        e1.record(stream)
    stream.synchronize()
    if cuda.last_device_error(dev) != 0:
        raise RuntimeError("bench: a kernel reported a device-side error during the stack decode")
    return ds.result(s["steps"]), e0.elapsed_time(e1) * 1e-3, ds


def stack_ids0():
    return (np.arange(STACK["batch"], dtype=np.int32) * 97 + 5) % STACK["vocab"]


def run_ep(args, rank: int, local_rank: int, world: int):
    """N > 1: one MoE decode layer of configs[4], batch 32, routed experts split over the ranks
    (256/N per GPU), router and shared expert replicated, tokens data-parallel; the exchange is the
    backend's own peer-memory kernels (int8 rows out, fp32 rows back).  Strong scaling: the batch is
    fixed.  After the timed region rank 0 runs the same batch through a single-GPU layer holding all
    experts: every rank's output rows are compared with it bit for bit (`parity_ok`), and its time
    is the like-for-like one-GPU base (`base_n1`)."""
    import torch
    import torch.distributed as dist

    from peregrine_b200 import cuda
    from peregrine_b200.ep import EpLayerRunner, EpWorkspace, owned_range
    from peregrine_b200.synth import synth_tokens

    c = CFG
    dev = local_rank
    torch.cuda.set_device(dev)
    # libraries (the collective library's version banner) write to file descriptor 1: keep the real
    # stdout for the one JSON line and send everything else to stderr
    sys.stdout.flush()
    json_out = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    dist.init_process_group("nccl", device_id=torch.device("cuda", dev))
    if cuda.init([dev]) < 1:
        raise RuntimeError("bench: the CUDA backend could not initialise its device (no CPU fallback exists)")
    m_total = args.m if args.m > 1 else EP_BATCH
    m_local = m_total // world
    ml, _, t_up = resident_layer(dev, owned=owned_range(c["n_experts"], rank, world), rank=rank, world=world)
    ws = EpWorkspace(dev, rank, world, m_total, c["hidden"], c["k"])
    ws.connect()
    run = EpLayerRunner(ml, ws)
    stream = run.stream
    xs_full = synth_tokens(99, N_TOKENS * m_total, c["hidden"]).reshape(N_TOKENS, m_total, c["hidden"])
    xs_host = np.ascontiguousarray(xs_full[:, rank * m_local:(rank + 1) * m_local, :])
    with torch.cuda.stream(stream):
        xs = torch.from_numpy(xs_host).cuda(dev)
        x_pin = torch.from_numpy(xs_host).pin_memory()
        x_dev = torch.empty((m_local, c["hidden"]), dtype=torch.float32, device=dev)
    flush = Flusher(torch, dev, stream)
    stream.synchronize()

    def step(i):
        run.forward(xs[i % N_TOKENS])

    dist.barrier()
    torch.cuda.synchronize()
    n0 = cuda.kernel_launches()
    with ClockSampler(dev) as clocks:
        step_ms = timed_steps(torch, stream, flush, step, args.steps, args.warmup)
    torch.cuda.synchronize()
    dist.barrier()
    launches = int(round((cuda.kernel_launches() - n0) * args.steps / (args.steps + args.warmup)))
    total_ms = float(step_ms.sum())
    t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms = float(t.item())
    if cuda.last_device_error(dev) != 0:
        raise RuntimeError("bench: a kernel reported a device-side error")
    value = m_total * args.steps / (total_ms * 1e-3)
    n_union = len(ml.last_routing(m_total)[3])

    # ---- phase times: the four phases bracketed by events in a separate pass (each phase waits for
    # the other ranks' previous phase, so a phase's time includes what it waits for)
    ph_names = ["route_publish", "plan_dispatch", "experts_return", "combine"]
    ph = np.zeros(4)
    reps = min(args.steps, 100)
    for i in range(reps):
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
        with torch.cuda.stream(stream):
            flush()
            evs[0].record(stream)
            run.route(xs[i % N_TOKENS])
            evs[1].record(stream)
            run.dispatch()
            evs[2].record(stream)
            run.experts()
            evs[3].record(stream)
            run.finish()
            evs[4].record(stream)
        stream.synchronize()
        ph += np.array([evs[j].elapsed_time(evs[j + 1]) for j in range(4)])
    ph /= reps
    pt = torch.tensor(ph, dtype=torch.float64, device=dev)
    dist.all_reduce(pt, op=dist.ReduceOp.MAX)
    phase_ms = {n: float(v) for n, v in zip(ph_names, pt.tolist())}

    # ---- end to end: pinned host tokens in, home-token outputs back to the host, every step
    e2e_steps = min(args.steps, 200)
    e2e_t = 0.0
    for i in range(e2e_steps):
        with torch.cuda.stream(stream):
            flush()
        stream.synchronize()
        dist.barrier()
        t0 = time.perf_counter()
        with torch.cuda.stream(stream):
            x_dev.copy_(x_pin[i % N_TOKENS], non_blocking=True)
            host = run.forward(x_dev).to("cpu", non_blocking=False)
        e2e_t += time.perf_counter() - t0
        del host
    t = torch.tensor([e2e_t], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_t = float(t.item())

    # ---- parity and the one-GPU base: one check batch through the expert-parallel layer, gathered on
    # rank 0, against a single-GPU layer with all experts on rank 0's device
    check = 5
    with torch.cuda.stream(stream):
        mine = run.forward(xs[check]).clone()
    stream.synchronize()
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    parity_ok, base_n1 = None, None
    if rank == 0:
        ep_out = torch.cat(gathered, 0).cpu().numpy()
        full, _, _ = resident_layer(dev)
        with torch.cuda.stream(stream):
            xb = torch.from_numpy(xs_full).cuda(dev)
            ob = torch.empty((m_total, c["hidden"]), dtype=torch.float32, device=dev)
            full.forward_dev(ob.data_ptr(), xb[check].data_ptr(), m_total)
        stream.synchronize()
        want = ob.cpu().numpy()
        parity_ok = bool(np.array_equal(ep_out.view(np.uint32), want.view(np.uint32)))
        ms1 = timed_steps(torch, stream, flush,
                          lambda i: full.forward_dev(ob.data_ptr(), xb[i % N_TOKENS].data_ptr(), m_total), 40, 5)
        base_n1 = {"value": m_total * 1e3 / float(ms1.mean()), "unit": UNIT, "ms_per_step": float(ms1.mean()),
                   "what": "the same batch through a single-GPU layer holding all 256 experts, same run, rank 0"}
        full.free()
        del xb, ob
    # ---- the 8-layer stack, expert-parallel: every rank decodes its home tokens for 256 greedy steps;
    # the ids of all ranks must equal the ids of the same stack on one GPU (rank 0 runs that too)
    stack = None
    if m_total == STACK["batch"] and not args.no_extras:
        st = stack_model()
        ids0 = stack_ids0()
        ids_l, secs, ds = stack_decode(torch, cuda, dev, st, ids0[rank * m_local:(rank + 1) * m_local], ep=ws,
                                       meet=dist.barrier)
        tsec = torch.tensor([secs], dtype=torch.float64, device=dev)
        dist.all_reduce(tsec, op=dist.ReduceOp.MAX)
        ids_t = torch.from_numpy(np.ascontiguousarray(ids_l)).to(dev)
        parts = [torch.empty_like(ids_t) for _ in range(world)]
        dist.all_gather(parts, ids_t)
        ds.free()
        if rank == 0:
            ep_ids = torch.cat(parts, 1).cpu().numpy()
            one_ids, one_secs, ds1 = stack_decode(torch, cuda, dev, st, ids0)
            ds1.free()
            stack = {"value": STACK["batch"] * STACK["steps"] / float(tsec.item()), "unit": UNIT,
                     "seconds": float(tsec.item()), "batch": STACK["batch"], "steps": STACK["steps"], "layers": 8,
                     "ids_match_one_gpu": bool(np.array_equal(ep_ids, one_ids)),
                     "base_n1": {"value": STACK["batch"] * STACK["steps"] / one_secs, "seconds": one_secs},
                     "speedup_vs_n1": one_secs / float(tsec.item())}
            if not stack["ids_match_one_gpu"]:
                parity_ok = False
    total_b, _ = algorithmic_bytes(n_union, m_total)
    peak, peak_kind = measured_peaks()
    step_s = total_ms / args.steps * 1e-3
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int4 x int8 -> int32 -> f32", "data": "synthetic",
        "config": {"workload": ep_workload_text(m_total, world), "m": m_total,
                   "parallelism": f"ep{world}: home-token routing, picks published to all ranks, int8 rows to the "
                                  "owners and fp32 rows back through peer memory (own kernels, NVLink)",
                   "l2": "flushed before every step, untimed: 256 MiB written, then 256 MiB read",
                   "union": n_union, "upload_s": round(t_up, 1),
                   "note": "the N=1 line of this bench is configs[1] (M=1); base_n1 below is this workload on one GPU"},
        "parity_ok": parity_ok, "base_n1": base_n1,
        "ep_efficiency": (value / (world * base_n1["value"])) if base_n1 else None,
        "ep_speedup_vs_n1": (value / base_n1["value"]) if base_n1 else None,
        "phase_ms": phase_ms, "stack_8layer": stack,
        "roofline": {"bound": "hbm", "kernel": "whole layer step (all ranks)", "achieved": total_b / step_s / 1e9,
                     "peak": peak * world, "peak_kind": f"{peak_kind} copy bandwidth x {world} GPUs", "unit": "GB/s",
                     "frac": total_b / step_s / 1e9 / (peak * world), "traffic": None,
                     "algorithmic_bytes": total_b},
        "e2e": {"value": m_total * e2e_steps / e2e_t, "unit": UNIT, "h2d_bytes_per_step": m_local * c["hidden"] * 4,
                "d2h_bytes_per_step": m_local * c["hidden"] * 4, "steps": e2e_steps,
                "call": "EpLayerRunner.forward on this rank's home tokens (pinned host in, host out)"},
        "gpu_launches": launches, "clocks": clocks.summary(),
    }
    if rank == 0:
        print(json.dumps(line), file=json_out, flush=True)
        if parity_ok is False:
            print("bench: the expert-parallel output differs from the single-GPU layer", file=sys.stderr, flush=True)
    # teardown order matters: the process group goes first, then torch's tensors, and the backend
    # (which owns the stream and the exchange block) last
    ok_t = torch.tensor([0 if parity_ok is False else 1], device=dev)
    dist.broadcast(ok_t, 0)
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()
    del run, xs, x_dev, x_pin, flush
    torch.cuda.synchronize()
    ws.free()
    ml.free()
    cuda.shutdown()
    if int(ok_t.item()) == 0:
        sys.exit(1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--m", type=int, default=1, help="tokens per step (decode batch)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extras", action="store_true", help="N = 1: skip the other configurations")
    ap.add_argument("--profile-case", action="store_true",
                    help="profiler captures: only the timed steps of the chosen --m / --experts, no other legs")
    ap.add_argument("--experts", type=int, default=CFG["n_experts"],
                    help="routed experts resident (smaller values are for profiler captures only)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    args.warmup = max(args.warmup, 3)
    CFG["n_experts"] = args.experts
    if args.impl == "reference":
        run_reference(args, rank, world)
    elif world > 1:
        run_ep(args, rank, local_rank, world)
    else:
        run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
