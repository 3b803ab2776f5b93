#!/usr/bin/env python
"""Benchmark of the MoE expert-FFN decode path (the headline config: one decode layer).

One "step" is one decode pass of one MoE layer over M tokens (default M = 1):
router -> top-k -> batch union -> int4 x int8 gate/up + SwiGLU -> down ->
routing-weighted combine, all experts resident in HBM.

    python bench.py --gpus 1 --steps K --warmup W          # this backend
    python bench.py --impl reference --steps K --warmup W  # the reference's CPU int4 path (oracle port)

Prints ONE JSON line (rank 0).  Timing: CUDA events on the stream the kernels
are launched on, L2 flushed before every step (256 MiB written, then 256 MiB
read so that the flush leaves no dirty lines to write back; untimed), max over ranks.
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
N_TOKENS = 64           # distinct synthetic tokens cycled through the steps
FLUSH_BYTES = 256 << 20  # > 126 MB L2
# dram__bytes_read.sum + dram__bytes_write.sum of one gate/up + one down GEMV launch
# (ncu capture of the M = 1 step, profiles/decode_m1_layer_kernels.md):
# gate/up 141.59 MB read + 3.53 MB written, down 70.89 MB read + 1.16 MB written.
NCU_GEMV_TRAFFIC_BYTES_PER_STEP = 217_170_000


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def algorithmic_bytes(n_union: int, m: int):
    """Bytes one step must move: (|U| + shared) experts, router weights, x in and out."""
    from peregrine_b200.synth import expert_bytes

    c = CFG
    we = expert_bytes(c["hidden"], c["inter"], c["gs"])
    gu = we * 2 // 3
    dn = we // 3
    ne = n_union + c["n_shared"]
    total = ne * we + c["n_experts"] * c["hidden"] * 4 + 2 * m * c["hidden"] * 4
    return total, ne * gu, ne * dn


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


def host_layer(seed: int, distinct: int):
    from peregrine_b200.synth import synth_layer

    c = CFG
    return synth_layer(seed, c["hidden"], c["inter"], c["n_experts"], c["k"], c["gs"], shared=True,
                       norm_topk=c["norm_topk"], routed_scale=c["routed_scale"], zipf=True,
                       distinct_experts=distinct)


def cpu_pass(layer, xs, threads: int, budget_s: float, max_tokens: int = 4096):
    """Times the oracle's layer forward (the reference's CPU int4 path restated in C) one
    token at a time until `budget_s` of CPU work has been spent.  Returns tok/s, tokens."""
    import oracle as po

    def ow(m):
        return po.Weight(m.q, m.scale, 4, m.gs, m.i_n, m.o_n)

    experts = [(ow(e.gate), ow(e.up), ow(e.down)) for e in layer.experts]
    shared = (ow(layer.shared.gate), ow(layer.shared.up), ow(layer.shared.down))
    c = CFG

    def one(x):
        return po.moe_forward(x, layer.router_w, layer.router_bias, experts, shared, x.shape[0], c["hidden"], c["k"],
                              c["norm_topk"], c["routed_scale"], threads=threads)

    one(xs[0:1])  # warm-up (page in the weights touched, spin up the pool)
    n, spent, times = 0, 0.0, []
    while spent < budget_s and n < max_tokens:
        x = xs[n % len(xs)][None, :]
        t0 = time.perf_counter()
        one(x)
        dt = time.perf_counter() - t0
        times.append(dt)
        spent += dt
        n += 1
    med = float(np.median(times))
    return 1.0 / med, n, med


def run_reference(args, rank: int, world: int):
    """The reference's own CPU implementation of the path (oracle port), all host threads."""
    if rank != 0:
        return
    import oracle as po
    from peregrine_b200.synth import synth_tokens

    po.build()
    threads = os.cpu_count() or 1
    layer = host_layer(seed=1, distinct=32)
    xs = synth_tokens(2, N_TOKENS, CFG["hidden"])
    # each step = one token; warm-up + steps bounded so the run ends within minutes
    # a step is one decode token; the sample is bounded to ~60 s of CPU work
    tok_s, n, med = cpu_pass(layer, xs, threads, budget_s=60.0, max_tokens=args.steps)
    line = {
        "impl": "reference", "metric": METRIC, "value": tok_s, "unit": UNIT, "n_gpus": args.gpus, "steps": n,
        "warmup": 1, "ms_per_step": med * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int4 x int8 -> int32 -> f32", "data": "synthetic",
        "config": {"workload": "configs[1]: one MoE decode layer, hidden 6144, 256 experts top-8 + 1 shared, "
                               "moe_inter 2048, int4 group-32, M=1, Zipf(1.1) selection bias", "m": 1},
        "cpu_baseline": {"value": tok_s, "unit": UNIT, "cores": threads, "kind": "port",
                         "simd": "avx2" if po.simd_tier() == 1 else "scalar",
                         "sample": f"{n} decode tokens, median per-token time; 32 distinct expert blobs on the host"},
        "e2e": {"value": tok_s, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_ours(args, rank: int, local_rank: int, world: int):
    import torch

    from peregrine_b200 import cuda
    from peregrine_b200.resident import upload_expert
    from peregrine_b200.synth import synth_expert, synth_tokens, zipf_bias

    dist = None
    if world > 1:
        import torch.distributed as dist  # noqa: F811

        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    c = CFG
    m = args.m
    dev = local_rank
    torch.cuda.set_device(dev)
    if cuda.init([dev]) < 1:
        raise RuntimeError("bench: the CUDA backend could not initialise its device (no CPU fallback exists)")
    # ---- resident layer: every expert generated and uploaded separately
    rng = np.random.default_rng(1234 + rank)
    router_w = (rng.standard_normal((c["n_experts"], c["hidden"])).astype(np.float32) * np.float32(0.02))
    bias = zipf_bias(rng, c["n_experts"])
    ml = cuda.MoeLayer(dev, c["hidden"], c["inter"], c["n_experts"], c["k"], c["norm_topk"], c["routed_scale"],
                       router_w, bias)
    t_up = time.time()
    for e in range(c["n_experts"] + 1):
        ml.set_expert(e, upload_expert(dev, synth_expert(rng, c["hidden"], c["inter"], c["gs"]), c["hidden"],
                                       c["inter"]))
    t_up = time.time() - t_up
    stream = torch.cuda.ExternalStream(cuda.lib().coli_cuda_stream(dev), device=dev)
    xs_host = synth_tokens(99 + rank, N_TOKENS * m, c["hidden"]).reshape(N_TOKENS, m, c["hidden"])
    with torch.cuda.stream(stream):
        xs = torch.from_numpy(xs_host).cuda(dev)
        out = torch.empty((m, c["hidden"]), dtype=torch.float32, device=dev)
        flush = torch.empty(FLUSH_BYTES, dtype=torch.uint8, device=dev)
        drain = torch.zeros(FLUSH_BYTES // 4, dtype=torch.float32, device=dev)
    stream.synchronize()

    def flush_l2():
        # 1. write 256 MiB: every line of the 126 MB L2 now belongs to the flush buffer;
        # 2. read another 256 MiB: the dirty lines left by the write are written back and replaced
        #    by clean lines, so the timed step starts with a cold L2 and pays for no write-backs
        #    of the flush itself.
        flush.zero_()
        drain.sum()

    def step(i, timed_events=None):
        with torch.cuda.stream(stream):
            flush_l2()
            if timed_events:
                timed_events[0].record(stream)
            ml.forward_dev(out.data_ptr(), xs[i % N_TOKENS].data_ptr(), m)
            if timed_events:
                timed_events[1].record(stream)

    for i in range(args.warmup):
        step(i)
    stream.synchronize()
    if dist:
        dist.barrier()
    torch.cuda.synchronize()
    events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    n0 = cuda.kernel_launches()
    with ClockSampler(dev) as clocks:
        for i in range(args.steps):
            step(i, events[i])
        stream.synchronize()
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
    launches = cuda.kernel_launches() - n0
    step_ms = np.array([a.elapsed_time(b) for a, b in events])
    total_ms = float(step_ms.sum())
    if dist:
        t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    if cuda.last_device_error(dev) != 0:
        raise RuntimeError("bench: a kernel reported a device-side error")
    value = world * m * args.steps / (total_ms * 1e-3)

    # ---- per-kernel times (separate pass over the same steps, events around every launch)
    prof_steps = min(args.steps, 300)
    ml.set_profile(True)
    unions = []
    for i in range(prof_steps):
        step(i)
        unions.append(len(ml.last_routing(m)[3]))
    stage_ms, ncalls = ml.profile()
    ml.set_profile(False)
    n_union = float(np.mean(unions))
    total_b, gu_b, dn_b = algorithmic_bytes(n_union, m)
    # A pair of event records around one launch costs ~2.6 us by itself; the same pass brackets two
    # stages that launch nothing ("qrow_x_unfused", "unused"), so their mean is that cost measured
    # under identical conditions, and the launch duration is the bracket minus it.
    gemv_ms_raw = (stage_ms["gemv_gateup"] + stage_ms["gemv_down"]) / max(ncalls, 1)
    bracket_ms = 0.5 * (stage_ms["qrow_x_unfused"] + stage_ms["unused"]) / max(ncalls, 1)
    gemv_ms = gemv_ms_raw - 2.0 * bracket_ms
    gemv_bytes = gu_b + dn_b
    peak, peak_kind = measured_peaks()
    achieved = gemv_bytes / (gemv_ms * 1e-3) / 1e9 if gemv_ms > 0 else 0.0
    achieved_raw = gemv_bytes / (gemv_ms_raw * 1e-3) / 1e9 if gemv_ms_raw > 0 else 0.0
    roofline = {
        "bound": "hbm", "kernel": "gemv_w4a8_kernel (gate/up + down launches of one step)",
        "achieved": achieved, "peak": peak, "peak_kind": f"{peak_kind} copy bandwidth", "unit": "GB/s",
        "frac": achieved / peak, "frac_of_8000": achieved / 8000.0,
        "achieved_with_event_brackets": achieved_raw, "frac_with_event_brackets": achieved_raw / peak,
        "empty_event_bracket_ms": bracket_ms,
        "traffic": NCU_GEMV_TRAFFIC_BYTES_PER_STEP, "algorithmic_bytes": gemv_bytes,
        "launch_ms": {"gateup": stage_ms["gemv_gateup"] / max(ncalls, 1), "down": stage_ms["gemv_down"] / max(ncalls, 1)},
        "gbs": {"gateup": gu_b / (stage_ms["gemv_gateup"] / max(ncalls, 1) * 1e-3) / 1e9 if ncalls else 0,
                "down": dn_b / (stage_ms["gemv_down"] / max(ncalls, 1) * 1e-3) / 1e9 if ncalls else 0},
        "stage_ms": {k: v / max(ncalls, 1) for k, v in stage_ms.items()},
        "kernel_timing": f"separate pass of {prof_steps} steps with CUDA events around every launch; launch duration = "
                         "bracket - empty bracket of the same pass (launch_ms and gbs keep the brackets)",
    }

    # ---- end to end through the host-pointer call (H2D of x and D2H of the result inside)
    e2e_steps = min(args.steps, 300)
    for i in range(3):
        ml.forward(xs_host[i % N_TOKENS])
    e2e_t = 0.0
    for i in range(e2e_steps):
        with torch.cuda.stream(stream):
            flush_l2()
        stream.synchronize()
        t0 = time.perf_counter()
        ml.forward(xs_host[i % N_TOKENS])
        e2e_t += time.perf_counter() - t0
    if dist:
        t = torch.tensor([e2e_t], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_t = float(t.item())
    e2e = {"value": world * m * e2e_steps / e2e_t, "unit": UNIT, "h2d_bytes_per_step": m * c["hidden"] * 4,
           "d2h_bytes_per_step": m * c["hidden"] * 4, "steps": e2e_steps,
           "call": "coli_cuda_moe_layer_forward (host x in, host out back, blocking)"}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int4 x int8 -> int32 -> f32", "data": "synthetic",
        "config": {"workload": "configs[1]: one MoE decode layer, hidden 6144, 256 experts top-8 + 1 shared, "
                               "moe_inter 2048, int4 group-32, Zipf(1.1) selection bias, all experts resident",
                   "m": m, "l2": "flushed before every step, untimed: 256 MiB written, then 256 MiB read so no dirty lines remain",
                   "parallelism": "1 GPU" if world == 1 else f"{world} independent replicas (one layer copy per GPU)",
                   "mean_union": n_union, "upload_s": round(t_up, 1)},
        "hbm_gbs_whole_step": total_b / (total_ms / args.steps * 1e-3) / 1e9,
        "hbm_frac_of_8000_whole_step": total_b / (total_ms / args.steps * 1e-3) / 1e9 / 8000.0,
        "roofline": roofline, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks.summary(),
    }
    if world == 1 and m == 1:
        # the same layer at the batch of the expert-parallel runs, on this one GPU: the base the
        # N > 1 lines of this bench (strong scaling at batch 32) compare with
        xb_host = synth_tokens(7, 8 * EP_BATCH, c["hidden"]).reshape(8, EP_BATCH, c["hidden"])
        with torch.cuda.stream(stream):
            xb = torch.from_numpy(xb_host).cuda(dev)
            ob = torch.empty((EP_BATCH, c["hidden"]), dtype=torch.float32, device=dev)
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(40)]
        for i in range(45):
            with torch.cuda.stream(stream):
                flush_l2()
                if i >= 5:
                    evs[i - 5][0].record(stream)
                ml.forward_dev(ob.data_ptr(), xb[i % 8].data_ptr(), EP_BATCH)
                if i >= 5:
                    evs[i - 5][1].record(stream)
        stream.synchronize()
        ms32 = float(np.mean([a.elapsed_time(b) for a, b in evs]))
        line["ep_batch32"] = {"value": EP_BATCH / (ms32 * 1e-3), "unit": UNIT, "ms_per_step": ms32, "m": EP_BATCH,
                              "steps": 40}
        # configs[3]: one prefill chunk of 4096 tokens through the same layer (CTA-tiled kernel)
        pm = 4096
        xp_host = synth_tokens(11, pm, c["hidden"])
        with torch.cuda.stream(stream):
            xp = torch.from_numpy(xp_host).cuda(dev)
            op = torch.empty((pm, c["hidden"]), dtype=torch.float32, device=dev)
        pev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(5)]
        for i in range(7):
            with torch.cuda.stream(stream):
                flush_l2()
                if i >= 2:
                    pev[i - 2][0].record(stream)
                ml.forward_dev(op.data_ptr(), xp.data_ptr(), pm)
                if i >= 2:
                    pev[i - 2][1].record(stream)
        stream.synchronize()
        pms = float(np.mean([a.elapsed_time(b) for a, b in pev]))
        pops = 2.0 * 3 * c["hidden"] * c["inter"] * pm * (c["k"] + 1)
        line["prefill_4096"] = {"value": pm / (pms * 1e-3), "unit": UNIT, "ms_per_step": pms, "m": pm, "steps": 5,
                                "int8_tops": pops / (pms * 1e-3) / 1e12,
                                "note": "group-32 format: every 32-element block dot is folded into fp32 on the "
                                        "CUDA cores in reference order, which bounds this kernel, not the tensor pipe"}
        del xp, op
    if rank == 0 and world == 1 and not args.no_cpu:
        import oracle as po

        po.build()
        threads = min(os.cpu_count() or 1, 16)  # the reference's default worker count
        layer = host_layer(seed=1, distinct=32)
        tok_s, n, med = cpu_pass(layer, xs_host[:, 0, :], threads, budget_s=12.0)
        line["cpu_baseline"] = {"value": tok_s, "unit": UNIT, "cores": threads, "kind": "port",
                                "simd": "avx2" if po.simd_tier() == 1 else "scalar",
                                "sample": f"{n} decode tokens (M=1) of the same layer shape, median per-token time, "
                                          "32 distinct expert blobs on the host"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist:
        dist.barrier()
        dist.destroy_process_group()
    torch.cuda.synchronize()
    ml.free()
    cuda.shutdown()


EP_BATCH = 32  # configs[4]: decode batch of the expert-parallel runs


def run_ep(args, rank: int, local_rank: int, world: int):
    """N > 1: one MoE decode layer of configs[4], batch 32, routed experts split over the ranks
    (256/N per GPU), router and shared expert replicated, NCCL all-gather / sum-reduction around
    the expert kernels.  Strong scaling: the batch is fixed."""
    import torch
    import torch.distributed as dist

    from peregrine_b200 import cuda
    from peregrine_b200.ep import EpLayerRunner, owned_range
    from peregrine_b200.resident import upload_expert
    from peregrine_b200.synth import synth_expert, synth_tokens, zipf_bias

    c = CFG
    dev = local_rank
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=torch.device("cuda", dev))
    if cuda.init([dev]) < 1:
        raise RuntimeError("bench: the CUDA backend could not initialise its device (no CPU fallback exists)")
    m_total = args.m if args.m > 1 else EP_BATCH
    m_local = m_total // world
    rng = np.random.default_rng(1234)  # router identical on every rank
    router_w = (rng.standard_normal((c["n_experts"], c["hidden"])).astype(np.float32) * np.float32(0.02))
    bias = zipf_bias(rng, c["n_experts"])
    ml = cuda.MoeLayer(dev, c["hidden"], c["inter"], c["n_experts"], c["k"], c["norm_topk"], c["routed_scale"],
                       router_w, bias)
    ml.set_ep(rank, world)
    for e in owned_range(c["n_experts"], rank, world):
        ml.set_expert(e, upload_expert(dev, synth_expert(np.random.default_rng(5000 + e), c["hidden"], c["inter"],
                                                         c["gs"]), c["hidden"], c["inter"]))
    ml.set_shared(upload_expert(dev, synth_expert(np.random.default_rng(4999), c["hidden"], c["inter"], c["gs"]),
                                c["hidden"], c["inter"]))
    run = EpLayerRunner(ml, dev, rank, world, m_total)
    stream = run.stream
    xs_host = synth_tokens(99, N_TOKENS * m_total, c["hidden"]).reshape(N_TOKENS, m_total, c["hidden"])
    xs_host = np.ascontiguousarray(xs_host[:, rank * m_local:(rank + 1) * m_local, :])
    with torch.cuda.stream(stream):
        xs = torch.from_numpy(xs_host).cuda(dev)
        flush = torch.empty(FLUSH_BYTES, dtype=torch.uint8, device=dev)
        drain = torch.zeros(FLUSH_BYTES // 4, dtype=torch.float32, device=dev)
        x_pin = torch.from_numpy(xs_host).pin_memory()
        x_dev = torch.empty((m_local, c["hidden"]), dtype=torch.float32, device=dev)
    stream.synchronize()

    def step(i, ev=None):
        with torch.cuda.stream(stream):
            flush.zero_()
            drain.sum()
            if ev:
                ev[0].record(stream)
            run.forward(xs[i % N_TOKENS])
            if ev:
                ev[1].record(stream)

    for i in range(args.warmup):
        step(i)
    stream.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    n0 = cuda.kernel_launches()
    with ClockSampler(dev) as clocks:
        for i in range(args.steps):
            step(i, events[i])
        stream.synchronize()
    torch.cuda.synchronize()
    dist.barrier()
    launches = cuda.kernel_launches() - n0
    total_ms = float(sum(a.elapsed_time(b) for a, b in events))
    t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms = float(t.item())
    if cuda.last_device_error(dev) != 0:
        raise RuntimeError("bench: a kernel reported a device-side error")
    value = m_total * args.steps / (total_ms * 1e-3)
    n_union = len(ml.last_routing(m_total)[3])
    # end to end: pinned host tokens in, home-token outputs back to the host, every step
    e2e_steps = min(args.steps, 200)
    e2e_t = 0.0
    for i in range(e2e_steps):
        with torch.cuda.stream(stream):
            flush.zero_()
            drain.sum()
        stream.synchronize()
        dist.barrier()
        t0 = time.perf_counter()
        with torch.cuda.stream(stream):
            x_dev.copy_(x_pin[i % N_TOKENS], non_blocking=True)
            out = run.forward(x_dev)
            host = out.to("cpu", non_blocking=False)
        e2e_t += time.perf_counter() - t0
        del host
    t = torch.tensor([e2e_t], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_t = float(t.item())
    total_b, gu_b, dn_b = algorithmic_bytes(n_union, m_total)
    peak, peak_kind = measured_peaks()
    step_s = total_ms / args.steps * 1e-3
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int4 x int8 -> int32 -> f32", "data": "synthetic",
        "config": {"workload": f"configs[4] MoE layer, expert-parallel: decode batch {m_total} fixed, hidden 6144, "
                               f"256 routed experts top-8 split {c['n_experts'] // world} per GPU + replicated "
                               "shared expert, moe_inter 2048, int4 group-32, Zipf(1.1) selection bias",
                   "m": m_total, "parallelism": f"ep{world}: all-gather of tokens, sum-reduction of pair rows (NCCL)",
                   "l2": "flushed before every step, untimed: 256 MiB written, then 256 MiB read",
                   "union": n_union,
                   "note": "the N=1 line of this bench is configs[1] (M=1); its ep_batch32 entry is the "
                           "single-GPU time of this same batch-32 layer"},
        "roofline": {"bound": "hbm", "kernel": "whole layer step (all ranks)", "achieved": total_b / step_s / 1e9,
                     "peak": peak * world, "peak_kind": f"{peak_kind} copy bandwidth x {world} GPUs", "unit": "GB/s",
                     "frac": total_b / step_s / 1e9 / (peak * world), "traffic": None,
                     "algorithmic_bytes": total_b},
        "e2e": {"value": m_total * e2e_steps / e2e_t, "unit": UNIT, "h2d_bytes_per_step": m_local * c["hidden"] * 4,
                "d2h_bytes_per_step": m_local * c["hidden"] * 4, "steps": e2e_steps,
                "call": "EpLayerRunner.forward on this rank's home tokens (pinned host in, host out)"},
        "gpu_launches": int(launches), "clocks": clocks.summary(),
    }
    if rank == 0:
        print(json.dumps(line), flush=True)
    # teardown order matters: the collectives were enqueued on the backend's stream, so the process
    # group goes first, then torch's tensors, and the backend (which owns that stream) last
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()
    del run, xs, flush, drain, x_dev, x_pin
    torch.cuda.synchronize()
    ml.free()
    cuda.shutdown()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--m", type=int, default=1, help="tokens per step (decode batch)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
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
