#!/usr/bin/env python
"""Benchmark of the NVFP4 linear path on B200.

    python bench.py --gpus N --steps K --warmup W            # this repo's CUDA path
    python bench.py --impl reference --gpus N --steps K ...   # the CPU oracle on the host cores

Workload (default): the 64-layer NVFP4 linear stack of a 32B-class decoder (hidden 5120, 64 query
/ 8 KV heads of 128, intermediate 25600) at M = 2048 tokens, tensor-parallel over N GPUs
(column-split q/k/v/gate/up, row-split o/down, one NCCL all-reduce after each row-split
projection). A step is one pass of all 64 layers over one batch of M tokens; the metric is
tokens/s of the whole job. ``--workload decode`` runs the same stack at M = 1.

One JSON line is printed by rank 0. ``value`` has inputs resident in HBM; ``e2e`` copies the
step's activations from pinned host memory and reads the result back inside the timed region.
``roofline`` is for the dominant kernel (the tcgen05 NVFP4 GEMM at M = 2048, the streaming GEMV at
M = 1), timed with CUDA events on its launch stream inside the timed region. ``cpu_baseline`` times
the CPU oracle on a bounded sample of the same workload. Data is synthetic (seeded N(0, 0.02^2)
weights, N(0, 1) activations).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "nvfp4_layer_stack_tokens_per_s"
UNIT = "tok/s"
FP4_OVER_BF16 = 4.0          # nominal dense FP4 : BF16 tensor ratio on B200 (9 : 2.25 PFLOP/s)
NOMINAL_FP4_TFLOPS = 9000.0
NOMINAL_HBM_GBS = 8000.0


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_baseline_sample(spec, m_tokens: int, seconds_target: float = 12.0, threads: int = 0):
    """The CPU oracle (row-parallel over all host threads, f64 accumulation, same arithmetic as the
    reference's velox-cpu) on a bounded sample: a row slice of one gate projection. Returns
    (tokens/s the whole stack would reach at that MAC rate, cores, description)."""
    import numpy as np
    from oracle import oracle as O

    # an explicit count: launchers such as torchrun export OMP_NUM_THREADS=1, which would otherwise
    # turn "all host threads" into one
    cores = threads if threads > 0 else (len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity")
                                         else (os.cpu_count() or 1))
    threads = cores
    k, n = spec.hidden, 256
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    payload = O.encode_nvfp4_rne(w)
    m = min(m_tokens, 64)
    x = rng.standard_normal((m, k)).astype(np.float32)
    # calibrate, then size the sample to the time target
    t0 = time.perf_counter()
    O.linear(x, payload, O.FMT_NVFP4, n, k, 0, n, m, threads=threads,
             act=O.ACT_NVFP4 if m_tokens > 16 else O.ACT_BF16, divisor=256.0)
    dt = max(time.perf_counter() - t0, 1e-4)
    reps = max(1, min(20000, int(seconds_target / dt)))
    t0 = time.perf_counter()
    for _ in range(reps):
        O.linear(x, payload, O.FMT_NVFP4, n, k, 0, n, m, threads=threads,
                 act=O.ACT_NVFP4 if m_tokens > 16 else O.ACT_BF16, divisor=256.0)
    dt = time.perf_counter() - t0
    macs = reps * m * n * k
    # at decode width the oracle re-decodes the weights every call, exactly as velox-cpu does
    mac_per_token = spec.flops_per_token() / 2
    tok_s = (macs / dt) / mac_per_token * (1.0 if m_tokens > 16 else 1.0)
    sample = (f"{reps} x oracle linear NVFP4 rows 256 of [25600,{k}] at m={m} ({macs / 1e9:.1f} GMAC in "
              f"{dt:.1f} s), scaled by the stack's {mac_per_token / 1e9:.1f} GMAC per token")
    return tok_s, cores, sample, dt / reps


def run_reference(args):
    from velox_inferer_b200.stack import StackSpec

    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    spec = StackSpec(layers=args.layers)
    m = 1 if args.workload == "decode" else args.m
    vals = []
    cores, sample = os.cpu_count() or 1, ""
    for i in range(args.warmup + args.steps):
        tok_s, cores, sample, step_s = cpu_baseline_sample(spec, m, seconds_target=max(2.0, 60.0 / (args.warmup + args.steps)))
        if i >= args.warmup:
            vals.append((tok_s, step_s))
    tok_s = sum(v[0] for v in vals) / len(vals)
    line = {
        "impl": "reference", "metric": METRIC, "value": tok_s, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * m / tok_s,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f64 accumulate over NVFP4",
        "data": "synthetic",
        "config": workload_config(args, spec, m, args.gpus > 1 and args.tp == "fused"),
        "cpu_baseline": {"value": tok_s, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tok_s, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(args, spec, m, fused_tp=False):
    return {"workload": f"{spec.layers}-layer NVFP4 linear stack (hidden {spec.hidden}, q {spec.q_dim}, kv {spec.kv_dim}, "
                        f"intermediate {spec.intermediate}), M={m}, attention = passthrough of q",
            "tokens_per_step": m, "layers": spec.layers,
            "parallelism": f"tp{args.gpus}: column-split q/k/v/gate/up, row-split o/down, "
                           + ("bf16 partial tiles stored into the owning rank's rows by the GEMM epilogue over NVLink "
                              "(reduce-scatter), NVFP4 norm output stored into every rank (all-gather), "
                              "signal-pad barriers" if fused_tp else "bf16 all-reduce (NCCL) after o and down"),
            "activations": "NVFP4 tensor-core operands written by the producing kernels (ActQuant::Nvfp4, "
                           "per-use divisors 256/128/16); f32 residual stream; bf16 step input and output",
            "l2": "each step streams the layers' distinct weights, far larger than the 126 MB L2"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="prefill", choices=["prefill", "decode", "linear"],
                    help="prefill / decode: the layer stack at M = --m / M = 1; linear: only the single "
                         "[25600, 5120] NVFP4 linear at M = 1 and M = 2048 (the profiling target)")
    ap.add_argument("--m", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=64)
    ap.add_argument("--no-components", action="store_true", help="skip the single-linear GEMV / GEMM lines")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--tp", choices=("fused", "nccl"), default="fused",
                    help="N > 1: communication fused into the GEMM epilogue and the norm over symmetric memory, "
                         "or one NCCL all-reduce after o and down")
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of replaying a CUDA graph")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 0)

    if args.impl == "reference":
        run_reference(args)
        return

    import torch
    import torch.distributed as dist

    from velox_inferer_b200 import ActPolicy, Sm100Backend, WeightFormat, WeightView
    from velox_inferer_b200.stack import LinearStack, StackSpec

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    b = Sm100Backend(local)
    if args.workload == "linear":
        print(json.dumps({"metric": "nvfp4_single_linear", "n_gpus": 1, "data": "synthetic",
                          "components": components(b, measured_peaks(), graph=not args.no_graph)}), flush=True)
        return
    spec = StackSpec(layers=args.layers)
    m = 1 if args.workload == "decode" else args.m
    peaks = measured_peaks()

    stack = LinearStack(b, spec, max_tokens=m, rank=rank, world=world, a4=True, seed=0)
    gen = torch.Generator().manual_seed(1234)
    x_host = torch.randn(m, spec.hidden, generator=gen).to(torch.bfloat16).pin_memory()
    y_host = torch.empty(m, spec.hidden, dtype=torch.bfloat16).pin_memory()
    x_dev = x_host.to(b.device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    fused_tp = False
    if world > 1 and args.tp == "fused":
        try:
            fused_tp = stack.enable_fused_tp(m)
        except Exception as exc:  # symmetric memory not available here: the NCCL step still is
            print(f"[bench] fused tensor parallelism not available ({exc}); using NCCL all-reduce",
                  file=sys.stderr, flush=True)
    forward = (lambda: stack.forward_fused_tp(x_dev)) if fused_tp else (lambda: stack.forward(x_dev, m))
    for _ in range(max(args.warmup, 3)):
        forward()
    barrier()

    # A step is hundreds of launches (and, with several ranks, two all-reduces per layer): it is
    # captured once and replayed as one CUDA graph, as the reference runs its step
    # (crates/velox-cuda/src/lib.rs:2130-2204), unless --no-graph is given or capture fails. Event
    # timing of single kernels is not possible inside a graph, so the roofline pass runs eagerly.
    step = forward
    use_graph = not args.no_graph
    if use_graph:
        try:
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                forward()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                forward()
            step = graph.replay
            for _ in range(3):
                step()
        except Exception as exc:  # capture not possible here: time eager launches instead
            print(f"[bench] CUDA graph capture failed ({exc}); launching eagerly", file=sys.stderr, flush=True)
            use_graph = False
            step = forward
        barrier()
    if b.lib.velox_sm100_debug_status() != 0:
        raise SystemExit("tensor-core kernel reported a timed-out wait")

    # ---- device-resident timing ----
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = b.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    launches = b.launch_count() - launches0
    if use_graph:
        launches = stack.launches_per_step * args.steps
    t = torch.tensor([ms], device=b.device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())

    # ---- the same steps again with every main kernel bracketed by CUDA events on its launch
    #      stream (the library's timing hooks): per-kernel durations for the roofline ----
    b.timing_enable(True)
    stack.kv_side_streams = False   # one stream: the event brackets of concurrent kernels would overlap
    barrier()
    for _ in range(args.steps):
        forward()
    barrier()
    timed = b.timing_collect()
    b.timing_enable(False)
    stack.kv_side_streams = True
    clocks = sampler.stop() if rank == 0 else None

    # ---- end to end: pinned host -> device, all layers, result back to the host ----
    barrier()
    e0.record()
    for _ in range(args.steps):
        x_dev.copy_(x_host, non_blocking=True)
        if use_graph:
            step()
            out = stack.fabric.out if fused_tp else stack.outb
        else:
            out = forward()
        y_host.copy_(out[: m * spec.hidden].view(m, spec.hidden), non_blocking=True)
    e1.record()
    barrier()
    t = torch.tensor([e0.elapsed_time(e1) / args.steps], device=b.device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item())

    def shutdown():
        # A captured graph holds the communicator's kernels: drop it and drain the device before the
        # process group goes away, and never let teardown outlive the measurement by more than a
        # few seconds (a rank stuck here would keep the whole launcher alive).
        nonlocal step
        if world > 1:
            threading.Timer(20.0, lambda: os._exit(0)).start()
            step = None
            if use_graph:
                graph.reset()
            torch.cuda.synchronize()
            dist.barrier()
            dist.destroy_process_group()
            os._exit(0)

    if rank != 0:
        shutdown()
        return

    # ---- roofline of the dominant kernel ----
    per_rank_flops = spec.flops_per_token() * m / world
    per_rank_bytes = stack.weight_bytes
    if m > 16:
        k_ms, k_n = timed["gemm_nvfp4"]
        peak = peaks["bf16_tflops"] * FP4_OVER_BF16
        achieved = per_rank_flops * args.steps / (k_ms * 1e-3) / 1e12 if k_ms > 0 else 0.0
        roofline = {"bound": "tensor", "kernel": "gemm_kernel<mxf4nvf4> (tcgen05 block-scaled NVFP4)",
                    "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                    "peak_source": f"{peaks['source']} bf16 cuBLAS {peaks['bf16_tflops']} TFLOP/s x {FP4_OVER_BF16:g} "
                                   "(no FP4 GEMM peak is measured on this pool; nominal dense FP4 : BF16 ratio)",
                    "frac_of_nominal_fp4": achieved / NOMINAL_FP4_TFLOPS,
                    "launches": int(k_n), "avg_launch_us": 1e3 * k_ms / max(k_n, 1),
                    # DRAM bytes of one [25600, 5120] M = 2048 launch from the committed ncu capture
                    # (79.7 MB read + 71.8 MB written; algorithmic 79.6 MB + 104.9 MB of output)
                    "traffic": 151.5e6, "traffic_of": "profiles/gemm_nvfp4_25600x5120_m2048.md",
                    "act_quant_ms_per_step": timed["act_quant"][0] / args.steps}
    else:
        k_ms, k_n = timed["gemv"]
        achieved = per_rank_bytes * args.steps / (k_ms * 1e-3) / 1e9 if k_ms > 0 else 0.0
        roofline = {"bound": "hbm", "kernel": "gemv_nvfp4_tc_kernel (tcgen05 block-scaled decode)", "achieved": achieved,
                    "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                    "peak_source": f"{peaks['source']} copy bandwidth",
                    "frac_of_nominal_hbm": achieved / NOMINAL_HBM_GBS,
                    "launches": int(k_n), "avg_launch_us": 1e3 * k_ms / max(k_n, 1),
                    # DRAM bytes of one [25600, 5120] M = 1 launch from the committed ncu capture
                    "traffic": 75.9e6, "traffic_of": "profiles/gemv_nvfp4_tc_25600x5120_m1.md"}

    line = {
        "metric": METRIC, "value": m / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "nvfp4 x nvfp4 -> f32 accumulate (bf16 in/out)",
        "data": "synthetic", "config": workload_config(args, spec, m, fused_tp),
        "e2e": {"value": m / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": y_host.numel() * 2},
        "gpu_launches": int(launches), "cuda_graph": bool(use_graph), "clocks": clocks, "roofline": roofline,
        "tflops_per_gpu": per_rank_flops / (ms * 1e-3) / 1e12,
        "weights_gb_per_gpu": per_rank_bytes / 1e9,
    }

    if world == 1 and not args.no_components:
        line["components"] = components(b, peaks)
    if world == 1 and not args.no_cpu_baseline:
        tok_s, cores, sample, _ = cpu_baseline_sample(spec, m)
        # the reference's own CPU backend is single-threaded: the same sample on one thread beside it
        tok_1, _, sample_1, _ = cpu_baseline_sample(spec, m, seconds_target=4.0, threads=1)
        line["cpu_baseline"] = {"value": tok_s, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample,
                                "single_thread": {"value": tok_1, "unit": UNIT, "cores": 1, "sample": sample_1}}
    else:
        line["cpu_baseline"] = None
    print(json.dumps(line), flush=True)
    sys.stdout.flush()
    shutdown()


def _time_replays(replay, launches_per_replay, gpu_index=0, warm_s=0.2, timed_s=0.3):
    """Microseconds per launch of `replay`, with the clocks seen meanwhile. The device first runs the
    same work for `warm_s`, so that its clocks are those this workload settles at rather than those
    the previous phase of the benchmark left behind (a power-capped prefill step, or an idle GPU);
    the timed region then lasts about `timed_s`, long enough for the clock sampler to see it."""
    import time

    import torch

    replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    replay()
    e1.record()
    torch.cuda.synchronize()
    per_replay_s = max(e0.elapsed_time(e1) * 1e-3, 1e-6)
    sampler = ClockSampler(gpu_index)   # (sees the warm-up too: the same work, and nvidia-smi takes a moment to start)
    sampler.start()
    t_end = time.time() + warm_s
    while time.time() < t_end:
        for _ in range(8):
            replay()
        torch.cuda.synchronize()
    n = max(3, int(timed_s / per_replay_s))
    e0.record()
    for _ in range(n):
        replay()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    return e0.elapsed_time(e1) * 1e3 / (n * launches_per_replay), clocks


def components(b, peaks, graph=True):
    """Single NVFP4 linear [25600, 5120]: decode GEMV (M = 1, weight copies rotated so they never
    sit in L2) and prefill GEMM (M = 2048), timed with CUDA events."""
    import torch

    from velox_inferer_b200 import ActPolicy, WeightFormat, WeightView

    n, k = 25600, 5120
    copies = 6   # 6 x 73.7 MB > 3 x the 126 MB L2
    views = []
    gen = torch.Generator(device=b.device).manual_seed(0)
    for _ in range(copies):
        w = torch.randn(n, k, generator=gen, device=b.device) * 0.02
        views.append(WeightView.full(b.encode_nvfp4(w), WeightFormat.NVFP4, n, k).with_act(ActPolicy.allow_a4(256.0)))
        del w
    out = {}
    payload = WeightFormat.NVFP4.payload_bytes(n, k)
    stream = torch.cuda.Stream()
    for m, twin in ((1, False), (1, True), (2048, False)):
        xb = torch.randn(m, k, device=b.device).to(torch.bfloat16)
        yb = torch.empty(m, n, dtype=torch.bfloat16, device=b.device)
        rounds = 5 if m == 1 else 2
        if twin:
            # the FP4 activation twin a norm or a producing linear hands over: no quantiser launch
            q4 = b.q4_blob(m, k)
            b.add_rms_norm_q4(xb.float().reshape(-1).contiguous(), None, torch.ones(k, device=b.device), None, q4,
                              m, k, 1e-6, 256.0)
            call = lambda v: b.linear_q4(q4, 256.0, v, None, m, yb=yb)
        else:
            call = lambda v: b.linear_bf16(xb, v, None, m, yb=yb)
        with torch.cuda.stream(stream):
            for v in views:
                call(v)
        torch.cuda.synchronize()
        # replayed as one CUDA graph so that host launch latency is not in the measurement
        def burst():
            for _ in range(rounds):
                for v in views:
                    call(v)
        replay = burst
        if graph:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                burst()
            replay = g.replay
        if m == 1:
            us, clk = _time_replays(replay, rounds * copies, b.device.index or 0)
        else:
            # a burst: the kernel timed alone, against the burst peak; the sustained figure follows
            replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(3):
                replay()
            e1.record()
            torch.cuda.synchronize()
            us, clk = e0.elapsed_time(e1) * 1e3 / (3 * rounds * copies), None
        if m == 1:
            byts = payload + 2 * m * k + 2 * m * n
            gbs = byts / (us * 1e-6) / 1e9
            out["decode_gemv_m1_fp4_twin_in" if twin else "decode_gemv_m1"] = {
                "us_per_launch": us, "GB/s": gbs, "bytes": byts,
                "frac_of_measured_hbm": gbs / peaks["hbm_gbs"],
                "frac_of_nominal_8TBs": gbs / NOMINAL_HBM_GBS, "clocks": clk,
                "timing": "CUDA-graph replay of 30 launches over 6 rotated weight copies, 0.2 s of the same work first"
                          + ("; input is the NVFP4 blob a producer wrote" if twin
                             else "; bf16 input, includes the activation quantiser launch")}
        else:
            tf = 2.0 * m * n * k / (us * 1e-6) / 1e12
            out["prefill_gemm_m2048"] = {"us_per_launch": us, "TFLOP/s": tf,
                                         "frac_of_measured_bf16_x4": tf / (peaks["bf16_tflops"] * FP4_OVER_BF16),
                                         "frac_of_nominal_fp4": tf / NOMINAL_FP4_TFLOPS,
                                         "timing": "CUDA-graph replay, a burst of 36 launches; includes the activation "
                                                   "quantiser launch"}
            us_s, clk_s = _time_replays(replay, rounds * copies, b.device.index or 0)
            tf_s = 2.0 * m * n * k / (us_s * 1e-6) / 1e12
            out["prefill_gemm_m2048_sustained"] = {
                "us_per_launch": us_s, "TFLOP/s": tf_s,
                "frac_of_measured_bf16_sustained_x4": tf_s / (peaks["bf16_tflops_sustained"] * FP4_OVER_BF16),
                "frac_of_nominal_fp4": tf_s / NOMINAL_FP4_TFLOPS, "clocks": clk_s,
                "timing": "the same graph replayed for 0.2 s, then timed for 0.3 s: under the power cap"}
    del views
    out.update(_decode_other_formats(b, peaks, graph))
    return out


def _decode_other_formats(b, peaks, graph=True):
    """The same [25600, 5120] projection stored as FP8-E4M3 rows and as GGML Q4_K: decode launches at
    1 and 8 tokens with bf16 activations (the rounding every policy admits), seeded synthetic bytes
    (finite codes, sane scales), weight copies rotated so that they never sit in L2."""
    import torch

    from velox_inferer_b200 import ActPolicy, WeightFormat, WeightView

    n, k = 25600, 5120
    out = {}
    gen = torch.Generator(device=b.device).manual_seed(1)
    stream = torch.cuda.Stream()
    for name, fmt, policies in (("fp8", WeightFormat.FP8_ROW_BF16, (("a16", ActPolicy.a16_only()), ("a8", ActPolicy.allow_a8()))),
                                ("q4k", WeightFormat.GGML_Q4_K, (("a16", ActPolicy.a16_only()),))):
        payload = fmt.payload_bytes(n, k)
        copies = 4 if name == "fp8" else 6   # > 3 x the 126 MB L2 either way
        bufs = []
        for _ in range(copies):
            buf = torch.randint(0, 120, (payload + 256,), generator=gen, dtype=torch.uint8, device=b.device)
            if name == "fp8":
                off = (n * k + 255) // 256 * 256
                buf[off:off + 2 * n].view(torch.bfloat16).fill_(0.01)      # bf16 row scales
            else:
                blocks = buf[:payload].view(-1, 144)
                blocks[:, 1] = 0x20                                        # f16 d and dmin: small, finite
                blocks[:, 3] = 0x20
            bufs.append(buf)
        for pname, policy in policies:
            views = [WeightView.full(buf, fmt, n, k).with_act(policy) for buf in bufs]
            for m in (1, 8):
                xb = torch.randn(m, k, device=b.device).to(torch.bfloat16)
                yb = torch.empty(m, n, dtype=torch.bfloat16, device=b.device)
                call = lambda v: b.linear_bf16(xb, v, None, m, yb=yb)
                rounds = 4
                with torch.cuda.stream(stream):
                    for v in views:
                        call(v)
                torch.cuda.synchronize()

                def burst():
                    for _ in range(rounds):
                        for v in views:
                            call(v)
                replay, g = burst, None
                if graph:
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=stream):
                        burst()
                    replay = g.replay
                us, clk = _time_replays(replay, rounds * copies, b.device.index or 0)
                byts = payload + 2 * m * k + 2 * m * n
                gbs = byts / (us * 1e-6) / 1e9
                act = b.linear_act(views[0], m)
                out[f"decode_gemv_{name}_{pname}_m{m}"] = {
                    "us_per_launch": us, "GB/s": gbs, "bytes": byts, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"],
                    "activation_rounding": str(act), "clocks": clk,
                    "timing": f"CUDA-graph replay of {rounds * copies} launches over {copies} rotated weight copies, "
                              "0.2 s of the same work first"}
                del g
        del bufs
    return out


if __name__ == "__main__":
    main()
