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
M = 1), timed with CUDA events on its launch stream inside the timed region; at N = 1 its
``components`` carry the rest of the headline metric (single-linear decode GEMV GB/s and prefill
TFLOP/s, the M sweep, the MLP, the other stored formats, the decode stack). With N > 1 an untimed
check of a two-layer stack runs first and is printed as ``config.tp_check``. ``cpu_baseline`` times
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
    reference's velox-cpu) on a bounded sample: an NVFP4 linear of the stack's width K with 256
    weight rows (a matrix of its own, built with the stack's weight construction) at up to 64
    tokens. Returns (tokens/s the whole stack would reach at that MAC rate, cores, description)."""
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
    sample = (f"{reps} x oracle linear on an NVFP4 [{n},{k}] matrix (the stack's K and weight construction; not a "
              f"slice of a stack matrix) at m={m}: {macs / 1e9:.1f} GMAC in {dt:.1f} s, scaled to tokens/s by the "
              f"stack's {mac_per_token / 1e9:.1f} GMAC per token (extrapolated, not a whole step)")
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
        "config": workload_config(args, spec, m, args.tp if args.gpus > 1 and args.tp != "nccl" else False),
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
                              "(reduce-scatter), NVFP4 norm output stored into every rank (all-gather), ordered by "
                              "per-phase flags in peer memory (bounded waits)" if fused_tp == "flags" else
                              "the same flags raised and awaited by one-warp barrier kernels between the phases "
                              "(bounded waits)" if fused_tp == "kernel" else
                              "the same with torch's signal-pad barrier kernels between the phases" if fused_tp == "barrier" else
                              "bf16 all-reduce (NCCL) after o and down"),
            "activations": "NVFP4 tensor-core operands written by the producing kernels (ActQuant::Nvfp4, "
                           "per-use divisors 256/128/16); f32 residual stream; bf16 step input and output",
            "l2": "each step streams the layers' distinct weights, far larger than the 126 MB L2"}


def tp_check(b, args, rank, world, m):
    """Untimed correctness check of the sharded step at this rank count, on a two-layer stack of the
    benchmark's geometry: the fused step equals the library-collective step with the same arithmetic
    bit for bit (twice: buffers and flags are reused), every rank ends with the same output, and
    both stay as close to the unsharded step (run on every rank's own GPU) as the all-reduce step."""
    import torch
    import torch.distributed as dist

    from velox_inferer_b200.stack import ChunkedStack, LinearStack, StackSpec

    spec = StackSpec(layers=2)
    gen = torch.Generator().manual_seed(4321)
    xb = torch.randn(m, spec.hidden, generator=gen).to(torch.bfloat16).to(b.device)
    n = m * spec.hidden

    def rel_rms(a, c):
        return float(((a.float() - c.float()).pow(2).mean().sqrt() / c.float().pow(2).mean().sqrt()).item())

    chk = LinearStack(b, spec, max_tokens=m, rank=rank, world=world, a4=True, seed=0)
    allreduce = chk.forward(xb, m).view(-1)[:n].clone()
    gathered = chk.forward_gathered(xb, m).view(-1)[:n].clone()
    out = {"layers": spec.layers, "m": m}
    fused_ok = None
    if args.tp != "nccl" and chk.enable_fused_tp(m, sync_mode=args.tp):
        fused_ok = True
        for _ in range(2):
            fused = chk.forward_fused_tp(xb).view(-1)[:n].clone()
            torch.cuda.synchronize()
            fused_ok = fused_ok and bool(torch.equal(fused, gathered)) and b.debug_status() == 0
        mine = fused
        if args.chunks > 1 and world <= 4:
            ch = ChunkedStack(b, spec, m, rank, world, chunks=args.chunks, seed=0)
            ok = ch.enable_fused_tp(m, sync_mode="kernel" if args.tp == "flags" else args.tp)
            for _ in range(2):
                chunked = ch.forward_fused_tp(xb).view(-1)[:n].clone()
                torch.cuda.synchronize()
                ok = ok and bool(torch.equal(chunked, gathered)) and b.debug_status() == 0
            fused_ok = fused_ok and ok
            out["chunks"] = args.chunks
            del ch
    else:
        mine = gathered
    flag = torch.tensor([1 if fused_ok in (True, None) else 0], device=b.device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    out["fused_equals_gathered_bitwise"] = None if fused_ok is None else bool(flag.item())
    ref = mine.clone()
    dist.broadcast(ref, src=0)
    same = torch.tensor([1 if torch.equal(ref, mine) else 0], device=b.device)
    dist.all_reduce(same, op=dist.ReduceOp.MIN)
    out["ranks_hold_equal_output"] = bool(same.item())
    del chk
    whole = LinearStack(b, spec, max_tokens=m, rank=0, world=1, a4=True, seed=0).forward(xb, m).view(-1)[:n].clone()
    out["rel_rms_vs_unsharded"] = round(rel_rms(mine, whole), 5)
    out["rel_rms_allreduce_vs_unsharded"] = round(rel_rms(allreduce, whole), 5)
    out["note"] = ("sharded steps round each shard's partial sums to bf16 and NVFP4 activation quantisation reacts to "
                   "last-bit differences, so agreement with the unsharded step is statistical; the exact check is "
                   "fused == gathered")
    out["ok"] = bool(out["ranks_hold_equal_output"] and out["fused_equals_gathered_bitwise"] is not False
                     and out["rel_rms_vs_unsharded"] <= 2.0 * out["rel_rms_allreduce_vs_unsharded"] + 0.01)
    del whole
    torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="prefill", choices=["prefill", "decode", "linear"],
                    help="prefill / decode: the layer stack at M = --m / M = 1; linear: only the single-linear "
                         "components (the profiling target)")
    ap.add_argument("--m", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=64)
    ap.add_argument("--no-components", action="store_true", help="skip the single-linear GEMV / GEMM lines")
    ap.add_argument("--components", default="all",
                    help="comma-separated subset of: nvfp4,sweep,mlp,formats,decode_stack (default all)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-tp-check", action="store_true")
    ap.add_argument("--tp", choices=("flags", "kernel", "barrier", "nccl", "fused"), default="kernel",
                    help="N > 1: communication fused into the GEMM epilogue and the norm over symmetric memory, "
                         "ordered by the library's own one-warp flag-barrier kernels between the phases (kernel, "
                         "the default: bounded waits on flags in peer memory), by flags that the GEMM and norm "
                         "kernels themselves raise and poll (flags; 'fused' is the same), by torch's signal-pad "
                         "barrier kernels (barrier); or one NCCL all-reduce after o and down (nccl)")
    ap.add_argument("--chunks", type=int, default=1,
                    help="N = 2 or 4, fused step: token chunks that run side by side on streams of their own, so that "
                         "one chunk's transfers overlap another's compute (1, the default: the whole step as one chain)")
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of replaying a CUDA graph")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 0)
    if args.tp == "fused":
        args.tp = "flags"

    if args.impl == "reference":
        run_reference(args)
        return

    import torch
    import torch.distributed as dist

    from velox_inferer_b200 import Sm100Backend
    from velox_inferer_b200.stack import ChunkedStack, LinearStack, StackSpec

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
    peaks = measured_peaks()
    if args.workload == "linear":
        print(json.dumps({"metric": "nvfp4_single_linear", "n_gpus": 1, "data": "synthetic",
                          "components": components(b, peaks, None, args, graph=not args.no_graph)}), flush=True)
        return
    spec = StackSpec(layers=args.layers)
    m = 1 if args.workload == "decode" else args.m

    check = None
    if world > 1 and m > 16 and not args.no_tp_check:
        check = tp_check(b, args, rank, world, m)
        if not check["ok"]:
            raise SystemExit(f"[bench] the sharded step failed its correctness check: {check}")

    # (token chunks are measured at 2 and 4 GPUs only: the one run at 8 never printed a result and was
    # killed with its call; no device wait can last that long, so it stopped on the host, where is not known)
    chunked = 1 < world <= 4 and args.tp != "nccl" and args.chunks > 1 and m % (args.chunks * world * 128) == 0
    if chunked:
        stack = ChunkedStack(b, spec, m, rank, world, chunks=args.chunks, seed=0)
    else:
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
    if world > 1 and args.tp != "nccl":
        try:
            fused_tp = stack.enable_fused_tp(m, sync_mode="kernel" if chunked and args.tp == "flags" else args.tp)
        except Exception as exc:  # symmetric memory not available here: the NCCL step still is
            print(f"[bench] fused tensor parallelism not available ({exc}); using NCCL all-reduce",
                  file=sys.stderr, flush=True)
    forward = (lambda: stack.forward_fused_tp(x_dev)) if fused_tp else (lambda: stack.forward(x_dev, m))
    for i in range(max(args.warmup, 3)):
        forward()
        if i == 0 and world > 1:
            # Every device-side wait of the sharded step gives up after two seconds; a step has hundreds of
            # them, so a step in which they all ran out would take many minutes. Look after the first one.
            torch.cuda.synchronize()
            bad = torch.tensor([b.debug_status()], dtype=torch.int32, device=b.device)
            dist.all_reduce(bad, op=dist.ReduceOp.MAX)
            if int(bad.item()) != 0:
                raise SystemExit(f"a bounded device wait ran out in the first step (status {int(bad.item())}): "
                                 "the step is not timed")
    barrier()

    # A step is hundreds of launches: it is captured once and replayed as one CUDA graph, as the
    # reference runs its step (crates/velox-cuda/src/lib.rs:2130-2204), unless --no-graph is given
    # or capture fails. Event timing of single kernels is not possible inside a graph, so the
    # roofline pass runs eagerly.
    step = forward
    use_graph = not args.no_graph
    graph = None
    if use_graph:
        try:
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                forward()
            torch.cuda.synchronize()
            barrier()
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
    if b.debug_status() != 0:
        raise SystemExit("a kernel reported a wait that ran out")

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
    barrier()
    for _ in range(args.steps):
        forward()
    barrier()
    timed = b.timing_collect()
    b.timing_enable(False)
    clocks = sampler.stop() if rank == 0 else None

    # ---- end to end: pinned host -> device, all layers, result back to the host. The fused sharded
    #      step reads only this rank's token rows and every rank ends with the whole output, so a rank
    #      copies its own rows in and out (the job moves each byte once). ----
    own = fused_tp and world > 1
    nchunks = args.chunks if chunked else 1
    mc = m // nchunks
    rows = mc // world if own else m          # rows of each chunk this rank copies
    spans = [(c * mc + rank * rows, rows) for c in range(nchunks)] if own else [(0, m)]
    h = spec.hidden
    result = (lambda: stack.out) if chunked else (lambda: stack.fabric.out if fused_tp else stack.outb)

    def e2e_pass(with_step):
        barrier()
        e0.record()
        for _ in range(args.steps):
            for r0, n in spans:
                x_dev.view(-1)[r0 * h:(r0 + n) * h].copy_(x_host[r0:r0 + n].view(-1), non_blocking=True)
            if with_step:
                out = (step() or result()) if use_graph else forward()
            else:
                out = result()
            for r0, n in spans:
                y_host[r0:r0 + n].copy_(out.view(-1)[r0 * h:(r0 + n) * h].view(n, h), non_blocking=True)
        e1.record()
        barrier()
        tt = torch.tensor([e0.elapsed_time(e1) / args.steps], device=b.device)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt.item())

    e2e_ms = e2e_pass(True)
    copy_ms = e2e_pass(False)

    def shutdown():
        # A captured graph holds the communicator's kernels: drop it and drain the device before the
        # process group goes away, and never let teardown outlive the measurement by more than a
        # few seconds (a rank stuck here would keep the whole launcher alive).
        nonlocal step, graph
        if world > 1:
            threading.Timer(20.0, lambda: os._exit(0)).start()
            step = None
            if graph is not None:
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
                    "frac_is": "of 4 x measured bf16 cuBLAS burst",
                    "peak_source": f"{peaks['source']} bf16 cuBLAS {peaks['bf16_tflops']} TFLOP/s x {FP4_OVER_BF16:g}: no "
                                   "FP4 GEMM peak is measured on this pool, 4 is the nominal dense FP4 : BF16 ratio",
                    "frac_of_nominal_fp4_9pf": achieved / NOMINAL_FP4_TFLOPS,
                    "launches": int(k_n), "avg_launch_us": 1e3 * k_ms / max(k_n, 1),
                    "traffic": STACK_GEMM_TRAFFIC_PER_LAUNCH if world == 1 else None,
                    "traffic_of": STACK_GEMM_TRAFFIC_OF if world == 1 else
                                  "no capture of the sharded step's launches (ncu runs on one GPU only)",
                    "act_quant_ms_per_step": timed["act_quant"][0] / args.steps}
    else:
        k_ms, k_n = timed["gemv"]
        achieved = per_rank_bytes * args.steps / (k_ms * 1e-3) / 1e9 if k_ms > 0 else 0.0
        roofline = {"bound": "hbm", "kernel": "gemv_nvfp4_tc_kernel (tcgen05 block-scaled decode)", "achieved": achieved,
                    "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                    "frac_is": "of measured copy bandwidth",
                    "peak_source": f"{peaks['source']} copy bandwidth",
                    "frac_of_nominal_hbm_8tbs": achieved / NOMINAL_HBM_GBS,
                    "launches": int(k_n), "avg_launch_us": 1e3 * k_ms / max(k_n, 1),
                    "traffic": None,
                    "traffic_of": "single [25600, 5120] M = 1 launch: 75.9 MB per launch against 73.8 MB algorithmic "
                                  "(profiles/gemv_nvfp4_tc_25600x5120_m1.md); the step's launches were not captured"}

    # where the eager, event-bracketed pass spent its step: the GEMMs, the norms (each including the time
    # it waited for peers' flags) and everything between kernels
    roofline["eager_step_ms"] = {k: round(timed[k][0] / args.steps, 3) for k in ("gemm_nvfp4", "gemv", "norm")
                                 if timed[k][1] > 0}
    cfg = workload_config(args, spec, m, args.tp if fused_tp else False)
    if chunked:
        cfg["parallelism"] += f"; the step's tokens run as {nchunks} chunks side by side on streams of their own"
    if check is not None:
        cfg["tp_check"] = check
    line = {
        "metric": METRIC, "value": m / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "nvfp4 x nvfp4 -> f32 accumulate (bf16 in/out)",
        "data": "synthetic", "config": cfg,
        "e2e": {"value": m / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
                "copy_only_ms_per_step": copy_ms,
                "h2d_bytes_per_step": sum(n for _, n in spans) * h * 2 * world,
                "d2h_bytes_per_step": sum(n for _, n in spans) * h * 2 * world,
                "copies": (f"each of the {world} ranks copies its own {rows * nchunks} token rows in and out" if own
                           else "the whole step input in, the whole output out")},
        "gpu_launches": int(launches), "cuda_graph": bool(use_graph), "clocks": clocks, "roofline": roofline,
        "tflops_per_gpu": per_rank_flops / (ms * 1e-3) / 1e12,
        "weights_gb_per_gpu": per_rank_bytes / 1e9,
    }

    if world == 1 and not args.no_components:
        roofline["components"] = components(b, peaks, stack, args)
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


# DRAM bytes per GEMM launch of the prefill step on one GPU, from an ncu capture of the step's own
# launches (four layers of the same stack: the layers are identical, so the per-launch average is the
# 64-layer step's): 89.8 MB read + 8.0 MB written on average over the step's four launches
# (q|k|v 36.2, o 33.2, gate|up 172.6, down 149.9 MB; the stored operands they must read are 35.4, 33.0,
# 153.4 and 103.2 MB). See the file named beside it.
STACK_GEMM_TRAFFIC_PER_LAUNCH = 97_717_568
STACK_GEMM_TRAFFIC_OF = ("profiles/stack_prefill_gemm_dram_traffic.md: dram__bytes_read.sum + dram__bytes_write.sum, "
                         "mean over the 16 gemm_kernel launches of one 4-layer step")


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


def _timed_cell(b, calls, graph=True, burst_only=False, rounds=None):
    """`calls`: functions that each queue one unit of work on a rotated weight copy. They are run
    back to back (a few rounds), captured as one CUDA graph so that host launch latency is not in
    the measurement, and timed per unit. Returns (microseconds per unit, clock record)."""
    import torch

    stream = torch.cuda.Stream()
    rounds = rounds or max(2, 24 // len(calls))
    with torch.cuda.stream(stream):
        for c in calls:
            c()
    torch.cuda.synchronize()

    def burst():
        for _ in range(rounds):
            for c in calls:
                c()
    replay, g = burst, None
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            burst()
        replay = g.replay
    if burst_only:
        replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / (3 * rounds * len(calls)), None
    return _time_replays(replay, rounds * len(calls), b.device.index or 0)


def _mhz(clk):
    return None if not clk else clk.get("sm_mhz")


def _hbm_cell(us, byts, peaks, clk, **extra):
    gbs = byts / (us * 1e-6) / 1e9
    d = {"us": round(us, 2), "GB/s": round(gbs, 1), "frac_measured_hbm": round(gbs / peaks["hbm_gbs"], 3),
         "frac_nominal_8tbs": round(gbs / NOMINAL_HBM_GBS, 3), "sm_mhz": _mhz(clk)}
    d.update(extra)
    return d


def _tensor_cell(us, flops, peaks, clk, fp4=True, sustained=False, **extra):
    tf = flops / (us * 1e-6) / 1e12
    base = peaks["bf16_tflops_sustained" if sustained else "bf16_tflops"]
    d = {"us": round(us, 2), "TFLOP/s": round(tf, 1)}
    if fp4:
        d["frac_4x_measured_bf16" + ("_sustained" if sustained else "")] = round(tf / (base * FP4_OVER_BF16), 3)
        d["frac_nominal_fp4_9pf"] = round(tf / NOMINAL_FP4_TFLOPS, 3)
    else:
        d["frac_measured_bf16" + ("_sustained" if sustained else "")] = round(tf / base, 3)
    d["sm_mhz"] = _mhz(clk)
    d.update(extra)
    return d


def _kernel_class(b, call):
    """Which kernel family served a call: runs it once with the library's timing hooks on."""
    import torch

    torch.cuda.synchronize()
    b.timing_collect()
    b.timing_enable(True)
    call()
    t = b.timing_collect()
    b.timing_enable(False)
    names = [k for k in ("gemv", "gemm_nvfp4", "gemm_fp8", "gemm_bf16") if t[k][1] > 0]
    return "+".join(names) or "other"


def components(b, peaks, stack, args, graph=True):
    """The rest of the headline metric, one GPU: single-linear decode GEMV and prefill GEMM on
    [25600, 5120] (BASELINE configs 0 and 1, with the M sweep), the SwiGLU MLP (config 2), FP8 rows and
    Q4_K on [14336, 4096] (config 3), and the decode stack (config 4 at M = 1). Weight copies are
    rotated so that no launch finds its weights in L2; every cell is a CUDA-graph replay timed with
    CUDA events after 0.2 s of the same work, with the SM clock seen meanwhile."""
    import torch

    from velox_inferer_b200 import ActPolicy, WeightFormat, WeightView

    want = set((args.components if args else "all").split(","))
    on = lambda name: "all" in want or name in want
    NV, F8, Q4 = WeightFormat.NVFP4, WeightFormat.FP8_ROW_BF16, WeightFormat.GGML_Q4_K
    dev = b.device
    out = {"timing": "CUDA-graph replay over rotated weight copies (> 3 x L2 in total), 0.2 s of the same work first, "
                     "CUDA events; us is per linear (per MLP / per token where said)"}
    gen = torch.Generator(device=dev).manual_seed(0)

    def nvfp4_views(n, k, copies, div):
        vs = []
        for _ in range(copies):
            w = torch.randn(n, k, generator=gen, device=dev) * 0.02
            vs.append(WeightView.full(b.encode_nvfp4(w), NV, n, k).with_act(ActPolicy.allow_a4(div)))
            del w
        return vs

    def blob_of(m, k, div):
        q4 = b.q4_blob(m, k)
        x = torch.randn(m, k, generator=gen, device=dev)
        b.add_rms_norm_q4(x.reshape(-1).contiguous(), None, torch.ones(k, device=dev), None, q4, m, k, 1e-6, div)
        return q4

    if on("nvfp4") or on("sweep"):
        n, k = 25600, 5120
        views = nvfp4_views(n, k, 6, 256.0)   # 6 x 73.7 MB
        payload = NV.payload_bytes(n, k)
        byts = lambda m: payload + 2 * m * k + 2 * m * n
        flops = lambda m: 2.0 * m * n * k
        if on("nvfp4"):
            c0 = {}
            m = 1
            xb = torch.randn(m, k, generator=gen, device=dev).to(torch.bfloat16)
            yb = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
            q4 = blob_of(m, k, 256.0)
            us, clk = _timed_cell(b, [lambda v=v: b.linear_q4(q4, 256.0, v, None, m, yb=yb) for v in views], graph)
            c0["fp4_blob_in"] = _hbm_cell(us, byts(m), peaks, clk, note="activations arrive as the NVFP4 blob a producer wrote")
            us, clk = _timed_cell(b, [lambda v=v: b.linear_bf16(xb, v, None, m, yb=yb) for v in views], graph)
            c0["bf16_in"] = _hbm_cell(us, byts(m), peaks, clk, note="bf16 x in, NVFP4 rounding (AllowA4): quantiser launch included")
            a16 = [v.with_act(ActPolicy.a16_only()) for v in views]
            us, clk = _timed_cell(b, [lambda v=v: b.linear_bf16(xb, v, None, m, yb=yb) for v in a16], graph)
            c0["bf16_in_a16only"] = _hbm_cell(us, byts(m), peaks, clk, note="bf16 activations kept (A16Only view): unpacking GEMV")
            out["config0_decode_gemv_nvfp4_25600x5120_m1"] = c0
            m = 2048
            xb = torch.randn(m, k, generator=gen, device=dev).to(torch.bfloat16)
            yb = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
            calls = [lambda v=v: b.linear_bf16(xb, v, None, m, yb=yb) for v in views]
            us, _ = _timed_cell(b, calls, graph, burst_only=True)
            us_s, clk = _timed_cell(b, calls, graph)
            q4 = blob_of(m, k, 256.0)
            us_q, _ = _timed_cell(b, [lambda v=v: b.linear_q4(q4, 256.0, v, None, m, yb=yb) for v in views], graph,
                                  burst_only=True)
            out["config1_prefill_gemm_nvfp4_25600x5120_m2048"] = {
                "burst": _tensor_cell(us, flops(m), peaks, None, note="bf16 x in: quantiser launch included; a burst of launches"),
                "burst_fp4_blob_in": _tensor_cell(us_q, flops(m), peaks, None,
                                                  note="the GEMM launch alone: activations arrive as the NVFP4 blob a producer wrote"),
                "sustained": _tensor_cell(us_s, flops(m), peaks, clk, sustained=True, note="0.5 s under the power cap")}
            del xb, yb, q4
        if on("sweep"):
            sweep = {}
            for m in (1, 4, 16, 64, 256, 2048):
                xb = torch.randn(m, k, generator=gen, device=dev).to(torch.bfloat16)
                yb = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
                q4 = blob_of(m, k, 256.0)
                kern = _kernel_class(b, lambda: b.linear_q4(q4, 256.0, views[0], None, m, yb=yb))
                us, clk = _timed_cell(b, [lambda v=v: b.linear_q4(q4, 256.0, v, None, m, yb=yb) for v in views], graph)
                cell = _hbm_cell(us, byts(m), peaks, clk, kernel=kern)
                cell["TFLOP/s"] = round(flops(m) / (us * 1e-6) / 1e12, 1)
                sweep[f"m{m}"] = cell
                del xb, yb
            sweep["crossover"] = ("the dispatcher streams (decode kernel, weight rows as MMA M) up to 16 tokens and for "
                                  "17-64 tokens where its cost model expects few GEMM tiles with a long K; otherwise the "
                                  "GEMM (tokens as MMA M): 'kernel' says which ran")
            out["config1_m_sweep_fp4_blob_in"] = sweep
        del views
        torch.cuda.empty_cache()

    if on("mlp"):
        w, k = 25600, 5120
        mlps = []
        for _ in range(2):   # 2 x 221 MB
            gu = torch.randn(2 * w, k, generator=gen, device=dev) * 0.02
            parent = WeightView.full(b.encode_nvfp4(gu), NV, 2 * w, k).with_act(ActPolicy.allow_a4(256.0))
            del gu
            dn = torch.randn(k, w, generator=gen, device=dev) * 0.02
            down = WeightView.full(b.encode_nvfp4(dn), NV, k, w).with_act(ActPolicy.allow_a4(16.0))
            del dn
            mlps.append((parent.rows_view(0, w), parent.rows_view(w, w), down))
        mlp_bytes = NV.payload_bytes(2 * w, k) + NV.payload_bytes(k, w)
        cells = {}
        for m in (1, 16, 2048):
            q4 = blob_of(m, k, 256.0)
            hq = b.q4_blob(m, w)
            yb = torch.empty(m, k, dtype=torch.bfloat16, device=dev)

            def mlp(g, u, d):
                b.linear_swiglu_q4_to_q4(q4, 256.0, g, u, m, hq, 16.0)
                b.linear_q4(hq, 16.0, d, None, m, yb=yb)
            us, clk = _timed_cell(b, [lambda t=t: mlp(*t) for t in mlps], graph)
            if m <= 16:
                cells[f"m{m}"] = _hbm_cell(us, mlp_bytes + 2 * m * k * 2, peaks, clk, unit="per MLP (2 launches)")
            else:
                cells[f"m{m}"] = _tensor_cell(us, 6.0 * m * w * k, peaks, clk, sustained=True, unit="per MLP (2 launches)")
        cells["form"] = ("norm-written NVFP4 blob -> fused gate|up SwiGLU whose epilogue emits down's NVFP4 input -> down "
                         "(bf16 out); gate|up one [51200, 5120] parent")
        out["config2_mlp_nvfp4"] = cells
        del mlps
        torch.cuda.empty_cache()

    if on("formats"):
        n, k = 14336, 4096
        fm = {}
        for name, fmt, copies, policies in (("fp8_rows", F8, 7, (("a16", ActPolicy.a16_only()), ("a8", ActPolicy.allow_a8()))),
                                            ("q4_k", Q4, 12, (("a16", ActPolicy.a16_only()),))):
            payload = fmt.payload_bytes(n, k)
            bufs = []
            for _ in range(copies):   # > 3 x L2 in total
                buf = torch.randint(0, 120, (payload + 256,), generator=gen, dtype=torch.uint8, device=dev)
                if fmt is F8:
                    off = (n * k + 255) // 256 * 256
                    buf[off:off + 2 * n].view(torch.bfloat16).fill_(0.01)      # bf16 row scales
                else:
                    blocks = buf[:payload].view(-1, 144)
                    blocks[:, 1] = 0x20                                        # f16 d and dmin: small, finite
                    blocks[:, 3] = 0x20
                bufs.append(buf)
            for pname, policy in policies:
                views = [WeightView.full(buf, fmt, n, k).with_act(policy) for buf in bufs]
                for m in (1, 8, 512):
                    xb = torch.randn(m, k, generator=gen, device=dev).to(torch.bfloat16)
                    yb = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
                    kern = _kernel_class(b, lambda: b.linear_bf16(xb, views[0], None, m, yb=yb))
                    us, clk = _timed_cell(b, [lambda v=v: b.linear_bf16(xb, v, None, m, yb=yb) for v in views], graph)
                    cell = _hbm_cell(us, payload + 2 * m * k + 2 * m * n, peaks, clk, kernel=kern,
                                     act=str(b.linear_act(views[0], m)))
                    if m > 16:
                        cell["TFLOP/s"] = round(2.0 * m * n * k / (us * 1e-6) / 1e12, 1)
                    fm[f"{name}_{pname}_m{m}"] = cell
                    del xb, yb
            del bufs
        fm["data"] = "seeded random stored bytes with finite codes and sane scales; bf16 x in (quantiser launches included)"
        out["config3_14336x4096"] = fm
        torch.cuda.empty_cache()

    if on("decode_stack") and stack is not None:
        spec = stack.spec
        x1 = torch.randn(1, spec.hidden, generator=gen, device=dev).to(torch.bfloat16)
        fwd = lambda: stack.forward(x1, 1)
        for _ in range(2):
            fwd()
        us, clk = _timed_cell(b, [fwd], graph, rounds=2)          # us per step = per token
        cell = _hbm_cell(us, stack.weight_bytes, peaks, clk)
        cell["tok/s"] = round(1e6 / us, 1)
        cell["ms_per_token"] = round(us / 1e3, 3)
        cell["launches_per_token"] = int(stack.launches_per_step)
        out["config4_decode_stack_m1"] = cell
    return out


if __name__ == "__main__":
    main()
