"""One rank of the multi-GPU checks of the fused tensor-parallel step (started by
test_gpu_tp_fused.py through torch.distributed.run).

Exact checks, phase by phase and for whole steps:
  * the partial-sum tiles a row-split linear scatters into the owners' slots are the bits the same
    linear writes to a local buffer, and those match the oracle's linear on this rank's K-slice;
  * the residual after the fused norm is the f32 sum, in rank order, of the slots, and the NVFP4 blob
    every rank holds afterwards is the oracle's quantiser applied to the norm's bf16 result;
  * whole steps of `forward_fused_tp` equal `forward_gathered` (library all-gather, same arithmetic)
    bit for bit, repeatedly, and every rank ends with the same output; so do the same steps run as
    two token chunks on streams of their own;
and, because a sharded step rounds each shard's partial sums to bf16, a statistical check against the
unsharded step on one GPU."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from oracle import oracle as O  # noqa: E402
from velox_inferer_b200 import Sm100Backend  # noqa: E402
from velox_inferer_b200.stack import (DIV_NORM_OUT, DIV_O_IN, ChunkedStack, LinearStack, StackSpec,
                                      fused_step_schedule)  # noqa: E402


def rel_rms(a, c):
    return ((a - c).pow(2).mean().sqrt() / c.pow(2).mean().sqrt()).item()


def decode_blob(q4, m, k, divisor):
    """The values an NVFP4 activation blob stands for: it has the layout of an NVFP4 weight [m, k]."""
    plane = (m * k // 2 + 255) // 256 * 256
    payload = np.zeros(plane + m * k // 16 + 4, dtype=np.uint8)
    payload[: m * k // 2] = q4[0].cpu().numpy()[: m * k // 2]
    payload[plane:plane + m * k // 16] = q4[1].cpu().numpy()[: m * k // 16]
    payload[plane + m * k // 16:] = np.frombuffer(np.float32(divisor).tobytes(), dtype=np.uint8)
    return O.decode_rows(O.FMT_NVFP4, payload, m, k, 0, m)


def check_phases(b, stack, xb, rank, world):
    """The first layer's norm -> q|k|v -> o-scatter -> norm, one launch at a time."""
    s, f = stack.spec, stack.fabric
    h, m, rows = s.hidden, f.m, f.rows
    r0 = rank * rows
    l = stack.layers[0]
    sched = [e for e in fused_step_schedule(len(stack.layers)) if e[1] == 0]
    x_own = stack.x[: rows * h]
    x_own.copy_(xb.reshape(-1)[r0 * h:(r0 + rows) * h])
    b.tp_step_begin(f.epoch)
    # norm (no addend) -> every rank's blob
    _, _, wait, signal = sched[0]
    b.tp_norm_q4(x_own, f.slots, 0, rows * h, stack.norm_w, f.codes_ptrs, f.atoms_ptrs, r0, rows, h, s.norm_eps,
                 DIV_NORM_OUT, sync=f.sync(wait, signal))
    # q|k|v wait for all rows of the blob
    stack._qkv(l, (f.codes, f.atoms), m, True, sync=f.sync(sched[1][2], -1))
    torch.cuda.synchronize()
    # the blob on this rank = the oracle's quantiser on the bf16 norm of ALL rows
    full = xb.float().cpu().numpy().reshape(m, h)
    normed = O.quantize_activations(O.rms_norm(full, np.ones(h, np.float32), s.norm_eps).reshape(-1), h, O.ACT_BF16)
    codes, scales = O.act_codes_nvfp4(normed.reshape(m, h), DIV_NORM_OUT)
    got_codes = f.codes.cpu().numpy().reshape(m, h // 2)
    # the kernel's f32 norm and the oracle's f64 norm round a few values to neighbouring bf16 numbers
    assert np.mean(got_codes != codes) < 2e-3, np.mean(got_codes != codes)
    # o: scatter into the owners' slots; the same linear into a local buffer
    b.tp_linear_q4_scatter(stack.qq, DIV_O_IN, l.o, m, f.maps, rows, sync=f.sync(-1, sched[2][3]))
    b.linear_q4(stack.qq, DIV_O_IN, l.o, None, m, yb=stack.pb)
    b.tp_wait(f.sync(sched[2][3], -1))
    torch.cuda.synchronize()
    assert b.debug_status() == 0
    gathered = [torch.empty_like(stack.pb) for _ in range(world)]
    dist.all_gather(gathered, stack.pb)
    for src in range(world):
        slot = f.slots[src * rows * h:(src + 1) * rows * h]
        assert torch.equal(slot, gathered[src][r0 * h:(r0 + rows) * h]), ("slot", src)
    # this rank's partial sums against the oracle on its K-slice (input: the q blob it holds, decoded)
    qv = decode_blob(stack.qq, m, s.q_dim // world, DIV_O_IN)
    toks = np.unique(np.concatenate([np.arange(8), np.arange(m - 8, m)]))
    want = O.linear(np.ascontiguousarray(qv[toks]), l.o.buf.cpu().numpy(), O.FMT_NVFP4, h, l.o.k, 0, h, len(toks),
                    act=O.ACT_EXACT)
    got = stack.pb.float().cpu().numpy().reshape(m, h)[toks]
    assert O.max_err(got, want) <= 2.0 ** -8, O.max_err(got, want)      # bf16 output: half a unit in the last place
    # norm: residual += slots in rank order (f32), blob = quantiser(bf16 norm)
    x_before = x_own.clone()
    part = f.slots[: rows * h].float()
    for src in range(1, world):
        part = part + f.slots[src * rows * h:(src + 1) * rows * h].float()
    b.tp_norm_q4(x_own, f.slots, world, rows * h, stack.norm_w, f.codes_ptrs, f.atoms_ptrs, r0, rows, h, s.norm_eps,
                 DIV_NORM_OUT, sync=f.sync(sched[3][2], sched[3][3]))
    b.tp_wait(f.sync(sched[3][3], -1))
    torch.cuda.synchronize()
    assert b.debug_status() == 0
    assert torch.equal(x_own, x_before + part)
    # every rank's rows of the blob: the single-GPU norm + quantiser on the gathered residual, bit for bit
    xs = [torch.empty_like(x_own) for _ in range(world)]
    dist.all_gather(xs, x_own.contiguous())
    x_all = torch.cat(xs)
    q4 = b.q4_blob(m, h)
    yb = torch.zeros(m * h, dtype=torch.bfloat16, device=b.device)
    b.add_rms_norm_q4(x_all, None, stack.norm_w, yb, q4, m, h, s.norm_eps, DIV_NORM_OUT)
    torch.cuda.synchronize()
    assert torch.equal(f.codes, q4[0]) and torch.equal(f.atoms, q4[1])
    wc, _ = O.act_codes_nvfp4(yb.float().cpu().numpy().reshape(m, h), DIV_NORM_OUT)
    assert np.array_equal(f.codes.cpu().numpy().reshape(m, h // 2), wc)      # = the oracle's quantiser on the bf16 norm
    torch.cuda.synchronize()
    dist.barrier()                # nobody starts the next step (which overwrites the blobs) while a peer still compares


def main() -> None:
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    b = Sm100Backend(local)
    spec = StackSpec(layers=3, hidden=512, intermediate=1024, heads=4 * world // 2, kv_heads=world, head_dim=128)
    m = 128 * world * 2
    stack = LinearStack(b, spec, max_tokens=m, rank=rank, world=world, a4=True, seed=5)
    x = torch.from_numpy(np.random.default_rng(9).standard_normal((m, spec.hidden)).astype(np.float32))
    xb = x.to(torch.bfloat16).to(b.device)
    ref = stack.forward(xb, m).float().clone()
    exact = stack.forward_gathered(xb, m).clone()
    whole = LinearStack(b, spec, max_tokens=m, rank=0, world=1, a4=True, seed=5).forward(xb, m).float().clone()
    err_nccl = rel_rms(ref, whole)
    assert err_nccl <= 0.08, ("all-reduce step vs unsharded", err_nccl)
    for mode in ("flags", "kernel", "barrier"):
        assert stack.enable_fused_tp(m, sync_mode=mode)
        if mode == "flags":
            check_phases(b, stack, xb, rank, world)
        for _ in range(3):                                   # repeatedly: buffers and flags are reused between steps
            got = stack.forward_fused_tp(xb).clone()
            torch.cuda.synchronize()
            assert b.debug_status() == 0
            assert torch.equal(got.view(-1)[: m * spec.hidden], exact.view(-1)[: m * spec.hidden]), mode
        err = rel_rms(got.float(), whole)
        assert err <= 0.08 and err <= 2.0 * err_nccl + 0.01, ("fused step vs unsharded", err, "all-reduce step", err_nccl)
        # the same as a CUDA graph, replayed
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            stack.forward_fused_tp(xb)
        torch.cuda.synchronize()
        dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            stack.forward_fused_tp(xb)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        assert b.debug_status() == 0
        assert torch.equal(stack.fabric.out.view(-1)[: m * spec.hidden], exact.view(-1)[: m * spec.hidden]), (mode, "graph")
        graph.reset()
        del graph
        # every rank holds the same full output
        mine = got.contiguous()
        others = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(others, mine)
        for o in others:
            assert torch.equal(o, mine)
        dist.barrier()
    # the same step as two token chunks side by side on streams of their own, eagerly and as a graph
    chunked = ChunkedStack(b, spec, m, rank, world, chunks=2, seed=5)
    assert chunked.enable_fused_tp(m, sync_mode="kernel")
    for _ in range(3):
        got = chunked.forward_fused_tp(xb).clone()
        torch.cuda.synchronize()
        assert b.debug_status() == 0
        assert torch.equal(got[: m * spec.hidden], exact.view(-1)[: m * spec.hidden]), "chunked"
    dist.barrier()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        chunked.forward_fused_tp(xb)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    assert b.debug_status() == 0
    assert torch.equal(chunked.out[: m * spec.hidden], exact.view(-1)[: m * spec.hidden]), "chunked graph"
    graph.reset()
    del graph
    dist.barrier()
    if rank == 0:
        print("TP_FUSED_OK", world, err, err_nccl, flush=True)
    torch.cuda.synchronize()
    dist.barrier()
    os._exit(0)


if __name__ == "__main__":
    try:
        main()
    except BaseException:      # the launcher's own report drops a rank's traceback: say it where the test looks
        import traceback

        print(f"TP_FUSED_FAIL rank {os.environ.get('RANK')}:\n{traceback.format_exc()}", flush=True)
        os._exit(1)
