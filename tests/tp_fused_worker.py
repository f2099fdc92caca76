"""One rank of the two-GPU check of the fused tensor-parallel step (started by
test_gpu_tp_fused.py through torch.distributed.run): the step with the reduce-scatter fused into
the row-split GEMMs and the all-gather into the norm must agree with the NCCL all-reduce step."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from velox_inferer_b200 import Sm100Backend  # noqa: E402
from velox_inferer_b200.stack import LinearStack, StackSpec  # noqa: E402


def main() -> None:
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    b = Sm100Backend(local)
    spec = StackSpec(layers=3, hidden=512, intermediate=1024, heads=4, kv_heads=2, head_dim=128)
    m = 128 * world * 2
    stack = LinearStack(b, spec, max_tokens=m, rank=rank, world=world, a4=True, seed=5)
    x = torch.from_numpy(np.random.default_rng(9).standard_normal((m, spec.hidden)).astype(np.float32))
    xb = x.to(torch.bfloat16).to(b.device)
    ref = stack.forward(xb, m).float().clone()
    # The same weights unsharded on this GPU. A sharded step rounds each shard's partial sums to
    # bf16, and FP4 activation quantisation downstream turns those last-bit differences into
    # occasional one-step code changes, so the comparison is statistical: relative RMS error of a
    # few percent, and the fused step no further from the unsharded one than the all-reduce step.
    whole = LinearStack(b, spec, max_tokens=m, rank=0, world=1, a4=True, seed=5).forward(xb, m).float().clone()

    def rel_rms(a, c):
        return ((a - c).pow(2).mean().sqrt() / c.pow(2).mean().sqrt()).item()

    err_nccl = rel_rms(ref, whole)
    assert err_nccl <= 0.08, ("all-reduce step vs unsharded", err_nccl)
    assert stack.enable_fused_tp(m)
    for _ in range(2):                                   # twice: buffers are reused between steps
        got = stack.forward_fused_tp(xb).float().clone()
        torch.cuda.synchronize()
        assert b.lib.velox_sm100_debug_status() == 0
        assert torch.isfinite(got).all()
        err = rel_rms(got, whole)
        assert err <= 0.08 and err <= 2.0 * err_nccl + 0.01, ("fused step vs unsharded", err, "all-reduce step", err_nccl)
    # every rank holds the same full output
    mine = got.contiguous()
    others = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(others, mine)
    for o in others:
        assert torch.equal(o, mine)
    if rank == 0:
        print("TP_FUSED_OK", err, err_nccl, flush=True)
    torch.cuda.synchronize()
    dist.barrier()
    os._exit(0)


if __name__ == "__main__":
    main()
