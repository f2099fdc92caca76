"""The flag protocol of the fused tensor-parallel step, run on CPU ranks (gloo, world size 2 and
3): every launch of `fused_step_schedule` becomes a host function that waits on the flag row the
schedule names, reads and writes tagged stand-ins for the buffers the kernels share (blob rows,
partial-sum slots, output rows), and raises the row the schedule names. The tags prove both
directions of every dependency: a reader finds exactly the version its step and layer expect, never
an older one (read too early) nor a newer one (overwritten too early), under random delays.

A second case takes a rank out for a whole step: the others' waits run out after their limit, each
records the status code the kernels use (6) and finishes its step instead of hanging - the
host-side form of the failure the device-side bounded waits are for. No GPU is involved."""
import os
import random
import time

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from velox_inferer_b200.stack import TpFabric, fused_step_schedule

ST_TIMEOUT_PEER = 6


class HostRank:
    """One rank's view of the shared tables (tensors in shared memory, one row per rank)."""

    def __init__(self, rank, world, flags, blob, slots, outp, limit_s):
        self.rank, self.world, self.flags, self.blob, self.slots, self.outp = rank, world, flags, blob, slots, outp
        self.limit_s, self.epoch, self.status, self.errors = limit_s, 0, 0, []

    def wait(self, phase):
        if phase < 0:
            return
        t0 = time.time()
        for src in range(self.world):
            while int(self.flags[self.rank, phase, src]) - self.epoch < 0:
                if time.time() - t0 > self.limit_s:
                    self.status = ST_TIMEOUT_PEER
                    return
                time.sleep(0.0002)

    def signal(self, phase):
        if phase >= 0:
            for d in range(self.world):
                self.flags[d, phase, self.rank] = self.epoch

    def expect(self, what, got, want):
        if self.status == 0 and got != want:
            self.errors.append((what, self.epoch, got, want))

    def run_step(self, layers, jitter, drop_wait=None):
        self.epoch += 1
        for op, li, wait, signal in fused_step_schedule(layers):
            if op != drop_wait:
                self.wait(wait)
            if jitter:
                time.sleep(random.random() * 0.002)
            tag = self.epoch * 1000 + li * 10
            if op == "norm":
                first = wait < 0 or wait % TpFabric.PHASES_PER_LAYER == 3       # the norm ahead of q|k|v
                if wait >= 0:                                                   # reads every source's slot
                    want = tag + 1 if not first else self.epoch * 1000 + (li - 1) * 10 + 2
                    for src in range(self.world):
                        self.expect("slot", int(self.slots[self.rank, src]), want)
                for d in range(self.world):                                     # its rows of every rank's blob
                    self.blob[d, self.rank] = tag + (3 if first else 4)
            elif op in ("qkv", "gate_up"):                                      # reads all rows of its own blob
                for owner in range(self.world):
                    self.expect("blob", int(self.blob[self.rank, owner]), tag + (3 if op == "qkv" else 4))
            elif op in ("o_scatter", "down_scatter"):                           # its slot on every owner
                for d in range(self.world):
                    self.slots[d, self.rank] = tag + (1 if op == "o_scatter" else 2)
            elif op == "finish":
                for src in range(self.world):
                    self.expect("slot", int(self.slots[self.rank, src]), self.epoch * 1000 + (li - 1) * 10 + 2)
                for d in range(self.world):
                    self.outp[d, self.rank] = self.epoch
            elif op == "wait":
                for owner in range(self.world):
                    self.expect("out", int(self.outp[self.rank, owner]), self.epoch)
            self.signal(signal)


def _rank_main(rank, world, port, shared, layers, steps, skip, limit_s, out, drop_wait):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        random.seed(100 + rank)
        r = HostRank(rank, world, *shared, limit_s)
        t0 = time.time()
        statuses = []
        for step in range(steps):
            if (rank, step) == skip:
                r.epoch += 1                      # this rank never runs the step: no waits, no signals
                statuses.append(-1)
                continue
            r.status = 0
            r.run_step(layers, jitter=True, drop_wait=drop_wait)
            statuses.append(r.status)
        result = [None] * world
        dist.all_gather_object(result, (statuses, r.errors[:4], time.time() - t0))
        if rank == 0:
            with open(out, "w") as f:
                f.write(repr(result))
    finally:
        dist.destroy_process_group()


def _run(world, layers, steps, skip, limit_s, tmp_path, port_base, drop_wait=None):
    phases = TpFabric.PHASES_PER_LAYER * layers + 1
    shared = (torch.zeros(world, phases, 8, dtype=torch.int32).share_memory_(),     # flag tables
              torch.zeros(world, world, dtype=torch.int64).share_memory_(),          # blob[rank][row owner]
              torch.zeros(world, world, dtype=torch.int64).share_memory_(),          # slots[owner][source]
              torch.zeros(world, world, dtype=torch.int64).share_memory_())          # out[rank][row owner]
    out = str(tmp_path / "result.txt")
    mp.spawn(_rank_main, args=(world, port_base + os.getpid() % 2000, shared, layers, steps, skip, limit_s, out,
                                  drop_wait),
             nprocs=world, join=True)
    return eval(open(out).read())


def test_schedule_orders_every_shared_buffer_in_both_directions(tmp_path):
    for world, port in ((2, 33500), (3, 35500)):
        result = _run(world, layers=3, steps=4, skip=None, limit_s=20.0, tmp_path=tmp_path, port_base=port)
        for statuses, errors, _ in result:
            assert statuses == [0, 0, 0, 0]
            assert errors == []


def test_a_rank_that_skips_a_step_costs_the_others_a_bounded_wait_and_a_status(tmp_path):
    result = _run(2, layers=2, steps=3, skip=(1, 1), limit_s=0.15, tmp_path=tmp_path, port_base=37500)
    (st0, _, secs0), (st1, _, _) = result
    assert st1[1] == -1
    assert st0[0] == 0 and st0[1] == ST_TIMEOUT_PEER      # the step without the peer reports, and ends
    assert secs0 < 20.0


def test_the_tags_notice_a_launch_that_does_not_wait(tmp_path):
    """The checker checks: with the wait of one kind of launch left out, some rank reads a buffer
    version it should not."""
    for op, port in (("qkv", 39500), ("norm", 41500)):
        result = _run(2, layers=3, steps=6, skip=None, limit_s=20.0, tmp_path=tmp_path, port_base=port, drop_wait=op)
        assert any(errors for _, errors, _ in result), op
