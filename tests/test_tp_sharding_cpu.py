"""Tensor-parallel sharding of NVFP4 weights, checked on CPU ranks (gloo, world size 2) against
the unsharded oracle: the column split is a row view re-based as its own parent, the row split a
K-slice re-layout of stored bytes; neither re-quantises, so decoded values are identical and the
all-reduced partial products equal the unsharded product up to f32 summation order."""
import os

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle as O
from velox_inferer_b200.stack import slice_k_nvfp4, slice_rows_nvfp4


def _payload(n, k, seed):
    w = (np.random.default_rng(seed).standard_normal((n, k)) * 0.02).astype(np.float32)
    return O.encode_nvfp4_rne(w)


def test_column_and_row_slices_decode_to_the_same_values():
    n, k = 512, 640
    p = _payload(n, k, 0)
    full = O.decode_rows(O.FMT_NVFP4, p, n, k, 0, n)
    pt = torch.from_numpy(p.copy())
    for world in (2, 4):
        rows = n // world
        for r in range(world):
            shard = slice_rows_nvfp4(pt, n, k, r * rows, rows).numpy()
            got = O.decode_rows(O.FMT_NVFP4, shard, rows, k, 0, rows)
            assert np.array_equal(got, full[r * rows:(r + 1) * rows])
    for world in (2, 5):
        kl = k // world
        for r in range(world):
            shard = slice_k_nvfp4(pt, n, k, r * kl, kl).numpy()
            got = O.decode_rows(O.FMT_NVFP4, shard, n, kl, 0, n)
            assert np.array_equal(got, full[:, r * kl:(r + 1) * kl])


def _rank_main(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n_col, n_row, k, m = 256, 128, 256, 3
        x = (np.random.default_rng(5).standard_normal((m, k))).astype(np.float32)
        x = O.quantize_activations(x, k, O.ACT_BF16).reshape(m, k)
        p_col, p_row = _payload(n_col, k, 1), _payload(n_row, n_col, 2)
        # column split: this rank's rows of the first projection
        rows = n_col // world
        shard = slice_rows_nvfp4(torch.from_numpy(p_col.copy()), n_col, k, rank * rows, rows).numpy()
        h = O.linear(x, shard, O.FMT_NVFP4, rows, k, 0, rows, m)            # [m, rows]
        # row split: this rank's K-slice of the second projection, input = its own columns of h
        kshard = slice_k_nvfp4(torch.from_numpy(p_row.copy()), n_row, n_col, rank * rows, rows).numpy()
        part = torch.from_numpy(O.linear(h, kshard, O.FMT_NVFP4, n_row, rows, 0, n_row, m))
        dist.all_reduce(part)
        if rank == 0:
            h_full = O.linear(x, p_col, O.FMT_NVFP4, n_col, k, 0, n_col, m)
            want = O.linear(h_full, p_row, O.FMT_NVFP4, n_row, n_col, 0, n_row, m)
            err = O.max_err(part.numpy(), want)
            with open(out, "w") as f:
                f.write(repr(err))
    finally:
        dist.destroy_process_group()


def test_two_rank_megatron_split_matches_unsharded_oracle(tmp_path):
    out = str(tmp_path / "err.txt")
    port = 29500 + os.getpid() % 2000
    mp.spawn(_rank_main, args=(2, port, out), nprocs=2, join=True)
    assert float(open(out).read()) <= 1e-6


def _bf16(a):
    return O.quantize_activations(np.asarray(a, dtype=np.float32).reshape(-1), 1, O.ACT_BF16).reshape(np.shape(a))


def _fused_rank_main(rank, world, port, out):
    """The data flow of the fused tensor-parallel step, restated with the oracle on CPU ranks: the
    row-split projection's bf16 partial rows go to the rank that owns those token rows (scatter),
    the owner adds the slots in rank order to its rows of the residual, normalises them, quantises
    to NVFP4, and every rank ends up with all rows of the blob (gather)."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        hidden, kfull, m, div = 128, 256, 256, 256.0
        own = m // world
        rng = np.random.default_rng(11)
        resid = rng.standard_normal((m, hidden)).astype(np.float32)          # residual stream, all rows
        act = _bf16(rng.standard_normal((m, kfull)).astype(np.float32))      # input of the row-split projection
        p_row = _payload(hidden, kfull, 3)
        ks = kfull // world
        kshard = slice_k_nvfp4(torch.from_numpy(p_row.copy()), hidden, kfull, rank * ks, ks).numpy()
        part = _bf16(O.linear(act[:, rank * ks:(rank + 1) * ks].copy(), kshard, O.FMT_NVFP4, hidden, ks, 0, hidden, m))
        # scatter: every rank's partial rows of owner o end up in o's slot for that source rank
        gathered = [torch.empty(m, hidden) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(part))
        slots = [g.numpy()[rank * own:(rank + 1) * own] for g in gathered]    # slots[src]: my rows from src
        x_own = resid[rank * own:(rank + 1) * own].copy()
        total = slots[0].copy()
        for s in slots[1:]:
            total = (total + s).astype(np.float32)                            # rank order, f32
        x_own = (x_own + total).astype(np.float32)
        normed = _bf16(O.rms_norm(x_own, np.ones(hidden, np.float32), 1e-6))
        codes, scales = O.act_codes_nvfp4(normed, div)
        # gather: all rows of the blob on every rank
        all_codes = [torch.empty(own, hidden // 2, dtype=torch.uint8) for _ in range(world)]
        all_scales = [torch.empty(own, hidden // 16, dtype=torch.uint8) for _ in range(world)]
        dist.all_gather(all_codes, torch.from_numpy(codes))
        dist.all_gather(all_scales, torch.from_numpy(scales))
        blob_codes = torch.cat(all_codes).numpy()
        blob_scales = torch.cat(all_scales).numpy()
        # what the unsharded sequence gives when the shards' partials are added in rank order
        parts = []
        for r in range(world):
            kr = slice_k_nvfp4(torch.from_numpy(p_row.copy()), hidden, kfull, r * ks, ks).numpy()
            parts.append(_bf16(O.linear(act[:, r * ks:(r + 1) * ks].copy(), kr, O.FMT_NVFP4, hidden, ks, 0, hidden, m)))
        tot = parts[0].copy()
        for q in parts[1:]:
            tot = (tot + q).astype(np.float32)
        want_norm = _bf16(O.rms_norm((resid + tot).astype(np.float32), np.ones(hidden, np.float32), 1e-6))
        want_codes, want_scales = O.act_codes_nvfp4(want_norm, div)
        ok = np.array_equal(blob_codes, want_codes) and np.array_equal(blob_scales, want_scales)
        # and it stays close to the product with the unsharded weights
        full = O.linear(act, p_row, O.FMT_NVFP4, hidden, kfull, 0, hidden, m)
        err = O.max_err(tot, full)
        with open(f"{out}.{rank}", "w") as f:
            f.write(repr((bool(ok), float(err))))
    finally:
        dist.destroy_process_group()


def test_two_rank_scatter_norm_gather_equals_rank_ordered_sum(tmp_path):
    out = str(tmp_path / "fused")
    port = 31500 + os.getpid() % 2000
    mp.spawn(_fused_rank_main, args=(2, port, out), nprocs=2, join=True)
    for r in range(2):
        ok, err = eval(open(f"{out}.{r}").read())
        assert ok
        assert err <= 1e-2          # bf16 rounding of the two partial sums
