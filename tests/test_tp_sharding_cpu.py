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
