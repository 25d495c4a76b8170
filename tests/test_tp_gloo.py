"""Tensor-parallel sharding on CPU: two gloo ranks each run their shard through
the CPU oracle, row-parallel partials are summed with a gloo allreduce, and the
result must match the unsharded oracle (the layout under test is the one
tgaf_weight_upload applies on each rank)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from talu_b200 import tp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from oracle import gaf_oracle as oracle
    rng = np.random.default_rng(0)           # every rank builds the same full weights
    G, bits, M = 64, 4, 3
    hidden, ffn = 512, 1024
    w_up = rng.standard_normal((ffn, hidden), dtype=np.float32) * np.float32(0.02)
    w_down = rng.standard_normal((hidden, ffn), dtype=np.float32) * np.float32(0.02)
    up = oracle.quantize(w_up, G, bits, nthreads=1)
    down = oracle.quantize(w_down, G, bits, nthreads=1)
    x = rng.standard_normal((M, hidden), dtype=np.float32)

    # column-parallel up: this rank's rows; its output is this rank's slice of the hidden state
    s_up = tp.shard_slice(ffn, hidden, G, bits, tp.SHARD_COL, rank, world)
    h_local = oracle.matmul_f32(x, *tp.slice_arrays(*up, G, bits, s_up), G, bits, nthreads=1)
    # row-parallel down: this rank's columns take exactly that slice; outputs are partial sums
    s_dn = tp.shard_slice(hidden, ffn, G, bits, tp.SHARD_ROW, rank, world)
    assert (s_dn.k0, s_dn.k1) == (s_up.n0, s_up.n1)
    y_part = oracle.matmul_f32(h_local, *tp.slice_arrays(*down, G, bits, s_dn), G, bits, nthreads=1)
    y = torch.from_numpy(y_part.copy())
    dist.all_reduce(y)                        # the one exchange step of the path

    h_full = oracle.matmul_f32(x, *up, G, bits, nthreads=1)
    y_full = oracle.matmul_f32(h_full, *down, G, bits, nthreads=1)
    np.save(os.path.join(out_dir, f"err_{rank}.npy"),
            np.array([np.abs(y.numpy() - y_full).max(), np.abs(y_full).max()]))
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_col_then_row_parallel_matches_unsharded(tmp_path, world):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        err, scale = np.load(tmp_path / f"err_{r}.npy")
        assert err <= 1e-4 * max(1.0, scale), (r, err, scale)


def test_shard_slice_rules():
    # qkv / gate / up: rows; o / down: columns on group boundaries
    s = tp.shard_slice(10240, 8192, 64, 4, tp.SHARD_COL, 3, 8)
    assert (s.n0, s.n1, s.k0, s.k1) == (3840, 5120, 0, 8192)
    s = tp.shard_slice(8192, 28672, 64, 4, tp.SHARD_ROW, 7, 8)
    assert (s.n0, s.n1, s.k0, s.k1) == (0, 8192, 25088, 28672) and s.k % 64 == 0
    with pytest.raises(ValueError):
        tp.shard_slice(10, 8192, 64, 4, tp.SHARD_COL, 0, 4)          # N not divisible
    with pytest.raises(ValueError):
        tp.shard_slice(8, 192, 64, 4, tp.SHARD_ROW, 0, 2)            # K/P not a whole number of groups
    with pytest.raises(ValueError):
        tp.shard_slice(8, 128, 64, 4, tp.SHARD_ROW, 2, 2)            # rank out of range
    full = tp.shard_slice(8, 128, 64, 4, tp.SHARD_NONE, 0, 1)
    assert (full.n, full.k) == (8, 128)
    # every (row, column) of the full weight belongs to exactly one rank
    for kind in (tp.SHARD_COL, tp.SHARD_ROW):
        cover = np.zeros((16, 256), np.int32)
        for r in range(4):
            sl = tp.shard_slice(16, 256, 64, 4, kind, r, 4)
            cover[sl.n0:sl.n1, sl.k0:sl.k1] += 1
        assert (cover == 1).all()
