"""The multi-rank host logic on CPU: two gloo ranks shard the rows of a scan, each checks its
slice against the oracle, and the gathered result equals the unsharded one."""

import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from rnn_with_grm_b200.sharding import all_row_ranges, row_range

ROOT = Path(__file__).resolve().parent.parent


def test_row_ranges_cover_every_row_once():
    for n_rows in (0, 1, 7, 64, 4096):
        for world in (1, 2, 3, 8):
            ranges = all_row_ranges(n_rows, world)
            assert ranges[0][0] == 0 and ranges[-1][1] == n_rows
            assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
            sizes = [stop - start for start, stop in ranges]
            assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)
    assert row_range(64, 3, 8) == (24, 32)
    with pytest.raises(ValueError):
        row_range(8, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    from oracle import grm_oracle as go
    from rnn_with_grm_b200.sharding import gather_rows, shard_rows

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(0)                      # same inputs on every rank
        rows, T, K, H = 5, 24, 8, 6
        k, q = rng.standard_normal((rows, T, K)), rng.standard_normal((rows, T, K))
        v, m = rng.standard_normal((rows, T, H)), rng.standard_normal((rows, H, K))
        full_h, full_m = go.chunk_update_sequential(k, v, q, m, 0.97)
        mine = [shard_rows(torch.from_numpy(a), rank, world).numpy() for a in (k, v, q, m)]
        h, m_out = go.chunk_update_sequential(*mine, 0.97)  # stands in for the rank's GPU work
        gathered_h = gather_rows(torch.from_numpy(h), rows)
        gathered_m = gather_rows(torch.from_numpy(m_out), rows)
        ok = np.array_equal(gathered_h.numpy(), full_h) and np.array_equal(gathered_m.numpy(), full_m)
        # timing convention of the benchmark: MAX over ranks of the per-rank time
        t = torch.tensor([float(rank + 1)])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ok = ok and float(t) == float(world)
        Path(out_dir, f"rank{rank}.ok").write_text("1" if ok else "0")
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_shard_and_gather(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert [Path(tmp_path, f"rank{r}.ok").read_text() for r in range(world)] == ["1", "1"]
