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


def test_scale_out_plan_covers_every_row_once_and_samples_sit_inside():
    from rnn_with_grm_b200 import scale_out as so

    shape = so.ScaleOutShape()
    assert (shape.rows, shape.tokens, shape.dim, shape.segment, shape.top_k, shape.segments) == (4096, 32768, 128, 1024, 8, 32)
    assert shape.batch_tokens == 256 * 32768 and shape.scan_bytes_per_row() == 32768 * 1024
    for world in (1, 2, 4, 8):
        covered = []
        for rank in range(world):
            slabs = so.plan_slabs(shape, rank, world, 256)
            assert len(slabs) == 16 // world and all(b - a == 256 for a, b in slabs)
            ragged = so.plan_slabs(shape, rank, world, 296)          # the last slab of a rank takes what is left
            assert sum(b - a for a, b in ragged) == 4096 // world and all(b - a == 296 for a, b in ragged[:-1])
            covered += [r for a, b in slabs for r in (a, b)]
            start, stop = row_range(shape.rows, rank, world)
            picks = so.sample_rows(shape, rank, world, 2)
            assert picks == [start, stop - 1]
            assert so.sample_rows(shape, rank, world, 3)[1] == start + round((stop - 1 - start) / 2)
        assert covered[0] == 0 and covered[-1] == 4096 and covered[1:-1:2] == covered[2::2]
    small = so.ScaleOutShape(rows=10, heads=2, tokens=256, dim=8, segment=64, top_k=2)
    assert so.plan_slabs(small, 1, 3, 2) == [(4, 6), (6, 7)] and so.sample_rows(small, 2, 3, 5) == [7, 8, 9]
    assert so.n_slabs_for(small, 3, 2) == 2
    # the routed matrices of a row: min(top_k, j) for segment j
    assert so.scale_out_bytes(small, 1) == small.scan_bytes_per_row() + 4 * 8 * 8 * 4 + (0 + 1 + 2 + 2) * 8 * 8 * 4


def test_verification_rows_regenerate_from_their_seed_and_round_trip_through_the_gather_vector():
    from rnn_with_grm_b200 import scale_out as so

    shape = so.ScaleOutShape(rows=6, heads=2, tokens=128, dim=16, segment=32, top_k=3)
    a, b = so.host_row_inputs(shape, 4), so.host_row_inputs(shape, 4)
    assert all(torch.equal(x, y) for x, y in zip(a, b))
    assert not torch.equal(a[0], so.host_row_inputs(shape, 5)[0])
    q, k, v, online = a
    assert q.dtype == torch.bfloat16 and tuple(q.shape) == (128, 16) and tuple(online.shape) == (4, 16)
    assert float((q.float().norm(dim=-1) - 1).abs().max()) < 1e-2
    hidden = torch.randn(128, 16).to(torch.bfloat16)
    m_out, fused = torch.randn(16, 16), torch.randn(4, 16)
    indices = torch.tensor([[-1, -1, -1], [0, -1, -1], [0, 1, -1], [2, 0, 1]])
    flat = so.pack_sample(hidden, m_out, fused, indices)
    assert flat.numel() == so.sample_vector_len(shape)
    h2, m2, f2, i2 = so.unpack_sample(flat, shape)
    assert torch.equal(h2, hidden.float()) and torch.equal(m2, m_out) and torch.equal(f2, fused) and torch.equal(i2, indices)


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
        # verification rows of the scale-out form: every rank contributes the same number of flat sample
        # vectors, rank 0 reads them back in global row order
        from rnn_with_grm_b200 import scale_out as so
        shape = so.ScaleOutShape(rows=6, heads=2, tokens=64, dim=8, segment=32, top_k=2)
        picks = so.sample_rows(shape, rank, world, 2)
        local = torch.stack([torch.full((so.sample_vector_len(shape),), float(row)) for row in picks])
        everyone = gather_rows(local, len(picks) * world)
        expected = [row for r in range(world) for row in so.sample_rows(shape, r, world, 2)]
        ok = ok and everyone[:, 0].tolist() == [float(r) for r in expected] and expected == sorted(expected)
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
