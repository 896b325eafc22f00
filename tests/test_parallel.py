"""Multi-rank host logic on CPU: world_size-2 gloo processes shard the
independent (kv head, batch) units, work on their block with no data-path
collective, and regather."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from nntile_b200 import parallel


def test_shard_range_partitions_exactly():
    for n in (0, 1, 7, 32, 96, 512):
        for world in (1, 2, 3, 4, 8):
            blocks = [parallel.shard_range(n, r, world) for r in range(world)]
            assert blocks[0][0] == 0 and blocks[-1][1] == n
            assert all(blocks[i][1] == blocks[i + 1][0] for i in range(world - 1))
            sizes = [hi - lo for lo, hi in blocks]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        parallel.shard_range(4, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        H, G, B, S, D = 4, 2, 3, 8, 16
        full = torch.randn(H, G, B, S, D)
        mine = parallel.shard_units(full, rank, world)
        assert mine.shape[0] == H//world
        local = mine*2.0                      # stand-in for the per-unit kernel
        whole = parallel.regather(local, axis=0)
        assert torch.equal(whole, full*2.0)
        t = parallel.max_over_ranks(float(rank + 1), "cpu")
        assert t == float(world)
        np.save(os.path.join(out_dir, f"ok{rank}.npy"), np.array([1]))
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_shard_and_regather(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}.npy").exists() for r in range(world))


def test_shard_units_falls_back_to_batch_axis():
    x = torch.zeros(3, 1, 4, 2, 2)
    assert parallel.shard_units(x, 1, 2).shape == (3, 1, 2, 2, 2)
    with pytest.raises(ValueError):
        parallel.shard_units(torch.zeros(3, 1, 3, 2, 2), 0, 2)


def test_chunk_ranges_cover_units():
    from nntile_b200.parallel import chunk_ranges
    for n, c in ((8, 8), (8, 3), (5, 8), (1, 4), (12, 5)):
        r = chunk_ranges(n, c)
        assert len(r) == min(n, c)
        assert r[0][0] == 0 and r[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(r, r[1:]))
        assert all(hi > lo for lo, hi in r)
