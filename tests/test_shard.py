"""Multi-rank host logic on CPU: the unit partition and the output all-gather with the gloo backend,
world size 2 (and 3 for the uneven case), spawned as child processes."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from pto_isa_b200 import shard


def test_unit_range_is_a_contiguous_partition():
    for units in (0, 1, 7, 8, 64, 1024, 1000):
        for world in (1, 2, 3, 4, 8):
            covered = []
            for r in range(world):
                b, e = shard.unit_range(units, world, r)
                assert 0 <= b <= e <= units
                covered.extend(range(b, e))
                for u in range(b, e):
                    assert shard.owner_of(u, units, world) == r
            assert covered == list(range(units))
            sizes = [shard.unit_range(units, world, r)[1] - shard.unit_range(units, world, r)[0] for r in range(world)]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard.unit_range(8, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, units):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        b, e = shard.unit_range(units, world, rank)
        # each unit's "output" is a small matrix that encodes its unit index
        local = torch.stack([torch.full((3, 5), float(u)) for u in range(b, e)]) if e > b else torch.empty(0, 3, 5)
        full = shard.all_gather_units(local, units)
        assert full.shape == (units, 3, 5)
        for u in range(units):
            assert bool((full[u] == float(u)).all())
        # timing convention of the benchmark: the step time is the maximum over ranks
        t = torch.tensor([1.0 + rank], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        assert t.item() == float(world)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,units", [(2, 8), (2, 5), (3, 7)])
def test_all_gather_units_gloo(world, units):
    mp.spawn(_worker, args=(world, _free_port(), units), nprocs=world, join=True)
