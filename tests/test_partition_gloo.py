"""Partition / all-gather logic on two CPU ranks (gloo); no GPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from lvar_b200 import partition as part


def test_unit_assignment_covers_every_unit_once():
    for n, w in ((32, 8), (32, 3), (5, 8), (1, 1), (64, 8)):
        seen = torch.cat([part.unit_indices(n, w, r) for r in range(w)])
        assert sorted(seen.tolist()) == list(range(n))
        assert part.units_per_rank(n, w) == [len(part.unit_indices(n, w, r)) for r in range(w)]
    with pytest.raises(ValueError):
        part.unit_indices(4, 2, 2)


def test_shard_unshard_roundtrip():
    x = torch.arange(2 * 3 * 4 * 5, dtype=torch.float32).view(2, 3, 4, 5)
    for w in (1, 2, 4, 6, 7):
        parts = [part.shard_units(x, w, r) for r in range(w)]
        assert all(p.shape[1:] == (1, 4, 5) for p in parts)
        assert torch.equal(part.unshard_units(parts, 2, 3), x)


def test_single_rank_gather_is_identity():
    s = torch.rand(6, 3, 4)
    assert part.all_gather_units(s, 6) is s
    with pytest.raises(ValueError):
        part.all_gather_units(s[:2], 6)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, n_units: int, ok):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(7)
        full = torch.rand(n_units, 4, 9, generator=g)  # same on every rank
        mine = full.index_select(0, part.unit_indices(n_units, world, rank))
        got = part.all_gather_units(mine, n_units)
        ok[rank] = int(torch.equal(got, full))
        # wrong unit count must be rejected before any collective is issued
        try:
            part.all_gather_units(full, n_units)
            ok[rank] = 0
        except ValueError:
            pass
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_units", [32, 5])
def test_all_gather_units_two_ranks(n_units):
    world = 2
    ok = mp.get_context("spawn").Array("i", [0] * world)
    mp.spawn(_worker, args=(world, _free_port(), n_units, ok), nprocs=world, join=True)
    assert list(ok) == [1] * world
