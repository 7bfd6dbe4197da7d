"""The one exchange step of the path on two GPUs: an NCCL all-gather of per-head block scores followed by
the (deterministic) shared block mask, identical on both ranks and equal to the single-process result.
Needs two CUDA devices; skipped otherwise."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, ok):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from lvar_b200 import kernels as K, partition as part, policy as P
        n_units, nq, nk, k_total = 6, 8, 21, 7
        g = torch.Generator().manual_seed(3)
        scores = torch.rand(n_units, nq, nk, generator=g)           # same on every rank
        always = P.sink_local_blocks(nq, nk, 128, 200, 1500, 0, nq * 128)
        mine = scores.index_select(0, part.unit_indices(n_units, world, rank)).to(dev)
        mask, gathered = part.shared_block_mask(mine, n_units, always.to(dev), k_total)
        torch.cuda.synchronize()
        total = torch.zeros(nq, nk)
        for u in range(n_units):
            total = total + scores[u]
        want = K.build_block_mask(total.view(1, 1, nq, nk).to(dev), always.to(dev), k_total)[0, 0]
        good = torch.equal(gathered.cpu(), scores) and torch.equal(mask.cpu(), want.cpu().bool())
        # both ranks must hold the same mask bit for bit
        both = [torch.empty_like(mask, dtype=torch.uint8) for _ in range(world)]
        dist.all_gather(both, mask.to(torch.uint8))
        good = good and torch.equal(both[0], both[1])
        ok[rank] = int(good)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two CUDA devices")
def test_shared_block_mask_two_gpus():
    world = 2
    ok = mp.get_context("spawn").Array("i", [0] * world)
    mp.spawn(_worker, args=(world, _free_port(), ok), nprocs=world, join=True)
    assert list(ok) == [1] * world
