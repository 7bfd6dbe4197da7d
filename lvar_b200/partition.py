"""Partitioning of the path over the GPUs of one box: one process per GPU, (batch, head) units dealt
round-robin to ranks, no collective on the data path.  The single exchange step is an all-gather of
per-head block scores for the case where ONE key selection must serve all heads (a shared block mask):
a few hundred KB per GPU, NCCL over NVLink on GPUs, gloo in the CPU tests.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def unit_indices(n_units: int, world: int, rank: int) -> torch.Tensor:
    """Flat (batch*H + head) ids owned by `rank`: rank, rank + world, rank + 2*world, ..."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of size {world}")
    return torch.tensor(list(range(rank, n_units, world)), dtype=torch.long)


def units_per_rank(n_units: int, world: int) -> List[int]:
    return [len(range(r, n_units, world)) for r in range(world)]


def shard_units(x: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """[B, H, ...] -> this rank's units as [U, 1, ...] (each unit is its own 'batch' with one head)."""
    B, H = x.shape[:2]
    flat = x.reshape(B * H, 1, *x.shape[2:])
    return flat.index_select(0, unit_indices(B * H, world, rank).to(x.device))


def unshard_units(parts: List[torch.Tensor], B: int, H: int) -> torch.Tensor:
    """Inverse of shard_units given every rank's [U_r, 1, ...] part (ordered by rank)."""
    world = len(parts)
    out = torch.empty((B * H, *parts[0].shape[2:]), dtype=parts[0].dtype, device=parts[0].device)
    for r, p in enumerate(parts):
        out[unit_indices(B * H, world, r).to(out.device)] = p.reshape(p.shape[0], *p.shape[2:])
    return out.view(B, H, *out.shape[1:])


def all_gather_units(local: torch.Tensor, n_units: int, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """All-gathers per-unit tensors [U_r, ...] of every rank into [n_units, ...] in unit order.

    Ranks may own different numbers of units (n_units not divisible by the world size): parts are padded
    to the largest count for the collective and the padding is dropped afterwards.  With a world of 1
    (or no process group) this is the identity."""
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        if local.shape[0] != n_units:
            raise ValueError(f"single-rank gather expects all {n_units} units, got {local.shape[0]}")
        return local
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    counts = units_per_rank(n_units, world)
    if local.shape[0] != counts[rank]:
        raise ValueError(f"rank {rank} owns {counts[rank]} units but passed {local.shape[0]}")
    cap = max(counts)
    send = local.contiguous()
    if send.shape[0] < cap:
        pad = torch.zeros((cap - send.shape[0], *send.shape[1:]), dtype=send.dtype, device=send.device)
        send = torch.cat([send, pad], dim=0)
    recv = torch.empty((world * cap, *send.shape[1:]), dtype=send.dtype, device=send.device)
    dist.all_gather_into_tensor(recv, send, group=group)
    recv = recv.view(world, cap, *send.shape[1:])
    out = torch.empty((n_units, *send.shape[1:]), dtype=send.dtype, device=send.device)
    for r in range(world):
        out[unit_indices(n_units, world, r).to(out.device)] = recv[r, :counts[r]]
    return out


def shared_block_mask(local_scores: torch.Tensor, n_units: int, always: Optional[torch.Tensor], k_total: int,
                      group: Optional[dist.ProcessGroup] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """One block mask for all heads from every rank's block scores.

    local_scores: fp32 [U_r, nq, nk] (CUDA).  Gathers the scores of all units, sums them over units in
    unit order (a fixed order, so every rank computes bit-identical totals) and runs the deterministic
    mask kernel redundantly on each rank.  Returns (mask [nq, nk] bool, gathered scores [n_units, nq, nk])."""
    from . import kernels as K
    gathered = all_gather_units(local_scores, n_units, group)
    total = torch.zeros_like(gathered[0])
    for u in range(n_units):  # fixed summation order
        total = total + gathered[u]
    mask = K.build_block_mask(total.view(1, 1, *total.shape), always, k_total)[0, 0]
    return mask, gathered
