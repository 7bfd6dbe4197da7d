"""CPU restatement of ScaleKV's cache compaction (reference: models/scalekv/scale_kv.py).

Test infrastructure only: imported by tests/, never by the product path.  Parity is pinned by
tests/golden/scalekv_ref.npz, produced by running the reference's own ScaleKVCluster class (compiled out of
scale_kv.py, whose module-level import of the model package does not resolve) on seeded inputs.

Every function works in the dtype of its inputs, like the reference: with bf16 tensors the logits, their
division by sqrt(D), the sum over the window queries and the average pool are each rounded to bf16.
"""
from __future__ import annotations

import math
from typing import List, Tuple

import torch
import torch.nn.functional as F

SCALE_TOKENS = [1, 4, 16, 36, 64, 144, 256, 400, 576, 1024, 1600, 2304, 4096]


def window_indices(current_scale_size: int, current_scale_start: int, key_len: int, window_size: int) -> List[int]:
    """scale_kv.py:38-147: centres of a sqrt(window_size)^2 grid of patches of the current scale's token map
    (most recent tokens when no square grid fits), unique, ascending."""
    side, grid = math.isqrt(current_scale_size), math.isqrt(window_size)
    if side * side != current_scale_size or grid * grid != window_size or side < grid:
        n = min(window_size, key_len)
        return list(range(key_len - n, key_len))
    hp = wp = side // grid
    cells = []
    for i in range(grid):
        for j in range(grid):
            hc = max(0, min(side - 1, i * hp + (hp - 1) // 2))
            wc = max(0, min(side - 1, j * wp + (wp - 1) // 2))
            cells.append(min(max(hc * side + wc + current_scale_start, 0), key_len - 1))
    return sorted(set(cells))[:window_size]


def window_scores(q: torch.Tensor, k: torch.Tensor, window: List[int]) -> torch.Tensor:
    """scale_kv.py:236-253: sum over the window queries of q_i . k_j / sqrt(D), -inf on the window columns."""
    B, H, Lq, D = q.shape
    key_len = k.shape[2]
    w = torch.tensor(window, dtype=torch.long)
    local = (w - (key_len - Lq)).clamp(0, Lq - 1)
    wq = q.index_select(2, local)
    logits = torch.matmul(wq, k.transpose(2, 3)) / math.sqrt(D)
    logits[..., w] = float("-inf")
    return logits.sum(dim=2)


def pooled_scores(scores: torch.Tensor, kernel_size: int, pooling: str) -> torch.Tensor:
    """scale_kv.py:255-258."""
    if pooling == "avgpool":
        return F.avg_pool1d(scores, kernel_size, padding=kernel_size // 2, stride=1)
    return F.max_pool1d(scores, kernel_size, padding=kernel_size // 2, stride=1)


def select_indices(q: torch.Tensor, k: torch.Tensor, window: List[int], max_capacity: int, kernel_size: int = 5,
                   pooling: str = "maxpool") -> Tuple[torch.Tensor, torch.Tensor]:
    """scale_kv.py:232-276: (ascending indices [B,H,max_capacity], pooled scores with -inf on the window)."""
    B, H, key_len, _ = k.shape
    pooled = pooled_scores(window_scores(q, k, window), kernel_size, pooling).clone()
    w = torch.tensor(window, dtype=torch.long)
    pooled[..., w] = float("-inf")
    keep = min(max_capacity - len(window), key_len - len(window))
    # stable descending order: among equal scores the lower index wins
    order = torch.sort(pooled.float(), dim=-1, descending=True, stable=True).indices[..., :keep]
    combined = torch.cat([order, w.view(1, 1, -1).expand(B, H, -1)], dim=-1)
    return torch.sort(combined, dim=-1).values, pooled


def compact(q, k, v, scale_ind: int, max_capacity: int, window_size: int = 16, kernel_size: int = 5,
            pooling: str = "maxpool"):
    """K, V gathered at the selected indices (scale_kv.py:278-296)."""
    key_len = k.shape[2]
    size = SCALE_TOKENS[scale_ind]
    start = max(0, key_len - size)
    win = window_indices(key_len - start, start, key_len, window_size)
    idx, _ = select_indices(q, k, win, max_capacity, kernel_size, pooling)
    ex = idx.unsqueeze(-1).expand(-1, -1, -1, k.shape[-1])
    return torch.gather(k, 2, ex), torch.gather(v, 2, ex), idx
