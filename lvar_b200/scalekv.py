"""ScaleKV KV-cache compaction on the sm_100a kernels: the host logic of the reference's
``ScaleKVCluster`` (models/scalekv/scale_kv.py:12-301) with the scoring, selection and gather on the
device.  Same constructor, same ``update_kv(key_states, query_states, value_states, scale_ind)`` and the
same capacity rules; tensors are CUDA bf16 [B, H, L, D] with D in {64, 128}.

The window (a sqrt(window_size) x sqrt(window_size) grid of tokens of the current scale) is the same for
every batch entry and head, so it is computed once on the host.  For every other case the reference
handles (non-square scale or window, window indices that collapse under clamping) this module raises
instead of guessing.
"""
from __future__ import annotations

import math
import warnings
from typing import List, Sequence

import torch

from . import kernels as K

SCALE_TOKENS = [1, 4, 16, 36, 64, 144, 256, 400, 576, 1024, 1600, 2304, 4096]


def window_indices(current_scale_size: int, current_scale_start: int, key_len: int, window_size: int) -> List[int]:
    """Centres of the grid patches of the current scale's token map, as global key indices
    (scale_kv.py:38-147 for the square case; unique and ascending)."""
    side = math.isqrt(current_scale_size)
    grid = math.isqrt(window_size)
    if side * side != current_scale_size or grid * grid != window_size or side < grid:
        n = min(window_size, key_len)  # the reference's fallback: the most recent tokens
        return list(range(key_len - n, key_len))
    hp = wp = side // grid
    out = []
    for i in range(grid):
        for j in range(grid):
            hc = max(0, min(side - 1, i * hp + (hp - 1) // 2))
            wc = max(0, min(side - 1, j * wp + (wp - 1) // 2))
            out.append(min(max(hc * side + wc + current_scale_start, 0), key_len - 1))
    return sorted(set(out))[:window_size]


class ScaleKVCluster:
    """Per-layer compaction state (scale_kv.py:12-36)."""

    def __init__(self, cache_sizes: Sequence[Sequence[int]], window_size: int = 16, base_capacity: int = 121,
                 kernel_size: int = 5, pooling: str = "maxpool", layer_idx: int = 0):
        if not isinstance(window_size, int) or window_size <= 0:
            raise ValueError("window_size must be a positive integer.")
        if not isinstance(base_capacity, int) or base_capacity <= 0:
            raise ValueError("base_capacity must be a positive integer.")
        if not isinstance(kernel_size, int) or kernel_size <= 0:
            raise ValueError("kernel_size must be a positive integer.")
        if pooling not in ("maxpool", "avgpool", "pool"):
            raise ValueError("pooling must be 'maxpool' or 'avgpool'.")
        if not isinstance(layer_idx, int) or layer_idx < 0:
            raise ValueError("layer_idx must be a non-negative integer.")
        if not isinstance(cache_sizes, (list, tuple)) or not cache_sizes:
            raise ValueError("cache_sizes must be a non-empty list.")
        self.window_size = window_size
        self.base_capacity = base_capacity
        self.kernel_size = kernel_size
        self.pooling = "avgpool" if pooling == "pool" else pooling
        self.layer_idx = layer_idx
        self.has_reached_base = False
        self.cache_sizes = cache_sizes
        self.SCALE = list(SCALE_TOKENS)
        self.max_capacity = base_capacity

    def _capacity(self, scale_ind: int) -> int:
        """Cache budget of this layer at this scale (scale_kv.py:172-190)."""
        cap_scale = 11 if scale_ind == 12 else scale_ind
        idx = max(0, min(cap_scale + 2, len(self.cache_sizes) - 1))
        if self.layer_idx >= len(self.cache_sizes[idx]):
            warnings.warn(f"Layer {self.layer_idx}: layer_idx out of bounds for cache_sizes[{idx}]. Using base_capacity.")
            return self.base_capacity
        return int(self.cache_sizes[idx][self.layer_idx])

    def select_indices(self, key_states: torch.Tensor, query_states: torch.Tensor, scale_ind: int) -> torch.Tensor:
        """int32 [B, H, max_capacity], ascending: the window tokens and the best of the rest
        (scale_kv.py:195-276)."""
        B, H, key_len, D = key_states.shape
        scale_ind = max(0, min(scale_ind, len(self.SCALE) - 1))
        size = self.SCALE[scale_ind]
        start = max(0, key_len - size)
        win = window_indices(key_len - start, start, key_len, self.window_size)
        if self.max_capacity < len(win):
            warnings.warn(f"Layer {self.layer_idx}: max_capacity ({self.max_capacity}) is less than the window "
                          f"({len(win)}). Will only keep the window tokens.", UserWarning)
            self.max_capacity = len(win)
        window = torch.tensor(win, dtype=torch.int32, device=key_states.device)
        if self.max_capacity == len(win):
            return window.view(1, 1, -1).expand(B, H, -1).contiguous()
        offset = key_len - query_states.shape[2]
        scores = K.scalekv_scores(query_states, key_states, window, offset)
        pooled = K.scalekv_pool(scores, window, self.kernel_size, self.pooling)
        keep = min(self.max_capacity, key_len)
        return K.topk_indices(pooled, keep, ascending_index=True)

    def update_kv(self, key_states: torch.Tensor, query_states: torch.Tensor, value_states: torch.Tensor,
                  scale_ind: int):
        """Returns (K, V) compacted to this layer's budget, or the inputs when they already fit
        (scale_kv.py:163-301)."""
        key_len = key_states.shape[2]
        if key_len <= self.base_capacity and not self.has_reached_base:
            return key_states, value_states
        self.has_reached_base = True
        if scale_ind == 12:
            self.has_reached_base = False
        self.max_capacity = self._capacity(scale_ind)
        if key_len <= self.max_capacity:
            return key_states, value_states
        idx = self.select_indices(key_states, query_states, scale_ind)
        return K.gather_rows(key_states, idx), K.gather_rows(value_states, idx)
