"""Sparse-attention policy (which keys each query group attends to) on top of the kernels:

* ``SparseDiffAttn`` - the column-sum -> top-k -> delta-attention policy ("CS4A") with the interface of
  the reference class of the same name (models/sparvar/sparse_attn.py:862-1167): at the decision
  scale it runs dense attention + column sums, keeps the top keys per query group and caches
  ``O_dense - delta``; at later scales it reuses the (group-remapped) key lists plus a static local
  band and adds the new delta onto the upsampled cache.
* ``SparseFlexAttn`` - the static sink + local-window block mask policy ("CSLA") with the interface of
  models/sparvar/basic_sparvar.py:47-194, running the block-sparse kernel instead of flex_attention.

The static index tables (local bands, block masks, group remap tables) are built once on the host,
like the reference does in its constructors; everything per call runs on the GPU without a host
synchronisation (the reference reads ``counts[0][0][0]`` back on every sparse layer,
sparse_attn.py:1058).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn.functional as F

from . import kernels as K
from .sparse_attn_config import GLOBAL_CONFIG, get_kernel_config_attn

INFINITY_SCALES = [1, 2, 4, 6, 8, 12, 16, 20, 24, 32, 40, 48, 64]


# --------------------------------------------------------------------------------------------------
# static tables
# --------------------------------------------------------------------------------------------------
def cumulative_tokens(scales: Sequence[int]) -> List[int]:
    """[0, s0^2, s0^2+s1^2, ...]: start of each scale on the KV axis."""
    out = [0]
    for s in scales:
        out.append(out[-1] + s * s)
    return out


def indices_count(top_keys: float, kv_len: int, multiple_of: int) -> int:
    """Keys kept per query group at the decision scale (sparse_attn.py:1012)."""
    return int(multiple_of * round((top_keys * kv_len) / multiple_of))


def group_remap_table(n_target: int, n_source: int) -> torch.Tensor:
    """For each of ``n_target`` query groups the nearest of ``n_source`` groups by centre position,
    float32 arithmetic with round-half-to-even as in sparse_attn.py:403-404."""
    centres = (torch.arange(n_target, dtype=torch.float32) + 0.5) / n_target * n_source - 0.5
    return torch.round(centres).long().clamp_(0, n_source - 1)


def local_band(scales: Sequence[int], scale_ind: int, win: int, bm: int, counts_multiple_of: int
               ) -> Tuple[torch.Tensor, int]:
    """See :func:`_local_band`; results are cached (every layer of a model asks for the same tables)."""
    key = (tuple(scales), scale_ind, win, bm, counts_multiple_of)
    if key not in _BAND_CACHE:
        _BAND_CACHE[key] = _local_band(scales, scale_ind, win, bm, counts_multiple_of)
    band, length = _BAND_CACHE[key]
    return band.clone(), length


_BAND_CACHE: Dict[tuple, Tuple[torch.Tensor, int]] = {}


def _local_band(scales: Sequence[int], scale_ind: int, win: int, bm: int, counts_multiple_of: int
                ) -> Tuple[torch.Tensor, int]:
    """Static local prior of one scale: for each group of ``bm`` queries a contiguous run of KV
    indices that starts at the smallest key any of its queries sees through a clamp-padded
    ``win x win`` window on the scale's own grid; all runs share one length (the largest group union
    rounded up to ``counts_multiple_of``) and are shifted left where they would pass the end of the KV
    axis.  Same result as build_crossscale_indices + aggregate_group_indices
    (sparse_attn.py:677-857) without per-group Python loops."""
    side = scales[scale_ind]
    cum = cumulative_tokens(scales)
    base, kv_len, q_len = cum[scale_ind], cum[scale_ind + 1], side * side
    G = math.ceil(q_len / bm)
    r_lo, r_hi = (win - 1) // 2, win - 1 - (win - 1) // 2
    off = torch.arange(-r_lo, r_hi + 1)
    y = torch.arange(side).view(side, 1, 1, 1)
    x = torch.arange(side).view(1, side, 1, 1)
    ny = (y + off.view(1, 1, -1, 1)).clamp(0, side - 1)
    nx = (x + off.view(1, 1, 1, -1)).clamp(0, side - 1)
    local = (ny * side + nx).reshape(q_len, -1)  # token ids inside the scale, [q_len, win*win]
    grp = (torch.arange(q_len) // bm).view(-1, 1).expand_as(local)
    member = torch.zeros(G, q_len, dtype=torch.bool)
    member[grp.reshape(-1), local.reshape(-1)] = True
    n_union = member.sum(dim=1)
    first = member.float().argmax(dim=1) + base
    if counts_multiple_of:
        n_union = (n_union + counts_multiple_of - 1) // counts_multiple_of * counts_multiple_of
    length = int(n_union.max()) if G else 0
    last = torch.clamp(first + (length - 1), max=kv_len - 1)
    return (last - (length - 1)).view(-1, 1) + torch.arange(length).view(1, -1), length


def csla_block_mask(scale_schedule: Sequence[Tuple[int, int]], kernel_schedule: Sequence[int], q_scale_idx: int,
                    attn_sink_scale: int, block_size: int = 128) -> torch.Tensor:
    """Block mask [ceil(S_q/block), ceil(S_k/block)] of the static sink + local-window policy: a block
    is kept if any (query, key) pair inside it is kept, a pair being kept if the key lies in the
    first ``attn_sink_scale`` scales or within ``kernel // 2`` (per key scale; negative = never) of the
    query's rescaled position in both axes (basic_sparvar.py:109-173).  Built per key scale from the
    window corners instead of a dense S_q x S_k mask."""
    Hq, Wq = scale_schedule[q_scale_idx]
    sched = list(scale_schedule[:q_scale_idx + 1])
    starts = [0]
    for h, w in sched:
        starts.append(starts[-1] + h * w)
    S_q, S_k = Hq * Wq, starts[-1]
    nq, nk = (S_q + block_size - 1) // block_size, (S_k + block_size - 1) // block_size
    mask = torch.zeros(nq, nk, dtype=torch.bool)
    sink = starts[attn_sink_scale] if attn_sink_scale > 0 else 0
    if sink > 0:
        mask[:, :(sink + block_size - 1) // block_size] = True
    q = torch.arange(S_q)
    qb = q // block_size
    qy, qx = (q // Wq).float(), (q % Wq).float()
    for s, (Hk, Wk) in enumerate(sched):
        half = kernel_schedule[s] // 2  # floor division: -1 // 2 == -1 switches the scale off
        if half < 0:
            continue
        cy = torch.round(qy / Hq * Hk).long()
        cx = torch.round(qx / Wq * Wk).long()
        d = torch.arange(-half, half + 1)
        ky = cy.view(-1, 1, 1) + d.view(1, -1, 1)
        kx = cx.view(-1, 1, 1) + d.view(1, 1, -1)
        ok = (ky >= 0) & (ky < Hk) & (kx >= 0) & (kx < Wk)
        kv = starts[s] + ky * Wk + kx
        rows = qb.view(-1, 1, 1).expand_as(kv)[ok]
        mask[rows, kv[ok] // block_size] = True
    return mask


def sink_local_blocks(nq: int, nk: int, block: int, sink_tokens: int, q_offset: int, window_blocks: int = 0,
                      q_len: Optional[int] = None) -> torch.Tensor:
    """Always-kept blocks of the top-k block policy: KV blocks holding tokens < ``sink_tokens`` and, for
    query block i, the KV blocks that intersect its own position range on the KV axis
    [q_offset + i*block, q_offset + (i+1)*block), widened by ``window_blocks`` blocks on each side."""
    i = torch.arange(nq).view(-1, 1)
    j = torch.arange(nk).view(1, -1)
    lo = q_offset + i * block
    hi = q_offset + (i + 1) * block - 1
    if q_len is not None:
        hi = torch.clamp(hi, max=q_offset + q_len - 1)
    b0 = lo // block - window_blocks
    b1 = hi // block + window_blocks
    return (j < (sink_tokens + block - 1) // block) | ((j >= b0) & (j <= b1))


# --------------------------------------------------------------------------------------------------
# per-layer state
# --------------------------------------------------------------------------------------------------
class AttnStorage:
    """Per-layer cache that lives for one image: key lists, their (host-known) count and the output
    cache (the parts of the reference's AttnStorage this path uses, sparse_attn.py:223-321; no offload)."""

    def __init__(self, layer_num: int):
        self.layer_num = layer_num
        self.indices: Optional[torch.Tensor] = None
        self.counts: Optional[torch.Tensor] = None
        self.count_value: int = 0
        self.out_cache: Optional[torch.Tensor] = None

    def clear(self) -> None:
        self.indices = self.counts = self.out_cache = None
        self.count_value = 0


class LayerCounter:
    """Position of the running layer inside the generation loop (sparse_attn_layer_counter.py:4-74)."""

    def __init__(self, num_layers: int = 0, num_sparse_submodules_per_layer: int = 1):
        self.num_layers = num_layers
        self.num_submodules_per_layer = num_sparse_submodules_per_layer
        self.cur_inference_step = 0
        self.cur_layer = 0
        self.cur_layer_submodule = 0

    def increment(self) -> None:
        self.cur_layer_submodule += 1
        if self.cur_layer_submodule >= self.num_submodules_per_layer:
            self.cur_layer_submodule = 0
            self.cur_layer += 1
            if self.num_layers and self.cur_layer >= self.num_layers:
                self.cur_layer = 0
                self.cur_inference_step += 1

    def reset(self) -> None:
        self.cur_inference_step = self.cur_layer = self.cur_layer_submodule = 0


# --------------------------------------------------------------------------------------------------
# CS4A
# --------------------------------------------------------------------------------------------------
class SparseDiffAttn:
    """Column-sum driven delta attention for one transformer layer.

    ``forward(q, k, v, scale, do_full_step=False, scale_ind=0, layer_ind=0)`` as in
    models/sparvar/sparse_attn.py:1146-1167; q/k/v are bf16 [B,H,L,D] CUDA tensors."""

    def __init__(self, layer_num: int = 0, layer_counter: Optional[LayerCounter] = None, use_o_cache: bool = True,
                 scales: Sequence[int] = tuple(INFINITY_SCALES), spsd_scale: int = 10,
                 wind_size: Optional[Sequence[int]] = None, speedup: bool = False, top_keys: Optional[float] = None):
        self.layer_num = layer_num
        self.layer_counter = layer_counter or LayerCounter()
        self.use_o_cache = use_o_cache
        self.spsd_scale = spsd_scale
        self.scales = list(scales)
        self.storage = AttnStorage(layer_num)
        cfg = GLOBAL_CONFIG["attn"]
        geo = get_kernel_config_attn()
        self.bm, self.multiple_of, self.indices_pad_to = geo["bm"], geo["counts_multiple_of"], geo["indices_pad_to"]
        self.top_keys = cfg["top_keys"] if top_keys is None else top_keys
        n_sparse = len(self.scales) - (spsd_scale + 1)
        if wind_size is None:
            ws_all = cfg.get("cs4a_ws", [1] * 11 + [7, 9])
            wind_size = ws_all[len(ws_all) - n_sparse:] if n_sparse else []
        assert len(wind_size) == n_sparse, "w/ local prior sparse, window size list mismatch sparse scales!"
        self.cum = cumulative_tokens(self.scales)
        self.local_inds: Dict[int, Tuple[torch.Tensor, int]] = {}
        for i in range(n_sparse):
            s = spsd_scale + 1 + i
            band, count = local_band(self.scales, s, wind_size[i], self.bm, self.multiple_of)
            self.local_inds[s] = (band.to(torch.int32), count)
        self._device_cache: Dict[tuple, torch.Tensor] = {}
        self.speedup = speedup

    # -- helpers ----------------------------------------------------------------------------------
    def _band_on(self, scale_ind: int, device) -> Tuple[torch.Tensor, int]:
        band, count = self.local_inds[scale_ind]
        key = (scale_ind, str(device))
        if key not in self._device_cache:
            self._device_cache[key] = band.to(device)
        return self._device_cache[key], count

    def _remap_on(self, Gk: int, Gs: int, device) -> torch.Tensor:
        key = (Gk, Gs, str(device))
        if key not in self._device_cache:
            self._device_cache[key] = group_remap_table(Gk, Gs).to(device=device, dtype=torch.int32)
        return self._device_cache[key]

    def _pad_lists(self, inds: torch.Tensor, k_len: int) -> torch.Tensor:
        """Pads the list dimension to k_len columns (zeros where the reference leaves torch.empty)."""
        have = inds.shape[-1]
        if have >= k_len:
            return inds[..., :k_len].contiguous()
        return F.pad(inds, (0, k_len - have))

    # -- steps ------------------------------------------------------------------------------------
    def _full_step(self, q, k, v, scale):
        from .sparse_attn_ops import csp_attn, dense_colsum_attn_q, dense_colsum_attn_s
        o, bs = (dense_colsum_attn_s if self.speedup else dense_colsum_attn_q)(q, k, v, scale)
        k_len = k.shape[-2]
        count = indices_count(self.top_keys, k_len, self.multiple_of)
        inds, counts = K.topk_indices(bs, count, out_cols=k_len, with_counts=True)
        self.storage.indices, self.storage.counts, self.storage.count_value = inds, counts, count
        if self.use_o_cache:
            self.storage.out_cache = csp_attn(q, k, v, scale, inds, counts, o, -1)
        return o

    def _sparse_step(self, q, k, v, scale, scale_ind):
        from .sparse_attn_ops import csp_attn, csp_attn_resized
        st = self.storage
        assert st.indices is not None, "sparse step before the decision (full) step of this layer"
        B, H, q_len, _ = q.shape
        k_len = k.shape[-2]
        inds, s_count = st.indices[:B], st.count_value
        Gk, Gs = (q_len + self.bm - 1) // self.bm, inds.shape[2]
        cnt = max(self.indices_pad_to, (s_count + self.indices_pad_to - 1) // self.indices_pad_to * self.indices_pad_to)
        band, band_count = self._band_on(scale_ind, inds.device)
        total = s_count + band_count
        assert total % self.multiple_of == 0, f"after add local sparse index, mismatch multiple_of={self.multiple_of}"
        lists, counts = K.sparse_step_lists(inds, self._remap_on(Gk, Gs, inds.device), band, cnt, k_len,
                                            count_value=total)
        if scale_ind != len(self.scales) - 1:
            st.indices, st.counts, st.count_value = lists, counts, total
        if self.use_o_cache:
            # the cache is resized to this scale's grid inside the attention launch
            return csp_attn_resized(q, k, v, scale, lists, counts, st.out_cache[:B].to(v.dtype), 1)
        return csp_attn(q, k, v, scale, lists, counts, torch.zeros_like(q), 1)

    def forward(self, q, k, v, scale, do_full_step: bool = False, inference_step: int = 0, scale_ind: int = 0,
                layer_ind: int = 0):
        if not GLOBAL_CONFIG["attn"]["is_enabled"]:
            from .sparse_attn_ops import dense_attn
            out, _ = dense_attn(q, k, v, scale)
        elif do_full_step:
            out = self._full_step(q, k, v, scale)
        else:
            out = self._sparse_step(q, k, v, scale, scale_ind)
        self.layer_counter.increment()
        return out

    __call__ = forward


# --------------------------------------------------------------------------------------------------
# CSLA
# --------------------------------------------------------------------------------------------------
class SparseFlexAttn:
    """Static sink + local-window block-sparse attention for one query scale
    (models/sparvar/basic_sparvar.py:47-194); ``forward(q, k, v, scale=None)``."""

    def __init__(self, scale_schedule, kernel_schedule, q_scale_idx, attn_sink_scale, block_size: int = 128,
                 num_heads: int = 16, device="cuda"):
        if block_size not in (64, 128):
            raise ValueError("the block-sparse kernel works on 128x128 or 64x64 blocks")
        self.block_size = block_size
        self.block_mask_cpu = csla_block_mask(scale_schedule, kernel_schedule, q_scale_idx, attn_sink_scale, block_size)
        self.block_mask = self.block_mask_cpu.to(device) if torch.cuda.is_available() else None
        self._orders: Dict[tuple, torch.Tensor] = {}

    def _order(self, B: int, H: int, device) -> torch.Tensor:
        """The mask is static and ragged (the window widens with the key scale), so the kernel's work items are
        handed out heaviest first; the order depends on (B, H) only and is built once."""
        key = (B, H, str(device))
        if key not in self._orders:
            self._orders[key] = K.heaviest_first_order(self.block_mask, B, H, self.block_size)
        return self._orders[key]

    def forward(self, q, k, v, scale=None):
        from .sparse_attn_ops import block_sparse_attn
        if self.block_mask is None or self.block_mask.device != q.device:
            self.block_mask = self.block_mask_cpu.to(q.device)
            self._orders.clear()
        return block_sparse_attn(q.to(v.dtype), k.to(v.dtype), v, self.block_mask, scale, self.block_size,
                                 work_order=self._order(q.shape[0], q.shape[1], q.device))

    __call__ = forward


# --------------------------------------------------------------------------------------------------
# which attention runs for (scale, layer)
# --------------------------------------------------------------------------------------------------
def build_csla_list(scales: Sequence[int] = tuple(INFINITY_SCALES), attn_config: Optional[dict] = None,
                    num_heads: int = 16, block_size: int = 128, device="cuda") -> List[Optional[SparseFlexAttn]]:
    """One entry per scale: ``None`` below the decision scale, a :class:`SparseFlexAttn` from it on (the
    ``spattn_compile_list`` of models/sparvar/sparvar_model.py:275-318, whose three modules are the scales from
    ``decision_scale`` to the last)."""
    cfg = GLOBAL_CONFIG["attn"] if attn_config is None else attn_config
    sched = [(s, s) for s in scales]
    win = list(cfg["win_size"])
    assert len(win) == len(scales), f"kernel_schedule mismatch {len(scales)} scales"
    first = cfg["decision_scale"]
    return [None if si < first else
            SparseFlexAttn(sched, win, q_scale_idx=si, attn_sink_scale=cfg["attn_sink"], block_size=block_size,
                           num_heads=num_heads, device=device)
            for si in range(len(scales))]


class SelfAttentionDispatch:
    """The attention call of one transformer layer during generation: picks, per (scale, layer), what
    ``SelfAttention.forward`` picks in models/sparvar/basic_sparvar.py:353-387 -

    * ``layer_ind > bound_layer`` and a static-mask module is given for the scale (scales from the decision
      scale on): sink + local-window block-sparse attention ("csla");
    * ``scale_ind == decision_scale`` and ``layer_ind <= bound_layer``: dense attention + column sums + top-k,
      O-cache ("cs4a_full");
    * ``scale_ind > decision_scale`` and ``layer_ind <= bound_layer``: column-sparse delta attention on the
      stored lists ("cs4a_sparse");
    * everything else: dense attention ("dense"; the reference calls ``torch.ops.chipmunk.dense_attn`` there).

    q, k, v are bf16 [B,H,L,D] (k, v: the whole KV cache up to this scale); returns o bf16 [B,H,Lq,D]."""

    def __init__(self, layer_ind: int, attn_config: Optional[dict] = None, scales: Sequence[int] = tuple(INFINITY_SCALES),
                 scale: float = 1.0, layer_counter: Optional[LayerCounter] = None):
        cfg = GLOBAL_CONFIG["attn"] if attn_config is None else attn_config
        self.layer_ind = layer_ind
        self.spsd_scale = cfg["decision_scale"]
        self.bound_layer = cfg["bound_layer"]
        self.scale = scale
        self.last_route: Optional[str] = None
        n_sparse = len(scales) - (self.spsd_scale + 1)
        ws = list(cfg.get("cs4a_ws", [1] * 11 + [7, 9]))
        self.sparse_attn = SparseDiffAttn(layer_ind, layer_counter, use_o_cache=True, scales=scales,
                                          spsd_scale=self.spsd_scale, wind_size=ws[len(ws) - n_sparse:] if n_sparse else [],
                                          speedup=bool(cfg.get("speedup", 0)), top_keys=cfg["top_keys"])

    def route(self, scale_ind: int, layer_ind: Optional[int] = None, spattn_fn=None) -> str:
        layer = self.layer_ind if layer_ind is None else layer_ind
        if spattn_fn is not None and layer > self.bound_layer:
            return "csla"
        if scale_ind == self.spsd_scale and layer <= self.bound_layer:
            return "cs4a_full"
        if scale_ind > self.spsd_scale and layer <= self.bound_layer:
            return "cs4a_sparse"
        return "dense"

    def forward(self, q, k, v, scale_ind: int = 0, layer_ind: Optional[int] = None, spattn_fn=None):
        layer = self.layer_ind if layer_ind is None else layer_ind
        r = self.last_route = self.route(scale_ind, layer, spattn_fn)
        if r == "csla":
            return spattn_fn(q, k, v, scale=self.scale)
        if r == "cs4a_full":
            return self.sparse_attn(q, k, v, scale=self.scale, do_full_step=True, scale_ind=scale_ind, layer_ind=layer)
        if r == "cs4a_sparse":
            return self.sparse_attn(q, k, v, scale=self.scale, scale_ind=scale_ind, layer_ind=layer)
        return K.dense_attn_fwd(q, k, v, self.scale, return_stats=False)[0]

    __call__ = forward
