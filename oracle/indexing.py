"""Mask / index construction of the path, restated on the CPU (see package docstring).

Integer and boolean results here are the bit-exact targets of the CUDA kernels and of the host-side
policy module.  Loops are kept literal where the reference loops; sizes in the tests are small enough.
"""
from __future__ import annotations

import math
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------------------------------
# top-k
# --------------------------------------------------------------------------------------------------
def topk_indices(scores: torch.Tensor, k: int, ascending_index: bool = False) -> torch.Tensor:
    """Indices of the k largest entries along the last dim.

    Stands for ``torch.topk(bs, k=indices_count, dim=-1).indices`` (models/sparvar/sparse_attn.py:1016).
    torch.topk leaves the order of equal values unspecified, so it is defined here: descending by
    value, equal values in ascending index order (a stable descending sort).  With
    ``ascending_index`` the selected set is returned sorted by index, the convention of ScaleKV's
    KV compaction (models/scalekv/scale_kv.py:276).  -0.0 and +0.0 compare equal.
    """
    order = torch.sort(scores.float(), dim=-1, descending=True, stable=True).indices[..., :k]
    if ascending_index:
        order = torch.sort(order, dim=-1).values
    return order.to(torch.int32)


def indices_count(top_keys: float, kv_len: int, multiple_of: int) -> int:
    """``int(multiple_of * round(top_keys * kv_len / multiple_of))`` (sparse_attn.py:1012); Python's
    round, i.e. half to even."""
    return int(multiple_of * round((top_keys * kv_len) / multiple_of))


def decision_step_indices(bs: torch.Tensor, top_keys: float, multiple_of: int, indices_pad_to: int,
                          fill: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """(inds [B,H,G,Lkv] int32, counts [B,H,G] int32) of the dense decision step
    (models/sparvar/sparse_attn.py:1012-1036).  The reference pads the list with ``torch.empty``
    (undefined values that are never read); here the tail is ``fill``."""
    B, H, G, Lkv = bs.shape
    cnt = indices_count(top_keys, Lkv, multiple_of)
    inds = topk_indices(bs, cnt)
    counts = torch.full((B, H, G), cnt, dtype=torch.int32)
    pad = (Lkv - cnt + indices_pad_to - 1) // indices_pad_to * indices_pad_to
    inds = torch.cat([inds, torch.full((B, H, G, pad), fill, dtype=torch.int32)], dim=-1)[..., :Lkv]
    return inds, counts


# --------------------------------------------------------------------------------------------------
# CS4A: cross-scale reuse of the decision-scale indices
# --------------------------------------------------------------------------------------------------
def group_remap_table(Gk: int, Gs: int) -> torch.Tensor:
    """Nearest source group of each target query group: round((g + 0.5) / Gk * Gs - 0.5) clamped,
    in float32 with round-half-to-even (sparse_attn.py:403-404)."""
    c = torch.arange(Gk, dtype=torch.float32) + 0.5
    return torch.round(c / Gk * Gs - 0.5).to(torch.int64).clamp_(0, Gs - 1)


def map_inds_counts_across_scales(inds_S: torch.Tensor, counts_S: torch.Tensor, cur_q_len: int, cur_k_len: int,
                                  bm: int = 192, indices_pad_to: int = 1) -> Tuple[torch.Tensor, torch.Tensor]:
    """The no-sink path of ``map_inds_counts_across_scales`` (sparse_attn.py:365-421), the only one
    the caller uses (sparse_attn.py:1067-1069)."""
    B, H, Gs, Ks = inds_S.shape
    Gk = (cur_q_len + bm - 1) // bm
    raw = int(counts_S[0, 0, 0])
    cnt = max(indices_pad_to, (raw + indices_pad_to - 1) // indices_pad_to * indices_pad_to)
    templ = inds_S.index_select(2, group_remap_table(Gk, Gs))
    if Ks >= cnt:
        out = templ[..., :cnt].clone()
    else:
        rep = math.ceil(cnt / Ks)
        out = templ.repeat_interleave(rep, dim=-1)[..., :cnt].clone()
    out = out.to(torch.int32).clamp_(0, max(0, cur_k_len - 1))
    return out, torch.full((B, H, Gk), cnt, dtype=torch.int32)


def local_window_indices(Hh: int, W: int, base: int, win: Tuple[int, int]) -> torch.Tensor:
    """Per-query clamp-padded 2-D window of absolute KV indices, [H*W, win_h*win_w]
    (sparse_attn.py:619-674, padding='clamp', dilation 1)."""
    hw, ww = win
    ry, rx = (hw - 1) // 2, (ww - 1) // 2
    rows = []
    for y in range(Hh):
        for x in range(W):
            r = []
            for dy in range(-ry, hw - ry):
                for dx in range(-rx, ww - rx):
                    ny = min(max(y + dy, 0), Hh - 1)
                    nx = min(max(x + dx, 0), W - 1)
                    r.append(ny * W + nx + base)
            rows.append(r)
    return torch.tensor(rows, dtype=torch.long)


def aggregate_group_indices(indices_abs: torch.Tensor, q_len: int, kv_len: int, bm: int,
                            counts_multiple_of: int) -> Tuple[torch.Tensor, int]:
    """Per query group: a CONTIGUOUS band starting at the group's smallest index, as long as the
    largest group union rounded up to ``counts_multiple_of``, shifted left when it would pass
    kv_len - 1 (sparse_attn.py:777-857)."""
    idx = indices_abs.clamp(0, kv_len - 1)
    G = math.ceil(q_len / bm)
    starts, counts = [], []
    for g in range(G):
        uniq = torch.unique(idx[g * bm:min((g + 1) * bm, q_len)].reshape(-1))
        c = int(uniq.numel())
        if counts_multiple_of:
            c = (c + counts_multiple_of - 1) // counts_multiple_of * counts_multiple_of
        starts.append(int(uniq[0]))
        counts.append(c)
    gc = max(counts) if counts else 0
    st = torch.tensor(starts, dtype=torch.long)
    tails = torch.minimum(st + (gc - 1), torch.tensor(kv_len - 1))
    return (tails[:, None] - (gc - 1)) + torch.arange(gc), gc


def local_band(scales: Sequence[int], scale_ind: int, win: int, bm: int, counts_multiple_of: int):
    """The static local prior of one sparse scale: ``build_crossscale_indices`` with
    window_spec {0: (win, win)} followed by ``aggregate_group_indices``
    (sparse_attn.py:921-938, 677-768)."""
    n_list = [s * s for s in scales]
    cum = [0] + list(np.cumsum(n_list))
    side = scales[scale_ind]
    per_query = local_window_indices(side, side, int(cum[scale_ind]), (win, win))
    kv_len = int(cum[scale_ind + 1])
    return aggregate_group_indices(per_query, n_list[scale_ind], kv_len, bm, counts_multiple_of)


def sparse_step_indices(inds: torch.Tensor, counts: torch.Tensor, q_len: int, k_len: int, band: torch.Tensor,
                        band_count: int, bm: int, multiple_of: int, indices_pad_to: int, fill: int = 0):
    """Index list of a sparse step: remapped decision-scale indices followed by the scale's local band,
    re-padded to k_len columns (sparse_attn.py:1056-1121)."""
    B, H = inds.shape[:2]
    s_count = int(counts[0, 0, 0])
    mapped, _ = map_inds_counts_across_scales(inds, counts, q_len, k_len, bm, indices_pad_to)
    G = mapped.shape[2]
    full = torch.cat([mapped, band.to(torch.int32).expand(B, H, -1, -1)], dim=-1)
    total = s_count + band_count
    assert total % multiple_of == 0
    new_counts = torch.full((B, H, G), total, dtype=torch.int32)
    pad = (k_len - total + indices_pad_to - 1) // indices_pad_to * indices_pad_to
    full = torch.cat([full, torch.full((B, H, G, pad), fill, dtype=torch.int32)], dim=-1)[..., :k_len]
    return full, new_counts


def upsample_ocache(o_cache: torch.Tensor, L_src: int, L_tgt: int) -> torch.Tensor:
    """Bilinear (align_corners=False) resize of [B,H,L_src,D] seen as a sqrt(L) x sqrt(L) grid
    (sparse_attn.py:324-362, mode='2d')."""
    B, H, _, Dh = o_cache.shape
    s, t = int(L_src ** 0.5), int(L_tgt ** 0.5)
    x = o_cache.view(B, H, s, s, Dh).permute(0, 1, 4, 2, 3).reshape(B * H, Dh, s, s)
    x = F.interpolate(x, size=(t, t), mode="bilinear", align_corners=False)
    return x.view(B, H, Dh, t, t).permute(0, 1, 3, 4, 2).reshape(B, H, -1, Dh)


# --------------------------------------------------------------------------------------------------
# CSLA: static sink + local-window block mask
# --------------------------------------------------------------------------------------------------
def csla_fine_mask(scale_schedule: Sequence[Tuple[int, int]], kernel_schedule: Sequence[int], q_scale_idx: int,
                   attn_sink_scale: int) -> torch.Tensor:
    """Fine [S_q, S_k] bool mask: kv in the sink scales, or inside the per-scale window around the
    query's rescaled position (models/sparvar/basic_sparvar.py:109-151)."""
    Hq, Wq = scale_schedule[q_scale_idx]
    sched = list(scale_schedule[:q_scale_idx + 1])
    kern = list(kernel_schedule[:q_scale_idx + 1])
    tokens = [h * w for h, w in sched]
    bounds = np.insert(np.cumsum(tokens), 0, 0)
    S_q, S_k = Hq * Wq, int(bounds[-1])
    sink = int(bounds[attn_sink_scale]) if attn_sink_scale > 0 else 0

    q_idx = torch.arange(S_q)[:, None]
    kv_idx = torch.arange(S_k)[None, :]
    b_t = torch.tensor(bounds, dtype=torch.int64)
    sc = torch.searchsorted(b_t, kv_idx.reshape(-1), right=True).reshape(1, S_k) - 1
    Hk = torch.tensor([h for h, _ in sched])[sc]
    Wk = torch.tensor([w for _, w in sched])[sc]
    start = b_t[sc]
    ks = torch.tensor(kern)[sc]
    rel = kv_idx - start
    kv_y, kv_x = rel // Wk, rel % Wk
    q_y, q_x = q_idx // Wq, q_idx % Wq
    cy = torch.round((q_y.float() / Hq) * Hk)
    cx = torch.round((q_x.float() / Wq) * Wk)
    half = torch.div(ks, 2, rounding_mode="floor")
    local = ((cy - kv_y).abs() <= half) & ((cx - kv_x).abs() <= half)
    return (kv_idx < sink) | local


def csla_block_mask(scale_schedule, kernel_schedule, q_scale_idx: int, attn_sink_scale: int,
                    block_size: int = 128) -> torch.Tensor:
    """Block-level mask [nq, nk]: a block is kept when ANY fine entry in it is set
    (basic_sparvar.py:154-173)."""
    fine = csla_fine_mask(scale_schedule, kernel_schedule, q_scale_idx, attn_sink_scale)
    S_q, S_k = fine.shape
    pq = (block_size - S_q % block_size) % block_size
    pk = (block_size - S_k % block_size) % block_size
    padded = F.pad(fine, (0, pk, 0, pq), "constant", False)
    nq, nk = padded.shape[0] // block_size, padded.shape[1] // block_size
    return padded.reshape(nq, block_size, nk, block_size).permute(0, 2, 1, 3).any(dim=(-1, -2))


# --------------------------------------------------------------------------------------------------
# block scores -> block mask (sink U local U top-k)
# --------------------------------------------------------------------------------------------------
def block_scores(cs: torch.Tensor, block: int) -> torch.Tensor:
    """[B,H,G,Lkv] column sums -> [B,H,G,ceil(Lkv/block)] sums over each KV block (float64 inside)."""
    B, H, G, Lkv = cs.shape
    nk = (Lkv + block - 1) // block
    pad = nk * block - Lkv
    x = F.pad(cs.double(), (0, pad))
    return x.view(B, H, G, nk, block).sum(-1)


def build_block_mask(scores: torch.Tensor, always: torch.Tensor, k_total: int) -> torch.Tensor:
    """Block mask with exactly max(k_total, |always row|) active KV blocks per query-block row:
    the always-kept blocks plus the highest-scoring remaining ones (descending score, lower block
    index wins a tie).  scores [B,H,nq,nk] fp32, always [nq,nk] bool -> [B,H,nq,nk] bool."""
    B, H, nq, nk = scores.shape
    out = always.bool().expand(B, H, nq, nk).clone()
    for b in range(B):
        for h in range(H):
            for i in range(nq):
                keep = always[i].bool()
                need = k_total - int(keep.sum())
                if need <= 0:
                    continue
                cand = torch.nonzero(~keep).flatten()
                need = min(need, cand.numel())
                s = scores[b, h, i, cand].float()
                order = torch.sort(s, descending=True, stable=True).indices[:need]
                out[b, h, i, cand[order]] = True
    return out


def sink_local_blocks(nq: int, nk: int, block: int, sink_tokens: int, q_offset: int, window_blocks: int = 0,
                      q_len: int = None) -> torch.Tensor:
    """Always-kept blocks of the benchmark mask recipe: KV blocks that intersect tokens < sink_tokens,
    and the KV blocks that intersect query block i's own KV range [q_offset + i*block,
    q_offset + (i+1)*block) widened by +-window_blocks blocks."""
    m = torch.zeros(nq, nk, dtype=torch.bool)
    n_sink = (sink_tokens + block - 1) // block
    m[:, :n_sink] = True
    for i in range(nq):
        lo = q_offset + i * block
        hi = q_offset + (i + 1) * block - 1
        if q_len is not None:
            hi = min(hi, q_offset + q_len - 1)
        b0 = max(0, lo // block - window_blocks)
        b1 = min(nk - 1, hi // block + window_blocks)
        m[i, b0:b1 + 1] = True
    return m


# --------------------------------------------------------------------------------------------------
# mask_to_indices / bitpack
# --------------------------------------------------------------------------------------------------
def mask_to_indices(mask: torch.Tensor, multiple_of: int, pad_to_multiple_of: int):
    """bool [b,h,m,n] -> (indices int32 [b,h,m,n rounded up to pad_to], counts int32 [b,h,m]).

    Order of the reference kernel (kernels/chipmunk/csrc/indexed_io/mask_to_indices.cu:21-88): lane t
    of one warp owns columns t, t+32, ... and writes its set columns, ascending, at the exclusive
    prefix of the lanes' counts - so the list is grouped by (column mod 32).  The count is rounded
    up to ``multiple_of`` and the list is padded with the first unset columns.  Entries past the
    count are undefined in the reference (torch.empty); here they are -1.  Checked against the reference
    kernel itself, compiled for sm_100a by ``oracle/build_ref.py``, in tests/test_gpu_reference_kernels.py.
    """
    b, h, m, n = mask.shape
    pad_n = (n + pad_to_multiple_of - 1) // pad_to_multiple_of * pad_to_multiple_of
    idx = torch.full((b, h, m, pad_n), -1, dtype=torch.int32)
    cnt = torch.zeros((b, h, m), dtype=torch.int32)
    mk = mask.bool().numpy()
    for bi in range(b):
        for hi in range(h):
            for mi in range(m):
                row = mk[bi, hi, mi]
                out: List[int] = []
                for lane in range(32):
                    out.extend(int(c) for c in range(lane, n, 32) if row[c])
                total = len(out)
                padded = (total + multiple_of - 1) // multiple_of * multiple_of
                if padded > total:
                    for c in range(n):
                        if not row[c]:
                            out.append(c)
                            if len(out) == padded:
                                break
                w = min(len(out), pad_n)
                idx[bi, hi, mi, :w] = torch.tensor(out[:w], dtype=torch.int32)
                cnt[bi, hi, mi] = padded
    return idx, cnt


def bitpack(mask: torch.Tensor):
    """Little-endian bit packing of a flattened bool tensor, zero padded to a byte
    (kernels/sparse_attn/sparse_attn_ops.py:300-335)."""
    flat = mask.flatten().to(torch.uint8).numpy()
    packed = np.packbits(flat, bitorder="little")
    return torch.from_numpy(packed.copy()), tuple(mask.shape)


def bitunpack(packed: torch.Tensor, shape):
    """Inverse of bitpack (sparse_attn_ops.py:338-366)."""
    total = int(np.prod(shape))
    bits = np.unpackbits(packed.numpy(), bitorder="little")[:total]
    return torch.from_numpy(bits.astype(bool)).view(*shape)
