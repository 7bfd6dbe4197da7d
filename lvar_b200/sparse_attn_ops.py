"""Operator API of the sparse-attention path: same function names, arguments, return conventions
and assertions as the reference's ``kernels/sparse_attn/sparse_attn_ops.py``, so that the reference's
attention blocks (``models/sparvar/sparse_attn.py``, ``basic_sparvar.py``) can import this module in
its place.  Every function runs hand-written sm_100a kernels through the C ABI; there is no Triton
branch, no FlashAttention call and no CPU path.  Tensors must be CUDA bf16 [B, H, L, D] with a
contiguous last dimension, D in {64, 128}, query heads == kv heads.
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch

from . import kernels as K
from .sparse_attn_config import GLOBAL_CONFIG, get_kernel_config_attn

__all__ = [
    "dense_attn", "dense_colsum_attn_s", "dense_colsum_attn_q", "naive_dense_colsum_attn", "csp_attn", "csp_attn_resized",
    "block_sparse_attn", "bitpack", "bitunpack", "copy_indices", "topk_indices", "scatter_add", "mask_to_indices",
]


def dense_attn(q, k, v, scale=None):
    """Dense (cross-)attention.  Returns ``(o, lse)`` where ``lse = (M, L)`` are fp32 [B,H,Lq,1]
    tensors in the reference's Triton convention (kernels/sparse_attn/sparse_attn_ops.py:21-59,
    triton/attn_dense.py:209-227): M = rowmax(qk*scale)*log2(e), L = sum_j exp2(qk_j*scale*log2e - M)."""
    o, M, L = K.dense_attn_fwd(q, k, v, scale)
    lse = (M.unsqueeze(-1), L.unsqueeze(-1))
    assert lse[0].shape == (q.shape[0], q.shape[1], q.shape[2], 1), "LSE shape mismatch"
    assert lse[1].shape == (q.shape[0], q.shape[1], q.shape[2], 1), "LSE shape mismatch"
    assert o.shape == q.shape, "Output shape mismatch"
    return o, lse


def _dense_colsum(q, k, v, scale):
    pad_to = get_kernel_config_attn()["bm"]
    if pad_to % 128 == 0:
        # one launch: the attention kernel sweeps the K tiles a second time for the column sums of its 128-row
        # query tiles; a group of pad_to rows is pad_to / 128 adjacent tiles, added in a fixed order
        if pad_to == 256:  # a work item of the kernel is exactly one group: its two tiles add into one row
            o, cs = K.dense_colsum_attn_fwd(q, k, v, scale, group_tiles=2)
        else:
            o, cs128 = K.dense_colsum_attn_fwd(q, k, v, scale)
            cs = K.sum_tiles(cs128, pad_to // 128)
    else:
        o, M, L = K.dense_attn_fwd(q, k, v, scale)
        cs = K.colsum_fwd(q, k, M, L, pad_to, scale)
    assert o.shape == q.shape, "Output shape mismatch - o: {}, q: {}".format(o.shape, q.shape)
    assert cs.shape == (q.shape[0], q.shape[1], (q.shape[-2] + pad_to - 1) // pad_to, k.shape[2]), \
        "CS shape mismatch - cs: {}, q: {}".format(cs.shape, q.shape)
    return o, cs


def dense_colsum_attn_s(q, k, v, scale=None):
    """Dense attention plus exact attention column sums, ``(o, cs)`` with ``cs`` fp32
    [B, H, ceil(Lq/bm), Lkv] (sparse_attn_ops.py:65-113).  The reference's "speed" and "quality"
    variants differ only in which of its kernels they combine; here both are the same exact two
    sweeps inside one launch: attention with row statistics, then a K Q^T-only column-sum sweep over the
    same resident Q tiles (a separate column-sum kernel serves group sizes that are not multiples of 128)."""
    return _dense_colsum(q, k, v, scale)


def dense_colsum_attn_q(q, k, v, scale=None):
    """See :func:`dense_colsum_attn_s` (sparse_attn_ops.py:119-149)."""
    return _dense_colsum(q, k, v, scale)


@torch.no_grad()
def naive_dense_colsum_attn(q, k, v, scale=None, q_group_size=192):
    """Materialising PyTorch definition of ``(o, cs)`` kept for debugging, as in the reference
    (sparse_attn_ops.py:179-200).  Not used by any fast path."""
    B, H, q_len, _ = q.shape
    k_len = k.size(-2)
    sm = 1 / math.sqrt(q.size(-1)) if scale is None else scale
    w = torch.softmax(q @ k.transpose(-2, -1) * sm, dim=-1)
    o = w @ v
    groups = (q_len + q_group_size - 1) // q_group_size
    pad = groups * q_group_size - q_len
    if pad:
        w = torch.nn.functional.pad(w, (0, 0, 0, pad))
    cs = w.view(B, H, groups, q_group_size, k_len).sum(dim=3).to(v.dtype)
    return o, cs


def csp_attn(q, k, v, scale, indices, indices_counts, o, o_scale):
    """Column-sparse attention delta accumulated onto ``o``: returns ``o + o_scale * delta`` where,
    for each group of ``bm`` query rows, delta is attention over the keys listed in
    ``indices[b,h,g,:indices_counts[b,h,g]]`` (sparse_attn_ops.py:273-292).  ``o`` itself is left
    untouched (the reference's Triton branch also returns a new tensor)."""
    assert indices.shape == (q.shape[0], q.shape[1], indices.shape[2], k.shape[-2]), \
        "Indices shape mismatch - indices: {}, q: {}, k: {}".format(indices.shape, q.shape, k.shape)
    assert indices_counts.shape == indices.shape[:-1], \
        "Indices counts shape mismatch - indices_counts: {}, indices: {}".format(indices_counts.shape, indices.shape)
    assert o.shape == q.shape, "Output shape mismatch - o: {}, q: {}".format(o.shape, q.shape)
    bm = get_kernel_config_attn()["bm"]
    return K.csp_attn_fwd(q, k, v, indices, indices_counts, o, int(o_scale), bm, scale)


def csp_attn_resized(q, k, v, scale, indices, indices_counts, o_cache, o_scale):
    """``csp_attn`` whose accumulate input is an O-cache of a coarser square token grid: the bilinear resize
    the policy does before every sparse step (upsample_Ocache, models/sparvar/sparse_attn.py:324-362) runs in
    the attention kernel's epilogue instead of as a launch of its own.  Same bits as
    ``csp_attn(..., upsample_ocache(o_cache, ...), o_scale)``."""
    assert indices.shape == (q.shape[0], q.shape[1], indices.shape[2], k.shape[-2]), \
        "Indices shape mismatch - indices: {}, q: {}, k: {}".format(indices.shape, q.shape, k.shape)
    assert indices_counts.shape == indices.shape[:-1], \
        "Indices counts shape mismatch - indices_counts: {}, indices: {}".format(indices_counts.shape, indices.shape)
    side = math.isqrt(o_cache.shape[-2])
    assert side * side == o_cache.shape[-2], "O-cache is not a square token grid: {}".format(o_cache.shape)
    bm = get_kernel_config_attn()["bm"]
    return K.csp_attn_fwd(q, k, v, indices, indices_counts, o_cache, int(o_scale), bm, scale, resize_from=side)


def block_sparse_attn(q, k, v, block_mask, scale=None, block_size=128, work_order=None):
    """Attention under a block mask of 128x128 (or 64x64) blocks ([nq,nk], [H,nq,nk] or [B,H,nq,nk], bool); the kernel
    behind ``SparseFlexAttn.forward`` in this package, standing in for
    ``flex_attention(q, k, v, block_mask=...)`` (models/sparvar/basic_sparvar.py:187-194).  ``work_order``
    (``kernels.heaviest_first_order``) hands the query tiles of a ragged mask out heaviest first."""
    return K.block_sparse_attn_fwd(q, k, v, block_mask, scale, block=block_size, work_order=work_order)


def bitpack(mask: torch.Tensor):
    """bool tensor -> (uint8 bit-packed 1-D tensor, original shape), little-endian within a byte
    (sparse_attn_ops.py:300-335)."""
    return K.bitpack(mask)


def bitunpack(packed: torch.Tensor, original_shape: Tuple[int, ...]):
    """Inverse of :func:`bitpack` (sparse_attn_ops.py:338-366)."""
    return K.bitunpack(packed, original_shape)


def copy_indices(bm_fc1, bm_mid_cache, indices, counts) -> None:
    raise NotImplementedError("copy_indices belongs to the sparse-MLP path, which this package does not cover")


def scatter_add(packed, unpacked, indices, counts, num_sms) -> None:
    raise NotImplementedError("scatter_add belongs to the sparse-MLP path, which this package does not cover")


def topk_indices(activations: torch.Tensor, indices_out: torch.Tensor, counts_out: torch.Tensor,
                 sparsity_amount: float, multiple_of: int, rk: float) -> None:
    """Fills ``indices_out[b, r, :count]`` with the columns of the largest activations of each row and
    ``counts_out[b, r]`` with count (sparse_attn_ops.py:381-389).  The reference kernel keeps roughly
    the top (1 - sparsity_amount) fraction through a sampled quantile, in a run-dependent order; this
    one keeps exactly ceil((1 - sparsity_amount) * cols) columns rounded up to ``multiple_of``, in
    descending order of value (lower index first among equals).

    ``rk`` > 0 (the reference's ``random_amount``, kernels/chipmunk/csrc/indexed_io/topk_indices.cu:108): every
    column outside the exact selection joins it with probability ``rk``, drawn from torch's CUDA generator (so
    ``torch.manual_seed`` makes it repeatable, which the reference's per-thread curand streams seeded from the
    data are not); the count is then padded to ``multiple_of`` with unselected columns, and the order within a
    row is that of ``mask_to_indices`` (the reference's is the order of its atomics)."""
    assert activations.dim() == 3, "activation must be 3-dimensional [batch, rows, cols]"
    assert indices_out.dim() == 3, "indices must be 3-dimensional [batch, rows, cols]"
    assert counts_out.dim() == 2, "counts must be 2-dimensional [batch, rows]"
    assert 0 <= sparsity_amount <= 1, "sparsity_amount must be between 0 and 1"
    assert 0 <= rk <= 1, "rk (random amount) must be between 0 and 1"
    cols = activations.shape[-1]
    keep = min(cols, math.ceil((1.0 - sparsity_amount) * cols))
    if rk > 0 and 0 < keep < cols:
        exact = K.topk_indices(activations.float(), keep)
        mask = torch.zeros(activations.shape, dtype=torch.bool, device=activations.device)
        mask.scatter_(-1, exact.long(), True)
        mask |= torch.rand(activations.shape, device=activations.device) < rk
        inds, counts = K.mask_to_indices(mask.unsqueeze(0), multiple_of, 1)
        indices_out[..., :cols].copy_(inds[0][..., :cols])
        counts_out.copy_(counts[0].clamp_max(cols))
        return
    keep = min(cols, (keep + multiple_of - 1) // multiple_of * multiple_of) if keep > 0 else 0
    inds, counts = K.topk_indices(activations.float(), keep, out_cols=indices_out.shape[-1], with_counts=True)
    indices_out.copy_(inds)
    counts_out.copy_(counts)


def mask_to_indices(mask: torch.Tensor, multiple_of: int, pad_to_multiple_of: int) -> List[torch.Tensor]:
    """bool [b,h,m,n] -> [indices, counts] in the reference kernel's order (sparse_attn_ops.py:402-407)."""
    return K.mask_to_indices(mask, multiple_of, pad_to_multiple_of)
