"""Attention arithmetic of the path in plain fp32/fp64 PyTorch on the CPU (see package docstring)."""
from __future__ import annotations

import math

import torch

LOG2E = 1.4426950408889634


def _scale(q, scale):
    return 1.0 / math.sqrt(q.shape[-1]) if scale is None else float(scale)


@torch.no_grad()
def dense_attn(q, k, v, scale=None, dtype=torch.float32):
    """softmax(q k^T * scale) v and the row statistics (M, L) in the reference's Triton convention.

    Follows ``_attn_fwd`` / ``_attention.forward`` (kernels/sparse_attn/triton/attn_dense.py:87-231):
    M = rowmax(qk) * scale * log2(e), L = sum_j exp2(qk_j * scale * log2e - M), o = acc / L.
    """
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    s = (q @ k.transpose(-1, -2)) * _scale(q, scale)
    m = s.max(dim=-1, keepdim=True).values
    p = torch.exp(s - m)
    l = p.sum(dim=-1, keepdim=True)
    o = (p @ v) / l
    return o, (m * LOG2E).squeeze(-1), l.squeeze(-1)


@torch.no_grad()
def dense_colsum_attn(q, k, v, scale=None, q_group_size=192, dtype=torch.float32):
    """(o, cs) with cs[b,h,g,:] = sum of softmax rows of query group g.

    Follows ``naive_dense_colsum_attn`` (kernels/sparse_attn/sparse_attn_ops.py:179-200) and
    ``reference_blocksums`` (kernels/sparse_attn/triton/attn_dense_colsum.py:487-500); computed per
    (batch, head) so the L x L matrix of only one head is alive at a time.
    """
    B, H, Lq, _ = q.shape
    Lkv = k.shape[-2]
    G = (Lq + q_group_size - 1) // q_group_size
    sc = _scale(q, scale)
    o = torch.empty(B, H, Lq, v.shape[-1], dtype=dtype)
    cs = torch.zeros(B, H, G, Lkv, dtype=dtype)
    for b in range(B):
        for h in range(H):
            w = torch.softmax((q[b, h].to(dtype) @ k[b, h].to(dtype).T) * sc, dim=-1)
            o[b, h] = w @ v[b, h].to(dtype)
            for g in range(G):
                cs[b, h, g] = w[g * q_group_size:min((g + 1) * q_group_size, Lq)].sum(dim=0)
    return o, cs


@torch.no_grad()
def block_sparse_attn(q, k, v, block_mask, scale=None, block=128, dtype=torch.float32):
    """Dense masked softmax under a block mask [.., nq, nk]; fully masked rows give 0.

    Stands for ``flex_attention(q, k, v, block_mask=...)`` as used by ``SparseFlexAttn.forward``
    (models/sparvar/basic_sparvar.py:187-194); flex_attention itself is third-party, so its result is
    defined here as softmax over the unmasked columns.
    """
    B, H, Lq, _ = q.shape
    Lkv = k.shape[-2]
    bm = block_mask.bool()
    while bm.dim() < 4:
        bm = bm.unsqueeze(0)
    bm = bm.expand(B, H, -1, -1)
    fine = bm.repeat_interleave(block, 2).repeat_interleave(block, 3)[:, :, :Lq, :Lkv]
    s = (q.to(dtype) @ k.to(dtype).transpose(-1, -2)) * _scale(q, scale)
    s = s.masked_fill(~fine, float("-inf"))
    m = s.max(dim=-1, keepdim=True).values
    m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
    p = torch.exp(s - m)
    l = p.sum(dim=-1, keepdim=True)
    o = (p @ v.to(dtype)) / torch.where(l > 0, l, torch.ones_like(l))
    return o


@torch.no_grad()
def csp_delta(q, k, v, indices, counts, scale=None, bm=192, dtype=torch.float32):
    """delta[b,h,rows of g] = softmax(q k[idx]^T * scale) v[idx], idx = indices[b,h,g,:counts[b,h,g]].

    Literal gather-then-softmax, i.e. the index list is a MULTISET (a key listed twice counts twice),
    which is what both reference kernels compute (kernels/sparse_attn/triton/attn_csp.py:56-98,
    kernels/chipmunk/csrc/attn/csp_attn.cu:137-304).  For duplicate-free lists this equals
    ``reference_sparse_o`` (attn_csp.py:437-471).  A count of 0 gives delta = 0
    (attn_csp.py:175-199: l_i starts at 1, acc at 0).
    """
    B, H, Lq, D = q.shape
    G = (Lq + bm - 1) // bm
    sc = _scale(q, scale)
    out = torch.zeros(B, H, Lq, v.shape[-1], dtype=dtype)
    for b in range(B):
        for h in range(H):
            for g in range(G):
                c = int(counts[b, h, g])
                if c == 0:
                    continue
                rows = slice(g * bm, min((g + 1) * bm, Lq))
                idx = indices[b, h, g, :c].long()
                s = (q[b, h, rows].to(dtype) @ k[b, h, idx].to(dtype).T) * sc
                out[b, h, rows] = torch.softmax(s, dim=-1) @ v[b, h, idx].to(dtype)
    return out


@torch.no_grad()
def csp_attn(q, k, v, scale, indices, counts, o, o_scale, bm=192):
    """o + o_scale * delta with the reference's rounding points: delta is rounded to the tensor dtype,
    then ``o + o_delta * o_scale`` is evaluated in that dtype
    (kernels/sparse_attn/sparse_attn_ops.py:281-288)."""
    delta = csp_delta(q, k, v, indices, counts, scale, bm).to(o.dtype)
    return o + delta * o_scale
