"""Torch-tensor front ends of the C ABI: pointer, stride and stream plumbing only.

Each function validates what the C side cannot see (dtype, device), allocates outputs with torch,
launches on the current CUDA stream and returns without synchronising.  Nothing here computes.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import AttnArgs, check, lib


_raw_stream = torch._C._cuda_getCurrentRawStream  # (device index) -> cudaStream_t of torch's current stream


def _stream_ptr(device: torch.device) -> int:
    return _raw_stream(device.index if device.index is not None else torch.cuda.current_device())


def _require_cuda_bf16(name: str, t: torch.Tensor) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor (lvar_b200 has no CPU path)")
    if t.dtype != torch.bfloat16:
        raise RuntimeError(f"{name} must be bfloat16, got {t.dtype}")
    if t.dim() != 4:
        raise RuntimeError(f"{name} must be 4-dimensional [B, H, L, D], got {tuple(t.shape)}")
    if t.stride(-1) != 1:
        raise RuntimeError(f"{name} must have a contiguous last dimension")


def _fill_qkv(a: AttnArgs, q, k, v, o, scale) -> int:
    """Fills the problem, tensor and scheduling fields; returns the stream to launch on."""
    B, H, Lq, D = q.shape
    if k.shape[0] != B or k.shape[1] != H or v.shape[:2] != k.shape[:2]:
        raise RuntimeError(f"q/k/v batch or head mismatch (query heads must equal kv heads): "
                           f"q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)}")
    if k.shape[-1] != D or v.shape[-1] != D or k.shape[2] != v.shape[2]:
        raise RuntimeError(f"q/k/v shape mismatch: q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)}")
    a.B, a.H, a.Lq, a.Lkv, a.D = B, H, Lq, k.shape[2], D
    a.scale = float(D ** -0.5 if scale is None else scale)
    a.q, (a.q_sb, a.q_sh, a.q_sl, _) = q.data_ptr(), q.stride()
    a.k, (a.k_sb, a.k_sh, a.k_sl, _) = k.data_ptr(), k.stride()
    a.v, (a.v_sb, a.v_sh, a.v_sl, _) = v.data_ptr(), v.stride()
    a.o, (a.o_sb, a.o_sh, a.o_sl, _) = o.data_ptr(), o.stride()
    a.wait_limit_ns = _lib.DEFAULT_WAIT_NS
    dev = q.get_device()
    stream = _raw_stream(dev)
    a.sched_scratch = _sched_scratch(dev, stream, q.device)
    return stream


_SCRATCH = {}


def _sched_scratch(dev: int, stream: int, device: torch.device) -> int:
    """Work counter of the persistent attention kernels: two zeroed int32 per (device, stream), returned as a
    device address.  The kernels leave the counter at zero, so it is allocated and cleared only once."""
    buf = _SCRATCH.get((dev, stream))
    if buf is None:
        if torch.cuda.is_current_stream_capturing():
            # allocated now, the counter and its zero fill would belong to the graph being captured
            raise RuntimeError("first launch of an lvar_b200 attention kernel on this stream happens inside a CUDA "
                               "graph capture: run one warm-up call on the capture stream before capturing")
        buf = torch.zeros(2, dtype=torch.int32, device=device)
        _SCRATCH[(dev, stream)] = buf
    return buf.data_ptr()


def new_status(device) -> torch.Tensor:
    """A zeroed device status word for the kernels' bounded waits."""
    return torch.zeros(1, dtype=torch.int32, device=device)


def read_status(status: torch.Tensor) -> Tuple[int, str]:
    """Synchronising read of a status word -> (code, description)."""
    code = int(status.item())
    return code, _lib.DEV_STATUS_NAMES.get(code, f"unknown status {code}")


def _output_like(q: torch.Tensor, out: Optional[torch.Tensor]) -> torch.Tensor:
    """The output tensor of an attention call: a fresh contiguous one, or the caller's ``out`` (bf16, q's shape
    and device, unit stride along the head dimension, every other stride a multiple of 8 elements and a 16-byte
    aligned base, e.g. a [B,H,L,D] view of a [B,L,H,D] buffer)."""
    if out is None:
        return torch.empty_like(q, memory_format=torch.contiguous_format)
    if out.dtype != torch.bfloat16 or out.device != q.device or out.shape != q.shape:
        raise RuntimeError(f"out must be a bfloat16 tensor of shape {tuple(q.shape)} on {q.device}")
    if out.stride(-1) != 1 or any(st % 8 for st in out.stride()[:-1]) or out.data_ptr() % 16:
        raise RuntimeError("out needs unit stride along the head dimension, other strides in multiples of 8 "
                           "elements and a 16-byte aligned base")
    return out


def dense_attn_fwd(q, k, v, scale=None, *, return_stats=True, status=None, wait_limit_ns=None, sched_flags=0,
                   out=None):
    """o = softmax(q k^T * scale) v; returns (o, M, L) with fp32 [B,H,Lq] statistics in base 2.  ``out``: an
    optional destination for o (see :func:`_output_like`)."""
    for n, t in (("q", q), ("k", k), ("v", v)):
        _require_cuda_bf16(n, t)
    o = _output_like(q, out)
    B, H, Lq, _ = q.shape
    M = L = None
    a = AttnArgs()
    stream = _fill_qkv(a, q, k, v, o, scale)
    if return_stats:
        M = torch.empty((B, H, Lq), dtype=torch.float32, device=q.device)
        L = torch.empty((B, H, Lq), dtype=torch.float32, device=q.device)
        a.M, a.L = M.data_ptr(), L.data_ptr()
    if status is not None:
        a.dev_status = status.data_ptr()
    if wait_limit_ns is not None:
        a.wait_limit_ns = int(wait_limit_ns)
    a.sched_flags = int(sched_flags)
    check(lib.lvar_dense_attn(C.byref(a), stream))
    return o, M, L


def dense_colsum_attn_fwd(q, k, v, scale=None, *, return_stats=False, status=None, group_tiles=1):
    """Dense attention plus, in the same launch, the attention column sums of every 128-row query tile
    (``group_tiles`` = 1) or of every 256-row group (2): returns (o, cs) with cs fp32
    [B,H,ceil(Lq/(128*group_tiles)),Lkv] (and M, L with return_stats)."""
    for n, t in (("q", q), ("k", k), ("v", v)):
        _require_cuda_bf16(n, t)
    if group_tiles not in (1, 2):
        raise RuntimeError("group_tiles must be 1 or 2")
    o = torch.empty_like(q, memory_format=torch.contiguous_format)
    B, H, Lq, _ = q.shape
    Lkv = k.shape[2]
    rows = 128 * group_tiles
    cs = (torch.zeros if group_tiles == 2 else torch.empty)((B, H, (Lq + rows - 1) // rows, Lkv),
                                                            dtype=torch.float32, device=q.device)
    a = AttnArgs()
    stream = _fill_qkv(a, q, k, v, o, scale)
    a.cs, a.cs_sb, a.cs_sh, a.cs_st = cs.data_ptr(), cs.stride(0), cs.stride(1), cs.stride(2)
    a.cs_group_tiles = group_tiles
    M = L = None
    if return_stats:
        M = torch.empty((B, H, Lq), dtype=torch.float32, device=q.device)
        L = torch.empty((B, H, Lq), dtype=torch.float32, device=q.device)
        a.M, a.L = M.data_ptr(), L.data_ptr()
    if status is not None:
        a.dev_status = status.data_ptr()
    check(lib.lvar_dense_colsum_attn(C.byref(a), stream))
    return (o, cs, M, L) if return_stats else (o, cs)


def dense_colsum_attn_given_fwd(q, k, v, M, L, scale=None, *, return_stats=False, status=None, group_tiles=1):
    """Dense attention and its column sums in ONE sweep from given row statistics (M, L as ``dense_attn_fwd``
    returns them): (o, cs) with cs fp32 [B,H,ceil(Lq/(128*group_tiles)),Lkv] normalised by the given statistics;
    with ``return_stats`` also this attention's own statistics (M, L times the measured row sums)."""
    for n, t in (("q", q), ("k", k), ("v", v)):
        _require_cuda_bf16(n, t)
    if group_tiles not in (1, 2):
        raise RuntimeError("group_tiles must be 1 or 2")
    B, H, Lq, _ = q.shape
    Lkv = k.shape[2]
    for n, t in (("M", M), ("L", L)):
        if t.dtype != torch.float32 or not t.is_cuda or t.numel() != B * H * Lq or not t.is_contiguous():
            raise RuntimeError(f"{n} must be a contiguous CUDA float32 tensor with B*H*Lq elements")
    o = torch.empty_like(q, memory_format=torch.contiguous_format)
    rows = 128 * group_tiles
    cs = (torch.zeros if group_tiles == 2 else torch.empty)((B, H, (Lq + rows - 1) // rows, Lkv),
                                                            dtype=torch.float32, device=q.device)
    a = AttnArgs()
    stream = _fill_qkv(a, q, k, v, o, scale)
    a.cs, a.cs_sb, a.cs_sh, a.cs_st = cs.data_ptr(), cs.stride(0), cs.stride(1), cs.stride(2)
    a.cs_group_tiles = group_tiles
    a.M_in, a.L_in = M.data_ptr(), L.data_ptr()
    Mo = Lo = None
    if return_stats:
        Mo = torch.empty((B, H, Lq), dtype=torch.float32, device=q.device)
        Lo = torch.empty((B, H, Lq), dtype=torch.float32, device=q.device)
        a.M, a.L = Mo.data_ptr(), Lo.data_ptr()
    if status is not None:
        a.dev_status = status.data_ptr()
    check(lib.lvar_dense_colsum_attn_given(C.byref(a), stream))
    return (o, cs, Mo, Lo) if return_stats else (o, cs)


def colsum_tiles_fwd(q, k, scale=None, *, stats=None, return_stats=False, status=None):
    """Attention column sums of every 128-row query tile without the attention output: fp32
    [B,H,ceil(Lq/128),Lkv].  ``stats`` = (M, L) as ``dense_attn_fwd`` returns them skips the statistics sweep;
    otherwise one launch takes them first (``return_stats`` hands them back)."""
    _require_cuda_bf16("q", q)
    _require_cuda_bf16("k", k)
    B, H, Lq, D = q.shape
    Lkv = k.shape[2]
    if k.shape[0] != B or k.shape[1] != H or k.shape[3] != D:
        raise RuntimeError(f"q/k shape mismatch: q {tuple(q.shape)}, k {tuple(k.shape)}")
    cs = torch.empty((B, H, (Lq + 127) // 128, Lkv), dtype=torch.float32, device=q.device)
    a = AttnArgs()
    a.B, a.H, a.Lq, a.Lkv, a.D = B, H, Lq, Lkv, D
    a.scale = float(D ** -0.5 if scale is None else scale)
    a.q, a.q_sb, a.q_sh, a.q_sl = q.data_ptr(), q.stride(0), q.stride(1), q.stride(2)
    a.k, a.k_sb, a.k_sh, a.k_sl = k.data_ptr(), k.stride(0), k.stride(1), k.stride(2)
    a.wait_limit_ns = _lib.DEFAULT_WAIT_NS
    stream = _raw_stream(q.get_device())
    a.sched_scratch = _sched_scratch(q.get_device(), stream, q.device)
    a.cs, a.cs_sb, a.cs_sh, a.cs_st = cs.data_ptr(), cs.stride(0), cs.stride(1), cs.stride(2)
    M = L = None
    if stats is not None:
        M, L = stats
        for n, t in (("M", M), ("L", L)):
            if t.dtype != torch.float32 or not t.is_cuda or t.numel() != B * H * Lq or not t.is_contiguous():
                raise RuntimeError(f"{n} must be a contiguous CUDA float32 tensor with B*H*Lq elements")
        a.M, a.L = M.data_ptr(), L.data_ptr()
    elif return_stats:
        M = torch.empty((B, H, Lq), dtype=torch.float32, device=q.device)
        L = torch.empty((B, H, Lq), dtype=torch.float32, device=q.device)
        a.M, a.L = M.data_ptr(), L.data_ptr()
    if status is not None:
        a.dev_status = status.data_ptr()
    check(lib.lvar_colsum_tiles(C.byref(a), 1 if stats is not None else 0, stream))
    return (cs, M, L) if return_stats else cs


def sum_tiles(cs128: torch.Tensor, per: int) -> torch.Tensor:
    """Column sums of groups of ``per`` adjacent 128-row query tiles: [B,H,T,Lkv] -> [B,H,ceil(T/per),Lkv],
    added in a fixed order (bit-reproducible)."""
    if per == 1:
        return cs128
    B, H, T, Lkv = cs128.shape
    G = (T + per - 1) // per
    if T != G * per:
        cs128 = torch.nn.functional.pad(cs128, (0, 0, 0, G * per - T))
    parts = cs128.view(B, H, G, per, Lkv)
    cs = parts[:, :, :, 0]
    for i in range(1, per):
        cs = cs + parts[:, :, :, i]
    return cs


def colsum_groups_fwd(q, k, M, L, group_rows, scale=None):
    """Column sums per group of ``group_rows`` query rows from given row statistics: the transposed sweep of
    the attention kernel when the group is a multiple of 128 rows, the stand-alone kernel otherwise."""
    if group_rows % 128 == 0:
        return sum_tiles(colsum_tiles_fwd(q, k, scale, stats=(M, L)), group_rows // 128)
    return colsum_fwd(q, k, M, L, group_rows, scale)


def heaviest_first_order(block_mask: torch.Tensor, B: int, H: int, block: int = 128) -> torch.Tensor:
    """Schedule order for a ragged block mask: the ids of the kernel's work items (pairs of 128-row query tiles,
    id = (b * H + h) * pairs_per_head + pair) sorted by their number of active KV tiles, heaviest first (ties by
    id), as int32 on the mask's device.  ``block_mask`` is [nq,nk], [H,nq,nk] or [B,H,nq,nk].  Build it once
    per mask (it runs a sort) and pass it as ``work_order``."""
    m = block_mask
    while m.dim() < 4:
        m = m.unsqueeze(0)
    nq, nk = m.shape[-2:]
    m = m.to(torch.bool)
    if block == 64:  # a 128-row tile is two mask rows, a 128-key tile two mask columns
        if nk % 2:
            m = torch.nn.functional.pad(m, (0, 1))
        m = m.view(*m.shape[:-1], -1, 2).any(-1)
        if nq % 2:
            m = torch.nn.functional.pad(m, (0, 0, 0, 1))
        m = m.view(*m.shape[:-2], -1, 2, m.shape[-1]).any(-2)
    tiles = m.sum(-1, dtype=torch.int32)                       # active KV tiles per 128-row query tile
    if tiles.shape[-1] % 2:
        tiles = torch.nn.functional.pad(tiles, (0, 1))
    pairs = tiles.view(*tiles.shape[:-1], -1, 2).sum(-1)       # [*, *, pairs_per_head]
    pairs = pairs.expand(B, H, pairs.shape[-1]).reshape(-1)
    return torch.sort(pairs, descending=True, stable=True).indices.to(torch.int32)


def block_sparse_attn_fwd(q, k, v, block_mask, scale=None, *, return_stats=False, status=None, block=128,
                          work_order=None, sched_flags=0, out=None):
    """Attention under a block mask of 128x128 (or 64x64) blocks: uint8/bool [nq,nk], [H,nq,nk] or [B,H,nq,nk].
    ``work_order``: optional int32 permutation of the work items (see :func:`heaviest_first_order`).
    ``out``: an optional destination for o (see :func:`_output_like`)."""
    for n, t in (("q", q), ("k", k), ("v", v)):
        _require_cuda_bf16(n, t)
    B, H, Lq, _ = q.shape
    Lkv = k.shape[2]
    if block not in (64, 128):
        raise RuntimeError("block must be 128 or 64")
    nq, nk = (Lq + block - 1) // block, (Lkv + block - 1) // block
    m = block_mask
    if m.dtype == torch.bool:
        m = m.view(torch.uint8)
    if m.dtype != torch.uint8 or not m.is_cuda:
        raise RuntimeError("block_mask must be a CUDA bool or uint8 tensor")
    while m.dim() < 4:
        m = m.unsqueeze(0)
    if m.shape[-2:] != (nq, nk) or m.shape[0] not in (1, B) or m.shape[1] not in (1, H):
        raise RuntimeError(f"block_mask shape {tuple(block_mask.shape)} does not match "
                           f"[{B}|1, {H}|1, {nq}, {nk}]")
    if m.stride(-1) != 1:
        m = m.contiguous()
    o = _output_like(q, out)
    a = AttnArgs()
    stream = _fill_qkv(a, q, k, v, o, scale)
    a.block_mask = m.data_ptr()
    a.bm_sb = m.stride(0) if m.shape[0] > 1 else 0
    a.bm_sh = m.stride(1) if m.shape[1] > 1 else 0
    a.bm_sq = m.stride(2)
    a.block_size = int(block)
    if work_order is not None:
        n_items = B * H * ((Lq + 255) // 256)
        if (work_order.dtype != torch.int32 or work_order.device != q.device or work_order.numel() != n_items
                or not work_order.is_contiguous()):
            raise RuntimeError(f"work_order must be a contiguous int32 tensor of {n_items} work item ids on {q.device}")
        a.work_order = work_order.data_ptr()
    M = L = None
    if return_stats:
        M = torch.empty((B, H, Lq), dtype=torch.float32, device=q.device)
        L = torch.empty((B, H, Lq), dtype=torch.float32, device=q.device)
        a.M, a.L = M.data_ptr(), L.data_ptr()
    if status is not None:
        a.dev_status = status.data_ptr()
    a.sched_flags = int(sched_flags)
    check(lib.lvar_block_sparse_attn(C.byref(a), stream))
    return (o, M, L) if return_stats else o


def csp_attn_fwd(q, k, v, indices, counts, o_in, o_scale, group_rows, scale=None, *, out=None, status=None,
                 resize_from: int = 0):
    """out = o_in + o_scale * softmax(q k[idx]^T * scale) v[idx] per query group of `group_rows` rows.

    ``resize_from`` = s > 0: ``o_in`` is a cache [B,H,s*s,D] over a square token grid and is resized bilinearly
    to the (square) query grid inside the same launch, with the bits of ``upsample_ocache`` + a plain call."""
    for n, t in (("q", q), ("k", k), ("v", v), ("o", o_in)):
        _require_cuda_bf16(n, t)
    B, H, Lq, _ = q.shape
    G = (Lq + group_rows - 1) // group_rows
    if indices.dtype != torch.int32 or counts.dtype != torch.int32 or not indices.is_cuda or not counts.is_cuda:
        raise RuntimeError("indices and counts must be CUDA int32 tensors")
    if tuple(indices.shape[:3]) != (B, H, G) or tuple(counts.shape) != (B, H, G):
        raise RuntimeError(f"indices {tuple(indices.shape)} / counts {tuple(counts.shape)} do not match "
                           f"[B={B}, H={H}, G={G}, *]")
    if indices.stride(-1) != 1 or counts.stride(-1) != 1:
        raise RuntimeError("indices and counts must have a contiguous last dimension")
    side = 0
    if resize_from:
        side = math.isqrt(Lq)
        if side * side != Lq:
            raise RuntimeError(f"resize_from needs a square query grid, Lq = {Lq}")
        want = (B, H, resize_from * resize_from, q.shape[3])
        if tuple(o_in.shape) != want:
            raise RuntimeError(f"Cache shape mismatch - o_in: {tuple(o_in.shape)}, expected {want}")
    elif o_in.shape != q.shape:
        raise RuntimeError("Output shape mismatch - o: {}, q: {}".format(tuple(o_in.shape), tuple(q.shape)))
    o = torch.empty_like(q, memory_format=torch.contiguous_format) if out is None else out
    a = AttnArgs()
    stream = _fill_qkv(a, q, k, v, o, scale)
    a.o_in_side, a.o_side = int(resize_from), side
    a.indices = indices.data_ptr()
    a.i_sb, a.i_sh, a.i_sg = indices.stride(0), indices.stride(1), indices.stride(2)
    a.counts = counts.data_ptr()
    a.c_sb, a.c_sh = counts.stride(0), counts.stride(1)
    a.group_rows = int(group_rows)
    a.o_in = o_in.data_ptr()
    a.oi_sb, a.oi_sh, a.oi_sl = o_in.stride(0), o_in.stride(1), o_in.stride(2)
    a.o_scale = int(o_scale)
    if status is not None:
        a.dev_status = status.data_ptr()
    check(lib.lvar_csp_attn(C.byref(a), stream))
    return o


def colsum_fwd(q, k, M, L, group_rows, scale=None, *, status=None):
    """cs[b,h,g,j] = sum over the rows of query group g of softmax(q k^T * scale)[., j]; fp32 out."""
    _require_cuda_bf16("q", q)
    _require_cuda_bf16("k", k)
    B, H, Lq, D = q.shape
    Lkv = k.shape[2]
    if k.shape[0] != B or k.shape[1] != H or k.shape[3] != D:
        raise RuntimeError(f"q/k shape mismatch: q {tuple(q.shape)}, k {tuple(k.shape)}")
    for n, t in (("M", M), ("L", L)):
        if t.dtype != torch.float32 or not t.is_cuda or t.numel() != B * H * Lq or not t.is_contiguous():
            raise RuntimeError(f"{n} must be a contiguous CUDA float32 tensor with B*H*Lq elements")
    G = (Lq + group_rows - 1) // group_rows
    cs = torch.empty((B, H, G, Lkv), dtype=torch.float32, device=q.device)
    sc = float(D ** -0.5 if scale is None else scale)
    check(lib.lvar_colsum(q.data_ptr(), k.data_ptr(), M.data_ptr(), L.data_ptr(), cs.data_ptr(),
                          B, H, Lq, Lkv, D, q.stride(0), q.stride(1), q.stride(2),
                          k.stride(0), k.stride(1), k.stride(2), cs.stride(0), cs.stride(1), cs.stride(2),
                          int(group_rows), sc, status.data_ptr() if status is not None else None,
                          _lib.DEFAULT_WAIT_NS, _stream_ptr(q.device)))
    return cs


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def block_scores(cs: torch.Tensor, block: int = 128) -> torch.Tensor:
    """[B,H,G,Lkv] fp32 column sums -> [B,H,G,ceil(Lkv/block)] fp32 per-KV-block sums."""
    _require(cs.is_cuda and cs.dtype == torch.float32 and cs.dim() == 4 and cs.stride(-1) == 1,
             "cs must be a CUDA float32 [B,H,G,Lkv] tensor with a contiguous last dimension")
    if not cs.is_contiguous():
        cs = cs.contiguous()
    B, H, G, Lkv = cs.shape
    nk = (Lkv + block - 1) // block
    out = torch.empty((B, H, G, nk), dtype=torch.float32, device=cs.device)
    check(lib.lvar_block_scores(cs.data_ptr(), out.data_ptr(), B * H * G, Lkv, int(block), cs.stride(2),
                                _stream_ptr(cs.device)))
    return out


def build_block_mask(scores: torch.Tensor, always: Optional[torch.Tensor], k_total: int, *, return_lists=False):
    """scores fp32 [B,H,nq,nk], always bool/uint8 [nq,nk] or None -> bool mask [B,H,nq,nk]
    (and, with return_lists, int32 lists [B,H,nq,nk] padded with -1 and counts [B,H,nq])."""
    _require(scores.is_cuda and scores.dtype == torch.float32 and scores.dim() == 4,
             "scores must be a CUDA float32 [B,H,nq,nk] tensor")
    scores = scores.contiguous()
    B, H, nq, nk = scores.shape
    a_ptr = None
    if always is not None:
        _require(always.is_cuda and tuple(always.shape) == (nq, nk), f"always must be a CUDA [{nq},{nk}] tensor")
        always = always.to(torch.uint8).contiguous() if always.dtype != torch.uint8 else always.contiguous()
        a_ptr = always.data_ptr()
    mask = torch.empty((B, H, nq, nk), dtype=torch.uint8, device=scores.device)
    lists = counts = None
    if return_lists:
        lists = torch.empty((B, H, nq, nk), dtype=torch.int32, device=scores.device)
        counts = torch.empty((B, H, nq), dtype=torch.int32, device=scores.device)
    check(lib.lvar_build_block_mask(scores.data_ptr(), a_ptr, mask.data_ptr(),
                                    lists.data_ptr() if lists is not None else None,
                                    counts.data_ptr() if counts is not None else None,
                                    B * H, nq, nk, int(k_total), _stream_ptr(scores.device)))
    mask = mask.view(torch.bool)
    return (mask, lists, counts) if return_lists else mask


def block_mask_from_colsums(cs: torch.Tensor, always: Optional[torch.Tensor], k_total: int, block: int = 128, *,
                            return_scores=False):
    """``build_block_mask(block_scores(cs, block), always, k_total)`` in one launch and one pass over the column
    sums: cs fp32 [B,H,G,Lkv] -> bool mask [B,H,G,ceil(Lkv/block)] (and the fp32 block scores with
    ``return_scores``; the same bits as ``block_scores`` gives)."""
    _require(cs.is_cuda and cs.dtype == torch.float32 and cs.dim() == 4 and cs.stride(-1) == 1,
             "cs must be a CUDA float32 [B,H,G,Lkv] tensor with a contiguous last dimension")
    if not cs.is_contiguous():
        cs = cs.contiguous()
    B, H, G, Lkv = cs.shape
    nk = (Lkv + block - 1) // block
    a_ptr = None
    if always is not None:
        _require(always.is_cuda and tuple(always.shape) == (G, nk), f"always must be a CUDA [{G},{nk}] tensor")
        always = always.to(torch.uint8).contiguous() if always.dtype != torch.uint8 else always.contiguous()
        a_ptr = always.data_ptr()
    mask = torch.empty((B, H, G, nk), dtype=torch.uint8, device=cs.device)
    scores = torch.empty((B, H, G, nk), dtype=torch.float32, device=cs.device) if return_scores else None
    check(lib.lvar_block_mask_from_colsums(cs.data_ptr(), cs.stride(2), a_ptr, mask.data_ptr(),
                                           scores.data_ptr() if scores is not None else None, None, None,
                                           B * H, G, Lkv, int(block), int(k_total), _stream_ptr(cs.device)))
    mask = mask.view(torch.bool)
    return (mask, scores) if return_scores else mask


def topk_indices(scores: torch.Tensor, k: int, *, ascending_index=False, out_cols: Optional[int] = None,
                 with_counts=False):
    """Exact deterministic top-k along the last dim of a float32 tensor -> int32 [..., out_cols]
    (first k entries valid, the rest 0) and optionally counts [...] filled with k."""
    _require(scores.is_cuda and scores.dtype == torch.float32 and scores.stride(-1) == 1,
             "scores must be a CUDA float32 tensor with a contiguous last dimension")
    n = scores.shape[-1]
    lead = scores.shape[:-1]
    flat = scores.reshape(-1, n)
    rows = flat.shape[0]
    cols = int(k if out_cols is None else out_cols)
    out = torch.empty((rows, cols), dtype=torch.int32, device=scores.device)
    counts = torch.full((rows,), int(k), dtype=torch.int32, device=scores.device) if with_counts else None
    if cols > 0:
        check(lib.lvar_topk_indices(flat.data_ptr(), rows, n, flat.stride(0), int(k),
                                    int(bool(ascending_index)),
                                    out.data_ptr(), out.stride(0), cols,
                                    counts.data_ptr() if counts is not None else None, int(k),
                                    _stream_ptr(scores.device)))
    out = out.view(*lead, cols)
    return (out, counts.view(*lead)) if with_counts else out


def mask_to_indices(mask: torch.Tensor, multiple_of: int, pad_to_multiple_of: int):
    """bool [b,h,m,n] -> [indices int32 [b,h,m,n rounded up to pad_to], counts int32 [b,h,m]]."""
    _require(mask.dim() == 4, "mask must be 4-dimensional [b, h, m, n]")
    _require(mask.dtype == torch.bool, "mask must be bool type")
    _require(mask.is_cuda, "mask must be a CUDA tensor (lvar_b200 has no CPU path)")
    mask = mask.contiguous()
    b, h, m, n = mask.shape
    pad_n = (n + pad_to_multiple_of - 1) // pad_to_multiple_of * pad_to_multiple_of
    indices = torch.empty((b, h, m, pad_n), dtype=torch.int32, device=mask.device)
    counts = torch.empty((b, h, m), dtype=torch.int32, device=mask.device)
    check(lib.lvar_mask_to_indices(mask.view(torch.uint8).data_ptr(), indices.data_ptr(), counts.data_ptr(),
                                   b * h * m, n, pad_n, int(multiple_of), _stream_ptr(mask.device)))
    return [indices, counts]


def bitpack(mask: torch.Tensor):
    _require(mask.is_cuda and mask.dtype == torch.bool, "mask must be a CUDA bool tensor")
    flat = mask.contiguous().view(torch.uint8)
    n = flat.numel()
    packed = torch.empty(((n + 7) // 8,), dtype=torch.uint8, device=mask.device)
    check(lib.lvar_bitpack(flat.data_ptr(), packed.data_ptr(), n, _stream_ptr(mask.device)))
    return packed, mask.shape


def bitunpack(packed: torch.Tensor, original_shape):
    _require(packed.is_cuda and packed.dtype == torch.uint8 and packed.dim() == 1, "packed must be CUDA uint8 1-D")
    total = 1
    for d in original_shape:
        total *= int(d)
    _require(packed.numel() * 8 >= total, "packed tensor too short for the requested shape")
    out = torch.empty((total,), dtype=torch.uint8, device=packed.device)
    check(lib.lvar_bitunpack(packed.contiguous().data_ptr(), out.data_ptr(), total, _stream_ptr(packed.device)))
    return out.view(torch.bool).view(*original_shape)


def upsample_ocache(o_cache: torch.Tensor, L_src: int, L_tgt: int) -> torch.Tensor:
    """Bilinear resize of a bf16 output cache [B,H,L_src,D] (square token grid) to [B,H,L_tgt,D]."""
    _require_cuda_bf16("o_cache", o_cache)
    B, H, L, D = o_cache.shape
    s, t = int(round(L_src ** 0.5)), int(round(L_tgt ** 0.5))
    _require(L == L_src and s * s == L_src and t * t == L_tgt, "L_src and L_tgt must be square token counts")
    src = o_cache if o_cache.is_contiguous() else o_cache.contiguous()
    dst = torch.empty((B, H, L_tgt, D), dtype=torch.bfloat16, device=o_cache.device)
    check(lib.lvar_upsample_ocache(src.data_ptr(), dst.data_ptr(), B * H, s, t, D, src.stride(1), src.stride(2),
                                   dst.stride(1), dst.stride(2), _stream_ptr(o_cache.device)))
    return dst


def sparse_step_lists(inds: torch.Tensor, remap: torch.Tensor, band: Optional[torch.Tensor], cnt: int, k_len: int,
                      *, src_cols: Optional[int] = None, count_value: Optional[int] = None):
    """Key lists of a sparse step: inds int32 [B,H,Gs,*] remapped to the groups in `remap` (int32 [Gk]),
    first `cnt` entries clamped to [0, k_len), followed by band int32 [Gk, band_count]; returns
    (lists int32 [B,H,Gk,k_len], counts int32 [B,H,Gk])."""
    _require(inds.is_cuda and inds.dtype == torch.int32 and inds.dim() == 4 and inds.stride(-1) == 1,
             "inds must be a CUDA int32 [B,H,Gs,cols] tensor with a contiguous last dimension")
    _require(remap.is_cuda and remap.dtype == torch.int32 and remap.dim() == 1, "remap must be CUDA int32 [Gk]")
    B, H, Gs, cols = inds.shape
    if inds.stride(0) != H * inds.stride(1):
        inds = inds.contiguous()
    Gk = remap.shape[0]
    band_count = 0
    if band is not None:
        _require(band.is_cuda and band.dtype == torch.int32 and band.dim() == 2 and band.shape[0] == Gk,
                 "band must be CUDA int32 [Gk, band_count]")
        band = band.contiguous()
        band_count = band.shape[1]
    out = torch.empty((B, H, Gk, k_len), dtype=torch.int32, device=inds.device)
    counts = torch.empty((B, H, Gk), dtype=torch.int32, device=inds.device)
    check(lib.lvar_sparse_step_lists(inds.data_ptr(), remap.data_ptr(), band.data_ptr() if band is not None else None,
                                     out.data_ptr(), counts.data_ptr(), B * H, Gs,
                                     int(cols if src_cols is None else src_cols), inds.stride(2), inds.stride(1),
                                     Gk, int(cnt), band_count, int(k_len), k_len,
                                     int(cnt + band_count if count_value is None else count_value),
                                     _stream_ptr(inds.device)))
    return out, counts


def scalekv_scores(q: torch.Tensor, k: torch.Tensor, window: torch.Tensor, offset: int) -> torch.Tensor:
    """ScaleKV window scores: fp32 [B,H,Lkv], -inf on the window's own columns.  q bf16 [B,H,Lq,D],
    k bf16 [B,H,Lkv,D], window int32 [w] (distinct key indices); the window queries are the query rows
    clamp(window - offset, 0, Lq - 1)."""
    _require_cuda_bf16("q", q)
    _require_cuda_bf16("k", k)
    B, H, Lq, D = q.shape
    Lkv = k.shape[2]
    _require(window.is_cuda and window.dtype == torch.int32 and window.dim() == 1, "window must be CUDA int32 [w]")
    window = window.contiguous()
    scores = torch.empty((B, H, Lkv), dtype=torch.float32, device=q.device)
    check(lib.lvar_scalekv_scores(q.data_ptr(), k.data_ptr(), window.data_ptr(), scores.data_ptr(), B, H, Lq, Lkv, D,
                                  q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
                                  window.shape[0], int(offset), _stream_ptr(q.device)))
    return scores


def scalekv_pool(scores: torch.Tensor, window: torch.Tensor, kernel_size: int, pooling: str) -> torch.Tensor:
    """max_pool1d / avg_pool1d(scores, kernel_size, padding kernel_size//2, stride 1) with the window columns
    then raised to +inf (see lvar_scalekv_pool)."""
    _require(scores.is_cuda and scores.dtype == torch.float32 and scores.is_contiguous(),
             "scores must be a contiguous CUDA float32 tensor")
    _require(pooling in ("maxpool", "avgpool"), "pooling must be 'maxpool' or 'avgpool'")
    Lkv = scores.shape[-1]
    rows = scores.numel() // Lkv
    pooled = torch.empty_like(scores)
    check(lib.lvar_scalekv_pool(scores.data_ptr(), window.data_ptr(), window.shape[0], pooled.data_ptr(), rows, Lkv,
                                int(kernel_size), int(pooling == "avgpool"), _stream_ptr(scores.device)))
    return pooled


def gather_rows(src: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """src bf16 [B,H,L,D], idx int32 [B,H,n] -> bf16 [B,H,n,D] = src[b,h,clamp(idx),:]."""
    _require_cuda_bf16("src", src)
    B, H, L, D = src.shape
    _require(idx.is_cuda and idx.dtype == torch.int32 and idx.dim() == 3 and idx.shape[:2] == (B, H),
             "idx must be CUDA int32 [B,H,n]")
    idx = idx.contiguous()
    n = idx.shape[2]
    dst = torch.empty((B, H, n, D), dtype=src.dtype, device=src.device)
    if n > 0:
        check(lib.lvar_gather_rows(src.data_ptr(), idx.data_ptr(), dst.data_ptr(), B, H, L, n, D, src.stride(0),
                                   src.stride(1), src.stride(2), n, _stream_ptr(src.device)))
    return dst


def qkv_prologue(qkv: torch.Tensor, scale_mul: Optional[torch.Tensor], rope_cos: Optional[torch.Tensor],
                 rope_sin: Optional[torch.Tensor], rope_start: int, k_cache: torch.Tensor, v_cache: torch.Tensor,
                 cache_pos: int) -> torch.Tensor:
    """Fused L2-normalise / per-head scale / 2-D RoPE / KV-cache append.  qkv bf16 [B,L,3,H,c] (any strides with
    a contiguous last dimension), scale_mul fp32 [H] or None, rope tables fp32 [P, c/2] or None; k_cache and
    v_cache bf16 [B,H,cap,c] receive rows cache_pos .. cache_pos+L-1.  Returns q bf16 [B,H,L,c]."""
    _require(qkv.is_cuda and qkv.dtype == torch.bfloat16 and qkv.dim() == 5 and qkv.shape[2] == 3 and
             qkv.stride(-1) == 1, "qkv must be a CUDA bfloat16 [B,L,3,H,c] tensor with a contiguous last dimension")
    B, L, _, H, c = qkv.shape
    for name, t in (("k_cache", k_cache), ("v_cache", v_cache)):
        _require_cuda_bf16(name, t)
        _require(t.shape[0] == B and t.shape[1] == H and t.shape[3] == c and cache_pos + L <= t.shape[2],
                 f"{name} must be [B,H,cap,c] with room for rows {cache_pos}..{cache_pos + L - 1}")
    if scale_mul is not None:
        _require(scale_mul.is_cuda and scale_mul.dtype == torch.float32 and scale_mul.numel() == H,
                 "scale_mul must be CUDA float32 with H entries")
        scale_mul = scale_mul.reshape(H).contiguous()
    if rope_cos is not None:
        for t in (rope_cos, rope_sin):
            _require(t is not None and t.is_cuda and t.dtype == torch.float32 and t.dim() == 2 and
                     t.shape[1] == c // 2 and t.is_contiguous() and rope_start + L <= t.shape[0],
                     "rope tables must be contiguous CUDA float32 [P, c/2] covering rope_start+L rows")
    q = torch.empty((B, H, L, c), dtype=torch.bfloat16, device=qkv.device)
    check(lib.lvar_qkv_prologue(qkv.data_ptr(), qkv.stride(0), qkv.stride(1), qkv.stride(2), qkv.stride(3),
                                scale_mul.data_ptr() if scale_mul is not None else None,
                                rope_cos.data_ptr() if rope_cos is not None else None,
                                rope_sin.data_ptr() if rope_cos is not None else None, int(rope_start),
                                q.data_ptr(), q.stride(0), q.stride(1), q.stride(2),
                                k_cache.data_ptr(), k_cache.stride(0), k_cache.stride(1), k_cache.stride(2),
                                v_cache.data_ptr(), v_cache.stride(0), v_cache.stride(1), v_cache.stride(2),
                                int(cache_pos), B, L, H, c, _stream_ptr(qkv.device)))
    return q
