"""Registers the ``torch.ops.chipmunk`` operators the reference's model code calls directly
(``torch.ops.chipmunk.dense_attn(q, k, v)`` at models/sparvar/basic_sparvar.py:384, and the ops its
``sparse_attn_ops`` module forwards to) with the schemas of kernels/chipmunk/csrc/chipmunk.cu:50-69,
implemented by this package's kernels.  Import this module once; importing it next to the
reference's own ``chipmunk`` extension is an error (the namespace can only be defined once).

Conventions kept from the reference's CUDA provider:
* ``dense_attn(q, k, v)`` takes no scale: head dim 128 uses 1.0 (cosine attention), head dim 64 uses
  0.125 (kernels/chipmunk/csrc/attn/dense_attn.cu:161-163,188-197); it returns ``[o, l_vec]`` with
  ``l_vec = 1 / sum_j exp(s_ij)`` as fp32 [B,H,Lq,1] (dense_attn.cu:227-236).
* ``dense_colsum_attn(q, k, v, p)`` normalises the column sums by the supplied ``p`` (an ``l_vec``) and
  returns ``[o, cs, l_vec]`` (kernels/chipmunk/csrc/attn/dense_colsum_attn.cu:270-280,354-522); ``cs``
  is fp32 here (bf16 there).
* ``csp_attn`` accumulates into ``o`` in place.
``dense_attn_scaled`` / ``dense_colsum_attn_scaled`` are the same operators with an explicit scale.
"""
from __future__ import annotations

import torch

from . import kernels as K
from .sparse_attn_config import get_kernel_config_attn

_LOG2E = 1.4426950408889634


def _default_scale(q) -> float:
    return 1.0 if q.shape[-1] == 128 else 0.125


def _l_vec(M, L):
    return (torch.exp2(-M) / L).unsqueeze(-1)


def _dense_attn(q, k, v):
    o, M, L = K.dense_attn_fwd(q, k, v, _default_scale(q))
    return [o, _l_vec(M, L)]


def _dense_attn_scaled(q, k, v, scale: float):
    o, M, L = K.dense_attn_fwd(q, k, v, scale)
    return [o, _l_vec(M, L)]


def _dense_colsum_attn_scaled(q, k, v, p, scale: float):
    B, H, Lq, _ = q.shape
    # p = 1/sum exp(s): in the kernels' base-2 form that is M' = -log2(p), L' = 1.  A p that underflowed to 0
    # (row maximum above 127 in base 2) is clamped to the smallest normal number instead of giving inf / NaN.
    Mp = (-torch.log2(p.reshape(B, H, Lq).float().clamp_min(torch.finfo(torch.float32).tiny))).contiguous()
    ones = torch.ones_like(Mp)
    bm = get_kernel_config_attn()["bm"]
    if bm % 128 == 0:
        # one sweep: the probabilities that feed P V are normalised with p as they are formed and their column
        # sums come from the same registers (the reference kernel's form, dense_colsum_attn.cu:270-280)
        if bm == 256:
            o, cs, M, L = K.dense_colsum_attn_given_fwd(q, k, v, Mp, ones, scale, return_stats=True, group_tiles=2)
        else:
            o, cs128, M, L = K.dense_colsum_attn_given_fwd(q, k, v, Mp, ones, scale, return_stats=True)
            cs = K.sum_tiles(cs128, bm // 128)
    else:
        o, M, L = K.dense_attn_fwd(q, k, v, scale)
        cs = K.colsum_fwd(q, k, Mp, ones, bm, scale)
    return [o, cs, _l_vec(M, L)]


def _dense_colsum_attn(q, k, v, p):
    return _dense_colsum_attn_scaled(q, k, v, p, _default_scale(q))


def _csp_attn(q, k, v, o, indices, indices_counts, o_scale: int):
    K.csp_attn_fwd(q, k, v, indices, indices_counts, o, int(o_scale), get_kernel_config_attn()["bm"],
                   _default_scale(q), out=o)


def _csp_attn_scaled(q, k, v, o, indices, indices_counts, o_scale: int, scale: float):
    K.csp_attn_fwd(q, k, v, indices, indices_counts, o, int(o_scale), get_kernel_config_attn()["bm"], scale, out=o)


def _mask_to_indices(mask, multiple_of: int, pad_to_multiple_of: int):
    return K.mask_to_indices(mask, multiple_of, pad_to_multiple_of)


def _topk_indices(activation, indices, counts, sparsity_amount: float, multiple_of: int, random_amount: float):
    from .sparse_attn_ops import topk_indices
    topk_indices(activation, indices, counts, sparsity_amount, multiple_of, random_amount)


_SCHEMAS = [
    ("dense_attn(Tensor q, Tensor k, Tensor v) -> Tensor[]", _dense_attn),
    ("dense_attn_scaled(Tensor q, Tensor k, Tensor v, float scale) -> Tensor[]", _dense_attn_scaled),
    ("dense_colsum_attn(Tensor q, Tensor k, Tensor v, Tensor p) -> Tensor[]", _dense_colsum_attn),
    ("dense_colsum_attn_scaled(Tensor q, Tensor k, Tensor v, Tensor p, float scale) -> Tensor[]",
     _dense_colsum_attn_scaled),
    ("csp_attn(Tensor q, Tensor k, Tensor v, Tensor(a!) o, Tensor indices, Tensor indices_counts, int o_scale) -> ()",
     _csp_attn),
    ("csp_attn_scaled(Tensor q, Tensor k, Tensor v, Tensor(a!) o, Tensor indices, Tensor indices_counts, "
     "int o_scale, float scale) -> ()", _csp_attn_scaled),
    ("mask_to_indices(Tensor mask, int multiple_of, int pad_to_multiple_of) -> Tensor[]", _mask_to_indices),
    ("topk_indices(Tensor activation, Tensor(a!) indices, Tensor(b!) counts, float sparsity_amount, "
     "int multiple_of, float random_amount) -> ()", _topk_indices),
]

_library = None


def register() -> None:
    """Defines and implements the operators (idempotent)."""
    global _library
    if _library is not None:
        return
    try:
        lib = torch.library.Library("chipmunk", "DEF")
    except RuntimeError as e:  # namespace already owned by another extension
        raise RuntimeError("torch.ops.chipmunk is already defined by another extension; "
                           "load either that extension or lvar_b200.torch_ops, not both") from e
    for schema, fn in _SCHEMAS:
        lib.define(schema)
        lib.impl(schema.split("(")[0], fn, "CUDA")
    _library = lib


register()
