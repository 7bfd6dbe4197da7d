"""CPU restatement of the QKV prologue of a self-attention layer during generation (reference:
models/sparvar/basic_sparvar.py:321-350 and models/infinity/basic_infinity.py:42-133).

Test infrastructure only.  Parity is pinned by tests/golden/prologue_ref.npz: the reference's own
precompute_rope2d_freqs_grid and apply_rotary_emb (compiled out of basic_infinity.py) run on seeded inputs
after torch's F.normalize, as SelfAttention.forward does.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch


def rope2d_tables(scales: Sequence[int], head_dim: int, max_edge: int = 128, base: float = 10000.0
                  ) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos, sin fp32 [sum(s*s), head_dim/2] for square scales with rope2d_normalized_by_hw == 2: the token at
    (y, x) of an s x s map takes the angles of grid point (round(y*S/s), round(x*S/s)) of the last scale S;
    first half of the row = y * theta_i, second half = x * theta_i, theta_i = base^(-2i / (head_dim/2))
    (basic_infinity.py:42-103)."""
    half = head_dim // 2
    inv_freq = 1.0 / (base ** (torch.arange(0, half, 2, dtype=torch.int64).float() / half))
    t = torch.arange(max_edge, dtype=torch.int64).float()
    f = torch.outer(t, inv_freq)                         # [max_edge, half/2]
    S = scales[-1]
    rows = []
    for s in scales:
        ys = (torch.arange(s) * (S / s)).round().int().long()
        ang = torch.cat([f[ys][:, None, :].expand(s, s, -1), f[ys][None, :, :].expand(s, s, -1)], dim=-1)
        rows.append(ang.reshape(s * s, half))
    ang = torch.cat(rows, 0)
    return torch.cos(ang), torch.sin(ang)


def qkv_prologue(qkv: torch.Tensor, scale_mul: Optional[torch.Tensor], cos: Optional[torch.Tensor],
                 sin: Optional[torch.Tensor], rope_start: int):
    """qkv bf16 [B,L,3,H,c] -> (q, k, v) bf16 [B,H,L,c]: normalise (fp32, eps 1e-12), q * scale_mul[h], rotate
    pairs (2i, 2i+1) with table rows rope_start.., round once to bf16 (basic_sparvar.py:321-350, 371-384)."""
    B, L, _, H, c = qkv.shape
    q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))  # [B,H,L,c]
    qf, kf = q.float(), k.float()
    if scale_mul is not None:
        qf = qf / qf.norm(dim=-1, keepdim=True).clamp_min(1e-12)
        kf = kf / kf.norm(dim=-1, keepdim=True).clamp_min(1e-12)
        qf = qf * scale_mul.view(1, H, 1, 1).float()
    if cos is not None:
        cs, sn = cos[rope_start:rope_start + L], sin[rope_start:rope_start + L]   # [L, c/2]

        def rot(x):
            x = x.reshape(B, H, L, c // 2, 2)
            return torch.stack([cs * x[..., 0] - sn * x[..., 1], sn * x[..., 0] + cs * x[..., 1]], dim=-1).reshape(B, H, L, c)
        qf, kf = rot(qf), rot(kf)
    return qf.bfloat16(), kf.bfloat16(), v.contiguous()
