"""The block-sparse kernel against PyTorch's own ``flex_attention`` on the same GPU.

The reference's static sink + local-window attention (``SparseFlexAttn``, models/sparvar/basic_sparvar.py:47-194)
turns its fine mask into a block-level lookup, hands it to ``create_block_mask`` and calls ``flex_attention``; this
package builds the same block mask on the host (pinned against the reference's by a golden fixture) and runs its
own block-sparse kernel.  ``flex_attention`` is PyTorch's, not the reference's, and no reference test pins its
output; here it is run on the very tensors the kernel gets: the scales a generation uses it for (40x40 and 48x48
query grids over the cumulative keys), 128-wide blocks, the reference's call (``scale`` passed through).
"""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("q_scale_idx,heads", [(10, 2), (11, 2)])
def test_block_sparse_kernel_matches_flex_attention(q_scale_idx, heads):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    try:
        from torch.nn.attention.flex_attention import create_block_mask, flex_attention
    except Exception as e:  # pragma: no cover
        pytest.skip(f"flex_attention unavailable: {e}")
    from lvar_b200 import policy as P
    scales = list(P.INFINITY_SCALES)
    sched = [(s, s) for s in scales]
    kernel_schedule = [1] * 11 + [7, 9]
    kernel_schedule[10] = 5
    mod = P.SparseFlexAttn(sched, kernel_schedule, q_scale_idx=q_scale_idx, attn_sink_scale=5, block_size=128,
                           num_heads=heads)
    bm = mod.block_mask_cpu.cuda()
    cum = P.cumulative_tokens(scales)
    Lq, Lkv, D, B = scales[q_scale_idx] ** 2, cum[q_scale_idx + 1], 128, 1
    assert bm.shape == ((Lq + 127) // 128, (Lkv + 127) // 128) and not bm.all() and bm.any(-1).all()
    g = torch.Generator(device="cuda").manual_seed(q_scale_idx)
    q = torch.randn(B, heads, Lq, D, generator=g, device="cuda")
    k = torch.randn(B, heads, Lkv, D, generator=g, device="cuda")
    v = torch.randn(B, heads, Lkv, D, generator=g, device="cuda").bfloat16()
    # the model's cosine attention: unit-norm q (times a per-head factor) and k, softmax scale 1
    q = (torch.nn.functional.normalize(q, dim=-1) * 8.0).bfloat16()
    k = torch.nn.functional.normalize(k, dim=-1).bfloat16()

    def mask_mod(b, h, q_idx, kv_idx):  # the reference's final_block_mask_mod: a lookup in the block-level mask
        return bm[q_idx // 128, kv_idx // 128]

    block_mask = create_block_mask(mask_mod, B=1, H=heads, Q_LEN=Lq, KV_LEN=Lkv, device="cuda", BLOCK_SIZE=128)
    try:
        theirs = torch.compile(flex_attention)(q, k, v, block_mask=block_mask, scale=1.0)
    except Exception:
        theirs = flex_attention(q, k, v, block_mask=block_mask, scale=1.0)  # eager form of the same operator
    ours = mod.forward(q, k, v, scale=1.0)
    torch.cuda.synchronize()
    d = (ours.float() - theirs.float()).abs()
    assert torch.isfinite(ours.float()).all()
    assert d.max().item() <= 4e-2 and d.mean().item() <= 2e-3, (d.max().item(), d.mean().item())
    # and both against fp32 masked softmax on one head
    fine = bm.repeat_interleave(128, 0)[:Lq].repeat_interleave(128, 1)[:, :Lkv]
    s = (q[0, 0].float() @ k[0, 0].float().T).masked_fill(~fine, float("-inf"))
    ref = torch.softmax(s, dim=-1) @ v[0, 0].float()
    for name, t in (("ours", ours), ("flex_attention", theirs)):
        e = (t[0, 0].float() - ref).abs()
        assert e.max().item() <= 2e-2 and e.mean().item() <= 2e-3, (name, e.max().item(), e.mean().item())
