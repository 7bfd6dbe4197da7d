"""The CPU restatement of the QKV prologue against the reference's F.normalize + apply_rotary_emb outputs
and RoPE tables (tests/golden/prologue_ref.npz).  No GPU."""
import pytest
import torch

from oracle import prologue as op

SCALES = [1, 2, 4, 6, 8, 12, 16, 20, 24, 32, 40, 48, 64]


def case(g, name):
    B, L, H, c, scale_ind = (int(x) for x in g[f"{name}_meta"])
    qkv = g[f"{name}_qkv"].view(B, L, 3, H, c).bfloat16()
    return B, L, H, c, scale_ind, qkv, g[f"{name}_scale_mul"], g[f"{name}_cos"], g[f"{name}_sin"]


@pytest.mark.parametrize("name", ["a", "b"])
def test_rope_tables_match_reference(golden_prologue, name):
    B, L, H, c, scale_ind, qkv, sm, cos, sin = case(golden_prologue, name)
    tc, ts = op.rope2d_tables(SCALES, c)
    assert tc.shape == (10521, c // 2)
    n = cos.shape[0]
    assert torch.equal(tc[:n], cos) and torch.equal(ts[:n], sin)
    assert torch.equal(tc[-64:], golden_prologue[f"{name}_cos_tail"])
    assert torch.equal(ts[-64:], golden_prologue[f"{name}_sin_tail"])


@pytest.mark.parametrize("name", ["a", "b"])
def test_prologue_matches_reference(golden_prologue, name):
    B, L, H, c, scale_ind, qkv, sm, cos, sin = case(golden_prologue, name)
    start = sum(s * s for s in SCALES[:scale_ind])
    q, k, v = op.qkv_prologue(qkv, sm, cos, sin, start)
    assert torch.equal(q.float(), golden_prologue[f"{name}_q_out"])
    assert torch.equal(k.float(), golden_prologue[f"{name}_k_out"])
    assert torch.equal(v, qkv[:, :, 2].permute(0, 2, 1, 3))
    # without normalisation and without rotation the prologue is a relayout
    q2, k2, _ = op.qkv_prologue(qkv, None, None, None, 0)
    assert torch.equal(q2, qkv[:, :, 0].permute(0, 2, 1, 3)) and torch.equal(k2, qkv[:, :, 1].permute(0, 2, 1, 3))
