"""Fused QKV prologue on the GPU against the CPU oracle (itself pinned on the reference's outputs)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from test_prologue_oracle import SCALES, case  # noqa: E402


@pytest.fixture(scope="module")
def K():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from lvar_b200 import kernels
    return kernels


def _close_bf16(got: torch.Tensor, want: torch.Tensor) -> None:
    """Equal except for a rare flip of the last bf16 bit (the fp32 sum of squares is taken in another order)."""
    g, w = got.float().cpu(), want.float()
    assert (g == w).float().mean().item() > 0.999
    assert ((g - w).abs() <= 2.0 ** -7 * w.abs() + 1e-30).all()


@pytest.mark.parametrize("name", ["a", "b"])
def test_prologue_matches_oracle_and_reference(K, golden_prologue, name):
    from oracle import prologue as op
    B, L, H, c, scale_ind, qkv, sm, cos, sin = case(golden_prologue, name)
    start = sum(s * s for s in SCALES[:scale_ind])
    cap, pos = start + L + 5, start
    k_cache = torch.full((B, H, cap, c), 7.0, dtype=torch.bfloat16, device="cuda")
    v_cache = torch.full((B, H, cap, c), 7.0, dtype=torch.bfloat16, device="cuda")
    q = K.qkv_prologue(qkv.cuda(), sm.cuda(), cos.cuda(), sin.cuda(), start, k_cache, v_cache, pos)
    _close_bf16(q, golden_prologue[f"{name}_q_out"])
    _close_bf16(k_cache[:, :, pos:pos + L], golden_prologue[f"{name}_k_out"])
    assert torch.equal(v_cache[:, :, pos:pos + L].cpu(), qkv[:, :, 2].permute(0, 2, 1, 3))
    # rows outside the appended range are untouched
    assert (k_cache[:, :, :pos] == 7).all() and (k_cache[:, :, pos + L:] == 7).all()
    assert (v_cache[:, :, :pos] == 7).all() and (v_cache[:, :, pos + L:] == 7).all()
    # relayout only
    q2 = K.qkv_prologue(qkv.cuda(), None, None, None, 0, k_cache, v_cache, 0)
    oq, ok, _ = op.qkv_prologue(qkv, None, None, None, 0)
    assert torch.equal(q2.cpu(), oq) and torch.equal(k_cache[:, :, :L].cpu(), ok)


def test_prologue_feeds_attention_like_the_reference_call_site(K, golden_prologue):
    """q, the appended K cache and V cache go straight into dense attention: same result as attention on the
    oracle's tensors (the reference casts its fp32 q and k to bf16 at this point)."""
    from oracle import prologue as op
    B, L, H, c, scale_ind, qkv, sm, cos, sin = case(golden_prologue, "b")
    start = sum(s * s for s in SCALES[:scale_ind])
    oq, ok, ov = op.qkv_prologue(qkv, sm, cos, sin, start)
    k_cache = torch.zeros((B, H, L, c), dtype=torch.bfloat16, device="cuda")
    v_cache = torch.zeros_like(k_cache)
    q = K.qkv_prologue(qkv.cuda(), sm.cuda(), cos.cuda(), sin.cuda(), start, k_cache, v_cache, 0)
    o, _, _ = K.dense_attn_fwd(q, k_cache, v_cache, 1.0)
    ref = torch.nn.functional.scaled_dot_product_attention(oq.float(), ok.float(), ov.float(), scale=1.0)
    assert (o.float().cpu() - ref).abs().max().item() <= 2e-2


def test_prologue_argument_errors(K):
    qkv = torch.zeros(1, 4, 3, 2, 64, dtype=torch.bfloat16, device="cuda")
    cache = torch.zeros(1, 2, 3, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="room for rows"):
        K.qkv_prologue(qkv, None, None, None, 0, cache, cache.clone(), 0)
    with pytest.raises(RuntimeError, match="bfloat16"):
        K.qkv_prologue(qkv.float(), None, None, None, 0, cache, cache.clone(), 0)
