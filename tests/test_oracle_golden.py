"""Pins the CPU oracle against outputs of the reference's own Python code (tests/golden/*.npz,
produced by tests/golden/make_golden.py).  CPU only."""
import numpy as np
import torch

from oracle import attention as oa
from oracle import indexing as oi

SCALES = [1, 2, 4, 6, 8, 12, 16, 20, 24, 32, 40, 48, 64]


def test_dense_colsum_matches_reference_naive(golden_attention):
    g = golden_attention
    for tag in ("a", "b"):
        q, k, v = g[f"colsum_{tag}_q"], g[f"colsum_{tag}_k"], g[f"colsum_{tag}_v"]
        bm = int(g[f"colsum_{tag}_bm"])
        o, cs = oa.dense_colsum_attn(q, k, v, None, q_group_size=bm)
        assert torch.allclose(o, g[f"colsum_{tag}_o"], atol=2e-6, rtol=1e-5)
        assert torch.allclose(cs, g[f"colsum_{tag}_cs"], atol=1e-6, rtol=1e-5)
        assert torch.allclose(cs, g[f"colsum_{tag}_blocksums"], atol=1e-6, rtol=1e-5)
        # the second formulation (M, L statistics) agrees with the first
        o2, M, L = oa.dense_attn(q, k, v)
        assert torch.allclose(o2, o, atol=2e-6, rtol=1e-5)
        s = (q @ k.transpose(-1, -2)) / np.sqrt(q.shape[-1])
        p = torch.exp2(s * oa.LOG2E - M[..., None]) / L[..., None]
        assert torch.allclose(p.sum(-1), torch.ones_like(M), atol=1e-5)


def test_csp_matches_reference_sparse_o(golden_attention):
    g = golden_attention
    q, k, v = g["csp_q"], g["csp_k"], g["csp_v"]
    delta = oa.csp_delta(q, k, v, g["csp_idx"], g["csp_counts"], None, bm=int(g["csp_bm"]))
    assert torch.allclose(delta, g["csp_o"], atol=2e-6, rtol=1e-5)
    # multiset semantics: listing every key twice leaves the softmax unchanged
    idx2 = torch.cat([g["csp_idx"], g["csp_idx"]], dim=-1)
    cnt2 = torch.full_like(g["csp_counts"], idx2.shape[-1])
    full = torch.full_like(g["csp_counts"], g["csp_idx"].shape[-1])
    d1 = oa.csp_delta(q, k, v, g["csp_idx"], full, None, bm=int(g["csp_bm"]))
    d2 = oa.csp_delta(q, k, v, idx2, cnt2, None, bm=int(g["csp_bm"]))
    assert torch.allclose(d1, d2, atol=1e-5)


def test_csp_attn_accumulate_rounding():
    torch.manual_seed(0)
    q, k, v = (torch.randn(1, 1, 70, 64).bfloat16() for _ in range(3))
    o = torch.randn(1, 1, 70, 64).bfloat16()
    idx = torch.arange(70, dtype=torch.int32).view(1, 1, 1, 70)
    cnt = torch.tensor([[[64]]], dtype=torch.int32)
    out = oa.csp_attn(q, k, v, None, idx, cnt, o, -1, bm=192)
    assert out.dtype == torch.bfloat16
    d = oa.csp_delta(q, k, v, idx, cnt, None, 192).bfloat16()
    assert torch.equal(out, o - d)


def test_local_bands_match_reference(golden_indices):
    g = golden_indices
    assert g["cum"].tolist() == [0, 1, 5, 21, 57, 121, 265, 521, 921, 1497, 2521, 4121, 6425, 10521]
    for bm, mult in ((192, 64), (192, 112), (256, 128)):
        for s, ws in ((11, 7), (12, 9)):
            band, cnt = oi.local_band(SCALES, s, ws, bm, mult)
            assert cnt == int(g[f"bandcount_bm{bm}_m{mult}_s{s}"])
            assert torch.equal(band, g[f"band_bm{bm}_m{mult}_s{s}"].long())
    # known answers: band shapes and end points for the two reference geometries
    b, c = oi.local_band(SCALES, 11, 7, 192, 64)
    assert (tuple(b.shape), c, int(b[0, 0]), int(b[0, -1]), int(b[-1, 0]), int(b[-1, -1])) == \
        ((12, 512), 512, 4121, 4632, 5913, 6424)
    b, c = oi.local_band(SCALES, 12, 9, 192, 112)
    assert (tuple(b.shape), c, int(b[0, 0]), int(b[0, -1]), int(b[-1, 0]), int(b[-1, -1])) == \
        ((22, 784), 784, 6425, 7208, 9737, 10520)


def test_local_window_indices_match_reference(golden_indices):
    g = golden_indices
    assert torch.equal(oi.local_window_indices(5, 7, 10, (3, 3)), g["lwi_5x7_w3_base10"].long())
    assert torch.equal(oi.local_window_indices(4, 4, 0, (5, 5)), g["lwi_4x4_w5_base0"].long())


def test_group_remap_matches_reference(golden_indices):
    g = golden_indices
    assert oi.group_remap_table(12, 9).tolist() == [0, 1, 1, 2, 3, 4, 4, 5, 6, 7, 7, 8]
    assert oi.group_remap_table(22, 12).tolist() == [0, 0, 1, 1, 2, 2, 3, 4, 4, 5, 5, 6, 6, 7, 7, 8, 8, 9, 10, 10,
                                                     11, 11]
    for tag in ("a", "b", "c"):
        qlen, klen, bm, pad = (int(x) for x in g[f"remap_{tag}_args"])
        out, cnt = oi.map_inds_counts_across_scales(g[f"remap_{tag}_in"], g[f"remap_{tag}_cnt"], qlen, klen, bm, pad)
        assert torch.equal(out, g[f"remap_{tag}_out"])
        assert torch.equal(cnt, g[f"remap_{tag}_outcnt"])


def test_indices_count_known_answers():
    assert [oi.indices_count(t, 4121, 64) for t in (0.05, 0.15, 0.2)] == [192, 640, 832]
    assert [oi.indices_count(t, 4121, 112) for t in (0.05, 0.15, 0.2)] == [224, 672, 784]


def test_upsample_matches_reference(golden_indices):
    g = golden_indices
    assert torch.allclose(oi.upsample_ocache(g["upsample_in"], 36, 64), g["upsample_out"], atol=1e-6)


def test_csla_block_mask_matches_reference(golden_csla):
    sched = [(s, s) for s in SCALES]
    win = [-1, -1, -1, -1, -1, -1, -1, -1, 1, 1, 3, 5, 7]
    for q_scale_idx, block in ((10, 128), (11, 128), (12, 128), (9, 64)):
        m = oi.csla_block_mask(sched, win, q_scale_idx, 5, block)
        assert torch.equal(m, golden_csla[f"csla_s{q_scale_idx}_b{block}"].bool())


def test_topk_tie_rule_and_decision_step():
    s = torch.tensor([[1.0, 3.0, 3.0, 2.0, 3.0, -0.0, 0.0]])
    assert oi.topk_indices(s, 4).tolist() == [[1, 2, 4, 3]]
    assert oi.topk_indices(s, 4, ascending_index=True).tolist() == [[1, 2, 3, 4]]
    assert oi.topk_indices(s, 7).tolist() == [[1, 2, 4, 3, 0, 5, 6]]
    bs = torch.rand(1, 2, 3, 1000)
    inds, counts = oi.decision_step_indices(bs, 0.2, 64, 4)
    assert inds.shape == (1, 2, 3, 1000) and counts.unique().tolist() == [192]
    ref = torch.topk(bs, 192, dim=-1).indices
    assert torch.equal(inds[..., :192].long().sort(-1).values, ref.sort(-1).values)


def test_mask_to_indices_order_and_padding():
    m = torch.zeros(1, 1, 1, 70, dtype=torch.bool)
    m[..., [0, 1, 32, 33, 64, 69]] = True
    idx, cnt = oi.mask_to_indices(m, 4, 8)
    assert idx.shape == (1, 1, 1, 72) and cnt.item() == 8
    # lane 0 owns 0,32,64; lane 1 owns 1,33; lane 5 owns 69; padding = first unset columns 2,3
    assert idx[0, 0, 0, :8].tolist() == [0, 32, 64, 1, 33, 69, 2, 3]


def test_bitpack_roundtrip():
    torch.manual_seed(1)
    m = torch.rand(3, 5, 7) > 0.5
    packed, shape = oi.bitpack(m)
    assert packed.dtype == torch.uint8 and packed.numel() == (m.numel() + 7) // 8
    assert torch.equal(oi.bitunpack(packed, shape), m)
    one = torch.zeros(9, dtype=torch.bool)
    one[0] = one[8] = True
    assert oi.bitpack(one)[0].tolist() == [1, 1]


def test_build_block_mask_counts_and_ties():
    scores = torch.tensor([[[[5.0, 1.0, 7.0, 7.0, 0.5, 7.0]]]])
    always = torch.tensor([[True, False, False, False, False, False]])
    m = oi.build_block_mask(scores, always, 3)
    assert m[0, 0, 0].tolist() == [True, False, True, True, False, False]
    assert oi.sink_local_blocks(2, 6, 128, 300, 512).tolist() == [
        [True, True, True, False, True, False], [True, True, True, False, False, True]]
