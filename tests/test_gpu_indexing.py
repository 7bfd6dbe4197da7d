"""GPU mask / index construction against the CPU oracle: bit-exact for masks, lists and counts."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from lvar_b200 import kernels
    return kernels


def _scores(shape, seed, ties=False):
    g = torch.Generator().manual_seed(seed)
    s = torch.rand(*shape, generator=g)
    if ties:  # few distinct values => many equal scores, exercising the tie rule
        s = torch.round(s * 16) / 16
    return s


@pytest.mark.parametrize("rows,n,k,ties", [
    (3, 1, 1, False), (4, 7, 0, False), (5, 100, 100, True), (6, 1000, 192, False), (6, 1000, 192, True),
    (2 * 2 * 3, 4121, 768, False), (4, 10521, 2176, True), (2, 24576, 2432, False), (3, 10521, 1052, True)])
def test_topk_indices_bit_exact(K, rows, n, k, ties):
    from oracle import indexing as oi
    s = _scores((rows, n), seed=n + k, ties=ties)
    s[0, : min(n, 3)] = -0.0 if ties else s[0, : min(n, 3)]
    for asc in (False, True):
        got, counts = K.topk_indices(s.cuda(), k, ascending_index=asc, out_cols=n, with_counts=True)
        ref = oi.topk_indices(s, k, ascending_index=asc)
        assert torch.equal(got[..., :k].cpu(), ref), f"asc={asc}"
        assert (got[..., k:] == 0).all() and (counts == k).all()


def test_topk_negative_and_special_values(K):
    from oracle import indexing as oi
    s = torch.tensor([[-1.0, -3.0, 0.0, -0.0, 2.5, float("inf"), -float("inf"), 2.5, 1e-38, -1e-38]])
    for k in range(0, 11):
        assert torch.equal(K.topk_indices(s.cuda(), k).cpu(), oi.topk_indices(s, k))


def test_decision_step_indices_match_oracle(K):
    """Decision-step list build: count, top-k by column sum, zero padding to Lkv columns."""
    from lvar_b200 import policy as P
    from oracle import indexing as oi
    bs = _scores((2, 4, 7, 4121), seed=1)
    count = P.indices_count(0.2, 4121, 128)
    inds, counts = K.topk_indices(bs.cuda(), count, out_cols=4121, with_counts=True)
    ref_i, ref_c = oi.decision_step_indices(bs, 0.2, 128, 4)
    assert torch.equal(inds.cpu(), ref_i) and torch.equal(counts.cpu(), ref_c)


@pytest.mark.parametrize("B,H,nq,nk,k_total,ties", [(2, 16, 32, 83, 17, False), (2, 4, 32, 83, 17, True),
                                                    (1, 2, 128, 192, 19, True), (1, 1, 3, 5, 9, False),
                                                    (2, 2, 4, 11, 6, True)])
def test_build_block_mask_bit_exact(K, B, H, nq, nk, k_total, ties):
    from lvar_b200 import policy as P
    from oracle import indexing as oi
    scores = _scores((B, H, nq, nk), seed=nq * nk, ties=ties)
    always = P.sink_local_blocks(nq, nk, 128, 521 if nk > 8 else 128, (nk - nq) * 128 if nk > nq else 0)
    mask, lists, counts = K.build_block_mask(scores.cuda(), always.cuda(), k_total, return_lists=True)
    ref = oi.build_block_mask(scores, always, k_total)
    assert torch.equal(mask.cpu(), ref)
    assert torch.equal(counts.cpu(), ref.sum(-1).int())
    want = max(k_total, int(always.sum(-1).max())) if k_total <= nk else nk
    assert int(counts.max()) <= max(want, int(always.sum(-1).max()))
    for b, h, i in ((0, 0, 0), (B - 1, H - 1, nq - 1)):
        n = int(counts[b, h, i])
        assert lists[b, h, i, :n].cpu().tolist() == torch.nonzero(ref[b, h, i]).flatten().tolist()
        assert (lists[b, h, i, n:] == -1).all()
    # no always-kept blocks at all
    m2 = K.build_block_mask(scores.cuda(), None, min(3, nk))
    assert torch.equal(m2.cpu(), oi.build_block_mask(scores, torch.zeros(nq, nk, dtype=torch.bool), min(3, nk)))


def test_block_scores_match_oracle(K):
    from oracle import indexing as oi
    cs = _scores((2, 3, 5, 1000), seed=2) * 3
    for block in (64, 128):
        got = K.block_scores(cs.cuda(), block).cpu()
        ref = oi.block_scores(cs, block).float()
        assert got.shape == ref.shape
        assert torch.allclose(got, ref, rtol=1e-6, atol=1e-6)
        assert torch.equal(got, K.block_scores(cs.cuda(), block).cpu())


@pytest.mark.parametrize("shape,mult,pad", [((1, 1, 1, 70), 4, 8), ((2, 3, 4, 1000), 64, 192), ((1, 2, 9, 4121), 112, 4),
                                           ((1, 1, 2, 31), 1, 1), ((1, 1, 3, 64), 128, 64)])
def test_mask_to_indices_matches_reference_order(K, shape, mult, pad):
    from oracle import indexing as oi
    g = torch.Generator().manual_seed(shape[-1])
    m = torch.rand(*shape, generator=g) < 0.3
    m[0, 0, 0] = False          # empty row: count 0
    if shape[2] > 1:
        m[0, 0, 1] = True       # full row: nothing to pad with
    idx, cnt = K.mask_to_indices(m.cuda(), mult, pad)
    ref_i, ref_c = oi.mask_to_indices(m, mult, pad)
    assert idx.shape == ref_i.shape and torch.equal(cnt.cpu(), ref_c)
    valid = ref_i >= 0
    assert torch.equal(idx.cpu()[valid], ref_i[valid])


def test_bitpack_roundtrip_and_layout(K):
    from oracle import indexing as oi
    g = torch.Generator().manual_seed(7)
    for shape in ((1,), (9,), (3, 5, 7), (2, 16, 22, 1000)):
        m = torch.rand(*shape, generator=g) < 0.5
        packed, shp = K.bitpack(m.cuda())
        assert torch.equal(packed.cpu(), oi.bitpack(m)[0])
        assert torch.equal(K.bitunpack(packed, shp).cpu(), m)


def test_upsample_ocache_matches_interpolate(K, golden_indices):
    """Bilinear O-cache resize against F.interpolate (what the reference calls) and its golden output."""
    from oracle import indexing as oi
    g = golden_indices
    got = K.upsample_ocache(g["upsample_in"].bfloat16().cuda(), 36, 64)
    ref = oi.upsample_ocache(g["upsample_in"].bfloat16().float(), 36, 64)
    assert (got.float().cpu() - ref).abs().max().item() <= 2e-2
    gen = torch.Generator().manual_seed(3)
    for (B, H, s, t, D) in ((2, 3, 40, 48, 128), (1, 2, 48, 64, 128), (1, 1, 5, 16, 64), (1, 2, 8, 8, 64)):
        x = torch.randn(B, H, s * s, D, generator=gen).bfloat16()
        got = K.upsample_ocache(x.cuda(), s * s, t * t).cpu()
        ref = oi.upsample_ocache(x.float(), s * s, t * t)
        assert got.shape == (B, H, t * t, D)
        d = (got.float() - ref).abs()
        # fp32 interpolation of bf16 inputs, one bf16 rounding of the result
        assert d.max().item() <= 2e-2 and d.mean().item() <= 2e-3


@pytest.mark.gpu
@pytest.mark.parametrize("src_cols,s_count", [(1521, 384), (96, 256), (640, 130)])
def test_sparse_step_lists_match_oracle(K, src_cols, s_count):
    """Remap + stretch + clamp + band append in one kernel, bit-exact against the CPU restatement."""
    from oracle import indexing as oi
    from lvar_b200 import policy as P
    torch.manual_seed(5)
    B, H, Gs, bm, mult, pad_to = 2, 3, 5, 256, 2, 4
    q_len, k_len = 9 * 256 - 17, 4000
    Gk = (q_len + bm - 1) // bm
    inds = torch.randint(0, 5000, (B, H, Gs, src_cols), dtype=torch.int32)
    counts = torch.full((B, H, Gs), s_count, dtype=torch.int32)
    band_count = 70
    band = (torch.arange(band_count)[None, :] + torch.arange(Gk)[:, None] * 11).to(torch.int32)
    want, want_counts = oi.sparse_step_indices(inds, counts, q_len, k_len, band, band_count, bm, mult, pad_to)
    cnt = max(pad_to, (s_count + pad_to - 1) // pad_to * pad_to)
    remap = P.group_remap_table(Gk, Gs).to(device="cuda", dtype=torch.int32)
    got, got_counts = K.sparse_step_lists(inds.cuda(), remap, band.cuda(), cnt, k_len,
                                          count_value=s_count + band_count)
    assert torch.equal(got.cpu(), want)
    assert torch.equal(got_counts.cpu(), want_counts)


@pytest.mark.parametrize("B,H,G,Lkv,block,k_total,peaked", [(2, 16, 32, 10521, 128, 17, True), (1, 2, 4, 680, 64, 6, False),
                                                             (1, 3, 5, 1000, 128, 3, True), (2, 1, 1, 77, 128, 1, False)])
def test_block_mask_from_colsums_equals_two_kernels(K, B, H, G, Lkv, block, k_total, peaked):
    """One pass over the column sums gives the block scores of block_scores bit for bit and the mask of
    build_block_mask; both are the oracle's on the same inputs (ragged last block, ties from a few distinct
    values)."""
    from oracle import indexing as oi
    g = torch.Generator().manual_seed(Lkv + G)
    cs = torch.rand(B, H, G, Lkv, generator=g)
    if peaked:
        cs = cs * torch.exp2(torch.randint(-20, 4, (B, H, G, Lkv), generator=g).float())
    else:
        cs = torch.round(cs * 4) / 4
    nk = (Lkv + block - 1) // block
    always = torch.rand(G, nk, generator=g) < 0.15
    csc = cs.cuda()
    scores = K.block_scores(csc, block)
    want = K.build_block_mask(scores, always.cuda(), k_total)
    mask, got_scores = K.block_mask_from_colsums(csc, always.cuda(), k_total, block, return_scores=True)
    assert torch.equal(got_scores, scores) and torch.equal(mask, want)
    assert torch.equal(K.block_mask_from_colsums(csc, always.cuda(), k_total, block), want)
    assert torch.equal(mask.cpu(), oi.build_block_mask(scores.cpu(), always, k_total))
    assert torch.equal(K.block_mask_from_colsums(csc, None, k_total, block),
                       K.build_block_mask(scores, None, k_total))


def test_topk_is_torch_topk_on_the_same_gpu(K):
    """The decision step of the reference takes ``torch.topk(bs, k, dim=-1).indices`` (models/sparvar/sparse_attn.py:
    1012-1039).  On scores without ties this package's kernel returns the same index SEQUENCE (descending by value);
    with ties, where torch.topk's order is not defined, the same multiset of values and the lower-index-first rule."""
    g = torch.Generator(device="cuda").manual_seed(17)
    for rows, n, k in ((64, 4121, 824), (32, 10521, 2176), (7, 257, 257), (5, 1000, 1)):
        s = torch.rand(rows, n, generator=g, device="cuda").argsort(-1).float() * 0.37 - 100.0  # distinct values
        got = K.topk_indices(s, k)
        ref = torch.topk(s, k, dim=-1).indices
        assert torch.equal(got.long(), ref)
    # ties: quantised scores
    s = (torch.randn(16, 4121, generator=g, device="cuda") * 4).round()
    k = 600
    got = K.topk_indices(s, k).long()
    ref = torch.topk(s, k, dim=-1)
    assert torch.equal(torch.gather(s, -1, got), ref.values)          # the same values, in descending order
    same_val = torch.gather(s, -1, got)
    inc = (got[:, 1:] > got[:, :-1]) | (same_val[:, 1:] != same_val[:, :-1])
    assert inc.all()                                                   # lower index first among equals
