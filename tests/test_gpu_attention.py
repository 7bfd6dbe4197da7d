"""GPU parity of the attention and column-sum kernels against the CPU oracle and the reference's golden
outputs, through the C ABI (lvar_b200.kernels / lvar_b200.sparse_attn_ops).

Tolerances (bf16 kernels against an fp32 oracle): outputs max-abs <= 2e-2 and mean-abs <= 2e-3;
column sums <= 1e-3 relative; row statistics 1e-4 relative.
"""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

O_MAX, O_MEAN, CS_REL = 2e-2, 2e-3, 1e-3


@pytest.fixture(scope="module")
def K():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from lvar_b200 import kernels
    return kernels


def _qkv(B, H, Lq, Lkv, D, seed=0, peaked=False):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H, Lq, D, generator=g)
    k = torch.randn(B, H, Lkv, D, generator=g)
    v = torch.randn(B, H, Lkv, D, generator=g)
    if peaked:  # seeded rank-8 component on K so that the column sums are peaked
        k = k + 2.0 * (torch.randn(B, H, Lkv, 8, generator=g) @ torch.randn(B, H, 8, D, generator=g))
    return q.bfloat16(), k.bfloat16(), v.bfloat16()


def _check_o(o_gpu, o_ref):
    d = (o_gpu.float().cpu() - o_ref.float()).abs()
    assert torch.isfinite(o_gpu.float()).all()
    assert d.max().item() <= O_MAX, f"max-abs {d.max().item():.3e}"
    assert d.mean().item() <= O_MEAN, f"mean-abs {d.mean().item():.3e}"


def _cs_rel(cs, ref):
    """Largest ELEMENT-WISE relative error of column sums against the fp64 oracle.  Sums below 1e-30 (the
    probability mass of a whole group on a key the peaked rows never look at) are compared absolutely."""
    ref = ref.double()
    return ((cs.double().cpu() - ref).abs() / ref.abs().clamp_min(1e-30)).max().item()


SCHED_PAIRS_ONLY, SCHED_SINGLE_ONE_SLOT = 1, 2  # lvar_attn_args.sched_flags


def _same_to_rounding(a, b):
    """Two bf16 results of the same attention whose probabilities were rounded to bf16 against different reference
    maxima and summed in a different order.  Each probability carries a 2^-9 relative rounding error into the
    output, weighted by |v| (up to about 4 here), whatever the size of the output itself, and the output is rounded
    once more: the two results may differ by as much as each may differ from the exact one (the 2e-2 bar, plus one
    bf16 ulp of outputs of magnitude 4 to 8), and agree far better on average."""
    a, b = a.float(), b.float()
    d = (a - b).abs()
    assert d.max().item() <= 3.2e-2, f"max-abs {d.max().item():.3e}"
    assert d.mean().item() <= 1.5e-3, f"mean-abs {d.mean().item():.3e}"


def _ok_status(K, st):
    code, text = K.read_status(st)
    assert code == 0, text


DENSE_SHAPES = [
    (1, 1, 1, 1, 128), (1, 2, 5, 7, 64), (1, 2, 129, 257, 128), (2, 3, 300, 1000, 128), (2, 3, 300, 1000, 64),
    (2, 16, 256, 680, 64),  # VAR-d16 last scale against all 10 scales
    (1, 2, 1600, 4121, 128),  # Infinity decision scale
]


@pytest.mark.parametrize("B,H,Lq,Lkv,D", DENSE_SHAPES)
def test_dense_attn_matches_oracle(K, B, H, Lq, Lkv, D):
    from oracle import attention as oa
    q, k, v = _qkv(B, H, Lq, Lkv, D, seed=Lq + Lkv)
    st = K.new_status("cuda")
    o, M, L = K.dense_attn_fwd(q.cuda(), k.cuda(), v.cuda(), None, status=st)
    _ok_status(K, st)
    o_ref, M_ref, L_ref = oa.dense_attn(q, k, v)
    _check_o(o, o_ref)
    assert torch.allclose(M.cpu(), M_ref, atol=1e-4, rtol=1e-4)
    assert torch.allclose(L.cpu(), L_ref, atol=0, rtol=1e-4)


def test_dense_attn_scale_one_cosine_like(K):
    """Cosine attention: unit-norm q and k scaled by a per-head factor, softmax scale 1."""
    from oracle import attention as oa
    q, k, v = _qkv(1, 4, 520, 1100, 128, seed=3)
    q = (torch.nn.functional.normalize(q.float(), dim=-1) * 8.0).bfloat16()
    k = torch.nn.functional.normalize(k.float(), dim=-1).bfloat16()
    o, M, L = K.dense_attn_fwd(q.cuda(), k.cuda(), v.cuda(), 1.0)
    o_ref, _, _ = oa.dense_attn(q, k, v, 1.0)
    _check_o(o, o_ref)


def test_dense_attn_strided_views(K):
    """q/k/v as slices of one packed [B, L, 3, H, D] projection (no copies needed)."""
    from oracle import attention as oa
    g = torch.Generator().manual_seed(5)
    packed = torch.randn(2, 384, 3, 4, 64, generator=g).bfloat16()
    q, k, v = (packed[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    pc = packed.cuda()
    qc, kc, vc = (pc[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    o, _, _ = K.dense_attn_fwd(qc, kc, vc)
    _check_o(o, oa.dense_attn(q, k, v)[0])


def test_golden_colsum_cases(K, golden_attention):
    """The reference's naive_dense_colsum_attn / reference_blocksums outputs on stored inputs."""
    g = golden_attention
    for tag in ("a", "b"):
        q, k, v = (g[f"colsum_{tag}_{n}"].bfloat16().cuda() for n in "qkv")
        bm = int(g[f"colsum_{tag}_bm"])
        o, M, L = K.dense_attn_fwd(q, k, v)
        cs = K.colsum_fwd(q, k, M, L, bm)
        _check_o(o, g[f"colsum_{tag}_o"])
        ref = g[f"colsum_{tag}_cs"]
        rel = ((cs.cpu() - ref).abs() / ref.abs().clamp_min(1e-30)).max().item()
        assert rel <= CS_REL, f"colsum relative error {rel:.3e}"


@pytest.mark.parametrize("B,H,Lq,Lkv,D,bm", [
    (1, 1, 1, 1, 64, 256), (1, 2, 31, 5, 128, 32), (2, 3, 300, 1000, 128, 192), (2, 3, 700, 1300, 64, 256),
    (2, 16, 256, 680, 64, 64), (1, 2, 1600, 4121, 128, 192), (1, 2, 1600, 4121, 128, 256)])
def test_colsum_matches_oracle(K, B, H, Lq, Lkv, D, bm):
    from oracle import attention as oa
    q, k, v = _qkv(B, H, Lq, Lkv, D, seed=bm + Lq, peaked=True)
    st = K.new_status("cuda")
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    o, M, L = K.dense_attn_fwd(qc, kc, vc, status=st)
    cs = K.colsum_fwd(qc, kc, M, L, bm, status=st)
    _ok_status(K, st)
    _, cs_ref = oa.dense_colsum_attn(q, k, v, None, q_group_size=bm, dtype=torch.float64)
    rel = ((cs.double().cpu() - cs_ref).abs() / cs_ref.abs().clamp_min(1e-300)).max().item()
    assert rel <= CS_REL, f"colsum relative error {rel:.3e}"
    assert torch.equal(cs, K.colsum_fwd(qc, kc, M, L, bm)), "colsum must be bit-reproducible"


def test_block_sparse_matches_oracle(K):
    from oracle import attention as oa
    for (B, H, Lq, Lkv, D, dens, seed) in [(2, 2, 700, 1500, 128, 0.4, 1), (1, 3, 130, 400, 64, 0.5, 2),
                                          (1, 2, 1024, 1024, 128, 0.15, 3)]:
        q, k, v = _qkv(B, H, Lq, Lkv, D, seed=seed)
        nq, nk = (Lq + 127) // 128, (Lkv + 127) // 128
        g = torch.Generator().manual_seed(seed)
        bm = torch.rand(B, H, nq, nk, generator=g) < dens
        bm[..., 0] = True
        bm[0, 0, -1] = False  # one fully masked row of blocks -> zeros
        st = K.new_status("cuda")
        o = K.block_sparse_attn_fwd(q.cuda(), k.cuda(), v.cuda(), bm.cuda(), status=st)
        _ok_status(K, st)
        _check_o(o, oa.block_sparse_attn(q, k, v, bm))
        assert o[0, 0, (nq - 1) * 128:].abs().max().item() == 0.0
    # broadcast mask [nq, nk]
    q, k, v = _qkv(2, 2, 300, 500, 128, seed=9)
    bm = torch.tensor([[1, 0, 1, 1], [0, 1, 0, 1], [1, 1, 1, 0]], dtype=torch.bool)
    o = K.block_sparse_attn_fwd(q.cuda(), k.cuda(), v.cuda(), bm.cuda())
    _check_o(o, oa.block_sparse_attn(q, k, v, bm))


def test_block_sparse_64_wide_blocks(K):
    """64x64 block masks: four mask entries per 128x128 MMA tile, including row halves with nothing to attend."""
    from oracle import attention as oa
    for (B, H, Lq, Lkv, D, dens, seed) in [(1, 2, 200, 500, 64, 0.4, 21), (2, 2, 700, 1500, 128, 0.3, 22)]:
        q, k, v = _qkv(B, H, Lq, Lkv, D, seed=seed)
        nq, nk = (Lq + 63) // 64, (Lkv + 63) // 64
        g = torch.Generator().manual_seed(seed)
        bm = torch.rand(B, H, nq, nk, generator=g) < dens
        bm[..., 0] = True
        bm[0, 0, 1] = False  # a 64-row half with no block at all -> zeros
        st = K.new_status("cuda")
        o, M, L = K.block_sparse_attn_fwd(q.cuda(), k.cuda(), v.cuda(), bm.cuda(), status=st, block=64,
                                          return_stats=True)
        _ok_status(K, st)
        _check_o(o, oa.block_sparse_attn(q, k, v, bm, block=64))
        assert o[0, 0, 64:128].abs().max().item() == 0.0
        assert (L[0, 0, 64:128] == 0).all()


def test_var_d16_config_end_to_end(K):
    """VAR-d16 shape (B2 H16 D64, last scale 16x16 against all 10 scales, Lkv 680): column sums -> 64x64
    block scores -> mask (scales <= 8x8, own position, top 25 % of the rest) -> block-sparse attention."""
    from lvar_b200 import policy as P
    from oracle import attention as oa
    from oracle import indexing as oi
    B, H, Lq, Lkv, D, blk = 2, 16, 256, 680, 64, 64
    q, k, v = _qkv(B, H, Lq, Lkv, D, seed=0)
    scale = 1.0 / 8.0
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    o_d, M, L = K.dense_attn_fwd(qc, kc, vc, scale)
    cs = K.colsum_fwd(qc, kc, M, L, blk, scale)
    _, cs_ref = oa.dense_colsum_attn(q, k, v, scale, q_group_size=blk, dtype=torch.float64)
    assert ((cs.double().cpu() - cs_ref).abs() / cs_ref).max().item() <= CS_REL
    nq, nk = 4, 11
    always = P.sink_local_blocks(nq, nk, blk, 155, 424, 0, Lq)
    assert torch.equal(always, oi.sink_local_blocks(nq, nk, blk, 155, 424, 0, Lq))
    k_total = int(always[0].sum()) + math.ceil(0.25 * int((~always[0]).sum()))
    scores = K.block_scores(cs, blk)
    mask = K.build_block_mask(scores, always.cuda(), k_total)
    assert torch.equal(mask.cpu(), oi.build_block_mask(scores.cpu(), always, k_total))  # identical score inputs
    o = K.block_sparse_attn_fwd(qc, kc, vc, mask, scale, block=blk)
    _check_o(o, oa.block_sparse_attn(q, k, v, mask.cpu(), scale, block=blk))


def test_block_sparse_csla_mask_last_scale(K):
    """Static sink + local-window block mask of the last Infinity scale (Lq 4096, Lkv 10521), one head."""
    from lvar_b200 import policy as P
    from oracle import attention as oa
    scales = P.INFINITY_SCALES
    mask = P.csla_block_mask([(s, s) for s in scales], [-1] * 8 + [1, 1, 3, 5, 7], 12, 5)
    q, k, v = _qkv(1, 1, 4096, 10521, 128, seed=12)
    o = K.block_sparse_attn_fwd(q.cuda(), k.cuda(), v.cuda(), mask.cuda(), 1.0 / math.sqrt(128))
    _check_o(o, oa.block_sparse_attn(q, k, v, mask))


def test_golden_csp_case(K, golden_attention):
    """The reference's reference_sparse_o output (bm=192, duplicate-free lists, one short list)."""
    g = golden_attention
    q, k, v = (g[f"csp_{n}"].bfloat16().cuda() for n in "qkv")
    zero = torch.zeros_like(q)
    o = K.csp_attn_fwd(q, k, v, g["csp_idx"].cuda(), g["csp_counts"].cuda(), zero, 1, int(g["csp_bm"]))
    _check_o(o, g["csp_o"])


@pytest.mark.parametrize("bm", [64, 128, 192, 256, 320])
def test_csp_attn_matches_oracle(K, bm):
    from oracle import attention as oa
    B, H, Lq, Lkv, D = 2, 2, 700, 900, 128
    q, k, v = _qkv(B, H, Lq, Lkv, D, seed=bm)
    G = (Lq + bm - 1) // bm
    g = torch.Generator().manual_seed(bm)
    cap = 384
    idx = torch.randint(0, Lkv, (B, H, G, cap), generator=g, dtype=torch.int32)  # duplicates on purpose
    counts = torch.randint(1, cap + 1, (B, H, G), generator=g, dtype=torch.int32)
    counts[0, 0, 0] = 0      # empty list: delta = 0
    counts[1, 1, -1] = cap   # full list
    counts[0, 1, 0] = 128    # exactly one tile
    o_in = torch.randn(B, H, Lq, D, generator=g).bfloat16()
    for o_scale in (1, -1):
        st = K.new_status("cuda")
        o = K.csp_attn_fwd(q.cuda(), k.cuda(), v.cuda(), idx.cuda(), counts.cuda(), o_in.cuda(), o_scale, bm,
                           status=st)
        _ok_status(K, st)
        ref = oa.csp_attn(q, k, v, None, idx, counts, o_in, o_scale, bm=bm)
        d = (o.float().cpu() - ref.float()).abs()
        # one bf16 ulp of |o_in| + |delta| <= ~5 is 3.1e-2 at the very top of the range; typical error far lower
        assert d.max().item() <= 3.2e-2 and d.mean().item() <= O_MEAN
        rows0 = slice(0, min(bm, Lq))
        assert torch.equal(o[0, 0, rows0].cpu(), o_in[0, 0, rows0]), "empty list must leave o untouched"


def test_csp_attn_all_keys_equals_dense(K):
    q, k, v = _qkv(1, 2, 512, 640, 64, seed=4)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    dense, _, _ = K.dense_attn_fwd(qc, kc, vc)
    idx = torch.arange(640, dtype=torch.int32).expand(1, 2, 2, 640).contiguous().cuda()
    counts = torch.full((1, 2, 2), 640, dtype=torch.int32, device="cuda")
    o = K.csp_attn_fwd(qc, kc, vc, idx, counts, torch.zeros_like(qc), 1, 256)
    assert (o.float() - dense.float()).abs().max().item() <= 8e-3


@pytest.mark.parametrize("B,H,Lq,Lkv,D", [(1, 2, 700, 900, 64), (2, 3, 1000, 1300, 128), (1, 1, 100, 77, 128)])
def test_fused_dense_colsum_matches_separate_kernels_and_oracle(K, B, H, Lq, Lkv, D):
    """One launch for attention and the column sums of its 128-row query tiles: the output is the dense kernel's
    bit for bit, the sums agree with the stand-alone column-sum kernel and with the fp64 oracle, ragged tiles
    and the single-tile tail items included."""
    from oracle import attention as oa
    q, k, v = _qkv(B, H, Lq, Lkv, D, seed=Lq, peaked=True)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    st = K.new_status("cuda")
    o, cs, M, L = K.dense_colsum_attn_fwd(qc, kc, vc, return_stats=True, status=st)
    _ok_status(K, st)
    # the same schedule (single tiles on one half of the CTA) gives the dense kernel's bits; the default dense
    # schedule splits a single tile's keys over both halves and agrees to rounding
    dense, M0, L0 = K.dense_attn_fwd(qc, kc, vc, sched_flags=SCHED_SINGLE_ONE_SLOT)
    assert torch.equal(o, dense) and torch.equal(M, M0) and torch.equal(L, L0)
    dense_s, M1, L1 = K.dense_attn_fwd(qc, kc, vc)
    _same_to_rounding(dense_s, dense)
    assert torch.allclose(M1, M0, rtol=1e-6, atol=1e-6) and torch.allclose(L1, L0, rtol=1e-5)
    sep = K.colsum_fwd(qc, kc, M0, L0, 128)
    assert cs.shape == sep.shape == (B, H, (Lq + 127) // 128, Lkv)
    assert ((cs - sep).abs() <= 1e-5 * sep.abs().max()).all()
    _, ref = oa.dense_colsum_attn(q, k, v, None, q_group_size=128, dtype=torch.float64)
    assert _cs_rel(cs, ref) <= CS_REL
    # twice in a row on the same stream: the work counter and every barrier phase start over cleanly
    o2, cs2 = K.dense_colsum_attn_fwd(qc, kc, vc)
    assert torch.equal(o2, o) and torch.equal(cs2, cs)
    # one row per 256-row group: the group's two tiles add into the row inside the launch, same bits as adding
    # the per-tile rows afterwards (odd tile counts leave the last group with one tile)
    o3, cs256 = K.dense_colsum_attn_fwd(qc, kc, vc, group_tiles=2)
    assert torch.equal(o3, o) and cs256.shape == (B, H, (Lq + 255) // 256, Lkv)
    assert torch.equal(cs256, K.sum_tiles(cs, 2))


@pytest.mark.parametrize("B,H,Lq,Lkv,D", [(1, 2, 700, 900, 64), (2, 3, 1000, 1300, 128), (1, 1, 100, 77, 128),
                                          (1, 2, 1, 300, 128), (2, 80, 512, 640, 64)])
def test_colsum_tiles_without_output_matches_fused_launch(K, B, H, Lq, Lkv, D):
    """Column sums alone (statistics sweep without P and PV, then the transposed sweep): the sums and the row
    statistics are the fused attention + column-sum launch's bit for bit; with the statistics supplied by the
    caller only the second sweep runs and agrees to rounding.  More work items than SMs in the last case."""
    from oracle import attention as oa
    q, k, v = _qkv(B, H, Lq, Lkv, D, seed=Lq + 1, peaked=True)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    _, want, M0, L0 = K.dense_colsum_attn_fwd(qc, kc, vc, return_stats=True)
    st = K.new_status("cuda")
    cs, M, L = K.colsum_tiles_fwd(qc, kc, return_stats=True, status=st)
    _ok_status(K, st)
    assert torch.equal(cs, want) and torch.equal(M, M0) and torch.equal(L, L0)
    st = K.new_status("cuda")
    cs2 = K.colsum_tiles_fwd(qc, kc, stats=(M0, L0), status=st)
    _ok_status(K, st)
    assert ((cs2 - want).abs() <= 1e-5 * want.abs().max()).all()
    assert torch.equal(K.colsum_tiles_fwd(qc, kc), cs)  # back to back on one stream
    if B * H <= 6:
        _, ref = oa.dense_colsum_attn(q, k, v, None, q_group_size=128, dtype=torch.float64)
        assert _cs_rel(cs, ref) <= CS_REL
        assert _cs_rel(cs2, ref) <= CS_REL


def test_colsum_groups_from_given_stats_and_argument_checks(K):
    """Groups that are multiples of 128 rows take the transposed sweep of the attention kernel and agree with
    the stand-alone kernel (which serves every multiple of 32); bad arguments are refused before any launch."""
    q, k, v = _qkv(2, 2, 900, 1100, 128, seed=21)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    _, M, L = K.dense_attn_fwd(qc, kc, vc)
    for group in (128, 256, 384):
        got = K.colsum_groups_fwd(qc, kc, M, L, group)
        want = K.colsum_fwd(qc, kc, M, L, group)
        assert got.shape == want.shape == (2, 2, (900 + group - 1) // group, 1100)
        assert ((got - want).abs() <= 1e-5 * want.abs().max()).all()
    assert torch.equal(K.colsum_groups_fwd(qc, kc, M, L, 96), K.colsum_fwd(qc, kc, M, L, 96))
    t = torch.arange(2 * 3 * 5 * 7, dtype=torch.float32, device="cuda").view(2, 3, 5, 7)
    assert torch.equal(K.sum_tiles(t, 2)[:, :, 2], t[:, :, 4]) and torch.equal(K.sum_tiles(t, 2)[:, :, 0], t[:, :, 0] + t[:, :, 1])
    with pytest.raises(RuntimeError):
        K.colsum_tiles_fwd(qc, kc[:, :1])                       # head mismatch
    with pytest.raises(RuntimeError):
        K.colsum_tiles_fwd(qc, kc, stats=(M[:, :, :-1].contiguous(), L))  # statistics of another shape
    with pytest.raises(RuntimeError):
        K.colsum_tiles_fwd(qc.float(), kc)                      # not bf16


@pytest.mark.parametrize("s_side,t_side,D,bm", [(12, 16, 128, 256), (5, 13, 64, 64), (16, 16, 128, 192), (20, 17, 64, 256)])
def test_csp_attn_with_resized_ocache_matches_two_launches(K, s_side, t_side, D, bm):
    """The O-cache resize inside the attention epilogue gives the bits of the stand-alone resize kernel followed
    by a plain column-sparse call (ragged last query tile, up- and down-sizing, equal grids)."""
    B, H, Lq, Lkv = 2, 2, t_side * t_side, 500
    q, k, v = _qkv(B, H, Lq, Lkv, D, seed=s_side)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    G = (Lq + bm - 1) // bm
    g = torch.Generator().manual_seed(t_side)
    idx = torch.randint(0, Lkv, (B, H, G, Lkv), generator=g, dtype=torch.int32).cuda()
    counts = torch.randint(0, 300, (B, H, G), generator=g, dtype=torch.int32).cuda()
    cache = torch.randn(B, H, s_side * s_side, D, generator=g).bfloat16().cuda()
    for o_scale in (1, -1):
        st = K.new_status("cuda")
        fused = K.csp_attn_fwd(qc, kc, vc, idx, counts, cache, o_scale, bm, resize_from=s_side, status=st)
        _ok_status(K, st)
        two = K.csp_attn_fwd(qc, kc, vc, idx, counts, K.upsample_ocache(cache, s_side * s_side, Lq), o_scale, bm)
        assert torch.equal(fused, two)
    with pytest.raises(RuntimeError):
        K.csp_attn_fwd(qc, kc, vc, idx, counts, cache[:, :, :-1], 1, bm, resize_from=s_side)


@pytest.mark.parametrize("D", [64, 128])
def test_csp_attn_lists_with_runs_of_consecutive_keys(K, D):
    """Tiles of 128 consecutive keys (the local band of a CS4A list) take the tile-copy path, the other tiles
    the row gather; a run that ends at the last key, one that is cut by the count and one that is off by
    one key in the middle sit next to them."""
    from oracle import attention as oa
    B, H, Lq, Lkv, bm = 1, 2, 512, 1000, 256
    q, k, v = _qkv(B, H, Lq, Lkv, D, seed=11)
    G = Lq // bm
    g = torch.Generator().manual_seed(11)
    run = lambda a: torch.arange(a, a + 128, dtype=torch.int32)
    rnd = lambda: torch.randint(0, Lkv, (128,), generator=g, dtype=torch.int32)
    broken = run(300).clone()
    broken[77] = 5
    lists = [
        torch.cat([rnd(), run(417), run(Lkv - 128), rnd(), run(40)]),       # runs between gathers, run at the end of K
        torch.cat([run(0), broken, run(545), run(100), rnd()]),             # a run with one foreign key
    ]
    idx = torch.zeros(B, H, G, Lkv, dtype=torch.int32)
    counts = torch.zeros(B, H, G, dtype=torch.int32)
    for h in range(H):
        for gi in range(G):
            li = lists[(h + gi) % 2]
            idx[0, h, gi, :li.numel()] = li
            counts[0, h, gi] = li.numel() if (h + gi) % 2 == 0 else li.numel() - 60  # cut inside the last tile
    o_in = torch.randn(B, H, Lq, D, generator=g).bfloat16()
    st = K.new_status("cuda")
    o = K.csp_attn_fwd(q.cuda(), k.cuda(), v.cuda(), idx.cuda(), counts.cuda(), o_in.cuda(), 1, bm, status=st)
    _ok_status(K, st)
    ref = oa.csp_attn(q, k, v, None, idx, counts, o_in, 1, bm=bm)
    d = (o.float().cpu() - ref.float()).abs()
    assert d.max().item() <= 3.2e-2 and d.mean().item() <= O_MEAN


def test_csp_attn_out_of_range_index_is_reported(K):
    q, k, v = _qkv(1, 1, 128, 200, 64, seed=6)
    idx = torch.arange(128, dtype=torch.int32).view(1, 1, 1, 128).clone()
    idx[..., 5] = 10_000
    counts = torch.full((1, 1, 1), 128, dtype=torch.int32)
    st = K.new_status("cuda")
    K.csp_attn_fwd(q.cuda(), k.cuda(), v.cuda(), idx.cuda(), counts.cuda(), torch.zeros_like(q).cuda(), 1, 256,
                   status=st)
    assert K.read_status(st)[0] == 5


def test_forced_wait_timeout_sets_status_and_context_survives(K):
    """A wait limit of zero makes the first unfinished wait give up: the kernel must return, report
    the status and leave the device usable (no trap, no hang)."""
    q, k, v = _qkv(1, 2, 512, 2048, 128, seed=8)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    st = K.new_status("cuda")
    K.dense_attn_fwd(qc, kc, vc, status=st, wait_limit_ns=0)
    torch.cuda.synchronize()
    assert K.read_status(st)[0] == 6
    st2 = K.new_status("cuda")
    o, _, _ = K.dense_attn_fwd(qc, kc, vc, status=st2)
    _ok_status(K, st2)
    ref = torch.nn.functional.scaled_dot_product_attention(qc, kc, vc)
    assert (o.float() - ref.float()).abs().max().item() <= O_MAX


def test_argument_errors(K):
    from lvar_b200._lib import LvarError
    q, k, v = (t.cuda() for t in _qkv(1, 1, 64, 64, 64))
    with pytest.raises(RuntimeError, match="bfloat16"):
        K.dense_attn_fwd(q.float(), k, v)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        K.dense_attn_fwd(q.cpu(), k, v)
    q96 = torch.randn(1, 1, 64, 96, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(LvarError, match="Head dimension must be 64 or 128"):
        K.dense_attn_fwd(q96, q96, q96)
    with pytest.raises(LvarError, match="scale"):
        K.dense_attn_fwd(q, k, v, -1.0)
    with pytest.raises(RuntimeError, match="mismatch"):
        K.dense_attn_fwd(q, k[:, :, :32], v)


# ----------------------------------------------------------------------------------------------
# full-size checks through size-independent properties (Infinity-2B last scale: Lq 4096, Lkv 10521)
# ----------------------------------------------------------------------------------------------
def test_full_size_properties(K):
    B, H, Lq, Lkv, D = 2, 16, 4096, 10521, 128
    q, k, v = (t.cuda() for t in _qkv(B, H, Lq, Lkv, D, seed=0, peaked=True))
    scale = 1.0 / math.sqrt(D)
    dense, M, L = K.dense_attn_fwd(q, k, v, scale)
    ref = torch.nn.functional.scaled_dot_product_attention(q[:1, :2].float(), k[:1, :2].float(), v[:1, :2].float(),
                                                           scale=scale)
    assert (dense[:1, :2].float() - ref).abs().max().item() <= O_MAX
    # a block mask of all ones walks the same tiles in the same order as the dense kernel
    ones = torch.ones(32, 83, dtype=torch.bool, device="cuda")
    assert torch.equal(K.block_sparse_attn_fwd(q, k, v, ones, scale), dense)
    # every softmax row sums to one => each group's column sums add up to the group's row count
    cs = K.colsum_fwd(q, k, M, L, 256, scale)
    assert cs.shape == (B, H, 16, Lkv)
    assert torch.allclose(cs.sum(-1), torch.full((B, H, 16), 256.0, device="cuda"), rtol=1e-3)
    assert (cs >= 0).all()
    # group sums at two group sizes are consistent with each other
    cs128 = K.colsum_fwd(q, k, M, L, 128, scale)
    assert torch.allclose(cs128.view(B, H, 16, 2, Lkv).sum(3), cs, rtol=1e-4, atol=1e-6)
    # the V path is linear, and scaling by a power of two is exact in bf16 and fp32:
    # attention(q, k, 2v) == 2 * attention(q, k, v) bit for bit
    a1 = K.block_sparse_attn_fwd(q[:1], k[:1], v[:1], ones, scale)
    a2 = K.block_sparse_attn_fwd(q[:1], k[:1], (v[:1].float() * 2).bfloat16(), ones, scale)
    assert torch.equal(a2.float(), a1.float() * 2)


# ----------------------------------------------------------------------------------------------
# scheduling variants: single tiles split over both halves of a CTA, caller-supplied work order
# ----------------------------------------------------------------------------------------------
@pytest.mark.parametrize("B,H,Lq,Lkv,D", [(1, 1, 100, 77, 128), (1, 3, 700, 1500, 128), (2, 2, 300, 1000, 64),
                                          (1, 1, 256, 128, 128), (2, 40, 512, 640, 64), (2, 45, 512, 900, 128)])
def test_split_single_tiles_agree_with_pairs_and_oracle(K, B, H, Lq, Lkv, D):
    """A single query tile of the last wave runs on both halves of the CTA, each half on half of the keys, and
    the partial results are merged in the epilogue: same result (to rounding) as the pair schedule and as single
    tiles on one half, for dense and block-sparse attention, row statistics included.  Odd tile counts, one
    tile (nothing for the second half) and more items than SMs are covered."""
    from oracle import attention as oa
    q, k, v = _qkv(B, H, Lq, Lkv, D, seed=Lq + Lkv + 7, peaked=True)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    st = K.new_status("cuda")
    o, M, L = K.dense_attn_fwd(qc, kc, vc, status=st)
    _ok_status(K, st)
    for flags in (SCHED_PAIRS_ONLY, SCHED_SINGLE_ONE_SLOT):
        o2, M2, L2 = K.dense_attn_fwd(qc, kc, vc, sched_flags=flags)
        _same_to_rounding(o, o2)
        assert torch.allclose(M, M2, rtol=1e-6, atol=1e-6) and torch.allclose(L, L2, rtol=1e-5)
    if B * H <= 6:
        o_ref, M_ref, L_ref = oa.dense_attn(q, k, v)
        _check_o(o, o_ref)
        assert torch.allclose(M.cpu(), M_ref, atol=1e-4, rtol=1e-4) and torch.allclose(L.cpu(), L_ref, rtol=1e-4)
    nq, nk = (Lq + 127) // 128, (Lkv + 127) // 128
    g = torch.Generator().manual_seed(Lq)
    bm = torch.rand(B, H, nq, nk, generator=g) < 0.5
    bm[..., 0] = True
    bm[0, 0, -1] = False
    bmc = bm.cuda()
    st = K.new_status("cuda")
    ob, Mb, Lb = K.block_sparse_attn_fwd(qc, kc, vc, bmc, return_stats=True, status=st)
    _ok_status(K, st)
    ob2, Mb2, Lb2 = K.block_sparse_attn_fwd(qc, kc, vc, bmc, return_stats=True, sched_flags=SCHED_PAIRS_ONLY)
    _same_to_rounding(ob, ob2)
    assert torch.allclose(Mb, Mb2, rtol=1e-6, atol=1e-6) and torch.allclose(Lb, Lb2, rtol=1e-5)
    assert torch.equal(ob, K.block_sparse_attn_fwd(qc, kc, vc, bmc))  # bit-reproducible
    if B * H <= 6:
        _check_o(ob, oa.block_sparse_attn(q, k, v, bm))


def test_work_order_heaviest_first(K):
    """A caller-supplied order of the work items changes when a query tile runs, not what it computes: with the
    pair schedule the output is bit-identical, with the default schedule (the END of the order runs as single
    tiles) it agrees to rounding.  The order is a permutation sorted by active KV tiles."""
    from lvar_b200 import policy as P
    from oracle import attention as oa
    scales = P.INFINITY_SCALES
    mask = P.csla_block_mask([(s, s) for s in scales], [-1] * 8 + [1, 1, 3, 5, 7], 11, 5).cuda()
    B, H, Lq, Lkv, D = 2, 12, 2304, 6425, 128
    q, k, v = _qkv(B, H, Lq, Lkv, D, seed=31)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    order = K.heaviest_first_order(mask, B, H)
    n_items = B * H * ((Lq + 255) // 256)
    assert order.dtype == torch.int32 and sorted(order.tolist()) == list(range(n_items))
    tiles = mask.sum(-1)
    per_pair = (tiles[0::2] + torch.nn.functional.pad(tiles[1::2], (0, tiles[0::2].numel() - tiles[1::2].numel())))
    w = per_pair[(order.long() % per_pair.numel())]
    assert (w[:-1] >= w[1:]).all(), "heaviest first"
    plain = K.block_sparse_attn_fwd(qc, kc, vc, mask, sched_flags=SCHED_PAIRS_ONLY)
    st = K.new_status("cuda")
    ordered = K.block_sparse_attn_fwd(qc, kc, vc, mask, work_order=order, sched_flags=SCHED_PAIRS_ONLY, status=st)
    _ok_status(K, st)
    assert torch.equal(plain, ordered)
    st = K.new_status("cuda")
    default = K.block_sparse_attn_fwd(qc, kc, vc, mask, work_order=order, status=st)
    _ok_status(K, st)
    _same_to_rounding(default, plain)
    _check_o(default[:1, :2], oa.block_sparse_attn(q[:1, :2], k[:1, :2], v[:1, :2], mask.cpu()))
    # 64-wide masks: the order counts 128-wide tiles
    m64 = torch.rand(Lq // 64, (Lkv + 63) // 64, generator=torch.Generator().manual_seed(2)) < 0.2
    m64[:, 0] = True
    o64 = K.heaviest_first_order(m64.cuda(), B, H, block=64)
    assert sorted(o64.tolist()) == list(range(n_items))
    a = K.block_sparse_attn_fwd(qc, kc, vc, m64.cuda(), block=64, sched_flags=SCHED_PAIRS_ONLY)
    b = K.block_sparse_attn_fwd(qc, kc, vc, m64.cuda(), block=64, work_order=o64, sched_flags=SCHED_PAIRS_ONLY)
    assert torch.equal(a, b)
    with pytest.raises(RuntimeError):
        K.block_sparse_attn_fwd(qc, kc, vc, mask, work_order=order[:-1].contiguous())


# ----------------------------------------------------------------------------------------------
# attention + column sums in one sweep from given row statistics
# ----------------------------------------------------------------------------------------------
@pytest.mark.parametrize("B,H,Lq,Lkv,D", [(1, 2, 700, 900, 64), (2, 3, 1000, 1300, 128), (1, 1, 100, 77, 128),
                                          (1, 2, 1, 300, 128), (2, 80, 512, 640, 64), (1, 2, 1600, 4121, 128)])
def test_one_sweep_colsum_from_given_stats(K, B, H, Lq, Lkv, D):
    """Given the dense kernel's row statistics, one sweep yields the attention output and the column sums of the very
    probabilities that feed P V: output within the bf16 bar of the oracle, column sums element-wise within 1e-3 of
    the fp64 oracle (peaked keys, ragged last tiles in both directions), bit-reproducible, and the statistics that
    come back are the ones that went in (to rounding)."""
    from oracle import attention as oa
    q, k, v = _qkv(B, H, Lq, Lkv, D, seed=Lq + 3, peaked=True)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    dense, M, L = K.dense_attn_fwd(qc, kc, vc)
    st = K.new_status("cuda")
    o, cs, M2, L2 = K.dense_colsum_attn_given_fwd(qc, kc, vc, M, L, return_stats=True, status=st)
    _ok_status(K, st)
    assert cs.shape == (B, H, (Lq + 127) // 128, Lkv)
    _same_to_rounding(o, dense)
    assert torch.equal(M2, M) and torch.allclose(L2, L, rtol=2e-3)  # row sums of bf16-free fp32 p: ~1 +- 1e-6
    two = K.colsum_tiles_fwd(qc, kc, stats=(M, L))
    assert ((cs - two).abs() <= 1e-4 * two.abs() + 1e-30).all()
    if B * H <= 6:
        o_ref, cs_ref = oa.dense_colsum_attn(q, k, v, None, q_group_size=128, dtype=torch.float64)
        _check_o(o, o_ref)
        assert _cs_rel(cs, cs_ref) <= CS_REL
    o3, cs3 = K.dense_colsum_attn_given_fwd(qc, kc, vc, M, L)
    assert torch.equal(o3, o) and torch.equal(cs3, cs)
    o4, cs256 = K.dense_colsum_attn_given_fwd(qc, kc, vc, M, L, group_tiles=2)
    assert torch.equal(o4, o) and torch.equal(cs256, K.sum_tiles(cs, 2))


def test_one_sweep_colsum_with_statistics_of_another_pass(K):
    """Statistics that are off by a per-row factor (another pass's normaliser): the output is still this attention's
    (it is divided by the measured row sums), the column sums scale with the given normaliser row by row, and the
    returned statistics are the true ones."""
    from oracle import attention as oa
    q, k, v = _qkv(1, 2, 300, 520, 128, seed=77, peaked=True)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    dense, M, L = K.dense_attn_fwd(qc, kc, vc)
    g = torch.Generator().manual_seed(1)
    f = torch.exp2(torch.randn(1, 2, 300, generator=g) * 2).cuda()   # given normaliser = true one x f
    o, cs, M2, L2 = K.dense_colsum_attn_given_fwd(qc, kc, vc, M, (L * f).contiguous(), return_stats=True)
    _same_to_rounding(o, dense)
    assert torch.allclose(L2, L, rtol=2e-3)
    s = (q.double() @ k.double().transpose(-1, -2)) / math.sqrt(128)
    w = torch.softmax(s, dim=-1) / f.cpu().double().unsqueeze(-1)
    ref = torch.stack([w[:, :, i * 128:(i + 1) * 128].sum(2) for i in range(3)], 2)
    assert _cs_rel(cs, ref) <= CS_REL


@pytest.mark.parametrize("bm,resize", [(192, 0), (256, 0), (192, 40), (256, 48)])
def test_csp_attn_many_work_items_per_sm(K, bm, resize):
    """Column-sparse attention with more work items than SMs (every CTA runs several items back to back), ragged
    last groups, with and without the O-cache resize, against the oracle on sampled heads."""
    from oracle import attention as oa
    from oracle import indexing as oi
    B, H, Lq, Lkv, D = 2, 6, 4096, 3000, 128
    q, k, v = _qkv(B, H, Lq, Lkv, D, seed=bm + resize, peaked=True)
    G = (Lq + bm - 1) // bm
    assert B * H * G > 148
    g = torch.Generator().manual_seed(bm)
    cap = 512
    idx = torch.randint(0, Lkv, (B, H, G, Lkv), generator=g, dtype=torch.int32)
    counts = torch.randint(1, cap + 1, (B, H, G), generator=g, dtype=torch.int32)
    counts[0, 0, 3] = 0
    src = resize * resize if resize else Lq
    o_in = torch.randn(B, H, src, D, generator=g).bfloat16()
    st = K.new_status("cuda")
    o = K.csp_attn_fwd(q.cuda(), k.cuda(), v.cuda(), idx.cuda(), counts.cuda(), o_in.cuda(), 1, bm, status=st,
                       resize_from=resize)
    _ok_status(K, st)
    for b, h in ((0, 0), (1, 5), (0, 3)):
        sl = (slice(b, b + 1), slice(h, h + 1))
        base = o_in[sl] if not resize else oi.upsample_ocache(o_in[sl].float(), src, Lq).bfloat16()
        ref = oa.csp_attn(q[sl], k[sl], v[sl], None, idx[sl], counts[sl], base, 1, bm=bm)
        d = (o[sl].float().cpu() - ref.float()).abs()
        assert d.max().item() <= 3.2e-2 and d.mean().item() <= O_MEAN, (b, h, d.max().item())
    assert torch.equal(o, K.csp_attn_fwd(q.cuda(), k.cuda(), v.cuda(), idx.cuda(), counts.cuda(), o_in.cuda(), 1, bm,
                                         resize_from=resize)), "bit-reproducible"


def test_output_into_a_strided_destination_matches_the_default_one(K):
    """`out=`: o written into a [B,H,L,D] view of a [B,L,H,D] buffer (the layout the next projection reads), and
    into a view whose rows start on 16-byte but not on 32-byte boundaries (the epilogue then falls back from
    256-bit to 128-bit stores); both bit-identical to the default contiguous output, for the block-sparse and the
    dense kernel, ragged last tiles included."""
    B, H, Lq, Lkv, D = 2, 3, 700, 1300, 128
    q, k, v = (t.cuda() for t in _qkv(B, H, Lq, Lkv, D, seed=77))
    nq, nk = (Lq + 127) // 128, (Lkv + 127) // 128
    g = torch.Generator().manual_seed(5)
    mask = (torch.rand(B, H, nq, nk, generator=g) < 0.4)
    mask[..., 0] = True
    mask = mask.cuda()
    ref_b = K.block_sparse_attn_fwd(q, k, v, mask)
    ref_d, _, _ = K.dense_attn_fwd(q, k, v)
    # (1) [B,L,H,D] buffer, 32-byte aligned rows
    buf = torch.full((B, Lq, H, D), float("nan"), dtype=torch.bfloat16, device="cuda")
    out = buf.permute(0, 2, 1, 3)
    assert K.block_sparse_attn_fwd(q, k, v, mask, out=out) is out
    assert torch.equal(out, ref_b)
    # (2) rows of D + 8 elements, first row 16 bytes into the buffer: 16-byte aligned only
    wide = torch.full((B, H, Lq, D + 8), float("nan"), dtype=torch.bfloat16, device="cuda")
    out2 = wide[..., 8:]
    assert out2.data_ptr() % 32 == 16
    K.block_sparse_attn_fwd(q, k, v, mask, out=out2)
    assert torch.equal(out2, ref_b)
    assert torch.isnan(wide[..., :8].float()).all(), "nothing outside the destination is written"
    wide.fill_(float("nan"))
    K.dense_attn_fwd(q, k, v, out=out2)
    assert torch.equal(out2, ref_d)
    with pytest.raises(RuntimeError):
        K.dense_attn_fwd(q, k, v, out=wide[..., 4:4 + D])  # base 8 bytes off


def test_seeded_sweep_of_ragged_shapes_against_the_oracle(K):
    """Twenty-four seeded random problems (ragged query and key lengths from 1 to ~900, both head dimensions, both
    mask block widths, masks with empty block rows, dense / block-sparse / fused column sums on the same tensors):
    every output within the output bar of the fp64 oracle (relative to max(1, |o|)), column sums within 1e-3
    element-wise."""
    from oracle import attention as oa
    rng = torch.Generator().manual_seed(20240607)

    def _check_o(o_gpu, o_ref):
        # rows that attend a handful of keys have outputs of magnitude 2 to 4, where one bf16 ulp (1.6e-2 to
        # 3.1e-2) is itself of the size of the absolute bar: the error is taken relative to max(1, |o|)
        d = (o_gpu.float().cpu() - o_ref.float()).abs() / o_ref.float().abs().clamp_min(1.0)
        assert torch.isfinite(o_gpu.float()).all()
        assert d.max().item() <= O_MAX and d.mean().item() <= O_MEAN, (d.max().item(), d.mean().item())

    def ri(lo, hi):
        return int(torch.randint(lo, hi + 1, (1,), generator=rng))

    for case in range(24):
        B, H, D = ri(1, 2), ri(1, 3), (64, 128)[case % 2]
        Lq, Lkv = ri(1, 900), ri(1, 900)
        if case % 6 == 0:
            Lq = ri(1, 3) * 128  # whole tiles
        if case % 8 == 1:
            Lkv = ri(1, 40)      # far less than one tile of keys
        q, k, v = _qkv(B, H, Lq, Lkv, D, seed=1000 + case, peaked=bool(case % 3 == 0))
        qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
        st = K.new_status("cuda")
        o, M, L = K.dense_attn_fwd(qc, kc, vc, status=st)
        _ok_status(K, st)
        o_ref, cs_ref = oa.dense_colsum_attn(q, k, v, D ** -0.5, q_group_size=128, dtype=torch.float64)
        _check_o(o, o_ref)
        o2, cs = K.dense_colsum_attn_fwd(qc, kc, vc, status=st)
        _ok_status(K, st)
        _check_o(o2, o_ref)
        assert _cs_rel(cs, cs_ref) <= CS_REL, f"case {case}: column sums {tuple(q.shape)} x {Lkv}"
        block = (128, 64)[(case // 2) % 2]
        nq, nk = (Lq + block - 1) // block, (Lkv + block - 1) // block
        bm = torch.rand(B, H, nq, nk, generator=rng) < 0.5
        bm[..., 0] = True
        if nq > 1:
            bm[0, 0, nq - 1] = False  # an empty block row: zeros
        ob = K.block_sparse_attn_fwd(qc, kc, vc, bm.cuda(), block=block, status=st)
        _ok_status(K, st)
        _check_o(ob, oa.block_sparse_attn(q, k, v, bm, block=block))


def test_overlapped_launches_keep_stream_order_for_data(K):
    """Attention launches may begin their set-up under the tail of the kernel before them (programmatic dependent
    launch).  A chain in which every launch consumes the output of the one before it, queued without any host
    synchronisation, gives the same bits as the same chain with plain launches, and a launch that follows a torch
    kernel writing its input sees that kernel's result."""
    from lvar_b200 import _lib
    B, H, L, D = 2, 4, 600, 128
    q, k, v = (t.cuda() for t in _qkv(B, H, L, L, D, seed=31))

    def chain(flags):
        x = q.clone()
        for _ in range(12):
            x, _, _ = K.dense_attn_fwd(x, k, v, sched_flags=flags)
            x = x * 2.0  # a torch kernel between two launches: writes the next launch's input
        torch.cuda.synchronize()
        return x

    a = chain(_lib.SCHED_SERIALIZE_LAUNCH)
    for _ in range(3):
        assert torch.equal(chain(0), a)
    # back-to-back launches of ours with nothing in between, each reading the previous one's output
    def chain2(flags):
        x = q.clone()
        outs = []
        for _ in range(12):
            x = K.block_sparse_attn_fwd(x, k, v, torch.ones(5, 5, dtype=torch.bool, device="cuda"), sched_flags=flags)
            outs.append(x)
        torch.cuda.synchronize()
        return outs[-1]
    assert torch.equal(chain2(0), chain2(_lib.SCHED_SERIALIZE_LAUNCH))
