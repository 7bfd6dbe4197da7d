"""The operator API (lvar_b200.sparse_attn_ops, torch.ops.chipmunk.*) and the policy classes on the GPU:
same call signatures, return conventions and assertions as the reference's modules."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from lvar_b200 import sparse_attn_ops
    return sparse_attn_ops


def _qkv(B, H, Lq, Lkv, D, seed=0):
    g = torch.Generator().manual_seed(seed)
    return tuple(torch.randn(B, H, n, D, generator=g).bfloat16() for n in (Lq, Lkv, Lkv))


def test_dense_attn_and_colsum_return_conventions(ops):
    from lvar_b200.sparse_attn_config import get_kernel_config_attn
    from oracle import attention as oa
    q, k, v = _qkv(2, 4, 600, 900, 128, seed=1)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    o, lse = ops.dense_attn(qc, kc, vc, scale=0.1)
    assert isinstance(lse, tuple) and lse[0].shape == (2, 4, 600, 1) and lse[1].shape == (2, 4, 600, 1)
    o_ref, M_ref, L_ref = oa.dense_attn(q, k, v, 0.1)
    assert (o.float().cpu() - o_ref).abs().max() <= 2e-2
    assert torch.allclose(lse[0].squeeze(-1).cpu(), M_ref, atol=1e-4, rtol=1e-4)
    bm = get_kernel_config_attn()["bm"]
    for fn in (ops.dense_colsum_attn_q, ops.dense_colsum_attn_s):
        o2, cs = fn(qc, kc, vc, 0.1)
        assert cs.shape == (2, 4, (600 + bm - 1) // bm, 900) and cs.dtype == torch.float32
        _, cs_ref = oa.dense_colsum_attn(q, k, v, 0.1, q_group_size=bm, dtype=torch.float64)
        assert ((cs.double().cpu() - cs_ref).abs() / cs_ref).max() <= 1e-3
        # same attention, but the two launches may schedule their last tiles differently: equal to rounding
        assert (o2.float() - o.float()).abs().max() <= 3.2e-2  # one bf16 ulp below 8
        assert (o2.float().cpu() - o_ref).abs().max() <= 2e-2
    # the materialising helper agrees with the kernels
    o3, cs3 = ops.naive_dense_colsum_attn(qc.float(), kc.float(), vc.float(), 0.1, q_group_size=bm)
    assert torch.allclose(cs3, cs, rtol=2e-3, atol=1e-6)


def test_csp_attn_signature_and_asserts(ops):
    from lvar_b200.sparse_attn_config import get_kernel_config_attn
    from oracle import attention as oa
    bm = get_kernel_config_attn()["bm"]
    q, k, v = _qkv(1, 2, 520, 640, 64, seed=2)
    G = (520 + bm - 1) // bm
    g = torch.Generator().manual_seed(2)
    inds = torch.stack([torch.randperm(640, generator=g) for _ in range(2 * G)]).view(1, 2, G, 640).int()
    counts = torch.full((1, 2, G), 256, dtype=torch.int32)
    o0 = torch.randn(1, 2, 520, 64, generator=g).bfloat16()
    o0c = o0.cuda()
    out = ops.csp_attn(q.cuda(), k.cuda(), v.cuda(), None, inds.cuda(), counts.cuda(), o0c, -1)
    assert torch.equal(o0c.cpu(), o0), "the input accumulator is not modified"
    ref = oa.csp_attn(q, k, v, None, inds, counts, o0, -1, bm=bm)
    assert (out.float().cpu() - ref.float()).abs().max() <= 3.2e-2
    with pytest.raises(AssertionError, match="Indices shape mismatch"):
        ops.csp_attn(q.cuda(), k.cuda(), v.cuda(), None, inds[..., :100].cuda(), counts.cuda(), o0c, 1)
    with pytest.raises(AssertionError, match="Indices counts shape mismatch"):
        ops.csp_attn(q.cuda(), k.cuda(), v.cuda(), None, inds.cuda(), counts[..., :1].cuda(), o0c, 1)
    with pytest.raises(AssertionError, match="Output shape mismatch"):
        ops.csp_attn(q.cuda(), k.cuda(), v.cuda(), None, inds.cuda(), counts.cuda(), o0c[:, :, :10], 1)


def test_index_ops_signatures(ops):
    from oracle import indexing as oi
    g = torch.Generator().manual_seed(3)
    m = torch.rand(1, 2, 3, 500, generator=g) < 0.2
    idx, cnt = ops.mask_to_indices(m.cuda(), 64, 192)
    ref_i, ref_c = oi.mask_to_indices(m, 64, 192)
    assert torch.equal(cnt.cpu(), ref_c) and torch.equal(idx.cpu()[ref_i >= 0], ref_i[ref_i >= 0])
    with pytest.raises(RuntimeError, match="mask must be bool type"):
        ops.mask_to_indices(m.int().cuda(), 64, 192)
    act = torch.rand(2, 5, 1000, generator=g)
    inds = torch.full((2, 5, 1000), -1, dtype=torch.int32, device="cuda")
    counts = torch.zeros(2, 5, dtype=torch.int32, device="cuda")
    ops.topk_indices(act.cuda(), inds, counts, 0.9, 64, 0.0)
    assert (counts == 128).all()
    assert torch.equal(inds[..., :128].cpu(), oi.topk_indices(act, 128))
    ops.topk_indices(act.cuda(), inds, counts, 0.0, 64, 0.0)
    assert (counts == 1000).all()
    ops.topk_indices(act.cuda(), inds, counts, 1.0, 64, 0.0)
    assert (counts == 0).all()
    # random extra keys: the exact top half is always inside, about rk of the rest joins, counts are padded to a
    # multiple of 64, and the draw repeats under the same seed
    inds.fill_(-1)
    torch.manual_seed(11)
    ops.topk_indices(act.cuda(), inds, counts, 0.5, 64, 0.1)
    first = (inds.clone(), counts.clone())
    assert (counts % 64 == 0).all() or (counts == 1000).all()
    exact = oi.topk_indices(act, 500)
    n_extra = 0
    for b in range(2):
        for r in range(5):
            c = int(counts[b, r])
            got = set(inds[b, r, :c].cpu().tolist())
            assert len(got) == c and set(exact[b, r].tolist()) <= got and max(got) < 1000 and min(got) >= 0
            n_extra += c - 500
    assert 10 * (0.1 * 500 - 35) <= n_extra <= 10 * (0.1 * 500 + 35 + 63)  # binomial(500, 0.1) per row, + padding
    torch.manual_seed(11)
    ops.topk_indices(act.cuda(), inds, counts, 0.5, 64, 0.1)
    assert torch.equal(counts, first[1])
    for b in range(2):
        for r in range(5):
            c = int(counts[b, r])
            assert torch.equal(inds[b, r, :c], first[0][b, r, :c])
    with pytest.raises(NotImplementedError):
        ops.copy_indices(None, None, None, None)
    packed, shp = ops.bitpack(m.cuda())
    assert torch.equal(ops.bitunpack(packed, shp).cpu(), m)


def test_torch_ops_chipmunk_namespace(ops):
    import lvar_b200.torch_ops  # noqa: F401  registers torch.ops.chipmunk.*
    from oracle import attention as oa
    q, k, v = _qkv(1, 2, 300, 520, 128, seed=4)
    q = (torch.nn.functional.normalize(q.float(), dim=-1) * 6).bfloat16()
    k = torch.nn.functional.normalize(k.float(), dim=-1).bfloat16()
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    o, l_vec = torch.ops.chipmunk.dense_attn(qc, kc, vc)  # head dim 128 => softmax scale 1.0
    o_ref, M, L = oa.dense_attn(q, k, v, 1.0)
    assert (o.float().cpu() - o_ref).abs().max() <= 2e-2
    assert l_vec.shape == (1, 2, 300, 1)
    assert torch.allclose(l_vec.squeeze(-1).cpu(), torch.exp2(-M) / L, rtol=1e-4)
    o2, cs, l2 = torch.ops.chipmunk.dense_colsum_attn(qc, kc, vc, l_vec)
    _, cs_ref = oa.dense_colsum_attn(q, k, v, 1.0, q_group_size=256, dtype=torch.float64)
    assert ((cs.double().cpu() - cs_ref).abs() / cs_ref).max() <= 1e-3
    # the output and the normaliser come from the one-sweep kernel here: equal to the dense kernel's to rounding
    assert (o2.float() - o.float()).abs().max() <= 3.2e-2 and (o2.float().cpu() - o_ref).abs().max() <= 2e-2
    assert torch.allclose(l2, l_vec, rtol=2e-3)
    # csp_attn accumulates in place
    inds = torch.arange(520, dtype=torch.int32).expand(1, 2, 2, 520).contiguous().cuda()
    counts = torch.full((1, 2, 2), 520, dtype=torch.int32, device="cuda")
    acc = o.clone()
    torch.ops.chipmunk.csp_attn(qc, kc, vc, acc, inds, counts, -1)
    assert acc.float().abs().max() <= 2e-2  # O_dense - delta over ALL keys ~ 0
    idx, cnt = torch.ops.chipmunk.mask_to_indices(torch.ones(1, 1, 2, 64, dtype=torch.bool, device="cuda"), 64, 64)
    assert cnt.tolist() == [[[64, 64]]]


def test_sparse_diff_attn_full_then_sparse_steps(ops):
    """CS4A over a small 5-scale schedule: decision step then two sparse steps, against the oracle's
    restatement of the same policy fed with the oracle's own column sums."""
    from lvar_b200 import policy as P
    from lvar_b200.sparse_attn_config import GLOBAL_CONFIG, get_kernel_config_attn
    from oracle import attention as oa
    from oracle import indexing as oi
    geo = get_kernel_config_attn()
    bm, mult, pad = geo["bm"], geo["counts_multiple_of"], geo["indices_pad_to"]
    scales = [2, 4, 16, 24, 32]
    cum = P.cumulative_tokens(scales)
    saved = GLOBAL_CONFIG["attn"]["top_keys"]
    GLOBAL_CONFIG["attn"]["top_keys"] = 0.4
    try:
        attn = P.SparseDiffAttn(layer_num=0, scales=scales, spsd_scale=2, wind_size=[3, 5])
        B, H, D = 1, 2, 64
        g = torch.Generator().manual_seed(11)
        kv = torch.randn(B, H, cum[-1], D, generator=g).bfloat16()
        vv = torch.randn(B, H, cum[-1], D, generator=g).bfloat16()
        qs = {s: torch.randn(B, H, scales[s] ** 2, D, generator=g).bfloat16() for s in (2, 3, 4)}
        scale = 1.0 / math.sqrt(D)
        # --- decision step
        k2, v2 = kv[:, :, :cum[3]], vv[:, :, :cum[3]]
        o = attn(qs[2].cuda(), k2.cuda(), v2.cuda(), scale, do_full_step=True, scale_ind=2)
        o_ref, cs_ref = oa.dense_colsum_attn(qs[2], k2, v2, scale, q_group_size=bm)
        assert (o.float().cpu() - o_ref).abs().max() <= 2e-2
        inds_ref, counts_ref = oi.decision_step_indices(cs_ref, 0.4, mult, pad)
        n = int(counts_ref[0, 0, 0])
        got = attn.storage.indices.cpu()
        # GPU and CPU column sums differ in the last bits: compare the selected SETS and tolerate swaps
        # only between candidates whose scores are within 1e-3 relative of the k-th score
        for h in range(H):
            a, b = set(got[0, h, 0, :n].tolist()), set(inds_ref[0, h, 0, :n].tolist())
            kth = cs_ref[0, h, 0].sort(descending=True).values[n - 1]
            for j in a ^ b:
                assert abs(cs_ref[0, h, 0, j] - kth) <= 1e-3 * kth
        cache_ref = oa.csp_attn(qs[2], k2, v2, scale, got, attn.storage.counts.cpu(), o_ref.bfloat16(), -1, bm=bm)
        assert (attn.storage.out_cache.float().cpu() - cache_ref.float()).abs().max() <= 3.2e-2
        # --- sparse steps (feed the oracle with the GPU's own lists so the comparison is exact in the indices)
        lists, counts, cache = attn.storage.indices.cpu(), attn.storage.counts.cpu(), attn.storage.out_cache.cpu()
        for s in (3, 4):
            ks, vs = kv[:, :, :cum[s + 1]], vv[:, :, :cum[s + 1]]
            out = attn(qs[s].cuda(), ks.cuda(), vs.cuda(), scale, scale_ind=s)
            band, band_count = oi.local_band(scales, s, {3: 3, 4: 5}[s], bm, mult)
            l_ref, c_ref = oi.sparse_step_indices(lists, counts, scales[s] ** 2, cum[s + 1], band, band_count, bm,
                                                  mult, pad)
            up = oi.upsample_ocache(cache.float(), cache.shape[-2], scales[s] ** 2).bfloat16()
            ref = oa.csp_attn(qs[s], ks, vs, scale, l_ref, c_ref, up, 1, bm=bm)
            assert (out.float().cpu() - ref.float()).abs().max() <= 3.2e-2
            if s == 3:
                assert torch.equal(attn.storage.indices.cpu(), l_ref)
                assert torch.equal(attn.storage.counts.cpu(), c_ref)
                lists, counts = l_ref, c_ref
    finally:
        GLOBAL_CONFIG["attn"]["top_keys"] = saved


def test_cs4a_layer_replays_as_a_cuda_graph(ops):
    """A layer's decision step and its two sparse steps captured in one CUDA graph: no host synchronisation,
    no allocation outside the graph's pool, the persistent kernels' work counters reset themselves.  Replays
    give the eager results bit for bit, also after the static inputs have been overwritten."""
    from lvar_b200 import policy as P
    scales = [2, 4, 16, 24, 32]
    cum = P.cumulative_tokens(scales)
    B, H, D = 1, 2, 64
    scale = 1.0 / math.sqrt(D)

    def inputs(seed):
        g = torch.Generator().manual_seed(seed)
        kv = torch.randn(B, H, cum[-1], D, generator=g).bfloat16().cuda()
        vv = torch.randn(B, H, cum[-1], D, generator=g).bfloat16().cuda()
        qs = [torch.randn(B, H, scales[s] ** 2, D, generator=g).bfloat16().cuda() for s in (2, 3, 4)]
        return kv, vv, qs

    def layer_steps(attn, kv, vv, qs):
        outs = []
        for i, s in enumerate((2, 3, 4)):
            outs.append(attn(qs[i], kv[:, :, :cum[s + 1]], vv[:, :, :cum[s + 1]], scale, do_full_step=(s == 2),
                             scale_ind=s))
        return outs

    eager = {seed: [o.clone() for o in layer_steps(P.SparseDiffAttn(layer_num=0, scales=scales, spsd_scale=2,
                                                                   wind_size=[3, 5]), *inputs(seed))]
             for seed in (1, 2)}
    attn = P.SparseDiffAttn(layer_num=0, scales=scales, spsd_scale=2, wind_size=[3, 5])
    kv, vv, qs = inputs(1)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):  # warm-up on the capture stream: caches, scratch and kernel attributes are set here
            layer_steps(attn, kv, vv, qs)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        outs = layer_steps(attn, kv, vv, qs)
    for seed in (1, 2, 1):
        kv2, vv2, qs2 = inputs(seed)
        kv.copy_(kv2)
        vv.copy_(vv2)
        for a, b in zip(qs, qs2):
            a.copy_(b)
        graph.replay()
        torch.cuda.synchronize()
        for got, want in zip(outs, eager[seed]):
            assert torch.equal(got, want)


def test_sparse_flex_attn_class(ops):
    from lvar_b200 import policy as P
    from oracle import attention as oa
    from oracle import indexing as oi
    sched = [(s, s) for s in (2, 4, 8, 16, 24)]
    win = [-1, -1, 1, 3, 5]
    mod = P.SparseFlexAttn(sched, win, q_scale_idx=4, attn_sink_scale=2, num_heads=2)
    S_q, S_k = 576, 4 + 16 + 64 + 256 + 576
    q, k, v = _qkv(1, 2, S_q, S_k, 64, seed=5)
    out = mod(q.cuda(), k.cuda(), v.cuda(), scale=0.125)
    mask = oi.csla_block_mask(sched, win, 4, 2, 128)
    assert torch.equal(mod.block_mask.cpu(), mask)
    assert (out.float().cpu() - oa.block_sparse_attn(q, k, v, mask, 0.125)).abs().max() <= 2e-2
