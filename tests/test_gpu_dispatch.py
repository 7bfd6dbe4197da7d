"""The per-(scale, layer) routing of self-attention during generation, and the random-init generation loop
around it, on the GPU.  Every route's output is checked against the CPU oracle's restatement of the same
policy (dense, CS4A decision step, CS4A sparse steps, CSLA), over a shortened scale schedule."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

SCALES = [2, 4, 16, 24, 32]
ATTN_CFG = dict(decision_scale=2, bound_layer=0, top_keys=0.4, cs4a_ws=[1, 1, 1, 3, 5], attn_sink=2,
                win_size=[-1, -1, 1, 3, 5], speedup=0)


@pytest.fixture(scope="module")
def P():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from lvar_b200 import policy
    return policy


def test_routing_and_outputs_over_a_short_schedule(P):
    from lvar_b200.sparse_attn_config import get_kernel_config_attn
    from oracle import attention as oa
    from oracle import indexing as oi
    geo = get_kernel_config_attn()
    bm, mult, pad = geo["bm"], geo["counts_multiple_of"], geo["indices_pad_to"]
    B, H, D = 1, 2, 64
    scale = 0.25
    cum = P.cumulative_tokens(SCALES)
    g = torch.Generator().manual_seed(5)
    kv = torch.randn(B, H, cum[-1], D, generator=g).bfloat16()
    vv = torch.randn(B, H, cum[-1], D, generator=g).bfloat16()
    kc, vc = kv.cuda(), vv.cuda()
    csla = P.build_csla_list(SCALES, ATTN_CFG, num_heads=H, device="cuda")
    assert [m is not None for m in csla] == [False, False, True, True, True]
    layers = [P.SelfAttentionDispatch(li, ATTN_CFG, SCALES, scale=scale) for li in range(2)]
    want_routes = {0: ["dense", "dense", "cs4a_full", "cs4a_sparse", "cs4a_sparse"],
                   1: ["dense", "dense", "csla", "csla", "csla"]}
    state = {}
    for si, side in enumerate(SCALES):
        Lq, Lk = side * side, cum[si + 1]
        q = torch.randn(B, H, Lq, D, generator=g).bfloat16()
        k, v = kv[:, :, :Lk], vv[:, :, :Lk]
        for li, d in enumerate(layers):
            o = d(q.cuda(), kc[:, :, :Lk], vc[:, :, :Lk], scale_ind=si, spattn_fn=csla[si])
            assert d.last_route == want_routes[li][si] == d.route(si, spattn_fn=csla[si])
            assert o.shape == q.shape and o.dtype == torch.bfloat16
            got = o.float().cpu()
            if d.last_route == "dense":
                ref = oa.dense_attn(q, k, v, scale)[0]
                tol = 2e-2
            elif d.last_route == "csla":
                mask = oi.csla_block_mask([(s, s) for s in SCALES], ATTN_CFG["win_size"], si, ATTN_CFG["attn_sink"], 128)
                assert torch.equal(csla[si].block_mask.cpu(), mask)
                ref = oa.block_sparse_attn(q, k, v, mask, scale)
                tol = 2e-2
            elif d.last_route == "cs4a_full":
                ref, cs_ref = oa.dense_colsum_attn(q, k, v, scale, q_group_size=bm)
                st = d.sparse_attn.storage
                n = oi.indices_count(ATTN_CFG["top_keys"], Lk, mult)
                assert st.count_value == n and int(st.counts[0, 0, 0]) == n
                # the selection, as SETS, up to swaps between candidates within 1e-3 of the k-th score
                sel_ref, _ = oi.decision_step_indices(cs_ref, ATTN_CFG["top_keys"], mult, pad)
                for h in range(H):
                    a, b = set(st.indices[0, h, 0, :n].tolist()), set(sel_ref[0, h, 0, :n].tolist())
                    kth = cs_ref[0, h, 0].sort(descending=True).values[n - 1]
                    for j in a ^ b:
                        assert abs(cs_ref[0, h, 0, j] - kth) <= 1e-3 * kth
                state = dict(lists=st.indices.cpu(), counts=st.counts.cpu(),
                             cache=oa.csp_attn(q, k, v, scale, st.indices.cpu(), st.counts.cpu(), ref.bfloat16(), -1, bm=bm))
                assert (st.out_cache.float().cpu() - state["cache"].float()).abs().max() <= 3.2e-2
                tol = 2e-2
            else:
                band, band_count = oi.local_band(SCALES, si, ATTN_CFG["cs4a_ws"][si], bm, mult)
                l_ref, c_ref = oi.sparse_step_indices(state["lists"], state["counts"], Lq, Lk, band, band_count, bm,
                                                      mult, pad)
                up = oi.upsample_ocache(state["cache"].float(), state["cache"].shape[-2], Lq).bfloat16()
                ref = oa.csp_attn(q, k, v, scale, l_ref, c_ref, up, 1, bm=bm).float()
                state["lists"], state["counts"] = l_ref, c_ref
                if si + 1 < len(SCALES):
                    assert torch.equal(d.sparse_attn.storage.indices.cpu(), l_ref)
                tol = 3.2e-2  # one bf16 ulp of the accumulate at |o| < 4
            assert (got - ref.float()).abs().max().item() <= tol, (si, li, d.last_route)


def test_reference_geometry_lists_match_golden_bands(P, golden_indices):
    """With attn.geometry = 'reference' the policy works on the reference's 192-row groups with counts in multiples
    of 64: the local bands are the golden tables of the reference's builder, the decision step keeps
    indices_count keys per group (832 at 4121 keys, top_keys 0.2) and the sparse step's lists are the oracle's."""
    from lvar_b200 import sparse_attn_config as cfg
    from oracle import attention as oa
    from oracle import indexing as oi
    saved = dict(cfg.GLOBAL_CONFIG["attn"])
    try:
        cfg.GLOBAL_CONFIG["attn"].update(geometry="reference", provider="triton", top_keys=0.2)
        assert cfg.get_kernel_config_attn() == {"bm": 192, "counts_multiple_of": 64, "indices_pad_to": 1}
        attn = P.SparseDiffAttn(layer_num=0)
        assert (attn.bm, attn.multiple_of) == (192, 64)
        for s in (11, 12):
            band, count = attn.local_inds[s]
            assert count == int(golden_indices[f"bandcount_bm192_m64_s{s}"])
            assert torch.equal(band, golden_indices[f"band_bm192_m64_s{s}"])
        cum = P.cumulative_tokens(P.INFINITY_SCALES)
        B, H, D = 1, 2, 128
        g = torch.Generator().manual_seed(8)
        kv = torch.randn(B, H, cum[12], D, generator=g).bfloat16()
        vv = torch.randn(B, H, cum[12], D, generator=g).bfloat16()
        kv = kv + (2.0 * (torch.randn(B, H, cum[12], 8, generator=g) @ torch.randn(B, H, 8, D, generator=g))).bfloat16()
        q10 = torch.randn(B, H, 1600, D, generator=g).bfloat16()
        q11 = torch.randn(B, H, 2304, D, generator=g).bfloat16()
        scale = 1.0 / math.sqrt(D)
        k10, v10 = kv[:, :, :cum[11]], vv[:, :, :cum[11]]
        o = attn(q10.cuda(), k10.cuda(), v10.cuda(), scale, do_full_step=True, scale_ind=10)
        o_ref, cs_ref = oa.dense_colsum_attn(q10, k10, v10, scale, q_group_size=192)
        assert (o.float().cpu() - o_ref).abs().max() <= 2e-2
        st = attn.storage
        assert st.count_value == 832 and tuple(st.indices.shape) == (B, H, 9, 4121)
        sel_ref, cnt_ref = oi.decision_step_indices(cs_ref, 0.2, 64, 1)
        assert torch.equal(st.counts.cpu(), cnt_ref)
        for h in range(H):
            for grp in range(9):
                a, b = set(st.indices[0, h, grp, :832].tolist()), set(sel_ref[0, h, grp, :832].tolist())
                kth = cs_ref[0, h, grp].sort(descending=True).values[831]
                for j in a ^ b:
                    assert abs(cs_ref[0, h, grp, j] - kth) <= 1e-3 * kth
        lists, counts = st.indices.cpu(), st.counts.cpu()
        out = attn(q11.cuda(), kv.cuda(), vv.cuda(), scale, scale_ind=11)
        band, band_count = oi.local_band(P.INFINITY_SCALES, 11, 7, 192, 64)
        l_ref, c_ref = oi.sparse_step_indices(lists, counts, 2304, cum[12], band, band_count, 192, 64, 1)
        assert torch.equal(attn.storage.indices.cpu(), l_ref) and torch.equal(attn.storage.counts.cpu(), c_ref)
        assert int(c_ref[0, 0, 0]) == 832 + 512 and tuple(l_ref.shape) == (B, H, 12, 6425)
        cache = oa.csp_attn(q10, k10, v10, scale, lists, counts, o_ref.bfloat16(), -1, bm=192)
        up = oi.upsample_ocache(cache.float(), 1600, 2304).bfloat16()
        ref = oa.csp_attn(q11, kv, vv, scale, l_ref, c_ref, up, 1, bm=192)
        assert (out.float().cpu() - ref.float()).abs().max() <= 3.2e-2
    finally:
        cfg.GLOBAL_CONFIG["attn"].clear()
        cfg.GLOBAL_CONFIG["attn"].update(saved)


def test_generation_loop_small(P):
    """A 4-block, width-256 instance of the generation loop over six scales: the routes follow the schedule,
    a captured CUDA graph of the whole generation replays the eager result bit for bit, and dense and sparse
    self-attention produce the same codes for the scales below the decision scale."""
    from lvar_b200 import infinity_loop as IL
    from lvar_b200 import sparse_attn_config as cfg
    saved = dict(cfg.GLOBAL_CONFIG["attn"])
    try:
        cfg.GLOBAL_CONFIG["attn"].update(decision_scale=3, bound_layer=1, top_keys=0.3, cs4a_ws=[1, 1, 1, 1, 3, 5],
                                         attn_sink=2, win_size=[-1, -1, 1, 1, 3, 5])
        lc = IL.LoopConfig(depth=4, width=256, heads=2, ffn=512, text_dim=64, text_len=8, code_dim=8,
                           scales=(1, 2, 4, 16, 24, 32))
        loop = IL.InfinityLoop(lc, batch=2, seed=1)
        text = torch.randn(2, 8, 64, generator=torch.Generator().manual_seed(3)).bfloat16().cuda()
        out = loop.generate(text, seed=4).clone()
        assert out.shape == (2, 8, 32, 32) and torch.isfinite(out).all()
        # 6 scales x 4 layers: dense below scale 3; from it on layers 0-1 CS4A, layers 2-3 CSLA
        assert loop.routes == {"dense": 12, "cs4a_full": 2, "cs4a_sparse": 4, "csla": 6}
        assert torch.equal(loop.generate(text, seed=4), out), "generation must be deterministic"
        loop.capture(text, seed=4)
        assert torch.equal(loop.replay(), out)
        other = torch.randn(2, 8, 64, generator=torch.Generator().manual_seed(9)).bfloat16().cuda()
        want = loop.generate(other, seed=4).clone()
        assert torch.equal(loop.replay(other), want)
        fl = loop.flops_per_batch()
        assert fl["linear"] > 0 and fl["self_attention_dense"] > 0
    finally:
        cfg.GLOBAL_CONFIG["attn"].clear()
        cfg.GLOBAL_CONFIG["attn"].update(saved)
