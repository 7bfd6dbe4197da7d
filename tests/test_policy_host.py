"""Host-side policy tables of the product (lvar_b200.policy) against the CPU oracle and the golden
outputs of the reference.  CPU only: builds tables, launches nothing."""
import torch

from lvar_b200 import policy as P
from lvar_b200 import sparse_attn_config as cfg
from oracle import indexing as oi

SCALES = [1, 2, 4, 6, 8, 12, 16, 20, 24, 32, 40, 48, 64]
WIN = [-1, -1, -1, -1, -1, -1, -1, -1, 1, 1, 3, 5, 7]


def test_cumulative_tokens_and_counts():
    assert P.cumulative_tokens(SCALES) == [0, 1, 5, 21, 57, 121, 265, 521, 921, 1497, 2521, 4121, 6425, 10521]
    for t in (0.05, 0.15, 0.2):
        for m in (64, 112, 128):
            assert P.indices_count(t, 4121, m) == oi.indices_count(t, 4121, m)


def test_local_band_matches_golden_and_oracle(golden_indices):
    for bm, mult in ((192, 64), (192, 112), (256, 128)):
        for s, ws in ((11, 7), (12, 9)):
            band, count = P.local_band(SCALES, s, ws, bm, mult)
            assert count == int(golden_indices[f"bandcount_bm{bm}_m{mult}_s{s}"])
            assert torch.equal(band, golden_indices[f"band_bm{bm}_m{mult}_s{s}"].long())
    # shapes the golden files do not hold: even windows, tiny groups, one group
    small = [1, 2, 3, 5, 8]
    for s, ws, bm, mult in ((4, 3, 16, 8), (4, 4, 24, 0), (3, 5, 7, 4), (4, 1, 64, 16), (2, 3, 192, 64)):
        band, count = P.local_band(small, s, ws, bm, mult)
        oband, ocount = oi.local_band(small, s, ws, bm, mult)
        assert count == ocount and torch.equal(band, oband)


def test_group_remap_table():
    for gk, gs in ((12, 9), (22, 12), (16, 7), (1, 5), (9, 9), (3, 1)):
        assert torch.equal(P.group_remap_table(gk, gs), oi.group_remap_table(gk, gs))


def test_csla_block_mask_matches_golden_and_oracle(golden_csla):
    sched = [(s, s) for s in SCALES]
    for q_scale_idx, block in ((10, 128), (11, 128), (12, 128), (9, 64)):
        m = P.csla_block_mask(sched, WIN, q_scale_idx, 5, block)
        assert torch.equal(m, golden_csla[f"csla_s{q_scale_idx}_b{block}"].bool())
    # non-square schedule, wide windows, no sink
    sched2 = [(1, 2), (2, 3), (3, 5), (6, 4), (8, 8)]
    for win, sink in (([1, 3, 3, 5, 3], 0), ([-1, -1, 1, 3, 7], 2), ([3, 3, 3, 3, 3], 4)):
        for block in (8, 16):
            assert torch.equal(P.csla_block_mask(sched2, win, 4, sink, block),
                               oi.csla_block_mask(sched2, win, 4, sink, block))


def test_sink_local_blocks_matches_oracle():
    for args in ((32, 83, 128, 521, 6425, 0, 4096), (4, 11, 64, 155, 424, 0, 256), (128, 192, 128, 0, 8192, 2, 16384),
                 (3, 9, 128, 300, 700, 1, 300)):
        assert torch.equal(P.sink_local_blocks(*args), oi.sink_local_blocks(*args))


def test_config_surface(tmp_path):
    assert set(cfg.BASE_CONFIG) >= {"attn", "mlp", "patchify", "offloading", "step_caching", "steps", "world_size"}
    assert cfg.GLOBAL_CONFIG["attn"]["win_size"] == [-1] * 8 + [1, 1, 3, 5, 7]
    geo = cfg.get_kernel_config_attn()
    assert set(geo) == {"bm", "counts_multiple_of", "indices_pad_to"}
    assert geo["bm"] % 32 == 0 and geo["counts_multiple_of"] == 128
    assert cfg.get_kernel_config_mlp() == {"bm": 128, "mbm": 128, "counts_multiple_of": 256}
    y = tmp_path / "c.yml"
    y.write_text("attn:\n  top_keys: 0.2\n  provider: cuda\n  cs4a_ws: [1,1,1,1,1,1,1,1,1,1,1,7,9]\n")
    saved = dict(cfg.GLOBAL_CONFIG["attn"])
    try:
        cfg.load_from_file(str(y))
        assert cfg.GLOBAL_CONFIG["attn"]["top_keys"] == 0.2
        assert cfg.GLOBAL_CONFIG["attn"]["attn_sink"] == 5  # untouched keys survive the deep merge
        assert cfg.get_kernel_config_attn() == geo          # one backend whatever the provider says
        cfg.GLOBAL_CONFIG["attn"]["provider"] = "rocm"
        try:
            cfg.get_kernel_config_attn()
            raise AssertionError("expected ValueError")
        except ValueError as e:
            assert "Invalid provider" in str(e)
    finally:
        cfg.GLOBAL_CONFIG["attn"].clear()
        cfg.GLOBAL_CONFIG["attn"].update(saved)


def test_sparse_diff_attn_tables():
    a = P.SparseDiffAttn(layer_num=0)
    geo = cfg.get_kernel_config_attn()
    assert sorted(a.local_inds) == [11, 12]
    for s in (11, 12):
        band, count = a.local_inds[s]
        oband, ocount = oi.local_band(SCALES, s, {11: 7, 12: 9}[s], geo["bm"], geo["counts_multiple_of"])
        assert count == ocount and torch.equal(band.long(), oband)
        assert count % geo["counts_multiple_of"] == 0


def test_dispatch_routes_follow_the_reference_branches():
    """13 scales x 32 layers: the route is the branch SelfAttention.forward takes in
    models/sparvar/basic_sparvar.py:353-387 with the yml's decision_scale 10 and bound_layer 10."""
    attn_cfg = dict(cfg.GLOBAL_CONFIG["attn"], decision_scale=10, bound_layer=10, top_keys=0.2)
    spattn = [None] * 10 + ["fn10", "fn11", "fn12"]  # spattn_compile_list: modules for the last three scales
    layers = [P.SelfAttentionDispatch(li, attn_cfg) for li in (0, 10, 11, 31)]
    counts = {}
    for si in range(13):
        for d in layers:
            li = d.layer_ind
            if spattn[si] is not None and li > 10:
                want = "csla"
            elif si == 10 and li <= 10:
                want = "cs4a_full"
            elif si > 10 and li <= 10:
                want = "cs4a_sparse"
            else:
                want = "dense"
            assert d.route(si, spattn_fn=spattn[si]) == want
            counts[want] = counts.get(want, 0) + 1
    assert counts == {"dense": 40, "cs4a_full": 2, "cs4a_sparse": 4, "csla": 6}
    # without a static-mask module (flex attention switched off) the late layers stay dense
    assert layers[-1].route(12, spattn_fn=None) == "dense"
    # a layer's CS4A module is built for the configured decision scale and windows
    assert sorted(layers[0].sparse_attn.local_inds) == [11, 12] and layers[0].sparse_attn.top_keys == 0.2


def test_geometry_override():
    saved = dict(cfg.GLOBAL_CONFIG["attn"])
    try:
        base = cfg.get_kernel_config_attn()
        assert base == {"bm": 256, "counts_multiple_of": 128, "indices_pad_to": 4}
        cfg.GLOBAL_CONFIG["attn"]["geometry"] = "reference"
        cfg.GLOBAL_CONFIG["attn"]["provider"] = "triton"
        assert cfg.get_kernel_config_attn() == {"bm": 192, "counts_multiple_of": 64, "indices_pad_to": 1}
        cfg.GLOBAL_CONFIG["attn"]["provider"] = "cuda"
        assert cfg.get_kernel_config_attn() == {"bm": 192, "counts_multiple_of": 112, "indices_pad_to": 4}
        a = P.SparseDiffAttn(layer_num=0, top_keys=0.2)
        assert (a.bm, a.multiple_of, a.indices_pad_to) == (192, 112, 4) and a.local_inds[11][1] == 560
        cfg.GLOBAL_CONFIG["attn"]["geometry"] = {"bm": 128}
        assert cfg.get_kernel_config_attn() == dict(base, bm=128)
        for bad in ({"bm": 100}, {"rows": 3}, "fast"):
            cfg.GLOBAL_CONFIG["attn"]["geometry"] = bad
            try:
                cfg.get_kernel_config_attn()
                raise AssertionError("expected ValueError")
            except ValueError:
                pass
    finally:
        cfg.GLOBAL_CONFIG["attn"].clear()
        cfg.GLOBAL_CONFIG["attn"].update(saved)


def test_heaviest_first_order_host():
    from lvar_b200 import kernels as K
    mask = P.csla_block_mask([(s, s) for s in SCALES], WIN, 12, 5)          # [32, 83], ragged rows
    order = K.heaviest_first_order(mask, 2, 3)
    pairs = mask.sum(-1).view(16, 2).sum(-1)
    assert order.dtype == torch.int32 and sorted(order.tolist()) == list(range(2 * 3 * 16))
    w = pairs[order.long() % 16]
    assert (w[:-1] >= w[1:]).all()
    # per-(batch, head) masks and an odd number of query tiles
    g = torch.Generator().manual_seed(0)
    m = torch.rand(2, 3, 5, 9, generator=g) < 0.4
    order = K.heaviest_first_order(m, 2, 3)
    t = torch.nn.functional.pad(m.sum(-1), (0, 1)).view(2, 3, 3, 2).sum(-1).reshape(-1)
    assert sorted(order.tolist()) == list(range(18)) and (t[order.long()][:-1] >= t[order.long()][1:]).all()
