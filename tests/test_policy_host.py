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


def test_upsample_matches_golden(golden_indices):
    out = P.upsample_ocache(golden_indices["upsample_in"], 36, 64)
    assert torch.allclose(out, golden_indices["upsample_out"], atol=1e-6)


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
