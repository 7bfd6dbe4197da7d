"""The CPU restatement of ScaleKV's compaction against what the reference's own class produced
(tests/golden/scalekv_ref.npz), and the host-side mirror of its window / capacity logic.  No GPU."""
import math

import pytest
import torch

from oracle import scalekv as osk

CASES = ["a", "b", "c", "d"]


def _case(g, name):
    scale_ind, cap, avg, bf16 = (int(x) for x in g[f"{name}_meta"])
    dt = torch.bfloat16 if bf16 else torch.float32
    q, k, v = (g[f"s{scale_ind}_{t}"].to(dt) for t in "qkv")
    return scale_ind, cap, ("avgpool" if avg else "maxpool"), q, k, v, g[f"{name}_window"].tolist(), g[f"{name}_idx"]


def tie_aware_equal(got: torch.Tensor, want: torch.Tensor, pooled: torch.Tensor, slack: float = 0.0) -> bool:
    """True when two selections (ascending index lists of one row) differ only in keys whose pooled score ties
    with (or lies within `slack`, relative, of) the lowest selected non-window score."""
    a, b = set(got.tolist()), set(want.tolist())
    if a == b:
        return True
    sel = pooled[torch.tensor(sorted(b))]
    thr = sel[torch.isfinite(sel)].min().item()
    return all(abs(pooled[j].item() - thr) <= slack * abs(thr) for j in a ^ b)


@pytest.mark.parametrize("name", CASES)
def test_oracle_selection_matches_reference(golden_scalekv, name):
    scale_ind, cap, pooling, q, k, v, window, want = _case(golden_scalekv, name)
    key_len = k.shape[2]
    size = osk.SCALE_TOKENS[scale_ind]
    assert osk.window_indices(size, key_len - size, key_len, 16) == window
    ko, vo, idx = osk.compact(q, k, v, scale_ind, cap, 16, 5, pooling)
    assert idx.shape == want.shape and ko.shape == (1, 2, cap, k.shape[-1])
    _, pooled = osk.select_indices(q, k, window, cap, 5, pooling)
    for h in range(2):
        assert torch.equal(idx[0, h], torch.sort(idx[0, h]).values)
        assert set(window) <= set(idx[0, h].tolist())
        if q.dtype == torch.float32:
            assert torch.equal(idx[0, h], want[0, h].long())                 # no ties in fp32: exact
        else:
            assert tie_aware_equal(idx[0, h], want[0, h], pooled[0, h].float())  # bf16 scores tie: any tied key
        assert torch.equal(ko[0, h], k[0, h][idx[0, h]]) and torch.equal(vo[0, h], v[0, h][idx[0, h]])


def test_window_indices_shapes_and_fallbacks():
    # 16 distinct patch centres of a 64x64 map that starts at key 6425
    w = osk.window_indices(4096, 6425, 10521, 16)
    assert len(w) == 16 == len(set(w)) and w == sorted(w) and 6425 <= w[0] and w[-1] < 10521
    # maps smaller than the grid, and non-square sizes: the most recent tokens
    assert osk.window_indices(4, 1, 5, 16) == list(range(0, 5))
    assert osk.window_indices(200, 100, 300, 16) == list(range(284, 300))


def test_host_mirror_agrees_with_oracle():
    sk = pytest.importorskip("lvar_b200.scalekv")
    for size, start, key_len in ((256, 265, 521), (4096, 6425, 10521), (4, 1, 5), (200, 100, 300)):
        assert sk.window_indices(size, start, key_len, 16) == osk.window_indices(size, start, key_len, 16)
    c = sk.ScaleKVCluster([[300, 310]] * 16, layer_idx=1)
    assert c._capacity(6) == 310 and c._capacity(12) == 310
    with pytest.raises(ValueError):
        sk.ScaleKVCluster([], layer_idx=0)
    with pytest.raises(ValueError):
        sk.ScaleKVCluster([[1]], pooling="median")
