"""ScaleKV compaction on the GPU against the CPU oracle and the reference's golden selections."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from test_scalekv_oracle import _case, tie_aware_equal  # noqa: E402


@pytest.fixture(scope="module")
def K():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from lvar_b200 import kernels
    return kernels


@pytest.mark.parametrize("name", ["c", "d"])
def test_scores_pool_and_selection_match_oracle(K, golden_scalekv, name):
    from oracle import scalekv as osk
    scale_ind, cap, pooling, q, k, v, window, want = _case(golden_scalekv, name)
    key_len, Lq = k.shape[2], q.shape[2]
    wdev = torch.tensor(window, dtype=torch.int32, device="cuda")
    scores = K.scalekv_scores(q.cuda(), k.cuda(), wdev, key_len - Lq)
    ref = osk.window_scores(q, k, window).float()
    got = scores.cpu()
    assert torch.equal(torch.isinf(got), torch.isinf(ref))
    fin = torch.isfinite(ref)
    # bf16 values: identical up to a rare flip of the last bf16 bit (fp32 summation order inside a dot product)
    assert (got[fin] - ref[fin]).abs().max().item() <= 2.0 ** -7 * ref[fin].abs().max().item()
    assert (got[fin] == ref[fin]).float().mean().item() > 0.97
    for pool in ("maxpool", "avgpool"):
        pooled = K.scalekv_pool(scores, wdev, 5, pool).cpu()
        pref = osk.pooled_scores(scores.cpu().to(torch.bfloat16), 5, pool).float()
        pref[..., window] = float("inf")
        assert torch.equal(pooled, pref)
    # the whole selection, against the oracle's pooled scores (ties and last-bit flips may swap keys)
    pooled = K.scalekv_pool(scores, wdev, 5, pooling)
    idx = K.topk_indices(pooled, cap, ascending_index=True).cpu()
    _, opooled = osk.select_indices(q, k, window, cap, 5, pooling)
    for h in range(2):
        assert torch.equal(idx[0, h], torch.sort(idx[0, h]).values) and len(set(idx[0, h].tolist())) == cap
        assert set(window) <= set(idx[0, h].tolist())
        assert tie_aware_equal(idx[0, h], want[0, h], opooled[0, h].float(), slack=2.0 ** -6)


def test_cluster_update_kv_end_to_end(K, golden_scalekv):
    from lvar_b200.scalekv import ScaleKVCluster
    scale_ind, cap, pooling, q, k, v, window, want = _case(golden_scalekv, "d")
    c = ScaleKVCluster([[cap] * 4 for _ in range(16)], window_size=16, base_capacity=121, kernel_size=5,
                       pooling=pooling, layer_idx=1)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    ko, vo = c.update_kv(kd, qd, vd, scale_ind)
    assert ko.shape == (1, 2, cap, k.shape[-1]) and vo.shape == ko.shape and c.max_capacity == cap
    idx = c.select_indices(kd, qd, scale_ind).cpu().long()
    for h in range(2):
        assert torch.equal(ko[0, h].cpu(), k[0, h][idx[0, h]]) and torch.equal(vo[0, h].cpu(), v[0, h][idx[0, h]])
    # below the base capacity, and when the cache already fits its budget, nothing is touched
    c2 = ScaleKVCluster([[5000] * 4 for _ in range(16)], layer_idx=0)
    k_small = kd[:, :, :100]
    assert c2.update_kv(k_small, qd[:, :, :100], vd[:, :, :100], 3)[0] is k_small
    assert c2.update_kv(kd, qd, vd, scale_ind)[0] is kd


def test_gather_rows_strided_and_clamped(K):
    g = torch.Generator().manual_seed(2)
    big = torch.randn(2, 3, 50, 3 * 64, generator=g).bfloat16().cuda()
    src = big[..., 64:128]                      # a strided view with a contiguous last dimension
    idx = torch.randint(-3, 60, (2, 3, 17), generator=g, dtype=torch.int32).cuda()
    out = K.gather_rows(src, idx)
    ref = torch.gather(src, 2, idx.clamp(0, 49).long().unsqueeze(-1).expand(-1, -1, -1, 64))
    assert torch.equal(out, ref)


def test_scalekv_argument_errors(K):
    q = torch.zeros(1, 1, 16, 64, dtype=torch.bfloat16, device="cuda")
    w = torch.arange(70, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="window"):
        K.scalekv_scores(q, q, w, 0)
    with pytest.raises(RuntimeError, match="bfloat16"):
        K.scalekv_scores(q.float(), q, w[:4], 0)
