"""This package's index kernels and the CPU oracle against the REFERENCE'S OWN CUDA kernels on the same GPU.

``oracle/build_ref.py`` compiles ``kernels/chipmunk/csrc/indexed_io/mask_to_indices.cu`` and ``topk_indices.cu``
from a reference checkout, unmodified, for sm_100a into ``oracle/_ref/`` (they are plain CUDA, unlike the
reference's attention kernels).  Where that library is present:

* ``mask_to_indices``: counts and every defined list entry are the reference kernel's, bit for bit, for this
  package's kernel and for the oracle's restatement of the reference's order;
* ``topk_indices``: the reference keeps the columns at or above a cutoff taken from a sorted sample of the row's
  first 1024 values, this package the exact top-k.  At the reference's own count per row the two select the same
  SET of columns (the order of the reference's list is that of its atomics), which is what makes the exact kernel
  a stand-in for it.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from oracle.build_ref import load_built
    mod = load_built()
    if mod is None:
        pytest.skip("oracle/_ref/lvar_ref_indexed_io.so has not been built (python oracle/build_ref.py <reference>)")
    return mod


@pytest.fixture(scope="module")
def K():
    from lvar_b200 import kernels
    return kernels


@pytest.mark.parametrize("n,multiple_of,pad_to", [(1000, 64, 192), (680, 112, 192), (4121, 64, 4), (96, 1, 1),
                                                  (33, 32, 64), (2048, 128, 128)])
def test_mask_to_indices_is_the_reference_kernels_output(ref, K, n, multiple_of, pad_to):
    from oracle import indexing as oi
    g = torch.Generator().manual_seed(n + multiple_of)
    b, h, m = 2, 3, 5
    mask = torch.rand(b, h, m, n, generator=g) < 0.3
    mask[0, 0, 0] = False                 # empty row: count 0
    mask[0, 0, 1, : n // 2] = True        # a dense half
    mask[1, 2, 4] = torch.rand(n, generator=g) < 0.9
    r_idx, r_cnt = ref.mask_to_indices(mask.cuda(), multiple_of, pad_to)
    torch.cuda.synchronize()
    o_idx, o_cnt = K.mask_to_indices(mask.cuda(), multiple_of, pad_to)
    c_idx, c_cnt = oi.mask_to_indices(mask, multiple_of, pad_to)
    assert r_idx.shape == o_idx.shape == c_idx.shape
    assert torch.equal(r_cnt, o_cnt) and torch.equal(r_cnt.cpu(), c_cnt)
    # entries the reference writes: the set columns, then as many unset columns as the padding needs and the row has
    written = torch.minimum(r_cnt.cpu(), mask.sum(-1).to(torch.int32) + (~mask).sum(-1).to(torch.int32))
    pos = torch.arange(r_idx.shape[-1]).expand_as(r_idx)
    live = pos < written.unsqueeze(-1)
    assert torch.equal(o_idx.cpu()[live], r_idx.cpu()[live])
    assert torch.equal(c_idx[live], r_idx.cpu()[live])


@pytest.mark.parametrize("cols,sparsity", [(2048, 0.9), (4121, 0.8), (10521, 0.95)])
def test_exact_topk_selects_the_reference_kernels_set_at_its_count(ref, K, cols, sparsity):
    g = torch.Generator().manual_seed(cols)
    batch, rows = 2, 4
    act = torch.randn(batch, rows, cols, generator=g).cuda()
    idx = torch.full((batch, rows, cols), -1, dtype=torch.int32, device="cuda")
    cnt = torch.zeros(batch, rows, dtype=torch.int32, device="cuda")
    ref.topk_indices(act, idx, cnt, sparsity, 1, 0.0)   # multiple_of 1: no padding entries, no random keys
    torch.cuda.synchronize()
    expect = (1.0 - sparsity) * cols
    for b in range(batch):
        for r in range(rows):
            c = int(cnt[b, r])
            # a quantile of 1024 sampled values: within a few standard errors of the asked fraction
            assert abs(c - expect) <= 6 * (sparsity * (1 - sparsity) / 1024) ** 0.5 * cols + 2, (c, expect)
            theirs = set(idx[b, r, :c].cpu().tolist())
            assert len(theirs) == c and min(theirs) >= 0 and max(theirs) < cols
            ours = K.topk_indices(act[b:b + 1, r:r + 1].contiguous(), c)
            assert set(ours.flatten().cpu().tolist()) == theirs
