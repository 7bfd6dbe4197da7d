"""The reference's OWN policy class running over this package's operator modules on the GPU.

``models/sparvar/sparse_attn.py`` of the reference (class SparseDiffAttn, lines 862-1167) is imported unmodified from
``baseline/_ref`` (see baseline/make_ref.py) with ``kernels.sparse_attn.sparse_attn_ops`` and
``kernels.sparse_attn.sparse_attn_config`` aliased to ``lvar_b200.sparse_attn_ops`` / ``lvar_b200.sparse_attn_config``
- the import swap a maintainer would make - and runs one decision step and two sparse steps of a layer.  Its
outputs, key lists, counts and O-cache are compared with this package's own ``policy.SparseDiffAttn`` on the same
inputs, in the library's default tile geometry and in the reference's (192-row groups).
Skipped when ``baseline/_ref`` has not been made (it is not part of the repository)."""
import importlib
import math
import sys
import types
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

REF = Path(__file__).resolve().parent.parent / "baseline" / "_ref"
ALIASED = ["matplotlib", "matplotlib.pyplot", "kernels", "kernels.sparse_attn", "kernels.sparse_attn.sparse_attn_ops",
           "kernels.sparse_attn.sparse_attn_config", "models", "models.sparvar", "models.sparvar.sparse_attn",
           "models.sparvar.sparse_attn_layer_counter"]


@pytest.fixture()
def reference_module():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    if not (REF / "models" / "sparvar" / "sparse_attn.py").exists():
        pytest.skip("baseline/_ref is absent: run `python baseline/make_ref.py <reference checkout>` first")
    from lvar_b200 import sparse_attn_config, sparse_attn_ops
    saved = {n: sys.modules.get(n) for n in ALIASED}
    saved_cfg = {k: (dict(v) if isinstance(v, dict) else v) for k, v in sparse_attn_config.GLOBAL_CONFIG.items()}
    mpl, plt = types.ModuleType("matplotlib"), types.ModuleType("matplotlib.pyplot")
    mpl.pyplot = plt
    sys.modules.update({"matplotlib": mpl, "matplotlib.pyplot": plt})
    for name, path in (("kernels", None), ("kernels.sparse_attn", None), ("models", REF / "models"),
                       ("models.sparvar", REF / "models" / "sparvar")):
        pkg = types.ModuleType(name)
        pkg.__path__ = [str(path)] if path else []
        sys.modules[name] = pkg
    sys.modules["kernels.sparse_attn.sparse_attn_ops"] = sparse_attn_ops
    sys.modules["kernels.sparse_attn.sparse_attn_config"] = sparse_attn_config
    sparse_attn_config.GLOBAL_CONFIG["offloading"]["global_disable_offloading"] = True  # as the reference's yml
    try:
        yield importlib.import_module("models.sparvar.sparse_attn")
    finally:
        for n, m in saved.items():
            if m is None:
                sys.modules.pop(n, None)
            else:
                sys.modules[n] = m
        for k, v in saved_cfg.items():
            sparse_attn_config.GLOBAL_CONFIG[k] = v


@pytest.mark.parametrize("geometry", [None, "reference"])
def test_reference_sparse_diff_attn_over_this_package(reference_module, geometry):
    from lvar_b200 import policy as P
    from lvar_b200 import sparse_attn_config as cfg
    ref_mod = reference_module
    cfg.GLOBAL_CONFIG["attn"].update(geometry=geometry, provider="triton", top_keys=0.2,
                                     cs4a_ws=[1] * 11 + [7, 9], decision_scale=10)
    geo = cfg.get_kernel_config_attn()
    counter = importlib.import_module("models.sparvar.sparse_attn_layer_counter").LayerCounter(1, 1)
    theirs = ref_mod.SparseDiffAttn(0, counter, use_o_cache=True, spsd_scale=10)
    ours = P.SparseDiffAttn(layer_num=0)
    for s in (11, 12):  # the reference's band builder and this package's agree on the static tables
        assert theirs.local_inds[s][1] == ours.local_inds[s][1]
        assert torch.equal(theirs.local_inds[s][0].to(torch.int32), ours.local_inds[s][0])

    cum = P.cumulative_tokens(P.INFINITY_SCALES)
    B, H, D = 2, 4, 128
    g = torch.Generator(device="cuda").manual_seed(13)
    k_all = torch.randn(B, H, cum[-1], D, generator=g, device="cuda")
    k_all = (k_all + 2.0 * torch.randn(B, H, cum[-1], 8, generator=g, device="cuda")
             @ torch.randn(B, H, 8, D, generator=g, device="cuda")).bfloat16()
    v_all = torch.randn(B, H, cum[-1], D, generator=g, device="cuda").bfloat16()
    scale = 1.0 / math.sqrt(D)
    for si in (10, 11, 12):
        q = torch.randn(B, H, P.INFINITY_SCALES[si] ** 2, D, generator=g, device="cuda").bfloat16()
        k, v = k_all[:, :, :cum[si + 1]].contiguous(), v_all[:, :, :cum[si + 1]].contiguous()
        o_ref = theirs(q, k, v, scale, do_full_step=(si == 10), scale_ind=si, layer_ind=0)
        o_own = ours(q, k, v, scale, do_full_step=(si == 10), scale_ind=si, layer_ind=0)
        assert o_ref.shape == o_own.shape == q.shape
        # one bf16 ulp at |o| < 4: the two classes resize the O-cache with different (both fp32) arithmetic and
        # may list equal-score keys in a different order
        assert (o_ref.float() - o_own.float()).abs().max().item() <= 3.2e-2, si
        assert (o_ref.float() - o_own.float()).abs().mean().item() <= 2e-3, si
        if si < 12:
            li, lc = theirs.storage.get_indices(), theirs.storage.get_counts()
            assert torch.equal(lc, ours.storage.counts)
            n = int(lc[0, 0, 0])
            assert n == ours.storage.count_value and n % geo["counts_multiple_of"] == 0
            a = li[..., :n].sort(-1).values
            b = ours.storage.indices[..., :n].sort(-1).values
            same = (a == b).all(-1)
            # torch.topk and this package's top-k may differ on keys with EQUAL scores only: nearly all lists agree
            assert same.float().mean().item() >= 0.98, f"scale {si}: {int((~same).sum())} of {same.numel()} lists differ"
        if si == 10:
            c_ref, c_own = theirs.storage.get_out_cache(), ours.storage.out_cache
            assert (c_ref.float() - c_own.float()).abs().max().item() <= 3.2e-2
