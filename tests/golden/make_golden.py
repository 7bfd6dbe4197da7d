"""Generates the golden fixtures in this directory by RUNNING THE REFERENCE'S OWN PYTHON CODE.

Run once where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/Lvar

The reference is imported in place (nothing is copied from it): ``kernels.sparse_attn`` directly,
``models/sparvar/sparse_attn.py`` through a namespace package with three stand-ins for things the
CPU container lacks (matplotlib, ``torch.cuda.Stream``), and the CSLA mask builder by compiling the
one method ``SparseFlexAttn.create_cross_scale_block_attn_mask`` out of ``basic_sparvar.py`` (the
module itself needs timm and flash-attn CUDA ops).  Inputs are seeded; inputs and the reference's
outputs are stored together so the tests never need the reference again.
"""
from __future__ import annotations

import ast
import importlib
import os
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
SCALES = [1, 2, 4, 6, 8, 12, 16, 20, 24, 32, 40, 48, 64]


def _install_stubs(ref: Path) -> None:
    sys.path.insert(0, str(ref))
    mpl = types.ModuleType("matplotlib")
    plt = types.ModuleType("matplotlib.pyplot")
    mpl.pyplot = plt
    sys.modules.setdefault("matplotlib", mpl)
    sys.modules.setdefault("matplotlib.pyplot", plt)
    if not torch.cuda.is_available():
        torch.cuda.Stream = lambda *a, **k: None  # module-level streams in sparse_attn.py
    # `models/__init__.py` imports a sub-package that does not exist in the checkout: bypass it.
    for name, rel in (("models", "models"), ("models.sparvar", "models/sparvar")):
        pkg = types.ModuleType(name)
        pkg.__path__ = [str(ref / rel)]
        sys.modules[name] = pkg


def _bf16_exact(*shape, gen, scale=1.0):
    """fp32 tensor whose values are exactly representable in bf16 (so GPU bf16 runs see the same data)."""
    return (torch.randn(*shape, generator=gen) * scale).bfloat16().float()


def make_attention(ref_ops, ref_colsum, ref_csp) -> dict:
    out = {}
    g = torch.Generator().manual_seed(1234)
    # --- colsum: naive_dense_colsum_attn (ops:179-200) + reference_blocksums (colsum.py:487-500)
    for tag, (B, H, Lq, Lkv, D, bm) in {"a": (1, 2, 200, 300, 64, 64), "b": (1, 2, 300, 450, 128, 192)}.items():
        q, k, v = (_bf16_exact(B, H, n, D, gen=g) for n in (Lq, Lkv, Lkv))
        scale = 1.0 / np.sqrt(D)
        o, cs = ref_ops.naive_dense_colsum_attn(q, k, v, scale, q_group_size=bm)
        O2, P = ref_colsum.dense_reference_o_and_p(q, k, v)
        Bs = ref_colsum.reference_blocksums(P, bm=bm)
        assert torch.allclose(cs, Bs, atol=1e-5, rtol=1e-5)
        out.update({f"colsum_{tag}_q": q, f"colsum_{tag}_k": k, f"colsum_{tag}_v": v, f"colsum_{tag}_o": o,
                    f"colsum_{tag}_cs": cs, f"colsum_{tag}_bm": torch.tensor(bm),
                    f"colsum_{tag}_blocksums": Bs, f"colsum_{tag}_o2": O2})
    # --- csp: reference_sparse_o (attn_csp.py:437-471), duplicate-free lists
    B, H, Lq, Lkv, D, bm = 1, 2, 400, 512, 64, 192
    q, k, v = (_bf16_exact(B, H, n, D, gen=g) for n in (Lq, Lkv, Lkv))
    G = (Lq + bm - 1) // bm
    cnt = 128
    idx = torch.stack([torch.randperm(Lkv, generator=g)[:cnt] for _ in range(B * H * G)]).view(B, H, G, cnt).int()
    counts = torch.full((B, H, G), cnt, dtype=torch.int32)
    counts[0, 1, 1] = 64
    o_ref = ref_csp.reference_sparse_o(q, k, v, idx, counts, bm=bm)
    out.update({"csp_q": q, "csp_k": k, "csp_v": v, "csp_idx": idx, "csp_counts": counts, "csp_o": o_ref,
                "csp_bm": torch.tensor(bm)})
    return out


def make_indices(sa) -> dict:
    out = {}
    n_list = [s * s for s in SCALES]
    cum = torch.tensor([0] + list(np.cumsum(n_list)))
    out["cum"] = cum
    # local bands (sparse_attn.py:921-938) for the three geometries of interest
    for bm, mult in ((192, 64), (192, 112), (256, 128)):
        for scale_ind, ws in ((11, 7), (12, 9)):
            idx_abs, _, kv_len, _ = sa.build_crossscale_indices(
                scales=SCALES, n_list=n_list, cum=cum[:scale_ind + 2], K=scale_ind, window_spec={0: (ws, ws)})
            gi, gc = sa.aggregate_group_indices(idx_abs, q_len=n_list[scale_ind], kv_len=kv_len, bm=bm,
                                                counts_multiple_of=mult)
            out[f"band_bm{bm}_m{mult}_s{scale_ind}"] = gi
            out[f"bandcount_bm{bm}_m{mult}_s{scale_ind}"] = torch.tensor(gc)
    # a small window table
    out["lwi_5x7_w3_base10"] = sa.local_window_indices(5, 7, 10, win=(3, 3))
    out["lwi_4x4_w5_base0"] = sa.local_window_indices(4, 4, 0, win=(5, 5))
    # cross-scale remap (sparse_attn.py:365-421), no-sink path
    g = torch.Generator().manual_seed(99)
    for tag, (Gs, Ks, cnt, qlen, klen, bm, pad) in {
        "a": (9, 4121, 832, 2304, 6425, 192, 1),
        "b": (12, 6425, 1344, 4096, 10521, 192, 1),
        "c": (7, 200, 256, 4096, 300, 256, 4),
    }.items():
        inds_S = torch.randint(0, klen, (1, 2, Gs, Ks), generator=g, dtype=torch.int32)
        counts_S = torch.full((1, 2, Gs), cnt, dtype=torch.int32)
        ik, ck = sa.map_inds_counts_across_scales(inds_S, counts_S, cur_q_len=qlen, cur_k_len=klen, bm=bm,
                                                  indices_pad_to=pad)
        out.update({f"remap_{tag}_in": inds_S, f"remap_{tag}_cnt": counts_S, f"remap_{tag}_out": ik,
                    f"remap_{tag}_outcnt": ck,
                    f"remap_{tag}_args": torch.tensor([qlen, klen, bm, pad])})
    # O-cache upsample (sparse_attn.py:324-362)
    oc = torch.randn(1, 2, 36, 8, generator=g)
    out["upsample_in"] = oc
    out["upsample_out"] = sa.upsample_Ocache(oc, 36, 64, upsample_mode="bilinear")
    return out


def make_csla(ref: Path) -> dict:
    """Compiles the single method create_cross_scale_block_attn_mask from the reference file and runs it
    on the CPU (basic_sparvar.py:74-185)."""
    import torch.nn.functional as F
    from torch.nn.attention.flex_attention import create_mask
    src = (ref / "models/sparvar/basic_sparvar.py").read_text()
    tree = ast.parse(src)
    fn = None
    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name == "create_cross_scale_block_attn_mask":
            fn = node
    assert fn is not None
    mod = ast.Module(body=[fn], type_ignores=[])
    ns = {"torch": torch, "np": np, "F": F, "create_mask": create_mask}
    exec(compile(mod, "basic_sparvar.create_cross_scale_block_attn_mask", "exec"), ns)
    method = ns["create_cross_scale_block_attn_mask"]
    out = {}
    sched = [(s, s) for s in SCALES]
    win = [-1, -1, -1, -1, -1, -1, -1, -1, 1, 1, 3, 5, 7]
    for q_scale_idx, block in ((10, 128), (11, 128), (12, 128), (9, 64)):
        holder = types.SimpleNamespace(block_size=block)
        final_mod = method(holder, scale_schedule=sched, kernel_schedule=win, q_scale_idx=q_scale_idx,
                           attn_sink_scale=5, device="cpu")
        cells = dict(zip(final_mod.__code__.co_freevars, (c.cell_contents for c in final_mod.__closure__)))
        out[f"csla_s{q_scale_idx}_b{block}"] = cells["block_level_mask"]
    return out


def make_scalekv(ref: Path) -> dict:
    """Runs the reference's ScaleKVCluster.update_kv (models/scalekv/scale_kv.py:12-301) on the CPU.  The class
    is compiled out of the file because the module's import of the model package does not resolve."""
    import math
    import warnings
    import torch.nn.functional as F
    src = (ref / "models/scalekv/scale_kv.py").read_text()
    cls = [n for n in ast.parse(src).body if isinstance(n, ast.ClassDef) and n.name == "ScaleKVCluster"][0]
    ns = {"torch": torch, "F": F, "math": math, "warnings": warnings}
    exec(compile(ast.Module(body=[cls], type_ignores=[]), "scale_kv.ScaleKVCluster", "exec"), ns)
    Cluster = ns["ScaleKVCluster"]
    tokens = [1, 4, 16, 36, 64, 144, 256, 400, 576, 1024, 1600, 2304, 4096]
    out = {}
    cases = (("a", torch.float32, 6, 300, "maxpool", 64), ("b", torch.float32, 7, 350, "avgpool", 128),
             ("c", torch.bfloat16, 6, 300, "maxpool", 64), ("d", torch.bfloat16, 7, 420, "maxpool", 128))
    for name, dtype, scale_ind, cap, pooling, D in cases:
        gen = torch.Generator().manual_seed(100 + scale_ind)  # cases of one scale share their inputs
        B, H = 1, 2
        key_len, Lq = sum(tokens[:scale_ind + 1]), tokens[scale_ind]
        q = _bf16_exact(B, H, Lq, D, gen=gen)
        k = _bf16_exact(B, H, key_len, D, gen=gen)
        v = _bf16_exact(B, H, key_len, D, gen=gen)
        cluster = Cluster([[cap] * 4 for _ in range(16)], window_size=16, base_capacity=121, kernel_size=5,
                          pooling=pooling, layer_idx=1)
        with warnings.catch_warnings():
            warnings.simplefilter("error")
            ko, vo = cluster.update_kv(k.to(dtype), q.to(dtype), v.to(dtype), scale_ind)
        assert ko.shape == (B, H, cap, D)
        window = cluster._select_window_indices(Lq, key_len - Lq, "cpu", B, H, key_len)[0, 0]
        # the indices the reference gathered: every key row is distinct, so rows identify them
        idx = torch.empty(B, H, cap, dtype=torch.int64)
        for b in range(B):
            for h in range(H):
                rows = {tuple(r.tolist()): j for j, r in enumerate(k[b, h].to(dtype).float())}
                idx[b, h] = torch.tensor([rows[tuple(r.tolist())] for r in ko[b, h].float()])
                assert torch.equal(vo[b, h].float(), v[b, h].to(dtype).float()[idx[b, h]])
        out[f"s{scale_ind}_q"], out[f"s{scale_ind}_k"], out[f"s{scale_ind}_v"] = q, k, v
        out[f"{name}_window"], out[f"{name}_idx"] = window, idx
        out[f"{name}_meta"] = torch.tensor([scale_ind, cap, int(pooling == "avgpool"), int(dtype == torch.bfloat16)])
    return out


def make_prologue(ref: Path) -> dict:
    """F.normalize + the reference's own precompute_rope2d_freqs_grid / apply_rotary_emb
    (models/infinity/basic_infinity.py:42-133, compiled out of the file: the module imports flash-attn)."""
    import torch.nn.functional as F
    src = (ref / "models/infinity/basic_infinity.py").read_text()
    fns = [n for n in ast.parse(src).body
           if isinstance(n, ast.FunctionDef) and n.name in ("precompute_rope2d_freqs_grid", "apply_rotary_emb")]
    assert len(fns) == 2
    ns = {"torch": torch, "np": np, "F": F}
    exec(compile(ast.Module(body=fns, type_ignores=[]), "basic_infinity.rope", "exec"), ns)
    out = {}
    sched = [(1, s, s) for s in SCALES]
    for name, c, scale_ind in (("a", 64, 3), ("b", 128, 5)):
        grid = ns["precompute_rope2d_freqs_grid"](dim=c, dynamic_resolution_h_w={1.0: {"1M": {"scales": sched}}},
                                                  rope2d_normalized_by_hw=2, pad_to_multiplier=1)
        gen = torch.Generator().manual_seed(50 + c)
        B, H, L = 2, 3, SCALES[scale_ind] ** 2
        qkv = _bf16_exact(B, L, 3, H, c, gen=gen)
        scale_mul = torch.rand(H, generator=gen) * 8 + 1
        q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3).bfloat16() for i in range(3))
        # as SelfAttention.forward under autocast: the norm is taken in fp32, so q and k become fp32
        qn = F.normalize(q.float(), dim=-1, eps=1e-12).mul(scale_mul.view(1, H, 1, 1)).contiguous()
        kn = F.normalize(k.float(), dim=-1, eps=1e-12).contiguous()
        qr, kr = ns["apply_rotary_emb"](qn, kn, sched, grid, 1, 2, scale_ind)
        table = grid[str(tuple(sched))]
        out[f"{name}_qkv"] = qkv.reshape(B, L, 3 * H * c)
        out[f"{name}_scale_mul"] = scale_mul
        out[f"{name}_q_out"], out[f"{name}_k_out"] = qr.bfloat16().float(), kr.bfloat16().float()
        used = sum(x * x for x in SCALES[:scale_ind + 1])
        # the table rows this case uses, and the last 64 rows of the table (64 x 64 map) to pin the builder
        out[f"{name}_cos"], out[f"{name}_sin"] = table[0, 0, 0, 0, :used], table[1, 0, 0, 0, :used]
        out[f"{name}_cos_tail"], out[f"{name}_sin_tail"] = table[0, 0, 0, 0, -64:], table[1, 0, 0, 0, -64:]
        out[f"{name}_meta"] = torch.tensor([B, L, H, c, scale_ind])
    return out


def main() -> None:
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/Lvar")
    ref = Path(sys.argv[1])
    _install_stubs(ref)
    ref_ops = importlib.import_module("kernels.sparse_attn.sparse_attn_ops")
    ref_colsum = importlib.import_module("kernels.sparse_attn.triton.attn_dense_colsum")
    ref_csp = importlib.import_module("kernels.sparse_attn.triton.attn_csp")
    sa = importlib.import_module("models.sparvar.sparse_attn")
    groups = {
        "attention_ref.npz": make_attention(ref_ops, ref_colsum, ref_csp),
        "indices_ref.npz": make_indices(sa),
        "csla_ref.npz": make_csla(ref),
        "scalekv_ref.npz": make_scalekv(ref),
        "prologue_ref.npz": make_prologue(ref),
    }
    for name, d in groups.items():
        arrays = {}
        for k, v in d.items():
            a = v.numpy() if isinstance(v, torch.Tensor) else np.asarray(v)
            if a.dtype == np.float64:
                a = a.astype(np.float32)
            if k.endswith(("_q", "_k", "_v", "_qkv", "_q_out", "_k_out")) and a.dtype == np.float32:
                # inputs are bf16-exact: keep the upper 16 bits only (the tests widen them back)
                a = (a.view(np.uint32) >> 16).astype(np.uint16)
            if a.dtype == np.int64 and a.size > 64 and np.abs(a).max() < 2**31:
                a = a.astype(np.int32)
            arrays[k] = a
        np.savez_compressed(HERE / name, **arrays)
        print(name, {k: a.shape for k, a in arrays.items()}, os.path.getsize(HERE / name), "bytes")


if __name__ == "__main__":
    main()
