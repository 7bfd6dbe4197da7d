"""Global configuration of the sparse-attention path, drop-in for the reference's
``kernels/sparse_attn/sparse_attn_config.py``: the same module-level ``GLOBAL_CONFIG`` dictionary
(same keys and defaults, YAML-overridable through ``load_from_file``) and the same helper names.

One thing differs on purpose: there is a single backend.  ``attn.provider`` is still read from YAML
files written for the reference ('triton' or 'cuda'; 'b200' is accepted too) but it only gets
validated; every value runs the sm_100a kernels of this package, and ``get_kernel_config_attn()``
publishes THEIR tile geometry (callers such as the reference's SparseDiffAttn read it at run time,
models/sparvar/sparse_attn.py:888-891,974-979).  The default geometry (256-row query groups, counts in
multiples of 128) selects keys for different row groups than the reference's 192-row groups; set
``GLOBAL_CONFIG['attn']['geometry'] = 'reference'`` to get the reference's groups and list lengths.
"""
from __future__ import annotations

import copy
from typing import Any, Dict

import yaml

_PROVIDERS = ("triton", "cuda", "b200")

_MLP = dict(is_enabled=True, is_fp8=False, top_keys=0.3, random_keys=0.05, full_step_every=10,
            block_mask_cache=2, first_n_dense_layers=2, provider="triton")
_PATCHIFY = dict(is_enabled=True, chunk_size_1=8, chunk_size_2=4)
_ATTN = dict(
    is_enabled=True,
    decision_scale=10, speedup=1, top_keys=0.05,            # CS4A: column-sum -> top-k at one scale
    attn_sink=5, win_size=[-1] * 8 + [1, 1, 3, 5, 7],        # CSLA: sink scales + per-scale window
    random_keys=0.01, local_voxels=0, local_1d_window=0,
    first_n_dense_layers=2, full_step_every=10, full_step_schedule=None,
    recompute_mask=True, should_compress_indices=True, should_keep_tail_dense=False,
    provider="triton",
    # CS4A / CSLA split and local-prior windows of models/sparvar/sparse-attn-config.yml
    bound_layer=10, cs4a_ws=[1] * 11 + [7, 9],
    # Tile geometry published by get_kernel_config_attn(): None = this library's own (256-row groups, counts in
    # multiples of 128), "reference" = the geometry the reference publishes for the configured provider
    # (192-row groups; counts in multiples of 64 for 'triton', 112 for 'cuda'), or a dict with the three keys.
    geometry=None,
)
_OFFLOADING = {
    "global_disable_offloading": False,
    "mlp.out_cache": False, "mlp.indices": False, "mlp.counts": False, "mlp.sparse_act_T": False,
    "mlp.blockmean_mid_cache": False,
    "attn.out_cache": True, "attn.indices": True, "attn.counts": False, "attn.lse_constants": False,
    "text_encoders": True,
}
_STEP_CACHING = dict(
    is_enabled=False,
    skip_step_schedule={7, 11, 13, 14, 15, 17, 18, 19, 21, 22, 23, 25, 26, 27, 29, 31, 33, 34, 35, 37, 38, 39,
                        41, 42, 43},
)

BASE_CONFIG: Dict[str, Any] = {
    "num_model_invocations_per_inference_step": 1,
    "should_profile": False,
    "generation_index": 0,
    "steps": 13,
    "world_size": 1,
    "mlp": _MLP,
    "patchify": _PATCHIFY,
    "attn": _ATTN,
    "offloading": _OFFLOADING,
    "step_caching": _STEP_CACHING,
}

GLOBAL_CONFIG: Dict[str, Any] = copy.deepcopy(BASE_CONFIG)


def _check_provider() -> str:
    provider = GLOBAL_CONFIG["attn"]["provider"]
    if provider not in _PROVIDERS:
        raise ValueError(f"Invalid provider: {provider}")
    return provider


def get_kernel_config_mlp() -> Dict[str, int]:
    """Sparse-MLP geometry of the reference (sparse_attn_config.py:74-80); the MLP kernels themselves
    are outside this package."""
    return {"bm": 128, "mbm": 128, "counts_multiple_of": 256}


def get_kernel_config_attn() -> Dict[str, int]:
    """Geometry of the attention kernels: ``bm`` query rows share one KV index list (and one colsum
    row), index counts are built as multiples of ``counts_multiple_of`` and index rows are padded to
    ``indices_pad_to`` entries.  Same keys as the reference (sparse_attn_config.py:82-98)."""
    provider = _check_provider()
    from ._lib import kernel_config_attn  # loads the CUDA library; raises if it is missing
    geo = kernel_config_attn()
    override = GLOBAL_CONFIG["attn"].get("geometry")
    if override is None or override == "b200":
        return geo
    if override == "reference":
        # kernels/sparse_attn/sparse_attn_config.py:82-98
        override = ({"bm": 192, "counts_multiple_of": 112, "indices_pad_to": 4} if provider == "cuda"
                    else {"bm": 192, "counts_multiple_of": 64, "indices_pad_to": 1})
    if not isinstance(override, dict) or set(override) - set(geo):
        raise ValueError(f"attn.geometry must be None, 'b200', 'reference' or a dict with keys {sorted(geo)}")
    geo.update({k: int(v) for k, v in override.items()})
    if geo["bm"] < 32 or geo["bm"] % 32 or geo["counts_multiple_of"] < 1 or geo["indices_pad_to"] < 1:
        raise ValueError(f"unsupported attention geometry {geo}: bm must be a positive multiple of 32")
    return geo


def update_global_config(config: Dict[str, Any]) -> None:
    """Shallow update of the top-level keys (sparse_attn_config.py:102-107)."""
    GLOBAL_CONFIG.update(config)


def _deep_update(dst: Dict[str, Any], src: Dict[str, Any]) -> None:
    for key, val in src.items():
        if isinstance(val, dict) and isinstance(dst.get(key), dict):
            _deep_update(dst[key], val)
        else:
            dst[key] = val


def load_from_file(config_file: str) -> None:
    """Deep-merge a YAML file into ``GLOBAL_CONFIG`` (sparse_attn_config.py:121-131)."""
    with open(config_file, "r") as f:
        loaded = yaml.safe_load(f)
    if loaded:
        _deep_update(GLOBAL_CONFIG, loaded)
        _check_provider()
        print(f"lvar_b200: using config file {config_file}")
        print(yaml.dump(loaded, sort_keys=False, allow_unicode=True, default_flow_style=False))
