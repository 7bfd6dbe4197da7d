"""Global configuration of the sparse-attention path, drop-in for the reference's
``kernels/sparse_attn/sparse_attn_config.py``: the same module-level ``GLOBAL_CONFIG`` dictionary
(same keys and defaults, YAML-overridable through ``load_from_file``) and the same helper names.

One thing differs on purpose: there is a single backend.  ``attn.provider`` is still read from YAML
files written for the reference ('triton' or 'cuda'; 'b200' is accepted too) but it only gets
validated; every value runs the sm_100a kernels of this package, and ``get_kernel_config_attn()``
publishes THEIR tile geometry (callers such as the reference's SparseDiffAttn read it at run time,
models/sparvar/sparse_attn.py:888-891,974-979).
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
    _check_provider()
    from ._lib import kernel_config_attn  # loads the CUDA library; raises if it is missing
    return kernel_config_attn()


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
