"""ctypes binding of ``liblvar_b200.so`` (the C ABI declared in ``include/lvar_b200.h``).

The library is the only compute path of this package: if it is missing, fails to load or lacks a
symbol, importing this module raises; nothing falls back to PyTorch or to the CPU.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "liblvar_b200.so"

LVAR_OK = 0
DEV_STATUS_NAMES = {
    0: "ok",
    1: "timeout: K/V loader",
    2: "timeout: MMA issuer",
    3: "timeout: softmax warpgroup",
    4: "timeout: drain",
    5: "KV index out of range",
    6: "forced timeout (wait limit 0)",
}
DEFAULT_WAIT_NS = 2_000_000_000
SCHED_PAIRS_ONLY, SCHED_SINGLE_ONE_SLOT, SCHED_SERIALIZE_LAUNCH = 1, 2, 4  # lvar_attn_args.sched_flags


class LvarError(RuntimeError):
    """A C-ABI call returned a non-zero code; the message is ``lvar_last_error()``."""

    def __init__(self, code: int, message: str):
        super().__init__(f"lvar_b200 error {code}: {message}")
        self.code = code


class AttnArgs(C.Structure):
    """Mirror of ``lvar_attn_args``; field order and types must match the header."""

    _fields_ = [
        ("B", C.c_int32), ("H", C.c_int32), ("Lq", C.c_int32), ("Lkv", C.c_int32), ("D", C.c_int32),
        ("scale", C.c_float),
        ("q", C.c_void_p), ("q_sb", C.c_int64), ("q_sh", C.c_int64), ("q_sl", C.c_int64),
        ("k", C.c_void_p), ("k_sb", C.c_int64), ("k_sh", C.c_int64), ("k_sl", C.c_int64),
        ("v", C.c_void_p), ("v_sb", C.c_int64), ("v_sh", C.c_int64), ("v_sl", C.c_int64),
        ("o", C.c_void_p), ("o_sb", C.c_int64), ("o_sh", C.c_int64), ("o_sl", C.c_int64),
        ("M", C.c_void_p), ("L", C.c_void_p),
        ("cs", C.c_void_p), ("cs_sb", C.c_int64), ("cs_sh", C.c_int64), ("cs_st", C.c_int64),
        ("cs_group_tiles", C.c_int32),
        ("block_mask", C.c_void_p), ("bm_sb", C.c_int64), ("bm_sh", C.c_int64), ("bm_sq", C.c_int64),
        ("block_size", C.c_int32),
        ("indices", C.c_void_p), ("i_sb", C.c_int64), ("i_sh", C.c_int64), ("i_sg", C.c_int64),
        ("counts", C.c_void_p), ("c_sb", C.c_int64), ("c_sh", C.c_int64),
        ("group_rows", C.c_int32),
        ("o_in", C.c_void_p), ("oi_sb", C.c_int64), ("oi_sh", C.c_int64), ("oi_sl", C.c_int64),
        ("o_scale", C.c_int32), ("o_in_side", C.c_int32), ("o_side", C.c_int32),
        ("sched_scratch", C.c_void_p), ("work_order", C.c_void_p),
        ("dev_status", C.c_void_p),
        ("wait_limit_ns", C.c_uint64),
        ("sched_flags", C.c_int32),
        ("M_in", C.c_void_p), ("L_in", C.c_void_p),
    ]


# name -> (restype, argtypes); every symbol the header declares is listed here and checked at load.
_SIGNATURES = {
    "lvar_dense_attn": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p]),
    "lvar_dense_colsum_attn": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p]),
    "lvar_dense_colsum_attn_given": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p]),
    "lvar_colsum_tiles": (C.c_int, [C.POINTER(AttnArgs), C.c_int32, C.c_void_p]),
    "lvar_block_sparse_attn": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p]),
    "lvar_csp_attn": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p]),
    "lvar_colsum": (C.c_int, [C.c_void_p] * 5 + [C.c_int32] * 5 + [C.c_int64] * 9 + [C.c_int32, C.c_float,
                                                                                    C.c_void_p, C.c_uint64, C.c_void_p]),
    "lvar_block_scores": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_int64, C.c_void_p]),
    "lvar_build_block_mask": (C.c_int, [C.c_void_p] * 5 + [C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "lvar_block_mask_from_colsums": (C.c_int, [C.c_void_p, C.c_int64] + [C.c_void_p] * 5 +
                                     [C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "lvar_topk_indices": (C.c_int, [C.c_void_p, C.c_int64, C.c_int32, C.c_int64, C.c_int32, C.c_int32, C.c_void_p,
                                    C.c_int64, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p]),
    "lvar_mask_to_indices": (C.c_int, [C.c_void_p] * 3 + [C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "lvar_bitpack": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]),
    "lvar_bitunpack": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]),
    "lvar_dense_colsum_attn_static": (C.c_int, [C.c_void_p] * 5 + [C.c_int32] * 5 + [C.c_int64] * 15 +
                                      [C.c_int32, C.c_float, C.c_void_p, C.c_uint64, C.c_void_p]),
    "lvar_sparse_step_lists": (C.c_int, [C.c_void_p] * 5 + [C.c_int64, C.c_int32, C.c_int32, C.c_int64, C.c_int64] +
                               [C.c_int32] * 6 + [C.c_void_p]),
    "lvar_scalekv_scores": (C.c_int, [C.c_void_p] * 4 + [C.c_int32] * 5 + [C.c_int64] * 6 + [C.c_int32] * 2 + [C.c_void_p]),
    "lvar_scalekv_pool": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_int64, C.c_int32, C.c_int32,
                                    C.c_int32, C.c_void_p]),
    "lvar_gather_rows": (C.c_int, [C.c_void_p] * 3 + [C.c_int32] * 5 + [C.c_int64] * 4 + [C.c_void_p]),
    "lvar_qkv_prologue": (C.c_int, [C.c_void_p] + [C.c_int64] * 4 + [C.c_void_p] * 3 + [C.c_int32] +
                          [C.c_void_p] + [C.c_int64] * 3 + [C.c_void_p] + [C.c_int64] * 3 + [C.c_void_p] + [C.c_int64] * 3 +
                          [C.c_int32] * 5 + [C.c_void_p]),
    "lvar_upsample_ocache": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_int32] +
                             [C.c_int64] * 4 + [C.c_void_p]),
    "lvar_last_error": (C.c_char_p, []),
    "lvar_version": (C.c_char_p, []),
    "lvar_kernel_config_attn": (None, [C.POINTER(C.c_int32)] * 3),
}


def _load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m lvar_b200.build` "
            "(there is no PyTorch or CPU fallback for these kernels)")
    lib = C.CDLL(os.fspath(LIB_PATH))
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name, None)
        if fn is None:
            raise ImportError(f"{LIB_PATH} does not export {name}")
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def exported_symbols() -> list[str]:
    return sorted(_SIGNATURES)


def check(code: int) -> None:
    if code != LVAR_OK:
        raise LvarError(code, lib.lvar_last_error().decode())


def version() -> str:
    return lib.lvar_version().decode()


def kernel_config_attn() -> dict:
    bm, mult, pad = C.c_int32(), C.c_int32(), C.c_int32()
    lib.lvar_kernel_config_attn(C.byref(bm), C.byref(mult), C.byref(pad))
    return {"bm": bm.value, "counts_multiple_of": mult.value, "indices_pad_to": pad.value}
