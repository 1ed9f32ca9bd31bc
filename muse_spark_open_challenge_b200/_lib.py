"""ctypes binding of libmsl.so (C ABI declared in include/msl.h).

There is no fallback: if the library is missing or a symbol is absent, importing raises, and every
wrapper raises `MslError` on a non-zero status.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libmsl.so")

OUT_BF16, OUT_F32, OUT_SWIGLU_BF16 = 0, 1, 2
ERR_DEVICE_TIMEOUT, ERR_CAPACITY = -5, -6
OPTIONS = {"gemm_splitk": 0, "gemm_wide": 1, "grouped_wide": 2}     # MSL_OPT_* of include/msl.h
ABI_VERSION = 2

_p, _i, _i64, _f = C.c_void_p, C.c_int, C.c_int64, C.c_float

# name -> (restype, argtypes), in the order of include/msl.h
SIGNATURES = {
    "msl_abi_version": (_i, []),
    "msl_status_string": (C.c_char_p, [_i]),
    "msl_set_option": (_i, [_i, _i]),
    "msl_get_option": (_i, [_i]),
    "msl_gemm_bf16": (_i, [_p, _i64, _p, _i64, _p, _i64, _i, _i, _i, _i, _i, _i, _i, _f, _p, _p]),
    "msl_gemm_splitk_plan": (_i, [_i, _i, _i, _i, _i]),
    "msl_gemm_bf16_splitk": (_i, [_p, _i64, _p, _i64, _p, _i64, _i, _i, _i, _i, _i, _i, _i, _f, _i, _p, _p, _p]),
    "msl_qk_rope_store": (_i, [_p, _i64, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i64, _p, _p]),
    "msl_boundary": (_i, [_p, _i64, _p, _p, _p, _p, _p, _p, _p, _i64, _i, _i, _f, _f, _p]),
    "msl_route_topk": (_i, [_p, _i64, _i, _p, _f, _p, _i, _i, _i, _i, _p, _p, _p, _p, _p, _p]),
    "msl_dispatch": (_i, [_p, _i64, _p, _p, _p, _p, _i, _i, _i, _i, _p, _i64, _p, _p, _p, _p]),
    "msl_route_dispatch": (_i, [_p, _i64, _i, _p, _f, _p, _p, _i64, _p, _i, _i, _i, _i, _i, _p, _p, _p, _p, _p, _p, _p,
                                _i64, _p, _p, _p, _p]),
    "msl_route_dispatch_static": (_i, [_p, _i64, _i, _p, _f, _p, _p, _i64, _p, _i, _i, _i, _i, _i, _p, _p, _p, _i64,
                                       _p, _p, _p, _p]),
    "msl_combine": (_i, [_p, _p, _p, _p, _p, _i64, _p, _i64, _i, _i, _i, _p, _p]),
    "msl_combine_boundary": (_i, [_p, _p, _p, _p, _p, _i64, _i, _i, _i, _p, _p, _p, _p, _p, _p, _p, _i64, _f, _f, _p,
                                  _p]),
    "msl_ep_plan": (_i, [_p, _i, _i, _i, _i, _p, _p, _p, _p]),
    "msl_peer_barrier": (_i, [_p, _i, _i, _i, _p, _p]),
    "msl_dispatch_peer": (_i, [_p, _i64, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _p, _p]),
    "msl_combine_peer": (_i, [_p, _i, _p, _p, _p, _p, _i64, _p, _i64, _i, _i, _i, _p]),
    "msl_kv_rows_copy": (_i, [_p, _p, _i64, _p, _p, _i64, _i64, _i, _p, _p]),
    "msl_nvfp4_padded_rows": (_i64, [_i, _i]),
    "msl_nvfp4_repack": (_i, [_p, _p, _p, _p, _i, _i, _i, _i, _p]),
    "msl_grouped_gemm_nvfp4": (_i, [_p, _i64, _p, _p, _p, _p, _p, _i64, _i, _i, _i, _i, _i, _i, _p, _p]),
    "msl_nvfp4_bs_tiles": (_i, [_i, _i]),
    "msl_nvfp4_bs_row_tiles": (_i64, [_i64, _i]),
    "msl_nvfp4_bs_sf_repack": (_i, [_p, _p, _i, _i, _i, _i, _p]),
    "msl_nvfp4_bs_quantize": (_i, [_p, _i64, _i64, _i, _p, _i, _p, _p, _p, _p]),
    "msl_grouped_gemm_nvfp4_bs": (_i, [_p, _p, _p, _i64, _p, _p, _p, _p, _p, _i64, _i, _i, _i, _i, _i, _i, _p, _p]),
    "msl_mma_peak": (_i, [_i, _i, _i, _p, _p]),
    "msl_unit_peak": (_i, [_i, _i, _i, _p, _p]),
    "msl_layer_prepared_bytes": (_i64, [_p]),
    "msl_layer_workspace_bytes": (_i64, [_p]),
    "msl_layer_prepare": (_i, [_p, _p, _p, _i64, _p, _p]),
    "msl_layer_prefill": (_i, [_p, _p, _p, _p, _p, _i64, _p, _p]),
    "msl_attention_fp8": (_i, [_p, _p, _p, _p, _i, _p, _p, _p, _p, _f, _i, _i, _i, _i, _i, _i, _i, _i, _i64, _p,
                               _i64, _p, _i64, _p, _p]),
    "msl_attention_split_plan": (_i, [_i, _i, _i, _i, _i, _i, _i]),
    "msl_attention_split_workspace": (_i64, [_i, _i, _i, _i]),
    "msl_attention_fp8_split": (_i, [_p, _p, _p, _p, _i, _p, _p, _p, _p, _f, _i, _i, _i, _i, _i, _i, _i, _i, _i64, _p,
                                     _i64, _p, _i64, _i, _p, _p, _p]),
}


class MslError(RuntimeError):
    pass


def load(path: str = LIB_PATH) -> C.CDLL:
    if not os.path.exists(path):
        raise MslError(f"{path} is missing: build it with `python -m muse_spark_open_challenge_b200.build` "
                       "(there is no non-CUDA fallback)")
    lib = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError if the symbol is not exported
        fn.restype, fn.argtypes = res, args
    return lib


_LIB = None


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        _LIB = load()
    return _LIB


def set_option(name: str, value: bool) -> bool:
    """Set a run-time option of the library (see MSL_OPT_* in include/msl.h); returns the old value."""
    old = bool(lib().msl_get_option(OPTIONS[name]))
    if lib().msl_set_option(OPTIONS[name], int(bool(value))) != 0:
        raise MslError(f"msl_set_option({name}) was rejected")
    return old


LAUNCHES = 0     # kernels of this library launched by this process (each successful entry point = one launch)


def check(rc: int, what: str) -> None:
    global LAUNCHES
    LAUNCHES += 1
    if rc != 0:
        raise MslError(f"{what}: {lib().msl_status_string(rc).decode()} ({rc})")
