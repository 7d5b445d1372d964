"""ctypes binding of ``libmxk.so`` (the C-ABI declared in ``include/mxk.h``).

There is no CPU or PyTorch fallback: if the shared library is missing the
import of this module raises, and every wrapper raises on a non-zero status.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("MXK_LIBRARY") or os.path.join(_HERE, "libmxk.so")

_p = ctypes.c_void_p
_i = ctypes.c_int
_z = ctypes.c_size_t
_f = ctypes.c_float

# name -> (restype, argtypes); mirrors include/mxk.h one to one.
SIGNATURES = {
    "mxk_status_string": (ctypes.c_char_p, [_i]),
    "mxk_abi_version": (_i, []),
    "mxk_selftest_bounded_wait": (_i, [_p, _i, _p]),
    "mxk_linrec_f32_fwd": (_i, [_p, _i, _p, _p, _p, _p, _p, _p, _i, _i, _i, _p]),
    "mxk_linrec_c64_fwd": (_i, [_p, _i, _p, _p, _p, _p, _p, _p, _i, _i, _i, _p]),
    "mxk_linrec_bwd_workspace_bytes": (_z, [_i, _i, _i, _i, _i]),
    "mxk_linrec_f32_bwd": (_i, [_p, _i, _p, _p, _p, _p, _p, _p, _p, _p, _p, _z, _i, _i, _i, _p]),
    "mxk_linrec_c64_bwd": (_i, [_p, _i, _p, _p, _p, _p, _p, _p, _p, _p, _p, _z, _i, _i, _i, _i, _p]),
    "mxk_linrec_grouped_bwd_workspace_bytes": (_z, [_i, _i, _i, _i]),
    "mxk_linrec_f32_last": (_i, [_p, _i] + [_p] * 4 + [_i, _i, _i, _p]),
    "mxk_linrec_c64_last": (_i, [_p, _i] + [_p] * 4 + [_i, _i, _i, _p]),
    "mxk_linrec_f32_grouped_last": (_i, [_p] * 5 + [_i, _i, _i, _i, _p]),
    "mxk_linrec_f32_grouped_fwd": (_i, [_p] * 7 + [_i, _i, _i, _i, _p]),
    "mxk_linrec_f32_grouped_bwd": (_i, [_p] * 10 + [_z, _i, _i, _i, _i, _p]),
    "mxk_linrec_noalloc_max_elements": (_z, []),
    "mxk_linrec_c64_bwd_noalloc": (_i, [_p] * 9 + [_i, _i, _i, _i, _p]),
    "mxk_loglinrec_f32_fwd": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _p]),
    "mxk_loglinrec_f32_bwd": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _p]),
    "mxk_mingru_f32_fwd": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _p]),
    "mxk_mingru_f32_bwd": (_i, [_p] * 11 + [_i, _i, _i, _p]),
    "mxk_linattn_chunk_states_bytes": (_z, [_i, _i, _i, _i]),
    "mxk_linattn_bf16_fwd": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _f, _i, _p]),
    "mxk_linattn_bf16_bwd": (_i, [_p] * 14 + [_i, _i, _i, _i, _f, _i, _p]),
    "mxk_mlstm_bwd_workspace_bytes": (_z, [_i, _i, _i, _i]),
    "mxk_mlstm_f32_fwd": (_i, [_p] * 15 + [_i, _i, _i, _i, _f, _p]),
    "mxk_mlstm_f32_bwd": (_i, [_p] * 22 + [_z, _i, _i, _i, _i, _f, _p]),
    "mxk_gdelta_chunk_states_bytes": (_z, [_i, _i, _i, _i]),
    "mxk_gdelta_workspace_bytes": (_z, [_i, _i, _i, _i]),
    "mxk_gdelta_bf16_fwd": (_i, [_p] * 11 + [_z, _p, _i, _i, _i, _i, _p]),
    "mxk_gdelta_bf16_bwd": (_i, [_p] * 17 + [_i, _i, _i, _i, _p]),
    "mxk_norm_bwd_workspace_bytes": (_z, [ctypes.c_longlong, _i]),
    "mxk_norm_bf16_fwd": (_i, [_p, _p, _p, _p, _p, _p, ctypes.c_longlong, _i, _f, _i, _p]),
    "mxk_norm_bf16_bwd": (_i, [_p] * 9 + [_z, ctypes.c_longlong, _i, _i, _p]),
    "mxk_gated_residual_bf16_fwd": (_i, [_p, _p, _p, _p, ctypes.c_longlong, _p]),
    "mxk_gated_residual_bf16_bwd": (_i, [_p, _p, _p, _p, _p, ctypes.c_longlong, _p]),
    "mxk_l2norm_heads_bf16": (_i, [_p, _p, _p, ctypes.c_longlong, _i, _f, _p]),
    "mxk_mlstm_bf16_chunk_states_bytes": (_z, [_i, _i, _i, _i]),
    "mxk_mlstm_bf16_fwd": (_i, [_p] * 18 + [_i, _i, _i, _i, _f, _p]),
    "mxk_mlstm_bf16_bwd": (_i, [_p] * 26 + [_i, _i, _i, _i, _f, _p]),
    "mxk_gelu_bf16": (_i, [_p, _p, _p, ctypes.c_longlong, _p]),
    "mxk_colsum_workspace_bytes": (_z, [ctypes.c_longlong, _i]),
    "mxk_colsum_bf16": (_i, [_p, _p, _p, _z, ctypes.c_longlong, _i, _p]),
    "mxk_adam_bf16": (_i, [_p, _p, _p, _p, ctypes.c_longlong, _f, _f, _f, _f, _i, _f, _p]),
    "mxk_adam_bf16_master": (_i, [_p, _p, _p, _p, _p, ctypes.c_longlong, _f, _f, _f, _f, _i, _f, _p]),
}


class MxkError(RuntimeError):
    def __init__(self, fn, status, text):
        super().__init__(f"{fn} failed with status {status}: {text}")
        self.status = status


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m memorax_b200.build` "
            "(nvcc, sm_100a). memorax_b200 has no fallback path.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def status_string(status: int) -> str:
    return lib.mxk_status_string(int(status)).decode()


def check(fn_name: str, status: int) -> None:
    if status != 0:
        raise MxkError(fn_name, status, status_string(status))


def call(fn_name: str, *args) -> None:
    """Invoke a status-returning entry point and raise MxkError on failure."""
    check(fn_name, getattr(lib, fn_name)(*args))
