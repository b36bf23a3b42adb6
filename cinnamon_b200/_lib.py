"""ctypes binding of libcinnamon_b200.so (the C ABI in include/cinnamon_b200.h).

There is no fallback: if the library is missing or a symbol is absent the
import raises, and every call checks the status code the library returns.
"""
from __future__ import annotations

import ctypes
import os

from .build import LIB_PATH as _DEFAULT_LIB_PATH

OK, ERR_INVALID, ERR_CUDA, ERR_UNSUPPORTED, ERR_DEVICE = 0, 1, 2, 3, 4
BF16, F32, F16, F32_BF16 = 0, 1, 2, 3
DIV_FULL, DIV_RN = 0, 1
B_NK, B_KN = 0, 1

_vp, _i64, _i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int

# name -> argument types; the list mirrors include/cinnamon_b200.h one to one
SIGNATURES = {
    "cinn_version": [],
    "cinn_last_error": [],
    "cinn_quant_rowwise": [_vp, _i32, _i64, _i64, _i64, _i64, _vp, _vp, _i32, _i32, _i32, _vp],
    "cinn_quant_rowwise_dual": [_vp, _i32, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _i32, _i32, _vp],
    "cinn_selfcheck_division": [_vp, _vp],
    "cinn_quant_rowwise_with_block": [_vp, _i32, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _i32, _i32, _vp],
    "cinn_quant_rowwise_with_block_t": [_vp, _i32, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _i32, _i32, _vp],
    "cinn_set_wait_limit_cycles": [ctypes.c_longlong],
    "cinn_quant_blockwise_t": [_vp, _i32, _i64, _i64, _i64, _vp, _vp, _vp, _i32, _i32, _vp],
    "cinn_quant_blockwise": [_vp, _i32, _i64, _i64, _i64, _i64, _vp, _vp, _i32, _i32, _i32, _i32, _vp],
    "cinn_requant_row_to_block": [_vp, _vp, _i64, _i64, _vp, _vp, _i32, _i32, _vp],
    "cinn_dequant": [_vp, _vp, _vp, _i32, _i64, _i64, _i32, _i32, _vp],
    "cinn_swiglu_quant_rowwise": [_vp, _i32, _i64, _i64, _vp, _vp, _i32, _vp],
    "cinn_swiglu_quant_rowwise_n": [_vp, _i32, _i64, _i64, _vp, _vp, _vp, _i32, _vp],
    "cinn_transpose_bytes": [_vp, _i64, _vp, _i64, _i64, _vp],
    "cinn_fp8_gemm": [_vp, _vp, _i64, _vp, _vp, _i64, _i64, _vp, _i64, _i64, _i64, _i32, _i32, _vp],
    "cinn_grouped_gemm_16bit": [_vp, _vp, _i32, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _i32, _vp],
    "cinn_fp8_grouped_gemm_dgrad": [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _i32, _vp],
    "cinn_moe_combine": [_vp, _i32, _vp, _vp, _vp, _i64, _i64, _i32, _i64, _vp],
    "cinn_zero_rows_outside": [_vp, _i64, _i64, _vp, _vp, _i64, _vp],
    "cinn_moe_combine_backward": [_vp, _i32, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i32, _i64, _vp],
    "cinn_moe_route_workspace_ints": [_i64, _i32],
    "cinn_moe_route": [_vp, _vp, _i64, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "cinn_moe_route_static_max_ints": [],
    "cinn_moe_route_static": [_vp, _vp, _i64, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "cinn_gather_rows": [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp],
    "cinn_sparse_attn_fwd": [_vp, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, ctypes.c_float, _vp],
    "cinn_sparse_attn_bwd": [_vp, _i32, _vp, _vp, _vp, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64,
                             ctypes.c_float, _vp],
    "cinn_lightning_indexer": [_vp, _vp, _vp, _i32, _vp, _i64, _i64, _i64, _i64, _i64, _vp, _vp, _vp, _vp],
    "cinn_scatter_rows": [_vp, _vp, _vp, _i64, _i64, _i64, _vp],
    "cinn_set_gemm_sm_limit": [_i32],
    "cinn_p2p_dispatch": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i32, _i32, _i64, _vp],
    "cinn_p2p_return": [_vp, _vp, _vp, _vp, _i64, _i64, _i32, _i32, _i64, _vp],
    "cinn_p2p_plan": [_vp, _vp, _vp, _i32, _i32, _i32, _i32, ctypes.c_uint, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "cinn_p2p_dispatch_signal": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i32, _i32, _i64, _vp, _i32, _i32,
                                 ctypes.c_uint, _vp, _i32, _i32, _i32, _vp],
    "cinn_p2p_row_table_wait": [_vp, _vp, _vp, _i64, _i64, _i32, _i32, _i64, _vp, _vp, _i32, _i32, ctypes.c_uint, _vp],
    "cinn_p2p_barrier": [_vp, _i32, _i32, ctypes.c_uint, _vp],
    "cinn_fp8_grouped_gemm_scatter": [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _i32, _vp],
    "cinn_p2p_row_table": [_vp, _vp, _vp, _i64, _i64, _i32, _i32, _i64, _vp, _vp],
    "cinn_fp8_grouped_wgrad_scratch_bytes": [_i64, _i64, _i64],
    "cinn_fp8_grouped_wgrad_fused_scratch_bytes": [_i64, _i64, _i64, _i64],
    "cinn_fp8_grouped_wgrad_fused": [_vp, _i32, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _i64, _vp, _i32, _i32, _vp, _vp, _vp],
    "cinn_fp8_grouped_wgrad": [_vp, _i32, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _i64, _vp, _i32, _i32, _vp],
    "cinn_swiglu": [_vp, _vp, _i32, _i64, _i64, _vp],
    "cinn_swiglu_backward": [_vp, _vp, _vp, _i32, _i64, _i64, _vp],
    "cinn_moe_combine_add": [_vp, _i32, _vp, _vp, _vp, _i32, _vp, _i64, _i64, _i32, _i64, _vp],
    "cinn_device_status": [ctypes.POINTER(ctypes.c_int), _i32],
    "cinn_fp8_grouped_gemm": [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _i32, _vp],
}


class LibraryError(RuntimeError):
    pass


def _load() -> ctypes.CDLL:
    LIB_PATH = os.environ.get("CINN_LIB_PATH") or _DEFAULT_LIB_PATH    # override: an alternative build of the library
    if not os.path.exists(LIB_PATH):
        raise LibraryError(
            f"{LIB_PATH} is missing: build it with `python -m cinnamon_b200.build` "
            "(there is no CPU or PyTorch fallback for these kernels)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)            # AttributeError if the symbol is not exported
        fn.argtypes = argtypes
        fn.restype = (ctypes.c_char_p if name == "cinn_last_error"
                      else ctypes.c_longlong if name == "cinn_set_wait_limit_cycles"
                      else ctypes.c_int64 if name in ("cinn_moe_route_workspace_ints", "cinn_moe_route_static_max_ints",
                                                 "cinn_fp8_grouped_wgrad_scratch_bytes", "cinn_fp8_grouped_wgrad_fused_scratch_bytes")
                      else ctypes.c_int)
    return lib


lib = _load()


def last_error() -> str:
    return (lib.cinn_last_error() or b"").decode("utf-8", "replace")


def check(status: int, what: str) -> None:
    """Turns a status code into the exception the reference would raise:
    invalid arguments are AssertionError (the reference uses `assert`), everything
    else is RuntimeError."""
    if status == OK:
        return
    msg = f"{what}: {last_error()} (status {status})"
    if status == ERR_INVALID:
        raise AssertionError(msg)
    raise LibraryError(msg)
