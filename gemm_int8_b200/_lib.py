"""ctypes binding of the C ABI declared in include/gemm_int8_b200.h.

The library is looked up next to this file, like the reference looks up gemm_int8_CUDA*.so next to its
package (gemm_int8/__init__.py:5-13), and its absence is an ImportError: there is no fallback path.
"""
from __future__ import annotations

import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libgemm_int8_b200.so")

STATUS_NAMES = {
    0: "GI8_OK",
    1: "GI8_ERR_INVALID_ARGUMENT",
    2: "GI8_ERR_UNSUPPORTED_SHAPE",
    3: "GI8_ERR_MISALIGNED",
    4: "GI8_ERR_CUDA",
    5: "GI8_ERR_UNSUPPORTED_DEVICE",
    6: "GI8_ERR_WORKSPACE",
    7: "GI8_ERR_DEVICE_TIMEOUT",
}

# Every symbol include/gemm_int8_b200.h declares: name -> (restype, argtypes)
_i64, _p, _f, _i = ctypes.c_int64, ctypes.c_void_p, ctypes.c_float, ctypes.c_int
SYMBOLS = {
    "gi8_version": (_i, []),
    "gi8_last_error": (ctypes.c_char_p, []),
    "gi8_matmul": (_i, [_p, _p, _p, _i64, _i64, _i64, _f, _p]),
    "gi8_matmul_i32": (_i, [_p, _p, _p, _i64, _i64, _i64, _p]),
    "gi8_matmul_scaled": (_i, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _p, _i64, _p]),
    "gi8_matmul_scaled_workspace_bytes": (_i64, [_i64, _i64, _i64]),
    "gi8_matmul_scaled_static": (_i, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _p]),
    "gi8_matmul_blockwise": (_i, [_p, _p, _p, _i64, _p, _i64, _p, _i64, _i64, _i64, _p]),
    "gi8_matmul_blockwise_f32": (_i, [_p, _p, _p, _i64, _p, _i64, _p, _i64, _i64, _i64, _p]),
    "gi8_matmul_blockwise_f32_scatter": (_i, [_p, _p, _p, _i64, _p, _i64, _p, _i, _i, _i64, _i64, _i64, _p]),
    "gi8_sum_parts_bf16": (_i, [_p, _i, _i64, _p, _i64, _p]),
    "gi8_matmul_blockwise_allgather": (_i, [_p, _p, _p, _i64, _p, _i64, _p, _i, _i64, _i64, _i64, _i64, _i64, _p]),
    "gi8_peer_alloc": (_i, [_p, _i64]),
    "gi8_peer_free": (_i, [_p]),
    "gi8_peer_export": (_i, [_p, _p]),
    "gi8_peer_import": (_i, [_p, _p]),
    "gi8_peer_release": (_i, [_p]),
    "gi8_quantize_token_block": (_i, [_p, _i, _p, _p, _i64, _i64, _p]),
    "gi8_quantize_token": (_i, [_p, _i, _p, _p, _i64, _i64, _p]),
    "gi8_hadamard_quantize_token_block": (_i, [_p, _i, _p, _p, _i64, _i64, _i64, _p]),
    "gi8_force_variant": (_i, [ctypes.c_char_p]),
    "gi8_pick_variant": (ctypes.c_char_p, [_i, _i64, _i64, _i64]),
    "gi8_device_status": (_i, [ctypes.POINTER(ctypes.c_uint32)]),
    "gi8_device_check": (_i, []),
    "gi8_selftest_wait_timeout": (_i, [_p]),
    "gi8_reload_env": (_i, []),
}


def load(path: str = LIB_PATH) -> ctypes.CDLL:
    if not os.path.exists(path):
        raise ImportError(
            f"Could not find the compiled CUDA library {path}; build it with "
            "`python gemm_int8_b200/_build.py` (needs nvcc). There is no CPU fallback."
        )
    lib = ctypes.CDLL(path)
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export a declared symbol
        fn.restype = res
        fn.argtypes = args
    return lib


class GemmInt8Error(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, status: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")
        self.status = status


def check(lib: ctypes.CDLL, status: int) -> None:
    if status != 0:
        msg = lib.gi8_last_error().decode("utf-8", "replace")
        raise GemmInt8Error(status, msg)
