"""ctypes binding of libi8linear.so (the C ABI declared in include/i8linear.h).

The product path has no CPU or eager fallback: if the shared library is missing or a call
returns an error code, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("I8L_LIBRARY_PATH") or os.path.join(_PKG_DIR, "libi8linear.so")

OK = 0
ERR_NAMES = {-1: "SHAPE", -2: "ALIGN", -3: "ARCH", -4: "CUDA", -5: "TIMEOUT", -6: "ARG"}

GRAN_TILE128, GRAN_GROUP128, GRAN_ROW, GRAN_TILE128X256 = 0, 1, 2, 5
QMODE_TRITON, QMODE_RNE, QMODE_FUSED, QMODE_ROWRCP, QMODE_TRITON_BF16S = 0, 1, 2, 3, 4
HAD_NONE, HAD_128, HAD_FULL = 0, 128, -1
ASCALE_TILE, ASCALE_GROUP, ASCALE_TILE256 = 0, 1, 2
BSCALE_CHANNEL, BSCALE_TILE, BSCALE_GROUP = 0, 1, 2
GEMM_EXACT_ORDER, GEMM_DIVIDE, GEMM_OUT_F32, GEMM_PRODUCT_FIRST = 1, 2, 4, 8
MAX_RANKS = 8

_P, _I64, _I, _F = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float

SIGNATURES = {
    "i8l_quant_tile": [_P, _I64, _I64, _I64, _I, _I, _I, _P, _P, _P, _P, _P],
    "i8l_quant_row": [_P, _I64, _I64, _I, _I, _P, _P, _P],
    "i8l_quant_col_t": [_P, _I64, _I64, _I, _P, _P, _P, _P],
    "i8l_quant_col_t_static": [_P, _I64, _I64, _I, _P, _P, _P],
    "i8l_quant_col_t_rot": [_P, _I64, _I64, _I, _P, _P, _P, _P],
    "i8l_gemm_block": [_P, _P, _P, _P, _I, _I, _I, _P, _F, _P, _I64, _I64, _I64, _I64, _I, _P, _P],
    "i8l_gemm_rowcol": [_P, _P, _P, _P, _I, _P, _F, _P, _I64, _I64, _I64, _I64, _I, _P, _P],
    "i8l_fused_gemm": [_P, _P, _P, _I64, _I64, _I64, _I64, _I, _I, _P, _P],
    "i8l_gemm_dump_i32": [_P, _P, _I, _P, _I64, _I64, _I64, _I64, _I, _P, _P],
    "i8l_gemm_block_scatter": [_P, _P, _P, _P, _I, _F, _P, _I, _I, _I64, _I64, _I64, _P, _P],
    "i8l_sum_slots": [_P, _P, _I, _I64, _I64, _P],
    "i8l_set_cta_limit": [_I],
    "i8l_test_set_wait_limit": [ctypes.c_uint32, _I],
    "i8l_version": [],
}


class I8LError(RuntimeError):
    def __init__(self, code: int, text: str):
        super().__init__(f"libi8linear error {ERR_NAMES.get(code, code)}: {text}")
        self.code = code


_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library (once).  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m triton_int8_b200.build` "
                "(there is no fallback implementation)")
        lib = ctypes.CDLL(LIB_PATH)
        for name, argtypes in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = _I
        lib.i8l_last_error.argtypes = []
        lib.i8l_last_error.restype = ctypes.c_char_p
        _lib = lib
    return _lib


def call(name: str, *args) -> None:
    lib = load()
    rc = getattr(lib, name)(*args)
    if rc != OK:
        raise I8LError(rc, lib.i8l_last_error().decode())
