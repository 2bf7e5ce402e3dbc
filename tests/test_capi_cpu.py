"""CPU-only checks of the boundary: the shared library loads, exports every symbol the header
declares, and argument validation fails with the documented codes before any device work."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from triton_int8_b200 import build, _lib
    build.build()
    return _lib.load()


def test_every_declared_symbol_is_exported(lib):
    hdr = open(os.path.join(ROOT, "include", "i8linear.h")).read()
    declared = set(re.findall(r"I8L_API\s+[\w\s\*]+?\b(i8l_\w+)\s*\(", hdr))
    assert len(declared) >= 8
    for name in declared:
        assert hasattr(lib, name), name
    from triton_int8_b200 import _lib
    assert declared == set(_lib.SIGNATURES) | {"i8l_last_error"}


def test_argument_validation_without_a_gpu(lib):
    buf = ctypes.create_string_buffer(1 << 16)
    p = ctypes.addressof(buf)
    p += (16 - p % 16) % 16
    rc = lib.i8l_quant_tile(p, 1, 100, 128, 0, 0, 0, p, p, None, None, None)
    assert rc == -1 and b"multiples of 128" in lib.i8l_last_error()
    rc = lib.i8l_quant_tile(p + 1, 1, 128, 128, 0, 0, 0, p, p, None, None, None)
    assert rc == -2
    rc = lib.i8l_quant_tile(p, 1, 128, 128, 0, 0, 64, p, p, None, None, None)
    assert rc == -6
    rc = lib.i8l_gemm_block(p, p, p, p, 0, 0, 0, None, 1.0, p, 1, 128, 128, 100, 0, None, None)
    assert rc == -1
    rc = lib.i8l_gemm_block(p, p, None, p, 0, 0, 0, None, 1.0, p, 1, 128, 128, 128, 0, None, None)
    assert rc == -6
    rc = lib.i8l_quant_row(p, 128, 3000, 0, -1, p, p, None)
    assert rc == -1


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_no_cpu_fallback(lib):
    from triton_int8_b200 import I8LError, block_channel
    with pytest.raises(ValueError):
        block_channel.triton_per_block_quant(torch.zeros(1, 128, 128, dtype=torch.bfloat16))
    buf = ctypes.create_string_buffer(1 << 16)
    p = ctypes.addressof(buf); p += (16 - p % 16) % 16
    rc = lib.i8l_quant_tile(p, 1, 128, 128, 0, 0, 0, p, p, None, None, None)
    assert rc in (-3, -4)   # no device / wrong architecture: an error, never a CPU result
