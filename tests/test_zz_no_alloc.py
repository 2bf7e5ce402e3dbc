"""The allocation-free column quantizer (i8l_quant_col_t_static), called straight through the C ABI.

Some callers cannot give the library scratch memory because they may not allocate on the device at
that point (a memory-pool callback, a sandboxed plugin, a capture section).  For them the library
carries a fixed 65536-float scratch array of its own.  This test checks that the entry point gives
bit-identical output to the regular i8l_quant_col_t on two calls in a row whose inputs differ, so
stale scratch contents from the first call would be caught, and that oversized requests are refused.
It lives in its own file, collected last, so a failure here cannot hide any other test's result.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, name, x, scratch=None):
    rows, cols = x.shape
    qt = torch.empty((cols, rows), dtype=torch.int8, device=x.device)
    st = torch.empty((cols,), dtype=torch.float32, device=x.device)
    stream = torch.cuda.current_stream().cuda_stream
    if scratch is None:
        rc = lib.i8l_quant_col_t_static(x.data_ptr(), rows, cols, 0, qt.data_ptr(), st.data_ptr(), stream)
    else:
        rc = lib.i8l_quant_col_t(x.data_ptr(), rows, cols, 0, qt.data_ptr(), st.data_ptr(), scratch.data_ptr(), stream)
    assert rc == 0, lib.i8l_last_error().decode()
    return qt, st


def test_static_scratch_variant_matches_regular_entry_point_twice():
    from triton_int8_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(77)
    big = (torch.randn(512, 1280, device=dev, generator=g) * 3.0).to(torch.bfloat16)
    small = (torch.randn(256, 1280, device=dev, generator=g) * 0.01).to(torch.bfloat16)  # smaller maxima than `big`
    scratch = torch.empty(1280, dtype=torch.float32, device=dev)
    for x in (big, small):          # two calls in a row on the shared built-in scratch
        q_ref, s_ref = _call(lib, "regular", x, scratch)
        q, s = _call(lib, "static", x)
        torch.cuda.synchronize()
        assert torch.equal(q, q_ref), "int8 output differs from i8l_quant_col_t"
        assert torch.equal(s, s_ref), "scales differ from i8l_quant_col_t (bit-exact expected)"


def test_static_scratch_variant_at_the_size_limit_and_against_the_oracle():
    """cols == 65536, the largest the built-in scratch admits, and the values themselves against the CPU
    restatement of the per-channel quantizer applied to x^T (not only against the sibling entry point)."""
    from oracle import ref_semantics as R
    from triton_int8_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(78)
    x = (torch.randn(128, 65536, device=dev, generator=g) * 2.0).to(torch.bfloat16)
    x[5, 40000] = 77.0
    q, s = _call(lib, "static", x)
    torch.cuda.synchronize()
    q_ref, s_ref = R.quant_token(x.cpu().t().contiguous())
    assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu(), s_ref.view(-1))


def test_static_scratch_variant_rejects_oversize():
    from triton_int8_b200 import _lib
    lib = _lib.load()
    x = torch.zeros(128, 128, dtype=torch.bfloat16, device="cuda:0")
    rc = lib.i8l_quant_col_t_static(x.data_ptr(), 128, 65536 + 128, 0, x.data_ptr(), x.data_ptr(), None)
    assert rc == -1 and b"exceeds the built-in scratch" in lib.i8l_last_error()
