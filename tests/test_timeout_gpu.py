"""The bounded waits of the GEMM kernels, exercised end to end without a fault, a trap or a hang.

Every wait on an mbarrier inside the GEMMs gives up after a number of polls; the kernel then returns
and writes I8L_ERR_TIMEOUT into the caller's status word.  The test hook i8l_test_set_wait_limit lowers
the limit to a few hundred polls and makes each CTA's operand producer leave out one load, so the waits
that depend on that load run out.  Checked: the launch returns, the status word holds TIMEOUT, the
context stays usable, and the next normal GEMM on the same stream is bit-exact.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"

if torch.cuda.is_available():
    from triton_int8_b200 import _lib as L
    from triton_int8_b200 import kernels as K

TIMEOUT = -5


def _operands(M, N, Kd, seed=3):
    g = torch.Generator().manual_seed(seed)
    a = torch.randint(-127, 128, (1, M, Kd), generator=g, dtype=torch.int8).to(DEV)
    b = torch.randint(-127, 128, (N, Kd), generator=g, dtype=torch.int8).to(DEV)
    return a, b


def _exact_i32(a, b):
    return torch._int_mm(a[0].cpu(), b.cpu().t().contiguous())


@pytest.mark.parametrize("kind,M,N,Kd", [
    ("block_fast", 2048, 4096, 512),    # 256 tiles on 148 CTAs: a second tile follows the withheld load
    ("block_exact", 256, 512, 1024),
    ("rowcol_single", 384, 512, 1024),  # M not a multiple of 256: one CTA per tile
    ("rowcol_pair", 256, 256, 1024),    # CTA pair (cta_group::2), one tile
    ("dump", 128, 256, 512),
])
def test_wait_runs_out_and_the_next_gemm_is_exact(kind, M, N, Kd):
    lib = L.load()
    a, b = _operands(M, N, Kd)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    a_tile = torch.ones(1, M // 128, Kd // 128, device=DEV)
    a_row = torch.ones(1, M, device=DEV)
    b_ch = torch.ones(N, device=DEV)

    def launch(st):
        if kind == "block_fast":
            return K.gemm_block(a, b, a_tile, b_ch, status=st, flags=L.GEMM_OUT_F32)
        if kind == "block_exact":
            return K.gemm_block(a, b, a_tile, b_ch, status=st, flags=L.GEMM_OUT_F32 | L.GEMM_EXACT_ORDER)
        if kind == "dump":
            return K.gemm_dump_i32(a, b, status=st)
        return K.gemm_rowcol(a, b, a_row, b_ch, status=st, flags=L.GEMM_OUT_F32)

    assert lib.i8l_test_set_wait_limit(256, 1) == 0
    try:
        launch(status)
        torch.cuda.synchronize()          # returns: no wait is unbounded
    finally:
        assert lib.i8l_test_set_wait_limit(0, 0) == 0
    assert status.item() == TIMEOUT
    status.zero_()
    out = launch(status)                   # same stream, same context: must be unaffected
    torch.cuda.synchronize()
    assert status.item() == 0
    ref = _exact_i32(a, b)
    if kind == "dump":
        assert torch.equal(out[0].cpu(), ref)
    else:                                  # unit scales: the fp32 result is the exact integer (|P| < 2^24 here)
        assert torch.equal(out[0].cpu(), ref.float())


def test_status_word_of_the_wrappers_reports_and_clears():
    """Without an explicit status argument the wrappers report into the per-device word that
    check_status() reads: it raises once and is clear afterwards."""
    lib = L.load()
    a, b = _operands(256, 256, 512)
    a_tile = torch.ones(1, 2, 4, device=DEV)
    b_ch = torch.ones(256, device=DEV)
    K.check_status(DEV)
    assert lib.i8l_test_set_wait_limit(256, 1) == 0
    try:
        K.gemm_block(a, b, a_tile, b_ch)
        torch.cuda.synchronize()
    finally:
        assert lib.i8l_test_set_wait_limit(0, 0) == 0
    with pytest.raises(L.I8LError, match="TIMEOUT"):
        K.check_status(DEV)
    K.check_status(DEV)                    # cleared by the raise
    K.gemm_block(a, b, a_tile, b_ch)
    K.check_status(DEV)
