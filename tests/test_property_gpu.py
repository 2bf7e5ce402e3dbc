"""Property tests over random shapes (multiples of 128) and batch sizes: every variant's exact mode must
equal the CPU oracle bit for bit, the default mode must stay within the bf16 tolerance."""
import pytest
import torch
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from oracle import ref_semantics as R

pytestmark = pytest.mark.gpu
DEV = "cuda"

if torch.cuda.is_available():
    from triton_int8_b200 import block_channel as BC
    from triton_int8_b200 import double_channel as DC
    from triton_int8_b200 import fused as FU
    from triton_int8_b200 import kernels as K

dims = st.integers(min_value=1, max_value=5).map(lambda v: 128 * v)
SET = dict(max_examples=12, deadline=None, suppress_health_check=list(HealthCheck), derandomize=True)


def _mk(seed, *shape, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(torch.bfloat16)


@settings(**SET)
@given(B=st.integers(1, 3), M=dims, N=dims, Kd=dims, seed=st.integers(0, 10**6))
def test_block_channel_exact_equals_oracle(B, M, N, Kd, seed):
    a, w, b3 = _mk(seed, B, M, Kd), _mk(seed + 1, N, Kd, std=0.05), _mk(seed + 2, B, N, Kd)
    got = BC.fwd_32(a.to(DEV), w.to(DEV), exact=True)
    assert torch.equal(got.cpu(), R.block_channel_fwd_32(a, w))
    got = BC.bwd_33(a.to(DEV), b3.to(DEV), exact=True)
    assert torch.equal(got.cpu(), R.block_channel_bwd_33(a, b3))
    fast = BC.fwd_32(a.to(DEV), w.to(DEV))
    assert R.rel_fro(fast.cpu().float(), R.block_channel_fwd_32(a, w, return_fp32=True)) < 1e-2


@settings(**SET)
@given(B=st.integers(1, 2), M=dims, N=dims, Kd=dims, seed=st.integers(0, 10**6))
def test_double_channel_and_fused_equal_oracle(B, M, N, Kd, seed):
    a, w, b3 = _mk(seed, B, M, Kd), _mk(seed + 1, N, Kd, std=0.05), _mk(seed + 2, B, N, Kd)
    assert torch.equal(DC.fwd_32(a.to(DEV), w.to(DEV), hadamard=128).cpu(), _dc_ref(a, w, 128))
    assert torch.equal(DC.bwd_33(a.to(DEV), b3.to(DEV), hadamard=None).cpu(), R.double_channel_bwd_33(a, b3, use_hadamard=False))
    assert torch.equal(FU.fused_int8_gemm(a.to(DEV), w.to(DEV), out_dtype=torch.float32, exact=True).cpu(),
                       R.fused_fwd_32(a, w, return_fp32=True))
    assert torch.equal(FU.fused_int8_gemm(a.to(DEV), b3.to(DEV), out_dtype=torch.float32, exact=True).cpu(),
                       R.fused_bwd_33(a, b3, return_fp32=True))


def _dc(t, block):
    return R.quant_row(R.hadamard(t, block))


def _dc_ref(a, w, block):
    """double_channel forward with a blockwise rotation: rescale by 1/block in bf16 like the reference's 1/K pass."""
    aq, a_s = _dc(a, block)
    wq, w_s = _dc(w, block)
    return R.gemm_rowcol(aq, wq, a_s, w_s).to(torch.bfloat16) * (1.0 / block)


@settings(**SET)
@given(M=dims, N=dims, Kd=dims, bb=st.booleans(), seed=st.integers(0, 10**6))
def test_int32_accumulators_random_shapes(M, N, Kd, bb, seed):
    g = torch.Generator().manual_seed(seed)
    aq = torch.randint(-128, 128, (2, M, Kd), generator=g, dtype=torch.int8)
    bq = torch.randint(-128, 128, (2, N, Kd) if bb else (N, Kd), generator=g, dtype=torch.int8)
    assert torch.equal(K.gemm_dump_i32(aq.to(DEV), bq.to(DEV)).cpu(), R.gemm_i32(aq, bq))
