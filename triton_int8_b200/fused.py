"""fused variant: bf16 in, bf16 out, scales recomputed per 128-wide K step.

The reference's single Triton kernel (triton/fused_triton_fwd32.py:23-96,
triton/fused_triton_bwd33.py:24-86) re-quantises every A tile N/128 times and every B tile M/128
times.  Its integers and scales depend only on the operand tile, so this implementation
quantises each operand once (scale 127/(amax+1e-5), no clamp) and feeds the block-scaled tensor-core
GEMM with the reference's `acc += dot / (s_a * s_b)` arithmetic: identical results, no repeated work.
"""
from __future__ import annotations

import torch

from . import _lib as L
from . import kernels as K
from .block_channel import calc_diff  # noqa: F401


def fused_int8_gemm(A_bf: torch.Tensor, B_bf: torch.Tensor, out_dtype=torch.bfloat16, exact: bool = False,
                    single_kernel: bool = False):
    """A_bf [B, M, K]; B_bf [N, K] (fwd: per (row, 128-K) scales, triton/fused_triton_fwd32.py:57-59)
    or [B, N, K] (bwd: per 128x128 tile, triton/fused_triton_bwd33.py:54-56).  exact=True divides per
    element in the reference's operation order (bit-equal fp32); the default multiplies by the rounded
    reciprocal of s_a*s_b and fuses the accumulation (same integers, ~1e-7 relative difference).
    single_kernel=True runs i8l_fused_gemm, one kernel from bf16 to the result as in the reference; the default
    quantizes each operand once and feeds the block-scaled GEMM, which is faster on all but small shapes."""
    if single_kernel:
        # the reference's own structure: one launch, tiles re-quantized inside the GEMM for every output tile that
        # consumes them (same integers and scales as below, N/128 resp. M/128 times the quantization work)
        flags = (L.GEMM_EXACT_ORDER if exact else 0) | (L.GEMM_OUT_F32 if out_dtype == torch.float32 else 0)
        return K.fused_gemm(A_bf, B_bf, flags)
    aq, a_s, _, _ = K.quant_tile(A_bf, L.GRAN_TILE128, L.QMODE_FUSED)
    flags = L.GEMM_DIVIDE | (L.GEMM_EXACT_ORDER if exact else 0) | (L.GEMM_OUT_F32 if out_dtype == torch.float32 else 0)
    if B_bf.dim() == 2:
        bq, b_s, _, _ = K.quant_tile(B_bf[None], L.GRAN_GROUP128, L.QMODE_FUSED)
        return K.gemm_block(aq, bq[0], a_s, b_s[0], L.ASCALE_TILE, L.BSCALE_GROUP, flags=flags)
    bq, b_s, _, _ = K.quant_tile(B_bf, L.GRAN_TILE128, L.QMODE_FUSED)
    return K.gemm_block(aq, bq, a_s, b_s, L.ASCALE_TILE, L.BSCALE_TILE, flags=flags)


def fwd_32(a: torch.Tensor, b: torch.Tensor, *, single_kernel: bool = False):
    """triton/fused_triton_fwd32.py:104-108 (inputs must already be on the GPU)."""
    assert a.dim() == 3 and b.dim() == 2
    return fused_int8_gemm(a, b, single_kernel=single_kernel)


def bwd_33(a: torch.Tensor, b: torch.Tensor, *, single_kernel: bool = False):
    """triton/fused_triton_bwd33.py:94-98."""
    assert a.dim() == 3 and b.dim() == 3
    return fused_int8_gemm(a, b, single_kernel=single_kernel)
