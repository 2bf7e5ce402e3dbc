"""double_channel variant: per-token activation scale x per-output-channel weight scale, int32
accumulation over the whole K, optional full-length Hadamard rotation in front.

Mirrors triton/double-channle_fwd32.py and triton/double_channel_bwd33.py of the reference.  The
rotation the reference obtains from the external fast_hadamard_transform extension is fused into
the row quantizer here, and the torch glue between its two quantizer passes (max, clamp, 127/amax,
amax/127) as well as the trailing `C * (1/K)` pass are part of the kernels.
"""
from __future__ import annotations

import torch

from . import _lib as L
from . import kernels as K
from .block_channel import calc_diff  # noqa: F401  (same helper in every reference file)


def _had(hadamard) -> int:
    if hadamard in (None, False, 0, "none"):
        return L.HAD_NONE
    if hadamard in (True, "full", -1):
        return L.HAD_FULL
    if hadamard == 128:
        return L.HAD_128
    raise ValueError(f"hadamard must be None, 'full' or 128, got {hadamard!r}")


def triton_per_row_quant_2d(x: torch.Tensor, BLOCK_N: int = 2048, hadamard=None):
    """x bf16 [M, N] -> (int8 [M, N], fp32 scale_inv [M]).  triton/double-channle_fwd32.py:140-175.
    BLOCK_N is accepted for signature compatibility; the kernel needs no column blocking and N only
    has to be a multiple of 128."""
    assert x.dim() == 2
    return K.quant_row(x, L.QMODE_ROWRCP, _had(hadamard))


def triton_per_row_quant_3d(x: torch.Tensor, BLOCK_N: int = 2048, hadamard=None, **_unused):
    """x bf16 [B, M, N] -> (int8 [B, M, N], fp32 scale_inv [B, M]).
    triton/double-channle_fwd32.py:229-266, triton/double_channel_bwd33.py:142-176."""
    assert x.dim() == 3
    return K.quant_row(x, L.QMODE_ROWRCP, _had(hadamard))


def triton_gemm(A_int8, B_int8, A_scale, B_scale, out_dtype=torch.bfloat16, post_scale: float = 1.0, bias=None):
    """C = (float(A_q . B_q^T) * A_scale[m]) * B_scale[n]; B_int8 [N, K] / B_scale [N]
    (triton/double-channle_fwd32.py:62-90) or B_int8 [B, N, K] / B_scale [B, N]
    (triton/double_channel_bwd33.py:60-87)."""
    flags = L.GEMM_OUT_F32 if out_dtype == torch.float32 else 0
    return K.gemm_rowcol(A_int8, B_int8, A_scale, B_scale, bias, post_scale, flags)


def int8_gemm_pipeline(A_bf, B_bf, out_dtype=torch.bfloat16, hadamard="full", bias=None):
    """Rotate, quantize per row, multiply, rescale by 1/K (1/128 for blockwise rotation).
    triton/double-channle_fwd32.py:269-285, triton/double_channel_bwd33.py:186-201."""
    had = _had(hadamard)
    Kd = A_bf.shape[-1]
    post = 1.0 / Kd if had == L.HAD_FULL else (1.0 / 128 if had == L.HAD_128 else 1.0)
    aq, a_s = triton_per_row_quant_3d(A_bf, hadamard=hadamard)
    bq, b_s = K.quant_row(B_bf, L.QMODE_ROWRCP, had)
    return triton_gemm(aq, bq, a_s, b_s, out_dtype, post_scale=post, bias=bias)


def fwd_32(a: torch.Tensor, b: torch.Tensor, *, hadamard="full", bias=None):
    """a bf16 [B, M, K], b bf16 [N, K] -> bf16 [B, M, N].  triton/double-channle_fwd32.py:295-311."""
    assert a.dim() == 3 and b.dim() == 2
    return int8_gemm_pipeline(a, b, torch.bfloat16, hadamard, bias)


def bwd_33(a: torch.Tensor, b: torch.Tensor, *, hadamard="full"):
    """a bf16 [B, M, K], b bf16 [B, N, K] -> bf16 [B, M, N].  triton/double_channel_bwd33.py:204-220."""
    assert a.dim() == 3 and b.dim() == 3
    return int8_gemm_pipeline(a, b, torch.bfloat16, hadamard)
