"""block_channel variant: activation scaled per 128x128 tile, weight per output channel.

Same function names and argument meaning as the reference's triton/block_channel_fwd32.py and
triton/block_channel_bwd33.py; the bodies call the sm_100a kernels through the C ABI.  Unlike
the reference the pipeline neither synchronises the device nor prints timings
(triton/block_channel_fwd32.py:218-238).
"""
from __future__ import annotations

import torch

from . import _lib as L
from . import kernels as K

_QMODE = {"half_up": L.QMODE_TRITON, "rne": L.QMODE_RNE}


def calc_diff(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """1 - 2<x,y>/(|x|^2+|y|^2) in float64 (triton/block_channel_fwd32.py:244-248)."""
    x, y = x.double(), y.double()
    return 1 - 2 * (x * y).sum() / (x * x + y * y).sum()


def triton_per_block_quant(x: torch.Tensor, round: str = "half_up", hadamard: int = 0):
    """x bf16 [B, M, K] -> (int8 [B, M, K], fp32 scale [B, M/128, K/128]).
    triton/block_channel_fwd32.py:194-212."""
    assert x.dim() == 3
    q, s, _, _ = K.quant_tile(x, L.GRAN_TILE128, _QMODE[round], hadamard)
    return q, s


def triton_per_group_quant(x: torch.Tensor, round: str = "rne", hadamard: int = 0):
    """x bf16 [B, M, K] -> (int8, fp32 scale [B, M, K/128]): one scale per (row, 128 K elements),
    the grouping of the reference's commented helper tilelang/block_channel_fwd.py:206-213."""
    assert x.dim() == 3
    q, s, _, _ = K.quant_tile(x, L.GRAN_GROUP128, _QMODE[round], hadamard)
    return q, s


def triton_per_block256_quant(x: torch.Tensor):
    """x bf16 [B, M, K] -> (int8, fp32 scale [B, M/128, K/256]) with the scale rounded to bf16: the
    activation quantizer in front of the reference's TileLang forward GEMM
    (tilelang/block_channel_fwd.py:152-204, 128 x 256 groups, bf16 scale tensor)."""
    assert x.dim() == 3
    q, s, _, _ = K.quant_tile(x, L.GRAN_TILE128X256, L.QMODE_TRITON_BF16S, 0)
    return q, s


def triton_per_token_quant_bf16scale(x: torch.Tensor):
    """Per-row quantizer whose stored scale is rounded to bf16 (tilelang/block_channel_fwd.py:94-149)."""
    assert x.dim() == 2
    q, s = K.quant_row(x, L.QMODE_TRITON_BF16S, 0)
    return q, s.view(-1, 1)


def triton_per_token_quant(x: torch.Tensor, round: str = "half_up", hadamard: int = 0):
    """x bf16 [N, K] -> (int8 [N, K], fp32 scale [N, 1]).  triton/block_channel_fwd32.py:132-157.
    Unlike the reference, K does not have to be a power of two."""
    assert x.dim() == 2 and x.shape[1] % 128 == 0
    q, s = K.quant_row(x, _QMODE[round], hadamard)
    return q, s.view(-1, 1)


def triton_gemm(A_int8, B_int8, A_scale, B_scale, out_dtype=torch.bfloat16, exact: bool = False,
                bias=None, post_scale: float = 1.0, product_first: bool = False):
    """C[b] = sum_kb float(A_q[b,:,kb] . B_q[:,kb]^T) * A_scale * B_scale.

    B_int8 2-D [N, K] with B_scale [N, 1] or [N]  -> triton/block_channel_fwd32.py:68-96;
    B_int8 3-D [B, N, K] with B_scale [B, N/128, K/128] -> triton/block_channel_bwd33.py:58-84.
    A_scale [B, M/128, K/128] (per tile) or [B, M, K/128] (per row group).
    """
    B, M, Kd = A_int8.shape
    a_kind = L.ASCALE_TILE if A_scale.shape[1] == M // 128 and M != M // 128 else L.ASCALE_GROUP
    if a_kind == L.ASCALE_TILE and A_scale.shape[2] * 256 == Kd:
        a_kind = L.ASCALE_TILE256
    if B_int8.dim() == 2:
        N = B_int8.shape[0]
        if B_scale.numel() == N:
            b_kind = L.BSCALE_CHANNEL
        elif B_scale.numel() == (N // 128) * (Kd // 128):
            b_kind = L.BSCALE_TILE
        else:
            b_kind = L.BSCALE_GROUP
    else:
        N = B_int8.shape[1]
        b_kind = L.BSCALE_TILE if B_scale.shape[1] == N // 128 else L.BSCALE_GROUP
    flags = (L.GEMM_EXACT_ORDER if exact else 0) | (L.GEMM_OUT_F32 if out_dtype == torch.float32 else 0)
    if exact and product_first:   # the TileLang kernels' order: float(P) * (a_s * b_s)
        flags |= L.GEMM_PRODUCT_FIRST
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise TypeError("out_dtype must be bfloat16 or float32")
    return K.gemm_block(A_int8, B_int8, A_scale, B_scale, a_kind, b_kind, bias, post_scale, flags)


def int8_gemm_pipeline(A_bf, B_bf, out_dtype=torch.bfloat16, **kw):
    """Quantize both operands, multiply.  2-D B_bf: forward pipeline
    (triton/block_channel_fwd32.py:216-240); 3-D B_bf: backward pipeline
    (triton/block_channel_bwd33.py:148-172)."""
    return fwd_32(A_bf, B_bf, out_dtype=out_dtype, **kw) if B_bf.dim() == 2 else bwd_33(A_bf, B_bf, out_dtype=out_dtype, **kw)


def fwd_32(a: torch.Tensor, b: torch.Tensor, *, scaling: str = "tile128", round: str = "half_up",
           hadamard: int = 0, bias=None, exact: bool = False, out_dtype=torch.bfloat16):
    """a bf16 [B, M, K], b bf16 [N, K] -> bf16 [B, M, N] = a @ b^T through int8.
    triton/block_channel_fwd32.py:252-254.  Defaults are the reference's live code
    (per-tile activation scale, round half up); scaling="row128", round="rne" select the
    per-(row, 128) grouping with round-to-nearest-even; scaling="tile128x256_bf16scale" the numerics of
    the reference's TileLang forward; hadamard=128 rotates both operands in
    128-wide groups along K first (the product is rescaled by 1/128)."""
    if scaling == "tile128x256_bf16scale":
        # numerics of the reference's TileLang forward (tilelang/block_channel_fwd.py:271-292): activation
        # scale per 128 x 256, both scale tensors rounded to bf16, a_s * b_s formed first in every K step
        if hadamard or round != "half_up":
            raise ValueError("tile128x256_bf16scale is defined without rotation and with round half up")
        aq, a_s = triton_per_block256_quant(a)
        bq, b_s = triton_per_token_quant_bf16scale(b)
        return triton_gemm(aq, bq, a_s, b_s, out_dtype, exact=exact, bias=bias, product_first=True)
    quant_a = triton_per_block_quant if scaling == "tile128" else triton_per_group_quant
    aq, a_s = quant_a(a, round=round, hadamard=hadamard)
    bq, b_s = triton_per_token_quant(b, round=round, hadamard=hadamard)
    return triton_gemm(aq, bq, a_s, b_s, out_dtype, exact=exact, bias=bias,
                       post_scale=1.0 / hadamard if hadamard else 1.0)


def bwd_33(a: torch.Tensor, b: torch.Tensor, *, scaling: str = "tile128", round: str = "half_up",
           hadamard: int = 0, exact: bool = False, out_dtype=torch.bfloat16):
    """a bf16 [B, M, K], b bf16 [B, N, K] -> bf16 [B, M, N] = a @ b^T per batch, both operands
    scaled per 128x128 tile.  triton/block_channel_bwd33.py:175-177."""
    tilelang = scaling == "tilelang_tile128"   # tilelang/block_channel_bwd.py:197-223: tile scales, a_s * b_s first
    quant = triton_per_block_quant if scaling in ("tile128", "tilelang_tile128") else triton_per_group_quant
    aq, a_s = quant(a, round=round, hadamard=hadamard)
    bq, b_s = quant(b, round=round, hadamard=hadamard)
    return triton_gemm(aq, bq, a_s, b_s, out_dtype, exact=exact, post_scale=1.0 / hadamard if hadamard else 1.0,
                       product_first=tilelang)
