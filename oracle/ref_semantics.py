"""CPU restatement (torch, fp32/int32 exact) of the reference's INT8 linear path.

TEST INFRASTRUCTURE, NOT PRODUCT: this file is the checker the CUDA path is
compared against and the timed CPU baseline.  The shipped package never imports
it.  Every function cites the reference lines it restates (paths are relative
to the reference project root).

Pinning: tests/golden/make_golden.py executes the reference's own Triton
kernels under TRITON_INTERPRET=1 and stores their outputs; test_oracle_golden
checks this restatement against those files bit for bit.  The Walsh-Hadamard
rotation is the one piece with no reference source (third-party extension
fast_hadamard_transform, unpinned, README.md:2): "parity unpinned" for it, the
butterfly order below is the definition the CUDA kernels follow.

Arithmetic notes that matter for bit-exactness:
  * Triton's `127.0 / amax` on fp32 is a true IEEE division; torch's
    `127.0 / tensor` is `reciprocal(tensor) * 127.0`.  Both appear in the
    reference and both are restated literally (`_div_true` vs `_rdiv_torch`).
  * `x * s + 0.5` is an unfused multiply followed by an add.
  * The int8 x int8 products are summed exactly in int32 (torch._int_mm).
"""
from __future__ import annotations

import math
import torch

BLK = 128


# --------------------------------------------------------------------------- helpers
def _div_true(num: float, t: torch.Tensor) -> torch.Tensor:
    """IEEE fp32 `num / t` (what a Triton kernel computes for `num / t`)."""
    return torch.full_like(t, num) / t


def _rdiv_torch(num: float, t: torch.Tensor) -> torch.Tensor:
    """torch's `num / t` for a Python scalar: reciprocal(t) * num."""
    return t.reciprocal() * num


def _round_half_up_i8(y: torch.Tensor, clamp: bool) -> torch.Tensor:
    r = torch.floor(y + 0.5)
    if clamp:
        r = torch.clamp(r, -128.0, 127.0)
    return r.to(torch.int8)


def calc_diff(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """1 - 2<x,y>/(|x|^2+|y|^2) in float64 (triton/block_channel_fwd32.py:244-248)."""
    x, y = x.double(), y.double()
    return 1 - 2 * (x * y).sum() / (x * x + y * y).sum()


def rel_fro(x: torch.Tensor, ref: torch.Tensor) -> float:
    x, ref = x.double(), ref.double()
    return float((x - ref).norm() / ref.norm().clamp_min(1e-300))


# --------------------------------------------------------------------------- quantizers
def quant_tile128(x: torch.Tensor, clamp: bool = True):
    """Per 128x128 tile absmax quantizer, round half up.

    triton/block_channel_fwd32.py:160-212 (`per_block_quant_kernel`,
    `triton_per_block_quant`); the copy in triton/block_channel_bwd33.py:87-138
    omits the clamp (:114), which never triggers.
    x: bf16 [B, M, K] -> int8 [B, M, K], fp32 scale [B, M/128, K/128] = 1/(127/amax).
    """
    B, M, K = x.shape
    v = x.float().view(B, M // BLK, BLK, K // BLK, BLK)
    amax = v.abs().amax(dim=(2, 4), keepdim=True)
    amax = torch.where(amax > 1e-4, amax, torch.full_like(amax, 1e-4))
    s = _div_true(127.0, amax)
    q = _round_half_up_i8(v * s, clamp).view(B, M, K)
    return q, _div_true(1.0, s).view(B, M // BLK, K // BLK)


def quant_token(w: torch.Tensor):
    """Per-row (output channel) absmax quantizer over the whole row.

    triton/block_channel_fwd32.py:101-157 (`per_token_quant_kernel`).
    w: bf16 [N, K] -> int8 [N, K], fp32 scale [N, 1].
    """
    v = w.float()
    amax = v.abs().amax(dim=1, keepdim=True)
    amax = torch.where(amax > 1e-4, amax, torch.full_like(amax, 1e-4))
    s = _div_true(127.0, amax)
    q = _round_half_up_i8(v * s, True)
    return q, _div_true(1.0, s)


def quant_row(x: torch.Tensor):
    """double_channel two-pass per-row quantizer (any leading dims).

    triton/double-channle_fwd32.py:93-266 and triton/double_channel_bwd33.py:90-176:
    amax over the row (max of 2048-wide partial maxima == max of the row),
    clamp(min=1e-4), `scale_mul = 127.0/amax` evaluated by torch (reciprocal*127),
    `scale_inv = amax/127.0`, q = clamp(floor(x*scale_mul + 0.5), -128, 127).
    x: bf16 [..., K] -> int8 [..., K], fp32 scale_inv [...].
    """
    v = x.float()
    amax = torch.clamp(v.abs().amax(dim=-1), min=1e-4)
    scale_mul = _rdiv_torch(127.0, amax)
    scale_inv = amax / 127.0
    q = _round_half_up_i8(v * scale_mul.unsqueeze(-1), True)
    return q, scale_inv


def quant_tile128_rne(x: torch.Tensor):
    """The reference's unused torch helper: per 128x128 tile, round to nearest even,
    symmetric clamp (tilelang/block_channel_bwd.py:96-104).
    """
    B, M, K = x.shape
    v = x.float().view(B, M // BLK, BLK, K // BLK, BLK)
    amax = v.abs().amax(dim=(2, 4), keepdim=True).clamp(min=1e-4)
    s = _rdiv_torch(127.0, amax)
    q = (v * s).round().clamp(-127, 127).to(torch.int8).view(B, M, K)
    return q, _rdiv_torch(1.0, s).view(B, M // BLK, K // BLK)


def quant_rowgroup128_rne(x: torch.Tensor):
    """Per (row, 128-wide group) absmax, round to nearest even, symmetric clamp: the
    commented-out helper at tilelang/block_channel_fwd.py:206-213, evaluated in fp32
    like its live sibling tilelang/block_channel_bwd.py:96-104.
    x: bf16 [..., K] -> int8 [..., K], fp32 scale [..., K/128].
    """
    lead, K = x.shape[:-1], x.shape[-1]
    v = x.float().reshape(*lead, K // BLK, BLK)
    amax = v.abs().amax(dim=-1, keepdim=True).clamp(min=1e-4)
    s = _rdiv_torch(127.0, amax)
    q = (v * s).round().clamp(-127, 127).to(torch.int8).reshape(*lead, K)
    return q, _rdiv_torch(1.0, s).reshape(*lead, K // BLK)


def quant_token_rne(w: torch.Tensor):
    """Per-row helper with RNE (tilelang/block_channel_fwd.py:215-220), fp32 math."""
    v = w.float()
    amax = v.abs().amax(dim=1, keepdim=True).clamp(min=1e-4)
    s = _rdiv_torch(127.0, amax)
    q = (v * s).round().clamp(-127, 127).to(torch.int8)
    return q, _rdiv_torch(1.0, s)


def quant_rowgroup128(x: torch.Tensor):
    """Per (row, 128-wide group) absmax with the live Triton arithmetic (true division,
    round half up, clamp): the per-(row, 128) grouping of the 512x1024x1024 test configuration combined with the rounding
    of triton/block_channel_fwd32.py:181-192.
    """
    lead, K = x.shape[:-1], x.shape[-1]
    v = x.float().reshape(*lead, K // BLK, BLK)
    amax = v.abs().amax(dim=-1, keepdim=True)
    amax = torch.where(amax > 1e-4, amax, torch.full_like(amax, 1e-4))
    s = _div_true(127.0, amax)
    q = _round_half_up_i8(v * s, True).reshape(*lead, K)
    return q, _div_true(1.0, s).reshape(*lead, K // BLK)


def quant_rne_native(x: torch.Tensor, group: str):
    """The torch helpers of tilelang/block_channel_fwd.py with their arithmetic kept in the INPUT dtype
    (no upcast anywhere: for bf16 input the absmax, `127.0 / amax` = reciprocal * 127, the product
    x * scale, round() and the returned 1.0 / scale are all bf16 operations, each rounded to bf16):
      group "tile"     per 128x128 tile of x [B, M, K]       tilelang/block_channel_fwd.py:222-230
      group "row"      per row of x [M, K]                   tilelang/block_channel_fwd.py:215-220
      group "row128"   per (row, 128 columns) of x [M, K]    tilelang/block_channel_fwd.py:206-213 (commented out)
    The copy in tilelang/block_channel_bwd.py:96-104 upcasts the absmax to fp32 first, which promotes
    everything after it to fp32: that one is quant_tile128_rne above.  For fp32 input the two agree.
    Returns (int8 like x, scale in x.dtype)."""
    if group == "tile":
        B, M, K = x.shape
        v = x.reshape(B, M // BLK, BLK, K // BLK, BLK)
        amax = v.abs().amax(dim=(2, 4), keepdim=True)
        out_shape, s_shape = (B, M, K), (B, M // BLK, K // BLK)
    elif group == "row":
        M, K = x.shape
        v = x
        amax = v.abs().amax(dim=1, keepdim=True)
        out_shape, s_shape = (M, K), (M, 1)
    else:
        M, K = x.shape
        v = x.reshape(M, K // BLK, BLK)
        amax = v.abs().amax(dim=2, keepdim=True)
        out_shape, s_shape = (M, K), (M, K // BLK)
    s = _rdiv_torch(127.0, amax.clamp(min=1e-4))
    q = (v * s).round().clamp(-127, 127).to(torch.int8).reshape(out_shape)
    return q, _rdiv_torch(1.0, s).reshape(s_shape)


# --------------------------------------------------------------------------- TileLang variant numerics
def _bf16_rne(t: torch.Tensor) -> torch.Tensor:
    """fp32 -> bf16 (round to nearest even, what a GPU store does) -> fp32."""
    return t.to(torch.bfloat16).float()


def quant_tile128x256_bf16scale(x: torch.Tensor):
    """Activation quantizer in front of the TileLang forward GEMM: one scale per 128 rows x 256
    columns (tilelang/block_channel_fwd.py:185-188), live Triton arithmetic (true division, round
    half up, no clamp: :168-172), the stored reciprocal scale rounded to bf16 because the wrapper
    allocates a bf16 scale tensor and widens it afterwards (:191, :204).
    x bf16 [B, M, K] (K a multiple of 256) -> int8 [B, M, K], fp32 scale [B, M/128, K/256].
    Also returns the unrounded fp32 scale (what the kernel computes before the bf16 store)."""
    B, M, K = x.shape
    v = x.float().view(B, M // BLK, BLK, K // 256, 256)
    amax = v.abs().amax(dim=(2, 4), keepdim=True)
    amax = torch.where(amax > 1e-4, amax, torch.full_like(amax, 1e-4))
    s = _div_true(127.0, amax)
    q = _round_half_up_i8(v * s, False).view(B, M, K)
    inv = _div_true(1.0, s).view(B, M // BLK, K // 256)
    return q, _bf16_rne(inv), inv


def quant_token_bf16scale(w: torch.Tensor):
    """Per-row weight quantizer of the same file (tilelang/block_channel_fwd.py:94-121, bf16 scale
    tensor :133, widened :149).  w bf16 [N, K] -> int8 [N, K], fp32 scale [N, 1] (+ unrounded scale)."""
    v = w.float()
    amax = v.abs().amax(dim=1, keepdim=True)
    amax = torch.where(amax > 1e-4, amax, torch.full_like(amax, 1e-4))
    s = _div_true(127.0, amax)
    q = _round_half_up_i8(v * s, False)
    inv = _div_true(1.0, s)
    return q, _bf16_rne(inv), inv


def gemm_tilelang_fwd(aq, bq, a_s, b_s) -> torch.Tensor:
    """TileLang forward GEMM (tilelang/block_channel_fwd.py:66-83): per 128-wide K step the column
    factor is the PRODUCT a_s[b, mb, (k*128)//256] * b_s[n] (:75-76), then
    acc_f32[m, n] += float(P[m, n]) * factor[n] (:80-81), evaluated unfused (multiply, then add).
    aq [B, M, K], bq [N, K], a_s [B, M/128, K/256], b_s [N] or [N, 1] -> fp32 [B, M, N]."""
    B, M, K = aq.shape
    N = bq.shape[0]
    out = torch.zeros(B, M, N, dtype=torch.float32)
    bs = b_s.reshape(1, N)
    for b in range(B):
        for kb in range(K // BLK):
            P = int_mm(aq[b, :, kb * BLK:(kb + 1) * BLK], bq[:, kb * BLK:(kb + 1) * BLK]).float()
            fac = a_s[b, :, (kb * BLK) // 256].repeat_interleave(BLK).view(M, 1) * bs
            out[b] += P * fac
    return out


def gemm_tilelang_bwd(aq, bq, a_s, b_s) -> torch.Tensor:
    """TileLang backward GEMM (tilelang/block_channel_bwd.py:66-83): scalar factor
    a_s[b, mb, kb] * b_s[b, nb, kb] per tile and K step (:76), acc += float(P) * factor (:80-81).
    aq [B, M, K], bq [B, N, K], fp32 scales per 128x128 tile -> fp32 [B, M, N]."""
    B, M, K = aq.shape
    N = bq.shape[1]
    out = torch.zeros(B, M, N, dtype=torch.float32)
    for b in range(B):
        for kb in range(K // BLK):
            P = int_mm(aq[b, :, kb * BLK:(kb + 1) * BLK], bq[b, :, kb * BLK:(kb + 1) * BLK]).float()
            fac = a_s[b, :, kb].repeat_interleave(BLK).view(M, 1) * b_s[b, :, kb].repeat_interleave(BLK).view(1, N)
            out[b] += P * fac
    return out


def tilelang_fwd_32(a: torch.Tensor, b: torch.Tensor, return_fp32: bool = False):
    """tilelang/block_channel_fwd.py:271-292 (quantizers :277-278, GEMM :287-288)."""
    aq, a_s, _ = quant_tile128x256_bf16scale(a)
    bq, b_s, _ = quant_token_bf16scale(b)
    c = gemm_tilelang_fwd(aq, bq, a_s, b_s)
    return c if return_fp32 else c.to(torch.bfloat16)


def tilelang_bwd_33(a: torch.Tensor, b: torch.Tensor, return_fp32: bool = False):
    """tilelang/block_channel_bwd.py:197-223: both operands per 128x128 tile with fp32 scales
    (:141-157, the clamp-less kernel), scale product first."""
    aq, a_s = quant_tile128(a, clamp=False)
    bq, b_s = quant_tile128(b, clamp=False)
    c = gemm_tilelang_bwd(aq, bq, a_s, b_s)
    return c if return_fp32 else c.to(torch.bfloat16)


# --------------------------------------------------------------------------- Hadamard
def hadamard(x: torch.Tensor, block: int | None = None) -> torch.Tensor:
    """Un-normalised Walsh-Hadamard transform (Sylvester order) along the last dim.

    Stand-in for fast_hadamard_transform.hadamard_transform as called at
    triton/double-channle_fwd32.py:273-274,299-300 and
    triton/double_channel_bwd33.py:189-190,208-209 (scale 1.0, dtype preserved).
    fp32 butterflies with the span doubling 1, 2, 4, ... ; result rounded to
    x.dtype.  block=None transforms the whole row (power-of-two length);
    block=128 transforms each 128-wide group independently.
    """
    K = x.shape[-1]
    n = K if block is None else block
    assert n & (n - 1) == 0 and K % n == 0
    v = x.float().reshape(-1, K // n, n).clone()
    h = 1
    while h < n:
        w = v.view(v.shape[0], v.shape[1], n // (2 * h), 2, h)
        a, b = w[..., 0, :].clone(), w[..., 1, :].clone()
        w[..., 0, :] = a + b
        w[..., 1, :] = a - b
        h *= 2
    return v.reshape(x.shape).to(x.dtype)


# --------------------------------------------------------------------------- GEMMs
def int_mm(aq: torch.Tensor, bq: torch.Tensor) -> torch.Tensor:
    """Exact int8 x int8 -> int32, C = aq @ bq^T for 2-D operands [M,K], [N,K]."""
    M = aq.shape[0]
    if M <= 16 or M % 8:
        return aq.to(torch.int32) @ bq.to(torch.int32).t()
    return torch._int_mm(aq.contiguous(), bq.t())


def gemm_block_fwd(aq, bq, a_s, b_s) -> torch.Tensor:
    """Block-scaled GEMM, A scale per 128x128 tile, B scale per output channel.

    triton/block_channel_fwd32.py:12-66: per 128-wide K step
    `acc += (float(P) * a_s[b,mb,kb]) * b_s[n]`, fp32, left to right.
    aq int8 [B,M,K], bq int8 [N,K], a_s [B,M/128,K/128], b_s [N,1] -> fp32 [B,M,N].
    """
    B, M, K = aq.shape
    N = bq.shape[0]
    out = torch.zeros(B, M, N, dtype=torch.float32)
    bsv = b_s.reshape(1, N)
    for b in range(B):
        for kb in range(K // BLK):
            P = int_mm(aq[b, :, kb * BLK:(kb + 1) * BLK], bq[:, kb * BLK:(kb + 1) * BLK]).float()
            sa = a_s[b, :, kb].repeat_interleave(BLK).view(M, 1)
            out[b] += (P * sa) * bsv
    return out


def gemm_block_bwd(aq, bq, a_s, b_s) -> torch.Tensor:
    """Block-scaled batched GEMM, both scales per 128x128 tile.

    triton/block_channel_bwd33.py:8-56: `acc += (float(P) * a_s[b,mb,kb]) * b_s[b,nb,kb]`.
    aq [B,M,K], bq [B,N,K], a_s [B,M/128,K/128], b_s [B,N/128,K/128] -> fp32 [B,M,N].
    """
    B, M, K = aq.shape
    N = bq.shape[1]
    out = torch.zeros(B, M, N, dtype=torch.float32)
    for b in range(B):
        for kb in range(K // BLK):
            P = int_mm(aq[b, :, kb * BLK:(kb + 1) * BLK], bq[b, :, kb * BLK:(kb + 1) * BLK]).float()
            sa = a_s[b, :, kb].repeat_interleave(BLK).view(M, 1)
            sb = b_s[b, :, kb].repeat_interleave(BLK).view(1, N)
            out[b] += (P * sa) * sb
    return out


def gemm_block_general(aq, bq, a_s, b_s, a_group_m: int, b_kind: str) -> torch.Tensor:
    """Generalisation used for the per-(row, 128-K) grouping of the 512x1024x1024 configuration:
    a_s is [B,M/a_group_m,K/128] with a_group_m in {1,128}; b_kind 'channel' ([N] K-invariant),
    'tile' ([B?,N/128,K/128]) or 'rowgroup' ([N,K/128]).  Same operation order as above.
    bq is [N,K] (shared) or [B,N,K].
    """
    B, M, K = aq.shape
    batched_b = bq.dim() == 3
    N = bq.shape[-2]
    out = torch.zeros(B, M, N, dtype=torch.float32)
    for b in range(B):
        bqb = bq[b] if batched_b else bq
        for kb in range(K // BLK):
            P = int_mm(aq[b, :, kb * BLK:(kb + 1) * BLK], bqb[:, kb * BLK:(kb + 1) * BLK]).float()
            sa = a_s[b, :, kb]
            if a_group_m == 128:
                sa = sa.repeat_interleave(BLK)
            sa = sa.view(M, 1)
            if b_kind == "channel":
                sb = b_s.reshape(1, N)
            elif b_kind == "tile":
                bs = b_s[b] if b_s.dim() == 3 else b_s
                sb = bs[:, kb].repeat_interleave(BLK).view(1, N)
            else:
                bs = b_s[b] if b_s.dim() == 3 else b_s
                sb = bs[:, kb].reshape(1, N)
            out[b] += (P * sa) * sb
    return out


def gemm_rowcol(aq, bq, a_s, b_s) -> torch.Tensor:
    """Full-K int32 accumulate, epilogue `(float(acc) * a_s[m]) * b_s[n]`.

    triton/double-channle_fwd32.py:11-59 (bq [N,K], b_s [N]) and
    triton/double_channel_bwd33.py:11-58 (bq [B,N,K], b_s [B,N]).  Returns fp32;
    the reference stores it as bf16 and multiplies by 1/K in bf16 afterwards
    (triton/double-channle_fwd32.py:284,310).
    """
    B, M, K = aq.shape
    batched_b = bq.dim() == 3
    N = bq.shape[-2]
    out = torch.empty(B, M, N, dtype=torch.float32)
    for b in range(B):
        acc = int_mm(aq[b], bq[b] if batched_b else bq)
        bs = b_s[b] if batched_b else b_s
        out[b] = (acc.float() * a_s[b].view(M, 1)) * bs.reshape(1, N)
    return out


def gemm_i32(aq, bq) -> torch.Tensor:
    """Raw int32 accumulators over the whole K (aq [B,M,K]; bq [N,K] or [B,N,K])."""
    B = aq.shape[0]
    return torch.stack([int_mm(aq[b], bq[b] if bq.dim() == 3 else bq) for b in range(B)])


# --------------------------------------------------------------------------- entry points
def block_channel_fwd_32(a: torch.Tensor, b: torch.Tensor, return_fp32: bool = False):
    """triton/block_channel_fwd32.py:216-254 without the syncs and prints."""
    aq, a_s = quant_tile128(a, clamp=True)
    bq, b_s = quant_token(b)
    c = gemm_block_fwd(aq, bq, a_s, b_s)
    return c if return_fp32 else c.to(torch.bfloat16)


def block_channel_bwd_33(a: torch.Tensor, b: torch.Tensor, return_fp32: bool = False):
    """triton/block_channel_bwd33.py:148-177."""
    aq, a_s = quant_tile128(a, clamp=False)
    bq, b_s = quant_tile128(b, clamp=False)
    c = gemm_block_bwd(aq, bq, a_s, b_s)
    return c if return_fp32 else c.to(torch.bfloat16)


def double_channel_fwd_32(a: torch.Tensor, b: torch.Tensor, use_hadamard: bool = True):
    """triton/double-channle_fwd32.py:295-311: rotate, per-row quantize, GEMM to bf16,
    then `C * (1/K)` in bf16."""
    inv_k = 1.0 / a.shape[-1]
    if use_hadamard:
        a, b = hadamard(a), hadamard(b)
    aq, a_s = quant_row(a)
    bq, b_s = quant_row(b)
    c = gemm_rowcol(aq, bq, a_s, b_s).to(torch.bfloat16)
    return c * inv_k if use_hadamard else c


def double_channel_bwd_33(a: torch.Tensor, b: torch.Tensor, use_hadamard: bool = True):
    """triton/double_channel_bwd33.py:204-220."""
    return double_channel_fwd_32(a, b, use_hadamard)


def fused_fwd_32(a: torch.Tensor, b: torch.Tensor, return_fp32: bool = False):
    """triton/fused_triton_fwd32.py:23-108: per K step the A tile (128x128) gets one
    scale 127/(amax+1e-5), each B row gets its own scale over the 128-wide K slice,
    no clamp, `acc += float(P) / (s_a * s_b[n])`.
    a bf16 [B,M,K], b bf16 [N,K] -> [B,M,N]."""
    B, M, K = a.shape
    N = b.shape[0]
    av = a.float().view(B, M // BLK, BLK, K // BLK, BLK)
    sa = _div_true(127.0, av.abs().amax(dim=(2, 4), keepdim=True) + 1e-5)
    aq = torch.floor(av * sa + 0.5).to(torch.int8).view(B, M, K)
    sa = sa.view(B, M // BLK, K // BLK)
    bv = b.float().view(N, K // BLK, BLK)
    sb = _div_true(127.0, bv.abs().amax(dim=2, keepdim=True) + 1e-5)
    bq = torch.floor(bv * sb + 0.5).to(torch.int8).view(N, K)
    sb = sb.view(N, K // BLK)
    out = torch.zeros(B, M, N, dtype=torch.float32)
    for bi in range(B):
        for kb in range(K // BLK):
            P = int_mm(aq[bi, :, kb * BLK:(kb + 1) * BLK], bq[:, kb * BLK:(kb + 1) * BLK]).float()
            den = sa[bi, :, kb].repeat_interleave(BLK).view(M, 1) * sb[:, kb].view(1, N)
            out[bi] += P / den
    return out if return_fp32 else out.to(torch.bfloat16)


def fused_bwd_33(a: torch.Tensor, b: torch.Tensor, return_fp32: bool = False):
    """triton/fused_triton_bwd33.py:24-98 with its 128-wide tiles: both operands one
    scale 127/(amax+1e-5) per 128x128 tile, `acc += float(P) / (s_a * s_b)`."""
    B, M, K = a.shape
    N = b.shape[1]

    def q(t, R):
        v = t.float().view(B, R // BLK, BLK, K // BLK, BLK)
        s = _div_true(127.0, v.abs().amax(dim=(2, 4), keepdim=True) + 1e-5)
        return torch.floor(v * s + 0.5).to(torch.int8).view(B, R, K), s.view(B, R // BLK, K // BLK)

    aq, sa = q(a, M)
    bq, sb = q(b, N)
    out = torch.zeros(B, M, N, dtype=torch.float32)
    for bi in range(B):
        for kb in range(K // BLK):
            P = int_mm(aq[bi, :, kb * BLK:(kb + 1) * BLK], bq[bi, :, kb * BLK:(kb + 1) * BLK]).float()
            den = sa[bi, :, kb].repeat_interleave(BLK).view(M, 1) * sb[bi, :, kb].repeat_interleave(BLK).view(1, N)
            out[bi] += P / den
    return out if return_fp32 else out.to(torch.bfloat16)


# --------------------------------------------------------------------------- linear layer
def linear_block_channel(x, w, dy, hadamard128: bool = False, bias=None):
    """Y, dX, dW of a linear layer by composition of the two primitives:
    Y = fwd_32(X[1,M,K], W[N,K]); dX = fwd_32(dY[1,M,N], W^T[K,N]);
    dW = bwd_33(dY^T[1,N,M], X^T[1,K,M]).  With hadamard128 every operand is rotated
    in 128-wide groups along the contraction axis of its GEMM and the product is
    scaled by 1/128 (exact) before the bf16 cast.  Bias (not in the reference) is
    added in fp32 before the cast.  Returns bf16 (y, dx, dw).
    """
    rot = (lambda t: hadamard(t, 128)) if hadamard128 else (lambda t: t)
    post = 1.0 / 128 if hadamard128 else 1.0
    y = block_channel_fwd_32(rot(x)[None], rot(w), return_fp32=True)[0] * post
    if bias is not None:
        y = y + bias.float()
    wt, dyt, xt = w.t().contiguous(), dy.t().contiguous(), x.t().contiguous()
    dx = block_channel_fwd_32(rot(dy)[None], rot(wt), return_fp32=True)[0] * post
    dw = block_channel_bwd_33(rot(dyt)[None], rot(xt)[None], return_fp32=True)[0] * post  # rotated along M
    return y.to(torch.bfloat16), dx.to(torch.bfloat16), dw.to(torch.bfloat16)
