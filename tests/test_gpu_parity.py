"""GPU parity tests: every CUDA kernel, called through the C ABI, against the CPU oracle and the
golden vectors produced by the reference's own kernels.  Integer outputs and scales must match
bit for bit; bf16 results within 1e-2 relative Frobenius error (far tighter in practice)."""
import os

import numpy as np
import pytest
import torch

from golden_inputs import make_inputs
from oracle import ref_semantics as R

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from triton_int8_b200 import _lib as L
    from triton_int8_b200 import block_channel as BC
    from triton_int8_b200 import double_channel as DC
    from triton_int8_b200 import fused as FU
    from triton_int8_b200 import kernels as K

DEV = "cuda"
TOL_BF16 = 1e-2  # relative Frobenius error allowed for bf16 outputs (north-star tolerance)


def _golden(golden_dir, name):
    return np.load(os.path.join(golden_dir, name + ".npz"))


def _same(t: torch.Tensor, ref, what=""):
    ref = torch.as_tensor(np.asarray(ref)) if not isinstance(ref, torch.Tensor) else ref
    t = t.detach().cpu()
    assert t.shape == ref.shape, f"{what}: shape {tuple(t.shape)} vs {tuple(ref.shape)}"
    bad = (t != ref).sum().item()
    assert bad == 0, f"{what}: {bad} of {t.numel()} entries differ"


def _status():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


def _randq(g, *shape):
    return torch.randint(-127, 128, shape, generator=g, dtype=torch.int8)


# ------------------------------------------------------------------------------ quantizers
@pytest.mark.parametrize("case", ["small", "edge", "c1"])
def test_quant_tile_and_token_match_reference(golden_dir, case):
    a, w, b3 = make_inputs(case)
    aq_ref, as_ref = R.quant_tile128(a)
    q, s = BC.triton_per_block_quant(a.to(DEV))
    _same(q, aq_ref, "tile int8"); _same(s, as_ref, "tile scale")
    wq_ref, ws_ref = R.quant_token(w)
    q, s = BC.triton_per_token_quant(w.to(DEV))
    _same(q, wq_ref, "token int8"); _same(s, ws_ref, "token scale")
    if case != "c1":
        g = _golden(golden_dir, "block_channel_" + case)
        _same(BC.triton_per_block_quant(a.to(DEV))[0], g["aq"], "tile int8 vs golden")
        _same(BC.triton_per_block_quant(b3.to(DEV))[1], g["b_s_bwd"], "tile scale vs golden")


@pytest.mark.parametrize("gran", ["tile", "group"])
@pytest.mark.parametrize("mode", ["triton", "rne", "fused"])
def test_quant_tile_modes_and_transposed_output(gran, mode):
    g = torch.Generator().manual_seed(7)
    x = (torch.randn(2, 256, 384, generator=g) * 3).to(torch.bfloat16)
    x[0, :128, :128] = 0
    x[1, 5, 200] = 40.0
    G = L.GRAN_TILE128 if gran == "tile" else L.GRAN_GROUP128
    Mo = {"triton": L.QMODE_TRITON, "rne": L.QMODE_RNE, "fused": L.QMODE_FUSED}[mode]
    q, s, qt, st = K.quant_tile(x.to(DEV), G, Mo, 0, natural=True, transposed=True)

    def oracle(t):
        if mode == "triton":
            return R.quant_tile128(t) if gran == "tile" else R.quant_rowgroup128(t)
        if mode == "rne":
            return R.quant_tile128_rne(t) if gran == "tile" else R.quant_rowgroup128_rne(t)
        B, M, Kd = t.shape
        v = t.float().view(B, M // 128, 128, Kd // 128, 128) if gran == "tile" else t.float().view(B, M, Kd // 128, 128)
        am = v.abs().amax(dim=(2, 4) if gran == "tile" else 3, keepdim=True) + 1e-5
        sc = torch.full_like(am, 127.0) / am
        qq = torch.floor(v * sc + 0.5).to(torch.int8).view(B, M, Kd)
        return qq, sc.view(B, M // 128, Kd // 128) if gran == "tile" else sc.view(B, M, Kd // 128)

    q_ref, s_ref = oracle(x)
    _same(q, q_ref, "natural int8"); _same(s, s_ref, "natural scale")
    xt = x.transpose(1, 2).contiguous()
    qt_ref, st_ref = oracle(xt)
    _same(qt, qt_ref, "transposed int8"); _same(st, st_ref, "transposed scale")


def test_quant_row_modes_and_col_t():
    a, w, _ = make_inputs("dc_small")
    q, s = DC.triton_per_row_quant_3d(a.to(DEV))
    q_ref, s_ref = R.quant_row(a)
    _same(q, q_ref, "row int8"); _same(s, s_ref, "row scale")
    g = torch.Generator().manual_seed(11)
    w = (torch.randn(384, 1280, generator=g) * 0.02).to(torch.bfloat16)   # K not a power of two
    w[7] = 0
    q, s = BC.triton_per_token_quant(w.to(DEV))
    q_ref, s_ref = R.quant_token(w)
    _same(q, q_ref); _same(s, s_ref)
    q, s = BC.triton_per_token_quant(w.to(DEV), round="rne")
    q_ref, s_ref = R.quant_token_rne(w)
    _same(q, q_ref); _same(s, s_ref)
    qt, st = K.quant_col_t(w.to(DEV), L.QMODE_TRITON)          # W^T per input channel, for dX
    q_ref, s_ref = R.quant_token(w.t().contiguous())
    _same(qt, q_ref, "col_t int8"); _same(st, s_ref.view(-1), "col_t scale")
    qt, st = K.quant_col_t(w.to(DEV), L.QMODE_TRITON, hadamard=128)   # rotated along the rows of w (N)
    q_ref, s_ref = R.quant_token(R.hadamard(w.t().contiguous(), 128))
    _same(qt, q_ref, "rotated col_t int8"); _same(st, s_ref.view(-1), "rotated col_t scale")
    for had in (0, 128):   # the double_channel scale (127 / absmax as a reciprocal): transposed operands of its backward
        qt, st = K.quant_col_t(w.to(DEV), L.QMODE_ROWRCP, hadamard=had)
        wt = w.t().contiguous()
        q_ref, s_ref = R.quant_row((R.hadamard(wt, 128) if had else wt)[None])
        _same(qt, q_ref[0], f"rowrcp col_t int8, hadamard={had}"); _same(st, s_ref.view(-1), "rowrcp col_t scale")


@pytest.mark.parametrize("kind", ["tile128", "row128", "rowfull"])
def test_hadamard_fused_quantizers(kind):
    g = torch.Generator().manual_seed(13)
    if kind == "rowfull":
        x = torch.randn(2, 128, 2048, generator=g).to(torch.bfloat16)
        q, s = DC.triton_per_row_quant_3d(x.to(DEV), hadamard="full")
        q_ref, s_ref = R.quant_row(R.hadamard(x))
    elif kind == "row128":
        x = (torch.randn(256, 640, generator=g) * 0.02).to(torch.bfloat16)
        q, s = BC.triton_per_token_quant(x.to(DEV), hadamard=128)
        q_ref, s_ref = R.quant_token(R.hadamard(x, 128))
    else:
        x = torch.randn(2, 256, 384, generator=g).to(torch.bfloat16)
        q, s = BC.triton_per_block_quant(x.to(DEV), hadamard=128)
        q_ref, s_ref = R.quant_tile128(R.hadamard(x, 128))
    # same butterfly order as the oracle -> bit-equal; a different FWHT order could differ by 1 LSB on ties
    _same(q, q_ref, "rotated int8"); _same(s, s_ref, "rotated scale")


# ------------------------------------------------------------------------------ int32 accumulators
@pytest.mark.parametrize("shape", [(1, 128, 128, 128), (1, 128, 256, 256), (2, 256, 384, 640),
                                   (1, 2048, 4096, 512), (3, 128, 128, 1152)])
@pytest.mark.parametrize("b_batched", [False, True])
def test_gemm_int32_accumulators_bit_exact(shape, b_batched):
    B, M, N, Kd = shape
    g = torch.Generator().manual_seed(B * 1000 + M + N + Kd)
    aq = _randq(g, B, M, Kd)
    bq = _randq(g, B, N, Kd) if b_batched else _randq(g, N, Kd)
    st = _status()
    out = K.gemm_dump_i32(aq.to(DEV), bq.to(DEV), per_block=False, status=st)
    assert st.item() == 0
    _same(out, R.gemm_i32(aq, bq), "whole-K int32")
    outb = K.gemm_dump_i32(aq.to(DEV), bq.to(DEV), per_block=True, status=st)
    assert st.item() == 0
    ref = torch.stack([R.gemm_i32(aq[:, :, k:k + 128].contiguous(), bq[..., k:k + 128].contiguous())
                       for k in range(0, Kd, 128)], dim=1)
    _same(outb, ref, "per-K-block int32")


def test_gemm_int32_extreme_values():
    """All operands at +-127/-128: partial sums reach 128*128*128 per K block, K*16129 overall."""
    aq = torch.full((1, 128, 1024), -128, dtype=torch.int8)
    bq = torch.full((256, 1024), -128, dtype=torch.int8)
    bq[::2] = 127
    out = K.gemm_dump_i32(aq.to(DEV), bq.to(DEV))
    _same(out, R.gemm_i32(aq, bq))


# ------------------------------------------------------------------------------ scaled GEMMs
@pytest.mark.parametrize("case", ["small", "edge"])
def test_block_channel_exact_mode_equals_reference_kernels(golden_dir, case):
    g = _golden(golden_dir, "block_channel_" + case)
    a, w, b3 = make_inputs(case)
    aq, a_s = BC.triton_per_block_quant(a.to(DEV))
    wq, w_s = BC.triton_per_token_quant(w.to(DEV))
    c = BC.triton_gemm(aq, wq, a_s, w_s, out_dtype=torch.float32, exact=True)
    _same(c, g["c_fwd"], "fwd fp32 vs reference kernel output")
    bq, b_s = BC.triton_per_block_quant(b3.to(DEV))
    c2 = BC.triton_gemm(aq, bq, a_s, b_s, out_dtype=torch.float32, exact=True)
    _same(c2, g["c_bwd"], "bwd fp32 vs reference kernel output")
    # default (fast) path: same integers, scale factors regrouped -> within tolerance, bf16 output
    y = BC.fwd_32(a.to(DEV), w.to(DEV))
    assert R.rel_fro(y.cpu().float(), torch.as_tensor(g["c_fwd"])) < TOL_BF16
    y2 = BC.bwd_33(a.to(DEV), b3.to(DEV))
    assert R.rel_fro(y2.cpu().float(), torch.as_tensor(g["c_bwd"])) < TOL_BF16
    _same(BC.fwd_32(a.to(DEV), w.to(DEV), exact=True), torch.as_tensor(g["c_fwd"]).to(torch.bfloat16), "bf16 exact")


def test_block_channel_config1_both_wordings():
    """The 512x1024x1024 configuration (8 outlier columns): reference scaling (tile128, half up) and the
    per-(row,128)/RNE wording, forward + dX + dW by composition of the two primitives."""
    a, w, dy = make_inputs("c1")
    x = a[0]
    y_ref, dx_ref, dw_ref = R.linear_block_channel(x, w, dy[0])
    xd, wd, dyd = x.to(DEV), w.to(DEV), dy[0].to(DEV)
    y = BC.fwd_32(xd[None], wd)[0]
    dx = BC.fwd_32(dyd[None], wd.t().contiguous())[0]
    dw = BC.bwd_33(dyd.t().contiguous()[None], xd.t().contiguous()[None])[0]
    for got, ref, name in ((y, y_ref, "Y"), (dx, dx_ref, "dX"), (dw, dw_ref, "dW")):
        err = R.rel_fro(got.cpu().float(), ref.float())
        assert err < TOL_BF16, f"{name}: rel fro {err}"
    # row128 / rne wording
    aq, a_s = R.quant_rowgroup128_rne(a)
    wq, w_s = R.quant_token_rne(w)
    ref = R.gemm_block_general(aq, wq, a_s, w_s.view(-1), 1, "channel").to(torch.bfloat16)
    got = BC.fwd_32(xd[None], wd, scaling="row128", round="rne")
    assert R.rel_fro(got.cpu().float(), ref.float()) < TOL_BF16
    got_exact = BC.fwd_32(xd[None], wd, scaling="row128", round="rne", exact=True)
    _same(got_exact, ref, "row128/rne exact bf16")


def test_double_channel_matches_reference_kernels(golden_dir):
    g = _golden(golden_dir, "double_channel_small")
    a, w, b3 = make_inputs("dc_small")
    aq, a_s = DC.triton_per_row_quant_3d(a.to(DEV))
    wq, w_s = DC.triton_per_row_quant_2d(w.to(DEV))
    _same(aq, g["aq"]); _same(a_s, g["a_s"]); _same(wq, g["wq"]); _same(w_s, g["w_s"])
    _same(DC.triton_gemm(aq, wq, a_s, w_s, out_dtype=torch.float32), g["c_fwd"], "fwd fp32")
    bq, b_s = DC.triton_per_row_quant_3d(b3.to(DEV))
    _same(DC.triton_gemm(aq, bq, a_s, b_s, out_dtype=torch.float32), g["c_bwd"], "bwd fp32")
    # whole pipeline incl. the rotation and the bf16 `C * 1/K` pass, against the oracle
    _same(DC.fwd_32(a.to(DEV), w.to(DEV)), R.double_channel_fwd_32(a, w), "fwd_32 bf16")
    _same(DC.bwd_33(a.to(DEV), b3.to(DEV)), R.double_channel_bwd_33(a, b3), "bwd_33 bf16")
    _same(DC.fwd_32(a.to(DEV), w.to(DEV), hadamard=None), R.double_channel_fwd_32(a, w, use_hadamard=False))


def test_fused_matches_reference_kernels(golden_dir):
    g = _golden(golden_dir, "fused_small")
    a, w, b3 = make_inputs("small")
    _same(FU.fused_int8_gemm(a.to(DEV), w.to(DEV), out_dtype=torch.float32, exact=True), g["c_fwd"], "fused fwd fp32")
    _same(FU.fused_int8_gemm(a.to(DEV), b3.to(DEV), out_dtype=torch.float32, exact=True), g["c_bwd"], "fused bwd fp32")
    # default (fast) path: reciprocal instead of division, fused accumulation
    for got, ref in ((FU.fused_int8_gemm(a.to(DEV), w.to(DEV), out_dtype=torch.float32), g["c_fwd"]),
                     (FU.fused_int8_gemm(a.to(DEV), b3.to(DEV), out_dtype=torch.float32), g["c_bwd"])):
        assert R.rel_fro(got.cpu(), torch.as_tensor(ref)) < 1e-5
    assert R.rel_fro(FU.fwd_32(a.to(DEV), w.to(DEV)).cpu().float(), torch.as_tensor(g["c_fwd"])) < TOL_BF16
    assert R.rel_fro(FU.bwd_33(a.to(DEV), b3.to(DEV)).cpu().float(), torch.as_tensor(g["c_bwd"])) < TOL_BF16


def test_reference_acceptance_gate():
    """calc_diff < 1e-3 against the bf16 product on N(0,1) inputs: the reference's own check
    (triton/block_channel_fwd32.py:257-272 and siblings), at 2 x 1024^3."""
    g = torch.Generator().manual_seed(3)
    a = torch.randn(2, 1024, 1024, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(1024, 1024, generator=g).to(torch.bfloat16).to(DEV)
    b3 = torch.randn(2, 1024, 1024, generator=g).to(torch.bfloat16).to(DEV)
    ref_f = torch.matmul(a, w.t())
    ref_b = torch.matmul(a, b3.transpose(1, 2))
    for mod in (BC, DC, FU):
        assert mod.calc_diff(mod.fwd_32(a, w), ref_f) < 1e-3
        assert mod.calc_diff(mod.bwd_33(a, b3), ref_b) < 1e-3


def test_bias_and_hadamard128_forward():
    g = torch.Generator().manual_seed(5)
    x = torch.randn(1, 256, 512, generator=g).to(torch.bfloat16)
    w = (torch.randn(384, 512, generator=g) * 0.02).to(torch.bfloat16)
    bias = (torch.randn(384, generator=g) * 0.01).to(torch.bfloat16)
    y_ref, _, _ = R.linear_block_channel(x[0], w, torch.zeros(256, 384, dtype=torch.bfloat16), hadamard128=True, bias=bias)
    y = BC.fwd_32(x.to(DEV), w.to(DEV), hadamard=128, bias=bias.to(DEV))[0]
    assert R.rel_fro(y.cpu().float(), y_ref.float()) < TOL_BF16
    y = BC.fwd_32(x.to(DEV), w.to(DEV), hadamard=128, bias=bias.to(DEV), exact=True)[0]
    _same(y, y_ref, "hadamard128 + bias, exact order")


# ------------------------------------------------------------------------------ error behaviour
def test_errors_are_reported_not_swallowed():
    from triton_int8_b200 import I8LError
    x = torch.zeros(1, 100, 128, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(I8LError, match="SHAPE"):
        BC.triton_per_block_quant(x)
    with pytest.raises(ValueError):
        BC.triton_per_block_quant(torch.zeros(1, 128, 128, dtype=torch.bfloat16))   # CPU tensor: no fallback
    with pytest.raises(TypeError):
        BC.triton_per_block_quant(torch.zeros(1, 128, 128, device=DEV))             # fp32 input


@pytest.mark.parametrize("gran", ["tile", "group"])
def test_hadamard_along_tokens_for_transposed_operand(gran):
    """The dW operands are x^T rotated along the tokens (rows of x): bit-equal to the oracle applied to
    the materialised transpose."""
    g = torch.Generator().manual_seed(17)
    x = (torch.randn(2, 256, 384, generator=g) * 2).to(torch.bfloat16)
    x[0, 3, 5] = 60.0
    G = L.GRAN_TILE128 if gran == "tile" else L.GRAN_GROUP128
    _, _, qt, st = K.quant_tile(x.to(DEV), G, L.QMODE_TRITON, 128, natural=False, transposed=True)
    xt_rot = R.hadamard(x.transpose(1, 2).contiguous(), 128)
    q_ref, s_ref = R.quant_tile128(xt_rot) if gran == "tile" else R.quant_rowgroup128(xt_rot)
    _same(qt, q_ref, "rotated transposed int8"); _same(st, s_ref, "rotated transposed scale")


# ------------------------------------------------------------------------------ TileLang variant numerics
@pytest.mark.parametrize("case", ["small", "edge"])
def test_tilelang_variant_quantizers_and_gemm(golden_dir, case):
    """scaling="tile128x256_bf16scale": activation scale per 128 x 256, scales rounded to bf16, scale
    product first (tilelang/block_channel_fwd.py:33,75-81,185-204).  The quantizers are checked against
    the reference's own Triton kernels (golden, unrounded scales + the bf16 rounding a GPU store applies),
    the GEMM against the cited restatement."""
    g = _golden(golden_dir, "tilelang_quantizers")
    a, w, b3 = make_inputs(case)
    aq, a_s = BC.triton_per_block256_quant(a.to(DEV))
    wq, w_s = BC.triton_per_token_quant_bf16scale(w.to(DEV))
    _same(aq, g[f"{case}__aq"], "128x256 int8"); _same(wq, g[f"{case}__wq"], "row int8")
    _same(a_s, torch.as_tensor(g[f"{case}__a_s_f32"]).to(torch.bfloat16).float(), "128x256 scale (bf16-rounded)")
    _same(w_s, torch.as_tensor(g[f"{case}__w_s_f32"]).to(torch.bfloat16).float(), "row scale (bf16-rounded)")
    ref = R.tilelang_fwd_32(a, w, return_fp32=True)
    got = BC.fwd_32(a.to(DEV), w.to(DEV), scaling="tile128x256_bf16scale", exact=True, out_dtype=torch.float32)
    _same(got, ref, "TileLang forward numerics, exact order, fp32")
    fast = BC.fwd_32(a.to(DEV), w.to(DEV), scaling="tile128x256_bf16scale")
    assert R.rel_fro(fast.cpu().float(), ref) < TOL_BF16
    ref_b = R.tilelang_bwd_33(a, b3, return_fp32=True)
    got_b = BC.bwd_33(a.to(DEV), b3.to(DEV), scaling="tilelang_tile128", exact=True, out_dtype=torch.float32)
    _same(got_b, ref_b, "TileLang backward numerics, exact order, fp32")
    assert R.rel_fro(BC.bwd_33(a.to(DEV), b3.to(DEV), scaling="tilelang_tile128").cpu().float(), ref_b) < TOL_BF16


def test_rowcol_fp32_output_applies_post_scale_and_bias():
    """double_channel pipeline with an fp32 result: the 1/K rescale and the bias are applied in fp32
    (the reference multiplies its GEMM output, whatever its type, by 1/K:
    triton/double-channle_fwd32.py:284)."""
    a, w, _ = make_inputs("dc_small")
    bias = (torch.arange(w.shape[0], dtype=torch.float32) * 1e-3).to(torch.bfloat16)
    for had in ("full", 128, None):
        rot = (lambda t: R.hadamard(t)) if had == "full" else ((lambda t: R.hadamard(t, 128)) if had == 128 else (lambda t: t))
        aq, a_s = R.quant_row(rot(a)); wq, w_s = R.quant_row(rot(w))
        post = 1.0 / a.shape[-1] if had == "full" else (1.0 / 128 if had == 128 else 1.0)
        ref = R.gemm_rowcol(aq, wq, a_s, w_s) * post + bias.float()
        got = DC.int8_gemm_pipeline(a.to(DEV), w.to(DEV), out_dtype=torch.float32, hadamard=had, bias=bias.to(DEV))
        _same(got, ref, f"fp32 double_channel pipeline, hadamard={had}")


@pytest.mark.parametrize("mode", ["triton", "rne"])
def test_rotated_operand_pair_from_one_read(mode):
    """hadamard=128 with both outputs requested: q (rotated along the columns) and qt (the transpose,
    rotated along the rows) come from one kernel that reads each tile once; both must equal the oracle,
    and the two single-output kernels, bit for bit."""
    g = torch.Generator().manual_seed(23)
    x = (torch.randn(2, 384, 256, generator=g) * 2).to(torch.bfloat16)
    x[0, :128, :128] = 0
    x[1, 130, 7] = -90.0
    x[0, 200:210, 129] = 33.0
    Mo = L.QMODE_TRITON if mode == "triton" else L.QMODE_RNE
    oracle = R.quant_tile128 if mode == "triton" else R.quant_tile128_rne
    q, s, qt, st = K.quant_tile(x.to(DEV), L.GRAN_TILE128, Mo, 128, natural=True, transposed=True)
    q_ref, s_ref = oracle(R.hadamard(x, 128))
    qt_ref, st_ref = oracle(R.hadamard(x.transpose(1, 2).contiguous(), 128))
    _same(q, q_ref, "q"); _same(s, s_ref, "scale"); _same(qt, qt_ref, "qt"); _same(st, st_ref, "scale_t")
    q1, s1, _, _ = K.quant_tile(x.to(DEV), L.GRAN_TILE128, Mo, 128, natural=True, transposed=False)
    _, _, qt1, st1 = K.quant_tile(x.to(DEV), L.GRAN_TILE128, Mo, 128, natural=False, transposed=True)
    assert torch.equal(q, q1) and torch.equal(s, s1) and torch.equal(qt, qt1) and torch.equal(st, st1)


@pytest.mark.parametrize("spread", ["smooth", "wild"])
def test_fast_block_epilogue_accuracy_deep_k(spread):
    """The fast block-scaled epilogue turns the int32 partials into floats by an integer add of a magic
    number and lets the accumulators carry a bounded multiple of that number, removed at the tile end.
    At K = 32768 (256 K blocks), with per-tile scales that are smooth or jump by three decades from one
    K block to the next, the fp32 result must stay within 1e-4 (relative Frobenius) of the float64 value of
    sum_kb P_kb * a_s * b_s, like the reference-order mode."""
    M, N, Kd = 256, 512, 32768
    g = torch.Generator().manual_seed(41)
    aq, bq = _randq(g, 1, M, Kd), _randq(g, N, Kd)
    if spread == "smooth":
        a_s = torch.rand(1, M // 128, Kd // 128, generator=g) * 0.5 + 0.75
    else:
        a_s = 10.0 ** (torch.rand(1, M // 128, Kd // 128, generator=g) * 3.0 - 1.5)
    b_s = torch.rand(N, generator=g) + 0.5
    ref = torch.zeros(M, N, dtype=torch.float64)
    for kb in range(Kd // 128):
        P = R.int_mm(aq[0, :, kb * 128:(kb + 1) * 128], bq[:, kb * 128:(kb + 1) * 128]).double()
        ref += P * a_s[0, :, kb].double().repeat_interleave(128).view(M, 1)
    ref *= b_s.double().view(1, N)
    args = (aq.to(DEV), bq.to(DEV), a_s.to(DEV), b_s.to(DEV))
    fast = K.gemm_block(*args, flags=L.GEMM_OUT_F32)[0].cpu().double()
    exact = K.gemm_block(*args, flags=L.GEMM_OUT_F32 | L.GEMM_EXACT_ORDER)[0].cpu().double()
    e_fast, e_exact = R.rel_fro(fast, ref), R.rel_fro(exact, ref)
    assert e_exact < 1e-6, e_exact
    assert e_fast < 1e-4, (e_fast, e_exact)
    # tile x tile scales (the dW layout) through the same kind
    b_t = torch.rand(N // 128, Kd // 128, generator=g) + 0.5
    ref2 = torch.zeros(M, N, dtype=torch.float64)
    for kb in range(Kd // 128):
        P = R.int_mm(aq[0, :, kb * 128:(kb + 1) * 128], bq[:, kb * 128:(kb + 1) * 128]).double()
        ref2 += P * a_s[0, :, kb].double().repeat_interleave(128).view(M, 1) * b_t[:, kb].double().repeat_interleave(128).view(1, N)
    fast2 = K.gemm_block(args[0], args[1], args[2], b_t.to(DEV), b_kind=L.BSCALE_TILE, flags=L.GEMM_OUT_F32)[0].cpu().double()
    assert R.rel_fro(fast2, ref2) < 1e-4


def test_single_kernel_fused_matches_reference_kernels(golden_dir):
    """i8l_fused_gemm: bf16 in, result out, operand tiles quantized inside the GEMM.  Reference operation
    order: bit-equal to the reference's fused kernels (golden); default order: equal to the two-step path."""
    g = _golden(golden_dir, "fused_small")
    a, w, b3 = make_inputs("small")
    ad, wd, bd = a.to(DEV), w.to(DEV), b3.to(DEV)
    _same(FU.fused_int8_gemm(ad, wd, out_dtype=torch.float32, exact=True, single_kernel=True), g["c_fwd"], "single-kernel fwd fp32")
    _same(FU.fused_int8_gemm(ad, bd, out_dtype=torch.float32, exact=True, single_kernel=True), g["c_bwd"], "single-kernel bwd fp32")
    for other in (wd, bd):
        one = FU.fused_int8_gemm(ad, other, out_dtype=torch.float32, single_kernel=True)
        two = FU.fused_int8_gemm(ad, other, out_dtype=torch.float32)
        assert R.rel_fro(one.cpu(), two.cpu()) < 1e-6
        assert torch.equal(FU.fused_int8_gemm(ad, other, single_kernel=True), FU.fused_int8_gemm(ad, other).to(torch.bfloat16)) or \
            R.rel_fro(FU.fused_int8_gemm(ad, other, single_kernel=True).cpu().float(), two.cpu()) < TOL_BF16
    # a shape with more tiles than SMs and a deeper K, against the exact product (the reference's gate)
    gen = torch.Generator().manual_seed(9)
    a2 = torch.randn(1, 2048, 2048, generator=gen).to(torch.bfloat16).to(DEV)
    w2 = torch.randn(1536, 2048, generator=gen).to(torch.bfloat16).to(DEV)
    y = FU.fwd_32(a2, w2, single_kernel=True)
    assert FU.calc_diff(y, torch.matmul(a2, w2.t())) < 1e-3
    assert R.rel_fro(y.cpu().float(), FU.fwd_32(a2, w2).cpu().float()) < 1e-2
    K.check_status(DEV)


def test_fast_block_epilogue_more_than_512_k_blocks():
    """K = 73728 = 576 K blocks: the factors of a tile are handed over in two chunks (512 + 64); int32
    partials via the dump entry, fp32 result against float64."""
    M, N, Kd = 128, 256, 128 * 576
    g = torch.Generator().manual_seed(43)
    aq, bq = _randq(g, 1, M, Kd), _randq(g, N, Kd)
    a_s = torch.rand(1, 1, Kd // 128, generator=g) + 0.5
    b_s = torch.rand(N, generator=g) + 0.5
    P = K.gemm_dump_i32(aq.to(DEV), bq.to(DEV), per_block=True)[0].cpu()          # [KB, M, N]
    ref = (P.double() * a_s[0, 0].double().view(-1, 1, 1)).sum(0) * b_s.double().view(1, N)
    for b_scale, kind in ((b_s, L.BSCALE_CHANNEL),):
        fast = K.gemm_block(aq.to(DEV), bq.to(DEV), a_s.to(DEV), b_scale.to(DEV), b_kind=kind, flags=L.GEMM_OUT_F32)[0].cpu().double()
        assert R.rel_fro(fast, ref) < 1e-4
    K.check_status(DEV)


@pytest.mark.parametrize("cols", [384, 8192, 8192 + 384])
def test_rotated_row_quantizer_both_kernels(cols):
    """Per-row scale with the 128-point rotation: rows of up to 8192 elements take the kernel that keeps the
    rotated row in registers, longer rows the two-sweep kernel; both must equal the oracle bit for bit."""
    g = torch.Generator().manual_seed(cols)
    w = (torch.randn(160, cols, generator=g) * 0.05).to(torch.bfloat16)
    w[3] = 0
    w[7, cols - 1] = 9.0
    q, s = K.quant_row(w.to(DEV), L.QMODE_TRITON, 128)
    q_ref, s_ref = R.quant_token(R.hadamard(w, 128))
    _same(q, q_ref, "rotated row int8"); _same(s, s_ref.view(-1), "rotated row scale")
