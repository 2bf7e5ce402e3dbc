"""Full-size runs of the BASELINE configurations on the GPU, checked through properties that do not
need a full CPU recomputation: quantisation groups are local (a row, or a 128x128 tile), so the oracle
evaluated on a slice of rows / tiles must reproduce the same slice of the full-size GPU result."""
import pytest
import torch

from oracle import ref_semantics as R

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = 1e-2

if torch.cuda.is_available():
    from triton_int8_b200 import block_channel as BC
    from triton_int8_b200 import double_channel as DC
    from triton_int8_b200 import kernels as K, _lib as L
    from triton_int8_b200.linear import Int8Config, linear_backward, linear_forward


def _gen(shape, seed, std=1.0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return torch.randn(*shape, device=DEV, generator=g) * std


def test_config2_double_channel_forward_full_size():
    """X [8192,4096] ~N(0,1) with 0.5 % outlier channels x30, W [4096,4096] ~N(0,0.02), bias ~N(0,0.01)."""
    M, Kd, N = 8192, 4096, 4096
    x = _gen((M, Kd), 20260001)
    cols = torch.randperm(Kd, device=DEV, generator=torch.Generator(device=DEV).manual_seed(1))[:21]
    x[:, cols] *= 30
    x = x.to(torch.bfloat16)
    w = _gen((N, Kd), 20260002, 0.02).to(torch.bfloat16)
    bias = _gen((N,), 20260003, 0.01).to(torch.bfloat16)
    for had in ("full", None):
        y = DC.fwd_32(x[None], w, hadamard=had, bias=bias)[0]
        rows = torch.arange(0, M, 67, device=DEV)[:96]               # per-token scales: any row subset is exact
        xs, ws = x[rows].cpu(), w.cpu()
        c = R.double_channel_fwd_32(xs[None], ws, use_hadamard=had is not None)[0]
        ref = (c.float() + bias.cpu().float()).to(torch.bfloat16)
        assert torch.equal(y[rows].cpu(), ref), f"hadamard={had}: {(y[rows].cpu() != ref).sum().item()} entries differ"
        exact = x.float() @ w.float().t() + bias.float()
        diff = R.calc_diff(y.float(), exact).item()
        if had == "full":       # the rotation spreads the outlier channels: the reference's gate holds
            assert diff < 1e-3
        else:                   # plain per-token scaling on outlier data is what the rotation is for
            assert diff < 2e-2


@pytest.mark.parametrize("n", [2048, 4096, 8192])
def test_config2_square_sweep(n):
    a = _gen((1, n, n), n).to(torch.bfloat16)
    w = _gen((n, n), n + 1, 0.02).to(torch.bfloat16)
    y = DC.fwd_32(a, w)
    assert R.calc_diff(y.float(), a.float() @ w.float().t()) < 1e-3
    y2 = BC.fwd_32(a, w)
    assert R.calc_diff(y2.float(), a.float() @ w.float().t()) < 1e-3


def test_config3_hadamard_block_channel_full_size():
    """M=16384, K=4096, N=11008; X ~N(0,1) with 1e-3 of the entries replaced by 10*t3 outliers;
    128-point rotation + block_channel; forward, dX and dW."""
    M, Kd, N = 16384, 4096, 11008
    g = torch.Generator(device=DEV).manual_seed(20260002)
    x = torch.randn(M, Kd, device=DEV, generator=g)
    mask = torch.rand(M, Kd, device=DEV, generator=g) < 1e-3
    t3 = torch.randn(M, Kd, device=DEV, generator=g) / torch.sqrt(
        (torch.randn(3, M, Kd, device=DEV, generator=g) ** 2).mean(0))
    x = torch.where(mask, 10 * t3, x).to(torch.bfloat16)
    del t3, mask
    w = _gen((N, Kd), 5, 0.02).to(torch.bfloat16)
    dy = _gen((M, N), 6, 1e-3).to(torch.bfloat16)
    cfg = Int8Config(hadamard=128)
    y, saved = linear_forward(x, w, None, cfg)
    dx, dw = linear_backward(dy, w, saved, cfg)
    # forward: two 128-row blocks against the oracle (tile scales are local to the block)
    rb = slice(128 * 7, 128 * 9)
    rot = lambda t: R.hadamard(t, 128)
    y_ref = (R.block_channel_fwd_32(rot(x[rb].cpu())[None], rot(w.cpu()), return_fp32=True)[0] / 128).to(torch.bfloat16)
    assert R.rel_fro(y[rb].cpu().float(), y_ref.float()) < TOL
    # dX: same row blocks of dY against the oracle (W^T per-input-channel scales need the whole W)
    wt = w.t().contiguous().cpu()
    dx_ref = (R.block_channel_fwd_32(rot(dy[rb].cpu())[None], rot(wt), return_fp32=True)[0] / 128).to(torch.bfloat16)
    assert R.rel_fro(dx[rb].cpu().float(), dx_ref.float()) < TOL
    # dW (rotated along the tokens): one 128-channel block x two 128-wide K blocks, contraction over all M
    nb, kb = slice(128 * 3, 128 * 4), slice(128 * 5, 128 * 7)
    dw_ref = (R.block_channel_bwd_33(rot(dy[:, nb].t().contiguous().cpu())[None], rot(x[:, kb].t().contiguous().cpu())[None],
                                      return_fp32=True)[0] / 128).to(torch.bfloat16)
    assert R.rel_fro(dw[nb, kb].cpu().float(), dw_ref.float()) < TOL
    # all three against the exact products (the reference's own gate)
    assert R.calc_diff(y.float(), x.float() @ w.float().t()) < 1e-3
    assert R.calc_diff(dx.float(), dy.float() @ w.float()) < 1e-3
    assert R.calc_diff(dw.float(), dy.float().t() @ x.float()) < 1e-3


def test_config4_llama7b_layer_chain_full_tokens():
    """Seven linears of a Llama-2-7B decoder layer at M=8192, forward then backward, each checked on a
    row-block slice against the oracle and as a whole against the bf16 product."""
    M = 8192
    shapes = [(4096, 4096)] * 4 + [(4096, 11008)] * 2 + [(11008, 4096)]
    for i, (Kd, N) in enumerate(shapes):
        x = _gen((M, Kd), 100 + i).to(torch.bfloat16)
        w = _gen((N, Kd), 200 + i, 0.02).to(torch.bfloat16)
        dy = _gen((M, N), 300 + i, 1e-3).to(torch.bfloat16)
        y, saved = linear_forward(x, w, None)
        dx, dw = linear_backward(dy, w, saved)
        rb = slice(128 * (i + 1), 128 * (i + 2))
        y_ref = R.block_channel_fwd_32(x[rb].cpu()[None], w.cpu())[0]
        assert R.rel_fro(y[rb].cpu().float(), y_ref.float()) < TOL
        assert R.calc_diff(y.float(), x.float() @ w.float().t()) < 1e-3
        assert R.calc_diff(dx.float(), dy.float() @ w.float()) < 1e-3
        assert R.calc_diff(dw.float(), dy.float().t() @ x.float()) < 1e-3


def test_int32_accumulators_at_scale_checksum():
    """8192 x 4096 x 8192 int8 GEMM: row and column checksums of the int32 result must equal the
    checksums computed from the operands in int64 (sum_n C[m,n] = A[m,:] . sum_n B[n,:])."""
    M, N, Kd = 8192, 4096, 8192
    g = torch.Generator(device=DEV).manual_seed(9)
    a = torch.randint(-127, 128, (1, M, Kd), device=DEV, dtype=torch.int8, generator=g)
    b = torch.randint(-127, 128, (N, Kd), device=DEV, dtype=torch.int8, generator=g)
    c = K.gemm_dump_i32(a, b)[0].to(torch.int64)
    # fp64 is exact here: |values| < 2^53
    row_ck = a[0].double() @ b.double().sum(0)
    col_ck = a[0].double().sum(0) @ b.double().t()
    assert torch.equal(c.sum(1).double(), row_ck) and torch.equal(c.sum(0).double(), col_ck)
