"""Int8Linear / autograd against the oracle's composition of fwd_32 and bwd_33 (GPU)."""
import pytest
import torch

from oracle import ref_semantics as R

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = 1e-2

if torch.cuda.is_available():
    from triton_int8_b200.linear import Int8Config, Int8Linear, linear_backward, linear_forward


def _data(M, K, N, seed=0, outliers=True):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g)
    if outliers:
        x[:, torch.randperm(K, generator=g)[:4]] *= 20
    w = torch.randn(N, K, generator=g) * 0.02
    dy = torch.randn(M, N, generator=g) * 1e-3
    b = torch.randn(N, generator=g) * 0.01
    return [t.to(torch.bfloat16) for t in (x, w, dy, b)]


@pytest.mark.parametrize("shape", [(256, 512, 384), (512, 1024, 1024), (1024, 384, 640)])
def test_linear_fwd_bwd_matches_oracle(shape):
    M, K, N = shape
    x, w, dy, b = _data(M, K, N)
    y_ref, dx_ref, dw_ref = R.linear_block_channel(x, w, dy, bias=b)
    lin = Int8Linear(K, N, bias=True, device=DEV)
    with torch.no_grad():
        lin.weight.copy_(w); lin.bias.copy_(b)
    xd = x.to(DEV).requires_grad_(True)
    y = lin(xd)
    y.backward(dy.to(DEV))
    assert R.rel_fro(y.cpu().float(), y_ref.float()) < TOL
    assert R.rel_fro(xd.grad.cpu().float(), dx_ref.float()) < TOL
    assert R.rel_fro(lin.weight.grad.cpu().float(), dw_ref.float()) < TOL
    assert torch.allclose(lin.bias.grad.float().cpu(), dy.float().sum(0), rtol=2e-2, atol=1e-4)


def test_linear_exact_mode_is_bit_equal_to_oracle():
    M, K, N = 256, 512, 384
    x, w, dy, _ = _data(M, K, N, seed=4)
    cfg = Int8Config(exact=True)
    y_ref, dx_ref, dw_ref = R.linear_block_channel(x, w, dy)
    y, saved = linear_forward(x.to(DEV), w.to(DEV), None, cfg)
    dx, dw = linear_backward(dy.to(DEV), w.to(DEV), saved, cfg)
    assert torch.equal(y.cpu(), y_ref) and torch.equal(dx.cpu(), dx_ref) and torch.equal(dw.cpu(), dw_ref)


def test_linear_3d_input_and_nn_linear_state_dict():
    lin_ref = torch.nn.Linear(256, 384, bias=True).to(torch.bfloat16)
    lin = Int8Linear.from_linear(lin_ref.to(DEV))
    assert set(lin.state_dict()) == set(lin_ref.state_dict())
    x = torch.randn(2, 64, 256, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = lin(x)
    assert y.shape == (2, 64, 384)
    y.float().square().mean().backward()
    assert x.grad.shape == x.shape and lin.weight.grad.shape == lin.weight.shape
    ref = torch.nn.functional.linear(x.detach(), lin.weight.detach(), lin.bias.detach())
    assert R.calc_diff(y.detach().cpu(), ref.cpu()) < 1e-3


def test_linear_hadamard128_forward_and_dx():
    M, K, N = 256, 512, 384
    x, w, dy, _ = _data(M, K, N, seed=9)
    cfg = Int8Config(hadamard=128)
    y, saved = linear_forward(x.to(DEV), w.to(DEV), None, cfg)
    dx, dw = linear_backward(dy.to(DEV), w.to(DEV), saved, cfg)
    rot = lambda t: R.hadamard(t, 128)
    y_ref = (R.block_channel_fwd_32(rot(x)[None], rot(w), return_fp32=True)[0] / 128).to(torch.bfloat16)
    dx_ref = (R.block_channel_fwd_32(rot(dy)[None], rot(w.t().contiguous()), return_fp32=True)[0] / 128).to(torch.bfloat16)
    dw_ref = (R.block_channel_bwd_33(rot(dy.t().contiguous())[None], rot(x.t().contiguous())[None],
                                      return_fp32=True)[0] / 128).to(torch.bfloat16)
    assert R.rel_fro(y.cpu().float(), y_ref.float()) < TOL
    assert R.rel_fro(dx.cpu().float(), dx_ref.float()) < TOL
    assert R.rel_fro(dw.cpu().float(), dw_ref.float()) < TOL
    # the rotation pays off on outlier-heavy inputs: closer to the exact product than without it
    exact = x.float() @ w.float().t()
    y0, _ = linear_forward(x.to(DEV), w.to(DEV), None, Int8Config())
    assert R.rel_fro(y.cpu().float(), exact) < R.rel_fro(y0.cpu().float(), exact)


def test_llama7b_layer_shapes_chain_small_tokens():
    """All seven linear shapes of a Llama-2-7B decoder layer (q,k,v,o 4096->4096, gate/up 4096->11008,
    down 11008->4096), forward then backward, at a reduced token count; outputs against the bf16 product
    with the reference's own gate (calc_diff < 1e-3)."""
    M = 256
    shapes = [(4096, 4096)] * 4 + [(4096, 11008)] * 2 + [(11008, 4096)]
    g = torch.Generator(device=DEV).manual_seed(2)
    for K, N in shapes:
        lin = Int8Linear(K, N, bias=False, device=DEV)
        x = torch.randn(M, K, device=DEV, generator=g).to(torch.bfloat16).requires_grad_(True)
        dy = (torch.randn(M, N, device=DEV, generator=g) * 1e-3).to(torch.bfloat16)
        y = lin(x)
        y.backward(dy)
        w = lin.weight.detach().float()
        assert R.calc_diff(y.detach().float(), x.detach().float() @ w.t()) < 1e-3
        assert R.calc_diff(x.grad.float(), dy.float() @ w) < 1e-3
        assert R.calc_diff(lin.weight.grad.float(), dy.float().t() @ x.detach().float()) < 1e-3


@pytest.mark.parametrize("had", [0, 128, -1])
def test_linear_double_channel_matches_oracle_composition(had):
    """scaling='double_channel': Y, dX and dW are the reference's double_channel product
    (triton/double-channle_fwd32.py:295-311) applied to (X, W), (dY, W^T) and (dY^T, X^T)."""
    from triton_int8_b200.linear import Int8Config, linear_backward, linear_forward
    M, Kd, N = 256, 512, 1024
    g = torch.Generator().manual_seed(5)
    x = torch.randn(M, Kd, generator=g).to(torch.bfloat16)
    x[:, ::61] *= 20
    w = (torch.randn(N, Kd, generator=g) * 0.02).to(torch.bfloat16)
    dy = (torch.randn(M, N, generator=g) * 1e-3).to(torch.bfloat16)
    bias = (torch.randn(N, generator=g) * 0.01).to(torch.bfloat16)

    def ref(a, b, with_bias=None):   # a [R, C], b [S, C] -> [R, S]
        if had == 128:
            aq, a_s = R.quant_row(R.hadamard(a[None], 128))
            bq, b_s = R.quant_row(R.hadamard(b, 128))
            c = R.gemm_rowcol(aq, bq, a_s, b_s).to(torch.bfloat16) * (1.0 / 128)
        else:
            c = R.double_channel_fwd_32(a[None], b, use_hadamard=had == -1)
        c = c[0]
        if with_bias is not None:   # bf16 result, then the bias added in fp32 and rounded again
            c = (c.float() + with_bias.float()).to(torch.bfloat16)
        return c

    cfg = Int8Config(scaling="double_channel", hadamard=had)
    y, saved = linear_forward(x.to(DEV), w.to(DEV), bias.to(DEV), cfg)
    dx, dw = linear_backward(dy.to(DEV), w.to(DEV), saved, cfg)
    assert torch.equal(y.cpu(), ref(x, w, bias))
    assert torch.equal(dx.cpu(), ref(dy, w.t().contiguous()))
    assert torch.equal(dw.cpu(), ref(dy.t().contiguous(), x.t().contiguous()))
    exact = dy.float() @ w.float()
    assert R.rel_fro(dx.cpu().float(), exact) < 5e-2
