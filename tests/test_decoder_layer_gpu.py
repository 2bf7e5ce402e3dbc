"""A Llama-2-7B-shaped decoder layer at M = 8192 tokens whose seven linears run through the INT8 path,
chained: every linear's input is the previous linear's output after the block's glue (norm, attention,
SiLU gate, residual), and its dY is the real upstream gradient.  Checked (a) per linear, on the
activations and gradients that actually flowed, against the CPU oracle on a row block; (b) end to end
against a bf16 nn.Linear twin with the same weights."""
import pytest
import torch

from oracle import ref_semantics as R

pytestmark = pytest.mark.gpu
DEV = "cuda"

if torch.cuda.is_available():
    from triton_int8_b200 import kernels as K
    from triton_int8_b200.decoder_layer import DecoderLayer


def _layers(hidden, heads, mlp, seed=0):
    torch.manual_seed(seed)
    q = DecoderLayer(hidden, heads, mlp, device=DEV)
    ref = DecoderLayer(hidden, heads, mlp, device=DEV, linear_cls=torch.nn.Linear)
    ref.load_state_dict(q.state_dict())
    return q, ref


@pytest.mark.parametrize("hidden,heads,mlp,batch,seq", [(512, 4, 1408, 2, 256), (4096, 32, 11008, 4, 2048)])
def test_decoder_layer_chain_forward_backward(hidden, heads, mlp, batch, seq):
    layer, twin = _layers(hidden, heads, mlp)
    g = torch.Generator(device=DEV).manual_seed(1)
    x = torch.randn(batch, seq, hidden, device=DEV, generator=g).to(torch.bfloat16)
    dout = (torch.randn(batch, seq, hidden, device=DEV, generator=g) * 1e-3).to(torch.bfloat16)

    seen = {}

    def keep(name):
        def fwd_hook(mod, inp, out):
            seen[name] = [inp[0].detach(), out.detach(), None]
            out.register_hook(lambda grad, n=name: seen[n].__setitem__(2, grad.detach()))
        return fwd_hook

    for name, lin in layer.linears().items():
        lin.register_forward_hook(keep(name))
    xq = x.clone().requires_grad_(True)
    out = layer(xq)
    out.backward(dout)
    K.check_status(DEV)
    xr = x.clone().requires_grad_(True)
    out_ref = twin(xr)
    out_ref.backward(dout)

    # (a) each linear on what actually flowed through it: a 256-row block of Y and dX against the oracle
    rb = slice(256, 512)
    for name, lin in layer.linears().items():
        inp, y, dy = seen[name]
        inp2, y2, dy2 = inp.reshape(-1, inp.shape[-1]), y.reshape(-1, y.shape[-1]), dy.reshape(-1, dy.shape[-1])
        w = lin.weight.detach()
        y_ref = R.block_channel_fwd_32(inp2[rb].cpu()[None], w.cpu())[0]
        assert R.rel_fro(y2[rb].cpu().float(), y_ref.float()) < 1e-2, name
        # the reference's gate on the chained activations (post-norm, attention output, SiLU-gated product)
        assert R.calc_diff(y2.float(), inp2.float() @ w.float().t()) < 1e-3, name
        assert R.calc_diff(lin.weight.grad.float(), dy2.float().t() @ inp2.float()) < 1e-3, name

    # (b) the whole block against its bf16 twin: output, input gradient and all seven weight gradients
    assert R.calc_diff(out.float(), out_ref.float()) < 1e-3
    assert R.calc_diff(xq.grad.float(), xr.grad.float()) < 2e-3
    for name, lin in layer.linears().items():
        d = R.calc_diff(lin.weight.grad.float(), getattr(twin, name).weight.grad.float()).item()
        assert d < 5e-3, (name, d)
