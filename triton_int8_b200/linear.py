"""nn.Linear drop-in built on the INT8 kernels: Y, dX and dW each run as one quantize -> int8
tensor-core GEMM -> fused rescale pass.

The reference defines only the two primitives fwd_32 (3-D x 2-D) and bwd_33 (3-D x 3-D); a linear
layer is their composition
    Y  = fwd_32(X[1,M,K],   W[N,K])            (triton/block_channel_fwd32.py:252)
    dX = fwd_32(dY[1,M,N],  W^T[K,N])
    dW = bwd_33(dY^T[1,N,M], X^T[1,K,M])       (triton/block_channel_bwd33.py:175)
Here the transposed int8 operands dY^T and X^T come out of the same kernel launch that quantises
dY and X (128x128 tile scales are transposition invariant), and W^T is quantised per input channel
by a column-scaled transposing kernel, so no bf16 transpose is ever materialised.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn

from . import _lib as L
from . import kernels as K


@dataclass(frozen=True)
class Int8Config:
    """scaling: 'tile128' (reference block_channel), 'row128' (one scale per row and 128
    contraction elements) or 'double_channel' (one scale per row of each operand over the whole
    contraction axis, int32 accumulation over all of it: triton/double-channle_fwd32.py:295-311 applied
    to Y, dX and dW; hadamard may then also be -1 = rotate over the whole contraction axis, which must be
    a power of two <= 32768); round: 'half_up' (reference) or 'rne'; hadamard: 0 or 128 (rotate both
    operands of every GEMM in 128-wide groups along that GEMM's contraction axis: K for Y, N for dX,
    the tokens for dW; each product is rescaled by 1/128);
    exact: reproduce the reference's fp32 operation order bit for bit (slower)."""
    scaling: str = "tile128"
    round: str = "half_up"
    hadamard: int = 0
    exact: bool = False

    @property
    def gran(self) -> int:
        return {"tile128": L.GRAN_TILE128, "row128": L.GRAN_GROUP128, "double_channel": L.GRAN_ROW}[self.scaling]

    @property
    def qmode(self) -> int:
        return {"half_up": L.QMODE_TRITON, "rne": L.QMODE_RNE}[self.round]

    @property
    def a_kind(self) -> int:
        return L.ASCALE_TILE if self.scaling == "tile128" else L.ASCALE_GROUP

    @property
    def bt_kind(self) -> int:
        return L.BSCALE_TILE if self.scaling == "tile128" else L.BSCALE_GROUP

    @property
    def flags(self) -> int:
        return L.GEMM_EXACT_ORDER if self.exact else 0

    @property
    def post(self) -> float:
        return 1.0 / self.hadamard if self.hadamard else 1.0

    @property
    def whole_k(self) -> bool:
        return self.scaling == "double_channel"

    def post_for(self, contraction: int) -> float:
        """Rescale that undoes the rotation of both operands: 1/128, or 1/length for a whole-axis rotation."""
        if not self.hadamard:
            return 1.0
        return 1.0 / contraction if self.hadamard == L.HAD_FULL else 1.0 / self.hadamard


DEFAULT = Int8Config()


def linear_forward(x2: torch.Tensor, weight: torch.Tensor, bias, cfg: Int8Config = DEFAULT, want_xt: bool = True):
    """x2 bf16 [M, K], weight bf16 [N, K] -> (y bf16 [M, N], saved) where saved holds the int8 X^T
    operand for dW (or None when want_xt is False)."""
    if cfg.whole_k:
        return _dc_forward(x2, weight, bias, cfg, want_xt)
    # one call yields X (groups / rotation along K) and, for dW, X^T (along the tokens); with per-tile scales
    # both come from a single read of X, rotated or not
    xq, xs, xqt, xst = K.quant_tile(x2[None], cfg.gran, cfg.qmode, cfg.hadamard, natural=True, transposed=want_xt)
    wq, ws = K.quant_row(weight, cfg.qmode, cfg.hadamard)
    y = K.gemm_block(xq, wq, xs, ws, cfg.a_kind, L.BSCALE_CHANNEL, bias, cfg.post, cfg.flags)[0]
    return y, (xqt, xst)


def _dc_transposed(t2: torch.Tensor, cfg: Int8Config):
    """t2 bf16 [R, C] -> (int8 t2^T [1, C, R], fp32 scale [1, C]): one scale per column of t2 over all rows.
    The transposing quantizer does it without a bf16 transpose, rotated in 128-wide groups along R or not;
    only a rotation over the whole of R goes through a transposed copy and the row quantizer."""
    if cfg.hadamard in (0, 128):
        q, s = K.quant_col_t(t2, L.QMODE_ROWRCP, cfg.hadamard)
        return q[None], s[None]
    return K.quant_row(t2.t().contiguous()[None], L.QMODE_ROWRCP, cfg.hadamard)


def _dc_forward(x2, weight, bias, cfg: Int8Config, want_xt: bool):
    """double_channel forward: per-token and per-output-channel scales over all of K."""
    Kd = x2.shape[1]
    xq, xs = K.quant_row(x2[None], L.QMODE_ROWRCP, cfg.hadamard)
    wq, ws = K.quant_row(weight, L.QMODE_ROWRCP, cfg.hadamard)
    y = K.gemm_rowcol(xq, wq, xs, ws, bias, cfg.post_for(Kd))[0]
    saved = (None, None)
    if want_xt:   # dW operand: X^T [K, M], one scale per input feature over all tokens
        saved = _dc_transposed(x2, cfg)
    return y, saved


def quantize_grad_output(dy2: torch.Tensor, cfg: Int8Config = DEFAULT, need_dx: bool = True, need_dw: bool = True):
    """One pass over dY [M, N] that yields the dX operand (dY, groups along N) and the dW operand
    (dY^T, groups along M).  Returns ((dyq, dys), (dyqt, dyst)); a pair not requested is (None, None)."""
    if cfg.whole_k:
        dy_op = K.quant_row(dy2[None], L.QMODE_ROWRCP, cfg.hadamard) if need_dx else (None, None)
        dyt_op = _dc_transposed(dy2, cfg) if need_dw else (None, None)
        return dy_op, dyt_op
    dyq, dys, dyqt, dyst = K.quant_tile(dy2[None], cfg.gran, cfg.qmode, cfg.hadamard,
                                        natural=need_dx, transposed=need_dw)
    return (dyq, dys), (dyqt, dyst)


def grad_input(dy_op, weight: torch.Tensor, cfg: Int8Config = DEFAULT) -> torch.Tensor:
    """dX = dY W, bf16 [M, K]; W^T is quantised per input channel."""
    dyq, dys = dy_op
    if cfg.whole_k:   # W^T [K, N], one scale per input channel over all of N
        wtq, wts = _dc_transposed(weight, cfg)
        return K.gemm_rowcol(dyq, wtq[0], dys, wts[0], None, cfg.post_for(weight.shape[0]))[0]
    wtq, wts = K.quant_col_t(weight, cfg.qmode, cfg.hadamard)   # rotated along N when hadamard is on
    return K.gemm_block(dyq, wtq, dys, wts, cfg.a_kind, L.BSCALE_CHANNEL, None, cfg.post, cfg.flags)[0]


def grad_weight(dyt_op, saved_xt, cfg: Int8Config = DEFAULT) -> torch.Tensor:
    """dW = dY^T X, bf16 [N, K], both operands scaled in groups along M."""
    (dyqt, dyst), (xqt, xst) = dyt_op, saved_xt
    if cfg.whole_k:
        return K.gemm_rowcol(dyqt, xqt, dyst, xst, None, cfg.post_for(dyqt.shape[-1]))[0]
    return K.gemm_block(dyqt, xqt, dyst, xst, cfg.a_kind, cfg.bt_kind, None, cfg.post, cfg.flags)[0]


def linear_backward(dy2: torch.Tensor, weight: torch.Tensor, saved_xt, cfg: Int8Config = DEFAULT,
                    need_dx: bool = True, need_dw: bool = True):
    """dy2 bf16 [M, N] -> (dx bf16 [M, K] or None, dw bf16 [N, K] or None)."""
    dy_op, dyt_op = quantize_grad_output(dy2, cfg, need_dx, need_dw)
    dx = grad_input(dy_op, weight, cfg) if need_dx else None
    dw = grad_weight(dyt_op, saved_xt, cfg) if need_dw else None
    return dx, dw


class Int8LinearFn(torch.autograd.Function):
    """y = x @ weight^T + bias with all three GEMMs in INT8."""

    @staticmethod
    def forward(ctx, x, weight, bias, cfg: Int8Config):
        x2 = x.reshape(-1, x.shape[-1])
        # Every GEMM reports a device-side wait that gave up into the device's status word; look at it
        # here without blocking (the copy was started by the previous call) and raise if it is set.
        K.poll_status(x.device)
        need_w = weight.requires_grad
        y, saved_xt = linear_forward(x2, weight, bias, cfg, want_xt=need_w)
        ctx.cfg = cfg
        ctx.x_shape = x.shape
        ctx.has_bias = bias is not None
        ctx.save_for_backward(weight, *(saved_xt if need_w else ()))
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        weight, *saved = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        dx, dw = linear_backward(dy2, weight, tuple(saved) if saved else None, ctx.cfg, need_dx, need_dw)
        db = dy2.sum(0).to(dy.dtype) if ctx.has_bias and ctx.needs_input_grad[2] else None
        return (dx.view(ctx.x_shape) if dx is not None else None), dw, db, None


class Int8Linear(nn.Module):
    """Drop-in for nn.Linear (bf16 parameters, same state_dict keys).  Token count (product of the
    leading dims), in_features and out_features must be multiples of 128."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None,
                 dtype=torch.bfloat16, config: Int8Config = DEFAULT):
        super().__init__()
        if in_features % 128 or out_features % 128:
            raise ValueError("in_features and out_features must be multiples of 128")
        self.in_features, self.out_features, self.config = in_features, out_features, config
        self.weight = nn.Parameter(torch.empty(out_features, in_features, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=dtype)) if bias else None
        nn.init.normal_(self.weight, std=0.02)

    @classmethod
    def from_linear(cls, lin: nn.Linear, config: Int8Config = DEFAULT) -> "Int8Linear":
        m = cls(lin.in_features, lin.out_features, lin.bias is not None, lin.weight.device, torch.bfloat16, config)
        m.load_state_dict({k: v.to(torch.bfloat16) for k, v in lin.state_dict().items()})
        return m

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return Int8LinearFn.apply(x, self.weight, self.bias, self.config)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, {self.config}"
