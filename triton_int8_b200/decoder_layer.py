"""One Llama-style decoder layer whose seven linear maps (q, k, v, o, gate, up, down) are INT8 linears.

This is the chained use of the hot path: the output of one quantized linear, after the glue of a
transformer block (RMS norm, rotary-free causal attention, SiLU gating, residual adds), is the input
of the next, and the backward pass sends real upstream gradients, not synthetic ones, through dX and
dW of every linear.  The glue is ordinary PyTorch (it is not part of the path this library rebuilds);
all seven Y, dX and dW products run through `Int8LinearFn`, i.e. through fwd_32 / bwd_33 of the
reference (triton/block_channel_fwd32.py:252, triton/block_channel_bwd33.py:175) by composition.

The reference has no model code; shapes follow Llama-2-7B (hidden 4096, 32 heads, MLP 11008).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from .linear import DEFAULT, Int8Config, Int8Linear


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5, device=None, dtype=torch.bfloat16):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, device=device, dtype=dtype))

    def forward(self, x):
        v = x.float()
        return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype) * self.weight


class DecoderLayer(nn.Module):
    """linear_cls(in, out, bias=False, device=..., dtype=...) builds the seven projections: Int8Linear
    (default, with `config`) or nn.Linear for a bf16 twin with the same parameter names."""

    def __init__(self, hidden: int = 4096, heads: int = 32, mlp: int = 11008, device=None,
                 config: Int8Config = DEFAULT, linear_cls=None):
        super().__init__()
        if hidden % heads:
            raise ValueError("hidden must be a multiple of heads")
        self.heads = heads
        if linear_cls is None:
            def linear_cls(i, o):
                return Int8Linear(i, o, bias=False, device=device, config=config)
        else:
            base = linear_cls

            def linear_cls(i, o):
                return base(i, o, bias=False, device=device, dtype=torch.bfloat16)
        self.input_norm = RMSNorm(hidden, device=device)
        self.post_norm = RMSNorm(hidden, device=device)
        self.q_proj, self.k_proj = linear_cls(hidden, hidden), linear_cls(hidden, hidden)
        self.v_proj, self.o_proj = linear_cls(hidden, hidden), linear_cls(hidden, hidden)
        self.gate_proj, self.up_proj = linear_cls(hidden, mlp), linear_cls(hidden, mlp)
        self.down_proj = linear_cls(mlp, hidden)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x bf16 [batch, seq, hidden]; batch*seq must be a multiple of 128."""
        B, S, H = x.shape
        h = self.input_norm(x)
        split = lambda t: t.view(B, S, self.heads, H // self.heads).transpose(1, 2)  # noqa: E731
        att = F.scaled_dot_product_attention(split(self.q_proj(h)), split(self.k_proj(h)), split(self.v_proj(h)),
                                             is_causal=True)
        x = x + self.o_proj(att.transpose(1, 2).reshape(B, S, H))
        h = self.post_norm(x)
        return x + self.down_proj(F.silu(self.gate_proj(h)) * self.up_proj(h))

    def linears(self):
        return {n: getattr(self, n) for n in ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")}
