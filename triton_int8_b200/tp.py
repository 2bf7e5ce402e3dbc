"""Column-parallel INT8 linear over the GPUs of one node.

W [N, K] is split along N: rank r owns W[r*N/g:(r+1)*N/g].  X is replicated.  The forward
Y_r = X W_r^T and dW_r = dY_r^T X need no communication; dX = sum_r dY_r W_r is reduced with one
reduce-scatter along M (rank r keeps rows r*M/g..(r+1)*M/g), issued on a side stream so that it
overlaps the dW GEMM.  This is the only collective in the library (NCCL over NVLink/NVSwitch).
The reference has no multi-GPU code; the sharding follows from its primitives
(triton/block_channel_fwd32.py:252, triton/block_channel_bwd33.py:175).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .linear import DEFAULT, Int8Config, grad_input, grad_weight, linear_forward, quantize_grad_output


def shard_bounds(n: int, world: int, rank: int, multiple: int = 128) -> tuple[int, int]:
    """[lo, hi) of the rank's slice of an axis of length n; every slice must be a multiple of 128
    so that no 128-group straddles two shards."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if n % (world * multiple):
        raise ValueError(f"axis of length {n} cannot be split into {world} shards that are multiples of {multiple}")
    per = n // world
    return rank * per, (rank + 1) * per


def shard_weight(weight: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    lo, hi = shard_bounds(weight.shape[0], world, rank)
    return weight[lo:hi].contiguous()


def reduce_scatter_rows(partial: torch.Tensor, group=None, out: torch.Tensor | None = None) -> torch.Tensor:
    """Sum `partial` [M, K] over the group and keep this rank's M/g rows."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    M = partial.shape[0]
    shapes = [None] * world
    dist.all_gather_object(shapes, tuple(partial.shape), group=group) if _DEBUG_SHAPES else None
    if _DEBUG_SHAPES and any(s != shapes[0] for s in shapes):
        raise RuntimeError(f"reduce_scatter_rows: ranks disagree on the partial shape: {shapes}")
    lo, hi = shard_bounds(M, world, rank, multiple=1)
    if out is None:
        out = torch.empty((hi - lo,) + tuple(partial.shape[1:]), dtype=partial.dtype, device=partial.device)
    if world == 1:
        out.copy_(partial)
    elif dist.get_backend(group) == "nccl":
        dist.reduce_scatter_tensor(out, partial.contiguous(), op=dist.ReduceOp.SUM, group=group)
    else:  # CPU process groups (tests): gloo has no reduce_scatter_tensor
        buf = partial.float().contiguous()
        dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=group)
        out.copy_(buf[lo:hi].to(partial.dtype))
    return out


_DEBUG_SHAPES = False


def set_shape_checks(on: bool) -> None:
    """Cross-rank shape validation before each collective (one extra small all-gather)."""
    global _DEBUG_SHAPES
    _DEBUG_SHAPES = bool(on)


class ColumnParallelStep:
    """Forward + backward of one column-parallel linear with the dX reduce-scatter overlapped
    with the dW GEMM.  Holds the side stream and events; reuse one instance per layer."""

    def __init__(self, group=None, cfg: Int8Config = DEFAULT):
        self.group, self.cfg = group, cfg
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.comm_stream = torch.cuda.Stream() if self.world > 1 else None

    def forward(self, x: torch.Tensor, w_shard: torch.Tensor, bias_shard=None):
        return linear_forward(x, w_shard, bias_shard, self.cfg, want_xt=True)

    def backward(self, dy_shard: torch.Tensor, w_shard: torch.Tensor, saved_xt):
        """Returns (dx rows owned by this rank [M/g, K], dw_shard [N/g, K])."""
        dy_op, dyt_op = quantize_grad_output(dy_shard, self.cfg, True, True)
        dx_partial = grad_input(dy_op, w_shard, self.cfg)
        if self.world == 1:
            return dx_partial, grad_weight(dyt_op, saved_xt, self.cfg)
        main = torch.cuda.current_stream()
        self.comm_stream.wait_stream(main)
        with torch.cuda.stream(self.comm_stream):
            dx = reduce_scatter_rows(dx_partial, self.group)
            dx_partial.record_stream(self.comm_stream)
        dw = grad_weight(dyt_op, saved_xt, self.cfg)
        main.wait_stream(self.comm_stream)
        return dx, dw
