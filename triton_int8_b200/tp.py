"""Column-parallel INT8 linear over the GPUs of one node.

W [N, K] is split along N: rank r owns W[r*N/g:(r+1)*N/g].  X is replicated.  The forward
Y_r = X W_r^T and dW_r = dY_r^T X need no communication; dX = sum_r dY_r W_r is reduced with one
reduce-scatter along M (rank r keeps rows r*M/g..(r+1)*M/g), issued on a side stream so that it
overlaps the dW GEMM (NCCL over NVLink/NVSwitch), or, with `PeerSlots`, by the dX GEMM itself: its
epilogue stores each 128-row block straight into the owning rank's memory over NVLink (plain peer
stores into one slot per source rank) and the owner adds the slots up, so no collective kernel runs.
The reference has no multi-GPU code; the sharding follows from its primitives
(triton/block_channel_fwd32.py:252, triton/block_channel_bwd33.py:175).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import _lib as L
from . import kernels as K
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


class PeerSlots:
    """A bf16 [world, M/world, K] buffer on every rank, each mapped into all the others (one process per
    GPU, one node), for the reduce-scatter that the dX GEMM's epilogue does itself.

    Mapping: torch's symmetric memory when it can be set up, else CUDA IPC handles exchanged through
    the process group.  Ordering between ranks is a one-element NCCL all-reduce on the compute stream
    (`fence`): every rank's earlier work on that stream is complete before any rank's later work starts.
    """

    def __init__(self, rows_total: int, cols: int, group=None, device=None):
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > L.MAX_RANKS:
            raise ValueError(f"PeerSlots: at most {L.MAX_RANKS} ranks")
        shard_bounds(rows_total, self.world, self.rank)  # validates the split
        self.rows, self.cols = rows_total // self.world, cols
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self._keep = []   # objects that keep the peer mappings alive
        self.mapping = None
        numel = self.world * self.rows * cols
        try:
            import torch.distributed._symmetric_memory as symm
            buf = symm.empty((numel,), dtype=torch.bfloat16, device=self.device)
            hdl = symm.rendezvous(buf, group if group is not None else dist.group.WORLD)
            self.ptrs = [int(p) for p in hdl.buffer_ptrs]
            self._keep += [hdl]
            self.mapping = "symmetric_memory"
        except Exception as exc:  # noqa: BLE001 - any failure of the optional route selects the other one
            self._symm_error = repr(exc)
            buf = torch.empty((numel,), dtype=torch.bfloat16, device=self.device)
            self.ptrs = self._exchange_ipc(buf)
            self.mapping = "cuda_ipc"
        self.local = buf.view(self.world, self.rows, cols)
        self._flag = torch.zeros(1, dtype=torch.float32, device=self.device)
        if self.ptrs[self.rank] != buf.data_ptr():
            raise RuntimeError("PeerSlots: the local mapping does not match the local buffer")

    def _exchange_ipc(self, buf: torch.Tensor):
        storage = buf.untyped_storage()
        handle = storage._share_cuda_()   # (device, handle, size, offset, ...) of the allocation that holds buf
        offset_in_alloc = handle[3]
        infos = [None] * self.world
        dist.all_gather_object(infos, (handle, offset_in_alloc), group=self.group)
        ptrs = []
        for r, (h, off) in enumerate(infos):
            if r == self.rank:
                ptrs.append(buf.data_ptr())
                continue
            peer = torch.UntypedStorage._new_shared_cuda(*h)
            self._keep.append(peer)
            ptrs.append(peer.data_ptr())
        return ptrs

    def fence(self) -> None:
        """Stream-ordered barrier over the group."""
        dist.all_reduce(self._flag, group=self.group)

    def reduce_scatter_gemm(self, dyq, dys, wtq, wts, a_kind, post_scale, out=None) -> torch.Tensor:
        """dX rows of this rank = sum over ranks of (dY_r W_r) restricted to those rows."""
        if a_kind != L.ASCALE_TILE:
            raise ValueError("PeerSlots needs per-tile activation scales")
        self.fence()   # every rank has finished reading its slots of the previous step
        K.gemm_block_scatter(dyq, wtq, dys, wts, self.ptrs, self.rank, L.BSCALE_CHANNEL, post_scale)
        self.fence()   # every rank's stores have landed
        return K.sum_slots(self.local, out)


def gather_quantized_activations(x_rows: torch.Tensor, cfg: Int8Config = DEFAULT, group=None):
    """Each rank holds only ITS M/g rows of the replicated activation X (e.g. the slice it copied from the
    host): quantize them once, for both orientations, and all-gather the INT8 operands and their scales
    over NVLink instead of moving bf16 X to every rank.  Per-tile scales are local to a 128-row block, so
    the gathered operands equal bit for bit what every rank would have computed from the whole X.

    x_rows bf16 [M/g, K] -> ((xq [1, M, K], xs [1, M/128, K/128]), (xqt [1, K, M], xst [1, K/128, M/128])):
    the A operand of the forward GEMM and the saved B operand X^T of the dW GEMM.  tile128 scaling only.
    """
    if cfg.gran != L.GRAN_TILE128:
        raise ValueError("gather_quantized_activations: per-tile (tile128) scaling only")
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    # both orientations from one read of the rows (128-token groups never straddle a rank's rows)
    xq, xs, xqt, xst = K.quant_tile(x_rows[None], cfg.gran, cfg.qmode, cfg.hadamard, natural=True, transposed=True)
    return gather_row_sharded_operands(xq, xs, xqt, xst, group)


def gather_row_sharded_operands(xq, xs, xqt, xst, group=None):
    """All-gather of operands quantized from a row shard of X: xq [1, M/g, K] and its tile scales
    [1, M/g/128, K/128] concatenate along the rows in rank order; the transposed pieces xqt [1, K, M/g],
    xst [1, K/128, M/g/128] sit side by side along the token axis of X^T."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return (xq, xs), (xqt, xst)
    _, Ml, Kd = xq.shape
    M = Ml * world

    def gather(t):   # [1, ..] local -> [world, ..]
        out = torch.empty((world,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, t.contiguous(), group=group)
        return out
    xq_all = gather(xq).view(1, M, Kd)
    xs_all = gather(xs).view(1, M // 128, Kd // 128)
    xqt_all = gather(xqt).permute(1, 0, 2).reshape(1, Kd, M)
    xst_all = gather(xst).permute(1, 0, 2).reshape(1, Kd // 128, M // 128)
    return (xq_all, xs_all), (xqt_all, xst_all)


class ColumnParallelStep:
    """Forward + backward of one column-parallel linear with the dX reduce-scatter overlapped
    with the dW GEMM.  Holds the side stream and events; reuse one instance per layer."""

    def __init__(self, group=None, cfg: Int8Config = DEFAULT, peer_slots: PeerSlots | None = None,
                 comm_sms: int | None = None):
        self.group, self.cfg = group, cfg
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.comm_stream = torch.cuda.Stream() if self.world > 1 else None
        # The GEMMs are persistent, one CTA per SM; the dW GEMM that runs beside the reduce-scatter leaves
        # `comm_sms` SMs to the collective's CTAs (otherwise NCCL's kernel waits for the GEMM to end).  The
        # reduce-scatter moves about the same bytes per rank at every world size while the dW GEMM beside it
        # shrinks with 1/world, so the collective needs more SMs as the group grows; measured on the
        # M=32768, K=8192, N=28672 layer: 8 at 2 ranks (8 / 16 SMs: 14.2 / 14.5 ms per step), 16 at 4 ranks
        # (0 / 16 / 32 SMs: 7.79 / 7.39 / 7.55 ms), 32 at 8 ranks (0 / 16 / 24 / 32 / 48 SMs: 4.48 / 4.35 /
        # 4.40 / 3.94 / 4.01 ms).  None picks 4 SMs per rank, between 8 and 32.
        if comm_sms is None:
            comm_sms = min(32, max(8, 4 * self.world))
        self.comm_sms = comm_sms
        sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        self.dw_ctas = max(1, sms - comm_sms) if (self.world > 1 and comm_sms > 0) else 0
        self.peer_slots = peer_slots   # when given, the dX GEMM scatters its partials itself (no NCCL reduce-scatter)

    def forward(self, x: torch.Tensor, w_shard: torch.Tensor, bias_shard=None):
        return linear_forward(x, w_shard, bias_shard, self.cfg, want_xt=True)

    def forward_sharded(self, x_rows: torch.Tensor, w_shard: torch.Tensor, bias_shard=None):
        """As forward(), from this rank's M/g rows of X only: the int8 operands are all-gathered
        (gather_quantized_activations).  Returns (y [M, N/g], saved X^T operand)."""
        cfg = self.cfg
        (xq, xs), saved = gather_quantized_activations(x_rows, cfg, self.group)
        wq, ws = K.quant_row(w_shard, cfg.qmode, cfg.hadamard)
        y = K.gemm_block(xq, wq, xs, ws, cfg.a_kind, L.BSCALE_CHANNEL, bias_shard, cfg.post, cfg.flags)[0]
        return y, saved

    def backward(self, dy_shard: torch.Tensor, w_shard: torch.Tensor, saved_xt):
        """Returns (dx rows owned by this rank [M/g, K], dw_shard [N/g, K])."""
        dy_op, dyt_op = quantize_grad_output(dy_shard, self.cfg, True, True)
        if self.world > 1 and self.peer_slots is not None and not self.cfg.exact and self.cfg.a_kind == L.ASCALE_TILE:
            wtq, wts = K.quant_col_t(w_shard, self.cfg.qmode, self.cfg.hadamard)
            dx = self.peer_slots.reduce_scatter_gemm(dy_op[0], dy_op[1], wtq, wts, self.cfg.a_kind, self.cfg.post)
            return dx, grad_weight(dyt_op, saved_xt, self.cfg)
        dx_partial = grad_input(dy_op, w_shard, self.cfg)
        if self.world == 1:
            return dx_partial, grad_weight(dyt_op, saved_xt, self.cfg)
        main = torch.cuda.current_stream()
        self.comm_stream.wait_stream(main)
        with torch.cuda.stream(self.comm_stream):
            dx = reduce_scatter_rows(dx_partial, self.group)
            dx_partial.record_stream(self.comm_stream)
        with K.cta_limit(self.dw_ctas):
            dw = grad_weight(dyt_op, saved_xt, self.cfg)
        main.wait_stream(self.comm_stream)
        return dx, dw
