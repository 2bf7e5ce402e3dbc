"""Host-side logic of the column-parallel split, run as two gloo ranks on CPU: shard bounds, the
reduce-scatter wrapper, and the algebra dX = sum_r dY_r W_r / dW_r = dY_r^T X checked with the CPU
oracle standing in for the GEMMs (the product GEMMs themselves are CUDA-only)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import ref_semantics as R
from triton_int8_b200 import tp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, scenario, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        M, K, N = 256, 256, 512
        x = torch.randn(M, K, generator=g).to(torch.bfloat16)
        w = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)
        dy = (torch.randn(M, N, generator=g) * 1e-3).to(torch.bfloat16)
        lo, hi = tp.shard_bounds(N, world, rank)
        w_r, dy_r = tp.shard_weight(w, world, rank), dy[:, lo:hi].contiguous()
        assert w_r.shape == ((hi - lo), K)
        if scenario == "algebra":
            y_r, dx_part, dw_r = R.linear_block_channel(x, w_r, dy_r)
            dx_r = tp.reduce_scatter_rows(dx_part.float())
            y_full, dx_full, dw_full = R.linear_block_channel(x, w, dy)
            mlo, mhi = tp.shard_bounds(M, world, rank, multiple=1)
            # forward and dW shards are bit-equal to slices of the unsharded result (128-groups never straddle)
            ok = torch.equal(y_r, y_full[:, lo:hi]) and torch.equal(dw_r, dw_full[lo:hi])
            # dX differs by quantisation noise of the per-shard W^T scales: compare with the exact product
            exact = dy.float() @ w.float()
            err = R.rel_fro(dx_r, exact[mlo:mhi])
            q.put((rank, ok, err))
        elif scenario == "gather":
            # each rank quantizes only its rows of X (both orientations); the gathered operands must equal
            # what the whole X gives, bit for bit (tile scales are local to 128-row blocks)
            mlo, mhi = tp.shard_bounds(M, world, rank)
            x_l = x[mlo:mhi]
            q_l, s_l = R.quant_tile128(x_l[None])
            qt_l, st_l = R.quant_tile128(x_l.t().contiguous()[None])
            (xq, xs), (xqt, xst) = tp.gather_row_sharded_operands(q_l, s_l, qt_l, st_l)
            q_f, s_f = R.quant_tile128(x[None])
            qt_f, st_f = R.quant_tile128(x.t().contiguous()[None])
            ok = all(torch.equal(a_, b_) for a_, b_ in ((xq, q_f), (xs, s_f), (xqt, qt_f), (xst, st_f)))
            q.put((rank, ok, 0.0))
        elif scenario == "mismatch":
            tp.set_shape_checks(True)
            part = torch.zeros(M if rank == 0 else M // 2, K)
            try:
                tp.reduce_scatter_rows(part)
                q.put((rank, False, 0.0))
            except RuntimeError as e:
                q.put((rank, "disagree" in str(e), 0.0))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("scenario", ["algebra", "gather", "mismatch"])
def test_two_rank_column_parallel(scenario):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, scenario, q)) for r in range(2)]
    [p.start() for p in procs]
    res = [q.get(timeout=120) for _ in procs]
    [p.join(timeout=60) for p in procs]
    assert all(p.exitcode == 0 for p in procs)
    for rank, ok, err in res:
        assert ok, f"rank {rank}"
        assert err < 3e-2


def test_shard_bounds_validation():
    assert tp.shard_bounds(28672, 8, 3) == (3 * 3584, 4 * 3584)
    assert [tp.shard_bounds(28672, g, 0)[1] for g in (1, 2, 4, 8)] == [28672, 14336, 7168, 3584]
    with pytest.raises(ValueError):
        tp.shard_bounds(1024 + 128, 2, 0)      # shards would not be multiples of 128
    with pytest.raises(ValueError):
        tp.shard_bounds(1024, 2, 2)
