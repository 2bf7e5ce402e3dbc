"""Two-rank test of the reduce-scatter done by the dX GEMM's epilogue (peer-memory slots) against the
NCCL route and the exact product.  Needs two GPUs; skipped otherwise.  Ranks are child processes."""
import os
import socket
import subprocess
import sys
import textwrap

import pytest
import torch

pytestmark = pytest.mark.gpu

CHILD = textwrap.dedent("""
    import os, sys
    sys.path.insert(0, os.getcwd())
    import torch, torch.distributed as dist
    from triton_int8_b200 import tp, kernels as K
    from triton_int8_b200.linear import Int8Config
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    M, Kd, N = 1024, 512, 768
    g = torch.Generator().manual_seed(7)
    x = torch.randn(M, Kd, generator=g).bfloat16()
    w = (torch.randn(N, Kd, generator=g) * 0.05).bfloat16()
    dy = (torch.randn(M, N, generator=g) * 1e-2).bfloat16()
    lo, hi = tp.shard_bounds(N, world, rank)
    w_s, dy_s = w[lo:hi].contiguous().to(dev), dy[:, lo:hi].contiguous().to(dev)
    for had in (0, 128):
        cfg = Int8Config(hadamard=had)
        slots = tp.PeerSlots(M, Kd)
        nccl, peer = tp.ColumnParallelStep(cfg=cfg), tp.ColumnParallelStep(cfg=cfg, peer_slots=slots)
        _, xt = nccl.forward(x.to(dev), w_s)
        dx_a, dw_a = nccl.backward(dy_s, w_s, xt)
        for rep in range(2):   # the second call reuses the slots
            dx_b, dw_b = peer.backward(dy_s, w_s, xt)
        torch.cuda.synchronize()
        rows = slice(rank * (M // world), (rank + 1) * (M // world))
        ref = (dy.float() @ w.float())[rows].to(dev)
        rel = lambda u, v: ((u.float() - v.float()).norm() / v.float().norm()).item()
        assert dx_b.shape == dx_a.shape == ref.shape
        assert torch.equal(dw_a, dw_b)
        # the two routes add the same bf16 partials: NCCL in bf16, the slot sum in fp32
        assert rel(dx_b, dx_a) < 1e-2, rel(dx_b, dx_a)
        assert rel(dx_b, ref) < 6e-2 and rel(dx_b, ref) <= rel(dx_a, ref) * 1.05 + 1e-3, (rel(dx_b, ref), rel(dx_a, ref))
        # slot sum alone: equals an fp32 sum of the slots
        want = slots.local.float().sum(0).to(torch.bfloat16)
        assert torch.equal(K.sum_slots(slots.local), want)
    print(f"rank {rank} ok ({slots.mapping})")
    dist.destroy_process_group()
""")


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_slot_reduce_scatter_matches_nccl(tmp_path):
    script = tmp_path / "child.py"
    script.write_text(CHILD)
    port = _free_port()
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, cwd=os.getcwd(),
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        outs.append(out)
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {r} failed:\n{out[-3000:]}"
        assert f"rank {r} ok" in out


@pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a GPU")
@pytest.mark.parametrize("world", [2, 4])
def test_scatter_epilogue_and_slot_sum_on_one_gpu(world):
    """The ranks of a column-parallel dX emulated one after the other on one GPU: every "rank" runs the
    scatter-mode GEMM on its shard with all slot buffers in local memory; the slot sums must equal the
    sum of the plain GEMMs' outputs (same bf16 partials, fp32 sum), row block by row block."""
    from triton_int8_b200 import _lib as L
    from triton_int8_b200 import kernels as K
    dev = "cuda"
    M, Kd, N = 128 * world * 2, 384, 256 * world
    g = torch.Generator().manual_seed(11)
    dy = (torch.randn(M, N, generator=g) * 1e-2).bfloat16().to(dev)
    w = (torch.randn(N, Kd, generator=g) * 0.05).bfloat16().to(dev)
    rows = M // world
    bufs = [torch.zeros(world, rows, Kd, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    ptrs = [b.data_ptr() for b in bufs]
    partials = []
    for r in range(world):
        lo, hi = r * (N // world), (r + 1) * (N // world)
        dyq, dys, _, _ = K.quant_tile(dy[None, :, lo:hi].contiguous())
        wtq, wts = K.quant_col_t(w[lo:hi].contiguous())
        partials.append(K.gemm_block(dyq, wtq, dys, wts)[0])
        K.gemm_block_scatter(dyq, wtq, dys, wts, ptrs, r)
    torch.cuda.synchronize()
    for o in range(world):
        for r in range(world):   # slot r of owner o holds rank r's rows of block o, bit for bit
            assert torch.equal(bufs[o][r], partials[r][o * rows:(o + 1) * rows]), (o, r)
        want = torch.stack([p[o * rows:(o + 1) * rows].float() for p in partials]).sum(0).to(torch.bfloat16)
        assert torch.equal(K.sum_slots(bufs[o]), want)
    with pytest.raises(L.I8LError):   # M must split into 128-row multiples per rank
        K.gemm_block_scatter(dyq[:, :128], wtq, dys[:, :1], wts, ptrs, 0)
