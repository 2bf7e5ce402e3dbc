"""Seeded inputs shared by the golden-vector generator and the tests.

Every case returns (a[B,M,K], w[N,K], b3[B,N2,K]) as bf16 CPU tensors: `a` and `w` feed
fwd_32(a, w); `a` and `b3` feed bwd_33(a, b3).
"""
import torch


def _randn(g, *shape, std=1.0):
    return (torch.randn(*shape, generator=g, dtype=torch.float32) * std).to(torch.bfloat16)


def make_inputs(case: str):
    if case == "small":        # B=2, M=256, K=512 (power of two: the per-row kernel needs it), N=384
        g = torch.Generator().manual_seed(20260101)
        return _randn(g, 2, 256, 512), _randn(g, 384, 512), _randn(g, 2, 128, 512)
    if case == "edge":         # ties, an all-zero tile, a tile whose absmax is negative, tiny values
        g = torch.Generator().manual_seed(20260102)
        a = _randn(g, 1, 256, 256)
        a[0, :128, :128] = 0.0                                   # all-zero tile -> scale floor 1e-4
        a[0, 128:, :128] = a[0, 128:, :128].abs().clamp(max=2.0)
        a[0, 200, 5] = -127.0                                    # negative absmax -> s == 1 exactly
        a[0, 128:136, 8:16] = torch.tensor([2.5, -2.5, 63.5, -63.5, 0.5, -0.5, 126.5, -126.5],
                                           dtype=torch.bfloat16)  # exact ties with s == 1
        a[0, :128, 128:] = a[0, :128, 128:] * 1e-6               # amax below the 1e-4 floor
        w = _randn(g, 128, 256, std=0.02)
        w[3] = 0.0                                               # all-zero row
        w[5, 7] = -4.0
        b3 = _randn(g, 1, 128, 256)
        b3[0, :, 128:] = 0.0
        return a, w, b3
    if case == "dc_small":     # double_channel: K must be a multiple of 2048 (unmasked kernels)
        g = torch.Generator().manual_seed(20260103)
        a = _randn(g, 2, 128, 2048)
        a[0, 3] = 0.0
        a[1, 7, 100] = -300.0
        return a, _randn(g, 128, 2048, std=0.02), _randn(g, 2, 128, 2048)
    if case == "c1":           # 512x1024x1024 configuration: X ~ N(0,1) with 8 outlier columns x20, W ~ N(0,0.02), dY ~ N(0,1e-3)
        g = torch.Generator().manual_seed(20260000)
        x = torch.randn(512, 1024, generator=g)
        cols = torch.randperm(1024, generator=g)[:8]
        x[:, cols] *= 20.0
        w = torch.randn(1024, 1024, generator=g) * 0.02
        dy = torch.randn(512, 1024, generator=g) * 1e-3
        return x.to(torch.bfloat16)[None], w.to(torch.bfloat16), dy.to(torch.bfloat16)[None]
    raise KeyError(case)
