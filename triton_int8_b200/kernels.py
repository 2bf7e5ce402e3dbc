"""Tensor-level wrappers of the C ABI: allocate outputs with torch, pass raw pointers and the
current CUDA stream.  These are the building blocks of the fwd_32 / bwd_33 variants."""
from __future__ import annotations

import torch

from . import _lib as L


def _ptr(t):
    return None if t is None else t.data_ptr()


def _call(name: str, dev: torch.device, *args, tensors=()) -> None:
    """Launch on `dev`: the C side takes the device, its SM count and the stream from the current CUDA
    context, so the tensors' device is made current for the call (the trailing stream argument is that
    device's current stream), and every operand must live on it."""
    for t in tensors:
        if t is not None and t.device != dev:
            raise ValueError(f"{name}: operands on different devices ({t.device} vs {dev})")
    with torch.cuda.device(dev):
        L.call(name, *args, torch.cuda.current_stream(dev).cuda_stream)


# ---------------------------------------------------------------------------------------- status word
# The GEMM kernels bound every device-side wait; a wait that gives up makes the kernel return early and
# write I8L_ERR_TIMEOUT into a device int32.  One such word per device is passed to every GEMM launched
# from here.  check_status() reads it (synchronously); poll_status() is the cheap form for a training
# loop: it looks at a copy started by the previous poll and starts the next one, never blocking.
_STATUS: dict = {}


class _StatusWord:
    def __init__(self, dev):
        self.dev = dev
        self.word = torch.zeros(1, dtype=torch.int32, device=dev)
        self.host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.event = None


def _status_of(dev: torch.device) -> "_StatusWord":
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    st = _STATUS.get(key)
    if st is None:
        st = _STATUS[key] = _StatusWord(torch.device("cuda", key))
    return st


def device_status(dev) -> torch.Tensor:
    """The int32 status word that GEMMs on `dev` report into (0 = no wait has ever given up)."""
    return _status_of(torch.device(dev)).word


def _raise_if_set(st: "_StatusWord", code: int) -> None:
    if code:
        st.word.zero_()
        st.host.zero_()
        raise L.I8LError(code, f"a GEMM on {st.dev} gave up a bounded device-side wait; its output is incomplete")


def check_status(dev=None) -> None:
    """Synchronous check: raises I8LError (code TIMEOUT) if a GEMM on `dev` gave up a wait since the
    last check, and clears the word."""
    st = _status_of(torch.device(dev if dev is not None else ("cuda", torch.cuda.current_device())))
    st.event = None
    _raise_if_set(st, int(st.word.item()))


def poll_status(dev) -> None:
    """Non-blocking check for hot loops: raises if the copy started by an earlier poll has completed and
    shows a timeout; then starts the next copy.  Does nothing while the stream is being captured."""
    st = _status_of(torch.device(dev))
    if torch.cuda.is_current_stream_capturing():
        return
    if st.event is not None:
        if not st.event.query():
            return
        st.event = None
        _raise_if_set(st, int(st.host[0]))
    st.host.copy_(st.word, non_blocking=True)
    st.event = torch.cuda.Event()
    st.event.record(torch.cuda.current_stream(st.dev))


def _check_bf16(x: torch.Tensor, name: str) -> torch.Tensor:
    if not x.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (no CPU path exists)")
    if x.dtype != torch.bfloat16:
        raise TypeError(f"{name} must be bfloat16, got {x.dtype}")
    return x.contiguous()


def quant_tile(x: torch.Tensor, gran: int = L.GRAN_TILE128, qmode: int = L.QMODE_TRITON, hadamard: int = 0,
               natural: bool = True, transposed: bool = False):
    """x bf16 [B, R, C] -> (q, scale, qt, scale_t); entries not requested are None."""
    x = _check_bf16(x, "x")
    B, R, C = x.shape
    q = s = qt = st = None
    if natural:
        q = torch.empty((B, R, C), dtype=torch.int8, device=x.device)
        s_shape = {L.GRAN_TILE128: (B, R // 128, C // 128), L.GRAN_TILE128X256: (B, R // 128, C // 256)}.get(gran, (B, R, C // 128))
        s = torch.empty(s_shape, dtype=torch.float32, device=x.device)
    if transposed:
        qt = torch.empty((B, C, R), dtype=torch.int8, device=x.device)
        st = torch.empty((B, C // 128, R // 128) if gran == L.GRAN_TILE128 else (B, C, R // 128),
                         dtype=torch.float32, device=x.device)
    _call("i8l_quant_tile", x.device, x.data_ptr(), B, R, C, gran, qmode, hadamard, _ptr(q), _ptr(s), _ptr(qt), _ptr(st))
    return q, s, qt, st


def quant_row(x: torch.Tensor, qmode: int = L.QMODE_TRITON, hadamard: int = 0):
    """x bf16 [..., C] -> int8 [..., C], fp32 scale [...]."""
    x = _check_bf16(x, "x")
    C = x.shape[-1]
    rows = x.numel() // C
    q = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    s = torch.empty(x.shape[:-1], dtype=torch.float32, device=x.device)
    _call("i8l_quant_row", x.device, x.data_ptr(), rows, C, qmode, hadamard, q.data_ptr(), s.data_ptr())
    return q, s


def quant_col_t(x: torch.Tensor, qmode: int = L.QMODE_TRITON, hadamard: int = 0):
    """x bf16 [R, C] -> int8 x^T [C, R] with one scale per column of x, fp32 [C]; hadamard=128 rotates
    x^T in 128-wide groups along its contraction axis (the rows of x) first."""
    x = _check_bf16(x, "x")
    R, C = x.shape
    qt = torch.empty((C, R), dtype=torch.int8, device=x.device)
    st = torch.empty((C,), dtype=torch.float32, device=x.device)
    scratch = torch.empty((C,), dtype=torch.float32, device=x.device)
    if hadamard not in (0, 128):
        raise ValueError("quant_col_t: hadamard must be 0 or 128")
    _call("i8l_quant_col_t_rot" if hadamard else "i8l_quant_col_t", x.device, x.data_ptr(), R, C, qmode, qt.data_ptr(),
          st.data_ptr(), scratch.data_ptr())
    return qt, st


def _gemm_dims(aq: torch.Tensor, bq: torch.Tensor):
    if aq.dtype != torch.int8 or bq.dtype != torch.int8:
        raise TypeError("quantized operands must be int8")
    B, M, K = aq.shape
    b_batched = bq.dim() == 3
    N = bq.shape[-2]
    if bq.shape[-1] != K or (b_batched and bq.shape[0] != B):
        raise ValueError(f"operand shapes do not match: {tuple(aq.shape)} x {tuple(bq.shape)}")
    return B, M, N, K, b_batched


def gemm_block(aq, bq, a_s, b_s, a_kind=L.ASCALE_TILE, b_kind=L.BSCALE_CHANNEL, bias=None, post_scale=1.0,
               flags=0, status=None):
    """Block-scaled GEMM; returns bf16 (fp32 with GEMM_OUT_F32) [B, M, N]."""
    aq, bq = aq.contiguous(), bq.contiguous()
    B, M, N, K, bb = _gemm_dims(aq, bq)
    out = torch.empty((B, M, N), dtype=torch.float32 if flags & L.GEMM_OUT_F32 else torch.bfloat16, device=aq.device)
    a_s, b_s = a_s.contiguous(), b_s.contiguous()
    status = device_status(aq.device) if status is None else status
    _call("i8l_gemm_block", aq.device, aq.data_ptr(), bq.data_ptr(), a_s.data_ptr(), b_s.data_ptr(),
          a_kind, b_kind, int(bb), _ptr(bias), float(post_scale), out.data_ptr(), B, M, N, K, flags, _ptr(status),
          tensors=(bq, a_s, b_s, bias, status))
    return out


def gemm_rowcol(aq, bq, a_s, b_s, bias=None, post_scale=1.0, flags=0, status=None):
    aq, bq = aq.contiguous(), bq.contiguous()
    B, M, N, K, bb = _gemm_dims(aq, bq)
    out = torch.empty((B, M, N), dtype=torch.float32 if flags & L.GEMM_OUT_F32 else torch.bfloat16, device=aq.device)
    a_s, b_s = a_s.contiguous(), b_s.contiguous()
    status = device_status(aq.device) if status is None else status
    _call("i8l_gemm_rowcol", aq.device, aq.data_ptr(), bq.data_ptr(), a_s.data_ptr(), b_s.data_ptr(),
          int(bb), _ptr(bias), float(post_scale), out.data_ptr(), B, M, N, K, flags, _ptr(status),
          tensors=(bq, a_s, b_s, bias, status))
    return out


def fused_gemm(a_bf, b_bf, flags=0, status=None):
    """bf16 a [B, M, K] x bf16 b [N, K] or [B, N, K] -> bf16 (fp32 with GEMM_OUT_F32) [B, M, N] in ONE kernel:
    operand tiles are quantized on the fly per 128-wide K step inside the GEMM (nothing int8 reaches memory)."""
    a_bf, b_bf = _check_bf16(a_bf, "a"), _check_bf16(b_bf, "b")
    B, M, K = a_bf.shape
    bb = b_bf.dim() == 3
    N = b_bf.shape[-2]
    if b_bf.shape[-1] != K or (bb and b_bf.shape[0] != B):
        raise ValueError(f"operand shapes do not match: {tuple(a_bf.shape)} x {tuple(b_bf.shape)}")
    out = torch.empty((B, M, N), dtype=torch.float32 if flags & L.GEMM_OUT_F32 else torch.bfloat16, device=a_bf.device)
    status = device_status(a_bf.device) if status is None else status
    _call("i8l_fused_gemm", a_bf.device, a_bf.data_ptr(), b_bf.data_ptr(), out.data_ptr(), B, M, N, K, int(bb), flags,
          _ptr(status), tensors=(b_bf, status))
    return out


def gemm_dump_i32(aq, bq, per_block=False, status=None):
    aq, bq = aq.contiguous(), bq.contiguous()
    B, M, N, K, bb = _gemm_dims(aq, bq)
    shape = (B, K // 128, M, N) if per_block else (B, M, N)
    out = torch.empty(shape, dtype=torch.int32, device=aq.device)
    status = device_status(aq.device) if status is None else status
    _call("i8l_gemm_dump_i32", aq.device, aq.data_ptr(), bq.data_ptr(), int(bb), out.data_ptr(), B, M, N, K, int(per_block),
          _ptr(status), tensors=(bq, status))
    return out


def gemm_block_scatter(aq, bq, a_s, b_s, slot_ptrs, rank: int, b_kind=L.BSCALE_CHANNEL, post_scale=1.0, status=None):
    """Block-scaled GEMM [M, K] x [N, K]^T whose row block o goes to slot `rank` of the bf16
    [world, M/world, N] buffer at slot_ptrs[o] (device pointers, peers included).  Nothing is returned:
    the caller synchronises the ranks and sums its own buffer with sum_slots."""
    import ctypes
    aq, bq = aq.contiguous(), bq.contiguous()
    B, M, N, K, bb = _gemm_dims(aq, bq)
    if B != 1 or bb:
        raise ValueError("gemm_block_scatter: one batch, shared B operand")
    world = len(slot_ptrs)
    arr = (ctypes.c_void_p * world)(*[int(p) for p in slot_ptrs])
    a_s, b_s = a_s.contiguous(), b_s.contiguous()
    status = device_status(aq.device) if status is None else status
    _call("i8l_gemm_block_scatter", aq.device, aq.data_ptr(), bq.data_ptr(), a_s.data_ptr(),
          b_s.data_ptr(), b_kind, float(post_scale), ctypes.cast(arr, ctypes.c_void_p), world, int(rank),
          M, N, K, _ptr(status), tensors=(bq, a_s, b_s, status))


def sum_slots(slots: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """slots bf16 [world, rows, cols] -> bf16 [rows, cols], summed in slot order in fp32."""
    if slots.dtype != torch.bfloat16 or slots.dim() != 3 or not slots.is_contiguous():
        raise TypeError("sum_slots: contiguous bf16 [world, rows, cols]")
    world, rows, cols = slots.shape
    if out is None:
        out = torch.empty((rows, cols), dtype=torch.bfloat16, device=slots.device)
    _call("i8l_sum_slots", slots.device, slots.data_ptr(), out.data_ptr(), world, rows, cols, tensors=(out,))
    return out


class cta_limit:
    """Context manager: GEMMs launched inside use at most `n` CTAs, leaving the other SMs to a kernel
    running beside them (a collective on another stream).  n <= 0 means no limit."""

    def __init__(self, n: int):
        self.n = max(0, int(n))

    def __enter__(self):
        L.call("i8l_set_cta_limit", self.n)
        return self

    def __exit__(self, *exc):
        L.call("i8l_set_cta_limit", 0)
        return False
