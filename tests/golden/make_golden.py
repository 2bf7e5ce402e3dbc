"""Generate golden vectors by EXECUTING the reference's own Triton kernels on CPU.

Run once, in a container that has the reference checkout (its path in I8L_REFERENCE_DIR)
and triton installed:

    python tests/golden/make_golden.py

The kernels run under the Triton interpreter (TRITON_INTERPRET=1), so no GPU is
needed.  Outputs go to tests/golden/*.npz.  Inputs are regenerated from the seeds
stored in each file (see tests/golden/golden_inputs.py); outputs are stored in full
for small cases and as SHA-256 digests plus a strided sample for the larger one.

Interpreter caveats handled here: autotuned kernels are launched through `.fn[grid]`
with the 128^3 blocking the reference wrapper fixes; C is always fp32 (the interpreter
truncates on a bf16 store, a GPU rounds to nearest even), the bf16 cast is applied by
the consumer.  The external fast_hadamard_transform extension is absent, so the
double_channel goldens start from the ALREADY ROTATED operands (rotation on/off is a
test of this repository's own FWHT, not of the reference).
"""
import hashlib
import importlib.util
import os
import sys
import types

os.environ["TRITON_INTERPRET"] = "1"
import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from golden_inputs import make_inputs  # noqa: E402

REF = os.environ.get("I8L_REFERENCE_DIR")
if not REF or not os.path.isdir(REF):
    raise SystemExit("set I8L_REFERENCE_DIR to the checkout of the reference project")


def _load(name, rel):
    if "fast_hadamard_transform" not in sys.modules:
        stub = types.ModuleType("fast_hadamard_transform")
        stub.hadamard_transform = lambda x, scale=1.0: x  # never called here
        sys.modules["fast_hadamard_transform"] = stub
    spec = importlib.util.spec_from_file_location(name, os.path.join(REF, rel))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().numpy().tobytes()).hexdigest()


def block_channel(case):
    fwd = _load("ref_bc_fwd", "triton/block_channel_fwd32.py")
    bwd = _load("ref_bc_bwd", "triton/block_channel_bwd33.py")
    a, w, b3 = make_inputs(case)
    B, M, K = a.shape
    N = w.shape[0]
    aq, a_s = fwd.triton_per_block_quant(a)
    wq, w_s = fwd.triton_per_token_quant(w)
    C = torch.zeros(B, M, N, dtype=torch.float32)
    fwd.int8_gemm_kernel.fn[(M // 128, N // 128, B)](
        A_ptr=aq, B_ptr=wq, C_ptr=C, A_scale_ptr=a_s, B_scale_ptr=w_s,
        B=B, M=M, N=N, K=K,
        stride_am=aq.stride(1), stride_ak=aq.stride(2),
        stride_bn=wq.stride(0), stride_bk=wq.stride(1),
        stride_cm=C.stride(1), stride_cn=C.stride(2),
        stride_ab=aq.stride(0), stride_cb=C.stride(0),
        stride_a_scale_b=a_s.stride(0), stride_a_scale_m=a_s.stride(1), stride_a_scale_k=a_s.stride(2),
        stride_b_scale_n=w_s.stride(0),
        BLOCK_M=128, BLOCK_N=128, BLOCK_K=128)
    # bwd_33(a, b3): both operands tile-quantized by the bwd file's own kernel
    aq2, a_s2 = bwd.triton_per_block_quant(a)
    bq2, b_s2 = bwd.triton_per_block_quant(b3)
    N2 = b3.shape[1]
    C2 = torch.zeros(B, M, N2, dtype=torch.float32)
    bwd.int8_gemm_kernel.fn[(M // 128, N2 // 128, B)](
        A_ptr=aq2, B_ptr=bq2, C_ptr=C2, A_scales_ptr=a_s2, B_scales_ptr=b_s2,
        BATCH=B, M=M, N=N2, K=K,
        stride_ab=aq2.stride(0), stride_am=aq2.stride(1), stride_ak=aq2.stride(2),
        stride_bb=bq2.stride(0), stride_bn=bq2.stride(1), stride_bk=bq2.stride(2),
        stride_cb=C2.stride(0), stride_cm=C2.stride(1), stride_cn=C2.stride(2),
        stride_scale_a_b=a_s2.stride(0), stride_scale_am=a_s2.stride(1), stride_scale_ak=a_s2.stride(2),
        stride_scale_b_b=b_s2.stride(0), stride_scale_bn=b_s2.stride(1), stride_scale_bk=b_s2.stride(2),
        BLOCK_M=128, BLOCK_N=128, BLOCK_K=128)
    return dict(aq=aq, a_s=a_s, wq=wq, w_s=w_s, c_fwd=C, aq_bwd=aq2, a_s_bwd=a_s2,
                bq_bwd=bq2, b_s_bwd=b_s2, c_bwd=C2)


def double_channel(case):
    fwd = _load("ref_dc_fwd", "triton/double-channle_fwd32.py")
    bwd = _load("ref_dc_bwd", "triton/double_channel_bwd33.py")
    a, w, b3 = make_inputs(case)
    B, M, K = a.shape
    N = w.shape[0]
    aq, a_s = fwd.triton_per_row_quant_3d(a)
    wq, w_s = fwd.triton_per_row_quant_2d(w)
    C = torch.zeros(B, M, N, dtype=torch.float32)
    fwd.int8_gemm_kernel.fn[(M // 128, N // 128, B)](
        A_ptr=aq, B_ptr=wq, C_ptr=C, A_scale_ptr=a_s, B_scale_ptr=w_s,
        B=B, M=M, N=N, K=K,
        stride_am=aq.stride(1), stride_ak=aq.stride(2),
        stride_bn=wq.stride(0), stride_bk=wq.stride(1),
        stride_cm=C.stride(1), stride_cn=C.stride(2),
        stride_ab=aq.stride(0), stride_cb=C.stride(0),
        stride_a_scale_b=a_s.stride(0), stride_a_scale_m=a_s.stride(1),
        stride_b_scale_n=w_s.stride(0),
        BLOCK_M=128, BLOCK_N=128, BLOCK_K=128)
    bq, b_s = bwd.triton_per_row_quant_3d(b3)
    aq2, a_s2 = bwd.triton_per_row_quant_3d(a)
    N2 = b3.shape[1]
    C2 = torch.zeros(B, M, N2, dtype=torch.float32)
    bwd.int8_gemm_kernel.fn[(M // 128, N2 // 128, B)](
        A_ptr=aq2, B_ptr=bq, C_ptr=C2, A_scales_ptr=a_s2, B_scales_ptr=b_s,
        BATCH=B, M=M, N=N2, K=K,
        stride_ab=aq2.stride(0), stride_am=aq2.stride(1), stride_ak=aq2.stride(2),
        stride_bb=bq.stride(0), stride_bn=bq.stride(1), stride_bk=bq.stride(2),
        stride_cb=C2.stride(0), stride_cm=C2.stride(1), stride_cn=C2.stride(2),
        stride_scale_a_b=a_s2.stride(0), stride_scale_am=a_s2.stride(1),
        stride_scale_b_b=b_s.stride(0), stride_scale_bn=b_s.stride(1),
        BLOCK_M=128, BLOCK_N=128, BLOCK_K=128)
    return dict(aq=aq, a_s=a_s, wq=wq, w_s=w_s, c_fwd=C, bq_bwd=bq, b_s_bwd=b_s, c_bwd=C2)


def fused(case):
    fwd = _load("ref_fu_fwd", "triton/fused_triton_fwd32.py")
    bwd = _load("ref_fu_bwd", "triton/fused_triton_bwd33.py")
    a, w, b3 = make_inputs(case)
    B, M, K = a.shape
    N = w.shape[0]
    C = torch.zeros(B, M, N, dtype=torch.float32)
    fwd.fused_int8_gemm_kernel[(B, M // 128, N // 128)](
        A_bf_ptr=a, B_bf_ptr=w, C_ptr=C, K=K,
        stride_ab=a.stride(0), stride_am=a.stride(1), stride_ak=a.stride(2),
        stride_bn=w.stride(0), stride_bk=w.stride(1),
        stride_cb=C.stride(0), stride_cm=C.stride(1), stride_cn=C.stride(2),
        BLOCK_M=128, BLOCK_N=128, BLOCK_K=128)
    N2 = b3.shape[1]
    C2 = torch.zeros(B, M, N2, dtype=torch.float32)
    bwd.fused_int8_gemm_kernel.fn[(B, M // 128, N2 // 128)](
        A_bf_ptr=a, B_bf_ptr=b3, C_ptr=C2, K=K,
        stride_ab=a.stride(0), stride_am=a.stride(1), stride_ak=a.stride(2),
        stride_bb=b3.stride(0), stride_bn=b3.stride(1), stride_bk=b3.stride(2),
        stride_cb=C2.stride(0), stride_cm=C2.stride(1), stride_cn=C2.stride(2),
        BLOCK_M=128, BLOCK_N=128, BLOCK_K=128)
    return dict(c_fwd=C, c_bwd=C2)


def _extract(rel, names, uncomment=None):
    """Source text of the named top-level functions of a reference file, without importing the file
    (the TileLang files need a tilelang version that is not installed).  `uncomment` = (first, last)
    1-based line range of a commented-out function whose leading "# " is stripped and which is
    returned under the name `<name>_commented`."""
    import ast
    text = open(os.path.join(REF, rel)).read()
    lines = text.splitlines()
    out = []
    for node in ast.parse(text).body:
        if isinstance(node, ast.FunctionDef) and node.name in names:
            first = min([node.lineno] + [d.lineno for d in node.decorator_list])
            out.append("\n".join(lines[first - 1:node.end_lineno]))
    if uncomment:
        body = [l[2:] if l.startswith("# ") else l.lstrip("#") for l in lines[uncomment[0] - 1:uncomment[1]]]
        body[0] = body[0].replace("def per_token_cast_to_int8", "def per_token_cast_to_int8_commented")
        out.append("\n".join(body))
    return "\n\n".join(out)


def _module_from_source(name, source):
    """Import extracted source through a temporary file (triton.jit needs inspect.getsource to work)."""
    import tempfile
    d = tempfile.mkdtemp(prefix="i8l_golden_")
    path = os.path.join(d, name + ".py")
    with open(path, "w") as f:
        f.write("import torch\nimport triton\nimport triton.language as tl\nfrom typing import Tuple\n\n" + source + "\n")
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def torch_helpers():
    """The reference's pure-torch quantisation helpers, executed as they stand:
    tilelang/block_channel_bwd.py:96-104 (tile 128x128, amax upcast to fp32),
    tilelang/block_channel_fwd.py:215-230 (per row and per tile, arithmetic in the INPUT dtype) and the
    commented-out per-(row, 128) version at tilelang/block_channel_fwd.py:206-213.  Each is run on the
    bf16 inputs of the `small` and `edge` cases and on unrounded fp32 inputs."""
    fwd = _module_from_source("ref_tl_fwd_helpers", _extract(
        "tilelang/block_channel_fwd.py", {"per_token_cast_to_int8", "per_block_cast_to_int8"}, uncomment=(206, 213)))
    bwd = _module_from_source("ref_tl_bwd_helpers", _extract("tilelang/block_channel_bwd.py", {"per_block_cast_to_int8"}))
    out = {}
    g = torch.Generator().manual_seed(20260110)
    cases = {"small": make_inputs("small")[:2], "edge": make_inputs("edge")[:2],
             "f32": (torch.randn(2, 256, 512, generator=g) * 3.0, torch.randn(384, 512, generator=g) * 0.02)}
    for cname, (a, w) in cases.items():
        for fname, fn, arg in (("bwd_block", bwd.per_block_cast_to_int8, a), ("fwd_block", fwd.per_block_cast_to_int8, a),
                               ("fwd_token", fwd.per_token_cast_to_int8, w),
                               ("fwd_group", fwd.per_token_cast_to_int8_commented, w)):
            q, sc = fn(arg.clone())
            out[f"{cname}__{fname}__q"] = q
            out[f"{cname}__{fname}__s"] = sc.float()          # bf16 scales are stored widened (exact)
            out[f"{cname}__{fname}__s_dtype"] = torch.tensor([{torch.float32: 32, torch.bfloat16: 16}[sc.dtype]])
    return out


def tilelang_quantizers():
    """The Triton quantizers that feed the TileLang GEMM (tilelang/block_channel_fwd.py:94-121 per row,
    :152-183 per 128x256 tile), run under the interpreter.  The wrappers allocate bf16 scale tensors
    (:133, :191); the interpreter truncates on a bf16 store where a GPU rounds to nearest even, so the
    kernels are launched here with fp32 scale tensors and the consumer applies the bf16 rounding."""
    mod = _module_from_source("ref_tl_fwd_quant", _extract(
        "tilelang/block_channel_fwd.py", {"per_token_quant_kernel", "per_block_quant_kernel"}))
    out = {}
    for cname in ("small", "edge"):
        a, w, _ = make_inputs(cname)
        B, M, K = a.shape
        N = w.shape[0]
        aq = torch.empty_like(a, dtype=torch.int8)
        a_s = torch.empty((B, M // 128, K // 256), dtype=torch.float32)
        mod.per_block_quant_kernel[(B * (M // 128) * (K // 256),)](
            X_ptr=a, SCALE_ptr=a_s, OUT_ptr=aq, B=B, M=M, N=K,
            stride_b=a.stride(0), stride_m=a.stride(1), stride_n=a.stride(2),
            stride_sb=a_s.stride(0), stride_sm=a_s.stride(1), stride_sn=a_s.stride(2),
            stride_ob=aq.stride(0), stride_om=aq.stride(1), stride_on=aq.stride(2),
            BLOCK_M=128, BLOCK_N=256)
        wq = torch.empty_like(w, dtype=torch.int8)
        w_s = torch.empty((N, 1), dtype=torch.float32)
        mod.per_token_quant_kernel[(N // 128, 1)](
            X_ptr=w, SCALE_ptr=w_s, OUT_ptr=wq, M=N, N=K,
            stride_xm=w.stride(0), stride_xn=w.stride(1), stride_sm=w_s.stride(0), stride_sn=w_s.stride(1),
            stride_om=wq.stride(0), stride_on=wq.stride(1), BLOCK_M=128, BLOCK_N=K)
        out.update({f"{cname}__aq": aq, f"{cname}__a_s_f32": a_s, f"{cname}__wq": wq, f"{cname}__w_s_f32": w_s})
    return out


def save(name, case, outs, digest_only=False):
    rec = {"case": np.array(case)}
    for k, v in outs.items():
        if digest_only and v.numel() > 4096:
            rec[k + "__sha256"] = np.array(sha(v))
            rec[k + "__sample"] = v.flatten()[::997].contiguous().numpy()
        else:
            rec[k] = v.numpy()
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **rec)
    print("wrote", name, {k: getattr(v, "shape", None) for k, v in rec.items()})


if __name__ == "__main__":
    if "--helpers-only" in sys.argv:
        save("torch_helpers", "small+edge+f32", torch_helpers())
        save("tilelang_quantizers", "small+edge", tilelang_quantizers())
        raise SystemExit(0)
    save("block_channel_small", "small", block_channel("small"))
    save("block_channel_edge", "edge", block_channel("edge"))
    save("double_channel_small", "dc_small", double_channel("dc_small"))
    save("fused_small", "small", fused("small"))
    save("block_channel_c1", "c1", block_channel("c1"), digest_only=True)
    save("torch_helpers", "small+edge+f32", torch_helpers())
    save("tilelang_quantizers", "small+edge", tilelang_quantizers())
