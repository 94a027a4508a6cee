"""Generate tests/golden/*.npz by RUNNING the reference project's own code on the CPU.

Run in the development container only (it needs the reference checkout):

    python tests/golden/make_golden.py

What executes:
  * the reference's two CUDA kernel bodies, compiled for the CPU through a thread-index shim
    (oracle/build_ref.py -> oracle/_ref/libwf_ref_cpu.so);
  * the reference's Python module models/kernels/wavefront_cuda.py, loaded from the checkout with
    three edits applied to its syntax tree in memory: the JIT ``cpp_extension.load`` call is
    dropped, the two custom-op wrappers are replaced by functions that call the CPU-run kernels,
    and ``@torch.compile`` decorators are removed (the CPU inductor backend is not usable here).
    Everything else -- proj_params, fused_backward_math, both autograd Functions and
    wavefront_scan_cuda -- is the reference's code, unmodified.

Inputs are regenerated from seeds by oracle.inputs, so only outputs (and input checksums) are
stored.  Large cases store a strided subsample (every SUB-th element of the flattened array).
"""
import ast
import ctypes
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import build_ref, inputs  # noqa: E402

REF_PY = os.path.join(build_ref.REF_ROOT, "models", "kernels", "wavefront_cuda.py")
SUB = 13


def _load_cpu_kernels():
    lib = ctypes.CDLL(build_ref.build())
    return lib


def _c(t, ct):
    return t.ctypes.data_as(ctypes.POINTER(ct))


def make_ops(lib):
    """wf_fwd_op / wf_bwd_op with the reference's signatures, backed by the CPU-run kernels."""
    def kind(t):
        return {torch.float32: ("f32", np.float32, ctypes.c_float),
                torch.float64: ("f64", np.float64, ctypes.c_double),
                torch.bfloat16: ("bf16", np.float32, ctypes.c_float)}[t.dtype]

    def to_np(t, npdt):
        return np.ascontiguousarray(t.detach().float().numpy() if t.dtype == torch.bfloat16 else t.detach().numpy(), dtype=npdt)

    def wf_fwd_op(hs, x, deltaT, deltaL, BT, BL, AT, AL):
        sfx, npdt, ct = kind(hs)
        B, H, W, E, N = hs.shape
        out = np.empty(hs.shape, npdt)
        getattr(lib, "wf_ref_fwd_" + sfx)(B, H, W, E, N, _c(out, ct), *[_c(to_np(t, npdt), ct) for t in (x, deltaT, deltaL, BT, BL, AT, AL)])
        hs.copy_(torch.from_numpy(out).to(hs.dtype))

    def wf_bwd_op(hs, x, deltaT, deltaL, AT, AL, grad_output, dDAT, dDAL, omega):
        sfx, npdt, ct = kind(hs)
        B, H, W, E, N = hs.shape
        g = to_np(grad_output, npdt).copy()
        a = np.empty(hs.shape, npdt)
        l = np.empty(hs.shape, npdt)
        getattr(lib, "wf_ref_bwd_" + sfx)(B, H, W, E, N, *[_c(to_np(t, npdt), ct) for t in (hs, x, deltaT, deltaL, AT, AL)],
                                          _c(g, ct), _c(a, ct), _c(l, ct))
        grad_output.copy_(torch.from_numpy(g).to(hs.dtype))
        dDAT.copy_(torch.from_numpy(a).to(hs.dtype))
        dDAL.copy_(torch.from_numpy(l).to(hs.dtype))

    return wf_fwd_op, wf_bwd_op


def load_reference_module(lib):
    tree = ast.parse(open(REF_PY).read())
    body = []
    for node in tree.body:
        if isinstance(node, ast.Assign) and any(isinstance(t, ast.Name) and t.id == "wf_cuda" for t in node.targets):
            continue                                   # the JIT build of the CUDA extension
        if isinstance(node, ast.FunctionDef) and node.name in ("wf_fwd_op", "wf_bwd_op", "wf_fwd_fake", "wf_bwd_fake"):
            continue                                   # custom-op wrappers, replaced below
        if isinstance(node, ast.FunctionDef):
            node.decorator_list = [d for d in node.decorator_list
                                   if not (isinstance(d, ast.Attribute) and d.attr == "compile")]
        body.append(node)
    tree.body = body
    ns = {"__name__": "reference_wavefront_cuda", "__file__": REF_PY}
    ns["wf_fwd_op"], ns["wf_bwd_op"] = make_ops(lib)
    exec(compile(tree, REF_PY, "exec"), ns)
    return ns


def sub(t):
    a = t.detach().float().numpy() if t.dtype == torch.bfloat16 else t.detach().numpy()
    flat = a.reshape(-1)
    return flat[::SUB].copy() if flat.size > 20000 else flat.copy()


def checksum(inp):
    return np.array([float(inp[k].detach().double().sum()) for k in ("x", "dT", "dL", "AT", "AL", "BT", "BL", "C", "D", "gy")])


SCAN_CASES = [  # name, (B,H,W,E,N), seed, dtype, strided_bc
    ("tiny_f32", (2, 5, 4, 6, 4), 1, torch.float32, True),
    ("tiny_f64", (2, 5, 4, 6, 4), 1, torch.float64, False),
    ("rect_f32", (1, 9, 13, 32, 16), 2, torch.float32, True),
    ("sq7_f32", (2, 7, 7, 32, 16), 3, torch.float32, False),
    ("rect_bf16", (1, 9, 13, 32, 16), 2, torch.bfloat16, True),
    ("cfg0_f32", (2, 32, 32, 64, 16), 0, torch.float32, True),
]
GRADS = ("d_x", "d_dT", "d_dL", "d_AT", "d_AL", "d_BT", "d_BL", "d_C", "d_D")


def gen_scan(ns, out):
    for name, (B, H, W, E, N), seed, dt, strided in SCAN_CASES:
        inp = inputs.make_inputs(B, H, W, E, N, seed=seed, strided_bc=strided)
        leaves = [inp[k].to(dt).requires_grad_(True) for k in inputs.NAMES]
        y = ns["wf_cuda_fn_pr"].apply(*leaves)
        grads = torch.autograd.grad(y, leaves, inp["gy"].to(dt))
        rec = {"shape": np.array([B, H, W, E, N]), "seed": np.array(seed), "checksum": checksum(inp), "y": sub(y)}
        for k, g in zip(GRADS, grads):
            rec[k] = sub(g)
        np.savez_compressed(os.path.join(out, f"scan_{name}.npz"), **rec)
        print("scan", name, "ok |y|max", float(y.detach().abs().max()))


ENTRY_CASES = [  # name, (B,H,W,E,N), seed, dtype
    ("entry_f32", (2, 6, 5, 32, 16), 5, torch.float32),
    ("entry_bf16", (2, 6, 5, 32, 16), 5, torch.bfloat16),
]
WNAMES = ("AT_log", "AL_log", "x_proj_w", "dt_projT_w", "dt_projT_b", "dt_projL_w", "dt_projL_b", "D")


def gen_entry(ns, out):
    for name, (B, H, W, E, N), seed, dt in ENTRY_CASES:
        w = inputs.make_module_params(E, N, seed=seed)
        g = torch.Generator().manual_seed(seed + 100)
        x0 = torch.randn(B, H, W, E, generator=g)
        gy = torch.randn(B, H, W, E, generator=g)
        rec = {"shape": np.array([B, H, W, E, N]), "seed": np.array(seed)}
        for recomp in ("partial", "full"):
            x = x0.to(dt).requires_grad_(True)
            ws = [w[k].clone().requires_grad_(True) for k in WNAMES]      # parameters stay fp32, as in the module
            y = ns["wavefront_scan_cuda"](x, *ws, recomp)
            grads = torch.autograd.grad(y, [x] + ws, gy.to(dt))
            rec[f"{recomp}_y"] = sub(y)
            rec[f"{recomp}_d_x"] = sub(grads[0])
            for k, gr in zip(WNAMES, grads[1:]):
                rec[f"{recomp}_d_{k}"] = sub(gr)
        # also pin proj_params on its own
        outs = ns["proj_params"](x0.to(dt), w["AT_log"], w["AL_log"], *[w[k].to(dt) for k in WNAMES[2:7]])
        for k, t in zip(("dT", "dL", "AT", "AL", "BT", "BL", "C"), outs):
            rec[f"proj_{k}"] = sub(t.contiguous())
        np.savez_compressed(os.path.join(out, f"{name}.npz"), **rec)
        print("entry", name, "ok")


if __name__ == "__main__":
    lib = _load_cpu_kernels()
    ns = load_reference_module(lib)
    gen_scan(ns, HERE)
    gen_entry(ns, HERE)
