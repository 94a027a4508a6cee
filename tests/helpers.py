"""Shared helpers for the tests: golden loading, subsampling and error measures."""
import os

import numpy as np
import torch

from oracle import inputs

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
SUB = 13          # must match tests/golden/make_golden.py
GRADS = ("d_x", "d_dT", "d_dL", "d_AT", "d_AL", "d_BT", "d_BL", "d_C", "d_D")

# name -> (strided B/C, dtype name); shapes and seeds are read from the fixture itself
SCAN_GOLDEN = {
    "tiny_f32": (True, "f32"), "tiny_f64": (False, "f64"), "rect_f32": (True, "f32"),
    "sq7_f32": (False, "f32"), "rect_bf16": (True, "bf16"), "cfg0_f32": (True, "f32"),
}


def sub(a):
    """The subsample rule used when the fixtures were written."""
    if isinstance(a, torch.Tensor):
        a = a.detach().float().cpu().numpy() if a.dtype == torch.bfloat16 else a.detach().cpu().numpy()
    flat = np.asarray(a).reshape(-1)
    return flat[::SUB] if flat.size > 20000 else flat


def load_scan_golden(name):
    g = np.load(os.path.join(GOLDEN, f"scan_{name}.npz"))
    B, H, W, E, N = (int(v) for v in g["shape"])
    strided, _ = SCAN_GOLDEN[name]
    inp = inputs.make_inputs(B, H, W, E, N, seed=int(g["seed"]), strided_bc=strided)
    chk = np.array([float(inp[k].double().sum()) for k in ("x", "dT", "dL", "AT", "AL", "BT", "BL", "C", "D", "gy")])
    np.testing.assert_allclose(chk, g["checksum"], rtol=1e-12, atol=1e-12,
                               err_msg="input generator drifted from the one the fixtures were made with")
    return inp, g


def rel_err(a, ref):
    """max-abs error relative to the scale (max-abs) of the reference array."""
    a = np.asarray(a, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(a - ref).max() / max(np.abs(ref).max(), 1e-30))


def bf16_round_inputs(inp):
    return {k: v.to(torch.bfloat16).float() for k, v in inp.items()}
