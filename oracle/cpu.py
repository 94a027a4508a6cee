"""ctypes wrapper around the C oracle (test infrastructure only)."""
import ctypes
import os

import numpy as np
import torch

from . import build as _build

_LIB = None
_SUFFIX = {"f64": ("_f64", np.float64, ctypes.c_double),
           "f32": ("_f32", np.float32, ctypes.c_float),
           "bf16e": ("_bf16e", np.float32, ctypes.c_float)}
GRAD_NAMES = ("d_x", "d_dT", "d_dL", "d_AT", "d_AL", "d_BT", "d_BL", "d_C", "d_D")


def lib():
    global _LIB
    if _LIB is None:
        path = _build.build()
        _LIB = ctypes.CDLL(path)
        _LIB.m2d_oracle_num_threads.restype = ctypes.c_int
    return _LIB


def num_threads():
    return int(lib().m2d_oracle_num_threads())


def set_threads(n):
    lib().m2d_oracle_set_threads(ctypes.c_int(int(n)))


def _np(t, npdt):
    if isinstance(t, torch.Tensor):
        t = t.detach().to("cpu")
        if t.dtype == torch.bfloat16:
            t = t.float()
        t = t.numpy()
    return np.ascontiguousarray(t, dtype=npdt)


def _ptr(a, ct):
    return a.ctypes.data_as(ctypes.POINTER(ct)) if a is not None else None


def _prep(mode, inp):
    sfx, npdt, ct = _SUFFIX[mode]
    a = {k: _np(inp[k], npdt) for k in ("x", "dT", "dL", "AT", "AL", "BT", "BL", "C", "D")}
    B, H, W, E = a["x"].shape
    N = a["AT"].shape[1]
    return sfx, npdt, ct, a, (B, H, W, E, N)


def forward(inp, mode="f64", return_hs=False):
    """y (and optionally hs) for a dict of inputs x,dT,dL,AT,AL,BT,BL,C,D.  Returns numpy arrays."""
    sfx, npdt, ct, a, (B, H, W, E, N) = _prep(mode, inp)
    y = np.empty((B, H, W, E), dtype=npdt)
    hs = np.empty((B, H, W, E, N), dtype=npdt) if return_hs else None
    fn = getattr(lib(), "m2d_oracle_fwd" + sfx)
    fn.restype = ctypes.c_int
    rc = fn(B, H, W, E, N, _ptr(a["x"], ct), _ptr(a["dT"], ct), _ptr(a["dL"], ct),
            _ptr(a["AT"], ct), _ptr(a["AL"], ct), _ptr(a["BT"], ct), _ptr(a["BL"], ct),
            _ptr(a["C"], ct), _ptr(a["D"], ct), _ptr(y, ct), _ptr(hs, ct))
    if rc != 0:
        raise RuntimeError(f"m2d_oracle_fwd{sfx} failed ({rc})")
    return (y, hs) if return_hs else y


def backward(inp, gy=None, mode="f64"):
    """The nine gradients as a dict of numpy arrays (keys GRAD_NAMES)."""
    sfx, npdt, ct, a, (B, H, W, E, N) = _prep(mode, inp)
    g = _np(inp["gy"] if gy is None else gy, npdt)
    out = dict(d_x=np.empty((B, H, W, E), npdt), d_dT=np.empty((B, H, W, E), npdt),
               d_dL=np.empty((B, H, W, E), npdt), d_AT=np.empty((E, N), npdt), d_AL=np.empty((E, N), npdt),
               d_BT=np.empty((B, H, W, N), npdt), d_BL=np.empty((B, H, W, N), npdt),
               d_C=np.empty((B, H, W, N), npdt), d_D=np.empty((E,), npdt))
    fn = getattr(lib(), "m2d_oracle_bwd" + sfx)
    fn.restype = ctypes.c_int
    rc = fn(B, H, W, E, N, _ptr(a["x"], ct), _ptr(a["dT"], ct), _ptr(a["dL"], ct),
            _ptr(a["AT"], ct), _ptr(a["AL"], ct), _ptr(a["BT"], ct), _ptr(a["BL"], ct),
            _ptr(a["C"], ct), _ptr(a["D"], ct), _ptr(g, ct),
            *[_ptr(out[k], ct) for k in GRAD_NAMES])
    if rc != 0:
        raise RuntimeError(f"m2d_oracle_bwd{sfx} failed ({rc})")
    return out
