"""The reference's GPU pipeline around its own CUDA kernels (test / benchmark infrastructure only).

``oracle/_ref/wf_ref_cuda.so`` is the reference project's extension built unmodified from its
sources (oracle/build_ref_cuda.py).  The reference's Python glue around the two kernels cannot
travel (the checkout is not present on the GPU machine), so the functions below restate it with
plain torch ops, step for step:

  forward   models/kernels/wavefront_cuda.py:148-160   (allocate hs, wf_fwd, readout)
  backward  models/kernels/wavefront_cuda.py:163-196   (recompute hs, dD, dC, dHS, wf_bwd,
                                                         fused_backward_math :97-139, d_x)

The reference kernels launch on the legacy default stream without error checks, so callers
synchronise around these functions.
"""
import torch

from . import build_ref_cuda

_EXT = None


def ext():
    global _EXT
    if _EXT is None:
        _EXT = build_ref_cuda.load()
    return _EXT


def available():
    return build_ref_cuda.find() is not None and torch.cuda.is_available()


def forward(x, dT, dL, AT, AL, BT, BL, C, D):
    B, H, W, E = x.shape
    N = AT.shape[1]
    hs = torch.empty((B, H, W, E, N), dtype=x.dtype, device=x.device)
    ext().wf_fwd(hs, x, dT, dL, BT, BL, AT, AL)
    return (hs * C.unsqueeze(-2)).sum(dim=-1) + x * D


def backward(x, dT, dL, AT, AL, BT, BL, C, D, gy):
    B, H, W, E = x.shape
    N = AT.shape[1]
    gy = gy.to(x.dtype)
    hs = torch.empty((B, H, W, E, N), dtype=x.dtype, device=x.device)
    ext().wf_fwd(hs, x, dT, dL, BT, BL, AT, AL)
    dD = (gy * x).sum(dim=(0, 1, 2))
    dC = (gy.unsqueeze(-1) * hs).sum(dim=-2)
    dHS = gy.unsqueeze(-1) * C.unsqueeze(-2)
    dDAT = torch.empty_like(hs)
    dDAL = torch.empty_like(hs)
    omega = torch.empty((2, B, H, E, N), dtype=hs.dtype, device=hs.device)
    ext().wf_bwd(hs, x, dT, dL, AT, AL, dHS, dDAT, dDAL, omega)
    del hs, omega
    # post-kernel gradient math
    gT = torch.exp(dT.unsqueeze(-1) * AT)
    gL = torch.exp(dL.unsqueeze(-1) * AL)
    dzT = dDAT * gT
    dzL = dDAL * gL
    del dDAT, dDAL, gT, gL
    d_AT = (dzT * dT.unsqueeze(-1)).sum(dim=(0, 1, 2))
    d_AL = (dzL * dL.unsqueeze(-1)).sum(dim=(0, 1, 2))
    d_dT = (dzT * AT).sum(dim=-1)
    d_dL = (dzL * AL).sum(dim=-1)
    del dzT, dzL
    rows = torch.arange(H, device=x.device).view(1, H, 1, 1, 1)
    cols = torch.arange(W, device=x.device).view(1, 1, W, 1, 1)
    hT = dHS * (rows > 0)
    hL = dHS * ((cols > 0) | (rows == 0))
    d_dT = d_dT + (hT * BT.unsqueeze(-2) * x.unsqueeze(-1)).sum(dim=-1)
    d_dL = d_dL + (hL * BL.unsqueeze(-2) * x.unsqueeze(-1)).sum(dim=-1)
    tT = hT * dT.unsqueeze(-1)
    tL = hL * dL.unsqueeze(-1)
    d_BT = (tT * x.unsqueeze(-1)).sum(dim=-2)
    d_BL = (tL * x.unsqueeze(-1)).sum(dim=-2)
    d_x = (tT * BT.unsqueeze(-2)).sum(dim=-1) + (tL * BL.unsqueeze(-2)).sum(dim=-1) + gy * D
    return d_x, d_dT, d_dL, d_AT, d_AL, d_BT, d_BL, dC, dD
