"""Seeded synthetic inputs for the wavefront scan (test infrastructure only).

One CPU ``torch.Generator``, fp32 draws in a fixed order:
``x, dT, dL, BT, BL, C, AT, AL, D_skip, gy``.

  x              ~ N(0, 1)                          (B,H,W,E)
  dT, dL         = softplus(N(-2, 0.5))             (B,H,W,E), independent draws
  BT, BL, C      ~ N(0, 1/N)  (std N**-0.5)         (B,H,W,N)
  AT, AL         = -exp(U(log 1, log 16))           (E,N)
  D_skip         ~ N(0, 1)                          (E)
  gy             ~ N(0, 1)                          (B,H,W,E)  upstream gradient

The reference op takes separate "top" and "left" parameter sets
(models/kernels/wavefront_cuda.py:148 in the reference), so a benchmark description that names a
single delta/B/A is instantiated twice, with independent draws.
"""
import math

import torch
import torch.nn.functional as F

NAMES = ("x", "dT", "dL", "AT", "AL", "BT", "BL", "C", "D")


def make_inputs(B, H, W, E, N=16, seed=0, strided_bc=False, dt_rank=None):
    """Return a dict of fp32 CPU tensors.  With ``strided_bc`` the BT/BL/C tensors are views into
    one (B,H,W,2R+3N) buffer with the offsets the reference's ``proj_params`` produces
    (models/kernels/wavefront_cuda.py:78-82)."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    x = torch.randn(B, H, W, E, generator=g)
    dT = F.softplus(torch.randn(B, H, W, E, generator=g) * 0.5 - 2.0)
    dL = F.softplus(torch.randn(B, H, W, E, generator=g) * 0.5 - 2.0)
    std = N ** -0.5
    BT = torch.randn(B, H, W, N, generator=g) * std
    BL = torch.randn(B, H, W, N, generator=g) * std
    C = torch.randn(B, H, W, N, generator=g) * std
    lo, hi = math.log(1.0), math.log(16.0)
    AT = -torch.exp(torch.rand(E, N, generator=g) * (hi - lo) + lo)
    AL = -torch.exp(torch.rand(E, N, generator=g) * (hi - lo) + lo)
    D = torch.randn(E, generator=g)
    gy = torch.randn(B, H, W, E, generator=g)
    if strided_bc:
        R = dt_rank if dt_rank is not None else math.ceil(E / 16)
        K = 2 * R + 3 * N
        buf = torch.zeros(B, H, W, K)
        buf[..., 2 * R:2 * R + N] = BT
        buf[..., 2 * R + N:2 * R + 2 * N] = BL
        buf[..., 2 * R + 2 * N:] = C
        BT = buf[..., 2 * R:2 * R + N]
        BL = buf[..., 2 * R + N:2 * R + 2 * N]
        C = buf[..., 2 * R + 2 * N:]
    return dict(x=x, dT=dT, dL=dL, AT=AT, AL=AL, BT=BT, BL=BL, C=C, D=D, gy=gy)


def make_module_params(E, N=16, seed=0, dt_rank=None):
    """Weights shaped like the ones ``M2DBlock`` owns (models/mamba2d.py:68-112 in the reference):
    A_log = log(1..N) per channel, x_proj (2R+3N, E), dt_proj weight (E,R) and bias (E), D = 1."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    R = dt_rank if dt_rank is not None else math.ceil(E / 16)
    A = torch.arange(1, N + 1, dtype=torch.float32).repeat(E, 1)
    AT_log = torch.log(A) + 0.05 * torch.randn(E, N, generator=g)
    AL_log = torch.log(A) + 0.05 * torch.randn(E, N, generator=g)
    bound = E ** -0.5
    x_proj_w = (torch.rand(2 * R + 3 * N, E, generator=g) * 2 - 1) * bound
    dt_std = R ** -0.5
    dtT_w = (torch.rand(E, R, generator=g) * 2 - 1) * dt_std
    dtL_w = (torch.rand(E, R, generator=g) * 2 - 1) * dt_std
    dt = torch.exp(torch.rand(E, generator=g) * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3)).clamp(min=1e-4)
    inv_dt = dt + torch.log(-torch.expm1(-dt))
    D = torch.ones(E) + 0.1 * torch.randn(E, generator=g)
    return dict(AT_log=AT_log, AL_log=AL_log, x_proj_w=x_proj_w, dt_projT_w=dtT_w, dt_projT_b=inv_dt.clone(),
                dt_projL_w=dtL_w, dt_projL_b=inv_dt.clone(), D=D)
