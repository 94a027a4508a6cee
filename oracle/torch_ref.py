"""PyTorch restatement of the wavefront scan for autograd cross-checks (test infrastructure only).

``scan_naive`` is a loop over cells, vectorised over (b, e, n), written so that fp64 autograd
through it yields all nine gradients.  ``proj_params_ref`` restates the projection step that
precedes the scan.  Reference lines restated (paths inside the reference project):

  recurrence      models/kernels/wf_cuda/wf_cuda.cu:41-69
  readout         models/kernels/wavefront_cuda.py:156
  projections     models/kernels/wavefront_cuda.py:63-95
  entry           models/kernels/wavefront_cuda.py:315-347
"""
import torch
import torch.nn.functional as F


def scan_naive(x, dT, dL, AT, AL, BT, BL, C, D, return_hs=False):
    """x,dT,dL (B,H,W,E); AT,AL (E,N); BT,BL,C (B,H,W,N); D (E) -> y (B,H,W,E)."""
    Bsz, H, W, E = x.shape
    gT = torch.exp(dT.unsqueeze(-1) * AT)                       # (B,H,W,E,N)
    gL = torch.exp(dL.unsqueeze(-1) * AL)
    uT = (dT.unsqueeze(-1) * BT.unsqueeze(-2)) * x.unsqueeze(-1)
    uL = (dL.unsqueeze(-1) * BL.unsqueeze(-2)) * x.unsqueeze(-1)
    rows = []
    for i in range(H):
        row = []
        for j in range(W):
            if i == 0 and j == 0:
                h = uL[:, 0, 0]
            elif i == 0:
                h = gL[:, 0, j] * row[j - 1] + uL[:, 0, j]
            elif j == 0:
                h = gT[:, i, 0] * rows[i - 1][0] + uT[:, i, 0]
            else:
                h = 0.5 * (gL[:, i, j] * row[j - 1] + uL[:, i, j] + gT[:, i, j] * rows[i - 1][j] + uT[:, i, j])
            row.append(h)
        rows.append(row)
    hs = torch.stack([torch.stack(r, dim=1) for r in rows], dim=1)   # (B,H,W,E,N)
    y = (hs * C.unsqueeze(-2)).sum(dim=-1) + x * D
    return (y, hs) if return_hs else y


def autograd_grads(inp, dtype=torch.float64):
    """All nine gradients by autograd through ``scan_naive`` in ``dtype``; dict keyed like
    ``oracle.cpu.GRAD_NAMES``."""
    names = ("x", "dT", "dL", "AT", "AL", "BT", "BL", "C", "D")
    leaves = [inp[k].detach().to(dtype).clone().contiguous().requires_grad_(True) for k in names]
    y = scan_naive(*leaves)
    grads = torch.autograd.grad(y, leaves, inp["gy"].to(dtype))
    keys = ("d_x", "d_dT", "d_dL", "d_AT", "d_AL", "d_BT", "d_BL", "d_C", "d_D")
    return y.detach(), dict(zip(keys, grads))


def proj_params_ref(x, AT_log, AL_log, x_proj_w, dt_projT_w, dt_projT_b, dt_projL_w, dt_projL_b):
    """Returns dT, dL, AT, AL, BT, BL, C like the reference's ``proj_params``: BT/BL/C are views
    into the x-projection output with row pitch 2R+3N."""
    N = AT_log.shape[1]
    R = dt_projT_w.shape[1]
    AT = -torch.exp(AT_log.float())
    AL = -torch.exp(AL_log.float())
    p = F.linear(x, x_proj_w)
    rT, rL, BT, BL, C = torch.split(p, [R, R, N, N, N], dim=-1)
    dT = F.softplus(F.linear(rT, dt_projT_w, dt_projT_b))
    dL = F.softplus(F.linear(rL, dt_projL_w, dt_projL_b))
    dt = x.dtype
    return dT.to(dt), dL.to(dt), AT.to(dt), AL.to(dt), BT.to(dt), BL.to(dt), C.to(dt)


def scan_from_weights(x, AT_log, AL_log, x_proj_w, dt_projT_w, dt_projT_b, dt_projL_w, dt_projL_b, D):
    """The whole op as the backbone calls it (entry signature of the reference), differentiable."""
    w = [t.to(x.dtype) for t in (x_proj_w, dt_projT_w, dt_projT_b, dt_projL_w, dt_projL_b)]
    dT, dL, AT, AL, BT, BL, C = proj_params_ref(x, AT_log, AL_log, *w)
    return scan_naive(x, dT, dL, AT, AL, BT, BL, C, D.to(x.dtype))
