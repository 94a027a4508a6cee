"""GPU parity of the fused projection kernels (include/m2d_proj.h) against the reference's
formulation of proj_params (models/kernels/wavefront_cuda.py:63-95) in fp64 PyTorch on the CPU,
differentiated by autograd.  Tolerances: 1e-4 x output scale in fp32, 2e-2 with bf16 tensors."""
import pytest
import torch

from oracle import inputs, torch_ref
from helpers import rel_err

pytestmark = pytest.mark.gpu

NAMES = ("AT_log", "AL_log", "x_proj_w", "dt_projT_w", "dt_projT_b", "dt_projL_w", "dt_projL_b")
OUTS = ("deltaT", "deltaL", "AT", "AL", "BT", "BL", "C")

# (pixels as B,H,W), E, dt_rank (None = E/16 rounded up)
CASES = [
    ((2, 28, 28), 64, None),     # R = 4
    ((2, 14, 14), 128, None),    # R = 8
    ((2, 7, 9), 320, None),      # R = 20, block of 320 threads
    ((1, 7, 7), 512, None),      # R = 32, block of 512 threads
    ((1, 5, 6), 576, None),      # R = 36: the widest shipped stage, two halves of 32 ranks
    ((3, 5, 4), 40, 4),          # channel count that is not a multiple of the warp size
    ((3, 5, 4), 40, None),       # R = 3: K = 54 is not a multiple of 4, PyTorch branch
    ((1, 9, 3), 96, 5),          # K = 2R+3N = 58 is not a multiple of 4: PyTorch branch of the backward
    ((2, 33, 31), 64, 4),        # pixel count that is not a multiple of the tile
    ((1, 1, 3), 64, 4),          # fewer pixels than one tile
    ((1, 2, 2), 512, None),      # fewer pixels than one tile, widest block
]


def _weights(E, R, seed):
    return inputs.make_module_params(E, 16, seed=seed, dt_rank=R)


def _run(fn, x, w, gs, device, dt):
    leaves = [x.to(device, dt).requires_grad_(True)] + \
             [(w[k].to(device) if k.endswith("_log") else w[k].to(device, dt)).requires_grad_(True) for k in NAMES]
    out = fn(*leaves)
    grads = torch.autograd.grad(list(out), leaves, [g.to(device, o.dtype) for g, o in zip(gs, out)])
    return [o.detach().double().cpu() for o in out], [g.double().cpu() for g in grads]


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("dt,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
def test_proj_params_forward_and_backward(case, dt, tol):
    from mamba2d_b200 import proj_params
    (B, H, W), E, R = case
    w = _weights(E, R, seed=E + (R or 0))
    g = torch.Generator().manual_seed(11)
    x = torch.randn(B, H, W, E, generator=g)
    if dt == torch.bfloat16:          # the fp64 check sees the values the kernels see
        x = x.bfloat16().float()
        w = {k: (v if k.endswith("_log") else v.bfloat16().float()) for k, v in w.items()}
    ref_out = torch_ref.proj_params_ref(x.double(), *[w[k].double() for k in NAMES])
    gs = [torch.randn(o.shape, generator=g) for o in ref_out]
    if dt == torch.bfloat16:
        gs = [t.bfloat16().float() for t in gs]
    want_out, want_g = _run(torch_ref.proj_params_ref, x, w, gs, "cpu", torch.float64)
    got_out, got_g = _run(proj_params, x, w, gs, "cuda", dt)
    for name, a, b in zip(OUTS, got_out, want_out):
        assert rel_err(a.numpy(), b.numpy()) < tol, name
    for name, a, b in zip(("x",) + NAMES, got_g, want_g):
        assert rel_err(a.numpy(), b.numpy()) < tol, "d_" + name


def test_proj_params_with_missing_upstream_gradients():
    """Only some outputs feed the loss: the absent gradients count as zero."""
    from mamba2d_b200 import proj_params
    E = 64
    w = _weights(E, None, seed=5)
    x = torch.randn(2, 6, 6, E, generator=torch.Generator().manual_seed(1))

    def run(fn, device, dt):
        leaves = [x.to(device, dt).requires_grad_(True)] + [w[k].to(device, dt if not k.endswith("_log") else torch.float32)
                                                            .requires_grad_(True) for k in NAMES]
        out = fn(*leaves)
        loss = (out[0] * 0.5).sum() + (out[6] ** 2).sum()          # deltaT and C only
        return [None if g is None else g.double().cpu()
                for g in torch.autograd.grad(loss, leaves, allow_unused=True)]

    want = run(lambda *a: torch_ref.proj_params_ref(*[t.double() for t in a]), "cpu", torch.float32)
    got = run(proj_params, "cuda", torch.float32)
    for name, a, b in zip(("x",) + NAMES, got, want):
        if b is None or float(b.abs().max()) == 0.0:
            assert a is None or float(a.abs().max()) == 0.0, name
        else:
            assert rel_err(a.numpy(), b.numpy()) < 1e-4, name


def test_projection_ops_pass_opcheck():
    from mamba2d_b200 import wavefront_cuda as wc
    E, R, N = 64, 4, 16
    w = {k: v.cuda() for k, v in _weights(E, R, seed=2).items()}
    proj = torch.randn(2, 5, 5, 2 * R + 3 * N, device="cuda")
    torch.library.opcheck(wc.dtproj_fwd_op, (proj, w["dt_projT_w"], w["dt_projT_b"], w["dt_projL_w"], w["dt_projL_b"], N))
    x = torch.randn(2, 5, 5, E, device="cuda")
    torch.library.opcheck(wc.xproj_wgrad_op, (proj, x, N, R))


def test_proj_params_under_autocast_takes_the_pytorch_branch():
    """Under autocast the x projection returns bf16 next to fp32 weights; the fused kernels want one
    dtype, so that case runs the PyTorch formulation (forward and hand-written backward) and must
    still agree with autograd of the reference's formulation under the same autocast."""
    from mamba2d_b200 import proj_params
    E = 64
    w = _weights(E, None, seed=8)
    g = torch.Generator().manual_seed(3)
    x0 = torch.randn(2, 6, 6, E, generator=g)

    def run(fn):
        leaves = [x0.cuda().requires_grad_(True)] + [w[k].cuda().requires_grad_(True) for k in NAMES]
        with torch.autocast("cuda", dtype=torch.bfloat16):
            out = fn(*leaves)
        gg = torch.Generator().manual_seed(4)
        gs = [torch.randn(o.shape, generator=gg).to(o.device, o.dtype) for o in out]
        grads = torch.autograd.grad(list(out), leaves, gs)
        return [o.detach().double().cpu() for o in out], [t.double().cpu() for t in grads]

    want_out, want_g = run(torch_ref.proj_params_ref)
    got_out, got_g = run(proj_params)
    for name, a, b in zip(OUTS, got_out, want_out):
        assert a.shape == b.shape and rel_err(a.numpy(), b.numpy()) < 2e-2, name
    for name, a, b in zip(("x",) + NAMES, got_g, want_g):
        assert rel_err(a.numpy(), b.numpy()) < 4e-2, "d_" + name


def test_fused_softplus_is_accurate_over_its_whole_range():
    """The kernel's softplus (max(z,0) + a series for log1p(exp(-|z|))) against fp64 over
    z in [-60, 60]: relative error below 1e-6 everywhere, including the tail below the threshold of
    20 where the reference's formulation switches to the identity."""
    from mamba2d_b200 import wavefront_cuda as wc
    E, R, N = 64, 4, 16
    P = 4096
    z = torch.linspace(-60.0, 60.0, P)
    proj = torch.zeros(1, 1, P, 2 * R + 3 * N)
    proj[0, 0, :, 0] = z              # rT[:, 0] carries z; WT = e_0 picks it out for every channel
    proj[0, 0, :, R] = -z             # and rL[:, 0] carries -z
    WT = torch.zeros(E, R)
    WT[:, 0] = 1.0
    b = torch.zeros(E)
    dT, dL = wc.dtproj_fwd_op(proj.cuda(), WT.cuda(), b.cuda(), WT.cuda(), b.cuda(), N)
    want = torch.nn.functional.softplus(z.double())
    for got, ref in ((dT[0, 0, :, 5].double().cpu(), want), (dL[0, 0, :, 9].double().cpu(), want.flip(0))):
        rel = ((got - ref).abs() / ref.clamp_min(1e-30)).max()
        assert float(rel) < 1e-6


@pytest.mark.parametrize("P,E,R", [(50176, 64, 4), (20000, 128, 8), (9999, 320, 20), (5000, 512, 32), (3000, 576, 36),
                                   (777, 40, 4), (64, 64, 4), (65, 192, 12)])
def test_xproj_weight_gradient_on_tensor_cores(P, E, R, monkeypatch):
    """bf16 problems that meet the alignment rules run on tcgen05 (the library says so itself); the
    result matches an fp64 product of the same bf16 operands and the CUDA-core kernel's."""
    import ctypes
    from mamba2d_b200 import _lib, wavefront_cuda as wc
    N = 16
    K = 2 * R + 3 * N
    g = torch.Generator().manual_seed(P + E)
    d_proj = torch.randn(P, K, generator=g).bfloat16().cuda()
    x = torch.randn(P, E, generator=g).bfloat16().cuda()
    monkeypatch.delenv("M2D_WGRAD_TC", raising=False)
    d = wc._proj_desc(d_proj, E, R, N)
    d.d_proj, d.x = d_proj.data_ptr(), x.data_ptr()
    assert _lib.lib().m2d_xproj_wgrad_on_tensor_cores(ctypes.byref(d)) == 1
    got = wc._xproj_wgrad(d_proj, x, N, R)
    torch.cuda.synchronize()
    want = d_proj.double().T @ x.double()
    scale = float(want.abs().max())
    assert float((got.double() - want).abs().max()) <= 2e-2 * scale
    monkeypatch.setenv("M2D_WGRAD_TC", "0")
    assert _lib.lib().m2d_xproj_wgrad_on_tensor_cores(ctypes.byref(d)) == 0
    simt = wc._xproj_wgrad(d_proj, x, N, R)
    torch.cuda.synchronize()
    assert float((got.double() - simt.double()).abs().max()) <= 1e-2 * scale     # both round their fp32 sums to bf16
