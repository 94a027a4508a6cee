"""GPU parity of the reverse-direction scan (start corner bottom-right).

The reference has no such kernel: it flips the activation (models/mamba2d.py:162-175 for odd
blocks, :190-200 for the second scan of double_scans), runs the top-left scan and flips back.  The
expected values here are therefore the CPU oracle run on flipped inputs, flipped back."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import cpu, inputs
from helpers import GRADS, bf16_round_inputs, rel_err
from test_scan_gpu import ORDER, TDT, TOL, to_dev

pytestmark = pytest.mark.gpu

PIXEL = ("x", "dT", "dL", "BT", "BL", "C", "gy")          # tensors with (B,H,W,.) layout
PIXEL_GRADS = ("d_x", "d_dT", "d_dL", "d_BT", "d_BL", "d_C")


def flipped(inp):
    return {k: (v.flip(1, 2).contiguous() if k in PIXEL else v) for k, v in inp.items()}


SHAPES = [
    (2, 32, 32, 64, 16),
    (2, 5, 4, 6, 4),        # ragged channels / states
    (1, 2, 2, 32, 16),
    (3, 7, 7, 64, 16),
    (1, 28, 28, 128, 16),   # several bands
    (1, 9, 13, 40, 12),
    (1, 13, 3, 32, 16),
    (1, 120, 72, 64, 16),   # chained CTAs
    (2, 56, 56, 64, 16),    # two cells per step in the forward
]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("kind", ["f32", "bf16"])
@pytest.mark.parametrize("strided", [False, True])
def test_reverse_forward_matches_flipped_oracle(shape, kind, strided):
    from mamba2d_b200 import scan_fwd
    inp = inputs.make_inputs(*shape, seed=sum(shape) + 2, strided_bc=strided)
    ref_in = flipped(bf16_round_inputs(inp) if kind == "bf16" else inp)
    y_ref = np.flip(cpu.forward(ref_in, "f64"), (1, 2))
    d = to_dev(inp, TDT[kind])
    y = scan_fwd(*[d[k] for k in ORDER], reverse=True).float().cpu().numpy()
    assert rel_err(y, y_ref) < TOL[kind]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("kind", ["f32", "bf16"])
@pytest.mark.parametrize("strided", [False, True])
def test_reverse_backward_matches_flipped_oracle(shape, kind, strided):
    from mamba2d_b200 import scan_bwd
    inp = inputs.make_inputs(*shape, seed=sum(shape) + 3, strided_bc=strided)
    ref_in = flipped(bf16_round_inputs(inp) if kind == "bf16" else inp)
    ref = cpu.backward(ref_in, mode="f64")
    d = to_dev(inp, TDT[kind])
    got = scan_bwd(*[d[k] for k in ORDER], d["gy"], reverse=True)
    for k, t in zip(GRADS, got):
        want = np.flip(ref[k], (1, 2)) if k in PIXEL_GRADS else ref[k]
        assert rel_err(t.float().cpu().numpy(), want) < TOL[kind], k


@pytest.mark.parametrize("recomp", ["partial", "full"])
@pytest.mark.parametrize("dt,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
def test_entry_bottom_right_equals_flip_scan_flip(recomp, dt, tol):
    """scan_start="BR" against the reference's way of getting that direction: flip, scan, flip."""
    from mamba2d_b200 import wavefront_scan_cuda
    B, H, W, E = 2, 14, 10, 64
    g = torch.Generator().manual_seed(5)
    x0 = torch.randn(B, H, W, E, generator=g)
    gy = torch.randn(B, H, W, E, generator=g).to("cuda", dt)
    p0 = inputs.make_module_params(E, 16, seed=6)
    names = ("AT_log", "AL_log", "x_proj_w", "dt_projT_w", "dt_projT_b", "dt_projL_w", "dt_projL_b", "D")

    def run(native):
        x = x0.to("cuda", dt).requires_grad_(True)
        p = {k: (v.to("cuda") if k.endswith("_log") else v.to("cuda", dt)).requires_grad_(True) for k, v in p0.items()}
        args = [p[k] for k in names]
        if native:
            y = wavefront_scan_cuda(x, *args, recomp, scan_start="BR")
        else:
            y = wavefront_scan_cuda(x.flip(1, 2), *args, recomp).flip(1, 2)
        y.backward(gy)
        return [y.detach()] + [t.grad for t in [x] + args]

    a, b = run(True), run(False)
    for name, u, v in zip(("y", "d_x") + tuple("d_" + n for n in names), a, b):
        assert rel_err(u.float().cpu().numpy(), v.float().cpu().numpy()) < tol, name


def test_entry_rejects_unknown_corner():
    from mamba2d_b200 import wavefront_scan_cuda
    p = {k: v.cuda() for k, v in inputs.make_module_params(32, 16, seed=1).items()}
    x = torch.randn(1, 4, 4, 32, device="cuda")
    with pytest.raises(ValueError):
        wavefront_scan_cuda(x, p["AT_log"], p["AL_log"], p["x_proj_w"], p["dt_projT_w"], p["dt_projT_b"],
                            p["dt_projL_w"], p["dt_projL_b"], p["D"], "partial", scan_start="TR")


def test_reverse_through_the_no_allocation_entry():
    from mamba2d_b200 import _lib, scan_fwd
    from mamba2d_b200.wavefront_cuda import _make_desc
    inp = inputs.make_inputs(2, 28, 28, 64, 16, seed=8)
    d = to_dev(inp, torch.float32)
    args = [d[k] for k in ORDER]
    want = scan_fwd(*args, reverse=True)
    desc, keep = _make_desc(*args, reverse=True)
    y = torch.empty_like(want)
    desc.y = y.data_ptr()
    rc = _lib.lib().m2d_scan_fwd_noalloc(ctypes.byref(desc), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.equal(y, want)
