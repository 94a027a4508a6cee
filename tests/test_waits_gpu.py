"""The bounded waits of the kernels give up cleanly, and one diverged image does not poison others.

Row-warps of a CTA and, on large maps with few images, CTAs that share an image wait on one another.
Every such wait has a limit; when one runs out the kernel still returns normally and leaves a
nonzero status word in its workspace.  A test hook (descriptor flag M2D_SCAN_TEST_WITHHOLD, honoured
only under M2D_TEST_HOOKS=1) makes exactly that happen: one producer never publishes its progress and
the limits are a few hundred tries.  Nothing here faults or hangs the GPU: a wait runs out and the
kernel ends."""
import ctypes

import pytest
import torch

from mamba2d_b200 import _lib
from mamba2d_b200 import wavefront_cuda as wc
from oracle import cpu, inputs
from helpers import rel_err

pytestmark = pytest.mark.gpu
ORDER = ("x", "dT", "dL", "AT", "AL", "BT", "BL", "C", "D")


def _launch_fwd(dev, flags):
    L = _lib.lib()
    d, keep = wc._make_desc(*[dev[k] for k in ORDER])
    d.flags = flags
    y = torch.empty_like(dev["x"])
    d.y = y.data_ptr()
    wc._workspace(d, L.m2d_scan_fwd_workspace(ctypes.byref(d)), dev["x"].device, keep)
    rc = L.m2d_scan_fwd(ctypes.byref(d), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, d, keep[-1], y


def test_a_withheld_counter_makes_the_wait_give_up(monkeypatch):
    monkeypatch.setenv("M2D_TEST_HOOKS", "1")
    inp = inputs.make_inputs(1, 96, 64, 64, 16, seed=3)      # one image on a large map: several CTAs share it
    dev = {k: v.cuda() for k, v in inp.items()}
    L = _lib.lib()
    d0, _ = wc._make_desc(*[dev[k] for k in ORDER])
    assert L.m2d_scan_fwd_chain(ctypes.byref(d0)) > 1
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    rc, d, ws, _ = _launch_fwd(dev, _lib.M2D_SCAN_TEST_WITHHOLD)
    stop.record()
    assert rc == 0
    torch.cuda.synchronize()
    assert start.elapsed_time(stop) < 2000.0                 # it returned promptly
    off = L.m2d_scan_fwd_status_offset(ctypes.byref(d))
    assert off >= 0 and wc._status_word(ws, off) != 0
    with pytest.raises(RuntimeError, match="timed out"):
        wc._check_status("fwd", d, ws)
    # the context is fine and the next, ordinary launch is correct
    rc, d, ws, y = _launch_fwd(dev, 0)
    assert rc == 0
    torch.cuda.synchronize()
    assert wc._status_word(ws, off) == 0
    assert rel_err(y.cpu().numpy(), cpu.forward(inp, "f64")) < 1e-4


def test_the_hook_is_refused_without_the_environment_variable(monkeypatch):
    monkeypatch.delenv("M2D_TEST_HOOKS", raising=False)
    inp = inputs.make_inputs(1, 96, 64, 64, 16, seed=3)
    dev = {k: v.cuda() for k, v in inp.items()}
    rc, _, _, _ = _launch_fwd(dev, _lib.M2D_SCAN_TEST_WITHHOLD)
    assert rc == -10


@pytest.mark.parametrize("shape", [(300, 6, 5, 64, 16), (400, 12, 9, 32, 16)])   # more (image, group) units than resident CTAs
def test_a_diverged_image_leaves_the_others_alone(shape):
    """Image 1 gets infinite inputs.  A CTA walks several images one after the other and carries state
    in registers and shared memory; nothing of a diverged image may leak into the next one (missing
    neighbours are taken as zero, never multiplied by a zero gate)."""
    from mamba2d_b200 import scan_bwd, scan_fwd
    inp = inputs.make_inputs(*shape, seed=8)
    dev = {k: v.cuda() for k, v in inp.items()}
    a = [dev[k] for k in ORDER]
    y0 = scan_fwd(*a)
    g0 = scan_bwd(*a, dev["gy"])
    bad = {k: v.clone() for k, v in dev.items()}
    bad["x"][1] = float("inf")
    bad["gy"][1] = float("inf")
    b = [bad[k] for k in ORDER]
    y1 = scan_fwd(*b)
    g1 = scan_bwd(*b, bad["gy"])
    torch.cuda.synchronize()
    keep = [i for i in range(shape[0]) if i != 1]
    assert torch.equal(y0[keep], y1[keep])
    for idx in (0, 1, 2, 5, 6, 7):       # the per-pixel gradients (the batch sums d_AT, d_AL, d_D include image 1)
        assert torch.isfinite(g1[idx][keep]).all()
        assert float((g0[idx][keep] - g1[idx][keep]).abs().max()) <= 1e-6 * float(g0[idx].abs().max())
