"""The forward entry point that takes no workspace (m2d_scan_fwd_noalloc).

It serves callers that can pass inputs and outputs but have no way to allocate or pass a scratch
buffer: the scratch sits in a fixed 32 MiB array inside the library.  The GPU test calls it through
the C ABI twice in a row (the array is shared by all calls and keeps whatever the previous call
left in it) and checks each result against the regular entry point, which gets its scratch from
the caller.  The file name sorts last on purpose: a run that stops at the first failure has then
already run every other test.
"""
import ctypes

import pytest
import torch

from mamba2d_b200 import _lib
from mamba2d_b200 import wavefront_cuda as wc
from oracle import inputs

ORDER = ("x", "dT", "dL", "AT", "AL", "BT", "BL", "C", "D")


def _call_noalloc(dev):
    """y from m2d_scan_fwd_noalloc for a dict of device tensors (no workspace in the descriptor)."""
    L = _lib.lib()
    with torch.cuda.device(dev["x"].device):
        d, keep = wc._make_desc(*[dev[k] for k in ORDER])
        y = torch.empty_like(dev["x"])
        d.y = y.data_ptr()
        d.workspace, d.workspace_bytes = None, 0
        rc = L.m2d_scan_fwd_noalloc(ctypes.byref(d), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    _lib.check(rc, "m2d_scan_fwd_noalloc")
    return y


@pytest.mark.gpu
@pytest.mark.parametrize("kind,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
def test_noalloc_forward_equals_regular_forward_back_to_back(kind, tol):
    # different problems back to back, all with several bands of rows so the ring is in use; each
    # reuses array slots the one before has written (the last two are narrow maps: the flat step loop
    # with two columns, one row per band with three)
    for shape, seed in (((3, 40, 24, 64, 16), 11), ((2, 19, 33, 96, 16), 12), ((5, 20, 2, 32, 16), 13), ((5, 13, 3, 32, 16), 14)):
        inp = inputs.make_inputs(*shape, seed=seed)
        dev = {k: v.to("cuda", kind) for k, v in inp.items()}
        want = wc.scan_fwd(*[dev[k] for k in ORDER])
        need = _lib.lib().m2d_scan_fwd_noalloc_need(ctypes.byref(wc._make_desc(*[dev[k] for k in ORDER])[0]))
        assert 256 < need <= _lib.NOALLOC_SCRATCH_BYTES      # more than the status word: the ring is in use
        got = _call_noalloc(dev)
        torch.cuda.synchronize()
        scale = float(want.float().abs().max())
        assert float((got.float() - want.float()).abs().max()) <= tol * scale


def test_noalloc_rejects_problems_beyond_its_capacity():
    """Decided from the shape alone, before any device work: runs without a GPU."""
    L = _lib.lib()
    d = _lib.ScanDesc()
    d.struct_bytes = ctypes.sizeof(_lib.ScanDesc)
    d.dtype = _lib.M2D_F32
    d.B, d.H, d.W, d.E, d.N = 16, 64, 4096, 64, 16           # ring: 32 CTAs x 4096 columns x 2 KiB = 256 MiB
    d.BT_pitch = d.BL_pitch = d.C_pitch = 16
    assert L.m2d_scan_fwd_noalloc_need(ctypes.byref(d)) > _lib.NOALLOC_SCRATCH_BYTES
    fake = ctypes.c_void_p(256)                               # never dereferenced: the size check comes first
    for name in ("x", "dT", "dL", "AT", "AL", "BT", "BL", "C", "D", "y"):
        setattr(d, name, fake)
    assert L.m2d_scan_fwd_noalloc(ctypes.byref(d), None) == -9
    assert "capacity" in _lib.strerror(-9)
