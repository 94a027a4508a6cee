"""Large maps with few images (the resolution sweep of the baseline description: B=1, D=64, fp32,
H=W from 128 to 2048): here every image is shared by a chain of CTAs, each owning every chain-th
band, and the chain closes into a ring when there are more bands than resident CTAs.  The forward is
checked against the reference project's own CUDA kernels on the same GPU up to 1024x1024 (their
state tensor would take 17 GB at 2048x2048) and against the fp64 CPU oracle at 2048x2048; the
backward against the reference's kernels at 256x256 and at a detection-style shape."""
import numpy as np
import pytest
import torch

from oracle import cpu, inputs, ref_gpu
from helpers import GRADS, rel_err

pytestmark = pytest.mark.gpu
ORDER = ("x", "dT", "dL", "AT", "AL", "BT", "BL", "C", "D")
HAVE_REF = ref_gpu.build_ref_cuda.find() is not None


def _dev(inp):
    return {k: v.to("cuda") for k, v in inp.items()}


@pytest.mark.skipif(not HAVE_REF, reason="reference CUDA extension not prebuilt")
@pytest.mark.parametrize("hw", [128, 256, 512, 1024])
def test_forward_resolution_sweep_matches_reference_kernels(hw):
    from mamba2d_b200 import scan_fwd
    inp = inputs.make_inputs(1, hw, hw, 64, 16, seed=hw)
    d = _dev(inp)
    a = [d[k] for k in ORDER]
    torch.cuda.synchronize()
    y_ref = ref_gpu.forward(*a)
    torch.cuda.synchronize()
    y = scan_fwd(*a)
    torch.cuda.synchronize()
    assert rel_err(y.cpu().numpy(), y_ref.cpu().numpy()) < 1e-4
    del y_ref
    torch.cuda.empty_cache()


def test_forward_2048_matches_oracle():
    from mamba2d_b200 import scan_fwd
    inp = inputs.make_inputs(1, 2048, 2048, 64, 16, seed=2048)
    d = _dev(inp)
    y = scan_fwd(*[d[k] for k in ORDER])
    torch.cuda.synchronize()
    y_ref = cpu.forward(inp, "f64")
    assert rel_err(y.cpu().numpy(), y_ref) < 1e-4


@pytest.mark.skipif(not HAVE_REF, reason="reference CUDA extension not prebuilt")
@pytest.mark.parametrize("shape", [(1, 256, 256, 64, 16), (2, 200, 336, 64, 16)])
def test_backward_large_map_matches_reference_kernels(shape):
    from mamba2d_b200 import scan_bwd
    inp = inputs.make_inputs(*shape, seed=sum(shape))
    d = _dev(inp)
    a = [d[k] for k in ORDER]
    torch.cuda.synchronize()
    g_ref = [t.cpu().numpy() for t in ref_gpu.backward(*a, d["gy"])]
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    g = scan_bwd(*a, d["gy"])
    torch.cuda.synchronize()
    for name, ours, ref in zip(GRADS, g, g_ref):
        assert rel_err(ours.cpu().numpy(), ref) < 1e-4, name


def test_reverse_direction_on_a_chained_map():
    """The bottom-right scan on a map that runs several CTAs per image, against the oracle on flipped inputs."""
    from mamba2d_b200 import scan_bwd, scan_fwd
    inp = inputs.make_inputs(1, 160, 96, 32, 16, seed=5)
    d = _dev(inp)
    a = [d[k] for k in ORDER]
    y = scan_fwd(*a, reverse=True)
    g = scan_bwd(*a, d["gy"], reverse=True)
    torch.cuda.synchronize()
    flipped = {k: (v.flip(1, 2).contiguous() if v.dim() == 4 else v) for k, v in inp.items()}
    y_ref = np.flip(cpu.forward(flipped, "f64"), (1, 2))
    g_ref = cpu.backward(flipped, mode="f64")
    assert rel_err(y.cpu().numpy(), y_ref) < 1e-4
    for name, ours in zip(GRADS, g):
        ref = g_ref[name]
        if ref.ndim == 4:
            ref = np.flip(ref, (1, 2))
        assert rel_err(ours.cpu().numpy(), ref) < 1e-4, name
