"""The reference's unchanged model file resolves its scan import to this package (needs the
reference checkout; skipped where it is absent)."""
import os
import sys

import pytest

REF = os.environ.get("M2D_REFERENCE_ROOT", "/root/reference")


@pytest.mark.skipif(not os.path.exists(os.path.join(REF, "models", "mamba2d.py")), reason="reference checkout not present")
def test_reference_block_imports_replacement():
    import mamba2d_b200.inject as inject
    from mamba2d_b200 import wavefront_cuda
    inject.install_droppath_shim()
    inject.install(REF)
    saved = {k: v for k, v in sys.modules.items() if k == "models" or k.startswith("models.")}
    try:
        import importlib
        m = importlib.import_module("models.mamba2d")
        assert m.wavefront_scan_cuda is wavefront_cuda.wavefront_scan_cuda
        blk = m.M2DBlock(d_model=32)
        assert blk.AT_log.shape == (32, 16) and blk.x_proj.weight.shape == (2 * 2 + 48, 32)
    finally:
        for k in [k for k in sys.modules if k == "models" or k.startswith("models.")]:
            if k not in saved:
                del sys.modules[k]


@pytest.mark.skipif(not os.path.exists(os.path.join(REF, "models", "mamba2d.py")), reason="reference checkout not present")
@pytest.mark.parametrize("corner", ["TL", "BR"])
@pytest.mark.parametrize("local_path", [False, True])
def test_block_without_flips_equals_reference_block(corner, local_path, monkeypatch):
    """native_scan_corner() removes the flip copies of a bottom-right block.  Checked on the CPU
    with a naive PyTorch scan standing in for the kernels (forward direction by definition,
    bottom-right by flipping around it): the reference's own forward() and the patched one must
    agree on the output and on every parameter gradient."""
    import importlib
    import torch
    import mamba2d_b200.inject as inject
    from mamba2d_b200 import wavefront_cuda
    from oracle import torch_ref

    def naive(x, *w, recomp="partial", scan_start="TL"):
        if len(w) == 9:
            *w, recomp = w
        if scan_start == "BR":
            return torch_ref.scan_from_weights(x.flip(1, 2), *w).flip(1, 2)
        return torch_ref.scan_from_weights(x, *w)

    inject.install_droppath_shim()
    inject.install(REF)
    saved = {k: v for k, v in sys.modules.items() if k == "models" or k.startswith("models.")}
    try:
        m = importlib.import_module("models.mamba2d")
        monkeypatch.setattr(m, "wavefront_scan_cuda", naive)
        monkeypatch.setattr(wavefront_cuda, "wavefront_scan_cuda", naive)
        torch.manual_seed(0)
        ref_blk = m.M2DBlock(d_model=16, scan_start=corner, local_path=local_path).double()

        class Patched(m.M2DBlock):
            pass
        inject.native_scan_corner(Patched)
        new_blk = Patched(d_model=16, scan_start=corner, local_path=local_path).double()
        new_blk.load_state_dict(ref_blk.state_dict())
        x = torch.randn(2, 5, 4, 16, dtype=torch.float64)
        gy = torch.randn(2, 5, 4, 16, dtype=torch.float64)
        outs = []
        for blk in (ref_blk, new_blk):
            xi = x.clone().requires_grad_(True)
            y = blk(xi)
            grads = torch.autograd.grad(y, [xi] + list(blk.parameters()), gy)
            outs.append([y.detach()] + list(grads))
        for a, b in zip(*outs):
            assert torch.allclose(a, b, rtol=1e-10, atol=1e-12)
    finally:
        for k in [k for k in sys.modules if k == "models" or k.startswith("models.")]:
            if k not in saved:
                del sys.modules[k]
