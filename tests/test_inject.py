"""The reference's unchanged model file resolves its scan import to this package (needs the
reference checkout; skipped where it is absent)."""
import os
import sys

import pytest

from mamba2d_b200 import refmodel

REF = refmodel.reference_root() or "/root/reference"     # the checkout, or the copy the build step stages


@pytest.mark.skipif(not os.path.exists(os.path.join(REF, "models", "mamba2d.py")), reason="reference checkout not present")
def test_reference_block_imports_replacement():
    import mamba2d_b200.inject as inject
    from mamba2d_b200 import wavefront_cuda
    refmodel.purge_models_modules()
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
@pytest.mark.parametrize("fuse_act2", [False, True])
def test_block_without_flips_equals_reference_block(corner, local_path, fuse_act2, monkeypatch):
    """native_scan_corner() removes the flip copies of a bottom-right block.  Checked on the CPU
    with a naive PyTorch scan standing in for the kernels (forward direction by definition,
    bottom-right by flipping around it): the reference's own forward() and the patched one must
    agree on the output and on every parameter gradient."""
    import importlib
    import torch
    import mamba2d_b200.inject as inject
    from mamba2d_b200 import wavefront_cuda
    from oracle import torch_ref

    def naive(x, *w, recomp="partial", scan_start="TL", act_out=None):
        if len(w) == 9:
            *w, recomp = w
        y = torch_ref.scan_from_weights(x.flip(1, 2), *w).flip(1, 2) if scan_start == "BR" else torch_ref.scan_from_weights(x, *w)
        return torch.nn.functional.gelu(y) if act_out == "gelu" else y

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
        inject.native_scan_corner(Patched, fuse_act2=fuse_act2)
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


@pytest.mark.skipif(not os.path.exists(os.path.join(REF, "models", "mamba2d.py")), reason="reference checkout not present")
@pytest.mark.parametrize("corner", ["TL", "BR"])
def test_double_scan_branch_without_flips_equals_reference_ssm(corner, monkeypatch):
    """The ``double_scans`` branch of the patched ``ssm`` against the reference's own ``ssm``
    (models/mamba2d.py:180-202).  The reference's constructor rejects ``double_scans=True`` together
    with any scan corner (:46-53), so the second parameter set is attached to a block built without
    it, the way the constructor would have created it (:115-150), and the flag is set afterwards."""
    import copy
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
        torch.manual_seed(1)
        blk = m.M2DBlock(d_model=16, scan_start=corner).double()
        donor = m.M2DBlock(d_model=16).double()
        for name in ("AT_log", "AL_log", "D"):
            setattr(blk, name + "_b", torch.nn.Parameter(getattr(donor, name).detach().clone() + 0.1))
        for name in ("x_proj", "dt_projT", "dt_projL"):
            setattr(blk, name + "_b", copy.deepcopy(getattr(donor, name)))
        blk.double_scans = True

        class Patched(m.M2DBlock):
            pass
        inject.native_scan_corner(Patched)
        x = torch.randn(2, 5, 4, 16, dtype=torch.float64)
        gy = torch.randn(2, 5, 4, 16, dtype=torch.float64)
        outs = []
        for ssm in (m.M2DBlock.ssm, Patched.ssm):
            xi = (x.flip(1, 2) if (corner == "BR" and ssm is m.M2DBlock.ssm) else x).clone().requires_grad_(True)
            # the reference block hands ssm() the flipped activation for a bottom-right block and flips
            # the result back (models/mamba2d.py:162-175); the patched one never flips
            y = ssm(blk, xi)
            if corner == "BR" and ssm is m.M2DBlock.ssm:
                y = y.flip(1, 2)
            params = [p for n, p in blk.named_parameters() if not n.startswith(("in_proj", "out_proj", "local"))]
            grads = torch.autograd.grad(y, [xi] + params, gy, allow_unused=True)
            dx = grads[0].flip(1, 2) if (corner == "BR" and ssm is m.M2DBlock.ssm) else grads[0]
            outs.append([y.detach(), dx] + [g for g in grads[1:] if g is not None])
        assert len(outs[0]) == len(outs[1]) and len(outs[0]) > 10
        for a, b in zip(*outs):
            assert torch.allclose(a, b, rtol=1e-10, atol=1e-12)
    finally:
        for k in [k for k in sys.modules if k == "models" or k.startswith("models.")]:
            if k not in saved:
                del sys.modules[k]
