"""The scan's callers: the reference project's unchanged block and classifier on top of this op.

The model code is not part of this repository; it is imported from a reference checkout or from the
unmodified copy the build step stages under baseline/_ref (skipped where neither exists)."""
import copy

import pytest
import torch

from mamba2d_b200 import refmodel
from oracle import build_ref_cuda, torch_ref
from helpers import rel_err

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(refmodel.reference_root() is None, reason="no copy of the reference's models/ package")]


def _naive(x, *w, recomp="partial", scan_start="TL"):
    if len(w) == 9:
        *w, recomp = w
    if scan_start == "BR":
        return torch_ref.scan_from_weights(x.flip(1, 2), *w).flip(1, 2)
    return torch_ref.scan_from_weights(x, *w)


@pytest.mark.parametrize("corner", ["TL", "BR"])
@pytest.mark.parametrize("native", [False, True])
def test_block_forward_backward_through_the_kernels(corner, native, monkeypatch):
    """One M2DBlock (models/mamba2d.py:157-202, with the local path) forward + backward on the GPU
    through the real kernels, against the same block in fp64 on the CPU with a naive scan."""
    m, _ = refmodel.import_reference_models(native_corner=native)
    torch.manual_seed(0)
    blk = m.M2DBlock(d_model=64, local_path=True, scan_start=corner)
    g = torch.Generator().manual_seed(1)
    x, gy = torch.randn(2, 12, 10, 64, generator=g), torch.randn(2, 12, 10, 64, generator=g)

    gblk = copy.deepcopy(blk).cuda()
    xg = x.cuda().requires_grad_(True)
    y = gblk(xg)
    got = [y.detach()] + list(torch.autograd.grad(y, [xg] + list(gblk.parameters()), gy.cuda()))

    m2, _ = refmodel.import_reference_models(native_corner=False)
    monkeypatch.setattr(m2, "wavefront_scan_cuda", _naive)
    cblk = m2.M2DBlock(d_model=64, local_path=True, scan_start=corner).double()
    cblk.load_state_dict(blk.state_dict())
    xc = x.double().requires_grad_(True)
    yc = cblk(xc)
    want = [yc.detach()] + list(torch.autograd.grad(yc, [xc] + list(cblk.parameters()), gy.double()))
    names = ["y", "d_x"] + [n for n, _ in cblk.named_parameters()]
    assert len(got) == len(want) == len(names)
    for n, a, b in zip(names, got, want):
        assert rel_err(a.cpu().numpy(), b.numpy()) < 2e-4, n
    refmodel.purge_models_modules()


@pytest.mark.skipif(build_ref_cuda.find() is None, reason="reference CUDA extension not prebuilt")
def test_classifier_logits_match_the_reference_kernels():
    """The whole M2D-T classifier (fp32, two images): the reference model calling this op against the
    same model, same weights, calling the reference's own kernels through its own Python module."""
    import importlib
    import bench
    g = torch.Generator().manual_seed(3)
    x = torch.randn(2, 3, 224, 224, generator=g).cuda().contiguous(memory_format=torch.channels_last)
    logits, state = {}, None
    for v in ("ours", "ours_native_corner", "ours_native_corner_fused_act", "reference"):
        if v == "reference":
            bench.load_reference_module()
            mods = (importlib.import_module("models.mamba2d"), importlib.import_module("models.utils"))
        else:
            mods = refmodel.import_reference_models(native_corner=(v != "ours"), fuse_act2=v.endswith("fused_act"))
        torch.manual_seed(0)
        model = refmodel.build_classifier("M2D-T", mods).cuda().eval()
        if state is None:
            state = {k: t.clone() for k, t in model.state_dict().items()}
        else:
            model.load_state_dict(state)
        with torch.inference_mode():
            logits[v] = model(x).float().cpu().numpy()
        del model
    refmodel.purge_models_modules()
    assert rel_err(logits["ours"], logits["reference"]) < 1e-3
    assert rel_err(logits["ours_native_corner"], logits["reference"]) < 1e-3
    assert rel_err(logits["ours_native_corner_fused_act"], logits["reference"]) < 1e-3


def test_block_under_autocast_takes_the_fused_projection_kernels(monkeypatch):
    """The shipped precision is bf16-mixed: inside the block the activation reaching the scan is bf16
    and the entry casts the projection weights to it, so the fused projection kernels (not the
    PyTorch formulation) must run, forward and backward, and the result must agree with the fp32 run."""
    from mamba2d_b200 import wavefront_cuda as wc
    m, _ = refmodel.import_reference_models()
    torch.manual_seed(0)
    blk = m.M2DBlock(d_model=64, local_path=True).cuda()
    g = torch.Generator().manual_seed(2)
    x, gy = torch.randn(4, 14, 14, 64, generator=g).cuda(), torch.randn(4, 14, 14, 64, generator=g).cuda()
    calls = {"fwd": 0, "bwd": 0}
    f0, b0 = wc._dtproj_fwd, wc._dtproj_bwd
    monkeypatch.setitem(wc._EAGER, wc.dtproj_fwd_op, lambda *a: (calls.__setitem__("fwd", calls["fwd"] + 1), f0(*a))[1])
    monkeypatch.setitem(wc._EAGER, wc.dtproj_bwd_op, lambda *a: (calls.__setitem__("bwd", calls["bwd"] + 1), b0(*a))[1])

    def run(autocast):
        xi = x.clone().requires_grad_(True)
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=autocast):
            y = blk(xi)
        grads = torch.autograd.grad(y.float(), [xi] + list(blk.parameters()), gy)
        return [y.detach().float()] + [t.float() for t in grads]

    ref = run(False)
    n_fp32 = dict(calls)
    got = run(True)
    assert n_fp32 == {"fwd": 1, "bwd": 1} and calls == {"fwd": 2, "bwd": 2}
    for k, (a, b) in enumerate(zip(got, ref)):
        # y and d_x at the bf16 bar; parameter gradients are long bf16 sums (some of them scalars)
        assert rel_err(a.cpu().numpy(), b.cpu().numpy()) < (3e-2 if k < 2 else 1e-1)
    refmodel.purge_models_modules()
