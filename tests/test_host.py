"""Host-side logic of the Python boundary that needs no GPU."""
import inspect

import pytest
import torch

from mamba2d_b200 import wavefront_cuda as wc
from oracle import inputs, torch_ref


def test_public_signature_matches_reference_entry():
    """Argument names and order of the reference's wavefront_scan_cuda
    (models/kernels/wavefront_cuda.py:315 in the reference); the two additions, the start corner and
    the output activation, come last and default to the reference's behaviour."""
    sig = inspect.signature(wc.wavefront_scan_cuda).parameters
    assert list(sig) == ["x", "AT_log", "AL_log", "x_proj_w", "dt_projT_w", "dt_projT_b", "dt_projL_w",
                         "dt_projL_b", "D", "recomp", "scan_start", "act_out"]
    assert sig["recomp"].default == "partial" and sig["scan_start"].default == "TL" and sig["act_out"].default is None
    pr = inspect.signature(wc.wf_cuda_fn_pr.forward).parameters
    assert list(pr)[1:] == ["x", "deltaT", "deltaL", "AT", "AL", "BT", "BL", "C", "D", "reverse", "a_log"]
    assert pr["reverse"].default is False and pr["a_log"].default is False
    assert list(inspect.signature(wc.proj_params).parameters) == \
        ["x", "AT_log", "AL_log", "x_proj_w", "dt_projT_w", "dt_projT_b", "dt_projL_w", "dt_projL_b"]


def test_value_errors_raised_before_any_device_work():
    w = inputs.make_module_params(32, 16, seed=1)
    ws = [w[k] for k in ("AT_log", "AL_log", "x_proj_w", "dt_projT_w", "dt_projT_b", "dt_projL_w", "dt_projL_b", "D")]
    with pytest.raises(ValueError, match="spatial dims"):
        wc.wavefront_scan_cuda(torch.randn(1, 1, 4, 32), *ws)
    with pytest.raises(ValueError, match="Unknown recomputation mode"):
        wc.wavefront_scan_cuda(torch.randn(1, 4, 4, 32), *ws, recomp="none")


def test_cpu_tensors_are_rejected_not_silently_computed():
    inp = inputs.make_inputs(1, 4, 4, 32, 16, seed=1)
    with pytest.raises(RuntimeError, match="no CPU path"):
        wc.scan_fwd(*[inp[k] for k in ("x", "dT", "dL", "AT", "AL", "BT", "BL", "C", "D")])


def test_shape_and_dtype_checks():
    inp = inputs.make_inputs(1, 4, 4, 32, 16, seed=1)
    a = {k: v.to("meta") for k, v in inp.items()}
    order = ("x", "dT", "dL", "AT", "AL", "BT", "BL", "C", "D")
    with pytest.raises(RuntimeError):
        wc._check_inputs(*[a[k] for k in order])               # not CUDA

    class FakeCuda(torch.Tensor):
        pass
    # shape check happens on metadata only
    bad = dict(inp)
    bad["dT"] = inp["dT"][:, :3]
    with pytest.raises(RuntimeError):
        wc._check_inputs(*[bad[k] for k in order])


def test_pixel_pitch_detection():
    inp = inputs.make_inputs(2, 5, 6, 64, 16, seed=2, strided_bc=True)
    t, pitch = wc._pixel_pitch(inp["BT"], 5, 6, 16)
    assert pitch == 2 * 4 + 3 * 16 and t.data_ptr() == inp["BT"].data_ptr()
    t, pitch = wc._pixel_pitch(inp["BT"].contiguous(), 5, 6, 16)
    assert pitch == 16
    weird = inp["BT"].permute(0, 2, 1, 3)                      # not a pixel-pitched view
    t, pitch = wc._pixel_pitch(weird, 6, 5, 16)
    assert pitch == 16 and t.is_contiguous()


def test_proj_params_equals_restatement_on_cpu():
    w = inputs.make_module_params(32, 16, seed=3)
    x = torch.randn(2, 4, 5, 32)
    names = ("AT_log", "AL_log", "x_proj_w", "dt_projT_w", "dt_projT_b", "dt_projL_w", "dt_projL_b")
    a = wc.proj_params(x, *[w[k] for k in names])
    b = torch_ref.proj_params_ref(x, *[w[k] for k in names])
    for u, v in zip(a, b):
        assert torch.equal(u, v)
    assert not a[4].is_contiguous()     # BT stays a view into the projection output


@pytest.mark.parametrize("dt,tol", [(torch.float32, 2e-6), (torch.bfloat16, 2e-2)])
def test_hand_written_projection_backward_equals_autograd(dt, tol):
    """proj_params is one autograd node with a hand-written backward; autograd through the plain
    PyTorch formulation (what the reference does, wavefront_cuda.py:63-95 and :235-302) is the
    check.  CPU tensors take the PyTorch branch of that backward."""
    E, N = 48, 16
    p = inputs.make_module_params(E, N, seed=2)
    names = ("AT_log", "AL_log", "x_proj_w", "dt_projT_w", "dt_projT_b", "dt_projL_w", "dt_projL_b")
    w = {k: (v if k.endswith("_log") else v.to(dt)) for k, v in p.items()}
    g = torch.Generator().manual_seed(3)
    x = torch.randn(2, 5, 4, E, generator=g).to(dt)

    def grads(fn):
        leaves = [x.clone().requires_grad_(True)] + [w[k].clone().requires_grad_(True) for k in names]
        out = fn(*leaves)
        gg = torch.Generator().manual_seed(4)
        gs = [torch.randn(o.shape, generator=gg).to(o.dtype) for o in out]
        return [o.detach() for o in out], torch.autograd.grad(list(out), leaves, gs)

    out_a, want = grads(torch_ref.proj_params_ref)
    out_b, got = grads(wc.proj_params)
    for a, b in zip(out_a, out_b):
        assert torch.equal(a, b)
    for name, a, b in zip(("x",) + names, want, got):
        assert a.dtype == b.dtype and a.shape == b.shape, name
        assert (a.float() - b.float()).abs().max() <= tol * a.float().abs().max(), name


def test_proj_params_gradients_survive_graph_capture():
    """proj_params traced by torch.compile (no code generator: backend "eager") must give the same
    gradients as eager mode: a custom autograd Function whose outputs alias saved tensors silently
    lost them there."""
    names = ("AT_log", "AL_log", "x_proj_w", "dt_projT_w", "dt_projT_b", "dt_projL_w", "dt_projL_b")
    w = inputs.make_module_params(32, 16, seed=4)
    x0 = torch.randn(2, 5, 4, 32, generator=torch.Generator().manual_seed(0))

    def loss(x, *ws):
        return sum((t * t).sum() for t in wc.proj_params(x, *ws))

    def run(fn):
        x = x0.clone().requires_grad_(True)
        ws = [w[k].clone().requires_grad_(True) for k in names]
        return torch.autograd.grad(fn(x, *ws), [x] + ws)

    want = run(loss)
    got = run(torch.compile(loss, backend="eager"))
    for name, a, b in zip(("x",) + names, got, want):
        assert float(b.abs().max()) > 0 and torch.allclose(a, b, rtol=1e-6, atol=0), name


def test_status_word_check_raises(monkeypatch):
    """The wrapper's reading of the status word, with a fake library and a host tensor standing in
    for the workspace: nonzero raises, zero passes, M2D_CHECK_STATUS=0 never looks."""
    import types
    import torch
    from mamba2d_b200 import wavefront_cuda as wc

    fake = types.SimpleNamespace(m2d_scan_fwd_chain=lambda d: 4, m2d_scan_fwd_status_offset=lambda d: 0,
                                 m2d_scan_bwd_chain=lambda d: 1, m2d_scan_bwd_status_offset=lambda d: 0)
    monkeypatch.setattr(wc._lib, "lib", lambda: fake)
    monkeypatch.setattr(torch.cuda, "is_current_stream_capturing", lambda: False)
    d = wc._lib.ScanDesc()
    bad = torch.zeros(256, dtype=torch.uint8)
    bad[0] = 1
    good = torch.zeros(256, dtype=torch.uint8)
    monkeypatch.setattr(wc, "_CHECK_STATUS", "auto")
    with pytest.raises(RuntimeError, match="timed out"):
        wc._check_status("fwd", d, bad)
    wc._check_status("fwd", d, good)
    wc._check_status("bwd", d, bad)              # one CTA per image: not looked at by default
    monkeypatch.setattr(wc, "_CHECK_STATUS", "1")
    with pytest.raises(RuntimeError, match="gradients are invalid"):
        wc._check_status("bwd", d, bad)
    monkeypatch.setattr(wc, "_CHECK_STATUS", "0")
    wc._check_status("fwd", d, bad)
