"""The op as the backbone calls it: wavefront_scan_cuda(x, weights..., recomp) with autograd,
against fixtures produced by the reference project's own Python + kernel code run on the CPU."""
import os

import numpy as np
import pytest
import torch

from oracle import inputs
from helpers import GOLDEN, rel_err, sub

pytestmark = pytest.mark.gpu

WNAMES = ("AT_log", "AL_log", "x_proj_w", "dt_projT_w", "dt_projT_b", "dt_projL_w", "dt_projL_b", "D")


def _load(name):
    g = np.load(os.path.join(GOLDEN, f"{name}.npz"))
    B, H, W, E, N = (int(v) for v in g["shape"])
    seed = int(g["seed"])
    w = inputs.make_module_params(E, N, seed=seed)
    gen = torch.Generator().manual_seed(seed + 100)
    x = torch.randn(B, H, W, E, generator=gen)
    gy = torch.randn(B, H, W, E, generator=gen)
    return g, w, x, gy


@pytest.mark.parametrize("name,dt,tol", [("entry_f32", torch.float32, 1e-4), ("entry_bf16", torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("recomp", ["partial", "full"])
def test_entry_matches_reference_fixture(name, dt, tol, recomp):
    from mamba2d_b200 import wavefront_scan_cuda
    g, w, x0, gy = _load(name)
    x = x0.to("cuda", dt).requires_grad_(True)
    ws = [w[k].clone().cuda().requires_grad_(True) for k in WNAMES]
    y = wavefront_scan_cuda(x, *ws, recomp)
    assert y.dtype == dt and y.shape == x.shape and y.is_contiguous()
    grads = torch.autograd.grad(y, [x] + ws, gy.to("cuda", dt))
    assert rel_err(sub(y), g[f"{recomp}_y"]) < tol
    assert rel_err(sub(grads[0]), g[f"{recomp}_d_x"]) < tol
    # weight gradients pass through bf16 GEMMs on both sides; allow the bf16 bar for those
    for k, gr in zip(WNAMES, grads[1:]):
        assert gr.dtype == torch.float32
        assert rel_err(sub(gr), g[f"{recomp}_d_{k}"]) < (tol if dt == torch.float32 else 4e-2), k


def test_entry_errors_match_reference():
    from mamba2d_b200 import wavefront_scan_cuda
    w = inputs.make_module_params(32, 16, seed=1)
    ws = [w[k].cuda() for k in WNAMES]
    with pytest.raises(ValueError):
        wavefront_scan_cuda(torch.randn(1, 1, 8, 32, device="cuda"), *ws)
    with pytest.raises(ValueError):
        wavefront_scan_cuda(torch.randn(1, 8, 1, 32, device="cuda"), *ws)
    with pytest.raises(ValueError):
        wavefront_scan_cuda(torch.randn(1, 4, 4, 32, device="cuda"), *ws, "sometimes")


def test_entry_autocast_and_inference_mode():
    from mamba2d_b200 import wavefront_scan_cuda
    w = inputs.make_module_params(64, 16, seed=2)
    ws = [w[k].cuda() for k in WNAMES]
    x = torch.randn(2, 8, 8, 64, device="cuda")
    with torch.inference_mode():
        y32 = wavefront_scan_cuda(x, *ws)
        y16 = wavefront_scan_cuda(x.bfloat16(), *ws)
    assert y16.dtype == torch.bfloat16
    assert rel_err(y16.float().cpu().numpy(), y32.cpu().numpy()) < 3e-2


def test_no_cpu_fallback():
    from mamba2d_b200 import scan_fwd
    inp = inputs.make_inputs(1, 4, 4, 32, 16, seed=1)
    with pytest.raises(RuntimeError):
        scan_fwd(*[inp[k] for k in ("x", "dT", "dL", "AT", "AL", "BT", "BL", "C", "D")])


@pytest.mark.parametrize("recomp", ["partial", "full"])
def test_entry_inside_a_compiled_graph(recomp):
    """torch.compile traces through the entry: the kernels appear as opaque registered operators
    (with fake implementations).  The aot_eager backend keeps the rest of the graph in plain
    PyTorch, so the test exercises tracing, functionalisation and autograd, not a code generator."""
    from mamba2d_b200 import wavefront_scan_cuda
    w = inputs.make_module_params(64, 16, seed=4)
    gen = torch.Generator().manual_seed(9)
    x0 = torch.randn(2, 9, 7, 64, generator=gen)
    gy = torch.randn(2, 9, 7, 64, generator=gen).cuda()

    def run(fn):
        x = x0.cuda().requires_grad_(True)
        ws = [w[k].clone().cuda().requires_grad_(True) for k in WNAMES]
        y = fn(x, *ws)
        return [y.detach()] + list(torch.autograd.grad(y, [x] + ws, gy))

    eager = run(lambda x, *ws: wavefront_scan_cuda(x, *ws, recomp))
    compiled = run(torch.compile(lambda x, *ws: wavefront_scan_cuda(x, *ws, recomp), backend="aot_eager"))
    for name, a, b in zip(("y", "d_x") + tuple("d_" + k for k in WNAMES), compiled, eager):
        assert rel_err(a.cpu().numpy(), b.cpu().numpy()) < 1e-5, name


@pytest.mark.parametrize("dt,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_entry_step_replays_from_a_cuda_graph(dt, tol):
    """Forward + backward of the entry captured in a CUDA graph: every call of the library is
    asynchronous on the capturing stream and allocates only through the caller's allocator, so the
    step can be replayed without Python in the loop.  With bf16 tensors the capture contains the
    tensor-core weight gradient, whose TMA descriptors are kernel arguments."""
    from mamba2d_b200 import wavefront_scan_cuda
    w = inputs.make_module_params(64, 16, seed=6)
    gen = torch.Generator().manual_seed(12)
    x = torch.randn(4, 14, 14, 64, generator=gen).to("cuda", dt).requires_grad_(True)
    gy = torch.randn(4, 14, 14, 64, generator=gen).to("cuda", dt)
    ws = [(w[k].clone().cuda() if k.endswith("_log") else w[k].clone().to("cuda", dt)).requires_grad_(True) for k in WNAMES]

    def step():
        for t in [x] + ws:
            t.grad = None
        y = wavefront_scan_cuda(x, *ws)
        y.backward(gy)
        return y

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            step()
    torch.cuda.current_stream().wait_stream(side)
    y_ref = step().detach().clone()
    g_ref = [t.grad.clone() for t in [x] + ws]
    graph = torch.cuda.CUDAGraph()
    for t in [x] + ws:
        t.grad = None
    with torch.cuda.graph(graph):
        y = wavefront_scan_cuda(x, *ws)
        y.backward(gy)
    with torch.no_grad():
        x.mul_(0.5)                        # new input values in the captured buffers
    graph.replay()
    with torch.no_grad():
        x.mul_(2.0)
    graph.replay()
    torch.cuda.synchronize()
    assert rel_err(y.detach().float().cpu().numpy(), y_ref.float().cpu().numpy()) < tol / 10
    for name, t, r in zip(("x",) + WNAMES, [x] + ws, g_ref):
        assert rel_err(t.grad.float().cpu().numpy(), r.float().cpu().numpy()) < tol, name


@pytest.mark.parametrize("recomp", ["partial", "full"])
def test_entry_inside_an_inductor_graph(recomp, monkeypatch):
    """The reference compiles its classifier's forward with the default code-generating backend
    (models/mamba2d_classifier.py:62).  Same check as above with that backend and a little PyTorch
    arithmetic around the op for the code generator to fuse; guards in particular against outputs
    that share storage with saved tensors losing their gradient under the graph compiler."""
    from mamba2d_b200 import wavefront_scan_cuda
    monkeypatch.setenv("CXX", "/usr/bin/g++")      # the host compiler the code generator may call
    monkeypatch.setenv("CC", "/usr/bin/gcc")
    torch._dynamo.reset()
    w = inputs.make_module_params(64, 16, seed=5)
    gen = torch.Generator().manual_seed(10)
    x0 = torch.randn(2, 8, 6, 64, generator=gen)
    gy = torch.randn(2, 8, 6, 64, generator=gen).cuda()

    def block(x, *ws):
        return torch.nn.functional.gelu(wavefront_scan_cuda(torch.nn.functional.gelu(x), *ws, recomp)) * 2.0

    def run(fn):
        x = x0.cuda().requires_grad_(True)
        ws = [w[k].clone().cuda().requires_grad_(True) for k in WNAMES]
        y = fn(x, *ws)
        return [y.detach()] + list(torch.autograd.grad(y, [x] + ws, gy))

    eager = run(block)
    compiled = run(torch.compile(block))
    for name, a, b in zip(("y", "d_x") + tuple("d_" + k for k in WNAMES), compiled, eager):
        assert float(b.abs().max()) > 0, name
        assert rel_err(a.cpu().numpy(), b.cpu().numpy()) < 1e-4, name


def test_entry_output_activation_with_and_without_gradients():
    """act_out="gelu": folded into the kernel where nothing is differentiated, an ordinary op under
    autograd; both equal gelu(entry)."""
    from mamba2d_b200 import wavefront_scan_cuda
    w = inputs.make_module_params(64, 16, seed=7)
    gen = torch.Generator().manual_seed(13)
    x = torch.randn(2, 11, 8, 64, generator=gen).cuda()
    gy = torch.randn(2, 11, 8, 64, generator=gen).cuda()
    ws = [w[k].clone().cuda() for k in WNAMES]
    with torch.no_grad():
        plain = torch.nn.functional.gelu(wavefront_scan_cuda(x, *ws))
        fused = wavefront_scan_cuda(x, *ws, act_out="gelu")
        fused_br = wavefront_scan_cuda(x, *ws, "full", scan_start="BR", act_out="gelu")
        plain_br = torch.nn.functional.gelu(wavefront_scan_cuda(x, *ws, "full", scan_start="BR"))
    assert rel_err(fused.cpu().numpy(), plain.cpu().numpy()) < 1e-5
    assert rel_err(fused_br.cpu().numpy(), plain_br.cpu().numpy()) < 1e-5
    xg = x.clone().requires_grad_(True)
    wg = [t.clone().requires_grad_(True) for t in ws]
    a = torch.autograd.grad(wavefront_scan_cuda(xg, *wg, act_out="gelu"), [xg] + wg, gy)
    b = torch.autograd.grad(torch.nn.functional.gelu(wavefront_scan_cuda(xg, *wg)), [xg] + wg, gy)
    for u, v in zip(a, b):
        assert rel_err(u.cpu().numpy(), v.cpu().numpy()) < 1e-5
    with pytest.raises(ValueError):
        wavefront_scan_cuda(x, *ws, act_out="relu")
