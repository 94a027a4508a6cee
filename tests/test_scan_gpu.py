"""GPU parity: the CUDA path (through the C ABI) against the CPU oracle and the committed
fixtures.  Tolerances are the ones the task states: max-abs error <= 1e-4 x output scale for
fp32, <= 2e-2 x output scale for bf16 inputs."""
import numpy as np
import pytest
import torch

from oracle import cpu, inputs
from helpers import GRADS, SCAN_GOLDEN, bf16_round_inputs, load_scan_golden, rel_err, sub

pytestmark = pytest.mark.gpu

TOL = {"f32": 1e-4, "bf16": 2e-2}
TDT = {"f32": torch.float32, "bf16": torch.bfloat16}
ORDER = ("x", "dT", "dL", "AT", "AL", "BT", "BL", "C", "D")


def to_dev(inp, dt):
    """Move a dict of fp32 CPU tensors to the GPU in dtype dt, keeping strided B/C views strided."""
    out = {}
    for k, v in inp.items():
        if not v.is_contiguous():
            base = v._base if v._base is not None else v
            gb = base.to("cuda", dt)
            out[k] = gb.as_strided(v.shape, v.stride(), v.storage_offset())
        else:
            out[k] = v.to("cuda", dt)
    return out


def run_fwd(inp, kind):
    from mamba2d_b200 import scan_fwd
    d = to_dev(inp, TDT[kind])
    y = scan_fwd(*[d[k] for k in ORDER])
    torch.cuda.synchronize()
    return y.float().cpu().numpy()


def run_bwd(inp, kind):
    from mamba2d_b200 import scan_bwd
    d = to_dev(inp, TDT[kind])
    g = scan_bwd(*[d[k] for k in ORDER], d["gy"])
    torch.cuda.synchronize()
    return {k: t.float().cpu().numpy() for k, t in zip(GRADS, g)}


FWD_SHAPES = [
    (2, 32, 32, 64, 16),    # benchmark config 0
    (2, 5, 4, 6, 4),        # ragged channels / states (scalar-load path)
    (1, 2, 2, 32, 16),      # smallest legal map
    (3, 7, 7, 64, 16),      # one band, several images chained
    (2, 14, 14, 96, 16),
    (1, 28, 28, 128, 16),   # several bands
    (1, 56, 56, 64, 16),
    (1, 9, 13, 40, 12),     # non-square, E and N not multiples of the warp tile
    (1, 13, 3, 32, 16),     # narrow map: band height limited by W
    (5, 3, 19, 32, 8),
    (1, 64, 64, 32, 16),
    (1, 200, 136, 64, 16),  # large map, one image: many CTAs chained along the bands of the image
    (2, 96, 40, 32, 16),
    (1, 2400, 24, 32, 16),  # more bands than resident CTAs: the chain closes into a ring
    (300, 13, 3, 32, 16),   # many narrow maps: batch mode with one row per band (a boundary is read two steps after it is written)
    (300, 11, 4, 32, 16),   # ... two rows per band
    (300, 20, 2, 32, 16),   # two columns: batch mode falls back to the flat step loop
]


@pytest.mark.parametrize("shape", FWD_SHAPES)
@pytest.mark.parametrize("kind", ["f32", "bf16"])
@pytest.mark.parametrize("strided", [False, True])
def test_forward_matches_oracle(shape, kind, strided):
    inp = inputs.make_inputs(*shape, seed=sum(shape), strided_bc=strided)
    if kind == "bf16":
        ref_in = bf16_round_inputs(inp)
    else:
        ref_in = inp
    y_ref = cpu.forward(ref_in, "f64")
    y = run_fwd(inp, kind)
    assert rel_err(y, y_ref) < TOL[kind]


@pytest.mark.parametrize("kind", ["f32", "bf16"])
def test_forward_scan_term_alone(kind):
    """With D = 0 the skip term cannot mask an error in the recurrence."""
    inp = inputs.make_inputs(2, 28, 28, 64, 16, seed=4)
    inp["D"] = torch.zeros_like(inp["D"])
    ref_in = bf16_round_inputs(inp) if kind == "bf16" else inp
    y_ref = cpu.forward(ref_in, "f64")
    y = run_fwd(inp, kind)
    assert rel_err(y, y_ref) < TOL[kind]


@pytest.mark.parametrize("name", sorted(SCAN_GOLDEN))
def test_forward_matches_reference_fixture(name):
    strided, kind = SCAN_GOLDEN[name]
    if kind == "f64":
        pytest.skip("fp64 is not a dtype of the CUDA path")
    inp, g = load_scan_golden(name)
    y = run_fwd(inp, kind)
    assert rel_err(sub(y), g["y"]) < TOL[kind]


BWD_SHAPES = [
    (2, 32, 32, 64, 16),
    (2, 5, 4, 6, 4),
    (1, 2, 2, 32, 16),
    (3, 7, 7, 64, 16),
    (2, 14, 14, 96, 16),
    (1, 28, 28, 128, 16),
    (1, 56, 56, 64, 16),
    (1, 9, 13, 40, 12),
    (1, 13, 3, 32, 16),
    (5, 3, 19, 32, 8),
    (1, 120, 72, 64, 16),   # large map, one image: chained CTAs in both sweeps of the backward
    (2, 96, 40, 32, 16),
    (1, 2000, 20, 32, 16),  # more bands than resident CTAs: the chain closes into a ring
    (300, 13, 3, 32, 16),   # many narrow maps: batch mode with one row per band
    (300, 11, 4, 32, 16),   # ... two rows per band
    (300, 20, 2, 32, 16),   # two columns: batch mode falls back to the flat step loops
]


@pytest.mark.parametrize("shape", BWD_SHAPES)
@pytest.mark.parametrize("kind", ["f32", "bf16"])
@pytest.mark.parametrize("strided", [False, True])
def test_backward_matches_oracle(shape, kind, strided):
    inp = inputs.make_inputs(*shape, seed=sum(shape) + 1, strided_bc=strided)
    ref_in = bf16_round_inputs(inp) if kind == "bf16" else inp
    ref = cpu.backward(ref_in, mode="f64")
    got = run_bwd(inp, kind)
    for k in GRADS:
        assert rel_err(got[k], ref[k]) < TOL[kind], k


@pytest.mark.parametrize("name", sorted(SCAN_GOLDEN))
def test_backward_matches_reference_fixture(name):
    strided, kind = SCAN_GOLDEN[name]
    if kind == "f64":
        pytest.skip("fp64 is not a dtype of the CUDA path")
    inp, g = load_scan_golden(name)
    got = run_bwd(inp, kind)
    for k in GRADS:
        assert rel_err(sub(got[k]), g[k]) < TOL[kind], k


def test_backward_twice_same_workspace_sizes():
    """Accumulators are re-zeroed on every call: two calls give the same answer."""
    inp = inputs.make_inputs(2, 14, 14, 64, 16, seed=9)
    a = run_bwd(inp, "f32")
    b = run_bwd(inp, "f32")
    for k in GRADS:
        assert rel_err(a[k], b[k]) < 1e-5, k


@pytest.mark.parametrize("kind", ["f32", "bf16"])
@pytest.mark.parametrize("reverse", [False, True])
def test_forward_with_output_gelu(kind, reverse):
    """The GELU the block applies after the scan, folded into the kernel's store, against the oracle's
    y passed through the erf-form GELU in fp64."""
    from mamba2d_b200 import scan_fwd
    from scipy.special import erf
    inp = inputs.make_inputs(3, 20, 9, 96, 16, seed=31)
    ref_in = bf16_round_inputs(inp) if kind == "bf16" else inp
    if reverse:
        flipped = {k: (v.flip(1, 2).contiguous() if v.dim() == 4 else v) for k, v in ref_in.items()}
        y_ref = np.flip(cpu.forward(flipped, "f64"), (1, 2))
    else:
        y_ref = cpu.forward(ref_in, "f64")
    want = 0.5 * y_ref * (1.0 + erf(y_ref / np.sqrt(2.0)))
    d = to_dev(inp, TDT[kind])
    got = scan_fwd(*[d[k] for k in ORDER], reverse=reverse, gelu_out=True)
    torch.cuda.synchronize()
    assert rel_err(got.float().cpu().numpy(), want) < TOL[kind]


@pytest.mark.parametrize("kind", ["f32", "bf16"])
def test_a_log_inside_the_kernels(kind):
    """AT / AL given as the fp32 parameters A_log: same y and gradients as with A = -exp(A_log) computed
    outside (rounded to the I/O type, as the reference's cast does), and d_A_log = d_A * A in fp32."""
    from mamba2d_b200 import scan_bwd, scan_fwd
    inp = inputs.make_inputs(3, 15, 11, 64, 16, seed=41)
    d = to_dev(inp, TDT[kind])
    g = torch.Generator().manual_seed(5)
    AT_log = (torch.rand(64, 16, generator=g) * 2.5).cuda()
    AL_log = (torch.rand(64, 16, generator=g) * 2.5).cuda()
    AT32, AL32 = -torch.exp(AT_log), -torch.exp(AL_log)
    a_out = dict(d, AT=AT32.to(TDT[kind]), AL=AL32.to(TDT[kind]))
    a_in = dict(d, AT=AT_log, AL=AL_log)
    y0 = scan_fwd(*[a_out[k] for k in ORDER])
    y1 = scan_fwd(*[a_in[k] for k in ORDER], a_log=True)
    g0 = scan_bwd(*[a_out[k] for k in ORDER], d["gy"])
    g1 = scan_bwd(*[a_in[k] for k in ORDER], d["gy"], a_log=True)
    torch.cuda.synchronize()
    tol = 1e-5 if kind == "f32" else 1e-2
    assert rel_err(y1.float().cpu().numpy(), y0.float().cpu().numpy()) < tol
    for name, u, v in zip(GRADS, g1, g0):
        if name in ("d_AT", "d_AL"):
            assert u.dtype == torch.float32
            v = v.float() * (AT32 if name == "d_AT" else AL32)
        assert rel_err(u.float().cpu().numpy(), v.float().cpu().numpy()) < tol, name
