"""The benchmark's full-size shapes (batch 128) through size-independent properties, plus an oracle
check on a slice: the CPU oracle cannot cover 128 images in seconds, but the scan is independent per
image, linear in x for fixed gates and linear in the upstream gradient."""
import numpy as np
import pytest
import torch

from oracle import cpu, inputs
from helpers import GRADS, rel_err

pytestmark = pytest.mark.gpu
ORDER = ("x", "dT", "dL", "AT", "AL", "BT", "BL", "C", "D")
STAGES = [(64, 56), (128, 28), (320, 14), (512, 7)]


def _dev(inp, dt):
    out = {}
    for k, v in inp.items():
        if not v.is_contiguous():
            base = v._base
            out[k] = base.to("cuda", dt).as_strided(v.shape, v.stride(), v.storage_offset())
        else:
            out[k] = v.to("cuda", dt)
    return out


@pytest.mark.parametrize("D,HW", STAGES)
def test_full_batch_properties_fp32(D, HW):
    from mamba2d_b200 import scan_bwd, scan_fwd
    inp = inputs.make_inputs(128, HW, HW, D, 16, seed=0, strided_bc=True)
    d = _dev(inp, torch.float32)
    a = [d[k] for k in ORDER]
    y = scan_fwd(*a)
    g = scan_bwd(*a, d["gy"])
    # (1) images are independent: the first and the last two images against the oracle run on them alone
    for sl in (slice(0, 2), slice(126, 128)):
        sub_in = {k: (v[sl].contiguous() if v.dim() == 4 else v) for k, v in inp.items()}
        y_ref = cpu.forward(sub_in, "f64")
        g_ref = cpu.backward(sub_in, mode="f64")
        assert rel_err(y[sl].cpu().numpy(), y_ref) < 1e-4
        for name, idx in (("d_x", 0), ("d_dT", 1), ("d_dL", 2), ("d_BT", 5), ("d_BL", 6), ("d_C", 7)):
            assert rel_err(g[idx][sl].cpu().numpy(), g_ref[name]) < 1e-4, name
    # (2) y is linear in x for fixed gates
    a2 = list(a)
    a2[0] = d["x"] * 2
    y2 = scan_fwd(*a2)
    assert float((y2 - 2 * y).abs().max() / y.abs().max()) < 1e-5
    # (3) every gradient is linear in the upstream gradient
    g3 = scan_bwd(*a, d["gy"] * -3.0)
    for name, u, v in zip(GRADS, g, g3):
        assert float((v + 3.0 * u).abs().max() / u.abs().max()) < 1e-4, name
    # (4) closed forms that need no recurrence: d_D = sum gy*x over (b,i,j)
    dD = (d["gy"].double() * d["x"].double()).sum(dim=(0, 1, 2))
    assert float((g[8].double() - dD).abs().max() / dD.abs().max()) < 1e-4
    # (5) batch sums: d_AT over all images equals the sum of per-half results
    h = 64
    lo = scan_bwd(*[t[:h].contiguous() if t.dim() == 4 else t for t in a], d["gy"][:h].contiguous())
    hi = scan_bwd(*[t[h:].contiguous() if t.dim() == 4 else t for t in a], d["gy"][h:].contiguous())
    for idx in (3, 4, 8):
        assert float((lo[idx] + hi[idx] - g[idx]).abs().max() / g[idx].abs().max()) < 1e-4


@pytest.mark.parametrize("D,HW", STAGES)
def test_full_batch_bf16_against_oracle(D, HW):
    """bf16 I/O at the benchmark's full batch, all four stage shapes: the first and the last two images
    against the fp64 oracle run on the same bf16-rounded inputs (2e-2 of the output scale), and the
    batch sums against the fp32 path on the same values."""
    from mamba2d_b200 import scan_bwd, scan_fwd
    inp = inputs.make_inputs(128, HW, HW, D, 16, seed=1, strided_bc=True)
    d16 = _dev(inp, torch.bfloat16)
    a = [d16[k] for k in ORDER]
    y = scan_fwd(*a)
    g = scan_bwd(*a, d16["gy"])
    rounded = {k: v.to(torch.bfloat16).float() for k, v in inp.items()}
    for sl in (slice(0, 2), slice(126, 128)):
        sub_in = {k: (v[sl].contiguous() if v.dim() == 4 else v) for k, v in rounded.items()}
        y_ref = cpu.forward(sub_in, "f64")
        g_ref = cpu.backward(sub_in, mode="f64")
        assert rel_err(y[sl].float().cpu().numpy(), y_ref) < 2e-2
        for name, idx in (("d_x", 0), ("d_dT", 1), ("d_dL", 2), ("d_BT", 5), ("d_BL", 6), ("d_C", 7)):
            assert rel_err(g[idx][sl].float().cpu().numpy(), g_ref[name]) < 2e-2, name
    d32 = {k: v.float() for k, v in d16.items()}
    g32 = scan_bwd(*[d32[k].contiguous() for k in ORDER], d32["gy"])
    for idx in (3, 4, 8):      # d_AT, d_AL, d_D: sums over all 128 images
        assert float((g[idx].float() - g32[idx]).abs().max() / g32[idx].abs().max()) < 2e-2


def test_custom_ops_pass_opcheck():
    """Schema, fake (meta) implementation and functionalisation of the two custom ops, as
    torch.compile needs them."""
    from mamba2d_b200 import wavefront_cuda as wc
    inp = inputs.make_inputs(2, 6, 5, 32, 16, seed=3)
    d = {k: v.cuda() for k, v in inp.items()}
    a = tuple(d[k] for k in ORDER)
    torch.library.opcheck(wc.scan_fwd_op, a, test_utils=("test_schema", "test_faketensor"))
    torch.library.opcheck(wc.scan_bwd_op, a + (d["gy"],), test_utils=("test_schema", "test_faketensor"))
