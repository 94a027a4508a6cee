"""Run one shape of the scan a few times on the current GPU: the command line used for ncu
captures and for one-off timings.

    python -m mamba2d_b200.profile_case --shape 128,56,56,64 [--dtype f32|bf16] [--bwd] [--iters 3]
    python -m mamba2d_b200.profile_case --sweep 64,128,256,512,1024 [--reference]
    python -m mamba2d_b200.profile_case --shape 2,200,336,64 --bwd --time [--reference]
    python -m mamba2d_b200.profile_case --shape 128,56,56,64 --bwd --time --corner BR
    python -m mamba2d_b200.profile_case --shape 128,56,56,64 --entry [--kernels]
    python -m mamba2d_b200.profile_case --shape 128,56,56,64 --entry --once      (one step, for ncu)

Inputs are seeded synthetic tensors (N = 16 states, BT/BL/C as strided views of one projection
buffer).  ``--time`` prints CUDA-event timings; ``--reference`` also times the reference
project's own CUDA extension when it has been prebuilt (oracle/_ref/), for comparison.
``--corner BR`` times the scan from the bottom-right corner and, beside it, the reference's way
of getting that direction: flip copies of every per-pixel tensor, the top-left scan, flip back.
``--entry`` times forward + backward of the module-level entry (projections included) in both
recomputation modes, and the same with the projections in plain PyTorch under autograd (the
reference's formulation) around the same scan kernels; ``--kernels`` adds the per-kernel device
times of one partial-recomputation step (torch.profiler, CUPTI activity records).
"""
import argparse
import math
import os
import sys

import torch
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORDER = ("x", "dT", "dL", "AT", "AL", "BT", "BL", "C", "D")


def make_inputs(B, H, W, E, N=16, seed=0, dtype=torch.float32, device="cuda", strided=True):
    """Same draws, in the same order, as the test-suite generator (x, dT, dL, BT, BL, C, AT, AL, D, gy)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(B, H, W, E, generator=g)
    dT = F.softplus(torch.randn(B, H, W, E, generator=g) * 0.5 - 2.0)
    dL = F.softplus(torch.randn(B, H, W, E, generator=g) * 0.5 - 2.0)
    std = N ** -0.5
    BT, BL, C = (torch.randn(B, H, W, N, generator=g) * std for _ in range(3))
    AT = -torch.exp(torch.rand(E, N, generator=g) * math.log(16.0))
    AL = -torch.exp(torch.rand(E, N, generator=g) * math.log(16.0))
    D = torch.randn(E, generator=g)
    gy = torch.randn(B, H, W, E, generator=g)
    out = {k: v.to(device, dtype) for k, v in dict(x=x, dT=dT, dL=dL, AT=AT, AL=AL, D=D, gy=gy).items()}
    if strided:
        R = math.ceil(E / 16)
        buf = torch.zeros(B, H, W, 2 * R + 3 * N)
        buf[..., 2 * R:2 * R + N], buf[..., 2 * R + N:2 * R + 2 * N], buf[..., 2 * R + 2 * N:] = BT, BL, C
        buf = buf.to(device, dtype)
        out["BT"], out["BL"], out["C"] = buf[..., 2 * R:2 * R + N], buf[..., 2 * R + N:2 * R + 2 * N], buf[..., 2 * R + 2 * N:]
    else:
        out["BT"], out["BL"], out["C"] = (t.to(device, dtype) for t in (BT, BL, C))
    return out


def timeit(fn, iters, warm=2):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def reference_ext():
    sys.path.insert(0, ROOT)
    try:
        from oracle import ref_gpu          # optional comparison only; never used by the product path
        return ref_gpu if ref_gpu.available() else None
    except Exception:
        return None


def run_corner(B, H, W, E, dtype, bwd, iters):
    """Native bottom-right scan against flip + top-left scan + flip at the level of the module:
    the module flips x once on the way in and y once on the way out (and, in training, the
    gradient on the way in and d_x on the way out)."""
    from mamba2d_b200 import scan_bwd, scan_fwd
    d = make_inputs(B, H, W, E, dtype=dtype)
    a = [d[k] for k in ORDER]
    native = timeit(lambda: scan_fwd(*a, reverse=True), iters)
    flips = timeit(lambda: scan_fwd(d["x"].flip(1, 2), *a[1:]).flip(1, 2), iters)
    line = f"B={B} {H}x{W} E={E} {str(dtype).split('.')[-1]} corner BR: fwd native {native:.3f} ms, flip+scan+flip {flips:.3f} ms"
    if bwd:
        native = timeit(lambda: scan_bwd(*a, d["gy"], reverse=True), iters)
        flips = timeit(lambda: scan_bwd(*a, d["gy"].flip(1, 2))[0].flip(1, 2), iters)
        line += f" | bwd native {native:.3f} ms, flip+scan+flip {flips:.3f} ms"
    print(line, flush=True)


def run_entry(B, H, W, E, dtype, iters, kernels=False, once=False):
    """wavefront_scan_cuda forward + backward with module-shaped weights (A_log = log(1..N), dt_rank = E/16)."""
    from mamba2d_b200 import wavefront_cuda as wc
    N, R = 16, math.ceil(E / 16)
    g = torch.Generator(device="cpu").manual_seed(0)
    x = torch.randn(B, H, W, E, generator=g).to("cuda", dtype).requires_grad_(True)
    gy = torch.randn(B, H, W, E, generator=g).to("cuda", dtype)
    A_log = torch.log(torch.arange(1, N + 1, dtype=torch.float32).repeat(E, 1)).cuda()
    mk = lambda *s, scale: ((torch.rand(*s, generator=g) * 2 - 1) * scale).to("cuda", dtype).requires_grad_(True)
    w = [A_log.clone().requires_grad_(True), A_log.clone().requires_grad_(True), mk(2 * R + 3 * N, E, scale=E ** -0.5),
         mk(E, R, scale=R ** -0.5), mk(E, scale=1.0), mk(E, R, scale=R ** -0.5), mk(E, scale=1.0),
         torch.ones(E, device="cuda", dtype=dtype, requires_grad=True)]

    def torch_proj(x, AT_log, AL_log, wx, wT, bT, wL, bL):   # the reference's formulation, differentiated by autograd
        p = F.linear(x, wx)
        rT, rL, BT, BL, C = torch.split(p, [R, R, N, N, N], dim=-1)
        return (F.softplus(F.linear(rT, wT, bT)), F.softplus(F.linear(rL, wL, bL)),
                (-torch.exp(AT_log.float())).to(x.dtype), (-torch.exp(AL_log.float())).to(x.dtype), BT, BL, C)

    class autograd_full(torch.autograd.Function):   # the reference's structure: graph + autograd.grad in backward
        @staticmethod
        def forward(ctx, x, *w):
            with torch.no_grad():
                p = torch_proj(x, *w[:7])
            ctx.save_for_backward(x, *w)
            return wc.scan_fwd_op(x, *p, w[7])

        @staticmethod
        def backward(ctx, gy):
            x, *w = ctx.saved_tensors
            with torch.enable_grad():
                leaves = [t.detach().requires_grad_(True) for t in (x, *w[:7])]
                proj = torch_proj(*leaves)
            p = [t.detach() for t in proj]
            gs = wc.scan_bwd_op(x, *p, w[7], gy)
            g = torch.autograd.grad(list(proj), leaves, [gs[1], gs[2], gs[3], gs[4], gs[5], gs[6], gs[7]])
            return (gs[0] + g[0], *g[1:], gs[8])

    def step(fn):
        for t in [x] + w:
            t.grad = None
        fn().backward(gy)

    if once:     # one partial-recomputation step and nothing else: the command line for ncu captures
        step(lambda: wc.wavefront_scan_cuda(x, *w, "partial"))
        torch.cuda.synchronize()
        print("ok")
        return
    line = f"B={B} {H}x{W} E={E} {str(dtype).split('.')[-1]} entry fwd+bwd:"
    for name, fn in (("partial", lambda: wc.wavefront_scan_cuda(x, *w, "partial")),
                     ("full", lambda: wc.wavefront_scan_cuda(x, *w, "full")),
                     ("partial, projections in PyTorch", lambda: wc.wf_cuda_fn_pr.apply(x, *torch_proj(x, *w[:7]), w[7])),
                     ("full, projections in PyTorch", lambda: autograd_full.apply(x, *w))):
        line += f" {name} {timeit(lambda: step(fn), iters):.3f} ms,"
    # the same partial-recomputation step captured once in a CUDA graph and replayed
    fn = lambda: wc.wavefront_scan_cuda(x, *w, "partial")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            step(fn)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    for t in [x] + w:
        t.grad = None
    with torch.cuda.graph(graph):
        fn().backward(gy)
    line += f" partial as a CUDA graph {timeit(graph.replay, iters):.3f} ms"
    print(line, flush=True)
    if kernels:
        from torch.profiler import ProfilerActivity, profile
        fn = lambda: wc.wavefront_scan_cuda(x, *w, "partial")
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(5):
                step(fn)
            torch.cuda.synchronize()
        rows = sorted((e for e in prof.key_averages() if e.device_time_total > 0), key=lambda e: -e.device_time_total)
        total = sum(e.device_time_total for e in rows)
        print(f"  device time per step {total / 5 / 1000:.3f} ms; kernels (average per launch, launches per step, share):")
        for e in rows[:14]:
            print(f"  {e.device_time_total / e.count:9.1f} us x{e.count // 5:<2d} {100 * e.device_time_total / total:5.1f} %  {e.key[:110]}")


def run_case(B, H, W, E, dtype, bwd, iters, timed, with_ref):
    from mamba2d_b200 import scan_bwd, scan_fwd
    d = make_inputs(B, H, W, E, dtype=dtype)
    a = [d[k] for k in ORDER]
    if not timed:
        for _ in range(iters):
            scan_fwd(*a)
            if bwd:
                scan_bwd(*a, d["gy"])
        torch.cuda.synchronize()
        print("ok")
        return
    line = f"B={B} {H}x{W} E={E} {str(dtype).split('.')[-1]}: fwd {timeit(lambda: scan_fwd(*a), iters):.3f} ms"
    if bwd:
        line += f", bwd {timeit(lambda: scan_bwd(*a, d['gy']), iters):.3f} ms"
    ref = reference_ext() if with_ref else None
    if ref is not None:
        c = [t.contiguous() for t in a]
        line += f" | reference extension fwd {timeit(lambda: ref.forward(*c), iters):.3f} ms"
        if bwd:
            line += f", bwd {timeit(lambda: ref.backward(*c, d['gy']), iters):.3f} ms"
    print(line, flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="128,56,56,64", help="B,H,W,E")
    ap.add_argument("--sweep", default=None, help="comma-separated H=W values at B=1, E=64 (forward)")
    ap.add_argument("--dtype", choices=("f32", "bf16"), default="f32")
    ap.add_argument("--bwd", action="store_true")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--time", action="store_true")
    ap.add_argument("--reference", action="store_true")
    ap.add_argument("--corner", choices=("TL", "BR"), default="TL")
    ap.add_argument("--entry", action="store_true")
    ap.add_argument("--kernels", action="store_true")
    ap.add_argument("--once", action="store_true")
    args = ap.parse_args()
    dtype = torch.float32 if args.dtype == "f32" else torch.bfloat16
    if args.sweep:
        for hw in (int(v) for v in args.sweep.split(",")):
            run_case(1, hw, hw, 64, dtype, False, args.iters, True, args.reference and hw <= 1024)
        return
    B, H, W, E = (int(v) for v in args.shape.split(","))
    if args.entry:
        run_entry(B, H, W, E, dtype, max(args.iters, 10), args.kernels, args.once)
        return
    if args.corner == "BR":
        run_corner(B, H, W, E, dtype, args.bwd, max(args.iters, 10))
        return
    run_case(B, H, W, E, dtype, args.bwd, args.iters, args.time, args.reference)


if __name__ == "__main__":
    main()
