#!/usr/bin/env python
"""Benchmark of the wavefront 2-D selective scan (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--dtype f32|bf16] [--impl ours|reference]

Workload ("config 2" of the baseline description): the isolated scan at the four M2D-T stage
shapes, batch 128 per GPU, N = 16 states:  (D, H=W) = (64,56) (128,28) (320,14) (512,7).
One step = forward + backward of all four shapes on one batch of seeded synthetic inputs.
An element is one output scalar y[b,i,j,e]; elements per step = sum of B*H*W*D = 49 774 592.

Prints ONE JSON line on rank 0.  `value` is device-resident throughput (CUDA events around the
timed steps, max over ranks); `e2e` is the same work driven from pinned host buffers with the
host<->device copies inside the timed region; `roofline` is for the dominant kernel (the backward
kernel at the 56x56 shape), `roofline_step` for everything launched in a step; `cpu_baseline` is
the C/OpenMP restatement under oracle/ timed on this machine's host cores on a bounded sample.

`--impl reference` times that CPU restatement as the reference arm: the reference project has no
CPU implementation of this path (its launcher has no host branch), so the restatement of its
kernel body is what can run on host cores.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

STAGES = [(64, 56), (128, 28), (320, 14), (512, 7)]   # (D, H=W)
BATCH = 128
NSTATE = 16
ORDER = ("x", "dT", "dL", "AT", "AL", "BT", "BL", "C", "D")
METRIC = "2D-scan fwd+bwd elements/s"
UNIT = "elements/s"
BYTES = {"f32": 4, "bf16": 2}

# DRAM bytes (read + write) of ONE launch of the dominant kernel, from an ncu capture of this same
# workload; see profiles/ for the capture summaries.  None = not captured for that dtype.
NCU_TRAFFIC = {"f32": 6.097e9, "bf16": None}   # profiles/m2d_bwd_kernel_f32_D64_56x56.md


def fwd_bytes(D, HW, s, B=BATCH, N=NSTATE):
    return s * (4 + 3 * N / D) * B * HW * HW * D


def bwd_bytes(D, HW, s, B=BATCH, N=NSTATE):
    return s * (7 + 6 * N / D) * B * HW * HW * D


def elements(B=BATCH):
    return sum(B * hw * hw * d for d, hw in STAGES)


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU, sampled every 200 ms while running."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
            except Exception:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        busy = [v for v in sm if mx and v > 0.5 * mx] or sm
        return {"sm_mhz": busy[len(busy) // 2] if busy else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(sm)}


def make_stage_inputs(dtype, device, pinned_host=False):
    """Seeded synthetic inputs for every stage shape (seed 0, draws as oracle.inputs documents)."""
    import torch
    from oracle import inputs as oin           # input generator only (no oracle compute)
    tdt = torch.float32 if dtype == "f32" else torch.bfloat16
    out = []
    for D, HW in STAGES:
        inp = oin.make_inputs(BATCH, HW, HW, D, NSTATE, seed=0, strided_bc=True)
        host, shared = {}, {}
        for k, v in inp.items():
            base = v if v.is_contiguous() else v._base
            if base.data_ptr() not in shared:      # BT, BL, C are views of ONE projection buffer
                hb = base.to(tdt)
                shared[base.data_ptr()] = hb.pin_memory() if pinned_host else hb
            host[k] = (shared[base.data_ptr()], v.shape, v.stride(), v.storage_offset(), v.is_contiguous())
        out.append(host)
    return out


def to_device(host, device):
    d, seen = {}, {}
    for k, (hb, shape, stride, off, contig) in host.items():
        key = hb.data_ptr()
        if key not in seen:
            seen[key] = hb.to(device, non_blocking=True)
        d[k] = seen[key] if contig else seen[key].as_strided(shape, stride, off)
    return d


def run_ours(args):
    import torch
    import torch.distributed as dist
    from mamba2d_b200 import scan_bwd, scan_fwd

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path for the product)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    host = make_stage_inputs(args.dtype, dev, pinned_host=True)
    devin = [to_device(h, dev) for h in host]
    torch.cuda.synchronize()
    s = BYTES[args.dtype]

    def step(record=None):
        for si, d in enumerate(devin):
            a = [d[k] for k in ORDER]
            if record is not None:
                record[si][0].record()
            scan_fwd(*a)
            if record is not None:
                record[si][1].record()
            scan_bwd(*a, d["gy"])
            if record is not None:
                record[si][2].record()

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()

    sampler = ClockSampler(local) if rank == 0 else None
    ev = [[[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in STAGES] for _ in range(args.steps)]
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for k in range(args.steps):
        step(ev[k])
    t1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms_total = t0.elapsed_time(t1)
    if world > 1:
        t = torch.tensor([ms_total], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps

    # per-kernel durations (averages over the timed steps, this rank)
    per = []
    for si, (D, HW) in enumerate(STAGES):
        f = sum(ev[k][si][0].elapsed_time(ev[k][si][1]) for k in range(args.steps)) / args.steps
        b = sum(ev[k][si][1].elapsed_time(ev[k][si][2]) for k in range(args.steps)) / args.steps
        per.append({"D": D, "HW": HW, "fwd_ms": round(f, 4), "bwd_ms": round(b, 4),
                    "fwd_GBs": round(fwd_bytes(D, HW, s) / f / 1e6, 1), "bwd_GBs": round(bwd_bytes(D, HW, s) / b / 1e6, 1),
                    "fb_GBs": round((fwd_bytes(D, HW, s) + bwd_bytes(D, HW, s)) / (f + b) / 1e6, 1)})

    # ---- end to end from pinned host buffers through the package's host-tensor API: every step copies
    # its inputs host -> device, runs forward + backward, and copies y and the nine gradients back;
    # copy-in, kernels and copy-out of consecutive calls overlap on three streams
    from mamba2d_b200 import HostScanPipeline
    e2e_steps = max(2, min(args.steps, 3))
    pipe = HostScanPipeline(dev, depth=4)
    host_views = [{k: (hb if contig else hb.as_strided(shape, stride, off)) for k, (hb, shape, stride, off, contig) in h.items()}
                  for h in host]
    outs_host = [None] * len(host_views)

    def e2e_step():
        for si, h in enumerate(host_views):
            t = pipe.submit(*[h[k] for k in ORDER], grad_output=h["gy"], out=outs_host[si])
            outs_host[si] = t.outputs

    e2e_step()
    pipe.synchronize()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    h2d0, d2h0, l0 = pipe.h2d_bytes, pipe.d2h_bytes, pipe.launches
    c0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    pipe.synchronize()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - c0
    h2d = (pipe.h2d_bytes - h2d0) // e2e_steps
    d2h = (pipe.d2h_bytes - d2h0) // e2e_steps
    e2e_launches = pipe.launches - l0
    if world > 1:
        t = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    clocks = sampler.stop() if sampler else None

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    peak, peak_kind = measured_peak()
    el = elements()
    dom = per[0]
    dom_bytes = bwd_bytes(*STAGES[0], s)
    step_bytes = sum(fwd_bytes(D, HW, s) + bwd_bytes(D, HW, s) for D, HW in STAGES)
    step_kernel_ms = sum(p["fwd_ms"] + p["bwd_ms"] for p in per)
    out = {
        "metric": METRIC, "value": el * world / (ms_step * 1e-3), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": args.dtype, "data": "synthetic",
        "config": {"workload": "isolated scan fwd+bwd at the four M2D-T stage shapes "
                               "(D,H=W)=(64,56),(128,28),(320,14),(512,7), batch 128 per GPU, N=16, BT/BL/C as "
                               "strided views (pitch 2R+3N)",
                   "elements_per_step_per_gpu": el, "l2": "each step streams >3 GB (inputs + state record), "
                   "far larger than the 126 MB L2, so no flush is needed between iterations",
                   "parallelism": f"batch-sharded replicas x{world}, no data-path collective"},
        "e2e": {"value": el * world * e2e_steps / e2e_s, "unit": UNIT, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "steps": e2e_steps, "gpu_launches": e2e_launches,
                "note": "HostScanPipeline: pinned host inputs -> device, fwd+bwd, y and all nine gradients -> pinned host, "
                        "every step; copy-in / kernels / copy-out of consecutive calls overlap on three streams"},
        "gpu_launches": args.steps * len(STAGES) * (2 if args.dtype == "f32" else 3),   # per shape: forward kernel, backward kernel (+ cast kernel for bf16)
        "roofline": {"bound": "hbm", "kernel": "m2d_bwd_kernel @ D=64,H=W=56,B=128", "achieved": dom_bytes / dom["bwd_ms"] / 1e6,
                     "peak": peak, "unit": "GB/s", "frac": dom_bytes / dom["bwd_ms"] / 1e6 / peak,
                     "peak_kind": peak_kind, "algorithmic_bytes": dom_bytes, "ms": dom["bwd_ms"],
                     "traffic": NCU_TRAFFIC[args.dtype]},
        "roofline_step": {"bound": "hbm", "achieved": step_bytes / step_kernel_ms / 1e6, "peak": peak, "unit": "GB/s",
                          "frac": step_bytes / step_kernel_ms / 1e6 / peak, "algorithmic_bytes": step_bytes},
        "per_shape": per,
        "clocks": clocks,
    }
    if world == 1 and not args.no_cpu:
        out["cpu_baseline"] = cpu_baseline(args.dtype)
    if world == 1 and not args.no_ref_gpu:
        out["reference_gpu"] = reference_gpu(devin, args.dtype)
    if world == 1:
        out["m2dt_scan_layers"] = m2dt_scan_layers(dev)
    print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


def cpu_baseline(dtype, sample_batch=64, repeat=1, threads=None):
    """The C/OpenMP restatement (oracle/) timed on the host cores over a bounded sample: forward +
    backward of the four stage shapes at a reduced batch."""
    import torch
    from oracle import cpu as ocpu
    from oracle import inputs as oin
    # all host cores this process may use (torchrun presets OMP_NUM_THREADS=1 for its ranks)
    ocpu.set_threads(threads or len(os.sched_getaffinity(0)))
    cores = ocpu.num_threads()
    el = 0
    t = 0.0
    for D, HW in STAGES:
        inp = oin.make_inputs(sample_batch, HW, HW, D, NSTATE, seed=0)
        if dtype == "bf16":
            inp = {k: v.to(torch.bfloat16).float() for k, v in inp.items()}
        for _ in range(repeat):
            c0 = time.perf_counter()
            ocpu.forward(inp, "f32")
            ocpu.backward(inp, mode="f32")
            t += time.perf_counter() - c0
            el += sample_batch * HW * HW * D
    return {"value": el / t, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"fwd+bwd of the four stage shapes at batch {sample_batch} (of 128), fp32 arithmetic, "
                      f"{repeat} pass(es), {t:.1f} s wall on {cores} threads",
            "seconds": t}


def m2dt_scan_layers(dev, batch=128, iters=5):
    """The scan layers of one M2D-T forward as the backbone calls them: wavefront_scan_cuda(x, weights)
    in bf16 under inference mode, projections included, 3 blocks at (D=64, 56x56) + 3 blocks at
    (D=128, 28x28) -- the only stages of the shipped M2D-T config that use the scan (stages 3-4 are
    attention).  Images/s of this part alone; the rest of the backbone is outside this repository."""
    import torch
    from mamba2d_b200 import wavefront_scan_cuda
    from oracle import inputs as oin
    names = ("AT_log", "AL_log", "x_proj_w", "dt_projT_w", "dt_projT_b", "dt_projL_w", "dt_projL_b", "D")
    layers = []
    for D, HW, blocks in ((64, 56, 3), (128, 28, 3)):
        g = torch.Generator().manual_seed(D)
        x = torch.randn(batch, HW, HW, D, generator=g).to(dev, torch.bfloat16)
        for k in range(blocks):
            w = oin.make_module_params(D, NSTATE, seed=10 * D + k)
            layers.append((x, [w[n].to(dev) for n in names]))
    def run():
        with torch.inference_mode():
            for x, ws in layers:
                wavefront_scan_cuda(x, *ws)
    for _ in range(2):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters

    # the same six layers in training: forward + backward with gradients for x and every weight
    train = []
    for x, ws in layers:
        train.append((x.clone().requires_grad_(True), [t.clone().requires_grad_(True) for t in ws], torch.randn_like(x)))

    def run_train():
        for x, ws, gy in train:
            for t in [x] + ws:
                t.grad = None
            wavefront_scan_cuda(x, *ws).backward(gy)
    for _ in range(2):
        run_train()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(iters):
        run_train()
    e1.record()
    torch.cuda.synchronize()
    train_ms = e0.elapsed_time(e1) / iters
    return {"images_per_s": batch / (ms * 1e-3), "ms": ms, "train_ms": train_ms, "train_images_per_s": batch / (train_ms * 1e-3),
            "batch": batch, "dtype": "bf16",
            "what": "6 scan layers of M2D-T (3x D=64@56x56, 3x D=128@28x28) through wavefront_scan_cuda incl. projections; "
                    "ms = forward under inference mode, train_ms = forward + backward"}


def reference_gpu(devin, dtype, iters=2):
    """The reference project's own CUDA extension (built unmodified into oracle/_ref/, sm_100) with its
    PyTorch glue restated in oracle/ref_gpu.py, timed on this GPU on the same inputs: forward + backward of
    the four stage shapes.  Reported beside our numbers; it is the GPU implementation being replaced."""
    import torch
    try:
        from oracle import ref_gpu
        if not ref_gpu.available():
            return {"unavailable": "oracle/_ref/wf_ref_cuda.so not prebuilt"}
        per, total = [], 0.0
        for (D, HW), d in zip(STAGES, devin):
            a = [d[k].contiguous() for k in ORDER]
            gy = d["gy"]
            ref_gpu.forward(*a)
            ref_gpu.backward(*a, gy)
            torch.cuda.synchronize()
            e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            f = b = 0.0
            for _ in range(iters):
                e[0].record()
                ref_gpu.forward(*a)
                e[1].record()
                ref_gpu.backward(*a, gy)
                e[2].record()
                torch.cuda.synchronize()
                f += e[0].elapsed_time(e[1]) / iters
                b += e[1].elapsed_time(e[2]) / iters
            per.append({"D": D, "HW": HW, "fwd_ms": round(f, 3), "bwd_ms": round(b, 3)})
            total += f + b
            torch.cuda.empty_cache()
        return {"value": elements() / (total * 1e-3), "unit": UNIT, "ms_per_step": total, "per_shape": per,
                "what": "reference wf_cuda extension (one launch per anti-diagonal) + its PyTorch readout / gradient math, "
                        "same GPU, same inputs (B/C made contiguous), device-resident, CUDA events"}
    except Exception as exc:   # the baseline is informative only
        return {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}


def run_reference(args):
    """Reference arm: the reference's algorithm on host cores (see module docstring)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    sample_batch = 8
    times, el = [], 0
    for k in range(args.warmup + args.steps):
        r = cpu_baseline(args.dtype, sample_batch=sample_batch)
        if k >= args.warmup:
            times.append(r["seconds"])
            el = r["value"] * r["seconds"]
    ms = 1e3 * sum(times) / len(times)
    value = el / (ms * 1e-3)
    out = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
           "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
           "dtype": args.dtype, "data": "synthetic",
           "config": {"workload": "isolated scan fwd+bwd at the four M2D-T stage shapes, N=16; each step is a bounded "
                                  f"sample at batch {sample_batch} of 128 on the host cores"},
           "cpu_baseline": {"value": value, "unit": UNIT, "cores": r["cores"], "kind": "port", "sample": r["sample"]},
           "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
           "gpu_launches": 0}
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--dtype", choices=("f32", "bf16"), default="f32")
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--no-cpu", action="store_true", help="skip the timed CPU baseline leg")
    ap.add_argument("--no-ref-gpu", action="store_true", help="skip timing the reference's CUDA extension")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
