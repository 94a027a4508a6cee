#!/usr/bin/env python
"""Benchmark of the wavefront 2-D selective scan (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--dtype f32|bf16] [--impl ours|reference]
    python bench.py --shape B,H,W,E [--dtype f32|bf16] [--bwd] [--once] [--iters K] [--corner BR [--flips]] [--entry]

Workload ("config 2" of the baseline description): the isolated scan at the four M2D-T stage
shapes, batch 128 per GPU, N = 16 states:  (D, H=W) = (64,56) (128,28) (320,14) (512,7).
One step = forward + backward of all four shapes on one batch of seeded synthetic inputs.
An element is one output scalar y[b,i,j,e]; elements per step = sum of B*H*W*D = 49 774 592.

Prints ONE JSON line on rank 0.  `value` is device-resident throughput (CUDA events around the
timed steps, max over ranks); `e2e` is the same work driven from pinned host buffers with the
host<->device copies inside the timed region; `roofline` is for the dominant kernel (the backward
kernel at the 56x56 shape), `roofline_step` for everything launched in a step; `cpu_baseline` is
the C/OpenMP restatement under oracle/ timed on this machine's host cores on a bounded sample.

Extra keys of the line (single-GPU runs): `other_dtype` (the same workload in the other I/O type),
`reference_gpu` (the reference project's own CUDA extension behind its own Python module, same GPU,
same inputs), `resolution_sweep` (forward at B=1, D=64, H=W = 64 ... 2048, ours and the reference
extension), `m2dt` (images/s of the reference's unchanged M2D-T classifier on top of this op; at
N > 1 the sum over ranks).

`--shape` runs one shape only (forward, and backward with `--bwd`) and prints CUDA-event times, or
with `--once` launches each kernel once and prints nothing but "ok": the command line of the ncu
captures under profiles/.

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
NCU_TRAFFIC = {"f32": 6.064e9, "bf16": 3.696e9}
NCU_TRAFFIC_FROM = "538d212"  # the commit whose kernels were captured


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


def time_config2(dtype, dev, steps, warmup, world, sampler_index=None, e2e_steps=20):
    """Device-resident and end-to-end timing of the config-2 workload in one I/O type on this rank.
    Returns a dict with ms_per_step (max over ranks), per-shape kernel times, e2e figures, clocks."""
    import torch
    import torch.distributed as dist
    from mamba2d_b200 import HostScanPipeline, scan_bwd, scan_fwd

    host = make_stage_inputs(dtype, dev, pinned_host=True)
    devin = [to_device(h, dev) for h in host]
    torch.cuda.synchronize()
    s = BYTES[dtype]

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

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()

    sampler = ClockSampler(sampler_index) if sampler_index is not None else None
    ev = [[[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in STAGES] for _ in range(steps)]
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for k in range(steps):
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
    ms_step = ms_total / steps

    # per-kernel durations (averages over the timed steps, this rank)
    per = []
    for si, (D, HW) in enumerate(STAGES):
        f = sum(ev[k][si][0].elapsed_time(ev[k][si][1]) for k in range(steps)) / steps
        b = sum(ev[k][si][1].elapsed_time(ev[k][si][2]) for k in range(steps)) / steps
        per.append({"D": D, "HW": HW, "fwd_ms": round(f, 4), "bwd_ms": round(b, 4),
                    "fwd_GBs": round(fwd_bytes(D, HW, s) / f / 1e6, 1), "bwd_GBs": round(bwd_bytes(D, HW, s) / b / 1e6, 1),
                    "fb_GBs": round((fwd_bytes(D, HW, s) + bwd_bytes(D, HW, s)) / (f + b) / 1e6, 1)})

    # ---- end to end from pinned host buffers through the package's host-tensor API: every step copies
    # its inputs host -> device, runs forward + backward, and copies y and the nine gradients back;
    # copy-in, kernels and copy-out of consecutive calls overlap on three streams
    pipe = HostScanPipeline(dev, depth=8)
    host_views = [{k: (hb if contig else hb.as_strided(shape, stride, off)) for k, (hb, shape, stride, off, contig) in h.items()}
                  for h in host]
    outs_host = [None] * len(host_views)

    def e2e_step():
        for si, h in enumerate(host_views):
            t = pipe.submit(*[h[k] for k in ORDER], grad_output=h["gy"], out=outs_host[si])
            outs_host[si] = t.outputs

    for _ in range(3):
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
    del pipe, outs_host, host_views
    return {"ms_step": ms_step, "per": per, "devin": devin, "clocks": clocks,
            "e2e": {"seconds": e2e_s, "steps": e2e_steps, "h2d": h2d, "d2h": d2h, "launches": e2e_launches}}


def summarise(dtype, r, world, steps):
    """value / roofline / per-shape figures of one time_config2 result."""
    s = BYTES[dtype]
    peak, peak_kind = measured_peak()
    el = elements()
    per = r["per"]
    dom = per[0]
    dom_bytes = bwd_bytes(*STAGES[0], s)
    step_bytes = sum(fwd_bytes(D, HW, s) + bwd_bytes(D, HW, s) for D, HW in STAGES)
    step_kernel_ms = sum(p["fwd_ms"] + p["bwd_ms"] for p in per)
    e = r["e2e"]
    return {
        "value": el * world / (r["ms_step"] * 1e-3), "ms_per_step": r["ms_step"],
        "e2e": {"value": el * world * e["steps"] / e["seconds"], "unit": UNIT, "h2d_bytes_per_step": e["h2d"],
                "d2h_bytes_per_step": e["d2h"], "steps": e["steps"], "gpu_launches": e["launches"],
                "note": "HostScanPipeline: pinned host inputs -> device, fwd+bwd, y and all nine gradients -> pinned host, "
                        "every step; copy-in / kernels / copy-out of consecutive calls overlap on three streams"},
        # per shape: forward kernel, backward kernel (+ cast kernel for bf16)
        "gpu_launches": steps * len(STAGES) * (2 if dtype == "f32" else 3),
        "roofline": {"bound": "hbm", "kernel": "m2d_bwd_kernel @ D=64,H=W=56,B=128", "achieved": dom_bytes / dom["bwd_ms"] / 1e6,
                     "peak": peak, "unit": "GB/s", "frac": dom_bytes / dom["bwd_ms"] / 1e6 / peak,
                     "peak_kind": peak_kind, "algorithmic_bytes": dom_bytes, "ms": dom["bwd_ms"],
                     "traffic": NCU_TRAFFIC[dtype], "traffic_from_commit": NCU_TRAFFIC_FROM if NCU_TRAFFIC[dtype] else None},
        "roofline_step": {"bound": "hbm", "achieved": step_bytes / step_kernel_ms / 1e6, "peak": peak, "unit": "GB/s",
                          "frac": step_bytes / step_kernel_ms / 1e6 / peak, "algorithmic_bytes": step_bytes},
        "per_shape": per,
    }


def run_ours(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path for the product)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    r = time_config2(args.dtype, dev, args.steps, args.warmup, world, sampler_index=local if rank == 0 else None)
    main = summarise(args.dtype, r, world, args.steps)
    m2dt = None if args.no_model else m2dt_images_per_s(dev, world, variants=("ours",) if world > 1 else None)
    m2ds = None if (args.no_model or args.no_train) else m2ds_train_step(dev, world, local)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    el = elements()
    out = {
        "metric": METRIC, "value": main["value"], "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": main["ms_per_step"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": args.dtype, "data": "synthetic",
        "config": {"workload": "isolated scan fwd+bwd at the four M2D-T stage shapes "
                               "(D,H=W)=(64,56),(128,28),(320,14),(512,7), batch 128 per GPU, N=16, BT/BL/C as "
                               "strided views (pitch 2R+3N)",
                   "elements_per_step_per_gpu": el, "l2": "each step streams >3 GB (inputs + state record), "
                   "far larger than the 126 MB L2, so no flush is needed between iterations",
                   "parallelism": f"batch-sharded replicas x{world}, no data-path collective"},
        "e2e": main["e2e"], "gpu_launches": main["gpu_launches"], "roofline": main["roofline"],
        "roofline_step": main["roofline_step"], "per_shape": main["per_shape"], "clocks": r["clocks"],
    }
    if m2dt is not None:
        out["m2dt"] = m2dt
    if m2ds is not None:
        out["m2ds_train"] = m2ds
    if world == 1:
        if not args.no_cpu:
            out["cpu_baseline"] = cpu_baseline(args.dtype)
        if not args.no_ref_gpu:
            out["reference_gpu"] = reference_gpu(r["devin"], args.dtype)
            out["resolution_sweep"] = resolution_sweep(dev)
        del r
        torch.cuda.empty_cache()
        other = "bf16" if args.dtype == "f32" else "f32"
        r2 = time_config2(other, dev, args.steps, args.warmup, world)
        o = summarise(other, r2, world, args.steps)
        out["other_dtype"] = {"dtype": other, "value": o["value"], "unit": UNIT, "ms_per_step": o["ms_per_step"],
                              "e2e": o["e2e"], "roofline": o["roofline"], "roofline_step": o["roofline_step"],
                              "per_shape": o["per_shape"]}
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


def _events():
    import torch
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def _time_ms(fn, iters, warm=2):
    import torch
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = _events()
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


_REF_MODULE = []


def load_reference_module():
    """The reference project's own ``models/kernels/wavefront_cuda.py`` (unmodified copy under
    baseline/_ref), imported for real with its JIT build answered by the prebuilt extension
    (oracle/_ref/wf_ref_cuda.so, the same two source files compiled ahead of time for sm_100).  Its
    projection and gradient helpers keep their ``@torch.compile`` decorators; if the code generator
    cannot run on this machine they fall back to eager execution."""
    import importlib
    import torch
    from torch.utils import cpp_extension
    from mamba2d_b200 import inject, refmodel
    from oracle import build_ref_cuda
    root = refmodel.reference_root()
    if root is None or build_ref_cuda.find() is None:
        raise RuntimeError("reference model copy (baseline/_ref) or prebuilt reference extension (oracle/_ref) missing")
    refmodel.purge_models_modules()
    inject.install_droppath_shim()
    if root not in sys.path:
        sys.path.insert(0, root)
    if _REF_MODULE:
        # imported before (its operators can be registered only once): put it back under its name
        importlib.import_module("models")
        importlib.import_module("models.kernels")
        sys.modules["models.kernels.wavefront_cuda"] = _REF_MODULE[0]
        return _REF_MODULE[0]
    os.environ.setdefault("CXX", "/usr/bin/g++")
    os.environ.setdefault("CC", "/usr/bin/gcc")
    torch._dynamo.config.suppress_errors = True
    prebuilt = build_ref_cuda.load()
    orig = cpp_extension.load
    cpp_extension.load = lambda *a, **k: prebuilt
    try:
        mod = importlib.import_module("models.kernels.wavefront_cuda")
    finally:
        cpp_extension.load = orig
    _REF_MODULE.append(mod)
    return mod


def m2dt_images_per_s(dev, world, batch=128, iters=5, variants=None):
    """Config 1: forward images/s of the reference's unchanged M2D-T classifier (blocks [3,3,9,3],
    widths [64,128,320,512], inter_flip, random weights), batch 128 per GPU, synthetic N(0,1) images,
    channels last, inference mode under bf16 autocast (the shipped precision is bf16-mixed).
    Variants: "ours" = the reference model calling this package's op, nothing else changed;
    "ours_native_corner" = the same with bottom-right blocks scanned in place instead of flipped;
    "ours_native_corner_fused_act" = that plus the GELU after the scan folded into the scan's store;
    "reference" = the reference model calling its own kernels (its own Python module, prebuilt
    extension).  All ranks run the same replica; the reported figure sums the ranks."""
    import torch
    import torch.distributed as dist
    from mamba2d_b200 import refmodel
    try:
        root = refmodel.reference_root()
        if root is None:
            return {"unavailable": "no copy of the reference's models/ package (baseline/_ref) on this machine"}
        g = torch.Generator().manual_seed(0)
        x = torch.randn(batch, 3, 224, 224, generator=g).to(dev).contiguous(memory_format=torch.channels_last)
        out, state = {"batch_per_gpu": batch, "dtype": "bf16 autocast", "n_gpus": world}, None
        logits = {}
        for v in variants or ("ours", "ours_native_corner", "ours_native_corner_fused_act", "reference"):
            try:
                if v == "reference":
                    import importlib
                    load_reference_module()                      # models.kernels.wavefront_cuda = the reference's
                    mods = (importlib.import_module("models.mamba2d"), importlib.import_module("models.utils"))
                else:
                    mods = refmodel.import_reference_models(root, native_corner=(v != "ours"), fuse_act2=v.endswith("fused_act"))
                torch.manual_seed(0)
                model = refmodel.build_classifier("M2D-T", mods).to(dev).eval()
                if state is None:
                    state = {k: t.clone() for k, t in model.state_dict().items()}
                else:
                    model.load_state_dict(state)

                def run():
                    with torch.inference_mode(), torch.autocast("cuda", dtype=torch.bfloat16):
                        return model(x)
                logits[v] = run().float()
                ms = _time_ms(run, iters)
                if world > 1:
                    t = torch.tensor([ms], device=dev)
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                    ms = float(t.item())
                out[v] = {"images_per_s": batch * world / (ms * 1e-3), "ms": ms}
                del model
                torch.cuda.empty_cache()
            except Exception as exc:
                out[v] = {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}
        if "ours" in logits and "reference" in logits:
            ref = logits["reference"]
            out["max_logit_difference_vs_reference"] = float((logits["ours"] - ref).abs().max() / ref.abs().max())
        refmodel.purge_models_modules()
        return out
    except Exception as exc:
        return {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}


def m2ds_train_step(dev, world, local, global_batch=1024, micro_batch=128, steps=2, warmup=2):
    """Config 4: one training step of the reference's unchanged M2D-S classifier (blocks [3,12,14,3],
    widths [96,192,384,576]) on top of this op: forward + backward + AdamW with the reference's
    parameter groups, cross-entropy on uniform random labels, bf16 autocast, global batch 1024 split
    evenly over the ranks (each rank accumulates over micro-batches of 128), weight gradients
    all-reduced by DistributedDataParallel over NCCL when there is more than one rank.  Strong
    scaling: the global batch is fixed.  Time per step is the max over ranks (CUDA events)."""
    import torch
    import torch.distributed as dist
    from mamba2d_b200 import refmodel
    try:
        if refmodel.reference_root() is None:
            return {"unavailable": "no copy of the reference's models/ package (baseline/_ref) on this machine"}
        mods = refmodel.import_reference_models(native_corner=False)
        torch.manual_seed(0)
        model = refmodel.build_classifier("M2D-S", mods).to(dev).train()
        net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local]) if world > 1 else model
        opt = refmodel.make_optimizer(net)
        n = global_batch // world
        g = torch.Generator().manual_seed(1 + int(os.environ.get("RANK", "0")))
        x = torch.randn(n, 3, 224, 224, generator=g).to(dev).contiguous(memory_format=torch.channels_last)
        labels = torch.randint(0, 1000, (n,), generator=g).to(dev)
        for _ in range(warmup):
            loss = refmodel.train_step(net, opt, x, labels, micro_batch)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = _events()
        e0.record()
        for _ in range(steps):
            loss = refmodel.train_step(net, opt, x, labels, micro_batch)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        out = {"ms_per_step": ms, "images_per_s": global_batch / (ms * 1e-3), "global_batch": global_batch,
               "micro_batch": micro_batch, "n_gpus": world, "scaling": "strong", "dtype": "bf16 autocast",
               "loss": float(loss), "peak_memory_GB": round(torch.cuda.max_memory_allocated(dev) / 2 ** 30, 1),
               "collective": "DistributedDataParallel bucketed NCCL all-reduce of the weight gradients" if world > 1 else "none"}
        del net, model, opt, x
        refmodel.purge_models_modules()
        torch.cuda.empty_cache()
        return out
    except Exception as exc:
        return {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}


def reference_gpu(devin, dtype, iters=10):
    """The reference project's own CUDA extension behind its own Python module
    (``wf_cuda_fn_pr`` of models/kernels/wavefront_cuda.py, unmodified), on this GPU and the same
    inputs: forward + backward of the four stage shapes.  Timed twice: with the module's
    ``@torch.compile`` helpers compiled (as shipped) and with them forced to eager execution."""
    import torch
    try:
        ref = load_reference_module()
        out = {}
        for mode in ("compiled", "eager"):
            per, total = [], 0.0
            with torch.compiler.set_stance("default" if mode == "compiled" else "force_eager"):
                for (D, HW), d in zip(STAGES, devin):
                    a = [d[k].contiguous().detach().requires_grad_(True) for k in ORDER]
                    gy = d["gy"]

                    def fwd():
                        return ref.wf_cuda_fn_pr.apply(*a)

                    def fwdbwd():
                        for t in a:
                            t.grad = None
                        fwd().backward(gy)
                    f = _time_ms(lambda: fwd(), iters)
                    fb = _time_ms(fwdbwd, iters)
                    per.append({"D": D, "HW": HW, "fwd_ms": round(f, 3), "bwd_ms": round(fb - f, 3)})
                    total += fb
                    del a
                    torch.cuda.empty_cache()
            out[mode] = {"value": elements() / (total * 1e-3), "unit": UNIT, "ms_per_step": total, "per_shape": per}
        out["iters"] = iters
        out["what"] = ("reference wf_cuda extension (one launch per anti-diagonal) behind the reference's own autograd Function "
                       "wf_cuda_fn_pr with its readout / gradient math, same GPU, same inputs (B/C made contiguous), "
                       "device-resident, CUDA events; bwd_ms = (forward + backward) - forward")
        return out
    except Exception as exc:   # the baseline is informative only
        return {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}


def resolution_sweep(dev, sizes=(64, 128, 256, 512, 1024, 2048)):
    """Config 3: forward at B=1, D=64, N=16, fp32, H=W from 64 to 2048; ours and, up to 1024 (its state
    tensor would take 17 GB at 2048), the reference's own extension with its readout."""
    import torch
    from mamba2d_b200 import scan_fwd
    from oracle import inputs as oin
    rows = []
    try:
        ref = load_reference_module()
    except Exception:
        ref = None
    for hw in sizes:
        inp = oin.make_inputs(1, hw, hw, 64, NSTATE, seed=hw)
        a = [inp[k].to(dev) for k in ORDER]
        row = {"HW": hw, "ours_ms": round(_time_ms(lambda: scan_fwd(*a), 10), 4)}
        if ref is not None and hw <= 1024:
            try:
                with torch.inference_mode():
                    row["reference_ms"] = round(_time_ms(lambda: ref.wf_cuda_fn_pr.apply(*a), 3), 3)
            except Exception as exc:
                row["reference_ms"] = f"{type(exc).__name__}"
        rows.append(row)
        del a
        torch.cuda.empty_cache()
    return rows


def run_shape(args):
    """One shape, for ncu captures and one-off timings (see the module docstring)."""
    import torch
    from mamba2d_b200 import scan_bwd, scan_fwd, wavefront_scan_cuda
    from oracle import inputs as oin
    B, H, W, E = (int(v) for v in args.shape.split(","))
    tdt = torch.float32 if args.dtype == "f32" else torch.bfloat16
    s = BYTES[args.dtype]
    peak, kind = measured_peak()
    if args.entry:
        # the op as the model calls it: projections + scan, forward + backward (partial recomputation)
        names = ("AT_log", "AL_log", "x_proj_w", "dt_projT_w", "dt_projT_b", "dt_projL_w", "dt_projL_b", "D")
        w = oin.make_module_params(E, NSTATE, seed=0)
        g = torch.Generator().manual_seed(0)
        x = torch.randn(B, H, W, E, generator=g).to("cuda", tdt).requires_grad_(True)
        gy = torch.randn(B, H, W, E, generator=g).to("cuda", tdt)
        ws = [(w[k].cuda() if k.endswith("_log") else w[k].to("cuda", tdt)).requires_grad_(True) for k in names]

        def step():
            for t in [x] + ws:
                t.grad = None
            wavefront_scan_cuda(x, *ws, "partial", scan_start=args.corner).backward(gy)
        if args.once:
            step()
            torch.cuda.synchronize()
            print("ok")
            return
        print(json.dumps({"shape": [B, H, W, E], "dtype": args.dtype, "corner": args.corner,
                          "entry_fwd_bwd_ms": round(_time_ms(step, args.iters, warm=3), 4)}), flush=True)
        return
    inp = oin.make_inputs(B, H, W, E, NSTATE, seed=0, strided_bc=True)
    dev = {}
    base = inp["BT"]._base.to("cuda", tdt)
    for k, v in inp.items():
        dev[k] = base.as_strided(v.shape, v.stride(), v.storage_offset()) if k in ("BT", "BL", "C") else v.to("cuda", tdt)
    a = [dev[k] for k in ORDER]
    rev = args.corner == "BR"
    if args.once:
        scan_fwd(*a, reverse=rev)
        if args.bwd:
            scan_bwd(*a, dev["gy"], reverse=rev)
        torch.cuda.synchronize()
        print("ok")
        return
    f = _time_ms(lambda: scan_fwd(*a, reverse=rev), args.iters, warm=3)
    out = {"shape": [B, H, W, E], "dtype": args.dtype, "corner": args.corner, "fwd_ms": round(f, 4),
           "fwd_frac_of_" + kind: round(s * (4 + 3 * NSTATE / E) * B * H * W * E / f / 1e6 / peak, 4)}
    if args.bwd:
        b = _time_ms(lambda: scan_bwd(*a, dev["gy"], reverse=rev), args.iters, warm=3)
        out["bwd_ms"] = round(b, 4)
        out["bwd_frac_of_" + kind] = round(s * (7 + 6 * NSTATE / E) * B * H * W * E / b / 1e6 / peak, 4)
    if rev and args.flips:
        # the reference's way to get this direction: flip copies around the top-left scan
        out["flip_scan_flip_fwd_ms"] = round(_time_ms(lambda: scan_fwd(dev["x"].flip(1, 2), *a[1:]).flip(1, 2), args.iters, warm=3), 4)
    print(json.dumps(out), flush=True)


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
    ap.add_argument("--no-model", action="store_true", help="skip the model-level legs (M2D-T images/s, M2D-S training step)")
    ap.add_argument("--no-train", action="store_true", help="skip the M2D-S training-step leg")
    ap.add_argument("--shape", default=None, help="B,H,W,E: run this one shape instead of the benchmark")
    ap.add_argument("--bwd", action="store_true", help="with --shape: also the backward")
    ap.add_argument("--once", action="store_true", help="with --shape: launch each kernel once, no timing")
    ap.add_argument("--iters", type=int, default=10, help="with --shape: timed iterations")
    ap.add_argument("--corner", choices=("TL", "BR"), default="TL", help="with --shape: scan start corner")
    ap.add_argument("--flips", action="store_true", help="with --shape --corner BR: also time flip + top-left scan + flip")
    ap.add_argument("--entry", action="store_true", help="with --shape: the module-level entry (projections + scan), forward + backward")
    args = ap.parse_args()
    if args.shape:
        run_shape(args)
        return
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
