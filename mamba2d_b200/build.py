"""Ahead-of-time build of the C-ABI library ``libm2d_scan.so`` for sm_100a.

    python -m mamba2d_b200.build [--force] [--verbose]

The shared object is written next to this file (in-tree, git-ignored).  Importing the package
never compiles; it only loads the prebuilt library.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
OUT = os.path.join(HERE, "libm2d_scan.so")
OBJ = os.path.join(HERE, "_obj")          # per-source objects (git-ignored, not shipped)
SOURCES = ["m2d_abi.cu", "m2d_scan_fwd.cu", "m2d_scan_bwd.cu", "m2d_scan_fwd_noalloc.cu", "m2d_proj.cu"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc():
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _deps():
    out = [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE) if f.endswith(".h")]
    for f in os.listdir(CSRC):
        if f.endswith((".cu", ".cuh")):
            out.append(os.path.join(CSRC, f))
    return out


def _compile(nvcc, src, obj):
    cmd = [nvcc, "-ccbin", "/usr/bin/g++"] if os.path.exists("/usr/bin/g++") else [nvcc]
    # (an alternative host compiler on PATH in some images cannot be used by nvcc; the system one is pinned)
    cmd += [*ARCH, "-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
            "-I", INCLUDE, "-I", CSRC, "-c", src, "-o", obj]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    return " ".join(cmd) + "\n" + res.stdout, res.returncode


def build(force=False, verbose=False):
    """Compile every source to an object (in parallel, only the stale ones) and link the library."""
    from concurrent.futures import ThreadPoolExecutor
    srcs = [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    headers = [d for d in _deps() if not d.endswith(".cu")]
    newest_header = max(os.path.getmtime(h) for h in headers)
    os.makedirs(OBJ, exist_ok=True)
    nvcc = _nvcc()
    jobs = []
    for src in srcs:
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        stale = force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), newest_header)
        jobs.append((src, obj, stale))
    if not any(j[2] for j in jobs) and os.path.exists(OUT) and all(os.path.getmtime(OUT) >= os.path.getmtime(j[1]) for j in jobs):
        return OUT
    logs, failed = [], False
    with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
        for text, rc in pool.map(lambda j: _compile(nvcc, j[0], j[1]) if j[2] else ("", 0), jobs):
            logs.append(text)
            failed = failed or rc != 0
    if not failed:
        cmd = [nvcc, "-ccbin", "/usr/bin/g++"] if os.path.exists("/usr/bin/g++") else [nvcc]
        cmd += [*ARCH, "-shared", *[j[1] for j in jobs], "-o", OUT, "-lcudart"]
        res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        logs.append(" ".join(cmd) + "\n" + res.stdout)
        failed = res.returncode != 0
    log = os.path.join(HERE, "build.log")
    with open(log, "w") as f:
        f.write("\n".join(logs))
    if verbose or failed:
        print("\n".join(logs))
    if failed:
        raise RuntimeError(f"nvcc failed; see {log}")
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv or "-v" in sys.argv))
