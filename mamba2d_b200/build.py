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
SOURCES = ["m2d_abi.cu", "m2d_scan_fwd.cu", "m2d_scan_bwd.cu", "m2d_scan_fwd_noalloc.cu"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc():
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _deps():
    out = [os.path.join(INCLUDE, "m2d_scan.h")]
    for f in os.listdir(CSRC):
        if f.endswith((".cu", ".cuh")) and f != "mufu_probe.cu":
            out.append(os.path.join(CSRC, f))
    return out


def build(force=False, verbose=False):
    srcs = [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    if not force and os.path.exists(OUT) and all(os.path.getmtime(OUT) >= os.path.getmtime(d) for d in _deps()):
        return OUT
    cmd = [_nvcc(), *ARCH, "-O3", "-lineinfo", "-std=c++17", "-shared", "-Xcompiler", "-fPIC",
           "-Xptxas", "-v", "-I", INCLUDE, "-I", CSRC, *srcs, "-o", OUT, "-lcudart"]
    env = dict(os.environ)
    # an alternative host compiler on PATH in some images cannot be used by nvcc; pin the system one
    if os.path.exists("/usr/bin/g++"):
        cmd[1:1] = ["-ccbin", "/usr/bin/g++"]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    log = os.path.join(HERE, "build.log")
    with open(log, "w") as f:
        f.write(" ".join(cmd) + "\n" + res.stdout)
    if verbose or res.returncode != 0:
        print(res.stdout)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed ({res.returncode}); see {log}")
    return OUT


def build_probe():
    """The stand-alone instruction-rate probe (csrc/mufu_probe.cu) -> mamba2d_b200/mufu_probe."""
    out = os.path.join(HERE, "mufu_probe")
    cmd = [_nvcc(), "-ccbin", "/usr/bin/g++", *ARCH, "-O3", os.path.join(CSRC, "mufu_probe.cu"), "-o", out]
    subprocess.run(cmd, check=True)
    return out


if __name__ == "__main__":
    if "--probe" in sys.argv:
        print(build_probe())
    else:
        print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv or "-v" in sys.argv))
