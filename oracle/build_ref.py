"""Build ``oracle/_ref/libwf_ref_cpu.so``: the reference project's own kernel source, run on the CPU.

TEST INFRASTRUCTURE ONLY.  The reference's recurrence exists only as CUDA kernels.  This recipe
takes the kernel part of ``models/kernels/wf_cuda/wf_cuda.cu`` (everything before the first host
launcher) straight from the reference checkout, appends ``ref_cpu_driver.inc`` and feeds the
result to g++ on standard input, with ``oracle/ref_shim`` first on the include path so that
``<torch/extension.h>`` resolves to the thread-index shim.  No reference source is written into
this repository; the only output is the shared object under ``oracle/_ref/`` (git-ignored).

The reference checkout is only present on the development machine; where it is absent this
script does nothing and the prebuilt library (if any) is used.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_ROOT = os.environ.get("M2D_REFERENCE_ROOT", "/root/reference")
REF_CU = os.path.join(REF_ROOT, "models", "kernels", "wf_cuda", "wf_cuda.cu")
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "libwf_ref_cpu.so")
MARK = "void wf_fwd_launcher("


def available():
    return os.path.exists(OUT)


def build(force=False, verbose=False):
    if not os.path.exists(REF_CU):
        return OUT if os.path.exists(OUT) else None
    if os.path.exists(OUT) and not force:
        return OUT
    text = open(REF_CU).read()
    cut = text.find(MARK)
    if cut < 0:
        raise RuntimeError("launcher marker not found in the reference kernel file")
    driver = open(os.path.join(HERE, "ref_cpu_driver.inc")).read()
    import torch
    tinc = os.path.join(os.path.dirname(torch.__file__), "include")
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = ["/usr/bin/g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-x", "c++", "-",
           "-I", os.path.join(HERE, "ref_shim"), "-I", tinc, "-o", OUT]
    if verbose:
        print(" ".join(cmd))
    subprocess.run(cmd, input=(text[:cut] + "\n" + driver).encode(), check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
