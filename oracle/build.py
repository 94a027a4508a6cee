"""Build the C oracle (``libm2d_oracle.so``) next to its source.  Test infrastructure only.

Uses the system gcc explicitly: an alternative compiler on PATH in some images lacks the OpenMP
spec file and cannot link ``-fopenmp``.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "m2d_oracle.c")
OUT = os.path.join(HERE, "libm2d_oracle.so")


def _gcc():
    for cand in ("/usr/bin/gcc", shutil.which("gcc")):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("no gcc found for the oracle build")


def build(force=False, verbose=False):
    deps = [SRC, os.path.join(HERE, "m2d_oracle_impl.h")]
    if (not force and os.path.exists(OUT)
            and all(os.path.getmtime(OUT) >= os.path.getmtime(d) for d in deps)):
        return OUT
    cmd = [_gcc(), "-O3", "-march=x86-64-v3", "-fopenmp", "-ffp-contract=off", "-shared", "-fPIC",
           SRC, "-o", OUT, "-lm"]
    if verbose:
        print(" ".join(cmd))
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
