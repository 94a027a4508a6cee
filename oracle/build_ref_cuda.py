"""Build ``oracle/_ref/wf_ref_cuda*.so``: the reference project's own CUDA extension, unmodified.

TEST / BENCHMARK INFRASTRUCTURE ONLY.  Compiles the two reference source files where they lie in
the reference checkout (models/kernels/wf_cuda/wf_cuda.cu and wf_cuda_bind.cpp) into a PyTorch
extension for sm_100 with the flags the reference passes to its JIT build
(models/kernels/wavefront_cuda.py:10-19: -O2 / -Xptxas -O3).  nvcc cross-compiles without a GPU.
Nothing is copied into this repository; the shared object (git-ignored) is the GPU baseline the
bench compares against and a second parity target on the GPU box.

Where the reference checkout is absent this script does nothing.
"""
import glob
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_ROOT = os.environ.get("M2D_REFERENCE_ROOT", "/root/reference")
SRC_DIR = os.path.join(REF_ROOT, "models", "kernels", "wf_cuda")
OUT_DIR = os.path.join(HERE, "_ref")
NAME = "wf_ref_cuda"


def find():
    hits = glob.glob(os.path.join(OUT_DIR, NAME + "*.so"))
    return hits[0] if hits else None


def build(force=False, verbose=False):
    srcs = [os.path.join(SRC_DIR, "wf_cuda_bind.cpp"), os.path.join(SRC_DIR, "wf_cuda.cu")]
    if not all(os.path.exists(s) for s in srcs):
        return find()
    if find() and not force:
        return find()
    os.makedirs(OUT_DIR, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    os.environ["CXX"] = "/usr/bin/g++"
    os.environ["CC"] = "/usr/bin/gcc"
    from torch.utils import cpp_extension
    build_dir = os.path.join("/tmp", "wf_ref_cuda_build")
    os.makedirs(build_dir, exist_ok=True)
    cpp_extension.load(name=NAME, sources=srcs, extra_cflags=["-O2", "-fvisibility=hidden"],
                       extra_cuda_cflags=["-Xptxas", "-O3", "-ccbin", "/usr/bin/g++"], build_directory=build_dir,
                       verbose=verbose, is_python_module=False)
    import shutil
    for f in glob.glob(os.path.join(build_dir, NAME + "*.so")):
        shutil.copy(f, OUT_DIR)
    return find()


def load():
    """Import the prebuilt extension as a Python module (needs a CUDA device to be useful)."""
    path = find()
    if not path:
        return None
    import importlib.util
    import torch  # noqa: F401  (registers the libraries the extension links against)
    spec = importlib.util.spec_from_file_location(NAME, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
