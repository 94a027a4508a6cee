"""The reference's unchanged model file resolves its scan import to this package (needs the
reference checkout; skipped where it is absent)."""
import os
import sys

import pytest

REF = os.environ.get("M2D_REFERENCE_ROOT", "/root/reference")


@pytest.mark.skipif(not os.path.exists(os.path.join(REF, "models", "mamba2d.py")), reason="reference checkout not present")
def test_reference_block_imports_replacement():
    import mamba2d_b200.inject as inject
    from mamba2d_b200 import wavefront_cuda
    inject.install_droppath_shim()
    inject.install(REF)
    saved = {k: v for k, v in sys.modules.items() if k == "models" or k.startswith("models.")}
    try:
        import importlib
        m = importlib.import_module("models.mamba2d")
        assert m.wavefront_scan_cuda is wavefront_cuda.wavefront_scan_cuda
        blk = m.M2DBlock(d_model=32)
        assert blk.AT_log.shape == (32, 16) and blk.x_proj.weight.shape == (2 * 2 + 48, 32)
    finally:
        for k in [k for k in sys.modules if k == "models" or k.startswith("models.")]:
            if k not in saved:
                del sys.modules[k]
