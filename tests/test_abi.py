"""The C-ABI library loads without a GPU and exports every symbol the headers under include/ declare;
argument validation and launch planning run on the host."""
import ctypes
import os
import re

import pytest

from mamba2d_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L():
    from mamba2d_b200 import build
    build.build()
    return _lib.lib()


def declared_symbols():
    inc = os.path.join(ROOT, "include")
    text = "".join(open(os.path.join(inc, f)).read() for f in sorted(os.listdir(inc)) if f.endswith(".h"))
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(m2d_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(L):
    syms = declared_symbols()
    assert set(_lib.EXPORTS) <= set(syms)
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for s in syms:
        assert getattr(raw, s) is not None, s


def test_version_and_strerror(L):
    assert L.m2d_abi_version() == _lib.ABI_VERSION
    assert _lib.strerror(0) == "ok"
    for code in range(-10, 0):
        assert _lib.strerror(code) not in ("ok", "unknown status")
    assert _lib.strerror(-99) == "unknown status"


def _desc(**kw):
    d = _lib.ScanDesc()
    d.struct_bytes = ctypes.sizeof(_lib.ScanDesc)
    d.dtype = _lib.M2D_F32
    d.B, d.H, d.W, d.E, d.N = 2, 8, 8, 64, 16
    d.BT_pitch = d.BL_pitch = d.C_pitch = 16
    for k, v in kw.items():
        setattr(d, k, v)
    return d


def test_descriptor_validation_without_a_device(L):
    d = _desc()
    assert L.m2d_scan_fwd(ctypes.byref(d), None) == -1          # NULL pointers
    assert L.m2d_scan_fwd(ctypes.byref(_desc(H=1)), None) == -3  # H < 2, as the reference's ValueError
    assert L.m2d_scan_fwd(ctypes.byref(_desc(W=1)), None) == -3
    assert L.m2d_scan_bwd(ctypes.byref(_desc(N=32)), None) == -4
    assert L.m2d_scan_fwd(ctypes.byref(_desc(dtype=7)), None) == -2
    assert L.m2d_scan_fwd(ctypes.byref(_desc(C_pitch=8)), None) == -5
    assert L.m2d_scan_fwd(ctypes.byref(_desc(struct_bytes=8)), None) == -8
    assert L.m2d_scan_fwd(ctypes.byref(_desc(flags=8)), None) == -10   # unknown flag bit
    assert L.m2d_scan_bwd(ctypes.byref(_desc(flags=_lib.M2D_SCAN_A_LOG)), None) == -1     # known to both entries
    assert L.m2d_scan_fwd(ctypes.byref(_desc(flags=_lib.M2D_SCAN_GELU_OUT)), None) == -1   # forward-only bit: next check
    assert L.m2d_scan_bwd(ctypes.byref(_desc(flags=_lib.M2D_SCAN_GELU_OUT)), None) == -10  # ... the backward refuses it
    assert L.m2d_scan_bwd(ctypes.byref(_desc(flags=_lib.M2D_SCAN_REVERSE)), None) == -1   # known bit: next check
    assert L.m2d_scan_fwd(None, None) == -1


def test_workspace_queries(L):
    # one band (no more rows than a CTA has row-warps): the forward needs the status word only
    assert L.m2d_scan_fwd_workspace(ctypes.byref(_desc(H=4))) == 256
    # several bands: a per-CTA ring of W slots of 2 KiB
    d = _desc(B=128, H=56, W=56)
    ws = L.m2d_scan_fwd_workspace(ctypes.byref(d))
    assert ws > 256 and ws % 256 == 0 and ws <= 256 + 128 * 2 * 56 * 2048
    # backward: state record B*groups*H*W*2 KiB plus accumulators
    wb = L.m2d_scan_bwd_workspace(ctypes.byref(d))
    assert wb >= 128 * 2 * 56 * 56 * 2048
    assert L.m2d_scan_fwd_workspace(ctypes.byref(_desc(H=1))) == 0    # invalid descriptor


def test_status_word_and_chain_queries(L):
    d = _desc(B=128, H=56, W=56)
    assert L.m2d_scan_fwd_status_offset(ctypes.byref(d)) == 0
    assert L.m2d_scan_bwd_status_offset(ctypes.byref(d)) == 0
    assert L.m2d_scan_fwd_chain(ctypes.byref(d)) == 1 and L.m2d_scan_bwd_chain(ctypes.byref(d)) == 1   # enough images: one CTA each
    d = _desc(B=1, H=256, W=256)
    assert L.m2d_scan_fwd_chain(ctypes.byref(d)) > 1 and L.m2d_scan_bwd_chain(ctypes.byref(d)) > 1
    assert L.m2d_scan_fwd_status_offset(ctypes.byref(_desc(H=1))) == -1 and L.m2d_scan_fwd_chain(ctypes.byref(_desc(H=1))) == 0
    # more bands than resident CTAs: the chain closes into a ring, which must stay shorter than one
    # row of steps (W / Rb - 1 with eight row-warps)
    d = _desc(B=1, H=2400, W=24, E=32)
    assert L.m2d_scan_fwd_chain(ctypes.byref(d)) == 24 // 8 - 1
    d = _desc(B=1, H=2400, W=200, E=32)
    assert L.m2d_scan_fwd_chain(ctypes.byref(d)) == 200 // 8 - 1


def test_chain_bound_over_shrink_sequences(L):
    """A planned chain and every chain a launch may fall back to obey the same rule: never more CTAs
    than bands, and a chain that closes into a ring stays below one row of steps per band height."""
    for nbands in (1, 2, 7, 10, 128, 300):
        for steps in (2, 3, 12, 24, 56, 1024):
            for rb in (1, 2, 6, 8):
                if rb > steps:
                    continue
                want = 296
                for _ in range(40):
                    c = L.m2d_scan_chain_bound(want, nbands, steps, rb)
                    assert 1 <= c <= nbands
                    assert c == nbands or c == 1 or c <= steps // rb - 1
                    assert c <= max(want, 1)
                    if c == 1:
                        break
                    want = c - c // 4 - 1 if c > 2 else 1      # how a refused cooperative launch shrinks it
                else:
                    raise AssertionError("the shrink sequence did not reach 1")
    assert L.m2d_scan_chain_bound(4, 0, 8, 2) == 0


def test_test_hook_flag_needs_the_environment(L, monkeypatch):
    monkeypatch.delenv("M2D_TEST_HOOKS", raising=False)
    assert L.m2d_scan_fwd(ctypes.byref(_desc(flags=_lib.M2D_SCAN_TEST_WITHHOLD)), None) == -10
    monkeypatch.setenv("M2D_TEST_HOOKS", "1")
    assert L.m2d_scan_fwd(ctypes.byref(_desc(flags=_lib.M2D_SCAN_TEST_WITHHOLD)), None) == -1   # accepted: next check


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_LIB", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.lib()


def _pdesc(**kw):
    d = _lib.ProjDesc()
    d.struct_bytes = ctypes.sizeof(_lib.ProjDesc)
    d.dtype = _lib.M2D_F32
    d.P, d.E, d.R, d.N = 1000, 64, 4, 16
    d.proj_pitch = 56
    for k, v in kw.items():
        setattr(d, k, v)
    return d


def test_projection_descriptor_validation_without_a_device(L):
    assert L.m2d_dtproj_fwd(ctypes.byref(_pdesc()), None) == -1                  # NULL pointers
    assert L.m2d_dtproj_bwd(ctypes.byref(_pdesc(struct_bytes=8)), None) == -8
    assert L.m2d_dtproj_fwd(ctypes.byref(_pdesc(dtype=5)), None) == -2
    assert L.m2d_dtproj_fwd(ctypes.byref(_pdesc(P=0)), None) == -3
    assert L.m2d_dtproj_fwd(ctypes.byref(_pdesc(E=_lib.PROJ_MAX_E + 4)), None) == -9
    assert L.m2d_dtproj_bwd(ctypes.byref(_pdesc(R=_lib.PROJ_MAX_R + 1, proj_pitch=400)), None) == -9
    assert L.m2d_xproj_wgrad(ctypes.byref(_pdesc(proj_pitch=55)), None) == -5     # narrower than 2R+3N
    ws = L.m2d_proj_workspace(ctypes.byref(_pdesc()))
    assert ws > 0 and ws % 256 == 0
    assert L.m2d_proj_workspace(ctypes.byref(_pdesc(R=0))) == 0                   # invalid descriptor
