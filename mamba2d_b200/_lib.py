"""ctypes binding of the C-ABI library (include/m2d_scan.h, include/m2d_proj.h).

The library is prebuilt by ``python -m mamba2d_b200.build``.  There is no fallback: if the shared
object is missing or a call fails, this module raises.
"""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("M2D_SCAN_LIB", os.path.join(HERE, "libm2d_scan.so"))   # override: an alternative build of the same ABI

M2D_F32, M2D_BF16 = 0, 1
M2D_SCAN_REVERSE = 1
M2D_SCAN_GELU_OUT = 2
M2D_SCAN_A_LOG = 4
M2D_SCAN_TEST_WITHHOLD = 0x100
ABI_VERSION = 3
NOALLOC_SCRATCH_BYTES = 32 << 20     # M2D_NOALLOC_SCRATCH_BYTES in include/m2d_scan.h

EXPORTS = ("m2d_abi_version", "m2d_strerror", "m2d_scan_fwd_workspace", "m2d_scan_bwd_workspace",
           "m2d_scan_fwd", "m2d_scan_bwd", "m2d_scan_fwd_noalloc", "m2d_scan_fwd_noalloc_need", "m2d_scan_fwd_status_offset",
           "m2d_scan_bwd_status_offset", "m2d_scan_fwd_chain", "m2d_scan_bwd_chain", "m2d_scan_chain_bound",
           "m2d_proj_workspace", "m2d_dtproj_fwd", "m2d_dtproj_bwd", "m2d_xproj_wgrad",
           "m2d_xproj_wgrad_on_tensor_cores")
PROJ_MAX_E, PROJ_MAX_R = 640, 64     # M2D_PROJ_MAX_E / M2D_PROJ_MAX_R in include/m2d_proj.h


class ScanDesc(ctypes.Structure):
    """Mirror of ``m2d_scan_desc``."""
    _fields_ = [
        ("struct_bytes", ctypes.c_uint32), ("dtype", ctypes.c_int32),
        ("B", ctypes.c_int32), ("H", ctypes.c_int32), ("W", ctypes.c_int32), ("E", ctypes.c_int32), ("N", ctypes.c_int32),
        ("flags", ctypes.c_uint32),
        ("x", ctypes.c_void_p), ("dT", ctypes.c_void_p), ("dL", ctypes.c_void_p),
        ("AT", ctypes.c_void_p), ("AL", ctypes.c_void_p),
        ("BT", ctypes.c_void_p), ("BL", ctypes.c_void_p), ("C", ctypes.c_void_p),
        ("BT_pitch", ctypes.c_int64), ("BL_pitch", ctypes.c_int64), ("C_pitch", ctypes.c_int64),
        ("D", ctypes.c_void_p), ("y", ctypes.c_void_p), ("gy", ctypes.c_void_p),
        ("d_x", ctypes.c_void_p), ("d_dT", ctypes.c_void_p), ("d_dL", ctypes.c_void_p),
        ("d_AT", ctypes.c_void_p), ("d_AL", ctypes.c_void_p),
        ("d_BT", ctypes.c_void_p), ("d_BL", ctypes.c_void_p), ("d_C", ctypes.c_void_p), ("d_D", ctypes.c_void_p),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_uint64),
    ]


class ProjDesc(ctypes.Structure):
    """Mirror of ``m2d_proj_desc``."""
    _fields_ = [
        ("struct_bytes", ctypes.c_uint32), ("dtype", ctypes.c_int32), ("P", ctypes.c_int64),
        ("E", ctypes.c_int32), ("R", ctypes.c_int32), ("N", ctypes.c_int32), ("reserved0", ctypes.c_int32),
        ("proj_pitch", ctypes.c_int64),
        ("x", ctypes.c_void_p), ("proj", ctypes.c_void_p), ("WT", ctypes.c_void_p), ("WL", ctypes.c_void_p),
        ("bT", ctypes.c_void_p), ("bL", ctypes.c_void_p), ("dT", ctypes.c_void_p), ("dL", ctypes.c_void_p),
        ("g_dT", ctypes.c_void_p), ("g_dL", ctypes.c_void_p), ("d_proj", ctypes.c_void_p),
        ("d_WT", ctypes.c_void_p), ("d_WL", ctypes.c_void_p), ("d_bT", ctypes.c_void_p), ("d_bL", ctypes.c_void_p),
        ("d_Wx", ctypes.c_void_p), ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_uint64),
    ]


_LIB = None


def lib():
    """Load (once) and return the shared library; raises if it is not built."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m mamba2d_b200.build` "
                "(there is no CPU or PyTorch fallback for the scan)")
        L = ctypes.CDLL(LIB_PATH)
        L.m2d_abi_version.restype = ctypes.c_int
        L.m2d_strerror.restype = ctypes.c_char_p
        L.m2d_strerror.argtypes = [ctypes.c_int]
        for name in ("m2d_scan_fwd_chain", "m2d_scan_bwd_chain"):
            getattr(L, name).restype = ctypes.c_int
            getattr(L, name).argtypes = [ctypes.POINTER(ScanDesc)]
        L.m2d_scan_chain_bound.restype = ctypes.c_int
        L.m2d_scan_chain_bound.argtypes = [ctypes.c_int] * 4
        for name in ("m2d_scan_fwd_workspace", "m2d_scan_bwd_workspace", "m2d_scan_fwd_noalloc_need"):
            getattr(L, name).restype = ctypes.c_uint64
            getattr(L, name).argtypes = [ctypes.POINTER(ScanDesc)]
        for name in ("m2d_scan_fwd_status_offset", "m2d_scan_bwd_status_offset"):
            getattr(L, name).restype = ctypes.c_int64
            getattr(L, name).argtypes = [ctypes.POINTER(ScanDesc)]
        for name in ("m2d_scan_fwd", "m2d_scan_bwd", "m2d_scan_fwd_noalloc"):
            getattr(L, name).restype = ctypes.c_int
            getattr(L, name).argtypes = [ctypes.POINTER(ScanDesc), ctypes.c_void_p]
        L.m2d_proj_workspace.restype = ctypes.c_uint64
        L.m2d_proj_workspace.argtypes = [ctypes.POINTER(ProjDesc)]
        for name in ("m2d_dtproj_fwd", "m2d_dtproj_bwd", "m2d_xproj_wgrad"):
            getattr(L, name).restype = ctypes.c_int
            getattr(L, name).argtypes = [ctypes.POINTER(ProjDesc), ctypes.c_void_p]
        L.m2d_xproj_wgrad_on_tensor_cores.restype = ctypes.c_int
        L.m2d_xproj_wgrad_on_tensor_cores.argtypes = [ctypes.POINTER(ProjDesc)]
        if L.m2d_abi_version() != ABI_VERSION:
            raise RuntimeError(f"libm2d_scan.so has ABI {L.m2d_abi_version()}, expected {ABI_VERSION}")
        _LIB = L
    return _LIB


def strerror(code):
    return lib().m2d_strerror(int(code)).decode()


def check(code, what):
    if code != 0:
        raise RuntimeError(f"{what}: {strerror(code)} (status {code})")
