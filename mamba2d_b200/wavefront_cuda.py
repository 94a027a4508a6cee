"""Drop-in replacement for the reference's ``models/kernels/wavefront_cuda.py``.

Same public names and call signatures as the reference module, so ``models/mamba2d.py`` (and the
copy under ``downstream/Mamba2D``) can import this module in its place unchanged:

  wavefront_scan_cuda(x, AT_log, AL_log, x_proj_w, dt_projT_w, dt_projT_b, dt_projL_w, dt_projL_b,
                      D, recomp="partial")                      reference: wavefront_cuda.py:315-347
  wf_cuda_fn_pr.apply(x, deltaT, deltaL, AT, AL, BT, BL, C, D)   reference: wavefront_cuda.py:146-196
  wf_cuda_fn_fr.apply(x, AT_log, AL_log, x_proj_w, ..., D)       reference: wavefront_cuda.py:199-313
  proj_params(x, AT_log, AL_log, x_proj_w, ...)                  reference: wavefront_cuda.py:63-95

What differs underneath: the reference launches one kernel per anti-diagonal, materialises the 5-D
hidden state and finishes the readout and the gradient arithmetic in PyTorch.  Here the forward and
the backward are one fused sm_100a kernel each, reached through the C ABI in ``include/m2d_scan.h``.
One extension beyond the reference's signatures: every entry takes a trailing ``scan_start`` /
``reverse`` argument (default: the reference's behaviour).  ``scan_start="BR"`` runs the scan from
the bottom-right corner in place, which is what the reference's ``M2DBlock.forward`` obtains with
two ``torch.flip`` copies around the block (models/mamba2d.py:162-175) and ``M2DBlock.ssm`` with a
third one for ``double_scans`` (:190-200).

There is no PyTorch or CPU fallback: tensors must live on a CUDA device and the prebuilt library
must be present, otherwise a ``RuntimeError`` is raised.
"""
import ctypes
import os

import torch
import torch.library
import torch.nn.functional as F

from . import _lib

__all__ = ["wavefront_scan_cuda", "wf_cuda_fn_pr", "wf_cuda_fn_fr", "proj_params", "scan_fwd", "scan_bwd"]

_DTYPES = {torch.float32: _lib.M2D_F32, torch.bfloat16: _lib.M2D_BF16}
# When to read the status word a launch leaves in its workspace (reading it synchronises):
# "1" after every call, "0" never, anything else (the default) only after launches that run several
# CTAs per image -- the ones whose bounded waits cross CTAs -- and never during stream capture.
_CHECK_STATUS = os.environ.get("M2D_CHECK_STATUS", "auto")


def _check_status(kind, d, ws):
    """Raise if a bounded wait inside the launch gave up (the results are then void)."""
    if _CHECK_STATUS == "0" or torch.cuda.is_current_stream_capturing():
        return
    L = _lib.lib()
    if _CHECK_STATUS != "1" and getattr(L, f"m2d_scan_{kind}_chain")(ctypes.byref(d)) <= 1:
        return
    off = getattr(L, f"m2d_scan_{kind}_status_offset")(ctypes.byref(d))
    if off >= 0 and _status_word(ws, off) != 0:
        what = "output is" if kind == "fwd" else "gradients are"
        raise RuntimeError(f"m2d_scan_{kind}: a wait between row-warps or CTAs timed out; the {what} invalid")


def _status_word(ws, off):
    return int(ws[off:off + 4].view(torch.int32).item())      # .item() synchronises


# -----------------------------------------------------------------------------
# Descriptor plumbing
# -----------------------------------------------------------------------------

def _pixel_pitch(t, H, W, N):
    """Return (tensor, pitch) with ``tensor`` laid out as (B,H,W,N) rows of ``pitch`` elements.

    Views into a wider (B,H,W,K) buffer -- what ``proj_params`` returns for BT, BL, C -- are passed
    through untouched; anything else is made contiguous."""
    s = t.stride()
    K = s[2]
    if s[3] == 1 and K >= N and s[1] == W * K and s[0] == H * W * K:
        return t, K
    return t.contiguous(), N


def _check_inputs(x, dT, dL, AT, AL, BT, BL, C, D, gy=None, a_log=False):
    if x.dim() != 4:
        raise RuntimeError(f"x must be (B,H,W,E), got {tuple(x.shape)}")
    if not x.is_cuda:
        raise RuntimeError("wavefront scan: tensors must be on a CUDA device (there is no CPU path)")
    if x.dtype not in _DTYPES:
        raise RuntimeError(f"wavefront scan: unsupported dtype {x.dtype} (float32 and bfloat16 only)")
    B, H, W, E = x.shape
    if AT.dim() != 2 or AT.shape[0] != E:
        raise RuntimeError(f"AT must be (E,N) with E={E}, got {tuple(AT.shape)}")
    N = AT.shape[1]
    want = {"deltaT": (dT, (B, H, W, E)), "deltaL": (dL, (B, H, W, E)), "AL": (AL, (E, N)),
            "BT": (BT, (B, H, W, N)), "BL": (BL, (B, H, W, N)), "C": (C, (B, H, W, N)), "D": (D, (E,))}
    if gy is not None:
        want["grad_output"] = (gy, (B, H, W, E))
    for name, (t, shape) in want.items():
        if tuple(t.shape) != shape:
            raise RuntimeError(f"{name} must have shape {shape}, got {tuple(t.shape)}")
    for name, t in [("x", x), ("AT", AT)] + [(k, v[0]) for k, v in want.items()]:
        expect = torch.float32 if (a_log and name in ("AT", "AL")) else x.dtype     # A_log is an fp32 parameter
        if t.dtype != expect:
            raise RuntimeError(f"{name} has dtype {t.dtype}, expected {expect}")
        if t.device != x.device:
            raise RuntimeError(f"{name} is on {t.device}, expected {x.device}")
    return B, H, W, E, N


def _make_desc(x, dT, dL, AT, AL, BT, BL, C, D, reverse=False, gelu_out=False, a_log=False):
    B, H, W, E = x.shape
    N = AT.shape[1]
    keep = []   # tensors that must outlive the launch call
    d = _lib.ScanDesc()
    d.struct_bytes = ctypes.sizeof(_lib.ScanDesc)
    d.dtype = _DTYPES[x.dtype]
    d.B, d.H, d.W, d.E, d.N = B, H, W, E, N
    d.flags = ((_lib.M2D_SCAN_REVERSE if reverse else 0) | (_lib.M2D_SCAN_GELU_OUT if gelu_out else 0)
               | (_lib.M2D_SCAN_A_LOG if a_log else 0))
    for name, t in (("x", x), ("dT", dT), ("dL", dL), ("AT", AT), ("AL", AL), ("D", D)):
        t = t.contiguous()
        keep.append(t)
        setattr(d, name, t.data_ptr())
    for name, t in (("BT", BT), ("BL", BL), ("C", C)):
        t, pitch = _pixel_pitch(t, H, W, N)
        keep.append(t)
        setattr(d, name, t.data_ptr())
        setattr(d, name + "_pitch", pitch)
    return d, keep


def _workspace(d, nbytes, device, keep):
    if nbytes:
        ws = torch.empty(int(nbytes), dtype=torch.uint8, device=device)
        keep.append(ws)
        d.workspace = ws.data_ptr()
        d.workspace_bytes = int(nbytes)


def scan_fwd(x, deltaT, deltaL, AT, AL, BT, BL, C, D, reverse=False, gelu_out=False, a_log=False):
    """Fused forward: y (B,H,W,E) in ``x.dtype``.  Inputs as ``wf_cuda_fn_pr.apply`` takes them.

    ``gelu_out=True`` returns ``gelu(y)`` (erf form), applied inside the kernel's store: what the
    reference block computes with a separate ``nn.GELU()`` pass after the scan (models/mamba2d.py:169).
    There is no backward for it; it is for inference.

    ``a_log=True``: ``AT`` / ``AL`` are the fp32 parameters ``AT_log`` / ``AL_log`` and the kernel uses
    ``A = -exp(A_log)`` (rounded to ``x.dtype`` as the reference's cast does,
    models/kernels/wavefront_cuda.py:72-73, :89-90), which saves the elementwise launches that compute A.

    ``reverse=True`` scans from the bottom-right corner: the result equals
    ``scan_fwd(*[t.flip(1, 2) for t in pixel_tensors], ...).flip(1, 2)`` without any copy.

    With few images on a large map the kernel runs several CTAs per image that wait on one another
    with bounded polling.  After such a launch the wrapper synchronises and raises if a wait gave
    up (status word in the workspace, see m2d_scan_fwd_status_offset); ``M2D_CHECK_STATUS=1``
    extends that check to every launch, ``M2D_CHECK_STATUS=0`` switches it off."""
    _check_inputs(x, deltaT, deltaL, AT, AL, BT, BL, C, D, a_log=a_log)
    L = _lib.lib()
    with torch.cuda.device(x.device):
        d, keep = _make_desc(x, deltaT, deltaL, AT, AL, BT, BL, C, D, reverse, gelu_out, a_log)
        y = torch.empty(x.shape, dtype=x.dtype, device=x.device)
        d.y = y.data_ptr()
        _workspace(d, L.m2d_scan_fwd_workspace(ctypes.byref(d)), x.device, keep)
        rc = L.m2d_scan_fwd(ctypes.byref(d), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    _lib.check(rc, "m2d_scan_fwd")
    _check_status("fwd", d, keep[-1])
    return y


def scan_bwd(x, deltaT, deltaL, AT, AL, BT, BL, C, D, grad_output, reverse=False, shared_storage=True, a_log=False):
    """Fused backward with recomputation.  Returns the nine gradients
    (d_x, d_deltaT, d_deltaL, d_AT, d_AL, d_BT, d_BL, d_C, d_D), all in ``x.dtype``.

    With ``shared_storage`` the reduced gradients are disjoint views of two allocations (per-pixel
    and per-channel ones), which lets the library zero them with two memsets; the registered
    operator asks for separate tensors, because operator outputs must not share storage.

    ``a_log=True``: ``AT`` / ``AL`` are the fp32 parameters A_log (see ``scan_fwd``) and ``d_AT`` / ``d_AL``
    come back as fp32 gradients with respect to them (``d_A * A``)."""
    B, H, W, E, N = _check_inputs(x, deltaT, deltaL, AT, AL, BT, BL, C, D, grad_output, a_log=a_log)
    L = _lib.lib()
    dev, dt = x.device, x.dtype
    with torch.cuda.device(dev):
        d, keep = _make_desc(x, deltaT, deltaL, AT, AL, BT, BL, C, D, reverse, False, a_log)
        gy = grad_output.contiguous()
        keep.append(gy)
        d.gy = gy.data_ptr()
        # the three per-pixel reduced gradients are carved out of one buffer and the three per-channel
        # ones out of another, in the order the library zeroes them: two memsets instead of six.  (One
        # buffer for all six would let the tiny d_D, which autograd may keep as D.grad, pin the
        # large per-pixel storage until the gradients are cleared.)
        npn, en = B * H * W * N, E * N
        dt_A = torch.float32 if a_log else dt                     # gradients of the fp32 parameter A_log are fp32
        if shared_storage:
            big = torch.empty(3 * npn, dtype=dt, device=dev)
            d_BT, d_BL, d_C = (big[k * npn:(k + 1) * npn].view(B, H, W, N) for k in range(3))
        else:
            d_BT, d_BL, d_C = (torch.empty((B, H, W, N), dtype=dt, device=dev) for _ in range(3))
        if shared_storage and dt_A == dt:
            small = torch.empty(2 * en + E, dtype=dt, device=dev)
            d_AT, d_AL = (small[k * en:(k + 1) * en].view(E, N) for k in range(2))
            d_D = small[2 * en:]
        else:
            d_AT, d_AL = (torch.empty((E, N), dtype=dt_A, device=dev) for _ in range(2))
            d_D = torch.empty((E,), dtype=dt, device=dev)
        outs = (torch.empty((B, H, W, E), dtype=dt, device=dev), torch.empty((B, H, W, E), dtype=dt, device=dev),
                torch.empty((B, H, W, E), dtype=dt, device=dev), d_AT, d_AL, d_BT, d_BL, d_C, d_D)
        for name, t in zip(("d_x", "d_dT", "d_dL", "d_AT", "d_AL", "d_BT", "d_BL", "d_C", "d_D"), outs):
            setattr(d, name, t.data_ptr())
        _workspace(d, L.m2d_scan_bwd_workspace(ctypes.byref(d)), dev, keep)
        rc = L.m2d_scan_bwd(ctypes.byref(d), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    _lib.check(rc, "m2d_scan_bwd")
    _check_status("bwd", d, keep[-1])
    return outs


# -----------------------------------------------------------------------------
# Custom operators (opaque to torch.compile; the reference registers mamba2d::wf_fwd / wf_bwd,
# wavefront_cuda.py:25-57)
# -----------------------------------------------------------------------------

_EAGER = {}     # operator -> its Python body


def _run(op, *args):
    """The registered operator while a compiler is tracing (it needs the opaque op and its fake);
    the operator's Python body directly in eager mode, where the dispatcher round trip of a custom
    operator costs more than the small stages' kernels."""
    return op(*args) if torch.compiler.is_compiling() else _EAGER[op](*args)


@torch.library.custom_op("mamba2d_b200::scan_fwd", mutates_args=())
def scan_fwd_op(x: torch.Tensor, deltaT: torch.Tensor, deltaL: torch.Tensor, AT: torch.Tensor, AL: torch.Tensor,
                BT: torch.Tensor, BL: torch.Tensor, C: torch.Tensor, D: torch.Tensor,
                reverse: bool = False, a_log: bool = False) -> torch.Tensor:
    return scan_fwd(x, deltaT, deltaL, AT, AL, BT, BL, C, D, reverse, False, a_log)


@scan_fwd_op.register_fake
def _scan_fwd_fake(x, deltaT, deltaL, AT, AL, BT, BL, C, D, reverse=False, a_log=False):
    return torch.empty_like(x, memory_format=torch.contiguous_format)


@torch.library.custom_op("mamba2d_b200::scan_bwd", mutates_args=())
def scan_bwd_op(x: torch.Tensor, deltaT: torch.Tensor, deltaL: torch.Tensor, AT: torch.Tensor, AL: torch.Tensor,
                BT: torch.Tensor, BL: torch.Tensor, C: torch.Tensor, D: torch.Tensor,
                grad_output: torch.Tensor, reverse: bool = False, a_log: bool = False) -> list[torch.Tensor]:
    return list(scan_bwd(x, deltaT, deltaL, AT, AL, BT, BL, C, D, grad_output, reverse, shared_storage=False, a_log=a_log))


@scan_bwd_op.register_fake
def _scan_bwd_fake(x, deltaT, deltaL, AT, AL, BT, BL, C, D, grad_output, reverse=False, a_log=False):
    B, H, W, E = x.shape
    N = AT.shape[1]
    mk = lambda *s: x.new_empty(s)
    mkA = (lambda *s: AT.new_empty(s)) if a_log else mk
    return [mk(B, H, W, E), mk(B, H, W, E), mk(B, H, W, E), mkA(E, N), mkA(E, N),
            mk(B, H, W, N), mk(B, H, W, N), mk(B, H, W, N), mk(E)]


# -----------------------------------------------------------------------------
# Projections.  The x projection and its data gradient are GEMMs and stay on the GEMM library; the
# rank-R dt projections with their softplus, their backward, and the weight gradient of the x
# projection (reductions over every pixel into a tiny matrix) are fused kernels of this library
# (include/m2d_proj.h).  CPU tensors and shapes outside the kernels' range take the plain PyTorch
# formulation, which is what the reference runs everywhere (wavefront_cuda.py:63-95).
# -----------------------------------------------------------------------------

def _proj_desc(proj, E, R, N):
    d = _lib.ProjDesc()
    d.struct_bytes = ctypes.sizeof(_lib.ProjDesc)
    d.dtype = _DTYPES[proj.dtype]
    d.P = proj.numel() // proj.shape[-1]
    d.E, d.R, d.N = E, R, N
    d.proj_pitch = proj.shape[-1]
    return d


def _proj_call(fn_name, d, device, keep):
    L = _lib.lib()
    with torch.cuda.device(device):
        _workspace(d, L.m2d_proj_workspace(ctypes.byref(d)), device, keep)
        rc = getattr(L, fn_name)(ctypes.byref(d), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    _lib.check(rc, fn_name)


def _fusable(x, proj_cols, R, *others):
    """The fused projection kernels cover CUDA tensors in fp32 / bf16 with E <= 640, a dt rank of at
    most 64 and (rounded up to a power of two) at most a quarter of the channels, and channel
    counts / row pitches that are multiples of 4 (every shipped model)."""
    E = x.shape[-1]
    rank_bucket = next((b for b in (4, 8, 16, 32, 64) if R <= b), None)
    # one dtype and one device for everything the kernels touch (under autocast the projection
    # output can be bf16 next to fp32 weights: that case takes the PyTorch formulation)
    if any(t.dtype != x.dtype or t.device != x.device for t in others):
        return False
    if (x.numel() // E) * max(E, proj_cols) >= (1 << 31) - (1 << 26):      # 31-bit element indices in the kernels
        return False
    return (x.is_cuda and x.dtype in _DTYPES and E <= _lib.PROJ_MAX_E and rank_bucket is not None
            and 4 * rank_bucket <= (E + 31) // 32 * 32 and E % 4 == 0 and proj_cols % 4 == 0)


def _dtproj_fwd(proj, WT, bT, WL, bL, d_state):
    """deltaT, deltaL = softplus(proj[..., :R] @ WT^T + bT), softplus(proj[..., R:2R] @ WL^T + bL)."""
    E, R = WT.shape
    proj = proj.contiguous()
    keep = [t.contiguous() for t in (WT, WL, bT, bL)]
    d = _proj_desc(proj, E, R, d_state)
    d.proj = proj.data_ptr()
    d.WT, d.WL, d.bT, d.bL = (t.data_ptr() for t in keep)
    dT = torch.empty(proj.shape[:-1] + (E,), dtype=proj.dtype, device=proj.device)
    dL = torch.empty_like(dT)
    d.dT, d.dL = dT.data_ptr(), dL.data_ptr()
    _proj_call("m2d_dtproj_fwd", d, proj.device, keep)
    return [dT, dL]


@torch.library.custom_op("mamba2d_b200::dtproj_fwd", mutates_args=())
def dtproj_fwd_op(proj: torch.Tensor, WT: torch.Tensor, bT: torch.Tensor, WL: torch.Tensor, bL: torch.Tensor,
                  d_state: int) -> list[torch.Tensor]:
    return _dtproj_fwd(proj, WT, bT, WL, bL, d_state)


@dtproj_fwd_op.register_fake
def _dtproj_fwd_fake(proj, WT, bT, WL, bL, d_state):
    shape = proj.shape[:-1] + (WT.shape[0],)
    return [proj.new_empty(shape), proj.new_empty(shape)]


def _dtproj_bwd(g_dT, g_dL, deltaT, deltaL, proj, WT, WL, g_BT, g_BL, g_C):
    """Backward of dtproj_fwd.  Returns [d_proj, d_WT, d_bT, d_WL, d_bL]: ``d_proj`` is the whole
    gradient of the x-projection output -- columns [0, 2R) from the kernel, the rest copied from the
    upstream gradients of BT, BL, C."""
    E, R = WT.shape
    N = g_BT.shape[-1]
    keep = [t.contiguous() for t in (g_dT, g_dL, deltaT, deltaL, proj, WT, WL)]
    d_proj = torch.empty_like(keep[4])
    for k, g in enumerate((g_BT, g_BL, g_C)):
        d_proj[..., 2 * R + k * N:2 * R + (k + 1) * N].copy_(g)
    d = _proj_desc(keep[4], E, R, N)
    d.g_dT, d.g_dL, d.dT, d.dL, d.proj, d.WT, d.WL = (t.data_ptr() for t in keep)
    d.d_proj = d_proj.data_ptr()
    outs = [d_proj, torch.empty_like(keep[5]), torch.empty(E, dtype=proj.dtype, device=proj.device),
            torch.empty_like(keep[6]), torch.empty(E, dtype=proj.dtype, device=proj.device)]
    d.d_WT, d.d_bT, d.d_WL, d.d_bL = (t.data_ptr() for t in outs[1:])
    _proj_call("m2d_dtproj_bwd", d, proj.device, keep)
    return outs


@torch.library.custom_op("mamba2d_b200::dtproj_bwd", mutates_args=())
def dtproj_bwd_op(g_dT: torch.Tensor, g_dL: torch.Tensor, deltaT: torch.Tensor, deltaL: torch.Tensor, proj: torch.Tensor,
                  WT: torch.Tensor, WL: torch.Tensor, g_BT: torch.Tensor, g_BL: torch.Tensor,
                  g_C: torch.Tensor) -> list[torch.Tensor]:
    return _dtproj_bwd(g_dT, g_dL, deltaT, deltaL, proj, WT, WL, g_BT, g_BL, g_C)


@dtproj_bwd_op.register_fake
def _dtproj_bwd_fake(g_dT, g_dL, deltaT, deltaL, proj, WT, WL, g_BT, g_BL, g_C):
    E = WT.shape[0]
    return [torch.empty_like(proj, memory_format=torch.contiguous_format), torch.empty_like(WT), WT.new_empty(E),
            torch.empty_like(WL), WL.new_empty(E)]


def _xproj_wgrad(d_proj, x, d_state, dt_rank):
    """d_Wx = d_proj^T @ x over all pixels: (2R+3N, E)."""
    E = x.shape[-1]
    keep = [d_proj.contiguous(), x.contiguous()]
    d = _proj_desc(keep[0], E, dt_rank, d_state)
    d.d_proj, d.x = keep[0].data_ptr(), keep[1].data_ptr()
    out = torch.empty(2 * dt_rank + 3 * d_state, E, dtype=x.dtype, device=x.device)
    d.d_Wx = out.data_ptr()
    _proj_call("m2d_xproj_wgrad", d, x.device, keep)
    return out


@torch.library.custom_op("mamba2d_b200::xproj_wgrad", mutates_args=())
def xproj_wgrad_op(d_proj: torch.Tensor, x: torch.Tensor, d_state: int, dt_rank: int) -> torch.Tensor:
    return _xproj_wgrad(d_proj, x, d_state, dt_rank)


@xproj_wgrad_op.register_fake
def _xproj_wgrad_fake(d_proj, x, d_state, dt_rank):
    return x.new_empty(2 * dt_rank + 3 * d_state, x.shape[-1])


_EAGER.update({scan_fwd_op: lambda *a: scan_fwd(*a[:10], False, *a[10:]),
               scan_bwd_op: lambda *a: list(scan_bwd(*a[:11], True, *a[11:])), dtproj_fwd_op: _dtproj_fwd,
               dtproj_bwd_op: _dtproj_bwd, xproj_wgrad_op: _xproj_wgrad})


def _proj_forward(x, AT_log, AL_log, x_proj_w, dt_projT_w, dt_projT_b, dt_projL_w, dt_projL_b, want_A=True):
    """``proj_params`` without an autograd graph.  Returns the seven outputs and what the
    hand-written backward needs: (proj, AT32, AL32) -- softplus' is recovered from deltaT / deltaL
    themselves, so the pre-activations are not kept.  Without ``want_A`` the two A outputs are the
    fp32 parameters A_log themselves (the scan kernels then apply ``-exp`` on their own) and AT32 /
    AL32 are None."""
    d_state, dt_rank, dt = AT_log.shape[1], dt_projT_w.shape[1], x.dtype
    AT32 = -torch.exp(AT_log.float()) if want_A else None
    AL32 = -torch.exp(AL_log.float()) if want_A else None
    proj = F.linear(x, x_proj_w)
    rT, rL, BT, BL, C = torch.split(proj, [dt_rank, dt_rank, d_state, d_state, d_state], dim=-1)
    if _fusable(x, proj.shape[-1], dt_rank, proj, dt_projT_w, dt_projT_b, dt_projL_w, dt_projL_b):
        deltaT, deltaL = _run(dtproj_fwd_op, proj, dt_projT_w, dt_projT_b, dt_projL_w, dt_projL_b, d_state)
    else:
        deltaT = F.softplus(F.linear(rT, dt_projT_w, dt_projT_b))
        deltaL = F.softplus(F.linear(rL, dt_projL_w, dt_projL_b))
    A_out = (AT32.to(dtype=dt), AL32.to(dtype=dt)) if want_A else (AT_log.float(), AL_log.float())
    out = (deltaT.to(dtype=dt), deltaL.to(dtype=dt), *A_out, BT.to(dtype=dt), BL.to(dtype=dt), C.to(dtype=dt))
    return out, (proj, AT32, AL32)


def _proj_backward(x, AT_log, AL_log, x_proj_w, dt_projT_w, dt_projL_w, deltaT, deltaL, saved,
                   d_dT, d_dL, d_AT, d_AL, d_BT, d_BL, d_C):
    """Gradients of ``proj_params`` (wavefront_cuda.py:63-95 in the reference) written out by hand:
    softplus', the two dt projections, the x projection and the ``-exp(A_log)`` transform.  A
    missing (None) upstream gradient counts as zero.
    Returns (d_x, d_AT_log, d_AL_log, d_x_proj_w, d_dt_projT_w, d_dt_projT_b, d_dt_projL_w, d_dt_projL_b)."""
    proj, AT32, AL32 = saved
    E, R, N = x.shape[-1], dt_projT_w.shape[1], AT_log.shape[1]
    dt = x.dtype
    zeros_like_delta = lambda: torch.zeros_like(deltaT)
    d_dT = zeros_like_delta() if d_dT is None else d_dT.to(dt)
    d_dL = zeros_like_delta() if d_dL is None else d_dL.to(dt)
    zeros_n = lambda: torch.zeros(proj.shape[:-1] + (N,), dtype=dt, device=proj.device)
    d_BT, d_BL, d_C = (zeros_n() if g is None else g for g in (d_BT, d_BL, d_C))
    if _fusable(x, proj.shape[-1], R, proj, dt_projT_w, dt_projL_w, deltaT, deltaL, d_dT, d_dL, d_BT, d_BL, d_C):
        d_proj, d_wT, d_bT, d_wL, d_bL = _run(dtproj_bwd_op, d_dT, d_dL, deltaT, deltaL, proj, dt_projT_w, dt_projL_w,
                                              d_BT, d_BL, d_C)
        d_wx = _run(xproj_wgrad_op, d_proj, x, N, R)
    else:
        # softplus'(z) = 1 - exp(-softplus(z)); values past the threshold of 20 give exactly 1
        sT = d_dT * (-torch.expm1(-deltaT.float())).to(dt)
        sL = d_dL * (-torch.expm1(-deltaL.float())).to(dt)
        rT, rL = proj[..., :R].to(dt), proj[..., R:2 * R].to(dt)       # (bf16 under autocast next to fp32 tensors)
        d_proj = torch.cat([sT @ dt_projT_w.to(dt), sL @ dt_projL_w.to(dt), d_BT.to(dt), d_BL.to(dt), d_C.to(dt)], dim=-1)
        d_wT = sT.reshape(-1, E).t() @ rT.reshape(-1, R)
        d_wL = sL.reshape(-1, E).t() @ rL.reshape(-1, R)
        d_bT, d_bL = sT.reshape(-1, E).sum(0), sL.reshape(-1, E).sum(0)
        d_wx = d_proj.reshape(-1, d_proj.shape[-1]).t() @ x.reshape(-1, E)
    d_x = d_proj @ x_proj_w.to(d_proj.dtype)
    # d(-exp(a))/da = -exp(a) = A.  (Callers that let the scan kernels apply -exp pass None here: the
    # kernels return d_A_log themselves.)
    d_AT_log = None if d_AT is None else (d_AT.float() * AT32).to(AT_log.dtype)
    d_AL_log = None if d_AL is None else (d_AL.float() * AL32).to(AL_log.dtype)
    return d_x, d_AT_log, d_AL_log, d_wx, d_wT, d_bT, d_wL, d_bL


class _proj_params_fn(torch.autograd.Function):
    """``proj_params`` as one autograd node with the hand-written backward."""

    @staticmethod
    def forward(ctx, x, AT_log, AL_log, x_proj_w, dt_projT_w, dt_projT_b, dt_projL_w, dt_projL_b):
        out, saved = _proj_forward(x, AT_log, AL_log, x_proj_w, dt_projT_w, dt_projT_b, dt_projL_w, dt_projL_b)
        if torch.compiler.is_compiling():
            # Outputs that share storage with a saved intermediate (BT/BL/C are views of the projection
            # output; a same-dtype .to() returns its argument) lose their gradient when the graph
            # compiler traces this Function (observed with PyTorch 2.11: zero gradients, no error).
            # Fresh copies cost three extra passes there; eager mode keeps the views.
            out = tuple(t.clone() for t in out)
        ctx.save_for_backward(x, AT_log, AL_log, x_proj_w, dt_projT_w, dt_projL_w, out[0], out[1], *saved)
        return out

    @staticmethod
    def backward(ctx, d_dT, d_dL, d_AT, d_AL, d_BT, d_BL, d_C):
        x, AT_log, AL_log, x_proj_w, dt_projT_w, dt_projL_w, deltaT, deltaL, proj, AT32, AL32 = ctx.saved_tensors
        g = _proj_backward(x, AT_log, AL_log, x_proj_w, dt_projT_w, dt_projL_w, deltaT, deltaL, (proj, AT32, AL32),
                           d_dT, d_dL, d_AT, d_AL, d_BT, d_BL, d_C)
        d_x, d_AT_log, d_AL_log, d_wx, d_wT, d_bT, d_wL, d_bL = g
        return d_x, d_AT_log, d_AL_log, d_wx, d_wT, d_bT, d_wL, d_bL


class _proj5_fn(torch.autograd.Function):
    """The input-dependent outputs of ``proj_params`` only (deltaT, deltaL, BT, BL, C): what the entry
    uses when the scan kernels take A_log directly."""

    @staticmethod
    def forward(ctx, x, x_proj_w, dt_projT_w, dt_projT_b, dt_projL_w, dt_projL_b, A_like):
        out, saved = _proj_forward(x, A_like, A_like, x_proj_w, dt_projT_w, dt_projT_b, dt_projL_w, dt_projL_b, want_A=False)
        out = (out[0], out[1], out[4], out[5], out[6])
        if torch.compiler.is_compiling():
            out = tuple(t.clone() for t in out)       # see _proj_params_fn.forward
        ctx.save_for_backward(x, x_proj_w, dt_projT_w, dt_projL_w, out[0], out[1], saved[0], A_like)
        return out

    @staticmethod
    def backward(ctx, d_dT, d_dL, d_BT, d_BL, d_C):
        x, x_proj_w, dt_projT_w, dt_projL_w, deltaT, deltaL, proj, A_like = ctx.saved_tensors
        g = _proj_backward(x, A_like, A_like, x_proj_w, dt_projT_w, dt_projL_w, deltaT, deltaL, (proj, None, None),
                           d_dT, d_dL, None, None, d_BT, d_BL, d_C)
        d_x, _, _, d_wx, d_wT, d_bT, d_wL, d_bL = g
        return d_x, d_wx, d_wT, d_bT, d_wL, d_bL, None


def proj_params(x, AT_log, AL_log, x_proj_w, dt_projT_w, dt_projT_b, dt_projL_w, dt_projL_b):
    """Input-dependent scan parameters from x (B,H,W,E).

    Returns deltaT, deltaL (B,H,W,E), AT, AL (E,N), BT, BL, C (B,H,W,N), all in ``x.dtype``;
    BT/BL/C are views into the x-projection output (pixel pitch 2R+3N), which the scan kernels
    read in place.  Differentiable: one autograd node whose backward is written by hand."""
    return _proj_params_fn.apply(x, AT_log, AL_log, x_proj_w, dt_projT_w, dt_projT_b, dt_projL_w, dt_projL_b)


# -----------------------------------------------------------------------------
# Autograd Functions
# -----------------------------------------------------------------------------

class wf_cuda_fn_pr(torch.autograd.Function):
    """Partial recomputation: projections are computed once and saved; the hidden state is
    recomputed inside the backward kernel.  With ``a_log`` the ``AT`` / ``AL`` arguments are the fp32
    parameters A_log and their gradients are gradients with respect to A_log."""

    @staticmethod
    def forward(ctx, x, deltaT, deltaL, AT, AL, BT, BL, C, D, reverse=False, a_log=False):
        y = _run(scan_fwd_op, x, deltaT, deltaL, AT, AL, BT, BL, C, D, reverse, a_log)
        ctx.save_for_backward(x, deltaT, deltaL, AT, AL, BT, BL, C, D)
        ctx.reverse, ctx.a_log = bool(reverse), bool(a_log)
        return y

    @staticmethod
    def backward(ctx, grad_output):
        x, deltaT, deltaL, AT, AL, BT, BL, C, D = ctx.saved_tensors
        grads = _run(scan_bwd_op, x, deltaT, deltaL, AT, AL, BT, BL, C, D, grad_output.to(x.dtype), ctx.reverse, ctx.a_log)
        return (*grads, None, None)


class wf_cuda_fn_fr(torch.autograd.Function):
    """Full recomputation: only x and the weights are saved; the projections are recomputed in
    backward.  The reference recomputes them under autograd and calls ``torch.autograd.grad``
    (wavefront_cuda.py:235-302); here their backward is written out (``_proj_backward``).  The scan
    kernels take A_log directly, so neither pass computes ``-exp(A_log)`` in PyTorch."""

    @staticmethod
    def forward(ctx, x, AT_log, AL_log, x_proj_w, dt_projT_w, dt_projT_b, dt_projL_w, dt_projL_b, D, reverse=False):
        with torch.no_grad():
            (deltaT, deltaL, AT, AL, BT, BL, C), _ = _proj_forward(
                x, AT_log, AL_log, x_proj_w, dt_projT_w, dt_projT_b, dt_projL_w, dt_projL_b, want_A=False)
        y = _run(scan_fwd_op, x, deltaT, deltaL, AT, AL, BT, BL, C, D, reverse, True)
        ctx.reverse = bool(reverse)
        ctx.save_for_backward(x, AT_log, AL_log, x_proj_w, dt_projT_w, dt_projT_b, dt_projL_w, dt_projL_b, D)
        return y

    @staticmethod
    def backward(ctx, grad_output):
        x, AT_log, AL_log, x_proj_w, dt_projT_w, dt_projT_b, dt_projL_w, dt_projL_b, D = ctx.saved_tensors
        grad_output = grad_output.to(x.dtype)
        with torch.no_grad():
            (deltaT, deltaL, AT, AL, BT, BL, C), saved = _proj_forward(
                x, AT_log, AL_log, x_proj_w, dt_projT_w, dt_projT_b, dt_projL_w, dt_projL_b, want_A=False)
            d_x_scan, d_dT, d_dL, d_AT_log, d_AL_log, d_BT, d_BL, d_C, d_D = _run(
                scan_bwd_op, x, deltaT, deltaL, AT, AL, BT, BL, C, D, grad_output, ctx.reverse, True)
            g = _proj_backward(x, AT_log, AL_log, x_proj_w, dt_projT_w, dt_projL_w, deltaT, deltaL, saved,
                               d_dT, d_dL, None, None, d_BT, d_BL, d_C)
        d_x = d_x_scan + g[0]
        return (d_x, d_AT_log.to(AT_log.dtype), d_AL_log.to(AL_log.dtype), *g[3:], d_D, None)


def wavefront_scan_cuda(x, AT_log, AL_log, x_proj_w, dt_projT_w, dt_projT_b, dt_projL_w, dt_projL_b, D, recomp="partial",
                        scan_start="TL", act_out=None):
    """The op as ``M2DBlock.ssm`` calls it.

    Args:
        recomp: ``"partial"`` saves the projections for backward; ``"full"`` saves only x and the
            weights and recomputes the projections in backward (less memory, slower).
        scan_start: ``"TL"`` (the reference's only direction) or ``"BR"``: scan from the bottom-right
            corner, equal to ``wavefront_scan_cuda(x.flip(1, 2), ...).flip(1, 2)`` without the copies.
        act_out: ``None`` or ``"gelu"``: return ``gelu(y)``, erf form, as the block's ``act2`` computes
            it (models/mamba2d.py:169).  Without gradients in play the activation is applied inside
            the kernel's store; otherwise it is an ordinary PyTorch op after the scan.
    Raises:
        ValueError: if H < 2 or W < 2, or for an unknown ``recomp`` (same conditions as the
            reference) or ``scan_start``.
    """
    if scan_start not in ("TL", "BR"):
        raise ValueError(f"Unknown scan start corner, got {scan_start}...")
    if act_out not in (None, "gelu"):
        raise ValueError(f"Unknown output activation, got {act_out}...")
    reverse = scan_start == "BR"
    _, H, W, _ = x.shape
    if H < 2 or W < 2:
        raise ValueError(f"Wavefront scan kernel requires spatial dims > 1. Got H={H}, W={W}.")

    x_proj_w = x_proj_w.to(x.dtype)
    dt_projT_w = dt_projT_w.to(x.dtype)
    dt_projT_b = dt_projT_b.to(x.dtype)
    dt_projL_w = dt_projL_w.to(x.dtype)
    dt_projL_b = dt_projL_b.to(x.dtype)
    D = D.to(x.dtype)

    if recomp not in ("partial", "full"):
        raise ValueError(f"Unknown recomputation mode, got {recomp}...")
    params = (x, AT_log, AL_log, x_proj_w, dt_projT_w, dt_projT_b, dt_projL_w, dt_projL_b, D)
    if act_out == "gelu" and not (torch.is_grad_enabled() and any(t.requires_grad for t in params)) \
            and not torch.compiler.is_compiling():
        # nothing to differentiate: one kernel for scan + activation
        (deltaT, deltaL, AT, AL, BT, BL, C), _ = _proj_forward(*params[:-1], want_A=False)
        return scan_fwd(x, deltaT, deltaL, AT, AL, BT, BL, C, D, reverse, gelu_out=True, a_log=True)
    if recomp == "partial":
        # the scan kernels take A_log directly (A = -exp(A_log) and its gradient are applied inside
        # them), so only the input-dependent projections are computed here
        deltaT, deltaL, BT, BL, C = _proj5_fn.apply(x, x_proj_w, dt_projT_w, dt_projT_b, dt_projL_w, dt_projL_b, AT_log)
        y = wf_cuda_fn_pr.apply(x, deltaT, deltaL, AT_log.float(), AL_log.float(), BT, BL, C, D, reverse, True)
    else:
        y = wf_cuda_fn_fr.apply(x, AT_log, AL_log, x_proj_w, dt_projT_w, dt_projT_b, dt_projL_w, dt_projL_b, D, reverse)
    return F.gelu(y) if act_out == "gelu" else y
