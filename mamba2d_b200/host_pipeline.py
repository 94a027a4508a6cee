"""Scan calls whose tensors live in HOST memory, pipelined over three CUDA streams.

The reference op only accepts device tensors (models/kernels/wavefront_cuda.py:315-347 raises
inside the extension otherwise); a caller that keeps activations on the host has to copy them in,
run the op and copy the results out, one after the other on one stream.  ``HostScanPipeline`` does
the same three stages on three streams, so that while one call's kernels run the next call's
inputs are already crossing PCIe in one direction and the previous call's results in the other:

    copy-in stream    H2D(k+1)
    compute stream    m2d_scan_fwd(k) [+ m2d_scan_bwd(k)]
    copy-out stream   D2H(k-1)

Throughput is then bounded by the slowest of the three stages instead of their sum.  Results are
identical to ``scan_fwd`` / ``scan_bwd`` on the same values: the kernels are the same C-ABI entry
points, launched on the pipeline's compute stream.  There is no CPU path here either: the copies
and kernels need a CUDA device.

    pipe = HostScanPipeline("cuda:0", depth=3)
    t = pipe.submit(x, dT, dL, AT, AL, BT, BL, C, D, grad_output=gy)     # host tensors, pinned for overlap
    ...                                                                  # submit more work
    t.wait()                                                             # t.y, t.grads are pinned host tensors
"""
import collections

import torch

from . import wavefront_cuda as _wc

__all__ = ["HostScanPipeline", "ScanTicket"]


class ScanTicket:
    """One submitted call.  ``y`` and ``grads`` (None for a forward-only call) are pinned host
    tensors; their contents are valid once ``wait()`` has returned (or ``done()`` is True)."""

    def __init__(self, y, grads, event, keep):
        self.y, self.grads = y, grads
        self._event = event
        # Device tensors of this call.  They were allocated on one stream and are used on another;
        # instead of telling the allocator (record_stream), they are simply kept alive until the
        # last stream is known to be done with them, and released only then.
        self._keep = keep

    @property
    def outputs(self):
        """The host buffers of this call (y first, then the nine gradients), reusable as ``out=``
        of a later ``submit`` once this ticket has been waited for."""
        return [self.y] + (list(self.grads) if self.grads is not None else [])

    def done(self):
        ok = self._event.query()
        if ok:
            self._keep = None
        return ok

    def wait(self):
        self._event.synchronize()
        self._keep = None
        return self


class HostScanPipeline:
    """Forward (and backward) scans on host tensors with copy-in, compute and copy-out overlapped.

    Args:
        device: CUDA device of the pipeline (default: the current one).
        depth: calls allowed in flight; ``submit`` blocks the host on the oldest one beyond that,
            which bounds the device memory held by queued work.
    """

    def __init__(self, device=None, depth=3):
        if not torch.cuda.is_available():
            raise RuntimeError("HostScanPipeline needs a CUDA device (there is no CPU path)")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError(f"HostScanPipeline needs a CUDA device, got {self.device}")
        if depth < 1:
            raise ValueError("depth must be >= 1")
        self.depth = int(depth)
        self.copy_in = torch.cuda.Stream(self.device)
        self.compute = torch.cuda.Stream(self.device)
        self.copy_out = torch.cuda.Stream(self.device)
        self._inflight = collections.deque()
        self.h2d_bytes = 0      # running totals over all submitted calls
        self.d2h_bytes = 0
        self.launches = 0       # kernels launched by the library on behalf of this pipeline

    # -- host -> device -------------------------------------------------------------------------
    def _upload(self, tensors):
        """Copy host tensors to the device on the copy-in stream.  Views that share one base buffer
        (BT, BL, C cut out of the projection output) are copied once, as that buffer, and re-viewed
        on the device with the same strides, so the kernels still read them in place."""
        bases, out = {}, []
        for t in tensors:
            if t.is_cuda:
                raise RuntimeError("HostScanPipeline takes host tensors; use scan_fwd / scan_bwd for device tensors")
            base = t._base if (t._base is not None and not t.is_contiguous()) else None
            if base is None:
                src = t if t.is_contiguous() else t.contiguous()
                key = (src.data_ptr(), tuple(src.shape), src.dtype)
                if key not in bases:
                    bases[key] = src.to(self.device, non_blocking=True)
                    self.h2d_bytes += src.numel() * src.element_size()
                out.append(bases[key])
            else:
                src = base if base.is_contiguous() else base.contiguous()
                key = (src.data_ptr(), tuple(src.shape), src.dtype)
                if key not in bases:
                    bases[key] = src.to(self.device, non_blocking=True)
                    self.h2d_bytes += src.numel() * src.element_size()
                off = t.storage_offset() - base.storage_offset()
                out.append(bases[key].as_strided(t.shape, t.stride(), off))
        return out

    # -- submit ---------------------------------------------------------------------------------
    def submit(self, x, deltaT, deltaL, AT, AL, BT, BL, C, D, grad_output=None, reverse=False, out=None):
        """Queue one call.  All tensor arguments are host tensors (pinned memory lets the copies
        overlap; pageable memory works but copies synchronously).  With ``grad_output`` the backward
        runs too and the ticket carries the nine gradients.  ``out`` may hold the pinned buffers of
        an earlier, finished ticket (``ticket.outputs``) to write into instead of allocating new
        ones.  The host inputs must stay unchanged until the ticket is done."""
        while len(self._inflight) >= self.depth:
            self._inflight.popleft().wait()
        host = [x, deltaT, deltaL, AT, AL, BT, BL, C, D] + ([grad_output] if grad_output is not None else [])
        with torch.cuda.device(self.device):
            with torch.cuda.stream(self.copy_in):
                dev = self._upload(host)
                e_in = torch.cuda.Event()
                e_in.record(self.copy_in)
            with torch.cuda.stream(self.compute):
                self.compute.wait_event(e_in)
                args = dev[:9]
                res = [_wc.scan_fwd(*args, reverse=reverse)]
                self.launches += 1
                if grad_output is not None:
                    res += list(_wc.scan_bwd(*args, dev[9], reverse=reverse))
                    self.launches += 1 if x.dtype == torch.float32 else 2
                e_c = torch.cuda.Event()
                e_c.record(self.compute)
            if out is None:
                out = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True) for t in res]
            elif len(out) != len(res) or any(o.shape != t.shape or o.dtype != t.dtype for o, t in zip(out, res)):
                raise ValueError("out= buffers do not match the shapes and dtypes of this call's results")
            with torch.cuda.stream(self.copy_out):
                self.copy_out.wait_event(e_c)
                for o, t in zip(out, res):
                    o.copy_(t, non_blocking=True)
                    self.d2h_bytes += t.numel() * t.element_size()
                e_out = torch.cuda.Event()
                e_out.record(self.copy_out)
        ticket = ScanTicket(out[0], tuple(out[1:]) if grad_output is not None else None, e_out, (dev, res))
        self._inflight.append(ticket)
        return ticket

    def synchronize(self):
        """Block until every submitted call has finished."""
        while self._inflight:
            self._inflight.popleft().wait()
        self.copy_out.synchronize()
