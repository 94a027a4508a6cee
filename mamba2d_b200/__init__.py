"""B200 (sm_100a) implementation of Mamba2D's wavefront 2-D selective scan.

``mamba2d_b200.wavefront_cuda`` mirrors the reference module ``models/kernels/wavefront_cuda.py``;
``mamba2d_b200.inject`` makes the reference's unchanged model code import it;
``mamba2d_b200.host_pipeline`` runs the same kernels on host-resident tensors with the PCIe copies
overlapped.
"""
from .host_pipeline import HostScanPipeline, ScanTicket  # noqa: F401
from .wavefront_cuda import (proj_params, scan_bwd, scan_fwd, wavefront_scan_cuda, wf_cuda_fn_fr,  # noqa: F401
                             wf_cuda_fn_pr)

__all__ = ["wavefront_scan_cuda", "wf_cuda_fn_pr", "wf_cuda_fn_fr", "proj_params", "scan_fwd", "scan_bwd",
           "HostScanPipeline", "ScanTicket"]
