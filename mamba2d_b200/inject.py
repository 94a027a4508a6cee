"""Make the reference project's unchanged model code call this package's scan.

The reference's ``models/mamba2d.py`` does ``from .kernels.wavefront_cuda import wavefront_scan_cuda``
(models/mamba2d.py:10) and its downstream copy does the same relative import
(downstream/Mamba2D/mamba2d.py:13).  Importing that module normally JIT-builds the reference's CUDA
extension.  ``install()`` pre-registers this package's ``wavefront_cuda`` under the module names
those imports resolve to, so the reference files load unmodified and ``M2DBlock.ssm`` reaches the
B200 kernels.

    import mamba2d_b200.inject as inject
    inject.install("/path/to/Mamba2D")          # adds the checkout to sys.path
    from models.mamba2d import Mamba2DBackbone
"""
import importlib
import sys
import types

from . import wavefront_cuda

TARGETS = ("models.kernels.wavefront_cuda", "Mamba2D.kernels.wavefront_cuda", "kernels.wavefront_cuda")


def _ensure_package(name, path=None):
    if name in sys.modules:
        return sys.modules[name]
    mod = types.ModuleType(name)
    mod.__path__ = [path] if path else []
    sys.modules[name] = mod
    return mod


def install(reference_root=None, extra_targets=()):
    """Register the replacement under every module path the reference imports it by.

    ``reference_root`` (optional) is put on ``sys.path`` so ``import models.mamba2d`` finds the
    reference checkout.  Returns the list of module names that now resolve to this package."""
    import os
    if reference_root and reference_root not in sys.path:
        sys.path.insert(0, reference_root)
    done = []
    for target in tuple(TARGETS) + tuple(extra_targets):
        parts = target.split(".")
        # the ``kernels`` sub-package must exist as a package object for the relative import
        if reference_root:
            kdir = os.path.join(reference_root, *parts[:-1]) if parts[0] != "Mamba2D" else \
                os.path.join(reference_root, "downstream", *parts[:-1])
        else:
            kdir = None
        if len(parts) > 2:
            try:
                importlib.import_module(parts[0])
            except Exception:
                _ensure_package(parts[0])
        _ensure_package(".".join(parts[:-1]), kdir)
        sys.modules[target] = wavefront_cuda
        done.append(target)
    return done


def install_droppath_shim():
    """``models/mamba2d.py`` imports ``timm.layers.DropPath``.  Where timm is not installed, provide
    a minimal stand-in (stochastic depth; identity in eval mode) so the backbone can be built."""
    try:
        import timm.layers  # noqa: F401
        return False
    except Exception:
        pass
    import torch
    import torch.nn as nn

    class DropPath(nn.Module):
        def __init__(self, drop_prob: float = 0.0, scale_by_keep: bool = True):
            super().__init__()
            self.drop_prob, self.scale_by_keep = drop_prob, scale_by_keep

        def forward(self, x):
            if self.drop_prob == 0.0 or not self.training:
                return x
            keep = 1 - self.drop_prob
            mask = x.new_empty((x.shape[0],) + (1,) * (x.ndim - 1)).bernoulli_(keep)
            if keep > 0.0 and self.scale_by_keep:
                mask.div_(keep)
            return x * mask

    timm = types.ModuleType("timm")
    layers = types.ModuleType("timm.layers")
    layers.DropPath = DropPath
    timm.layers = layers
    sys.modules.setdefault("timm", timm)
    sys.modules.setdefault("timm.layers", layers)
    return True


def native_scan_corner(block_cls, fuse_act2=False):
    """Optional: make the reference's ``M2DBlock`` scan from its start corner in place.

    The reference block obtains ``scan_start == "BR"`` by flipping the activation on the way in and
    the result on the way out (models/mamba2d.py:162-175); everything between those two flips other
    than the scan acts per pixel, and the local path is taken before the first flip and added after
    the second.  This replaces ``forward`` and ``ssm`` of the given class with versions that never
    flip and pass ``scan_start`` to the scan instead, which is the same function of the input with
    two full-activation copies less per odd block (and their two copies in backward).  The
    ``double_scans`` branch keeps the reference's arithmetic: its second scan runs on the flipped
    input and its result is averaged in as it comes, without being flipped back
    (models/mamba2d.py:190-200).

    With ``fuse_act2`` the GELU the block applies to the scan's output (``act2``,
    models/mamba2d.py:169) is requested from the scan itself (``act_out="gelu"``), which folds it
    into the kernel's store whenever no gradient is needed; ``double_scans`` blocks keep the separate
    activation, because it acts on the average of two scans.

    Returns the class.  Call it after ``install()`` and after importing the model module:

        from models.mamba2d import M2DBlock
        inject.native_scan_corner(M2DBlock)
    """
    scan = wavefront_cuda.wavefront_scan_cuda

    def ssm(self, x, act_out=None):
        corner = getattr(self, "scan_start", "TL")
        extra = {} if act_out is None else {"act_out": act_out}
        y = scan(x, self.AT_log, self.AL_log, self.x_proj.weight, self.dt_projT.weight, self.dt_projT.bias,
                 self.dt_projL.weight, self.dt_projL.bias, self.D, self.recomp, scan_start=corner, **extra)
        if self.double_scans:
            other = "TL" if corner == "BR" else "BR"
            y_b = scan(x, self.AT_log_b, self.AL_log_b, self.x_proj_b.weight, self.dt_projT_b.weight,
                       self.dt_projT_b.bias, self.dt_projL_b.weight, self.dt_projL_b.bias, self.D_b, self.recomp,
                       scan_start=other)
            y = (y + y_b.flip(1, 2)) / 2
        return y

    def forward(self, x):
        local = self.local_path(self.local_norm(x)) if self.local_path else None
        gelu2 = fuse_act2 and not self.double_scans and type(self.act2).__name__ == "GELU" \
            and getattr(self.act2, "approximate", "none") == "none"
        if gelu2:
            x = self.out_proj(self.ssm(self.act1(self.in_proj(x)), act_out="gelu"))
        else:
            x = self.out_proj(self.act2(self.ssm(self.act1(self.in_proj(x)))))
        return x if local is None else x + local

    block_cls.ssm = ssm
    block_cls.forward = forward
    return block_cls
