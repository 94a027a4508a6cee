"""Build the reference project's own, unchanged model classes on top of this package's scan.

The scan is one operator inside ``M2DBlock.ssm`` (models/mamba2d.py:180-202); its callers are
``M2DBlock.forward`` (:157-178), ``ResBlock`` (:205-261) and ``Mamba2DBackbone`` (:263-386), and the
classifier wraps the backbone as ``head(norm(backbone(x).mean([-2, -1])))``
(models/mamba2d_classifier.py:62-69).  None of that code lives in this repository: this module
imports it from a checkout of the reference (``reference_root()``), after ``inject.install`` has
made its ``from .kernels.wavefront_cuda import wavefront_scan_cuda`` resolve to this package.

The classifier here is a plain ``nn.Module`` with the reference's forward; the reference's own class
is a Lightning module and needs packages (lightning, torchmetrics, timm.loss) that are not part of
the scan's path.  The optimiser grouping is the reference's (models/mamba2d_classifier.py:73-99), and
``train_step`` is one optimiser step of the training configuration (forward + backward + AdamW, with
the weight-gradient all-reduce of DistributedDataParallel when the model is wrapped in it).
"""
import contextlib
import importlib
import os
import sys

import torch
import torch.nn as nn

from . import inject

_REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Architecture arguments of the shipped configs (configs/M2D-T-ImageNet.yaml:94-101,
# configs/M2D-S-ImageNet.yaml:94-101, :112).
ARCH = {
    "M2D-T": dict(n_blocks=[3, 3, 9, 3], embed_dim=[64, 128, 320, 512], drop_path_rate=0.175, head_dropout=0.0),
    "M2D-S": dict(n_blocks=[3, 12, 14, 3], embed_dim=[96, 192, 384, 576], drop_path_rate=0.4, head_dropout=0.4),
}


def reference_root():
    """Directory that holds the reference's ``models/`` package: ``$M2D_REFERENCE_ROOT``, else the
    unmodified copy the build step places under ``baseline/_ref`` (git-ignored), else None."""
    for cand in (os.environ.get("M2D_REFERENCE_ROOT"), os.path.join(_REPO, "baseline", "_ref"), "/root/reference"):
        if cand and os.path.exists(os.path.join(cand, "models", "mamba2d.py")):
            return cand
    return None


def purge_models_modules():
    """Forget every imported ``models.*`` module, so that the package can be imported again with a
    different scan behind it."""
    for k in [k for k in sys.modules if k == "models" or k.startswith("models.")]:
        del sys.modules[k]


def import_reference_models(root=None, native_corner=False, fuse_act2=False):
    """``(models.mamba2d, models.utils)`` of the reference with this package's scan injected.

    With ``native_corner`` the block class scans bottom-right blocks in place instead of flipping
    the activation around them (``inject.native_scan_corner``); ``fuse_act2`` also folds the GELU
    after the scan into the scan's store where no gradient is needed."""
    root = root or reference_root()
    if root is None:
        raise RuntimeError("no reference checkout found: set M2D_REFERENCE_ROOT or run __graft_entry__.build() "
                           "where the reference is present")
    purge_models_modules()
    inject.install_droppath_shim()
    inject.install(root)
    m = importlib.import_module("models.mamba2d")
    u = importlib.import_module("models.utils")
    if native_corner or fuse_act2:
        inject.native_scan_corner(m.M2DBlock, fuse_act2=fuse_act2)
    return m, u


class Classifier(nn.Module):
    """backbone -> global average pool -> LayerNorm -> head (models/mamba2d_classifier.py:62-69)."""

    def __init__(self, backbone, head):
        super().__init__()
        self.backbone, self.head = backbone, head
        self.norm = nn.LayerNorm(backbone.embed_dim[-1])
        if backbone.channel_last:
            self.to(memory_format=torch.channels_last)

    def forward(self, x):
        x = self.backbone(x)
        return self.head(self.norm(x.mean([-2, -1])))


def build_classifier(arch="M2D-T", modules=None, n_classes=1000, recomp="partial"):
    """The shipped architecture ``arch`` with random initial weights, built from the reference's classes."""
    m, u = modules or import_reference_models()
    cfg = ARCH[arch]
    backbone = m.Mamba2DBackbone(in_channels=3, channel_last=True, n_blocks=cfg["n_blocks"],
                                 ds_stages=["mf_stem", "mf_2", "mf_2", "mf_2"], embed_dim=cfg["embed_dim"],
                                 token_mixer=["2D_local", "2D_local", "RopeAttention", "RopeAttention"],
                                 drop_path_rate=cfg["drop_path_rate"], res_scale_init_values=[1.0, 1.0, 1.0, 1.0],
                                 inter_flip=True, recomp=recomp)
    head = u.MlpHead(dim=cfg["embed_dim"][3], n_classes=n_classes, head_dropout=cfg["head_dropout"])
    return Classifier(backbone, head)


def param_groups(model, weight_decay=0.05):
    """The reference's AdamW grouping: no decay for parameters flagged ``_no_weight_decay`` (the scan's
    A_log and D) and for anything one-dimensional (models/mamba2d_classifier.py:73-99)."""
    decay, no_decay = [], []
    for p in model.parameters():
        if not p.requires_grad:
            continue
        (no_decay if getattr(p, "_no_weight_decay", False) or p.dim() < 2 else decay).append(p)
    return [{"params": decay, "weight_decay": weight_decay}, {"params": no_decay, "weight_decay": 0.0}]


def make_optimizer(model, lr=0.004, weight_decay=0.05):
    """AdamW as the reference configures it (models/mamba2d_classifier.py:92-97)."""
    return torch.optim.AdamW(param_groups(model, weight_decay), lr=lr, betas=(0.9, 0.999), eps=1e-8)


def train_step(model, optimizer, images, labels, micro_batch, autocast_dtype=torch.bfloat16):
    """One optimiser step on this rank's share of the global batch: forward + backward over
    micro-batches (gradients accumulate; under DistributedDataParallel only the last micro-batch
    triggers the weight-gradient all-reduce), then AdamW.  Cross-entropy on hard labels, mean over the
    rank's whole share.  Returns the loss (a detached scalar tensor)."""
    n = images.shape[0]
    chunks = [(s, min(s + micro_batch, n)) for s in range(0, n, micro_batch)]
    optimizer.zero_grad(set_to_none=True)
    total = None
    ddp = isinstance(model, torch.nn.parallel.DistributedDataParallel)
    use_autocast = autocast_dtype is not None and images.is_cuda
    for k, (s, e) in enumerate(chunks):
        last = k == len(chunks) - 1
        sync = contextlib.nullcontext() if (last or not ddp) else model.no_sync()
        with sync:
            with torch.autocast("cuda", dtype=autocast_dtype, enabled=use_autocast):
                logits = model(images[s:e])
            loss = torch.nn.functional.cross_entropy(logits.float(), labels[s:e], reduction="sum") / n
            loss.backward()
        total = loss.detach() if total is None else total + loss.detach()
    optimizer.step()
    return total
