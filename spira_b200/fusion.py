"""Inference-time fusion: BatchNorm (eval), ReLU and residual adds that follow a ``SparseConv`` move into the
convolution kernel's epilogue.

The reference runs them as separate passes over the ``[T, C]`` activations (``spira/nn/normalizations.py:8-10``,
``spira/nn/activations.py:8-18``, ``scripts/models/spira/modules/blocks.py:81-84``).  ``fuse(model)`` rewrites, inside
every ``torch.nn.Sequential``, the pattern ``SparseConv -> BatchNorm [-> ReLU]`` (the layer must not be the 1x1x1
matrix-product case and the BatchNorm must be in eval mode) and leaves identity modules in their place, so the model's
structure and ``forward`` stay as they are.  Blocks that expose ``fuse_residual()`` (``spira_b200.models.ResBlock``)
additionally fold ``relu(main(x) + shortcut(x))`` into the last convolution of the main branch.
"""
from __future__ import annotations

import torch
from torch import nn

from spira_b200.nn.activations import ReLU
from spira_b200.nn.conv import SparseConv
from spira_b200.nn.normalizations import BatchNorm

__all__ = ["fuse", "bn_affine"]


def bn_affine(bn: nn.BatchNorm1d):
    """Eval-mode BatchNorm as ``y = x * scale + shift`` (fp32)."""
    var = bn.running_var.detach().float()
    mean = bn.running_mean.detach().float()
    gamma = bn.weight.detach().float() if bn.affine else torch.ones_like(var)
    beta = bn.bias.detach().float() if bn.affine else torch.zeros_like(var)
    scale = gamma / torch.sqrt(var + bn.eps)
    return scale, beta - mean * scale


def _fuse_sequential(seq: nn.Sequential) -> int:
    fused = 0
    mods = list(seq.named_children())
    i = 0
    while i < len(mods):
        name, m = mods[i]
        if isinstance(m, SparseConv) and m.is_trivial and m._folded is None and i + 1 < len(mods):
            bn_name, bn = mods[i + 1]
            if isinstance(bn, BatchNorm) and not bn.training and bn.track_running_stats:
                # a 1x1x1 stride-1 layer is a matrix product: the BatchNorm affine folds into its weight and bias
                scale, shift = bn_affine(bn)
                w = m.kernel.detach().view(m.in_channels, m.out_channels).float() * scale[None, :]
                b = shift if m.bias is None else m.bias.detach().float() * scale + shift
                m._folded = (w.to(m.kernel.dtype).contiguous(), b.to(m.kernel.dtype).contiguous())
                setattr(seq, bn_name, nn.Identity())
                fused += 1
                i += 2
                continue
        if isinstance(m, SparseConv) and not m.is_trivial and m._fused is None and i + 1 < len(mods):
            bn_name, bn = mods[i + 1]
            if isinstance(bn, BatchNorm) and not bn.training and bn.track_running_stats:
                scale, shift = bn_affine(bn)
                relu = False
                if i + 2 < len(mods) and type(mods[i + 2][1]) is ReLU:
                    relu = True
                    setattr(seq, mods[i + 2][0], nn.Identity())
                m.set_fused_epilogue(scale, shift, relu)
                setattr(seq, bn_name, nn.Identity())
                fused += 1
                i += 3 if relu else 2
                continue
        i += 1
    return fused


def fuse(model: nn.Module) -> nn.Module:
    """Fuses in place and returns ``model``; call it after ``model.eval()`` (and after ``.half()`` / ``.cuda()``)."""
    for mod in list(model.modules()):
        if isinstance(mod, nn.Sequential):
            _fuse_sequential(mod)
    for mod in list(model.modules()):
        if hasattr(mod, "fuse_residual"):
            mod.fuse_residual()
    return model
