"""Network definitions for the benchmark workloads, written against the public layer API only
(``SparseConv``, ``BatchNorm``, ``ReLU``, ``cat``) -- the same building blocks the reference's model zoo uses
(``scripts/models/spira/sparse_unet.py``, ``scripts/models/spira/modules/blocks.py``).

``map_schedule(...)`` returns the argument lists of ``KernelMapCache.add_all_kernel_maps`` for a network with
``n_down`` stride-2 levels, in the alternating order the builder expects (submanifold map of level i, then the
down-sampling map i -> i+1; ``scripts/end_to_end_experiment.py:107-112``).
"""
from __future__ import annotations

from typing import List, Sequence

import torch
from torch import nn

import spira_b200 as sp
from spira_b200 import nn as spnn

__all__ = ["SparseUNet", "SparseBackbone", "minkunet18", "indoor_resunet", "second_backbone", "map_schedule"]


def _conv_bn_relu(cin, cout, k, stride=1, transposed=False):
    return nn.Sequential(spnn.SparseConv(cin, cout, k, stride=stride, transposed=transposed), spnn.BatchNorm(cout), spnn.ReLU(True))


class ResBlock(nn.Module):
    """``relu(main(x) + shortcut(x))`` with ``main = conv-bn-relu-conv-bn`` (the reference's ``SparseResBlock``,
    scripts/models/spira/modules/blocks.py:51-84)."""

    def __init__(self, cin: int, cout: int, k: int = 3):
        super().__init__()
        self.main = nn.Sequential(spnn.SparseConv(cin, cout, k), spnn.BatchNorm(cout), spnn.ReLU(True),
                                  spnn.SparseConv(cout, cout, k), spnn.BatchNorm(cout))
        self.shortcut = nn.Identity() if cin == cout else nn.Sequential(spnn.SparseConv(cin, cout, 1), spnn.BatchNorm(cout))
        self.relu = spnn.ReLU(True)
        self._residual_fused = False

    def fuse_residual(self):
        """After ``spira_b200.fuse``: the add and the final ReLU run in the epilogue of the last main convolution."""
        last = self.main[3]
        if isinstance(last, spnn.SparseConv) and last._fused is not None and isinstance(self.main[4], nn.Identity):
            last._fused["relu"] = True
            self._residual_fused = True

    def forward(self, x):
        if self._residual_fused:
            s = self.shortcut(x)
            h = self.main[2](self.main[1](self.main[0](x)))
            return self.main[3](h, residual=s._features)
        return self.relu(self.main(x) + self.shortcut(x))


class SparseUNet(nn.Module):
    """Residual encoder-decoder: stem, ``len(enc)`` stride-2 stages, as many transposed up-sampling stages with
    skip concatenation, and a 1x1x1 classification head."""

    def __init__(self, in_channels: int, stem: int, enc: Sequence[int], dec: Sequence[int], num_classes: int,
                 kernel: int = 3, resample_kernel: int = 3):
        super().__init__()
        assert len(enc) == len(dec)
        self.n_down = len(enc)
        self.stem = nn.Sequential(_conv_bn_relu(in_channels, stem, kernel), _conv_bn_relu(stem, stem, kernel))
        widths = [stem] + list(enc)
        self.encoders = nn.ModuleList()
        for i in range(len(enc)):
            self.encoders.append(nn.Sequential(_conv_bn_relu(widths[i], widths[i], resample_kernel, stride=2),
                                               ResBlock(widths[i], widths[i + 1], kernel), ResBlock(widths[i + 1], widths[i + 1], kernel)))
        self.ups = nn.ModuleList()
        self.fuses = nn.ModuleList()
        cur = widths[-1]
        for i, d in enumerate(dec):
            skip = widths[len(enc) - 1 - i]
            self.ups.append(_conv_bn_relu(cur, d, resample_kernel, stride=2, transposed=True))
            self.fuses.append(nn.Sequential(ResBlock(d + skip, d, kernel), ResBlock(d, d, kernel)))
            cur = d
        self.head = spnn.SparseConv(cur, num_classes, 1, bias=True)

    def forward(self, x):
        skips = [self.stem(x)]
        for e in self.encoders:
            skips.append(e(skips[-1]))
        y = skips.pop()
        for up, fuse in zip(self.ups, self.fuses):
            y = fuse(sp.cat([up(y), skips.pop()]))
        return self.head(y)


class SparseBackbone(nn.Module):
    """SECOND-style 3D backbone: submanifold blocks separated by stride-2 down-sampling convolutions."""

    def __init__(self, in_channels: int, widths: Sequence[int], kernel: int = 3):
        super().__init__()
        self.n_down = len(widths) - 1
        layers: List[nn.Module] = [_conv_bn_relu(in_channels, widths[0], kernel), _conv_bn_relu(widths[0], widths[0], kernel)]
        for i in range(1, len(widths)):
            layers += [_conv_bn_relu(widths[i - 1], widths[i], kernel, stride=2),
                       _conv_bn_relu(widths[i], widths[i], kernel), _conv_bn_relu(widths[i], widths[i], kernel)]
        self.layers = nn.Sequential(*layers)

    def forward(self, x):
        return self.layers(x)


def minkunet18(in_channels: int = 4, num_classes: int = 19, resample_kernel: int = 3) -> SparseUNet:
    """MinkUNet18-style network: widths 32 | 32-64-128-256 | 256-128-96-96, 3^3 kernels everywhere."""
    return SparseUNet(in_channels, 32, [32, 64, 128, 256], [256, 128, 96, 96], num_classes, 3, resample_kernel)


def indoor_resunet(in_channels: int = 3, num_classes: int = 20) -> SparseUNet:
    """SparseResUNet-style indoor network: widths 32-64-128-256 down, mirrored up."""
    return SparseUNet(in_channels, 32, [64, 128, 256], [128, 64, 32], num_classes, 3, 3)


def second_backbone(in_channels: int = 5) -> SparseBackbone:
    return SparseBackbone(in_channels, [16, 32, 64, 128], 3)


def map_schedule(n_down: int, kernel: int = 3, resample_kernel: int = 3):
    """(kernel_sizes, source_strides, target_strides) for ``add_all_kernel_maps`` with ``init_stride = 1``."""
    kernel_sizes, source_strides, target_strides = [], [(1, 1, 1)], []
    s = 1
    for level in range(n_down + 1):
        kernel_sizes.append((kernel,) * 3)
        source_strides.append((s,) * 3)
        if level < n_down:
            kernel_sizes.append((resample_kernel,) * 3)
            s *= 2
            source_strides.append((s,) * 3)
            target_strides.append((s,) * 3)
    return kernel_sizes, source_strides, target_strides
