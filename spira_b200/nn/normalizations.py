"""BatchNorm over SparseTensor features (reference: spira/nn/normalizations.py:8-10)."""
__all__ = ['BatchNorm']

import torch

from spira_b200.utils.apply import fapply


class BatchNorm(torch.nn.BatchNorm1d):
    def forward(self, input):
        return fapply(input, super().forward)
