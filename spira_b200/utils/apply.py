"""``fapply``: run a feature-wise torch function on a SparseTensor (reference: spira/utils/apply.py:10-19)."""
from typing import Callable

import torch

__all__ = ["fapply"]


def fapply(input, fn: Callable[..., torch.Tensor], *args, **kwargs):
    from spira_b200.tensors import SparseTensor
    return SparseTensor(coordinates=input._coordinates, features=fn(input._features, *args, **kwargs), stride=input._stride)
