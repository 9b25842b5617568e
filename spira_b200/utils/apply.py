"""``fapply``: run a feature-wise torch function on a SparseTensor (reference: spira/utils/apply.py:10-19)."""
from typing import Callable

import torch

__all__ = ["fapply"]


def fapply(input, fn: Callable[..., torch.Tensor], *args, **kwargs):
    from spira_b200.tensors import SparseTensor
    from spira_b200 import compile as _compile
    output = SparseTensor(coordinates=input._coordinates, features=fn(input._features, *args, **kwargs), stride=input._stride)
    if _compile._recorder is not None:
        _compile._recorder.apply(fn, args, kwargs, input, output)
    return output
