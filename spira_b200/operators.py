"""``cat`` for skip connections (reference: spira/operators.py:11-13)."""
from typing import List

import torch

from spira_b200.tensors import SparseTensor

__all__ = ["cat"]


def cat(inputs: List[SparseTensor]) -> SparseTensor:
    from spira_b200 import compile as _compile
    feats = torch.cat([x._features for x in inputs], dim=1)
    output = SparseTensor(features=feats, coordinates=inputs[0]._coordinates, stride=inputs[0]._stride)
    if _compile._recorder is not None:
        _compile._recorder.cat(inputs, output)
    return output
