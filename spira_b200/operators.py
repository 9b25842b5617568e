"""``cat`` for skip connections (reference: spira/operators.py:11-13)."""
from typing import List

import torch

from spira_b200.tensors import SparseTensor

__all__ = ["cat"]


def cat(inputs: List[SparseTensor]) -> SparseTensor:
    feats = torch.cat([x._features for x in inputs], dim=1)
    return SparseTensor(features=feats, coordinates=inputs[0]._coordinates, stride=inputs[0]._stride)
