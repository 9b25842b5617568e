"""``SparseTensor``: packed integer coordinates + features + stride.

Same constructor, attributes (``_coordinates``, ``_features``, ``_stride``, ``_double``) and methods as the
reference class (spira/tensors.py:10-65), so model code written against it runs unchanged.
"""
__all__ = ['SparseTensor']

from typing import Tuple, Union

import torch

from spira_b200.utils.helpers import as_tuple


class SparseTensor(object):

    def __init__(self, coordinates: torch.Tensor, features: torch.Tensor,
                 stride: Union[int, Tuple[int, ...]] = 1, double: bool = False):
        self._coordinates = coordinates
        self._features = features
        self._double = double
        self._stride = as_tuple(stride, size=3, name="strides")

    def cuda(self):
        self._coordinates = self._coordinates.cuda()
        self._features = self._features.cuda()
        return self

    def to(self, dtype):
        self._features = self._features.to(dtype=dtype)
        return self

    def contiguous(self):
        self._coordinates = self._coordinates.contiguous()
        self._features = self._features.contiguous()
        return self

    def half(self):
        self._features = self._features.half()
        return self

    def __add__(self, other):
        from spira_b200 import compile as _compile
        output = SparseTensor(coordinates=self._coordinates, features=self._features + other._features, stride=self._stride)
        if _compile._recorder is not None:
            _compile._recorder.add(self, other, output)
        return output

    def order(self):
        """Packs ``[N,3]`` coordinates into sorted keys and permutes the features accordingly
        (reference: spira/tensors.py:55-65)."""
        from spira_b200.nn.functional import _C
        keys, perm = _C.cuda_flatten_sort(self._coordinates.contiguous(), self._double)
        self._features = _C.permute_rows(self._features, perm)
        self._coordinates = keys
        return self
