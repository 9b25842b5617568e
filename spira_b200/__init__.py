"""spira_b200: a B200-native (sm_100a) sparse-convolution engine with the Python API of
SPIN-Research-Group/Spira (``SparseTensor``, ``nn.SparseConv``, ``nn.KernelMapCache``, ``tune``).

All computation goes through the C-ABI library ``libspira_b200.so`` (``include/spira_b200.h``); there is no
CPU or eager fallback.  ``install_as_spira()`` registers the package under the name ``spira`` so that model
definitions written against the reference (``from spira import SparseTensor, cat; import spira.nn as spnn``)
run unchanged.
"""
from .utils.helpers import set_kernel_map_cache
from .utils.helpers import tune
from .tensors import *
from . import nn
from . import utils
from .operators import *
from .compat import install_as_spira
from .fusion import fuse
from .compile import compile_model, CompiledModel
from . import batch

__version__ = "0.1.0"
