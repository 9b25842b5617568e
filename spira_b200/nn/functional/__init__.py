from . import _C
from .convolution import *
from .indexing import *
from .memory import *
