from .conv import *
from .activations import *
from .normalizations import *
from . import functional
