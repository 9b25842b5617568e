from . import typing
from . import helpers
from . import apply
