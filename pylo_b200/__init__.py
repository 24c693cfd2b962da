"""pylo_b200: the learned-optimizer step of PyLO on hand-written sm_100a CUDA kernels."""

from . import _lib  # noqa: F401  (loads libpylo_b200.so; raises if it cannot)
from . import models, optim  # noqa: F401

__version__ = "0.1.0"
