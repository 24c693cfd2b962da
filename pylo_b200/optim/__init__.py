"""Optimizer classes with the reference's names (pylo/optim/__init__.py:21-76).

Only the CUDA classes exist here; importing this package fails loudly when the
CUDA library cannot be loaded, and there are no naive fallbacks behind the
aliases.
"""

from .AdafacLO_cuda import AdafacLO_CUDA, ELO_CUDA
from .CELO2_cuda import CELO2_CUDA, ELO_CELO2_CUDA
from .MuLO_cuda import MuLO_CUDA
from .velo_cuda import VeLO_CUDA

AdafacLO = AdafacLO_CUDA
ELO = ELO_CUDA
CELO2 = CELO2_CUDA
ELO_CELO2 = ELO_CELO2_CUDA
VeLO = VeLO_CUDA
MuLO = MuLO_CUDA

__all__ = ["AdafacLO_CUDA", "ELO_CUDA", "CELO2_CUDA", "ELO_CELO2_CUDA", "VeLO_CUDA", "MuLO_CUDA", "VeLO", "AdafacLO", "ELO", "CELO2",
           "ELO_CELO2", "MuLO"]
