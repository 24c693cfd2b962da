"""ELO_CUDA shares its kernels with AdafacLO_CUDA; re-exported under the reference's module name."""

from .AdafacLO_cuda import ELO_CUDA

__all__ = ["ELO_CUDA"]
