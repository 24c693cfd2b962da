"""ELO_CELO2_CUDA lives beside CELO2_CUDA (they share every kernel); re-exported under the reference's module name."""

from .CELO2_cuda import ELO_CELO2_CUDA

__all__ = ["ELO_CELO2_CUDA"]
