"""Pieces shared by the optimizer classes: factored-dims rules, Newton-Schulz, plan caching."""

from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import numpy as np
import torch

from .. import _lib as L
from ..plan import DeviceTable, make_tiles


def factored_dims_sorted(shape):
    """(dc, dr): indices of the second-largest and largest axis, ties broken by index
    (AdafacLO_cuda.py:52-73 with min_dim_size_to_factor=1, ELO_cuda.py:46-51)."""
    if len(shape) < 2:
        return None
    order = sorted((s, i) for i, s in enumerate(shape))
    return int(order[-2][1]), int(order[-1][1])


def factored_dims_argsort(shape):
    """(dc, dr) via ``np.argsort`` (CELO2_naive.py:42-47)."""
    if len(shape) < 2:
        return None
    order = np.argsort(shape)
    return int(order[-2]), int(order[-1])


def factored_dims_velo(shape):
    """(dc, dr) with VeLO's tie rule: equal sizes swap unless 4-D with axes (0, 1) (velo_cuda.py:121-131)."""
    if len(shape) < 2:
        return None
    order = np.argsort(shape)
    a, b = int(order[-2]), int(order[-1])
    if shape[a] == shape[b] and not (len(shape) == 4 and a == 0 and b == 1):
        return b, a
    return a, b


def newton_schulz(x: torch.Tensor, coeffs, iters: int = 5, eps: float = 1e-8) -> torch.Tensor:
    """Quintic Newton-Schulz iteration towards the orthogonal factor of ``x`` over its last two axes.

    Same arithmetic, in the same order, as CELO2_naive.py:59-73: work on the wide
    orientation, divide by (Frobenius norm + eps), then ``iters`` times
    ``a = x x^T; b = c1 a + c2 a a; x = c0 x + b x``.  It is a chain of dense fp32
    GEMMs and stays on ``torch.matmul``.
    """
    tall = x.shape[-2] > x.shape[-1]
    if tall:
        x = x.transpose(-2, -1)
    x = x / (torch.linalg.norm(x, dim=(-2, -1), keepdim=True) + eps)
    c0, c1, c2 = coeffs
    for _ in range(iters):
        a = x @ x.transpose(-2, -1)
        b = c1 * a + c2 * (a @ a)
        x = c0 * x + b @ x
    return x.transpose(-2, -1) if tall else x


def _split_tf32(x: torch.Tensor):
    """x = hi + lo (+ a remainder below 2^-22 |x|): hi is x rounded to nearest TF32 (10 mantissa bits), lo
    the exact difference rounded to TF32 as well, so that the tensor core's own truncation of its inputs
    loses nothing."""
    def to_tf32(t):
        return ((t.view(torch.int32) + 0x1000) & -8192).view(torch.float32)

    hi = to_tf32(x)
    return hi, to_tf32(x - hi)


def _mm_3xtf32(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a @ b from three TF32 tensor-core products, a_hi b_hi + (a_hi b_lo + a_lo b_hi).

    The dropped term a_lo b_lo is ~2^-22 of the result, so the product carries fp32-like accuracy while
    running on the tensor cores; the GEMMs themselves are the library's (cuBLAS through torch.matmul).
    """
    ah, al = _split_tf32(a)
    bh, bl = _split_tf32(b)
    return ah @ bh + (ah @ bl + al @ bh)


def newton_schulz_3xtf32(x: torch.Tensor, coeffs, iters: int = 5, eps: float = 1e-8) -> torch.Tensor:
    """:func:`newton_schulz` with every matrix product evaluated by :func:`_mm_3xtf32`.

    Optional (``ns_precision="3xtf32"``) and off by default: it is not the reference's arithmetic.  Measured
    against an fp64 evaluation its result is ~3e-5 off in relative Frobenius norm where the fp32 products
    are ~4e-6 off (the TF32 units accumulate less exactly); on a 4096 x 4096 matrix it is 2.7x faster.
    """
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        tall = x.shape[-2] > x.shape[-1]
        if tall:
            x = x.transpose(-2, -1)
        x = x / (torch.linalg.norm(x, dim=(-2, -1), keepdim=True) + eps)
        c0, c1, c2 = coeffs
        for _ in range(iters):
            a = _mm_3xtf32(x, x.transpose(-2, -1).contiguous())
            b = c1 * a + c2 * _mm_3xtf32(a, a)
            x = c0 * x + _mm_3xtf32(b, x)
        return x.transpose(-2, -1) if tall else x
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def require_cuda_param(p: torch.Tensor, who: str):
    if not p.is_cuda:
        raise RuntimeError(f"{who}: parameters must live on a CUDA device (there is no CPU path)")
    if p.dtype != torch.float32:
        raise RuntimeError(f"{who}: only fp32 parameters are supported, got {p.dtype}")
    if not p.is_contiguous():
        raise RuntimeError(f"{who}: parameters must be contiguous")


class ItemPlan:
    """Tile list + item table for the simple element-wise kernels (AdamW, CELO2 tail)."""

    def __init__(self, dtype, sizes: Sequence[int], device):
        self.items = np.zeros(len(sizes), dtype=dtype)
        self.items["n"] = sizes
        tiles, ranges = make_tiles(sizes)
        if "tile0" in dtype.names:
            for i, (t0, k) in enumerate(ranges):
                self.items["tile0"][i], self.items["n_tiles"][i] = t0, k
        self.ranges = ranges
        self.tiles = DeviceTable(tiles, device)
        self.n_tiles = len(tiles)
        self.table = DeviceTable(self.items, device)

    def upload(self):
        self.table.upload()
