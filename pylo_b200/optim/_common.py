"""Pieces shared by the optimizer classes: factored-dims rules, Newton-Schulz, plan caching."""

from __future__ import annotations

import ctypes as C_
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


def _gemm_tn(A, B, C, D, alpha, beta, status, stream, symmetric=False):
    """C[b] = alpha * A[b] @ B[b]^T + beta * D[b] through ``pylo_b200_gemm_tn_3xtf32`` (3-D fp32 tensors whose last axis is
    contiguous).  ``symmetric``: the result is known to be symmetric; only the tiles on and above the diagonal are
    computed and the rest is filled in by mirroring."""
    g = L.GemmDesc()
    g.A, g.B, g.C, g.D = A.data_ptr(), B.data_ptr(), C.data_ptr(), (D.data_ptr() if D is not None else None)
    g.batch, g.M, g.K = A.shape
    g.N = B.shape[1]
    g.lda, g.ldb, g.ldc, g.ldd = A.stride(1), B.stride(1), C.stride(1), (D.stride(1) if D is not None else 0)
    g.strideA, g.strideB, g.strideC = A.stride(0), B.stride(0), C.stride(0)
    g.strideD = D.stride(0) if D is not None else 0
    g.alpha, g.beta = float(alpha), float(beta)
    g.symmetric = int(bool(symmetric))
    L.check(L.lib.pylo_b200_gemm_tn_3xtf32(C_.byref(g), status.data_ptr() if status is not None else None, stream),
            "gemm_tn_3xtf32")
    if symmetric:
        L.check(L.lib.pylo_b200_transpose(C.data_ptr(), C.data_ptr(), g.M, g.N, g.ldc, g.ldc, g.strideC, g.strideC, g.batch, 1,
                                          stream), "transpose(mirror)")


def _transpose(src, dst, stream):
    """dst[b] = src[b]^T for 3-D fp32 tensors whose last axis is contiguous."""
    nb, r, c = src.shape
    L.check(L.lib.pylo_b200_transpose(src.data_ptr(), dst.data_ptr(), r, c, src.stride(1), dst.stride(1), src.stride(0),
                                      dst.stride(0), nb, 0, stream), "transpose")


def newton_schulz_eligible(rows: int, cols: int) -> bool:
    """Whether :func:`newton_schulz_tc` takes a matrix of this shape (else it goes to ``torch.matmul``): both sides
    multiples of 4 (rows are moved in 16-byte pieces) and the short side at least 64 (the kernel's tiles have 128
    rows; below half a tile the library product is the better tool)."""
    r, c = min(rows, cols), max(rows, cols)
    return r % 4 == 0 and c % 4 == 0 and r >= 64


def newton_schulz_tc(x: torch.Tensor, coeffs, iters: int = 5, eps: float = 1e-8, status=None, stream=None) -> torch.Tensor:
    """:func:`newton_schulz` with the three products of every round on the tensor cores.

    Same chain as CELO2_naive.py:59-73.  Each product is one launch of the library's own batched kernel
    (``pylo_b200_gemm_tn_3xtf32``: operands split into TF32 high and low parts inside the kernel, three tcgen05
    products accumulated in fp32, the scaled additions ``c1 a + c2 (a a)`` and ``c0 x + (b x)`` as its epilogue),
    which needs both operands with the contraction index contiguous; x^T is therefore kept beside x and refreshed
    once per round.  Not bit-identical to the fp32 products of ``torch.matmul`` (neither are two builds of cuBLAS);
    against an fp64 evaluation it is as close as they are.
    """
    shape = x.shape
    x = x.reshape((-1,) + tuple(shape[-2:]))
    tall = x.shape[-2] > x.shape[-1]
    if tall:
        x = x.transpose(-2, -1)
    x = (x / (torch.linalg.norm(x, dim=(-2, -1), keepdim=True) + eps)).contiguous()
    n_b, r, c = x.shape
    if stream is None:
        stream = torch.cuda.current_stream().cuda_stream
    c0, c1, c2 = (float(v) for v in coeffs)
    xt = torch.empty((n_b, c, r), dtype=torch.float32, device=x.device)
    a = torch.empty((n_b, r, r), dtype=torch.float32, device=x.device)
    b = torch.empty_like(a)
    x_next = torch.empty_like(x)
    for it in range(iters):
        _transpose(x, xt, stream)
        _gemm_tn(x, x, a, None, 1.0, 0.0, status, stream, symmetric=True)     # a = x x^T
        _gemm_tn(a, a, b, a, c2, c1, status, stream, symmetric=True)          # b = c1 a + c2 a a   (a is symmetric)
        _gemm_tn(b, xt, x_next, x, 1.0, c0, status, stream)                   # x = c0 x + b x
        x, x_next = x_next, x
    if tall:
        x = x.transpose(-2, -1)
    return x.reshape(shape)


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
