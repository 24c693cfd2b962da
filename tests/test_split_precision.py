"""CPU emulation of the operand split the tensor-core kernels use.

The kernels feed the tensor cores TF32 operands (11 significant bits) and recover fp32 fidelity by splitting every
operand into a high and a low part and accumulating three products per layer (lo x hi, hi x lo, hi x hi) in fp32.
This file restates the split with integer masks and checks, against fp64, that a 32-term dot product comes out
within a few 1e-7 of the sum of its terms' magnitudes - the same order as a plain fp32 FMA chain - and that a
single 11-bit product does not (so the test can tell the difference).
"""

import numpy as np
import pytest


def tf32_trunc(x: np.ndarray) -> np.ndarray:
    """What a TF32 operand keeps of an fp32 value: sign, exponent, 10 explicit mantissa bits."""
    return (x.astype(np.float32).view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32)


def split_tf32(x):
    hi = tf32_trunc(x)
    lo = tf32_trunc((x - hi).astype(np.float32))  # x - hi is exact in fp32; the tensor core then drops its low bits
    return hi, lo


def three_products(a, b, split):
    """sum_k a[m,k] b[n,k] with fp32 accumulation of lo x hi, hi x lo, hi x hi (in that order)."""
    ah, al = split(a)
    bh, bl = split(b)
    acc = np.zeros((a.shape[0], b.shape[0]), dtype=np.float32)
    for x, y in ((al, bh), (ah, bl), (ah, bh)):
        for k in range(a.shape[1]):  # products of 11-bit operands are exact in fp32; the sum rounds like fp32
            acc = (acc + np.outer(x[:, k], y[:, k]).astype(np.float32)).astype(np.float32)
    return acc


@pytest.mark.parametrize("name,split,scale", [("tf32", split_tf32, 1e-4), ("tf32", split_tf32, 1.0)])
def test_three_split_products_are_fp32_faithful(name, split, scale):
    rng = np.random.default_rng(0)
    a = (rng.standard_normal((128, 32)) * 3.0 * scale).astype(np.float32)
    b = (rng.uniform(-0.5, 0.5, (32, 32))).astype(np.float32)
    exact = a.astype(np.float64) @ b.astype(np.float64).T
    mag = np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64).T
    got = three_products(a, b, split)
    err = np.max(np.abs(got - exact) / mag)
    chain = np.zeros_like(got)
    for k in range(32):
        chain = (chain + np.outer(a[:, k], b[:, k]).astype(np.float32)).astype(np.float32)
    err_fp32 = np.max(np.abs(chain - exact) / mag)
    assert err < 1e-6, (name, err)
    assert err < 8 * max(err_fp32, 6e-8), (name, err, err_fp32)
    single = np.max(np.abs(split(a)[0].astype(np.float64) @ split(b)[0].astype(np.float64).T - exact) / mag)
    assert single > 1e-5  # one 11-bit product alone is three orders worse: the split is what buys the accuracy
