"""Parameter-shape lists of the benchmark configurations and seeded synthetic tensors for them.

Only *shapes* of public architectures are used (the optimizer's cost and
arithmetic depend on shapes, gradient values and meta-weights, not on what the
tensors mean); parameters, gradients and meta-weights are seeded random draws.
"""

from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import torch

Shape = Tuple[int, ...]


def mlp_784() -> List[Shape]:
    return [(128, 784), (128,), (128, 128), (128,), (10, 128), (10,)]


def celo2_4096() -> List[Shape]:
    return [(4096, 4096), (4096,)]


def vit_b16() -> List[Shape]:
    d, ff = 768, 3072
    s: List[Shape] = [(d, 3, 16, 16), (d,), (197, d), (d,)]  # patch embed w/b, positions, class token
    for _ in range(12):
        s += [(d,), (d,), (d, 3 * d), (3 * d,), (d, d), (d,), (d,), (d,), (d, ff), (ff,), (ff, d), (d,)]
    s += [(d,), (d,), (d, 1000), (1000,)]
    return s


def gpt2_medium() -> List[Shape]:
    d, ff, vocab, ctx = 1024, 4096, 50257, 1024
    s: List[Shape] = [(vocab, d), (ctx, d)]
    for _ in range(24):
        s += [(d,), (d,), (d, 3 * d), (3 * d,), (d, d), (d,), (d,), (d,), (d, ff), (ff,), (ff, d), (d,)]
    s += [(d,), (d,)]
    return s


def llama3_8b(layers: int = 32) -> List[Shape]:
    d, ff, kv, vocab = 4096, 14336, 1024, 128256
    s: List[Shape] = [(vocab, d)]
    for _ in range(layers):
        s += [(d, d), (kv, d), (kv, d), (d, d), (ff, d), (ff, d), (d, ff), (d,), (d,)]
    s += [(d,), (vocab, d)]
    return s


def llama3_block() -> List[Shape]:
    """One transformer block of Llama-3-8B (218 M params): a small multi-tensor case for kernel comparisons."""
    return llama3_8b(1)[1:-2]


WORKLOADS = {
    "llama3_block": llama3_block,
    "mlp_784": mlp_784,
    "celo2_4096": celo2_4096,
    "vit_b16": vit_b16,
    "gpt2_medium": gpt2_medium,
    "llama3_8b": llama3_8b,
}


def numel(shape: Shape) -> int:
    n = 1
    for d in shape:
        n *= d
    return n


def total_params(shapes: Sequence[Shape]) -> int:
    return sum(numel(s) for s in shapes)


def make_grad_pool(shapes: Sequence[Shape], scale: float, device, seed: int = 2, kind: str = "iid") -> Dict[Shape, torch.Tensor]:
    """One seeded gradient buffer per distinct shape (tensors of equal shape share it)."""
    gen = torch.Generator(device=device).manual_seed(seed)
    pool: Dict[Shape, torch.Tensor] = {}
    for s in shapes:
        if s in pool:
            continue
        g = torch.randn(s, generator=gen, device=device, dtype=torch.float32) * scale
        if kind == "outliers":  # 1 % of the entries times 100
            mask = torch.rand(s, generator=gen, device=device) < 0.01
            g = torch.where(mask, g * 100.0, g)
        elif kind == "rowlognormal" and len(s) >= 2:
            row = torch.exp(-7.0 + torch.randn((s[0],) + (1,) * (len(s) - 1), generator=gen, device=device))
            g = g / scale * row
        pool[s] = g
    return pool
