"""Seeded inputs and hyper-parameters of the golden cases.

Shared by ``make_golden.py`` (which runs the reference on them) and by the
tests (which run the oracle and the CUDA classes on the same inputs).  Inputs
come from ``torch.Generator`` on the CPU, which is deterministic for a given
torch build, so only outputs are stored in the ``.npz`` fixtures.

The first CELO2 / ELO cases take their shapes, seeds, scales, step counts and
hyper-parameters from the reference's own CUDA-vs-naive tests
(tests/test_celo2_cuda.py:38-128, tests/test_elo_cuda.py:36-109).
"""

import math

import torch

REF_SHAPES = [(64, 32), (32, 64), (32,)]


def _gen(seed):
    return torch.Generator().manual_seed(seed)


def init_values(case):
    g = _gen(case["init_seed"])
    scale = case.get("init_scale", 1.0)
    return [torch.randn(s, generator=g) * scale for s in case["shapes"]]


def grads_at(case, t):
    """Gradients of step ``t`` (1-based); independent of earlier calls."""
    g = _gen(case["grad_seed"] * 100003 + t)
    kind = case.get("grad_kind", "iid")
    scale = case.get("grad_scale", 1.0)
    out = []
    for s in case["shapes"]:
        x = torch.randn(s, generator=g) * scale
        if kind == "rowlognormal" and len(s) >= 2:
            row = torch.exp(case.get("log_mu", 0.0) + torch.randn((s[0],) + (1,) * (len(s) - 1), generator=g))
            x = x * row
        elif kind == "outliers":
            mask = torch.rand(s, generator=g) < 0.01
            x = torch.where(mask, x * 100.0, x)
        out.append(x)
    return out


def velo_loss(t):
    return 2.0 * math.exp(-t / 50.0) + 0.1


_CELO2_REF = dict(lr=1e-2, weight_decay=0.1, clip_grad=True, clip_norm=1.0)

CELO2_CASES = [
    # tests/test_celo2_cuda.py:72-95, the four parametrisations
    dict(name=f"celo2_ref_orth{int(o)}_exp{e}", family="celo2", shapes=REF_SHAPES, net_seed=0, init_seed=1,
         grad_seed=2, grad_scale=3.0, steps=50, record=[1, 10, 50],
         hparams=dict(_CELO2_REF, orthogonalize=o, exp_mult=e))
    for o in (True, False) for e in (0.0, 0.01)
] + [
    # tests/test_celo2_cuda.py:98-111
    dict(name="elo_celo2_ref", family="elo_celo2", shapes=REF_SHAPES, net_seed=0, init_seed=3, grad_seed=4,
         grad_scale=3.0, steps=50, record=[1, 10, 50], hparams=dict(lr=1e-3)),
    # tests/test_celo2_cuda.py:114-128
    dict(name="celo2_single_matrix", family="celo2", shapes=[(48, 24)], net_seed=0, init_seed=7, grad_seed=8,
         grad_scale=2.0, steps=50, record=[1, 10, 50], hparams=dict(lr=1e-2, orthogonalize=True)),
    # beyond the reference tests: structured gradients, odd sizes, 3-D/4-D tensors, an embedding group
    dict(name="celo2_structured", family="celo2", shapes=[(40, 96), (33, 7), (5, 6, 8), (12, 3, 4, 4), (17,)],
         net_seed=5, init_seed=11, init_scale=0.02, grad_seed=12, grad_kind="rowlognormal", log_mu=-7.0,
         steps=12, record=[1, 3, 12],
         hparams=dict(lr=1e-3, weight_decay=0.1, orthogonalize=True, exp_mult=0.01, clip_grad=False)),
    dict(name="elo_celo2_embedding", family="elo_celo2", shapes=[(50, 16), (16, 24), (24,)],
         is_embedding=[True, False, False], net_seed=6, init_seed=13, init_scale=0.02, grad_seed=14,
         grad_scale=1e-3, steps=8, record=[1, 8], hparams=dict(lr=1e-3, adam_lr_mult=20.0)),
]

_MLP_SHAPES = [(128, 784), (128,), (128, 128), (128,), (10, 128), (10,)]

ADAFAC_CASES = [
    # the CPU-runnable benchmark configuration: 784-128-128-10 MLP, 10 steps, lr 1e-3
    dict(name="adafaclo_mlp", family="adafaclo", shapes=_MLP_SHAPES, net_seed=0, init_seed=1, init_scale=0.05,
         grad_seed=2, grad_scale=1e-3, steps=10, record=[1, 10], sample_stride=29,
         hparams=dict(lr=1e-3, step_mult=0.01, exp_mult=0.001)),
    dict(name="adafaclo_small", family="adafaclo", shapes=[(64, 32), (32, 64), (32,), (6, 5, 4)], net_seed=3,
         init_seed=21, grad_seed=22, grad_kind="rowlognormal", log_mu=-3.0, steps=12, record=[1, 3, 12],
         hparams=dict(lr=1e-2, step_mult=0.01, exp_mult=0.001, weight_decay=0.05)),
] + [
    # tests/test_elo_cuda.py:72-92
    dict(name=f"elo_ref_clip{int(c)}_exp{e}", family="elo", shapes=REF_SHAPES, net_seed=0, init_seed=1, grad_seed=2,
         grad_scale=3.0, steps=50, record=[1, 10, 50],
         hparams=dict(lr=1e-2, exp_mult=e, weight_decay=0.1, clip_grad=c, clip_norm=1.0))
    for c in (False, True) for e in (0.001, 0.01)
]

VELO_CASES = [
    dict(name="velo_small", family="velo", shapes=[(48, 32), (32, 32), (16, 40), (32,), (3, 8, 8)], net_seed=4,
         lstm_hidden=64, bank_scale=0.05, init_seed=31, init_scale=0.02, grad_seed=32, grad_kind="outliers",
         grad_scale=1e-3, steps=12, record=[1, 3, 12], hparams=dict(lr=1.0, num_steps=200, weight_decay=0.01)),
]

ALL_CASES = CELO2_CASES + ADAFAC_CASES + VELO_CASES
