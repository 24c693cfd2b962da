"""The CPU oracle against trajectories of the reference's own naive classes (no GPU needed).

The fixtures were produced by tests/golden/make_golden.py from the unmodified
reference code.  With ``variant="naive"`` the oracle must reproduce them; the
bound is an absolute one on parameter values after up to 50 steps, the same
quantity the reference's CUDA-vs-naive tests bound by 1e-5
(tests/test_celo2_cuda.py:95).
"""

import pytest
import torch

import golden_util as G

TOL = 5e-6


@pytest.mark.parametrize("name", sorted(G.CASES))
def test_oracle_reproduces_reference_naive(name):
    torch.set_num_threads(1)
    meta, weights, golden, _ = G.load(name)
    case = G.CASES[name]
    assert meta["hparams"] == case["hparams"], "fixture is stale: rerun tests/golden/make_golden.py"
    out = G.run(case, G.make_oracle(case, weights, variant="naive"))
    assert G.max_abs_diff(out, golden, case.get("sample_stride")) < TOL


def test_oracle_velo_side_state_matches_reference():
    meta, weights, golden, extra = G.load("velo_small")
    case = G.CASES["velo_small"]
    o = G.make_oracle(case, weights, variant="naive")
    G.run(case, o)
    h, c = o.lstm_hidden_state
    assert torch.allclose(h, torch.from_numpy(extra["lstm_h"]), atol=1e-6)
    assert torch.allclose(c, torch.from_numpy(extra["lstm_c"]), atol=1e-6)
    assert torch.allclose(o.loss_buffer.means, torch.from_numpy(extra["loss_means"]), atol=1e-7)


def test_cuda_variant_differs_where_the_reference_classes_differ():
    """AdafacLO/ELO: the CUDA class reduces row_col_mean over the decay axis; the distance to naive is visible."""
    meta, weights, golden, _ = G.load("elo_ref_clip0_exp0.001")
    case = G.CASES["elo_ref_clip0_exp0.001"]
    out = G.run(case, G.make_oracle(case, weights, variant="cuda"))
    d = G.max_abs_diff(out, golden)
    assert 1e-5 < d < 1e-3  # the reference's own CUDA-vs-naive bound for ELO is 1e-3 (tests/test_elo_cuda.py:92)


def test_decay_reparam_known_answer():
    from oracle import pylo_oracle as O

    bm = O.decay_reparam((0.9, 0.99, 0.999), (0.15216392, 0.14245212, 0.06812963))
    assert torch.allclose(bm, torch.tensor([0.5420273, 0.9584414, 0.9980236]), atol=2e-6)
    bf = O.decay_reparam((0.9, 0.99, 0.999), (0.18621896, -0.10864615, -0.06185547))
    assert torch.allclose(bf, torch.tensor([0.3562182, 0.9966259, 0.9994613]), atol=2e-6)
