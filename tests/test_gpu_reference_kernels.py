"""The reference's OWN CUDA kernels as the checker (skipped when ``oracle/_ref/`` holds no built modules).

``oracle/build_ref.py`` compiles the reference's three CUDA extensions for sm_100a; ``oracle/ref_cuda.py`` drives
them the way the reference's ``*_CUDA`` classes do.  Two things are bound here, on two-dimensional and
one-dimensional tensors (the shapes the reference's kernels index correctly, and the ones its own CUDA tests use):

* the CPU oracle in its ``variant="cuda"`` mode against the reference's kernels: this pins, by OUTPUT of the
  reference, the places where its CUDA classes differ from its naive classes (``row_col_mean`` over the decay
  axis in AdafacLO / ELO, ``safe_rsqrt(v + 1e-9)`` for one-dimensional tensors, VeLO's weight decay with the
  multiplied step size);
* the CUDA classes of this package against the reference's kernels, same bounds as against the oracle except
  that the movement bound allows for the reference's fast-math build (approximate exp / division / rsqrt and
  floating-point atomics: it is not bit-reproducible itself).
"""

import pytest
import torch

import cases
import cuda_util as CU
from test_gpu_config_sizes import HP, _make_pair, _nets

pytestmark = pytest.mark.gpu

# row/column-structured gradients make the decay-axis behaviour of AdafacLO / ELO visible (iid gradients nearly
# cancel it); the (40,) and (257,) tensors take the one-dimensional branch
SHAPES = [(96, 64), (64, 160), (300, 200), (40,), (257,)]
FAMILIES = ["adafaclo", "elo", "celo2", "elo_celo2", "velo"]
MOVE_TOL_VS_FAST_MATH = 5e-5   # observed: <= 1.6e-6


def _ref_cuda():
    from oracle import ref_cuda

    if not ref_cuda.available():
        pytest.skip("the reference's CUDA extensions are not built (python oracle/build_ref.py)")
    return ref_cuda


def _reference_stepper(family, shapes, hp, nets):
    from oracle import pylo_oracle as O

    R = _ref_cuda()
    dev = torch.device("cuda")
    if family in ("adafaclo", "elo"):
        return R.adafaclo(nets.flat_weights(), dev, elo=(family == "elo"), **hp)
    if family in ("celo2", "elo_celo2"):
        kw = dict(hp)
        if family == "elo_celo2":
            kw = dict(dict(clip_grad=True, adam_lr_mult=20.0), **kw)
        return R.celo2(nets.flat_weights(), dev, shared_adam=(family == "elo_celo2"), **kw)
    rnn, mlp = nets
    return R.velo(O.rnn_weights_from_module(rnn), O.bank_from_module(mlp), shapes, dev, **hp)


def _run(family, case, steps, hp):
    """{step: tensors} of the reference's CUDA path, the CPU oracle and this package's CUDA class."""
    nets = _nets(family, lstm_hidden=64)
    init = cases.init_values(case)
    ours = [torch.nn.Parameter(v.cuda()) for v in init]
    via_ref = [v.clone().cuda() for v in init]
    via_cpu = [v.clone() for v in init]
    opt, ora = _make_pair(family, case["shapes"], ours, hp, nets)
    ref = _reference_stepper(family, case["shapes"], hp, nets)
    for t in range(1, steps + 1):
        grads = cases.grads_at(case, t)
        for p, g in zip(ours, grads):
            p.grad = g.cuda()
        if family == "velo":
            loss = cases.velo_loss(t)
            opt.step(torch.tensor(loss, dtype=torch.float32, device="cuda"))
            ora.step(via_cpu, grads, loss)
            ref.step(via_ref, [g.cuda() for g in grads], loss)
        else:
            opt.step()
            ora.step(via_cpu, grads)
            ref.step(via_ref, [g.cuda() for g in grads])
    torch.cuda.synchronize()
    return ({steps: [p.detach().cpu() for p in ours]}, {steps: via_cpu}, {steps: [p.cpu() for p in via_ref]}, init)


@pytest.mark.parametrize("family", FAMILIES)
def test_oracle_and_library_match_the_reference_kernels(family):
    case = dict(shapes=SHAPES, init_seed=51, init_scale=0.05, grad_seed=52, grad_kind="rowlognormal", log_mu=-3.0)
    hp = dict(HP[family])
    if family == "velo":
        hp.update(lr=1.0, num_steps=200, weight_decay=0.01)   # weight decay on: it is one of the pinned differences
    elif family == "adafaclo":
        hp.update(lr=1e-2, weight_decay=0.05)
    else:
        hp.update(lr=1e-2)
    ours, cpu, ref, init = _run(family, case, 3, hp)
    for name, got in (("oracle", cpu), ("library", ours)):
        res = CU.compare(got, ref, init)
        upd = CU.compare_updates(got, ref, init)
        CU.log_parity(f"reference_kernels[{family},{name}]", rel=res[3][0], move=res[3][1], update=upd[3])
        assert res[3][0] < 1e-5, (name, res)
        assert res[3][1] < MOVE_TOL_VS_FAST_MATH, (name, res)


def test_reference_kernels_show_the_decay_axis_behaviour():
    """The check above would be empty if the pinned difference were invisible: with structured gradients the
    reference's CUDA kernels must differ visibly from the oracle's ``variant="naive"`` mode (the naive classes'
    meaning) while agreeing with ``variant="cuda"``."""
    from oracle import pylo_oracle as O

    R = _ref_cuda()
    case = dict(shapes=[(96, 64), (64, 160)], init_seed=51, init_scale=0.05, grad_seed=52, grad_kind="rowlognormal", log_mu=-3.0)
    net = _nets("adafaclo")
    init = cases.init_values(case)
    hp = dict(lr=1e-2, step_mult=0.01, exp_mult=0.001)
    ref = R.adafaclo(net.flat_weights(), torch.device("cuda"), **hp)
    as_cuda = O.AdafacLOOracle(net.flat_weights(), variant="cuda", **hp)
    as_naive = O.AdafacLOOracle(net.flat_weights(), variant="naive", **hp)
    p_ref, p_cuda, p_naive = [v.clone().cuda() for v in init], [v.clone() for v in init], [v.clone() for v in init]
    for t in (1, 2, 3):
        grads = cases.grads_at(case, t)
        ref.step(p_ref, [g.cuda() for g in grads])
        as_cuda.step(p_cuda, grads)
        as_naive.step(p_naive, grads)
    got = {3: [p.cpu() for p in p_ref]}
    near = CU.compare({3: p_cuda}, got, init)[3][1]
    far = CU.compare({3: p_naive}, got, init)[3][1]
    CU.log_parity("decay_axis_visibility", cuda_variant=near, naive_variant=far)
    assert near < MOVE_TOL_VS_FAST_MATH and far > 20 * MOVE_TOL_VS_FAST_MATH, (near, far)
