"""GPU checks of the tensor-core variant of the AdafacLO / ELO apply kernel (``mlp_precision="3xtf32"``, the default).

The two hidden layers run as tcgen05 products with every operand split into a high and a low TF32 part; the
results must stay inside the same bounds as the scalar-FMA path: 1e-5 relative per element after one step, 1e-4
after the whole trajectory, movement within 2e-5 of its largest entry against the oracle, and within 1e-5 of the
movement against the scalar-FMA path of the library itself at the full 4096 x 4096 size.
"""

import pytest
import torch

import cases
import cuda_util as CU
import golden_util as G

pytestmark = pytest.mark.gpu

PRECISIONS = ["3xtf32"]
MOVE_TOL = 2e-5
ADAFAC_CASES = sorted(n for n, c in G.CASES.items() if c["family"] in ("adafaclo", "elo"))


def _net():
    from pylo_b200 import models

    torch.manual_seed(0)
    return models.MetaMLP(39, 32, 1)


def _make(family, params, **kw):
    from pylo_b200 import optim

    if family == "adafaclo":
        return optim.AdafacLO_CUDA(params, lr=1e-2, network=_net(), **kw)
    return optim.ELO_CUDA(params, lr=1e-2, weight_decay=0.1, clip_grad=True, network=_net(), **kw)


@pytest.mark.parametrize("prec", PRECISIONS)
@pytest.mark.parametrize("name", ADAFAC_CASES)
def test_tensor_core_path_matches_oracle(name, prec):
    meta, weights, golden, _ = G.load(name)
    case = G.CASES[name]
    ref = G.run(case, G.make_oracle(case, weights, variant="cuda"))
    got, opt, _ = CU.run_cuda(case, weights, mlp_precision=prec)
    opt.check_status()
    assert any(plan.tensor_cores and plan.n_ctiles for _, plan in opt._plans.values()), "no tensor took the tensor-core kernel"
    res = CU.compare(got, ref, cases.init_values(case))
    first, last = min(res), max(res)
    assert res[first][0] < 1e-5, res
    assert res[last][0] < 1e-4, res
    assert all(r[1] < MOVE_TOL for r in res.values()), res


@pytest.mark.parametrize("name", ADAFAC_CASES)
def test_scalar_fma_path_matches_oracle(name):
    """The CUDA-core path (``mlp_precision="fp32"``) is no longer the default, so it is pinned here."""
    meta, weights, golden, _ = G.load(name)
    case = G.CASES[name]
    ref = G.run(case, G.make_oracle(case, weights, variant="cuda"))
    got, opt, _ = CU.run_cuda(case, weights, mlp_precision="fp32")
    assert not any(plan.tensor_cores for _, plan in opt._plans.values())
    res = CU.compare(got, ref, cases.init_values(case))
    first, last = min(res), max(res)
    assert res[first][0] < 1e-5 and res[last][0] < 1e-4 and all(r[1] < MOVE_TOL for r in res.values()), res


# two-dimensional shapes that are factored (both sides >= 32) with ragged edges: columns that do not fill a
# block of 128, fewer rows than one work item, a single block; plus tensors that stay on the generic kernel
TC_RAGGED = [(257, 129), (129, 300), (64, 128), (33, 37), (40, 4100), (300, 1000), (7,), (5, 3)]


@pytest.mark.parametrize("prec", PRECISIONS)
@pytest.mark.parametrize("family", ["adafaclo", "elo"])
def test_tensor_core_ragged_shapes_match_oracle(family, prec):
    from oracle import pylo_oracle as O

    case = dict(name="tc_ragged", family=family, shapes=TC_RAGGED, net_seed=0, init_seed=5, init_scale=0.1, grad_seed=6,
                grad_scale=0.3, steps=3, record=[1, 3], hparams={})
    params = [torch.nn.Parameter(v.cuda()) for v in cases.init_values(case)]
    opt = _make(family, params, mlp_precision=prec)
    kw = dict(lr=1e-2, elo=(family == "elo"))
    if family == "elo":
        kw.update(weight_decay=0.1, clip_grad=True)
    ora = O.AdafacLOOracle(_net().flat_weights(), **kw)
    ref = [v.clone() for v in cases.init_values(case)]
    init = [v.clone() for v in ref]
    for t in (1, 2, 3):
        grads = cases.grads_at(case, t)
        for p, g in zip(params, grads):
            p.grad = g.cuda()
        opt.step()
        ora.step(ref, grads)
    opt.check_status()
    res = CU.compare({3: [p.detach().cpu() for p in params]}, {3: ref}, init)
    CU.log_parity(f"tc_ragged[{family},{prec}]", rel=res[3][0], move=res[3][1])
    assert res[3][0] < 1e-5 and res[3][1] < MOVE_TOL, res


@pytest.mark.parametrize("prec", PRECISIONS)
@pytest.mark.parametrize("family,extra", [("adafaclo", {}), ("adafaclo", {"weight_decay": 0.1}), ("elo", {})])
def test_tensor_core_and_fma_paths_agree_at_full_size(family, extra, prec):
    """4096 x 4096 and a 4096 x 1000 tensor (ragged last column block): the update through the tensor cores must
    equal the scalar-FMA one to 1e-5 of the largest movement (a few ulp of the parameter are discounted)."""
    shapes = [(4096, 4096), (4096, 1000)]
    outs, init = {}, None
    for which in ("fp32", prec):
        gen = torch.Generator(device="cuda").manual_seed(3)
        ps = [torch.nn.Parameter(torch.randn(*s, device="cuda", generator=gen) * 0.02) for s in shapes]
        init = [p.detach().clone() for p in ps]
        rows = [torch.exp(-7 + torch.randn(s[0], 1, device="cuda", generator=gen)) for s in shapes]
        opt = _make(family, ps, mlp_precision=which, **extra)
        for t in (1, 2):
            g = torch.Generator(device="cuda").manual_seed(100 + t)
            for p, r in zip(ps, rows):
                p.grad = torch.randn(*p.shape, device="cuda", generator=g) * r
            opt.step()
        opt.check_status()
        outs[which] = [p.detach().clone() for p in ps]
    for a, b, w0 in zip(outs["fp32"], outs[prec], init):
        moved = (a - w0).abs().max()
        assert moved > 0
        err = torch.clamp((a - b).abs() - 4 * 1.2e-7 * a.abs(), min=0).max()
        assert float(err / moved) < 1e-5, float(err / moved)
        assert torch.allclose(a, b, rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("prec", PRECISIONS)
def test_tensor_core_path_is_bit_reproducible(prec):
    outs = []
    for _ in range(2):
        gen = torch.Generator(device="cuda").manual_seed(3)
        p = torch.nn.Parameter(torch.randn(2048, 4096, device="cuda", generator=gen) * 0.02)
        opt = _make("adafaclo", [p], mlp_precision=prec)
        for _ in range(2):
            p.grad = torch.randn(2048, 4096, device="cuda", generator=gen) * 1e-3
            opt.step()
        opt.check_status()
        outs.append(p.detach().clone())
    assert torch.equal(outs[0], outs[1])


def test_unknown_mlp_precision_is_rejected():
    p = torch.nn.Parameter(torch.zeros(64, 64, device="cuda"))
    with pytest.raises(ValueError):
        _make("adafaclo", [p], mlp_precision="bf16")


@pytest.mark.parametrize("prec", PRECISIONS)
def test_reported_timeout_keeps_parameters_and_is_raised(prec):
    """The kernel ORs 1 into a device word when one of its bounded waits runs out, and a launch that finds the
    word set stores nothing.  Here the word is set from the host (no GPU misbehaviour involved): the launch must
    leave the parameters exactly as they were, check_status() must raise, a later step must raise by itself
    before it touches any state, and clear_status() must bring the optimizer back."""
    from pylo_b200 import _lib as L

    gen = torch.Generator(device="cuda").manual_seed(3)
    p = torch.nn.Parameter(torch.randn(256, 256, device="cuda", generator=gen) * 0.02)
    opt = _make("adafaclo", [p], mlp_precision=prec)
    p.grad = torch.randn(256, 256, device="cuda", generator=gen) * 1e-3
    opt.step()
    opt.check_status()
    plan = list(opt._plans.values())[0][1]
    plan.status[0] = 1
    with pytest.raises(L.PyloLibError):
        opt.check_status()
    before = p.detach().clone()
    opt.step()                 # this launch finds the word set; a copy of the word to pinned memory follows it
    torch.cuda.synchronize()
    assert torch.equal(p.detach(), before), "a launch that found the status word set must not write parameters"
    m_before = opt.state[p]["exp_avg"].clone()
    with pytest.raises(L.PyloLibError):
        opt.step()             # ... which this step looks at before its first kernel
    torch.cuda.synchronize()
    assert torch.equal(opt.state[p]["exp_avg"], m_before), "the refused step must not have touched the state"
    opt.clear_status()
    opt.step()
    opt.check_status()
    assert not torch.equal(p.detach(), before)
