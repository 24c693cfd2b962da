"""GPU checks beyond the golden trajectories: resume format, ragged shapes, full-size properties.

At the full benchmark size (4096 x 4096) the oracle would take minutes per family, so the checks there
are size-independent properties: two different code paths of the library (the float4 path and the
scalar generic path, selected by the alignment of the tensors) must agree, and repeated runs must be
bit-identical.
"""

import copy

import pytest
import torch

import cases
import cuda_util as CU
import golden_util as G

pytestmark = pytest.mark.gpu


def _nets(family):
    from pylo_b200 import models

    torch.manual_seed(0)
    if family in ("adafaclo", "elo"):
        return models.MetaMLP(39, 32, 1)
    if family in ("celo2", "elo_celo2"):
        return models.CELO2MLP()
    rnn, mlp = models.VeLORNN(lstm_hidden_size=32), models.VeLOMLP()
    with torch.no_grad():
        for name, p in mlp.named_parameters():
            if name.endswith("_") or "_." in name:
                p.mul_(0.05)
    return rnn, mlp


def _make(family, params, **kw):
    from pylo_b200 import optim

    if family == "adafaclo":
        return optim.AdafacLO_CUDA(params, lr=1e-2, network=_nets(family), **kw)
    if family == "elo":
        return optim.ELO_CUDA(params, lr=1e-2, weight_decay=0.1, clip_grad=True, network=_nets(family), **kw)
    if family == "celo2":
        return optim.CELO2_CUDA(params, lr=1e-2, weight_decay=0.1, clip_grad=True, network=_nets(family), **kw)
    if family == "elo_celo2":
        return optim.ELO_CELO2_CUDA(params, lr=1e-2, network=_nets(family), **kw)
    rnn, mlp = _nets(family)
    return optim.VeLO_CUDA(params, lr=kw.pop("lr", 1.0), num_steps=100, rnn=rnn, mlp=mlp, **kw)


def _step(opt, family, t):
    if family == "velo":
        opt.step(torch.tensor(cases.velo_loss(t), device="cuda"))
    else:
        opt.step()


FAMILIES = ["adafaclo", "elo", "celo2", "elo_celo2", "velo"]
# AdafacLO / ELO have two apply kernels for factored 2-D tensors: tensor cores (the default) and CUDA cores
VARIANTS = [(f, {}) for f in FAMILIES] + [("adafaclo", {"mlp_precision": "fp32"}), ("elo", {"mlp_precision": "fp32"})]
VARIANT_IDS = [f + ("-" + kw["mlp_precision"] if kw else "") for f, kw in VARIANTS]
RAGGED = [(33, 7), (1, 5), (5, 1), (17, 36), (3, 3, 3), (1,), (7,), (257, 129), (2, 4100), (70, 100), (33, 260)]


@pytest.mark.parametrize("family,extra", VARIANTS, ids=VARIANT_IDS)
def test_ragged_shapes_match_oracle(family, extra):
    """Sizes that are not multiples of 4 / 32 / 256, single rows and columns, one-element vectors."""
    case = dict(name="ragged", family=family, shapes=RAGGED, net_seed=0, init_seed=5, init_scale=0.1, grad_seed=6,
                grad_scale=0.3, steps=3, record=[1, 3], hparams={})
    dev = "cuda"
    params = [torch.nn.Parameter(v.to(dev)) for v in cases.init_values(case)]
    opt = _make(family, params, **extra)
    from oracle import pylo_oracle as O

    net = _nets(family)
    if family in ("adafaclo", "elo"):
        kw = dict(lr=1e-2, elo=(family == "elo"))
        if family == "elo":
            kw.update(weight_decay=0.1, clip_grad=True)
        ora = O.AdafacLOOracle(net.flat_weights(), **kw)
    elif family in ("celo2", "elo_celo2"):
        kw = dict(lr=1e-2, shared_adam=(family == "elo_celo2"))
        kw.update(dict(weight_decay=0.1, clip_grad=True) if family == "celo2" else dict(weight_decay=0.1, clip_grad=True, adam_lr_mult=20.0))
        ora = O.CELO2Oracle(net.flat_weights(), **kw)
    else:
        rnn, mlp = net
        ora = O.VeLOOracle(O.rnn_weights_from_module(rnn), O.bank_from_module(mlp), RAGGED, lr=1.0, num_steps=100)
    ref = [v.clone() for v in cases.init_values(case)]
    init = [v.clone() for v in ref]
    for t in (1, 2, 3):
        grads = cases.grads_at(case, t)
        for p, g in zip(params, grads):
            p.grad = g.to(dev)
        _step(opt, family, t)
        if family == "velo":
            ora.step(ref, grads, cases.velo_loss(t))
        else:
            ora.step(ref, grads)
    got = {3: [p.detach().cpu() for p in params]}
    res = CU.compare(got, {3: ref}, init)
    CU.log_parity(f"ragged[{family}]", rel=res[3][0], move=res[3][1])
    assert res[3][0] < 1e-5 and res[3][1] < 2e-5, res


@pytest.mark.parametrize("family,extra", VARIANTS, ids=VARIANT_IDS)
def test_resume_from_state_dict_continues_identically(family, extra):
    """Save after 3 steps, load into a fresh optimizer, continue: same parameters as the uninterrupted run
    (the contract of the reference's tests/test_optimizer_resume.py:134-164)."""
    shapes = [(40, 24), (24, 40), (24,)]
    case = dict(shapes=shapes, init_seed=9, grad_seed=10, grad_scale=0.5)

    def fresh():
        ps = [torch.nn.Parameter(v.cuda()) for v in cases.init_values(case)]
        return ps, _make(family, ps, **extra)

    pa, oa = fresh()
    for t in range(1, 7):
        for p, g in zip(pa, cases.grads_at(case, t)):
            p.grad = g.cuda()
        _step(oa, family, t)
        if t == 3:
            saved = copy.deepcopy(oa.state_dict())
            saved_p = [p.detach().clone() for p in pa]
    pb, ob = fresh()
    with torch.no_grad():
        for p, v in zip(pb, saved_p):
            p.copy_(v)
    ob.load_state_dict(saved)
    for t in range(4, 7):
        for p, g in zip(pb, cases.grads_at(case, t)):
            p.grad = g.cuda()
        _step(ob, family, t)
    for a, b in zip(pa, pb):
        assert torch.allclose(a, b, rtol=1e-6, atol=1e-7)


def test_state_keys_and_shapes_are_the_reference_format():
    shape = (12, 20)
    p = [torch.nn.Parameter(torch.randn(shape, device="cuda")), torch.nn.Parameter(torch.randn(20, device="cuda"))]
    for q in p:
        q.grad = torch.randn_like(q)
    opt = _make("adafaclo", p)
    opt.step()
    st = opt.state[p[0]]
    assert st["step"].dtype == torch.float64 and st["step"].device.type == "cpu" and float(st["step"]) == 1.0
    assert tuple(st["exp_avg"].shape) == (3,) + shape and tuple(st["exp_avg_sq"].shape) == shape
    assert tuple(st["exp_avg_sq_r"].shape) == (3, 12, 1) and tuple(st["exp_avg_sq_c"].shape) == (3, 1, 20)
    assert tuple(opt.state[p[1]]["exp_avg_sq_r"].shape) == (3, 20)
    opt = _make("celo2", p)
    opt.step()
    st = opt.state[p[0]]
    assert tuple(st["mom"].shape) == (3,) + shape and tuple(st["fac_r"].shape) == (3, 12, 1)
    assert set(opt.state[p[1]]) == {"exp_avg", "exp_avg_sq", "adam_step"}
    opt = _make("velo", p)
    opt.step(torch.tensor(1.0, device="cuda"))
    st = opt.state[p[0]]
    assert tuple(st["rms"].shape) == (1,) + shape and tuple(st["fac_vec_row"].shape) == (3, 12, 1)
    assert st["fac_vec_v"].numel() == 0 and tuple(opt.state[p[1]]["fac_vec_v"].shape) == (3, 20)
    sd = opt.state_dict()
    assert {"loss_buffer", "lstm_hidden_state", "num_steps"} <= set(sd)


@pytest.mark.parametrize("family", ["adafaclo", "celo2", "velo"])
def test_full_size_float4_and_generic_paths_agree(family):
    """4096 x 4096 (the single-tensor benchmark size): the same values once 16-byte aligned (float4 path)
    and once shifted by one float (scalar generic path) must give the same update."""
    n = 4096
    gen = torch.Generator(device="cuda").manual_seed(3)
    w0 = torch.randn(n, n, device="cuda", generator=gen) * 0.02
    row = torch.exp(-7 + torch.randn(n, 1, device="cuda", generator=gen))
    outs = []
    for shift in (0, 1):
        buf = torch.empty(n * n + 4, device="cuda")
        view = buf[shift:shift + n * n].view(n, n)
        view.copy_(w0)
        p = torch.nn.Parameter(view)
        kw = {"orthogonalize": False} if family == "celo2" else ({"lr": 1e3} if family == "velo" else {})
        opt = _make(family, [p], **kw)
        for t in (1, 2):
            g = torch.Generator(device="cuda").manual_seed(100 + t)
            p.grad = torch.randn(n, n, device="cuda", generator=g) * row
            _step(opt, family, t)
        outs.append(p.detach().clone())
        del opt
    a, b = outs
    moved = (a - w0).abs().max()
    assert moved > 0
    err = torch.clamp((a - b).abs() - 4 * 1.2e-7 * a.abs(), min=0).max()
    assert float(err / moved) < 1e-3
    assert torch.allclose(a, b, rtol=1e-5, atol=1e-7)


def test_full_size_is_bit_reproducible():
    n = 4096
    outs = []
    for _ in range(2):
        gen = torch.Generator(device="cuda").manual_seed(3)
        p = torch.nn.Parameter(torch.randn(n, n, device="cuda", generator=gen) * 0.02)
        opt = _make("adafaclo", [p])
        p.grad = torch.randn(n, n, device="cuda", generator=gen) * 1e-3
        opt.step()
        outs.append(p.detach().clone())
    assert torch.equal(outs[0], outs[1])


def test_celo2_with_3xtf32_newton_schulz_stays_within_the_reference_bound():
    meta, weights, golden, _ = G.load("celo2_ref_orth1_exp0.0")
    case = dict(G.CASES["celo2_ref_orth1_exp0.0"])
    case["hparams"] = dict(case["hparams"], ns_precision="3xtf32")
    got, opt, _ = CU.run_cuda(case, weights)
    opt.check_status()
    assert G.max_abs_diff(got, golden) < 1e-5   # the bound of tests/test_celo2_cuda.py:95


def test_elo_celo2_group_step_advances_without_gradients():
    """ELO_CELO2_cuda.py:215-216 advances ``group['step']`` for every group on every step, before it looks at the
    gradients; a group that has none on some step must therefore keep counting (its AdamW bias corrections and
    the ``step`` a checkpoint carries depend on it)."""
    a = torch.nn.Parameter(torch.randn(40, 24, device="cuda") * 0.02)
    b = torch.nn.Parameter(torch.randn(24, device="cuda") * 0.02)
    opt = _make("elo_celo2", [{"params": [a]}, {"params": [b]}])
    for t in (1, 2, 3):
        a.grad = torch.randn_like(a) * 1e-3
        b.grad = None if t == 2 else torch.randn_like(b) * 1e-3
        opt.step()
    assert [g["step"] for g in opt.param_groups] == [3, 3]
    assert opt.state_dict()["param_groups"][1]["step"] == 3


def test_mulo_cuda_equals_adafaclo_with_the_scaled_groups():
    """MuLO_CUDA only regroups (MuLO_cuda.py:32-61): stepping it must give what AdafacLO_CUDA gives over groups whose
    learning rates were divided by the width multipliers by hand."""
    from pylo_b200 import optim

    class Inf:
        def __init__(self, n, w):
            self.n, self.w = n, w

        def ninf(self):
            return self.n

        def width_mult(self):
            return self.w

    case = dict(shapes=[(48, 64), (64, 32), (64,)], init_seed=15, init_scale=0.05, grad_seed=16, grad_scale=0.2)
    mults = [(2, 4.0), (2, 2.0), (1, 1.0)]

    def params():
        ps = [torch.nn.Parameter(v.cuda()) for v in cases.init_values(case)]
        for p, (n, w) in zip(ps, mults):
            p.infshape = Inf(n, w)
        return ps

    pa, pb = params(), params()
    mulo = optim.MuLO_CUDA(pa, lr=1e-2, network=_nets("adafaclo"), momentum_dtype="bfloat16")
    by_hand = optim.AdafacLO_CUDA([{"params": [pb[0]], "lr": 1e-2 / 4.0}, {"params": [pb[1]], "lr": 1e-2 / 2.0},
                                   {"params": [pb[2]], "lr": 1e-2}], lr=1e-2, network=_nets("adafaclo"))
    for t in (1, 2):
        for a, b, g in zip(pa, pb, cases.grads_at(case, t)):
            a.grad, b.grad = g.cuda(), g.cuda()
        mulo.step()
        by_hand.step()
    for a, b, v in zip(pa, pb, cases.init_values(case)):
        assert torch.equal(a, b) and not torch.equal(a.detach().cpu(), v)
    # the momentum stays fp32 whatever momentum_dtype says, as in the reference class (AdafacLO_cuda.py:256,364-373)
    assert mulo.state[pa[0]]["exp_avg"].dtype == torch.float32
    assert mulo.defaults["momentum_dtype"] == torch.bfloat16
