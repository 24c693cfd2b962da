"""Kernel-level known answers: accumulator states and per-feature second moments after one step.

The trajectory tests bind the final parameters; these bind what the kernels leave behind on the way:
the momentum / second-moment / factored accumulators (the resume format) and the per-feature sums of
squares that the reference kernels accumulate with atomics (learned_optimizer.cu:100-190,
celo2_kernel.cu:130-199, velo_kernel.cu:170-256), against the CPU oracle.
"""

import pytest
import torch

import cases
import golden_util as G
from test_gpu_properties import _make, _nets, _step

pytestmark = pytest.mark.gpu

SHAPES = [(48, 40), (40, 48), (36, 36), (6, 10, 12), (40,)]


def _oracle(family):
    from oracle import pylo_oracle as O

    net = _nets(family)
    if family == "adafaclo":
        return O.AdafacLOOracle(net.flat_weights(), lr=1e-2)
    if family == "celo2":
        return O.CELO2Oracle(net.flat_weights(), lr=1e-2, weight_decay=0.1, clip_grad=True)
    rnn, mlp = net
    return O.VeLOOracle(O.rnn_weights_from_module(rnn), O.bank_from_module(mlp), SHAPES, lr=1.0, num_steps=100)


def _sums_of(plan, unit):
    """desc.sums of one unit as a tensor (a view into the plan's workspace)."""
    off = (int(plan.desc.host["sums"][unit]) - plan.workspace.data_ptr()) // 4
    return plan.workspace[off:off + 30].cpu()


@pytest.mark.parametrize("family", ["adafaclo", "celo2", "velo"])
def test_states_and_feature_moments_after_two_steps(family):
    case = dict(shapes=SHAPES, init_seed=41, init_scale=0.1, grad_seed=42, grad_scale=0.3, grad_kind="rowlognormal",
                log_mu=-2.0)
    params = [torch.nn.Parameter(v.cuda()) for v in cases.init_values(case)]
    opt = _make(family, params)
    ora = _oracle(family)
    ref = [v.clone() for v in cases.init_values(case)]
    for t in (1, 2):
        grads = cases.grads_at(case, t)
        for p, g in zip(params, grads):
            p.grad = g.cuda()
        _step(opt, family, t)
        ora.step(ref, grads, cases.velo_loss(t)) if family == "velo" else ora.step(ref, grads)
    torch.cuda.synchronize()
    keymap = {
        "adafaclo": {"exp_avg": "exp_avg", "exp_avg_sq": "exp_avg_sq", "exp_avg_sq_r": "exp_avg_sq_r", "exp_avg_sq_c": "exp_avg_sq_c"},
        "celo2": {"mom": "mom", "rms": "rms", "fac_r": "fac_r", "fac_c": "fac_c", "exp_avg": "exp_avg", "exp_avg_sq": "exp_avg_sq"},
        "velo": {"mom": "mom", "rms": "rms", "fac_vec_row": "fac_vec_row", "fac_vec_col": "fac_vec_col", "fac_vec_v": "fac_vec_v"},
    }[family]
    for i, p in enumerate(params):
        st_gpu, st_ref = opt.state[p], ora.state[i]
        for k_gpu, k_ref in keymap.items():
            if k_ref not in st_ref or k_gpu not in st_gpu or st_ref[k_ref].numel() == 0:
                continue
            a, b = st_gpu[k_gpu].detach().cpu().reshape(-1), st_ref[k_ref].reshape(-1)
            assert torch.allclose(a, b, rtol=2e-6, atol=1e-12), (family, i, k_gpu, float((a - b).abs().max()))
    # per-feature sums of squares of the last step (2-D tensors: one unit per tensor)
    plans = [v[1]["lo"] if isinstance(v[1], dict) else v[1] for v in getattr(opt, "_plans", {}).values()]
    if getattr(opt, "_plan", None):
        plans.append(opt._plan[1]["plan"])
    plan = plans[0]
    nf = 28 if family == "adafaclo" else 30
    lo_index = 0
    for i, p in enumerate(params):
        if family == "celo2" and p.dim() < 2:
            continue  # AdamW branch: no features
        if "second_moment" in ora.state[i] and p.dim() == 2:
            unit = [u for u, (ti, off) in enumerate(plan.unit_owner) if ti == lo_index and off == 0][0]
            got = _sums_of(plan, unit)[:nf].double()
            want = ora.state[i]["second_moment"].double().reshape(-1)[:nf]
            rel = ((got - want).abs() / (want.abs() + 1e-30)).max()
            assert rel < 2e-5, (family, i, float(rel))
        lo_index += 1
