"""Drive the CUDA optimizer classes over a golden case's seeded inputs."""

import json
import os

import torch

import cases
import golden_util as G


def make_cuda_optimizer(case, weights, params, **extra):
    import pylo_b200
    from pylo_b200 import models, optim

    fam, hp = case["family"], dict(case["hparams"])
    hp.update(extra)  # e.g. mlp_precision="3xtf32"
    dev = params[0].device
    if fam in ("celo2", "elo_celo2"):
        net = models.CELO2MLP()
        net.load_state_dict(weights)
        emb = case.get("is_embedding")
        groups = ([{"params": [p], "is_embedding": bool(e)} for p, e in zip(params, emb)] if emb else params)
        if fam == "elo_celo2":
            # the golden run used ELO_CELO2_naive, whose adam_lr_mult default is 1.0 (ELO_CELO2_naive.py:49)
            hp.setdefault("adam_lr_mult", 1.0)
            return optim.ELO_CELO2_CUDA(groups, network=net, **hp)
        return optim.CELO2_CUDA(groups, network=net, **hp)
    if fam in ("adafaclo", "elo"):
        net = models.MetaMLP(39, 32, 1)
        net.load_state_dict(weights)
        if fam == "elo":
            return optim.ELO_CUDA(params, network=net, **hp)
        return optim.AdafacLO_CUDA(params, network=net, **hp)
    if fam == "velo":
        rnn = models.VeLORNN(lstm_hidden_size=case["lstm_hidden"])
        rnn.load_state_dict({k[4:]: v for k, v in weights.items() if k.startswith("rnn.")})
        mlp = models.VeLOMLP()
        mlp.load_state_dict({k[4:]: v for k, v in weights.items() if k.startswith("mlp.")}, strict=False)
        return optim.VeLO_CUDA(params, rnn=rnn, mlp=mlp, **hp)
    raise ValueError(fam)


def run_cuda(case, weights, record=None, device="cuda", **extra):
    params = [torch.nn.Parameter(v.to(device)) for v in cases.init_values(case)]
    opt = make_cuda_optimizer(case, weights, params, **extra)
    record = record or case["record"]
    out = {}
    for t in range(1, max(record) + 1):
        for p, g in zip(params, cases.grads_at(case, t)):
            p.grad = g.to(device)
        if case["family"] == "velo":
            opt.step(torch.tensor(cases.velo_loss(t), dtype=torch.float32, device=device))
        else:
            opt.step()
        if t in record:
            out[t] = [p.detach().cpu().clone() for p in params]
    return out, opt, params


def compare(traj_a, traj_b, init):
    """Per recorded step: (worst relative error on parameters, worst error on the movement since init).

    The relative error of an element is taken against max(|reference|, rms of its tensor), so that
    elements that happen to sit next to zero do not turn fp32 rounding into a large ratio; the
    movement error discounts four ulps of the parameter itself.
    """
    res = {}
    for t in traj_b:
        worst_p, worst_u = 0.0, 0.0
        for a, b, p0 in zip(traj_a[t], traj_b[t], init):
            a, b, p0 = a.double().reshape(-1), b.double().reshape(-1), p0.double().reshape(-1)
            scale = torch.maximum(b.abs(), b.pow(2).mean().sqrt())
            err = (a - b).abs()
            worst_p = max(worst_p, float((err / (scale + 1e-30)).max()))
            mv = (b - p0).abs().max()
            worst_u = max(worst_u, float(torch.clamp(err - 4 * 1.2e-7 * b.abs(), min=0).max() / (mv + 1e-30)))
        res[t] = (worst_p, worst_u)
    return res


def update_error(a, b, p0):
    """Worst per-element relative error of the UPDATE ``p - p0`` of one tensor.

    ``a`` is the tensor under test, ``b`` the reference, ``p0`` the value both started from.  The error of an
    element is taken against max(|its reference update|, rms of the tensor's reference update), after four ulps
    of the parameter itself are discounted (the update is read back as a difference of two fp32 parameters, which
    carries that much rounding whatever the arithmetic that produced it).
    """
    a, b, p0 = a.double().reshape(-1), b.double().reshape(-1), p0.double().reshape(-1)
    du = b - p0
    err = torch.clamp((a - b).abs() - 4 * 1.2e-7 * b.abs(), min=0)
    scale = torch.maximum(du.abs(), du.pow(2).mean().sqrt())
    return float((err / (scale + 1e-30)).max())


def compare_updates(traj_a, traj_b, init):
    """{step: worst :func:`update_error` over the tensors} for two trajectories."""
    return {t: max(update_error(a, b, p0) for a, b, p0 in zip(traj_a[t], traj_b[t], init)) for t in traj_b}


def log_parity(test, **numbers):
    """Append observed error figures to the file named by PYLO_PARITY_LOG (used when tolerances are reviewed)."""
    path = os.environ.get("PYLO_PARITY_LOG")
    if path:
        with open(path, "a") as f:
            f.write(json.dumps({"test": test, **{k: (v if isinstance(v, (int, float, str)) else repr(v)) for k, v in numbers.items()}}) + "\n")
