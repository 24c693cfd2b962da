"""Drive the CUDA optimizer classes over a golden case's seeded inputs."""

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
