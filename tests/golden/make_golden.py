"""Generate the golden trajectories under tests/golden/ from the reference's own code.

Run once, where a checkout of the reference is available; point ``PYLO_REFERENCE`` at it
(default: a sibling directory ``reference`` next to this repository):

    python tests/golden/make_golden.py

It imports the reference's CPU-capable ``*_naive`` optimizer classes and
meta-model modules *unmodified*, runs them on seeded inputs and writes
``tests/golden/<case>.npz`` holding the meta-model weights, the seeds and
hyper-parameters (as a JSON string) and the parameter values after selected
steps.  Inputs are regenerated from the seeds by ``tests/golden/cases.py`` so
the fixtures stay small.

Two shims are applied to make ``import pylo`` work without network or the
``mup`` package, neither of which touches arithmetic:
* a stub ``mup.optim.process_param_groups`` (``pylo/optim/MuLO_naive.py:7``
  imports it at module import time);
* ``MetaMLP/VeLORNN/VeLOMLP.from_pretrained`` return seeded random-init
  modules (``AdafacLO_naive.py:183`` and ``Velo_naive.py:286-289`` call them
  unconditionally and the hub is unreachable).
"""

import json
import os
import sys
import types
import warnings

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import cases  # noqa: E402


def load_reference():
    default = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference")
    ref = os.environ.get("PYLO_REFERENCE", default)
    mup = types.ModuleType("mup")
    mup_optim = types.ModuleType("mup.optim")
    mup_optim.process_param_groups = lambda *a, **k: None
    mup.optim = mup_optim
    sys.modules.setdefault("mup", mup)
    sys.modules.setdefault("mup.optim", mup_optim)
    sys.path.insert(0, ref)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        import pylo  # noqa: F401
    return pylo


def run_trajectory(opt, params, grad_fn, steps, record, loss_fn=None):
    out = {}
    for t in range(1, steps + 1):
        for p, g in zip(params, grad_fn(t)):
            p.grad = g.clone()
        if loss_fn is None:
            opt.step()
        else:
            opt.step(loss_fn(t))
        if t in record:
            out[t] = [p.detach().clone().numpy() for p in params]
    return out


def save(name, weights, meta, traj, extra=None):
    arrays = {f"w_{k}": v.detach().numpy() for k, v in weights.items()}
    for t, plist in traj.items():
        for i, a in enumerate(plist):
            arrays[f"p_step{t}_{i}"] = a
    if extra:
        arrays.update(extra)
    arrays["meta"] = np.array(json.dumps(meta))
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **arrays)
    print(f"{name}: {os.path.getsize(path) / 1024:.0f} KiB")


def main():
    load_reference()
    from pylo.models.CELO2_MLP import CELO2MLP
    from pylo.models.Meta_MLP import MetaMLP
    from pylo.models.VeLO_MLP import VeLOMLP
    from pylo.models.VeLO_RNN import VeLORNN
    from pylo.optim.AdafacLO_naive import AdafacLO_naive
    from pylo.optim.CELO2_naive import CELO2_naive
    from pylo.optim.ELO_CELO2_naive import ELO_CELO2_naive
    from pylo.optim.ELO_naive import ELO_naive
    from pylo.optim.Velo_naive import VeLO_naive

    torch.set_num_threads(1)  # fixed reduction order inside torch CPU kernels

    # ---------------- CELO2 / ELO_CELO2 ----------------
    for case in cases.CELO2_CASES:
        torch.manual_seed(case["net_seed"])
        net = CELO2MLP()
        params = [torch.nn.Parameter(v) for v in cases.init_values(case)]
        cls = ELO_CELO2_naive if case["family"] == "elo_celo2" else CELO2_naive
        emb = case.get("is_embedding")
        if emb:
            groups = [{"params": [p], "is_embedding": bool(e)} for p, e in zip(params, emb)]
        else:
            groups = params
        opt = cls(groups, network=net, **case["hparams"])
        traj = run_trajectory(opt, params, lambda t, c=case: cases.grads_at(c, t), case["steps"], case["record"])
        save(case["name"], dict(net.state_dict()), case, traj)

    # ---------------- AdafacLO / ELO ----------------
    for case in cases.ADAFAC_CASES:
        torch.manual_seed(case["net_seed"])
        net = MetaMLP(input_size=39, hidden_size=32, hidden_layers=1)
        params = [torch.nn.Parameter(v) for v in cases.init_values(case)]
        if case["family"] == "elo":
            opt = ELO_naive(params, network=net, **case["hparams"])
        else:
            MetaMLP.from_pretrained = classmethod(lambda cls, *a, _n=net, **k: _n)
            opt = AdafacLO_naive(params, **case["hparams"])
        traj = run_trajectory(opt, params, lambda t, c=case: cases.grads_at(c, t), case["steps"], case["record"])
        sample = case.get("sample_stride")
        if sample:
            traj = {t: [a.reshape(-1)[::sample].copy() for a in pl] for t, pl in traj.items()}
        save(case["name"], dict(net.state_dict()), case, traj)

    # ---------------- VeLO ----------------
    for case in cases.VELO_CASES:
        torch.manual_seed(case["net_seed"])
        rnn = VeLORNN(lstm_hidden_size=case["lstm_hidden"])
        mlp = VeLOMLP()
        with torch.no_grad():
            for k, v in mlp.state_dict().items():
                if k.endswith("_") or "_." in k:
                    v.mul_(case["bank_scale"])
            # give the bias banks and the LSTM start state non-trivial values
            g = torch.Generator().manual_seed(case["net_seed"] + 1)
            for k, v in mlp.state_dict().items():
                if "bias_" in k:
                    v.copy_(torch.randn(v.shape, generator=g) * case["bank_scale"])
            for v in rnn.lstm_init_state:
                v.copy_(torch.randn(v.shape, generator=g) * 0.1)
        VeLORNN.from_pretrained = classmethod(lambda cls, *a, _n=rnn, **k: _n)
        VeLOMLP.from_pretrained = classmethod(lambda cls, *a, _n=mlp, **k: _n)
        params = [torch.nn.Parameter(v) for v in cases.init_values(case)]
        opt = VeLO_naive(params, **case["hparams"])
        weights = {("rnn." + k): v for k, v in rnn.state_dict().items()}
        weights.update({("mlp." + k): v for k, v in mlp.state_dict().items() if k.endswith("_") or "_." in k})
        traj = run_trajectory(
            opt, params, lambda t, c=case: cases.grads_at(c, t), case["steps"], case["record"],
            loss_fn=lambda t: torch.tensor(cases.velo_loss(t), dtype=torch.float32),
        )
        extra = {
            "lstm_h": opt.lstm_hidden_state[0].detach().numpy(),
            "lstm_c": opt.lstm_hidden_state[1].detach().numpy(),
            "loss_means": opt.loss_buffer["means"].numpy(),
            "loss_running_min": opt.loss_buffer["running_min"].numpy(),
        }
        save(case["name"], weights, case, traj, extra)


if __name__ == "__main__":
    main()
