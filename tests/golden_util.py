"""Load a golden fixture and drive the oracle (or any stepper) over its seeded inputs."""

import json
import os

import numpy as np
import torch

import cases
from oracle import pylo_oracle as O

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
CASES = {c["name"]: c for c in cases.ALL_CASES}


def load(name):
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    meta = json.loads(str(z["meta"]))
    weights = {k[2:]: torch.from_numpy(z[k]) for k in z.files if k.startswith("w_")}
    traj = {}
    for k in z.files:
        if k.startswith("p_step"):
            t, i = k[len("p_step"):].split("_")
            traj.setdefault(int(t), {})[int(i)] = z[k]
    traj = {t: [d[i] for i in sorted(d)] for t, d in traj.items()}
    extra = {k: z[k] for k in z.files if not (k.startswith("w_") or k.startswith("p_step") or k == "meta")}
    return meta, weights, traj, extra


def metamlp_weights(w):
    return tuple(w[k] for k in ("network.input.weight", "network.input.bias", "network.linear_0.weight",
                                "network.linear_0.bias", "network.output.weight", "network.output.bias"))


def celo2_weights(w):
    w_in = torch.cat([w[f"w0.{i}"] for i in range(14)], dim=0)
    return (w_in, w["b0"], w["dense_w.0"], w["dense_b.0"], w["dense_w.1"], w["dense_b.1"])


def velo_weights(w):
    rnn = {
        "mix2_w": w["rnn.mix_layer2.weight"], "mix2_b": w["rnn.mix_layer2.bias"],
        "fmix_w": w["rnn.final_mix_layer.weight"], "fmix_b": w["rnn.final_mix_layer.bias"],
        "lstm_w": w["rnn.lstm.linear.weight"], "lstm_b": w["rnn.lstm.linear.bias"],
        "ctrl_w": w["rnn.rnn_to_controls.weight"], "ctrl_b": w["rnn.rnn_to_controls.bias"],
        "step_w": w["rnn.step_size.weight"], "step_b": w["rnn.step_size.bias"],
        "h0": w["rnn.lstm_init_state.0"], "c0": w["rnn.lstm_init_state.1"],
    }
    keys = ["input_weights_", "input_bias_", "hidden_weights_.0", "hidden_bias_.0", "output_weights_", "output_bias_"]
    bank = torch.cat([w["mlp." + k].reshape(w["mlp." + k].shape[0], -1) for k in keys], dim=1)
    return rnn, bank


def make_oracle(case, weights, variant="cuda", dtype=torch.float32):
    fam, hp = case["family"], dict(case["hparams"])
    if fam in ("celo2", "elo_celo2"):
        if fam == "elo_celo2":
            # ELO_CELO2_naive's own defaults (ELO_CELO2_naive.py:40-60)
            base = dict(weight_decay=0.1, clip_grad=True, adam_lr_mult=1.0)
            base.update(hp)
            hp = base
        return O.CELO2Oracle(celo2_weights(weights), shared_adam=(fam == "elo_celo2"),
                             is_embedding=case.get("is_embedding"), dtype=dtype, **hp)
    if fam in ("adafaclo", "elo"):
        if fam == "elo":
            hp.setdefault("lr", 0.001)
        return O.AdafacLOOracle(metamlp_weights(weights), elo=(fam == "elo"), variant=variant, dtype=dtype, **hp)
    if fam == "velo":
        rnn, bank = velo_weights(weights)
        return O.VeLOOracle(rnn, bank, case["shapes"], variant=variant, dtype=dtype, **hp)
    raise ValueError(fam)


def run(case, stepper, record=None, dtype=torch.float32):
    """Drive ``stepper.step(params, grads[, loss])`` over the case; returns {step: [params]}."""
    params = [v.to(dtype) for v in cases.init_values(case)]
    record = record or case["record"]
    out = {}
    for t in range(1, max(record) + 1):
        grads = cases.grads_at(case, t)
        if case["family"] == "velo":
            stepper.step(params, grads, cases.velo_loss(t))
        else:
            stepper.step(params, grads)
        if t in record:
            out[t] = [p.clone() for p in params]
    return out


def max_abs_diff(traj, golden, stride=None):
    worst = 0.0
    for t, plist in golden.items():
        for a, b in zip(traj[t], plist):
            a = a.reshape(-1).double().numpy()
            if stride:
                a = a[::stride]
            worst = max(worst, float(np.max(np.abs(a - b.reshape(-1).astype(np.float64)))))
    return worst
