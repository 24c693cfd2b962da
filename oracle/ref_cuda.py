"""The reference's own CUDA kernels as a checker and as the timed "kernel to beat".  TEST INFRASTRUCTURE ONLY.

``oracle/build_ref.py`` compiles the reference's three CUDA extensions (pylo/csrc/learned_optimizer.cu,
celo2_kernel.cu, velo_kernel.cu) from the reference checkout into ``oracle/_ref/*.so``.  This module loads those
built modules and plugs their entry points (``cuda_lo.learned_optimizer_kernel``,
``celo2_cuda_kernel.celo2_kernel``, ``velo_cuda_kernel.velo_kernel_simple``) into the oracle classes of
``oracle/pylo_oracle.py``, whose Python-side state update then runs on the GPU with torch ops exactly as the
reference's ``*_CUDA`` classes do it (AdafacLO_cuda.py:291-407, CELO2_cuda.py:255-341, velo_cuda.py:490-755).  The
result is the reference's ``*_CUDA`` path: it pins the points where that path differs from the reference's naive
classes by OUTPUT of the reference's kernels, and it is what the product kernels are timed against.

Only tests, the smoke check and the benchmark's ``reference_cuda`` leg import this; the product never does.
"""

import importlib.machinery
import importlib.util
import os
import time

import torch

from . import pylo_oracle as O

REF_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")
MODULES = ("cuda_lo", "celo2_cuda_kernel", "velo_cuda_kernel")
_loaded = {}


def available():
    return all(os.path.exists(os.path.join(REF_DIR, m + ".so")) for m in MODULES)


def load(name):
    """Import one of the reference's built extension modules from ``oracle/_ref/``."""
    if name not in _loaded:
        path = os.path.join(REF_DIR, name + ".so")
        if not os.path.exists(path):
            raise FileNotFoundError(f"{path} is missing: run `python oracle/build_ref.py` where the reference checkout is")
        loader = importlib.machinery.ExtensionFileLoader(name, path)
        spec = importlib.util.spec_from_loader(name, loader)
        mod = importlib.util.module_from_spec(spec)
        loader.exec_module(mod)
        _loaded[name] = mod
    return _loaded[name]


def adafaclo(weights, device, **kw):
    """AdafacLO_CUDA / ELO_CUDA (``elo=True``) of the reference: torch state update + ``cuda_lo`` kernel."""
    return O.AdafacLOOracle(weights, device=device, ref_kernel=load("cuda_lo").learned_optimizer_kernel, **kw)


def celo2(weights, device, **kw):
    """CELO2_CUDA / ELO_CELO2_CUDA (``shared_adam=True``) of the reference."""
    return O.CELO2Oracle(weights, device=device, ref_kernel=load("celo2_cuda_kernel").celo2_kernel, **kw)


def velo(rnn, bank, shapes, device, **kw):
    """VeLO_CUDA of the reference (its LSTM front end restated with torch ops on the device)."""
    return O.VeLOOracle(rnn, bank, shapes, device=device, ref_kernel=load("velo_cuda_kernel").velo_kernel_simple, **kw)


def _time_steps(step, steps, warmup):
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        step()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / steps


def time_against_library(dev, seeded_networks, steps=5, warmup=2):
    """Reference ``*_CUDA`` path and this library on the same GPU, same shapes, CUDA events.

    Samples (bounded so that the leg takes seconds): one Llama-3-8B transformer block for AdafacLO (seven matrices,
    two vectors, 218 M parameters) and the 4096 x 4096 + 4096 CELO2 configuration with Newton-Schulz off (the
    Newton-Schulz products are the same library GEMMs on both sides).  Returns a dict for the benchmark line."""
    from pylo_b200 import optim
    from pylo_b200 import workloads as W

    out = {"status": "ok", "what": "the reference's CUDA extensions (built for sm_100a with the flags of its setup.py) "
                                   "driven as its *_CUDA classes drive them, against this library, same GPU",
           "timing": f"CUDA events, {steps} steps after {warmup} warm-up", "cases": []}
    cases = [("adafaclo", "llama3_block", W.llama3_block(), 1e-4), ("celo2", "celo2_4096", W.celo2_4096(), 1.0)]
    for fam, wl, shapes, gscale in cases:
        n = W.total_params(shapes)
        gen = torch.Generator(device=dev).manual_seed(1)
        init = [torch.randn(s, generator=gen, device=dev) * 0.02 for s in shapes]
        grads = [torch.randn(s, generator=gen, device=dev) * gscale for s in shapes]
        net = seeded_networks(fam)
        # reference path
        ref_p = [t.clone() for t in init]
        if fam == "adafaclo":
            ref = adafaclo(net.flat_weights(), dev, lr=1e-3, step_mult=0.01, exp_mult=0.001)
        else:
            ref = celo2(net.flat_weights(), dev, lr=1e-3, weight_decay=0.1, orthogonalize=False)
        ref_ms = _time_steps(lambda: ref.step(ref_p, grads), steps, warmup)
        # this library
        ours_p = [torch.nn.Parameter(t.clone()) for t in init]
        for p, g in zip(ours_p, grads):
            p.grad = g
        if fam == "adafaclo":
            opt = optim.AdafacLO_CUDA(ours_p, lr=1e-3, step_mult=0.01, exp_mult=0.001, network=net)
        else:
            opt = optim.CELO2_CUDA(ours_p, lr=1e-3, weight_decay=0.1, orthogonalize=False, network=net)
        our_ms = _time_steps(lambda: opt.step(), steps, warmup)
        worst = 0.0
        for a, b, p0 in zip(ours_p, ref_p, init):
            moved = float((b - p0).abs().max())
            worst = max(worst, float((a.detach() - b).abs().max()) / max(moved, 1e-30))
        out["cases"].append({"optimizer": fam, "shapes": wl, "params": n, "reference_ms_per_step": ref_ms,
                             "library_ms_per_step": our_ms, "speedup": ref_ms / our_ms,
                             "reference_params_per_s": n / (ref_ms * 1e-3), "library_params_per_s": n / (our_ms * 1e-3),
                             "max_difference_over_largest_movement": worst})
        del ref, opt, ref_p, ours_p, init, grads
        torch.cuda.empty_cache()
    return out
