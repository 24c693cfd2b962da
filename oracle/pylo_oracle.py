"""CPU oracle for the learned-optimizer ``step()`` hot path.  TEST INFRASTRUCTURE ONLY.

This file restates, with plain ``torch`` CPU tensor arithmetic, what the
reference's ``*_CUDA`` optimizer classes compute in one ``step()``: the Python
side state update *and* the arithmetic of the fused CUDA kernels they call.
The reference classes themselves hard-code ``device="cuda"`` and call a
CUDA-only extension, so they cannot run on a CPU; the pieces restated here are

* AdafacLO_CUDA / ELO_CUDA   pylo/optim/AdafacLO_cuda.py:291-407,
                             pylo/optim/ELO_cuda.py:179-288,
                             pylo/csrc/learned_optimizer.cu:35-97,223-300
* CELO2_CUDA / ELO_CELO2_CUDA pylo/optim/CELO2_cuda.py:180-341,
                             pylo/optim/ELO_CELO2_cuda.py:179-298,
                             pylo/csrc/celo2_kernel.cu:49-125,229-281,
                             pylo/optim/CELO2_naive.py:42-73
* VeLO_CUDA                  pylo/optim/velo_cuda.py:121-252,389-434,464-565,668-755,
                             pylo/csrc/velo_kernel.cu:73-164,288-367,
                             pylo/models/VeLO_RNN.py:43-66,110-135,
                             pylo/models/VeLO_MLP.py:92-126

Nothing in the shipped package imports this module.  It is used by the test
suite, by the smoke check and by the CPU-baseline leg of the benchmark, always
as the checker or the timed baseline, never as the product path.

Parity status: pinned.  ``tests/golden/make_golden.py`` runs the reference's own
``*_naive`` classes (imported from the reference checkout) on seeded inputs and
stores their trajectories; ``variant="naive"`` below switches the handful of
places where the reference's CUDA classes knowingly differ from its naive
classes (listed at ``Variant``), and in that mode this oracle must reproduce
those trajectories.  The ``variant="cuda"`` arithmetic shares every other line
with the pinned mode.  What stays unpinned by any reference test: the CUDA
classes on tensors with three or more dimensions, and all VeLO numerics beyond
what ``VeLO_naive`` shares with ``VeLO_CUDA``.

State layout is the ``*_CUDA`` one (decay axis leading), which is also the
resume format of the product classes, so states can be compared key by key.

Every oracle class takes ``device=`` (default CPU) and ``ref_kernel=``.  With a
``ref_kernel`` the Python-side state update restated here runs on that device
and the fused part of the step is done by the REFERENCE'S OWN CUDA extension
(built from the reference's sources by ``oracle/build_ref.py``, loaded by
``oracle/ref_cuda.py``) instead of the restatement in
``_feature_moments_and_apply``: the reference's ``*_CUDA`` path end to end, used
on a GPU as a second checker and as the timed "kernel to beat".
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

# Elements per block when the per-element feature matrix is materialised.
_CHUNK = 1 << 20

TIMESCALES = (1.0, 3.0, 10.0, 30.0, 100.0, 300.0, 1000.0, 3000.0, 10000.0, 30000.0, 100000.0)


# --------------------------------------------------------------------------------------
# small helpers
# --------------------------------------------------------------------------------------
def decay_reparam(initial: Sequence[float], offset: Sequence[float]) -> torch.Tensor:
    """``clip(1 - exp(10 * (log(1 - b0) / 10 + theta)), 0, 1)`` in fp32 (AdafacLO_cuda.py:29-34,153-177)."""
    b0 = torch.tensor(list(initial), dtype=torch.float32)
    theta = torch.tensor(list(offset), dtype=torch.float32)
    return torch.clip(1 - torch.exp((torch.log(1 - b0) / 10.0 + theta) * 10.0), 0.0, 1.0)


def clamp_decays(decays: Sequence[float]) -> torch.Tensor:
    """Raw decays clamped to [0, 1] in fp32 (CELO2_cuda.py:120-131)."""
    return torch.clamp(torch.tensor(list(decays), dtype=torch.float32), 0.0, 1.0)


def factored_dims_sorted(shape) -> Optional[Tuple[int, int]]:
    """(dc, dr) by ``sorted((size, index))`` (AdafacLO_cuda.py:52-73 with min size 1, ELO_cuda.py:46-51)."""
    if len(shape) < 2:
        return None
    order = sorted((s, i) for i, s in enumerate(shape))
    return int(order[-2][1]), int(order[-1][1])


def factored_dims_argsort(shape) -> Optional[Tuple[int, int]]:
    """(dc, dr) by ``np.argsort`` (CELO2_naive.py:42-47)."""
    if len(shape) < 2:
        return None
    order = np.argsort(shape)
    return int(order[-2]), int(order[-1])


def factored_dims_velo(shape) -> Optional[Tuple[int, int]]:
    """(dc, dr) with VeLO's tie rule (velo_cuda.py:121-131)."""
    if len(shape) < 2:
        return None
    order = np.argsort(shape)
    a, b = int(order[-2]), int(order[-1])
    if shape[a] == shape[b] and not (len(shape) == 4 and a == 0 and b == 1):
        return b, a
    return a, b


def safe_rsqrt(x: torch.Tensor) -> torch.Tensor:
    return torch.rsqrt(torch.clamp(x, min=1e-9))


def tanh_time_features(step0: float, dtype) -> torch.Tensor:
    """``tanh(t / tau - 1)`` for the 11 time scales, t 0-based (learned_optimizer.cu:27-32,245-248)."""
    t = torch.tensor(float(step0), dtype=torch.float32)
    return torch.tanh(t / torch.tensor(TIMESCALES, dtype=torch.float32) - 1.0).to(dtype)


def newton_schulz(x: torch.Tensor, coeffs, iters: int, eps: float) -> torch.Tensor:
    """Newton-Schulz orthogonalisation over the last two axes (CELO2_naive.py:59-73)."""
    flip = x.shape[-2] > x.shape[-1]
    if flip:
        x = x.transpose(-2, -1)
    x = x / (torch.linalg.norm(x, dim=(-2, -1), keepdim=True) + eps)
    c0, c1, c2 = coeffs
    for _ in range(iters):
        a = x @ x.transpose(-2, -1)
        b = c1 * a + c2 * (a @ a)
        x = c0 * x + b @ x
    return x.transpose(-2, -1) if flip else x


def _lead(v: torch.Tensor, ndim: int) -> torch.Tensor:
    return v.view([-1] + [1] * ndim)


@dataclass
class Variant:
    """Where the reference's CUDA classes and naive classes differ.

    ``cuda`` (default) follows the ``*_CUDA`` classes; ``naive`` follows the
    ``*_naive`` classes and exists so the restatement can be pinned against
    trajectories of the reference's own CPU-capable code.

    * ``fix_axis``: AdafacLO/ELO reduce ``row_col_mean`` over the decay axis for
      2-D tensors in the CUDA class (AdafacLO_cuda.py:342-343) and over the dc
      axis in the naive class (AdafacLO_naive.py:284-285).
    * ``naive_1d``: for 1-D tensors the CUDA class uses
      ``m * safe_rsqrt(v + 1e-9)`` (AdafacLO_cuda.py:358-360); AdafacLO_naive uses
      ``m * (v + 1e-6) ** -0.5`` (AdafacLO_naive.py:298) and VeLO_naive
      ``m * v ** -0.5`` (Velo_naive.py:487); the ``g`` feature keeps safe_rsqrt.
    * ``naive_wd``: VeLO_CUDA decays with ``lr * lr_mult`` (velo_kernel.cu:364-366);
      VeLO_naive with the group ``lr`` (Velo_naive.py:500-502).
    """

    name: str = "cuda"

    @property
    def naive(self) -> bool:
        return self.name == "naive"


# --------------------------------------------------------------------------------------
# shared state-update pieces
# --------------------------------------------------------------------------------------
def _update_factored(state, grad_sqr, fdims, beta_fac, key_r, key_c, reduce_axis):
    """Row/column EMA and the two rsqrt factor tensors for a tensor with >= 2 dims.

    ``reduce_axis`` is the axis of the leading-decay row accumulator over which
    ``row_col_mean`` is taken.
    """
    dc, dr = fdims
    w = 1 - _lead(beta_fac, grad_sqr.dim()).to(grad_sqr.dtype)
    fac_r, fac_c = state[key_r], state[key_c]
    fac_r.lerp_(grad_sqr.mean(dim=dr, keepdim=True)[None, ...], w)
    fac_c.lerp_(grad_sqr.mean(dim=dc, keepdim=True)[None, ...], w)
    row_col_mean = fac_r.mean(dim=reduce_axis, keepdim=True)
    row_factor = safe_rsqrt(fac_r / (row_col_mean + 1e-9))
    col_factor = safe_rsqrt(fac_c)
    return fac_r, fac_c, row_factor, col_factor


def _feature_moments_and_apply(n, nfeat, build, norm_eps, mlp, consume, norm_groups=None):
    """Two passes over the tensor in blocks: per-feature sum of squares, then the MLP.

    ``build(lo, hi)`` returns the ``[hi-lo, nfeat]`` feature block, ``mlp`` maps
    normalised features to outputs, ``consume(lo, hi, out)`` applies them.
    ``norm_groups``: optional ``(group_index[n] int64, n_groups, group_size)`` to
    normalise per group of elements instead of over the whole tensor.
    """
    first = build(0, min(n, 1))
    acc_dtype = torch.float64
    if norm_groups is None:
        s = torch.zeros(nfeat, dtype=acc_dtype)
        for lo in range(0, n, _CHUNK):
            f = build(lo, min(n, lo + _CHUNK))
            s += (f.to(acc_dtype) ** 2).sum(0)
        scale = torch.rsqrt((s / n).to(first.dtype) + norm_eps)
        for lo in range(0, n, _CHUNK):
            hi = min(n, lo + _CHUNK)
            consume(lo, hi, mlp(build(lo, hi) * scale))
        return s.to(first.dtype)
    gidx, ng, gsize = norm_groups
    s = torch.zeros(ng, nfeat, dtype=acc_dtype)
    for lo in range(0, n, _CHUNK):
        hi = min(n, lo + _CHUNK)
        s.index_add_(0, gidx[lo:hi], build(lo, hi).to(acc_dtype) ** 2)
    scale = torch.rsqrt((s / gsize).to(first.dtype) + norm_eps)
    for lo in range(0, n, _CHUNK):
        hi = min(n, lo + _CHUNK)
        consume(lo, hi, mlp(build(lo, hi) * scale[gidx[lo:hi]]))
    return s.to(first.dtype)


def _bcast_flat(t: torch.Tensor, shape) -> torch.Tensor:
    """Expand a keep-dim factor tensor ``[3]+shape[d->1]`` to ``[3, n]`` (a view where possible)."""
    return t.expand([t.shape[0]] + list(shape)).reshape(t.shape[0], -1)


# --------------------------------------------------------------------------------------
# AdafacLO / ELO
# --------------------------------------------------------------------------------------
class AdafacLOOracle:
    """One ``AdafacLO_CUDA.step()`` (``elo=False``) or ``ELO_CUDA.step()`` (``elo=True``).

    ``weights`` = (w_in[32,39], b_in[32], w_h[32,32], b_h[32], w_out[2,32], b_out[2]),
    ``nn.Linear`` orientation.
    """

    FEAT = 28

    def __init__(
        self,
        weights,
        lr=1.0,
        step_mult=0.01,
        exp_mult=0.001,
        weight_decay=0.0,
        beta_m=None,
        beta_rms=None,
        beta_fac=None,
        elo=False,
        clip_grad=False,
        clip_norm=1.0,
        variant="cuda",
        dtype=torch.float32,
        device="cpu",
        ref_kernel=None,
    ):
        self.dtype = dtype
        self.device = torch.device(device)
        self.ref_kernel = ref_kernel  # cuda_lo.learned_optimizer_kernel of the reference, or None
        self.w = [w.detach().to(dtype).to(self.device).contiguous() for w in weights]
        self.lr, self.step_mult, self.exp_mult, self.wd = lr, step_mult, exp_mult, weight_decay
        self.elo, self.clip_grad, self.clip_norm = elo, clip_grad, clip_norm
        if elo:
            self.beta_m = clamp_decays(beta_m or (0.9, 0.99, 0.999))
            self.beta_rms = clamp_decays(beta_rms or (0.999,))
            self.beta_fac = clamp_decays(beta_fac or (0.9, 0.99, 0.999))
        else:
            self.beta_m = beta_m if beta_m is not None else decay_reparam((0.9, 0.99, 0.999), (0.15216392, 0.14245212, 0.06812963))
            self.beta_rms = beta_rms if beta_rms is not None else decay_reparam((0.999,), (0.01079706,))
            self.beta_fac = beta_fac if beta_fac is not None else decay_reparam((0.9, 0.99, 0.999), (0.18621896, -0.10864615, -0.06185547))
        self.beta_m, self.beta_rms, self.beta_fac = (b.to(self.device) for b in (self.beta_m, self.beta_rms, self.beta_fac))
        self.variant = Variant(variant)
        self.state: List[Dict] = []

    def _init_state(self, g):
        shape = tuple(g.shape)
        st = {"step": 0.0}
        kw = dict(dtype=self.dtype, device=self.device)
        fd = factored_dims_sorted(shape)
        if fd is not None:
            dc, dr = fd
            rs, cs = list(shape), list(shape)
            rs[dr], cs[dc] = 1, 1
            st["exp_avg_sq_r"] = torch.zeros([3] + rs, **kw)
            st["exp_avg_sq_c"] = torch.zeros([3] + cs, **kw)
        else:
            st["exp_avg_sq_r"] = torch.zeros((3,) + shape, **kw)
            st["exp_avg_sq_c"] = torch.zeros((3,) + shape, **kw)
        st["exp_avg_sq"] = torch.zeros(shape, **kw)
        st["exp_avg"] = torch.zeros((3,) + shape, **kw)
        return st

    def _mlp(self, x):
        w_in, b_in, w_h, b_h, w_out, b_out = self.w
        h = torch.relu(x @ w_in.T + b_in)
        h = torch.relu(h @ w_h.T + b_h)
        return h @ w_out.T + b_out

    def step(self, params: List[torch.Tensor], grads: List[torch.Tensor]):
        if not self.state:
            self.state = [self._init_state(g) for g in grads]
        scale = 1.0
        if self.elo and self.clip_grad:
            scale = global_grad_scale(grads, self.clip_norm)
        for p, g0, st in zip(params, grads, self.state):
            g = g0.to(self.dtype)
            if self.elo:
                if scale != 1.0:
                    g = g * scale
                g = torch.nan_to_num(g)
            self._step_tensor(p, g, st)

    def _step_tensor(self, p, g, st):
        dt = self.dtype
        shape = tuple(g.shape)
        n = g.numel()
        st["step"] += 1.0
        grad_sqr = torch.square(g) + 1e-30
        fd = factored_dims_sorted(shape)
        w_rms = (1 - self.beta_rms).to(dt)
        if fd is not None:
            dc, dr = fd
            if self.variant.naive:
                axis = dc + 1
            else:
                axis = dc - 1 if dc > dr else dc
            fac_r, fac_c, rf, cf = _update_factored(
                st, grad_sqr, fd, self.beta_fac, "exp_avg_sq_r", "exp_avg_sq_c", axis
            )
            st["exp_avg_sq"].lerp_(grad_sqr, w_rms)
            rf_g = rf_m = _bcast_flat(rf, shape)
            cf_g = cf_m = _bcast_flat(cf, shape)
            fr, fc = _bcast_flat(fac_r, shape), _bcast_flat(fac_c, shape)
        else:
            w_fac = 1 - self.beta_fac.view(-1, 1).to(dt)
            st["exp_avg_sq_r"].lerp_(grad_sqr[None, ...], w_fac)
            st["exp_avg_sq_c"].lerp_(grad_sqr[None, ...], w_fac)
            st["exp_avg_sq"].lerp_(grad_sqr, w_rms)
            fr = st["exp_avg_sq_r"].reshape(3, -1)
            fc = st["exp_avg_sq_c"].reshape(3, -1)
            rf_g = safe_rsqrt(fr + 1e-9)
            rf_m = torch.pow(fr + 1e-6, -0.5) if self.variant.naive else rf_g
            cf_g = cf_m = None
        st["exp_avg"].lerp_(g[None, ...], 1 - _lead(self.beta_m, g.dim()).to(dt))

        if self.ref_kernel is not None:
            # AdafacLO_cuda.py:378-405 / ELO_cuda.py:262-286: the reference's fused kernel does the rest
            if fd is not None:
                row_factor, col_factor, kdc, kdr, vector_like = rf, cf, fd[0], fd[1], 0
            else:
                row_factor = safe_rsqrt(st["exp_avg_sq_r"] + 1e-9)
                col_factor, kdc, kdr, vector_like = torch.ones_like(row_factor), 0, 0, 1
            second = torch.zeros(28, dtype=dt, device=self.device)
            p_before = p.clone() if (self.elo and self.wd > 0) else None
            self.ref_kernel(g.contiguous(), p, st["exp_avg"], st["exp_avg_sq"], st["exp_avg_sq_r"], st["exp_avg_sq_c"],
                            row_factor.contiguous(), col_factor.contiguous(), second, *self.w, float(self.lr),
                            1.0 if self.elo else float(self.step_mult), float(self.exp_mult), 1e-6, st["step"] - 1.0, 0.0,
                            int(kdc), int(kdr), int(vector_like))
            st["second_moment"] = second
            if self.wd > 0:
                p.add_(p_before if self.elo else p, alpha=-self.wd * self.lr)
            return

        gf, pf = g.reshape(-1), p.reshape(-1)
        m = st["exp_avg"].reshape(3, -1)
        v = st["exp_avg_sq"].reshape(-1)

        def build(lo, hi):
            f = torch.empty(hi - lo, self.FEAT, dtype=dt)
            f[:, 0] = gf[lo:hi]
            f[:, 1] = pf[lo:hi]
            f[:, 2:5] = m[:, lo:hi].T
            f[:, 5] = v[lo:hi]
            rs = torch.rsqrt(v[lo:hi] + 1e-6)
            f[:, 6:9] = (m[:, lo:hi] * rs).T
            f[:, 9] = rs
            fg = rf_g[:, lo:hi] if cf_g is None else rf_g[:, lo:hi] * cf_g[:, lo:hi]
            fm = rf_m[:, lo:hi] if cf_m is None else rf_m[:, lo:hi] * cf_m[:, lo:hi]
            f[:, 10:13] = (fg * gf[lo:hi]).T
            f[:, 13:16] = fr[:, lo:hi].T
            f[:, 16:19] = fc[:, lo:hi].T
            f[:, 19:22] = torch.rsqrt(fr[:, lo:hi] + 1e-8).T
            f[:, 22:25] = torch.rsqrt(fc[:, lo:hi] + 1e-8).T
            f[:, 25:28] = (fm * m[:, lo:hi]).T
            return f

        time_feat = tanh_time_features(st["step"] - 1.0, dt)
        step_mult = 1.0 if self.elo else self.step_mult
        p_before = p.clone() if (self.elo and self.wd > 0) else None

        def mlp(x):
            x = torch.cat([x, time_feat.expand(x.shape[0], -1)], dim=1)
            return self._mlp(x)

        def consume(lo, hi, out):
            upd = out[:, 0] * torch.exp(out[:, 1] * self.exp_mult) * step_mult
            pf[lo:hi] -= self.lr * upd

        st["second_moment"] = _feature_moments_and_apply(n, self.FEAT, build, 1e-5, mlp, consume)
        if self.wd > 0:
            if self.elo:
                p.add_(p_before, alpha=-self.wd * self.lr)
            else:
                p.add_(p, alpha=-self.wd * self.lr)


def global_grad_scale(grads, clip_norm) -> float:
    """``clip_norm / max(||g||, clip_norm)`` over all tensors, fp32 (CELO2_cuda.py:180-188)."""
    total = torch.zeros((), dtype=torch.float32)
    for g in grads:
        total = total + g.detach().float().pow(2).sum()
    denom = torch.clamp(torch.sqrt(total), min=clip_norm)
    return (clip_norm / denom).item() if denom > 0 else 1.0


# --------------------------------------------------------------------------------------
# CELO2 / ELO_CELO2
# --------------------------------------------------------------------------------------
class CELO2Oracle:
    """One ``CELO2_CUDA.step()`` (``shared_adam=False``) or ``ELO_CELO2_CUDA.step()`` (``True``).

    ``weights`` = (w_in[30,8], b_in[8], w_h[8,8], b_h[8], w_out[8,3], b_out[3]),
    all **in-major** (the network computes ``x @ w``).

    For tensors with three or more dimensions the reference CUDA kernel reads
    the factor vectors of the wrong slice (celo2_kernel.cu:79-84,107-112) and
    normalises over all elements (celo2_kernel.cu:233) while every other step of
    the same class works on the last two axes; no reference test runs that
    case.  This oracle uses the naive class's meaning there (correct slice,
    normaliser over the last two axes, CELO2_naive.py:328-329); for 2-D tensors
    the two meanings coincide.
    """

    FEAT = 30

    def __init__(
        self,
        weights,
        lr=1e-3,
        weight_decay=0.0,
        adam_lr_mult=1.0,
        adam_weight_decay=None,
        adam_betas=(0.9, 0.95),
        adam_eps=1e-8,
        use_adamw_for_1d=True,
        orthogonalize=True,
        clip_grad=False,
        clip_norm=1.0,
        beta_m=(0.9, 0.99, 0.999),
        beta_rms=(0.95,),
        beta_fac=(0.9, 0.99, 0.999),
        exp_mult=0.0,
        rmsmult=1.0,
        ns_coeffs=(3.4445, -4.7750, 2.0315),
        ns_iters=5,
        ns_eps=1e-8,
        grad_clip_val=1000.0,
        shared_adam=False,
        is_embedding: Optional[Sequence[bool]] = None,
        dtype=torch.float32,
        device="cpu",
        ref_kernel=None,
    ):
        self.dtype = dtype
        self.device = torch.device(device)
        self.ref_kernel = ref_kernel  # celo2_cuda_kernel.celo2_kernel of the reference, or None
        self.w = [w.detach().to(dtype).to(self.device).contiguous() for w in weights]
        self.lr, self.wd = lr, weight_decay
        self.adam_lr_mult = adam_lr_mult
        self.adam_wd = adam_weight_decay if adam_weight_decay is not None else weight_decay
        self.adam_b1, self.adam_b2 = (float(b) for b in adam_betas)
        self.adam_eps = adam_eps
        self.use_adamw_for_1d = use_adamw_for_1d
        self.orthogonalize, self.clip_grad, self.clip_norm = orthogonalize, clip_grad, clip_norm
        self.beta_m, self.beta_rms, self.beta_fac = (clamp_decays(b).to(self.device) for b in (beta_m, beta_rms, beta_fac))
        self.exp_mult, self.rmsmult = exp_mult, rmsmult
        self.ns = (tuple(float(c) for c in ns_coeffs), ns_iters, ns_eps)
        self.grad_clip_val = grad_clip_val
        self.shared_adam = shared_adam
        self.is_embedding = is_embedding
        self.group_step = 0
        self.state: List[Dict] = []

    def _mlp(self, x):
        w_in, b_in, w_h, b_h, w_out, b_out = self.w
        h = torch.relu(x @ w_in + b_in)
        h = torch.relu(h @ w_h + b_h)
        return h @ w_out + b_out

    def _init_lo_state(self, st, shape):
        kw = dict(dtype=self.dtype, device=self.device)
        st["mom"] = torch.zeros((3,) + shape, **kw)
        st["rms"] = torch.zeros(shape, **kw)
        fd = factored_dims_argsort(shape)
        if fd is not None:
            dc, dr = fd
            rs, cs = list(shape), list(shape)
            rs[dr], cs[dc] = 1, 1
            st["fac_r"] = torch.zeros([3] + rs, **kw)
            st["fac_c"] = torch.zeros([3] + cs, **kw)

    def step(self, params, grads):
        if not self.state:
            self.state = [dict() for _ in grads]
        scale = global_grad_scale(grads, self.clip_norm) if self.clip_grad else 1.0
        self.group_step += 1
        for i, (p, g0, st) in enumerate(zip(params, grads, self.state)):
            g = g0.to(self.dtype)
            if scale != 1.0:
                g = g * scale
            g = torch.clamp(g, -self.grad_clip_val, self.grad_clip_val)
            forced = bool(self.is_embedding[i]) if self.is_embedding is not None else False
            is_1d = p.dim() <= 1 or forced
            if self.shared_adam:
                if not st:
                    self._init_lo_state(st, tuple(p.shape))
                self._update_mom_rms(st, g)
                if self.use_adamw_for_1d and is_1d:
                    self._adam_shared(p, st)
                    continue
                self._lo_tensor(p, g, st)
            else:
                if self.use_adamw_for_1d and is_1d:
                    self._adam_independent(p, g, st)
                    continue
                if p.dim() < 2:
                    raise ValueError("CELO2 needs use_adamw_for_1d=True for tensors with fewer than 2 dims")
                if "mom" not in st:
                    self._init_lo_state(st, tuple(p.shape))
                self._update_mom_rms(st, g)
                self._lo_tensor(p, g, st)

    def _update_mom_rms(self, st, g):
        st["mom"].lerp_(g[None, ...], _lead(1 - self.beta_m, g.dim()).to(self.dtype))
        st["rms"].lerp_(g * g, float(1 - self.beta_rms[-1]))

    def _adam_independent(self, p, g, st):
        """CELO2_cuda.py:234-253."""
        if "exp_avg" not in st:
            st["exp_avg"] = torch.zeros_like(p)
            st["exp_avg_sq"] = torch.zeros_like(p)
            st["adam_step"] = 0
        st["adam_step"] += 1
        t = st["adam_step"]
        b1, b2 = self.adam_b1, self.adam_b2
        st["exp_avg"].mul_(b1).add_(g, alpha=1 - b1)
        st["exp_avg_sq"].mul_(b2).addcmul_(g, g, value=1 - b2)
        m_bc = st["exp_avg"] / (1.0 - b1 ** t)
        v_bc = st["exp_avg_sq"] / (1.0 - b2 ** t)
        upd = m_bc / (torch.sqrt(v_bc) + self.adam_eps)
        p.add_(upd + self.adam_wd * p, alpha=-(self.adam_lr_mult * self.lr))

    def _adam_shared(self, p, st):
        """ELO_CELO2_cuda.py:244-253."""
        t = self.group_step
        b1, b2 = float(self.beta_m[0]), float(self.beta_rms[-1])
        m_bc = st["mom"][0] / (1.0 - b1 ** t)
        v_bc = st["rms"] / (1.0 - b2 ** t)
        upd = m_bc / (torch.sqrt(v_bc) + 1e-8)
        p.add_(upd + self.adam_wd * p, alpha=-(self.adam_lr_mult * self.lr))

    def _lo_tensor(self, p, g, st):
        dt = self.dtype
        shape = tuple(p.shape)
        n = p.numel()
        fd = factored_dims_argsort(shape)
        dc, dr = fd
        grad_sqr = g * g + 1e-30
        fac_r, fac_c, rf, cf = _update_factored(st, grad_sqr, fd, self.beta_fac, "fac_r", "fac_c", dc + 1)
        if self.ref_kernel is not None:
            # CELO2_cuda.py:301-339: the reference's fused kernel writes the raw step, the tail stays torch
            second = torch.zeros(self.FEAT, dtype=dt, device=self.device)
            step = torch.empty_like(p)
            self.ref_kernel(g.contiguous(), p, st["mom"], st["rms"], fac_r, fac_c, rf.contiguous(), cf.contiguous(), second,
                            *self.w, step, float(self.exp_mult), int(dc), int(dr), 0)
            st["second_moment"] = second
            self._tail(p, step, st)
            return
        rfb, cfb = _bcast_flat(rf, shape), _bcast_flat(cf, shape)
        fr, fc = _bcast_flat(fac_r, shape), _bcast_flat(fac_c, shape)
        gf, pf = g.reshape(-1), p.reshape(-1)
        m = st["mom"].reshape(3, -1)
        v = st["rms"].reshape(-1)

        def build(lo, hi):
            f = torch.empty(hi - lo, self.FEAT, dtype=dt)
            gg = gf[lo:hi]
            f[:, 0] = gg
            f[:, 1] = torch.clamp(gg, -0.1, 0.1)
            f[:, 2] = pf[lo:hi]
            f[:, 3:6] = m[:, lo:hi].T
            f[:, 6] = v[lo:hi]
            rs = torch.rsqrt(v[lo:hi] + 1e-8)
            f[:, 7:10] = (m[:, lo:hi] * rs).T
            f[:, 10] = rs
            fac = rfb[:, lo:hi] * cfb[:, lo:hi]
            f[:, 11:14] = (fac * gg).T
            f[:, 14] = gg * rs
            f[:, 15:18] = fr[:, lo:hi].T
            f[:, 18:21] = fc[:, lo:hi].T
            f[:, 21:24] = torch.rsqrt(fr[:, lo:hi] + 1e-8).T
            f[:, 24:27] = torch.rsqrt(fc[:, lo:hi] + 1e-8).T
            f[:, 27:30] = (fac * m[:, lo:hi]).T
            return f

        step_flat = torch.empty(n, dtype=dt)

        def consume(lo, hi, out):
            step_flat[lo:hi] = out[:, 0] * torch.exp(out[:, 1] * self.exp_mult)

        groups = None
        if p.dim() > 2:
            gsize = shape[-1] * shape[-2]
            groups = (torch.arange(n, dtype=torch.int64) // gsize, n // gsize, gsize)
        st["second_moment"] = _feature_moments_and_apply(n, self.FEAT, build, 1e-9, self._mlp, consume, groups)
        self._tail(p, step_flat.view(shape), st)

    def _tail(self, p, step, st):
        """Newton-Schulz, the second-moment normaliser over the last two axes, the update (CELO2_cuda.py:331-339)."""
        st["raw_step"] = step.clone()
        if self.orthogonalize:
            step = newton_schulz(step, *self.ns)
        ms = torch.mean(step ** 2, dim=(-2, -1), keepdim=True)
        step = step * torch.rsqrt(1e-9 + ms)
        step = step * self.rmsmult
        p.add_(step + self.wd * p, alpha=-self.lr)


# --------------------------------------------------------------------------------------
# VeLO
# --------------------------------------------------------------------------------------
def fractional_tanh_embed(x: float) -> torch.Tensor:
    ts = torch.tensor([0.03, 0.1, 0.2, 0.4, 0.6, 0.8, 0.9, 1.0, 1.1], dtype=torch.float32)
    return torch.tanh((torch.tensor(x, dtype=torch.float32) - ts) * 10)


def clip_log_abs(v, scale=1.0):
    return torch.clamp(torch.log(1e-8 + torch.abs(v * scale)), -5, 5) * 0.5


class LossBuffer:
    """``BufferLossAccumulators`` (velo_cuda.py:165-211) on fp32 CPU tensors."""

    def __init__(self, num_steps):
        halflife = torch.logspace(1, torch.log10(torch.tensor(num_steps, dtype=torch.float32)), 10)
        self.decays = torch.exp(-1.0 / halflife)
        self.means = torch.zeros(10, dtype=torch.float32)
        self.iteration = torch.tensor(0, dtype=torch.int32)
        self.running_min = 999999999999.0 * torch.ones(10, dtype=torch.float32)

    def update(self, loss):
        loss = torch.as_tensor(loss, dtype=torch.float32)
        d = self.decays
        cor = self.means / (1 - d ** (self.iteration + 1))
        approx_max = torch.where(self.iteration == 0, loss, torch.max(cor))
        loss = torch.minimum(torch.abs(approx_max) * 2, loss)
        self.means = self.means * d + loss * (1.0 - d)
        cor = self.means / (1 - d ** (self.iteration + 1))
        self.running_min = torch.minimum(self.running_min, cor)
        self.iteration = self.iteration + 1

    def features(self):
        cor = self.means / (1 - self.decays ** self.iteration)
        approx_max, cor_lo, rmin = cor[1:], cor[:-1], self.running_min[:-1]
        den = torch.maximum(torch.tensor(1e-8), approx_max - rmin)
        f = torch.clamp((cor_lo - rmin) / den - 1.0, -1, 1)
        return torch.where(self.iteration <= 2, f * 0, f)


class VeLOOracle:
    """One ``VeLO_CUDA.step(loss)``.

    ``rnn``: dict with ``mix2_w[H,30] mix2_b[H] fmix_w[H,30] fmix_b[H] lstm_w[4H,2H]
    lstm_b[4H] ctrl_w[B,H] ctrl_b[B] step_w[1,H] step_b[1] h0[1,H] c0[1,H]``;
    ``bank``: ``[B,159]`` in the column order input_weights(4x30) | input_bias |
    hidden_weights | hidden_bias | output_weights(3x4) | output_bias.
    """

    FEAT = 30

    def __init__(
        self,
        rnn: Dict[str, torch.Tensor],
        bank: torch.Tensor,
        shapes: Sequence[Tuple[int, ...]],
        lr=1e-3,
        exp_mult=0.001,
        step_mult=0.001,
        weight_decay=0.0,
        num_steps=10000,
        variant="cuda",
        dtype=torch.float32,
        device="cpu",
        ref_kernel=None,
    ):
        self.dtype = dtype
        self.device = torch.device(device)
        self.ref_kernel = ref_kernel  # velo_cuda_kernel.velo_kernel_simple of the reference, or None
        self.rnn = {k: v.detach().to(dtype).to(self.device) for k, v in rnn.items()}
        self.bank = bank.detach().to(dtype).to(self.device)
        self.lr, self.exp_mult, self.step_mult, self.wd = lr, exp_mult, step_mult, weight_decay
        self.num_steps = num_steps
        zero3, zero1 = (0.0, 0.0, 0.0), (0.0,)
        self.beta_m = decay_reparam((0.9, 0.99, 0.999), zero3).to(self.device)
        self.beta_rms = decay_reparam((0.999,), zero1).to(self.device)
        self.beta_fac = decay_reparam((0.9, 0.99, 0.999), zero3).to(self.device)
        self.variant = Variant(variant)
        self.loss_buffer = LossBuffer(num_steps)
        self.group_step = 0
        self.state = []
        for idx, shape in enumerate(shapes):
            shape = tuple(shape)
            st = {"layer_idx": idx}
            st["mom"] = torch.zeros((3,) + shape, dtype=dtype, device=self.device)
            st["rms"] = torch.zeros((1,) + shape, dtype=dtype, device=self.device)
            fd = factored_dims_velo(shape)
            if fd is not None:
                dc, dr = fd
                rs, cs = list(shape), list(shape)
                rs[dr], cs[dc] = 1, 1
                st["fac_vec_row"] = torch.zeros([3] + rs, dtype=dtype, device=self.device)
                st["fac_vec_col"] = torch.zeros([3] + cs, dtype=dtype, device=self.device)
                st["fac_vec_v"] = torch.zeros(0, dtype=dtype, device=self.device)
            else:
                st["fac_vec_row"] = torch.zeros(0, dtype=dtype, device=self.device)
                st["fac_vec_col"] = torch.zeros(0, dtype=dtype, device=self.device)
                st["fac_vec_v"] = torch.zeros((3,) + shape, dtype=dtype, device=self.device)
            rank = sum(1 for d in shape if d > 1)
            st["rank_onehot"] = torch.nn.functional.one_hot(torch.tensor(rank), num_classes=5).to(dtype).to(self.device)
            self.state.append(st)
        T = len(shapes)
        self.lstm_hidden_state = (self.rnn["h0"].repeat(T, 1), self.rnn["c0"].repeat(T, 1))

    # ---- per-tensor LSTM input (velo_cuda.py:213-252) ----
    def _tensor_features(self, p, st, fraction_left, loss_features):
        dt = self.dtype
        norm = torch.rsqrt(torch.clamp(torch.mean(p.to(dt) ** 2), min=1e-9))
        m = st["mom"].reshape(3, -1) * norm
        rms = st["rms"].reshape(1, -1) * norm
        mean_m = m.mean(dim=1, keepdim=True)
        var_m = ((m - mean_m) ** 2).mean(dim=1)
        mean_rms = rms.mean(dim=1)
        var_rms = ((rms - mean_m) ** 2).mean(dim=1)
        out = torch.empty(30, dtype=dt, device=self.device)
        out[0:9] = fraction_left
        out[9:18] = loss_features
        out[18:19] = clip_log_abs(mean_rms, 10.0)
        out[19:24] = st["rank_onehot"]
        out[24:27] = clip_log_abs(var_m, 10.0)
        out[27:30] = clip_log_abs(var_rms, 10.0)
        return out

    def _rnn_forward(self, x, state):
        """VeLO_RNN.py:110-135 with the LSTM cell of VeLO_RNN.py:43-66."""
        r = self.rnn
        pooled = torch.relu(x @ r["mix2_w"].T + r["mix2_b"]).max(dim=0, keepdim=True).values
        x = x @ r["fmix_w"].T + r["fmix_b"] + pooled
        h_prev, c_prev = state
        gates = torch.cat((x, h_prev), dim=-1) @ r["lstm_w"].T + r["lstm_b"]
        i, g, f, o = gates.chunk(4, -1)
        c = torch.sigmoid(f + 1) * c_prev + torch.sigmoid(i) * torch.tanh(g)
        h = torch.sigmoid(o) * torch.tanh(c)
        controls = h @ r["ctrl_w"].T + r["ctrl_b"]
        lr_mult = (h @ r["step_w"].T + r["step_b"]).squeeze(-1)
        return controls, lr_mult, (h, c)

    def step(self, params, grads, loss):
        dt = self.dtype
        self.loss_buffer.update(loss)
        loss_feat = self.loss_buffer.features().to(dt).to(self.device)
        fraction_left = fractional_tanh_embed(self.group_step / self.num_steps).to(dt).to(self.device)
        feats = [self._tensor_features(p, st, fraction_left, loss_feat) for p, st in zip(params, self.state)]
        x = torch.flip(torch.stack(feats), [0])
        self.rnn_inputs = x
        controls, lr_mult, self.lstm_hidden_state = self._rnn_forward(x, self.lstm_hidden_state)
        self.controls, self.lr_mult = controls, lr_mult
        self.group_step += 1
        for p, g0, st in zip(params, grads, self.state):
            g = torch.clip(g0.to(dt), -1000.0, 1000.0)
            self._step_tensor(p, g, st, controls, lr_mult)

    def _step_tensor(self, p, g, st, controls, lr_mult):
        dt = self.dtype
        shape = tuple(p.shape)
        n = p.numel()
        layer = st["layer_idx"]
        st["mom"].lerp_(g[None, ...], 1 - _lead(self.beta_m, g.dim()).to(dt))
        st["rms"].lerp_(g[None, ...] ** 2, 1 - _lead(self.beta_rms, g.dim()).to(dt))
        grad_sqr = torch.square(g) + 1e-30
        fd = factored_dims_velo(shape)
        if fd is not None:
            dc, dr = fd
            fac_r, fac_c, rf, cf = _update_factored(st, grad_sqr, fd, self.beta_fac, "fac_vec_row", "fac_vec_col", dc + 1)
            rf_g = rf_m = _bcast_flat(rf, shape)
            cfb = _bcast_flat(cf, shape)
            fr, fc = _bcast_flat(fac_r, shape), _bcast_flat(fac_c, shape)
        else:
            st["fac_vec_v"].lerp_(grad_sqr[None, ...], 1 - _lead(self.beta_fac, g.dim()).to(dt))
            fr = fc = st["fac_vec_v"].reshape(3, -1)
            rf_g = safe_rsqrt(fr + 1e-9)
            rf_m = torch.pow(fr, -0.5) if self.variant.naive else rf_g
            cfb = None

        w = (controls[-(1 + layer)][:, None] * self.bank).mean(0) * 100.0
        w_in, b_in = w[0:120].view(4, 30), w[120:124]
        w_h, b_h = w[124:140].view(4, 4), w[140:144]
        w_out, b_out = w[144:156].view(3, 4), w[156:159]
        st["mlp_weights"] = w.clone()

        if self.ref_kernel is not None:
            # velo_cuda.py:694-755: factors from the updated accumulators, then the reference's fused kernel
            if fd is not None:
                row_factor, col_factor, vr, vc, kdc, kdr, vector_like = rf, cf, fac_r, fac_c, fd[0], fd[1], 0
            else:
                vr = vc = st["fac_vec_v"]
                row_factor = safe_rsqrt(vr + 1e-9)
                col_factor, kdc, kdr, vector_like = torch.ones_like(row_factor), 0, 0, 1
            second = torch.zeros(self.FEAT, dtype=dt, device=self.device)
            self.ref_kernel(g.contiguous(), p, st["mom"], st["rms"], row_factor.contiguous(), col_factor.contiguous(), vr, vc,
                            second, w_in.contiguous(), b_in.contiguous(), w_h.contiguous(), b_h.contiguous(),
                            w_out.contiguous(), b_out.contiguous(), float(self.lr * float(lr_mult[-(1 + layer)])),
                            float(self.step_mult), float(self.exp_mult), 1e-6, float(self.wd), int(kdc), int(kdr),
                            int(vector_like))
            st["second_moment"] = second
            return

        gf, pf = g.reshape(-1), p.reshape(-1)
        m = st["mom"].reshape(3, -1)
        v = st["rms"].reshape(-1)

        def build(lo, hi):
            f = torch.empty(hi - lo, self.FEAT, dtype=dt)
            gg = gf[lo:hi]
            f[:, 0] = gg
            f[:, 1] = torch.clamp(gg, -0.1, 0.1)
            f[:, 2] = pf[lo:hi]
            f[:, 3:6] = m[:, lo:hi].T
            f[:, 6] = v[lo:hi]
            rs = torch.rsqrt(v[lo:hi] + 1e-6)
            f[:, 7:10] = (m[:, lo:hi] * rs).T
            f[:, 10] = rs
            fg = rf_g[:, lo:hi] if cfb is None else rf_g[:, lo:hi] * cfb[:, lo:hi]
            fm = rf_m[:, lo:hi] if cfb is None else rf_m[:, lo:hi] * cfb[:, lo:hi]
            f[:, 11:14] = (fg * gg).T
            f[:, 14] = gg * rs
            f[:, 15:18] = fr[:, lo:hi].T
            f[:, 18:21] = fc[:, lo:hi].T
            f[:, 21:24] = torch.rsqrt(fr[:, lo:hi] + 1e-8).T
            f[:, 24:27] = torch.rsqrt(fc[:, lo:hi] + 1e-8).T
            f[:, 27:30] = (fm * m[:, lo:hi]).T
            return f

        def mlp(x):
            h = torch.relu(x @ w_in.T + b_in)
            h = torch.relu(h @ w_h.T + b_h)
            return h @ w_out.T + b_out

        if self.variant.naive:
            # VeLO_naive scales by lr_mult and group lr separately and decays with the group lr.
            lr_eff, wd_lr = self.lr * lr_mult[-(1 + layer)], self.lr
        else:
            lr_eff = self.lr * float(lr_mult[-(1 + layer)])
            wd_lr = lr_eff
        param_scale = torch.sqrt(torch.mean(p.to(dt) ** 2) + 1e-9)

        def consume(lo, hi, out):
            upd = param_scale * out[:, 0] * torch.exp(out[:, 1] * self.exp_mult) * self.step_mult
            pf[lo:hi] -= lr_eff * upd
            if self.wd > 0:
                pf[lo:hi] -= self.wd * wd_lr * pf[lo:hi]

        st["second_moment"] = _feature_moments_and_apply(n, self.FEAT, build, 1e-5, mlp, consume)


def rnn_weights_from_module(rnn_module) -> Dict[str, torch.Tensor]:
    """Pull the dict ``VeLOOracle`` wants out of a ``VeLORNN``-shaped module."""
    sd = rnn_module.state_dict()
    return {
        "mix2_w": sd["mix_layer2.weight"],
        "mix2_b": sd["mix_layer2.bias"],
        "fmix_w": sd["final_mix_layer.weight"],
        "fmix_b": sd["final_mix_layer.bias"],
        "lstm_w": sd["lstm.linear.weight"],
        "lstm_b": sd["lstm.linear.bias"],
        "ctrl_w": sd["rnn_to_controls.weight"],
        "ctrl_b": sd["rnn_to_controls.bias"],
        "step_w": sd["step_size.weight"],
        "step_b": sd["step_size.bias"],
        "h0": sd["lstm_init_state.0"],
        "c0": sd["lstm_init_state.1"],
    }


def bank_from_module(mlp_module) -> torch.Tensor:
    """``[B,159]`` bank matrix from a ``VeLOMLP``-shaped module's state dict."""
    sd = mlp_module.state_dict()
    keys = ["input_weights_", "input_bias_", "hidden_weights_.0", "hidden_bias_.0", "output_weights_", "output_bias_"]
    return torch.cat([sd[k].reshape(sd[k].shape[0], -1) for k in keys], dim=1)
