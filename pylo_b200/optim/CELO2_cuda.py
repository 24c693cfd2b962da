"""CELO2_CUDA and ELO_CELO2_CUDA on the B200 kernels.

Drop-in for the reference classes of the same names
(pylo/optim/CELO2_cuda.py:54-341, pylo/optim/ELO_CELO2_cuda.py:39-298): same
constructor arguments, param-group keys, per-parameter state keys and shapes
(``mom (3,)+shape``, ``rms shape``, ``fac_r``, ``fac_c``; for the independent
AdamW branch ``exp_avg``, ``exp_avg_sq``, ``adam_step``), hence the same
``state_dict`` / resume format.

What differs is where the work runs.  The reference does the accumulator
updates with ~10 torch ops per tensor and then calls a two-kernel extension per
tensor.  Here every tensor of a param group goes through one multi-tensor
launch per phase: row/column sums of g^2, factor update, fused EMA + feature
moments, normaliser folding, network + raw step; then Newton-Schulz (still
``torch.matmul``), and one fused kernel pair for the final normalise-and-apply.
The global-norm clip factor is computed and consumed on the device, so the step
has no host synchronisation.
"""

from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np
import torch
from torch.optim import Optimizer

from .. import _lib as L
from ..models.CELO2_MLP import CELO2MLP
from ..plan import GradNorm, LoPlan, LoTensor, current_stream_ptr, one_minus
from ._common import (ItemPlan, factored_dims_argsort, newton_schulz, newton_schulz_eligible, newton_schulz_tc,
                      require_cuda_param)

_IN, _HID = 30, 8


class _Celo2Family(Optimizer):
    _shared_adam = False
    _name = "CELO2_CUDA"

    def _setup(self, params, defaults, initial_momentum_decays, initial_rms_decays, initial_adafactor_decays,
               ns_coeffs, ns_iters, ns_eps, ff_hidden_size, ff_hidden_layers, hf_key, checkpoint_path, network):
        if not torch.cuda.is_available():
            raise RuntimeError(f"{self._name} requires a CUDA device.")
        self.device = torch.device("cuda")
        Optimizer.__init__(self, params, defaults)
        dev = self.device
        clamp = lambda xs: torch.clamp(torch.tensor(xs, dtype=torch.float32, device=dev), 0.0, 1.0)
        self.beta_m, self.beta_rms, self.beta_fac = clamp(initial_momentum_decays), clamp(initial_rms_decays), clamp(initial_adafactor_decays)
        self.n_mom, self.n_rms, self.n_fac = (int(b.shape[-1]) for b in (self.beta_m, self.beta_rms, self.beta_fac))
        if self.n_mom != 3 or self.n_fac != 3:
            raise ValueError(f"{self._name} kernels are built for 3 momentum and 3 adafactor decays")
        self.ns_coeffs = tuple(float(c) for c in ns_coeffs)
        self.ns_iters, self.ns_eps = ns_iters, ns_eps
        # weights: explicit network > local checkpoint > hub > random init (CELO2_cuda.py:141-155)
        if network is not None:
            self.network = network
        elif checkpoint_path is not None:
            self.network = CELO2MLP(hidden_size=ff_hidden_size, hidden_layers=ff_hidden_layers)
            self.network.load_state_dict(torch.load(checkpoint_path, map_location="cpu"))
        elif hf_key is not None:
            self.network = CELO2MLP.from_pretrained(hf_key)
        else:
            self.network = CELO2MLP(hidden_size=ff_hidden_size, hidden_layers=ff_hidden_layers)
        self.network = self.network.to(dev)
        if sum(self.network.feature_dims) != _IN:
            raise ValueError(f"{self._name} kernel expects feature_dims summing to {_IN}, got {sum(self.network.feature_dims)}.")
        if self.network.hidden_size != _HID or len(self.network.dense_w) != 2:
            raise ValueError(f"{self._name} kernel only supports ff_hidden_size=8, ff_hidden_layers=2.")
        self.w_in, self.b_in, self.w_h, self.b_h, self.w_out, self.b_out = (
            t.to(dev) for t in self.network.flat_weights())
        self._w_flat = torch.cat([t.reshape(-1) for t in (self.w_in, self.b_in, self.w_h, self.b_h, self.w_out, self.b_out)]).contiguous()
        self._plans = {}
        self._gnorm = None
        # "3xtf32" (default): the Newton-Schulz products on the tensor cores (this library's kernel, operands split
        # into TF32 high and low parts, as accurate as fp32 products); "fp32": torch.matmul, the reference's arithmetic
        self.ns_precision = "3xtf32"
        #: device word the Newton-Schulz kernel ORs 4 into if one of its bounded waits ran out
        self._ns_status = torch.zeros(1, dtype=torch.int32, device=dev)
        #: Newton-Schulz launches of this library since construction (for the benchmark's launch count)
        self.extra_launches = 0
        self.process_group = None   # set (or set _sharded) when the tensors of the model are split over ranks
        self._sharded = False
        self.after_group = None     # optional callable(group index), called once a param group's kernels are enqueued
        self.before_group = None    # optional callable(group index), called before a param group's first kernel
        # fp32 values of 1 - beta, read back once (the reference evaluates them on the device every step)
        self._w_m, self._w_f = one_minus(self.beta_m), one_minus(self.beta_fac)
        self._w_v = float(1 - self.beta_rms[-1])
        self._b1_shared, self._b2_shared = float(self.beta_m[0]), float(self.beta_rms[-1])

    # ------------------------------------------------------------------ state
    def _init_lo_state(self, state, p):
        shape = tuple(p.shape)
        dev = p.device
        state["mom"] = torch.zeros((self.n_mom,) + shape, device=dev)
        state["rms"] = torch.zeros(shape, device=dev)
        fd = factored_dims_argsort(shape)
        if fd is not None:
            dc, dr = fd
            r_shape, c_shape = list(shape), list(shape)
            r_shape[dr], c_shape[dc] = 1, 1
            state["fac_r"] = torch.zeros([self.n_fac] + r_shape, device=dev)
            state["fac_c"] = torch.zeros([self.n_fac] + c_shape, device=dev)

    def load_state_dict(self, state_dict):
        super().load_state_dict(state_dict)
        self._plans = {}

    def add_param_group(self, param_group):
        super().add_param_group(param_group)
        self._plans = {}

    # ------------------------------------------------------------------ planning
    def _build_group_plan(self, gi, group, plist):
        lo, adam = [], []
        for p in plist:
            require_cuda_param(p, self._name)
            st = self.state[p]
            is_1d = p.dim() <= 1 or group["is_embedding"]
            to_adam = group["use_adamw_for_1d"] and is_1d
            if self._shared_adam:
                if len(st) == 0:
                    self._init_lo_state(st, p)
            elif to_adam:
                if "exp_avg" not in st:
                    st["exp_avg"] = torch.zeros_like(p)
                    st["exp_avg_sq"] = torch.zeros_like(p)
                    st["adam_step"] = 0
            else:
                if p.dim() < 2:
                    raise ValueError(f"{self._name}: tensors with fewer than 2 dims need use_adamw_for_1d=True")
                if "mom" not in st:
                    self._init_lo_state(st, p)
            (adam if to_adam else lo).append(p)
        plan = {"lo_params": lo, "adam_params": adam, "lo": None, "adam": None, "post": None}
        if lo:
            # raw-step buffers of equally shaped tensors are slices of one stacked tensor, so that
            # Newton-Schulz runs once per shape as a batched product instead of once per tensor
            by_shape = {}
            for ti, p in enumerate(lo):
                by_shape.setdefault(tuple(p.shape), []).append(ti)
            stacks, out_of = [], {}
            for shape, members in by_shape.items():
                stacked = torch.empty((len(members),) + shape, dtype=torch.float32, device=self.device)
                stacks.append((stacked, members))
                for j, ti in enumerate(members):
                    out_of[ti] = stacked[j]
            plan["stacks"] = stacks
            tensors = []
            for ti, p in enumerate(lo):
                st = self.state[p]
                fd = factored_dims_argsort(tuple(p.shape))
                if fd is None:
                    raise ValueError(f"{self._name}: tensors with fewer than 2 dims need use_adamw_for_1d=True")
                tensors.append(LoTensor(
                    p=p.data, m=st["mom"], v=st["rms"], fac_r=st["fac_r"], fac_c=st["fac_c"], fdims=fd,
                    rcm_axis=fd[0] + 1, out=out_of[ti], w=self._w_flat, slice_last2=True))
            plan["lo"] = LoPlan(L.FAM_CELO2, tensors, self.device)
            # the tail works on matrices: the last two axes of every tensor
            post_sizes, post_owner = [], []
            for ti, p in enumerate(lo):
                mat = p.shape[-1] * p.shape[-2]
                for k in range(p.numel() // mat):
                    post_sizes.append(mat)
                    post_owner.append((ti, k * mat))
            post = ItemPlan(L.POST_DTYPE, post_sizes, self.device)
            post.owner = post_owner
            post.owner_t = np.array([t for t, _ in post_owner], dtype=np.int64)
            post.owner_off = np.array([4 * o for _, o in post_owner], dtype=np.uint64)
            post.part = torch.zeros(max(post.n_tiles, 1), dtype=torch.float32, device=self.device)
            for i, (t0, k) in enumerate(post.ranges):
                post.items["part"][i] = post.part.data_ptr() + 4 * t0
            plan["post"] = post
        if adam:
            plan["adam"] = ItemPlan(L.ADAM_DTYPE, [p.numel() for p in adam], self.device)
        return plan

    def _params_struct(self, group, gnorm_ptr):
        prm = L.StepParams()
        prm.family = L.FAM_CELO2
        prm.nan_to_num, prm.wd_mode = 0, 0
        for k in range(3):
            prm.w_m[k], prm.w_f[k] = self._w_m[k], self._w_f[k]
        prm.w_v = self._w_v
        prm.eps_v, prm.eps_feat, prm.eps_norm = 0.0, 1e-8, 1e-9
        prm.clip_val = float(group["grad_clip_val"])
        prm.gnorm_sq = gnorm_ptr
        return prm

    def check_status(self):
        """Synchronise and raise if the Newton-Schulz kernel reported a wait that ran out (its output is incomplete)."""
        if int(self._ns_status.item()) != 0:
            raise L.PyloLibError(f"{self._name}: a wait inside the Newton-Schulz kernel timed out; the step is invalid")

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self, loss=None):
        stream = current_stream_ptr()
        gnorm_ptr = None
        if any(g["clip_grad"] for g in self.param_groups):
            all_p = [p for g in self.param_groups for p in g["params"] if p.grad is not None]
            sig = tuple(p.numel() for p in all_p)
            if self._gnorm is None or self._gnorm[0] != sig:
                self._gnorm = (sig, GradNorm(sig, self.device))
            total = self._gnorm[1].run([p.grad for p in all_p], stream)
            if self.process_group is not None or (torch.distributed.is_initialized() and self._sharded):
                torch.distributed.all_reduce(total, group=self.process_group)  # each rank holds its own tensors' share
            gnorm_ptr = total.data_ptr()

        for gi, group in enumerate(self.param_groups):
            if self._shared_adam:
                # every group advances on every step, with or without gradients (ELO_CELO2_cuda.py:215-216)
                group["step"] = group.get("step", 0) + 1
            plist = [p for p in group["params"] if p.grad is not None]
            if not plist:
                # a sharded step hangs collectives on this hook: every rank must reach it for every group, in order,
                # also a rank that owns nothing of the group
                if self.after_group is not None:
                    self.after_group(gi)
                continue
            sig = tuple((p.data_ptr(), bool(group["is_embedding"]), bool(group["use_adamw_for_1d"])) for p in plist)
            cached = self._plans.get(gi)
            if cached is None or cached[0] != sig:
                cached = (sig, self._build_group_plan(gi, group, plist))
                self._plans[gi] = cached
            plan = cached[1]
            if self.before_group is not None:
                self.before_group(gi)
            prm = self._params_struct(group, gnorm_ptr)
            clip_norm = float(group["clip_norm"]) if group["clip_grad"] else 0.0
            lr = float(group["lr"])

            lo: Optional[LoPlan] = plan["lo"]
            if lo is not None:
                lo.set_field("lr", lr)
                lo.set_field("wd", group["weight_decay"])
                lo.set_field("clip_norm", clip_norm)
                lo.set_field("exp_mult", group["exp_mult"])
                lo.refresh([p.grad for p in plan["lo_params"]])
                lo.run_front(prm, stream)
                lo.run_back(prm, stream)
                post = plan["post"]
                keep = [t.out for t in lo.tensors]
                if group["orthogonalize"]:
                    for stacked, members in plan["stacks"]:
                        on_tc = self.ns_precision == "3xtf32" and newton_schulz_eligible(*stacked.shape[-2:])
                        # batches of at most ~64 M elements keep the iteration's temporaries small
                        per = max(1, (64 << 20) // max(1, stacked[0].numel()))
                        for c0 in range(0, len(members), per):
                            part = stacked[c0:c0 + per]
                            if on_tc:
                                res = newton_schulz_tc(part, self.ns_coeffs, self.ns_iters, self.ns_eps, self._ns_status, stream)
                                self.extra_launches += 3 * self.ns_iters
                            else:
                                res = newton_schulz(part, self.ns_coeffs, self.ns_iters, self.ns_eps)
                            res = res.contiguous()
                            for j, ti in enumerate(members[c0:c0 + per]):
                                keep[ti] = res[j]
                it = post.items
                base_s = np.fromiter((k.data_ptr() for k in keep), dtype=np.uint64, count=len(keep))
                base_p = np.fromiter((p.data_ptr() for p in plan["lo_params"]), dtype=np.uint64, count=len(keep))
                it["step"][:] = base_s[post.owner_t] + post.owner_off
                it["p"][:] = base_p[post.owner_t] + post.owner_off
                it["lr"][:] = lr
                it["wd"][:] = group["weight_decay"]
                it["rmsmult"][:] = group["rmsmult"]
                post.upload()
                L.check(L.lib.pylo_b200_celo2_post_sums(post.table.ptr, post.tiles.ptr, post.n_tiles, stream), "celo2_post_sums")
                L.check(L.lib.pylo_b200_celo2_post_apply(post.table.ptr, post.tiles.ptr, post.n_tiles, stream), "celo2_post_apply")
                self._keep = keep

            adam: Optional[ItemPlan] = plan["adam"]
            if adam is not None:
                it = adam.items
                keepg = []
                for i, p in enumerate(plan["adam_params"]):
                    st = self.state[p]
                    g = p.grad
                    if not (g.dtype == torch.float32 and g.is_contiguous()):
                        g = g.to(torch.float32).contiguous()
                        keepg.append(g)
                    it["g"][i], it["p"][i] = g.data_ptr(), p.data_ptr()
                    if self._shared_adam:
                        t = group["step"]
                        b1, b2 = self._b1_shared, self._b2_shared
                        it["m"][i], it["v"][i] = st["mom"].data_ptr(), st["rms"].data_ptr()
                    else:
                        st["adam_step"] += 1
                        t = st["adam_step"]
                        b1, b2 = self.adam_beta1, self.adam_beta2
                        it["m"][i], it["v"][i] = st["exp_avg"].data_ptr(), st["exp_avg_sq"].data_ptr()
                    it["bc1"][i], it["bc2"][i] = 1.0 - b1 ** t, 1.0 - b2 ** t
                it["lr"][:] = group["adam_lr_mult"] * lr
                it["wd"][:] = group["adam_weight_decay"]
                it["clip_norm"][:] = clip_norm
                adam.upload()
                eps = 1e-8 if self._shared_adam else self.adam_eps
                L.check(L.lib.pylo_b200_adamw(adam.table.ptr, adam.tiles.ptr, adam.n_tiles, int(not self._shared_adam),
                                              b1, 1 - b1, b2, 1 - b2, eps, C.byref(prm), stream), "adamw")
                self._keepg = keepg
            if self.after_group is not None:
                self.after_group(gi)
        return loss


class CELO2_CUDA(_Celo2Family):
    """CELO2 learned optimizer; 1-D / embedding tensors take an AdamW step with their own moments."""

    _shared_adam = False
    _name = "CELO2_CUDA"

    def __init__(self, params, lr=1e-3, weight_decay=0.0, adam_lr_mult=1.0, adam_weight_decay=None,
                 adam_betas=(0.9, 0.95), adam_eps=1e-8, use_adamw_for_1d=True, orthogonalize=True, clip_grad=False,
                 clip_norm=1.0, ff_hidden_size=8, ff_hidden_layers=2, initial_momentum_decays=(0.9, 0.99, 0.999),
                 initial_rms_decays=(0.95,), initial_adafactor_decays=(0.9, 0.99, 0.999), exp_mult=0.0, rmsmult=1.0,
                 param_scale_mult=False, ns_coeffs=(3.4445, -4.7750, 2.0315), ns_iters=5, ns_eps=1e-8,
                 grad_clip_val=1000.0, hf_key: Optional[str] = "DiamondXL/celo2",
                 checkpoint_path: Optional[str] = None, network: Optional[CELO2MLP] = None, ns_precision: str = "3xtf32"):
        defaults = dict(
            lr=lr, weight_decay=weight_decay, adam_lr_mult=adam_lr_mult,
            adam_weight_decay=(adam_weight_decay if adam_weight_decay is not None else weight_decay),
            use_adamw_for_1d=use_adamw_for_1d, orthogonalize=orthogonalize, clip_grad=clip_grad, clip_norm=clip_norm,
            exp_mult=exp_mult, rmsmult=rmsmult, param_scale_mult=param_scale_mult, grad_clip_val=grad_clip_val,
            is_embedding=False)
        self.adam_beta1, self.adam_beta2 = (float(b) for b in adam_betas)
        self.adam_eps = adam_eps
        self._setup(params, defaults, initial_momentum_decays, initial_rms_decays, initial_adafactor_decays,
                    ns_coeffs, ns_iters, ns_eps, ff_hidden_size, ff_hidden_layers, hf_key, checkpoint_path, network)
        if ns_precision not in ("fp32", "3xtf32"):
            raise ValueError("ns_precision must be 'fp32' or '3xtf32'")
        self.ns_precision = ns_precision


class ELO_CELO2_CUDA(_Celo2Family):
    """ELO-CELO2: CELO2 forward with ELO defaults; the AdamW branch reuses mom[0] / rms of every tensor."""

    _shared_adam = True
    _name = "ELO_CELO2_CUDA"

    def __init__(self, params, lr=1e-3, weight_decay=0.1, clip_grad=True, clip_norm=1.0, adam_lr_mult=20.0,
                 adam_weight_decay=None, use_adamw_for_1d=True, orthogonalize=True, ff_hidden_size=8,
                 ff_hidden_layers=2, initial_momentum_decays=(0.9, 0.99, 0.999), initial_rms_decays=(0.95,),
                 initial_adafactor_decays=(0.9, 0.99, 0.999), exp_mult=0.0, rmsmult=1.0, param_scale_mult=False,
                 ns_coeffs=(3.4445, -4.7750, 2.0315), ns_iters=5, ns_eps=1e-8, grad_clip_val=1000.0,
                 hf_key: Optional[str] = "DiamondXL/elo-celo2", checkpoint_path: Optional[str] = None,
                 network: Optional[CELO2MLP] = None, ns_precision: str = "3xtf32"):
        defaults = dict(
            lr=lr, weight_decay=weight_decay, adam_lr_mult=adam_lr_mult,
            adam_weight_decay=(adam_weight_decay if adam_weight_decay is not None else weight_decay),
            use_adamw_for_1d=use_adamw_for_1d, orthogonalize=orthogonalize, clip_grad=clip_grad, clip_norm=clip_norm,
            exp_mult=exp_mult, rmsmult=rmsmult, param_scale_mult=param_scale_mult, grad_clip_val=grad_clip_val,
            is_embedding=False)
        self._setup(params, defaults, initial_momentum_decays, initial_rms_decays, initial_adafactor_decays,
                    ns_coeffs, ns_iters, ns_eps, ff_hidden_size, ff_hidden_layers, hf_key, checkpoint_path, network)
        if ns_precision not in ("fp32", "3xtf32"):
            raise ValueError("ns_precision must be 'fp32' or '3xtf32'")
        self.ns_precision = ns_precision
