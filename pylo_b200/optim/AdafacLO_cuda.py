"""AdafacLO_CUDA and ELO_CUDA on the B200 kernels.

Drop-in for pylo/optim/AdafacLO_cuda.py:76-288 and pylo/optim/ELO_cuda.py:54-288:
same constructor arguments, group keys and per-parameter state (``step`` as a
0-d CPU float64 tensor, ``exp_avg_sq_r``, ``exp_avg_sq_c``, ``exp_avg_sq``,
``exp_avg``), so ``state_dict()`` round-trips with the reference.

Two behaviours of the reference CUDA classes are kept on purpose because this
class replaces them, not the naive ones: ``row_col_mean`` is taken over the
decay axis for 2-D tensors (AdafacLO_cuda.py:342-343), and tensors with fewer
than two dims use ``safe_rsqrt(v + 1e-9)`` for both factored features
(AdafacLO_cuda.py:358-360).  For tensors with three or more dims the reference
kernel indexes the factor vectors as if the tensor were 2-D
(learned_optimizer.cu:70-86); here they are indexed by the element's true
coordinates.

``mlp_precision`` (an addition) selects how the network's two hidden layers are
evaluated on factored 2-D tensors: ``"3xtf32"`` (default) as tcgen05 tensor-core
products with every operand split into a high and a low TF32 part, three
products per layer, which reproduces the fp32 result to ~3e-7 of a dot
product's magnitude; ``"fp32"`` as scalar fp32 FMAs on the CUDA cores, the
arithmetic of the reference kernel.  Both meet the same parity bounds.
"""

from __future__ import annotations

from typing import Optional, Union

import torch
from torch.optim import Optimizer

from .. import _lib as L
from ..models.Meta_MLP import MetaMLP
from ..plan import GradNorm, LoPlan, LoTensor, current_stream_ptr, one_minus
from ._common import factored_dims_sorted, require_cuda_param


def _decay_to_param(x):
    return torch.log(1 - x) / 10.0


def _param_to_decay(x):
    return 1 - torch.exp(x * 10.0)


class _AdafacFamily(Optimizer):
    _name = "AdafacLO_CUDA"
    _elo = False

    def _finish_init(self, network: MetaMLP):
        net = network.network
        if not (hasattr(net, "input") and hasattr(net, "linear_0") and hasattr(net, "output")) or hasattr(net, "linear_1"):
            raise ValueError(f"{self._name} kernel only supports the 39->32->32->2 MetaMLP (hidden_layers=1).")
        flat = network.flat_weights()
        if tuple(flat[0].shape) != (32, 39):
            raise ValueError(f"{self._name} kernel only supports the 39->32->32->2 MetaMLP.")
        self._w_flat = torch.cat([t.reshape(-1) for t in flat]).to(self.device).contiguous()
        self._plans = {}
        self._gnorm = None
        if self.mlp_precision not in ("fp32", "3xtf32"):
            raise ValueError(f"mlp_precision must be 'fp32' or '3xtf32', got {self.mlp_precision!r}")
        self.process_group = None   # set (or set _sharded) when the tensors of the model are split over ranks
        self._sharded = False
        self.after_group = None     # optional callable(group index), called once a param group's kernels are enqueued
        self.before_group = None    # optional callable(group index), called before a param group's first kernel
        # fp32 values of 1 - beta, read back once (the reference evaluates them on the device every step)
        self._w_m, self._w_f = one_minus(self.beta_m), one_minus(self.beta_adafactor)
        self._w_v = one_minus(self.beta_rms)[0]

    def _init_state(self, state, p):
        """AdafacLO_cuda.py:227-256 / ELO_cuda.py:160-176."""
        shape = tuple(p.shape)
        state["step"] = torch.tensor(0.0, dtype=torch.float64)
        fd = factored_dims_sorted(shape)
        if fd is not None:
            dc, dr = fd
            r_shape, c_shape = list(shape), list(shape)
            r_shape[dr], c_shape[dc] = 1, 1
            state["exp_avg_sq_r"] = p.new_zeros([3] + r_shape)
            state["exp_avg_sq_c"] = p.new_zeros([3] + c_shape)
        else:
            state["exp_avg_sq_r"] = p.new_zeros((3,) + shape)
            state["exp_avg_sq_c"] = p.new_zeros((3,) + shape)
        state["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.preserve_format)
        state["exp_avg"] = p.new_zeros((3,) + shape)

    def load_state_dict(self, state_dict):
        super().load_state_dict(state_dict)
        self._plans = {}

    def add_param_group(self, param_group):
        super().add_param_group(param_group)
        self._plans = {}

    def _build_plan(self, plist):
        tensors = []
        for p in plist:
            require_cuda_param(p, self._name)
            st = self.state[p]
            if len(st) == 0:
                self._init_state(st, p)
            fd = factored_dims_sorted(tuple(p.shape))
            axis = 0
            if fd is not None:
                dc, dr = fd
                axis = dc - 1 if dc > dr else dc  # AdafacLO_cuda.py:342 (axis 0 is the decay axis)
            tensors.append(LoTensor(
                p=p.data, m=st["exp_avg"], v=st["exp_avg_sq"], fac_r=st["exp_avg_sq_r"], fac_c=st["exp_avg_sq_c"],
                fdims=fd, rcm_axis=axis, w=self._w_flat, peer_ptrs=getattr(p, "_pylo_peer_ptrs", None),
                peer_multicast=getattr(p, "_pylo_peer_multicast", False)))
        return LoPlan(L.FAM_ADAFAC, tensors, self.device, tensor_cores=(self.mlp_precision == "3xtf32"))

    def check_status(self):
        """Synchronise and raise if a tensor-core launch of an earlier step reported a timed-out wait."""
        for _, plan in self._plans.values():
            plan.check_status()

    def clear_status(self):
        """Acknowledge a reported tensor-core timeout so that the apply kernels store again."""
        for _, plan in self._plans.values():
            plan.clear_status()

    def _run_group(self, gi, group, plist, prm, lr, wd, exp_mult, step_mult, clip_norm, stream):
        sig = tuple(p.data_ptr() for p in plist)
        cached = self._plans.get(gi)
        if cached is None or cached[0] != sig:
            cached = (sig, self._build_plan(plist))
            self._plans[gi] = cached
        plan: LoPlan = cached[1]
        plan._poll_status()  # refuse the step before any state (the step counters included) is advanced
        steps = []
        for p in plist:
            st = self.state[p]["step"]
            st += 1
            steps.append(float(st) - 1.0)
        plan.set_field("lr", lr)
        plan.set_field("wd", wd)
        plan.set_field("exp_mult", exp_mult)
        plan.set_field("step_mult", step_mult)
        plan.set_field("clip_norm", clip_norm)
        plan.refresh([p.grad for p in plist], steps=steps)
        if self.before_group is not None:
            self.before_group(gi)
        plan.run_front(prm, stream)
        plan.run_back(prm, stream)
        if self.after_group is not None:
            self.after_group(gi)

    def _params_struct(self, gnorm_ptr, wd_mode, nan_to_num):
        prm = L.StepParams()
        prm.family = L.FAM_ADAFAC
        prm.nan_to_num, prm.wd_mode = int(nan_to_num), int(wd_mode)
        for k in range(3):
            prm.w_m[k], prm.w_f[k] = self._w_m[k], self._w_f[k]
        prm.w_v = self._w_v
        prm.eps_v, prm.eps_feat, prm.eps_norm = 1e-30, 1e-6, 1e-5
        prm.clip_val = float("inf")
        prm.gnorm_sq = gnorm_ptr
        return prm


class AdafacLO_CUDA(_AdafacFamily):
    """small_fc_lopt / AdafacLO learned optimizer (https://arxiv.org/abs/2203.11860)."""

    _name = "AdafacLO_CUDA"

    def __init__(self, params, lr: float = 1.0, min_dim_size_to_factor: int = 32, decay_rate: float = 0.8,
                 decay_offset: int = 0, beta2_cap: float = 0.999, initial_momentum_decays=(0.9, 0.99, 0.999),
                 initial_rms_decays=(0.999,), initial_adafactor_decays=(0.9, 0.99, 0.999),
                 momentum_decays=[0.15216392, 0.14245212, 0.06812963], rms_decays=[0.01079706],
                 adafactor_decays=[0.18621896, -0.10864615, -0.06185547],
                 momentum_dtype: Union[str, torch.dtype] = torch.float32, eps: Optional[float] = None,
                 weight_decay: float = 0.0, clipping_threshold: Optional[float] = None,
                 max_grad_norm: Optional[float] = None, unscaled_wd: bool = False, step_mult: float = 0.01,
                 exp_mult: float = 0.001, load_from_file: Optional[str] = None, *, foreach: Optional[bool] = False,
                 hf_key: Optional[str] = "btherien/mulo", network: Optional[MetaMLP] = None,
                 mlp_precision: str = "3xtf32"):
        if isinstance(momentum_dtype, str):
            if momentum_dtype not in ("float32", "float16", "bfloat16"):
                raise AssertionError(f"{momentum_dtype} dtype not supported")
            momentum_dtype = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}[momentum_dtype]
        # Accepted and recorded in the group defaults exactly as the reference does (AdafacLO_cuda.py:109-118,122-135).
        # The reference class then keeps the momentum in the gradient's dtype all the same: its state is allocated with
        # p.grad.new_zeros (AdafacLO_cuda.py:256) and the branch that would cast is switched off (AdafacLO_cuda.py:364-373).
        # So do we: exp_avg is fp32 whatever this argument says, and state_dict() round-trips with the reference.
        if foreach:
            raise NotImplementedError("foreach=True is not implemented (neither is it in the reference)")
        if not torch.cuda.is_available():
            raise RuntimeError("AdafacLO_CUDA requires a CUDA device.")
        defaults = dict(lr=lr, min_dim_size_to_factor=min_dim_size_to_factor, decay_rate=decay_rate,
                        decay_offset=decay_offset, beta2_cap=beta2_cap, momentum_dtype=momentum_dtype, eps=eps,
                        weight_decay=weight_decay, clipping_threshold=clipping_threshold, max_grad_norm=max_grad_norm,
                        unscaled_wd=unscaled_wd, foreach=foreach)
        super().__init__(params, defaults)
        self.device = torch.device("cuda")
        dev = self.device
        momentum_decays = torch.tensor(momentum_decays, device=dev)
        rms_decays = torch.tensor(rms_decays, device=dev)
        adafactor_decays = torch.tensor(adafactor_decays, device=dev)
        # `network=` is an addition: the reference always goes to the hub (AdafacLO_cuda.py:141)
        self.metamlp = (network if network is not None else MetaMLP.from_pretrained(hf_key)).to(dev)
        if load_from_file:
            loaded = torch.load(load_from_file)
            self.metamlp.load_state_dict(loaded["state_dict"])
            momentum_decays = loaded["decays"]["momentum_decays"]
            rms_decays = loaded["decays"]["rms_decays"]
            adafactor_decays = loaded["decays"]["adafactor_decays"]
        for prm in self.metamlp.parameters():
            prm.requires_grad = False

        def reparam(initial, offset):
            return torch.clip(_param_to_decay(_decay_to_param(torch.tensor(initial, device=dev)) + offset), 0.0, 1.0)

        self.beta_m = reparam(initial_momentum_decays, momentum_decays)
        self.beta_rms = reparam(initial_rms_decays, rms_decays)
        self.beta_adafactor = reparam(initial_adafactor_decays, adafactor_decays)
        self.step_mult, self.exp_mult = step_mult, exp_mult
        self.mlp_precision = mlp_precision
        self._finish_init(self.metamlp)

    def __setstate__(self, state):
        super().__setstate__(state)
        for group in self.param_groups:
            group.setdefault("foreach", None)
            for p in group["params"]:
                st = self.state.get(p, {})
                if len(st) != 0 and not torch.is_tensor(st["step"]):
                    st["step"] = torch.tensor(float(st["step"]), dtype=torch.float64)
        self._plans = {}

    @torch.no_grad()
    def step(self, loss=None):
        stream = current_stream_ptr()
        for gi, group in enumerate(self.param_groups):
            if group["max_grad_norm"] is not None:
                for p in group["params"]:
                    torch.nn.utils.clip_grad_norm_(p, group["max_grad_norm"])  # per tensor, as AdafacLO_cuda.py:214-215
            plist = [p for p in group["params"] if p.grad is not None]
            if not plist:
                # a sharded step hangs collectives on this hook: every rank must reach it for every group, in order,
                # also a rank that owns nothing of the group
                if self.after_group is not None:
                    self.after_group(gi)
                continue
            if any(p.grad.is_sparse for p in plist):
                raise RuntimeError("Sparse gradients not supported")
            wd = float(group["weight_decay"])
            prm = self._params_struct(None, wd_mode=1 if wd > 0 else 0, nan_to_num=False)
            if group["eps"] is not None:
                prm.eps_v = float(group["eps"])
            self._run_group(gi, group, plist, prm, float(group["lr"]), wd, self.exp_mult, self.step_mult, 0.0, stream)
        return loss


class ELO_CUDA(_AdafacFamily):
    """ELO (Adafactor-MLP) learned optimizer: raw decays, no step_mult, weight decay against the pre-step value."""

    _name = "ELO_CUDA"
    _elo = True

    def __init__(self, params, lr=0.001, exp_mult=0.001, weight_decay=0.0, hidden_size=32, hidden_layers=1,
                 initial_momentum_decays=(0.9, 0.99, 0.999), initial_rms_decays=(0.999,),
                 initial_adafactor_decays=(0.9, 0.99, 0.999), clip_grad=False, clip_norm=1.0,
                 hf_key: Optional[str] = "DiamondXL/elo", checkpoint_path: Optional[str] = None,
                 network: Optional[MetaMLP] = None, mlp_precision: str = "3xtf32"):
        if not torch.cuda.is_available():
            raise RuntimeError("ELO_CUDA requires a CUDA device.")
        self.device = torch.device("cuda")
        dev = self.device
        super().__init__(params, dict(lr=lr, exp_mult=exp_mult, weight_decay=weight_decay, clip_grad=clip_grad,
                                      clip_norm=clip_norm))
        clamp = lambda xs: torch.clamp(torch.tensor(xs, dtype=torch.float32, device=dev), 0.0, 1.0)
        self.beta_m, self.beta_rms, self.beta_adafactor = clamp(initial_momentum_decays), clamp(initial_rms_decays), clamp(initial_adafactor_decays)
        if network is not None:
            self.network = network
        elif checkpoint_path is not None:
            self.network = MetaMLP(input_size=39, hidden_size=hidden_size, hidden_layers=hidden_layers)
            self.network.load_state_dict(torch.load(checkpoint_path, map_location="cpu"))
        elif hf_key is not None:
            self.network = MetaMLP.from_pretrained(hf_key)
        else:
            self.network = MetaMLP(input_size=39, hidden_size=hidden_size, hidden_layers=hidden_layers)
        self.network = self.network.to(dev)
        for prm in self.network.parameters():
            prm.requires_grad = False
        self.mlp_precision = mlp_precision
        self._finish_init(self.network)

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
            plist = [p for p in group["params"] if p.grad is not None]
            if not plist:
                # a sharded step hangs collectives on this hook: every rank must reach it for every group, in order,
                # also a rank that owns nothing of the group
                if self.after_group is not None:
                    self.after_group(gi)
                continue
            if any(p.grad.is_sparse for p in plist):
                raise RuntimeError("Sparse gradients not supported")
            wd = float(group["weight_decay"])
            prm = self._params_struct(gnorm_ptr, wd_mode=2 if wd > 0 else 0, nan_to_num=True)
            clip_norm = float(group["clip_norm"]) if group["clip_grad"] else 0.0
            self._run_group(gi, group, plist, prm, float(group["lr"]), wd, float(group["exp_mult"]), 1.0, clip_norm, stream)
        return loss
