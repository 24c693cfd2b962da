"""VeLO_CUDA on the B200 kernels (VeLO: https://arxiv.org/abs/2211.09760).

Drop-in for pylo/optim/velo_cuda.py:255-755: same constructor arguments, the
same per-parameter state (``layer_idx``, ``mom (3,)+shape``, ``rms (1,)+shape``,
``fac_vec_row``, ``fac_vec_col``, ``fac_vec_v``, ``rank_onehot``), and a
``state_dict`` that carries ``loss_buffer``, ``lstm_hidden_state`` and
``num_steps`` like the reference's (velo_cuda.py:438-462).

One step is a fixed sequence of launches with no host synchronisation: loss
features; row/column sums of g^2; factor update; fused EMA + feature moments,
which also gathers the statistics of the *pre-update* state that the
per-tensor LSTM consumes (so the reference's extra sweep over p, mom and rms,
velo_cuda.py:213-252, costs no memory traffic here); the LSTM front end as a
handful of small batched kernels that end in the 256-way weight-bank mixing;
and the apply sweep, which reads each tensor's mixed weights and its
``lr_mult`` from device memory (the reference reads ``lr_mult`` back with
``.item()`` once per tensor, velo_cuda.py:747).
"""

from __future__ import annotations

import ctypes as C

import numpy as np
import torch
import torch.nn.functional as F
from torch.optim import Optimizer

from .. import _lib as L
from ..models.VeLO_MLP import VeLOMLP
from ..models.VeLO_RNN import VeLORNN
from ..plan import LoPlan, LoTensor, current_stream_ptr, one_minus
from ._common import factored_dims_velo, require_cuda_param


def _decay_to_param(x):
    return torch.log(1 - x) / 10.0


def _param_to_decay(x):
    return 1 - torch.exp(x * 10.0)


def fractional_tanh_embed(x: float) -> torch.Tensor:
    """tanh((x - t) * 10) for the nine time fractions of velo_cuda.py:155-162."""
    ts = torch.tensor([0.03, 0.1, 0.2, 0.4, 0.6, 0.8, 0.9, 1.0, 1.1], dtype=torch.float32)
    return torch.tanh((x - ts) * 10)


def init_loss_buffer(num_steps, device):
    """BufferLossAccumulators.init (velo_cuda.py:170-181)."""
    halflife = torch.logspace(1, torch.log10(torch.tensor(num_steps, dtype=torch.float32)), 10)
    decays = torch.exp(-1.0 / halflife)
    return {
        "means": torch.zeros(10, dtype=torch.float32, device=device),
        "iteration": torch.tensor(0, dtype=torch.int32, device=device),
        "running_min": 999999999999.0 * torch.ones(10, dtype=torch.float32, device=device),
        "decays": decays.to(device),
    }


class VeLO_CUDA(Optimizer):
    def __init__(self, params, momentum_decays=[0.0, 0.0, 0.0], rms_decays=[0.0], adafactor_decays=[0.0, 0.0, 0.0],
                 lr=1e-3, exp_mult=0.001, step_mult=0.001, input_size=30, hidden_size=4, hidden_layers=1,
                 initial_momentum_decays=(0.9, 0.99, 0.999), lstm_input_size=30, lstm_hidden_size=512,
                 param_inits=256, num_steps=10000, initial_rms_decays=(0.999,),
                 initial_adafactor_decays=(0.9, 0.99, 0.999), concat_weights=True, make_separate_weights=False,
                 split_weights=False, weight_decay=0.0, clip_grad=False, mup_lrs=None,
                 hf_key_rnn="Pauljanson002/VeLO_RNN", hf_key_mlp="Pauljanson002/VeLO_MLP", legacy=False,
                 rnn: VeLORNN = None, mlp: VeLOMLP = None, process_group=None, all_shapes=None, owned=None):
        if legacy:
            raise NotImplementedError("VeLO_CUDA(legacy=True): the reference's legacy path cannot run either "
                                      "(its processor needs arguments the step loop never passes)")
        if not torch.cuda.is_available():
            raise RuntimeError("VeLO_CUDA requires a CUDA device.")
        params = list(params)
        probe = params[0]
        if isinstance(probe, dict):
            probe["params"] = list(probe["params"])
            probe = probe["params"][0]
        if not probe.is_cuda:
            raise RuntimeError("VeLO_CUDA: parameters must live on a CUDA device (there is no CPU path)")
        self.device = probe.device
        dev = self.device

        def reparam(initial, offset):
            d = _param_to_decay(_decay_to_param(torch.tensor(initial, device=dev)) + torch.tensor(offset, device=dev))
            return torch.clip(d, 0.0, 1.0)

        defaults = dict(
            lr=lr, exp_mult=exp_mult, step_mult=step_mult,
            initial_momentum_decays=reparam(initial_momentum_decays, momentum_decays),
            lstm_hidden_size=lstm_hidden_size,
            initial_rms_decays=reparam(initial_rms_decays, rms_decays),
            initial_adafactor_decays=reparam(initial_adafactor_decays, adafactor_decays),
            param_inits=param_inits, concat_weights=concat_weights, make_separate_weights=make_separate_weights,
            input_size=input_size, hidden_size=hidden_size, hidden_layers=hidden_layers, split_weights=split_weights,
            clip_grad=clip_grad, mup_lrs=mup_lrs, weight_decay=weight_decay, legacy=legacy)
        super().__init__(params, defaults)
        self.legacy = False
        self.num_steps = num_steps
        self.loss_buffer = init_loss_buffer(num_steps, dev)
        # `rnn=` / `mlp=` are additions: the reference always goes to the hub (velo_cuda.py:338-341)
        self.rnn = (rnn if rnn is not None else VeLORNN.from_pretrained(hf_key_rnn)).to(dev)
        self.lstm_init_state = self.rnn.lstm_init_state
        self.network_stack = (mlp if mlp is not None else VeLOMLP.from_pretrained(hf_key_mlp)).to(dev)
        for prm in list(self.network_stack.parameters()) + list(self.rnn.parameters()):
            prm.requires_grad = False
        self._bank = self.network_stack.flat_bank().to(dev)
        sd = {k: v.detach().to(dev, torch.float32).contiguous() for k, v in self.rnn.state_dict().items()}
        self._rnn_w = sd
        self._H = int(sd["mix_layer2.weight"].shape[0])
        self._B = int(sd["rnn_to_controls.weight"].shape[0])
        if self._bank.shape != (self._B, 159) or sd["mix_layer2.weight"].shape[1] != 30:
            raise ValueError("VeLO_CUDA kernels are built for 30 LSTM inputs and the 30-4-4-3 per-element network")
        # Sharded use (one process per GPU, each owning whole tensors): `all_shapes` lists the shapes of ALL
        # tensors of the model in their global order, `owned` the global positions of the tensors passed
        # to this instance (same order).  The LSTM sees every tensor (it pools over them, VeLO_RNN.py:129-131),
        # so the per-tensor LSTM inputs are summed over the ranks and every rank runs the small LSTM itself.
        self._pg = process_group
        self._all_shapes = [tuple(s) for s in all_shapes] if all_shapes is not None else None
        self._owned = list(owned) if owned is not None else None
        if (self._all_shapes is None) != (self._owned is None):
            raise ValueError("VeLO_CUDA: pass all_shapes and owned together")
        self._plan = None
        g0 = self.param_groups[0]
        self._w_m, self._w_f = one_minus(g0["initial_momentum_decays"]), one_minus(g0["initial_adafactor_decays"])
        self._w_v = one_minus(g0["initial_rms_decays"])[0]
        self.init_state()

    @torch.no_grad()
    def init_state(self):
        """velo_cuda.py:357-387."""
        layer_idx = 0
        dev = self.device
        for group in self.param_groups:
            group["step"] = 0
            for p in group["params"]:
                if p.requires_grad is False:
                    continue
                st = self.state[p]
                shape = tuple(p.shape)
                if len(st) == 0:
                    st["layer_idx"] = layer_idx
                    st["mom"] = torch.zeros((3,) + shape, device=dev)
                    st["rms"] = torch.zeros((1,) + shape, device=dev)
                    fd = factored_dims_velo(shape)
                    empty = lambda: torch.tensor([], dtype=torch.float32, device=dev)
                    if fd is not None:
                        dc, dr = fd
                        r_shape, c_shape = list(shape), list(shape)
                        r_shape[dr], c_shape[dc] = 1, 1
                        st["fac_vec_row"] = torch.zeros([3] + r_shape, device=dev)
                        st["fac_vec_col"] = torch.zeros([3] + c_shape, device=dev)
                        st["fac_vec_v"] = empty()
                    else:
                        st["fac_vec_row"], st["fac_vec_col"] = empty(), empty()
                        st["fac_vec_v"] = torch.zeros((3,) + shape, device=dev)
                    rank = sum(1 for d in shape if d > 1)
                    st["rank_onehot"] = F.one_hot(torch.tensor(rank), num_classes=5).float().to(dev)
                layer_idx += 1
        if self._owned is not None:
            if len(self._owned) != layer_idx:
                raise ValueError("VeLO_CUDA: `owned` must name one global position per parameter")
            for group in self.param_groups:
                for p in group["params"]:
                    if p.requires_grad is not False:
                        self.state[p]["layer_idx"] = self._owned[self.state[p]["layer_idx"]]
            layer_idx = len(self._all_shapes)
        self.lstm_hidden_state = (
            self.lstm_init_state[0].detach().repeat(layer_idx, 1).to(dev).contiguous(),
            self.lstm_init_state[1].detach().repeat(layer_idx, 1).to(dev).contiguous(),
        )

    # ------------------------------------------------------------------ checkpointing
    def state_dict(self):
        sd = super().state_dict()
        sd["loss_buffer"] = self.loss_buffer
        sd["lstm_hidden_state"] = self.lstm_hidden_state
        sd["num_steps"] = self.num_steps
        return sd

    def load_state_dict(self, state_dict):
        state_dict = dict(state_dict)
        loss_buffer = state_dict.pop("loss_buffer")
        lstm_hidden_state = state_dict.pop("lstm_hidden_state")
        num_steps = state_dict.pop("num_steps")
        super().load_state_dict(state_dict)
        dev = self.device
        self.loss_buffer = {k: v.detach().clone().to(dev) for k, v in loss_buffer.items()}
        self.lstm_hidden_state = tuple(t.detach().clone().to(dev, torch.float32).contiguous() for t in lstm_hidden_state)
        self.num_steps = num_steps
        self._plan = None

    def add_param_group(self, param_group):
        super().add_param_group(param_group)
        self._plan = None

    # ------------------------------------------------------------------ planning
    def _build_plan(self, plist):
        dev = self.device
        T = len(self._all_shapes) if self._all_shapes is not None else len(plist)
        H, B = self._H, self._B
        f32 = dict(dtype=torch.float32, device=dev)
        buf = {
            "weights": torch.zeros(T, 160, **f32), "lr_mult": torch.zeros(T, **f32), "x_in": torch.zeros(T, 30, **f32),
            "pooled": torch.zeros(H, **f32), "xmix": torch.zeros(T, H, **f32), "gates": torch.zeros(T, 4 * H, **f32),
            "controls": torch.zeros(T, B, **f32), "loss9": torch.zeros(9, **f32), "fraction9": torch.zeros(9, **f32),
            "rank": torch.stack([self.state[p]["rank_onehot"] for p in plist]).contiguous(),
            "loss": torch.zeros(1, **f32),
        }
        # the nine time features are computed on the host (as the reference does) and cross through pinned staging
        # buffers, two in turn, so that the copy never stalls the host
        buf["frac_stage"] = [torch.zeros(9, dtype=torch.float32).pin_memory() for _ in range(2)]
        buf["frac_event"] = [None, None]
        buf["frac_turn"] = 0
        layers = [self.state[p]["layer_idx"] for p in plist]
        buf["layer_of"] = torch.tensor(layers, dtype=torch.int32, device=dev)
        tensors = []
        for i, p in enumerate(plist):
            require_cuda_param(p, "VeLO_CUDA")
            st = self.state[p]
            li = st["layer_idx"]
            if self._owned is None and li != i:
                raise RuntimeError("VeLO_CUDA: every parameter needs a gradient on every step")
            fd = factored_dims_velo(tuple(p.shape))
            common = dict(p=p.data, m=st["mom"], v=st["rms"], fdims=fd, w=buf["weights"][li], lr_mult=buf["lr_mult"][li:li + 1],
                          peer_ptrs=getattr(p, "_pylo_peer_ptrs", None),
                peer_multicast=getattr(p, "_pylo_peer_multicast", False))
            if fd is not None:
                tensors.append(LoTensor(fac_r=st["fac_vec_row"], fac_c=st["fac_vec_col"], rcm_axis=fd[0] + 1, **common))
            else:
                tensors.append(LoTensor(fac_r=st["fac_vec_v"], fac_c=None, **common))
        plan = LoPlan(L.FAM_VELO, tensors, dev)
        w = self._rnn_w
        r = L.VeloRnn()
        r.mix2_w, r.mix2_b = w["mix_layer2.weight"].data_ptr(), w["mix_layer2.bias"].data_ptr()
        r.fmix_w, r.fmix_b = w["final_mix_layer.weight"].data_ptr(), w["final_mix_layer.bias"].data_ptr()
        r.lstm_w, r.lstm_b = w["lstm.linear.weight"].data_ptr(), w["lstm.linear.bias"].data_ptr()
        r.ctrl_w, r.ctrl_b = w["rnn_to_controls.weight"].data_ptr(), w["rnn_to_controls.bias"].data_ptr()
        r.step_w, r.step_b = w["step_size.weight"].data_ptr(), w["step_size.bias"].data_ptr()
        r.bank = self._bank.data_ptr()
        for k in ("x_in", "pooled", "xmix", "gates", "controls", "weights", "lr_mult"):
            setattr(r, k, buf[k].data_ptr())
        r.T, r.H, r.B = T, H, B
        return {"plan": plan, "buf": buf, "rnn": r}

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self, loss):
        stream = current_stream_ptr()
        dev = self.device
        plist, lrs, wds, ems, sms = [], [], [], [], []
        fraction = None
        for group in self.param_groups:
            frac = group["step"] / self.num_steps
            if fraction is not None and frac != fraction:
                raise RuntimeError("VeLO_CUDA: param groups must advance in lock step")
            fraction = frac
            for p in group["params"]:
                if p.requires_grad is False:
                    continue
                if p.grad is None:
                    raise RuntimeError("VeLO_CUDA: every parameter needs a gradient on every step "
                                       "(the per-tensor LSTM sees all tensors, velo_cuda.py:399-418)")
                plist.append(p)
                lrs.append(group["lr"]); wds.append(group["weight_decay"])
                ems.append(group["exp_mult"]); sms.append(group["step_mult"])
        sig = tuple(p.data_ptr() for p in plist)
        if self._plan is None or self._plan[0] != sig:
            self._plan = (sig, self._build_plan(plist))
        ctx = self._plan[1]
        plan: LoPlan = ctx["plan"]
        buf, r = ctx["buf"], ctx["rnn"]

        # loss features (velo_cuda.py:183-211)
        if torch.is_tensor(loss):
            buf["loss"].copy_(loss.detach().reshape(-1)[:1].to(torch.float32), non_blocking=True)
        else:
            buf["loss"].fill_(float(loss))
        lb = self.loss_buffer
        L.check(L.lib.pylo_b200_velo_loss_features(lb["means"].data_ptr(), lb["iteration"].data_ptr(),
                                                   lb["running_min"].data_ptr(), lb["decays"].data_ptr(),
                                                   buf["loss"].data_ptr(), buf["loss9"].data_ptr(), stream), "velo_loss_features")
        turn = buf["frac_turn"]
        buf["frac_turn"] = turn ^ 1
        if buf["frac_event"][turn] is not None:
            buf["frac_event"][turn].synchronize()  # the copy issued two steps ago has long finished
        buf["frac_stage"][turn].copy_(fractional_tanh_embed(fraction))
        buf["fraction9"].copy_(buf["frac_stage"][turn], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        buf["frac_event"][turn] = ev

        prm = L.StepParams()
        prm.family, prm.nan_to_num, prm.wd_mode = L.FAM_VELO, 0, 3
        for k in range(3):
            prm.w_m[k], prm.w_f[k] = self._w_m[k], self._w_f[k]
        prm.w_v = self._w_v
        prm.eps_v, prm.eps_feat, prm.eps_norm = 0.0, 1e-6, 1e-5
        prm.clip_val = 1000.0
        prm.gnorm_sq = None

        plan.set_field("lr", lrs)
        plan.set_field("wd", wds)
        plan.set_field("exp_mult", ems)
        plan.set_field("step_mult", sms)
        plan.refresh([p.grad for p in plist])
        plan.run_front(prm, stream)

        h, c = self.lstm_hidden_state
        r.h, r.c = h.data_ptr(), c.data_ptr()
        sharded = self._owned is not None
        if sharded:
            buf["x_in"].zero_()
        L.check(L.lib.pylo_b200_velo_tensor_features(plan.desc.ptr, plan.n_tensors, buf["layer_of"].data_ptr(), int(r.T),
                                                     buf["rank"].data_ptr(), buf["fraction9"].data_ptr(),
                                                     buf["loss9"].data_ptr(), buf["x_in"].data_ptr(), stream),
                "velo_tensor_features")
        if sharded and torch.distributed.is_initialized() and torch.distributed.get_world_size(self._pg) > 1:
            torch.distributed.all_reduce(buf["x_in"], group=self._pg)
        L.check(L.lib.pylo_b200_velo_rnn(C.byref(r), stream), "velo_rnn")
        plan.run_back(prm, stream)
        for group in self.param_groups:
            group["step"] += 1
        return None
