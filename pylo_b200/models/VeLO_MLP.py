"""VeLOMLP: the 256-way weight bank of VeLO's per-element network.

Weight-layout contract (pylo/models/VeLO_MLP.py:63-90): bank tensors carry a
trailing underscore, ``input_weights_ (B, H, 30)``, ``input_bias_ (B, H)``,
``hidden_weights_.{i} (B, H, H)``, ``hidden_bias_.{i} (B, H)``,
``output_weights_ (B, 3, H)``, ``output_bias_ (B, 3)`` with B=256, H=4; the
working copies without underscore hold the weights mixed for the current
tensor.  ``update_params(control)`` sets each working tensor to
``mean_b(control[b] * bank[b]) * 100`` (VeLO_MLP.py:92-126).
"""

import torch
import torch.nn.functional as F
from torch import nn

from ._hub import HUB_KW, HubMixin


class VeLOMLP(nn.Module, HubMixin, **HUB_KW):
    def __init__(self, param_inits=256, input_size=30, hidden_size=4, hidden_layers=1, output_size=3):
        super().__init__()
        self.hidden_layers = hidden_layers

        def bank(*shape):
            return nn.Parameter(torch.randn(param_inits, *shape))

        def bank_bias(width):
            return nn.Parameter(torch.zeros(param_inits, width))

        self.input_weights_ = bank(hidden_size, input_size)
        self.input_bias_ = bank_bias(hidden_size)
        self.hidden_weights_ = nn.ParameterList(bank(hidden_size, hidden_size) for _ in range(hidden_layers))
        self.hidden_bias_ = nn.ParameterList(bank_bias(hidden_size) for _ in range(hidden_layers))
        self.output_weights_ = bank(output_size, hidden_size)
        self.output_bias_ = bank_bias(output_size)

        self.input_weights = nn.Parameter(torch.randn(hidden_size, input_size))
        self.input_bias = nn.Parameter(torch.zeros(hidden_size))
        self.hidden_weights = nn.ParameterList(
            nn.Parameter(torch.randn(hidden_size, hidden_size)) for _ in range(hidden_layers)
        )
        self.hidden_bias = nn.ParameterList(nn.Parameter(torch.zeros(hidden_size)) for _ in range(hidden_layers))
        self.output_weights = nn.Parameter(torch.randn(output_size, hidden_size))
        self.output_bias = nn.Parameter(torch.zeros(output_size))

    def _pairs(self):
        yield self.input_weights, self.input_weights_
        yield self.input_bias, self.input_bias_
        for i in range(self.hidden_layers):
            yield self.hidden_weights[i], self.hidden_weights_[i]
            yield self.hidden_bias[i], self.hidden_bias_[i]
        yield self.output_weights, self.output_weights_
        yield self.output_bias, self.output_bias_

    @torch.no_grad()
    def update_params(self, control):
        for work, stored in self._pairs():
            c = control.view(-1, *([1] * (stored.dim() - 1)))
            work.data.copy_((c * stored.data).mean(0) * 100.0)

    def forward(self, x):
        x = F.relu(F.linear(x, self.input_weights, self.input_bias))
        for w, b in zip(self.hidden_weights, self.hidden_bias):
            x = F.relu(F.linear(x, w, b))
        return F.linear(x, self.output_weights, self.output_bias)

    def flat_bank(self):
        """The bank as one ``(B, 159)`` fp32 matrix in kernel order.

        Column layout per bank row: input_weights (4x30 out-major) | input_bias 4 |
        hidden_weights.0 (4x4) | hidden_bias.0 4 | output_weights (3x4) | output_bias 3.
        """
        if self.hidden_layers != 1:
            raise ValueError("the VeLO kernel geometry is 30-4-4-3 (hidden_layers=1)")
        parts = [stored.detach().to(torch.float32).reshape(stored.shape[0], -1) for _, stored in self._pairs()]
        return torch.cat(parts, dim=1).contiguous()
