"""CELO2MLP: weight container of the CELO2 / ELO-CELO2 per-element network.

Weight-layout contract (pylo/models/CELO2_MLP.py:25,73-98): the first layer is
split per feature group, ``w0.{0..13}`` of shape ``(group_width, hidden)`` with
group widths (1,1,1,3,1,3,1,3,1,3,3,3,3,3); ``b0 (hidden,)``; then dense layers
``dense_w.{i}`` stored **(in, out)** (the network multiplies ``x @ w``) with
``dense_b.{i}``.  For the kernel geometry 30-8-8-3 that is ``dense_w.0 (8, 8)``
and ``dense_w.1 (8, 3)``.
"""

import torch
from torch import nn

from ._hub import HUB_KW, HubMixin

CELO2_FEATURE_DIMS = (1, 1, 1, 3, 1, 3, 1, 3, 1, 3, 3, 3, 3, 3)


class CELO2MLP(nn.Module, HubMixin, **HUB_KW):
    def __init__(
        self,
        feature_dims=CELO2_FEATURE_DIMS,
        hidden_size=8,
        hidden_layers=2,
        output_size=3,
        activation="relu",
    ):
        super().__init__()
        if activation not in ("relu", "tanh"):
            raise ValueError(f"Invalid MLP activation: {activation}")
        self.feature_dims = tuple(feature_dims)
        self.hidden_size = hidden_size
        self.hidden_layers = hidden_layers
        self.output_size = output_size
        self.activation = activation

        self.w0 = nn.ParameterList(
            nn.Parameter(torch.empty(width, hidden_size)) for width in self.feature_dims
        )
        self.b0 = nn.Parameter(torch.zeros(hidden_size))
        widths = [hidden_size] * hidden_layers + [output_size]
        self.dense_w = nn.ParameterList()
        self.dense_b = nn.ParameterList()
        for fan_in, fan_out in zip(widths[:-1], widths[1:]):
            self.dense_w.append(nn.Parameter(torch.empty(fan_in, fan_out)))
            self.dense_b.append(nn.Parameter(torch.zeros(fan_out)))
        self.reset_parameters()

    def reset_parameters(self):
        """Truncated normal with std 1/sqrt(fan_in) (CELO2_MLP.py:90-98)."""
        fan_in = sum(self.feature_dims)
        for w in self.w0:
            nn.init.trunc_normal_(w, std=fan_in ** -0.5)
        for w in self.dense_w:
            nn.init.trunc_normal_(w, std=w.shape[0] ** -0.5)

    def _act(self, x):
        return torch.relu(x) if self.activation == "relu" else torch.tanh(x)

    def forward(self, inps):
        """``inps``: list of ``[..., group_width]`` tensors (a prefix of the groups is allowed)."""
        acc = self.b0
        for x, w in zip(inps, self.w0):
            acc = acc + x @ w
        out = self._act(acc)
        last = len(self.dense_w) - 1
        for i, (w, b) in enumerate(zip(self.dense_w, self.dense_b)):
            out = out @ w + b
            if i != last:
                out = self._act(out)
        return out

    def flat_weights(self):
        """(w_in[30,8] in-major, b_in, w_h[8,8], b_h, w_out[8,3], b_out) as fp32 tensors.

        The split first layer is concatenated along the input axis
        (CELO2_cuda.py:172-177).
        """
        return tuple(
            t.detach().to(torch.float32).contiguous()
            for t in (
                torch.cat([w.detach() for w in self.w0], dim=0),
                self.b0,
                self.dense_w[0],
                self.dense_b[0],
                self.dense_w[1],
                self.dense_b[1],
            )
        )
