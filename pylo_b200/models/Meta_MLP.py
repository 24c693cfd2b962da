"""MetaMLP: weight container of the AdafacLO / ELO per-element network.

Weight-layout contract (pylo/models/Meta_MLP.py:30-43): an ``nn.Sequential``
called ``network`` whose children are ``input`` Linear(39, 32), ``relu_input``,
``linear_0`` Linear(32, 32), ``relu_0`` and ``output`` Linear(32, 2); weights
are ``nn.Linear`` style ``(out, in)``.  State-dict keys are therefore
``network.{input,linear_0,output}.{weight,bias}``, which is what a checkpoint
published for the reference holds.
"""

from collections import OrderedDict

import torch
from torch import nn

from ._hub import HUB_KW, HubMixin


class MetaMLP(nn.Module, HubMixin, **HUB_KW):
    def __init__(self, input_size=39, hidden_size=32, hidden_layers=1):
        super().__init__()
        layers = OrderedDict()
        layers["input"] = nn.Linear(input_size, hidden_size)
        layers["relu_input"] = nn.ReLU()
        for i in range(hidden_layers):
            layers[f"linear_{i}"] = nn.Linear(hidden_size, hidden_size)
            layers[f"relu_{i}"] = nn.ReLU()
        layers["output"] = nn.Linear(hidden_size, 2)
        self.network = nn.Sequential(layers)

    def forward(self, x):
        return self.network(x)

    def flat_weights(self):
        """(w_in[32,39], b_in, w_h[32,32], b_h, w_out[2,32], b_out) as fp32 tensors."""
        net = self.network
        return tuple(
            t.detach().to(torch.float32).contiguous()
            for t in (
                net.input.weight,
                net.input.bias,
                net.linear_0.weight,
                net.linear_0.bias,
                net.output.weight,
                net.output.bias,
            )
        )
