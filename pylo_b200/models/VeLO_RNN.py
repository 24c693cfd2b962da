"""VeLORNN: the per-tensor LSTM that emits VeLO's bank controls and step sizes.

Weight-layout contract (pylo/models/VeLO_RNN.py:96-108): ``mix_layer1``,
``mix_layer2``, ``final_mix_layer`` Linear(30, H); ``lstm.linear``
Linear(2H, 4H) over ``cat(x, h)`` with gate order i, g, f, o and a +1 forget
bias (VeLO_RNN.py:57-65); ``rnn_to_controls`` Linear(H, 256); ``step_size``
Linear(H, 1); ``lstm_init_state.{0,1} (1, H)``; H = 512.
``mix_layer1`` is carried for checkpoint compatibility and not used in the
forward pass (VeLO_RNN.py:128).
"""

import torch
import torch.nn.functional as F
from torch import nn

from ._hub import HUB_KW, HubMixin


class LSTM(nn.Module):
    def __init__(self, input_size, hidden_size):
        super().__init__()
        self.linear = nn.Linear(2 * input_size, 4 * hidden_size)

    def forward(self, x, prev_state):
        h_prev, c_prev = prev_state
        i, g, f, o = self.linear(torch.cat((x, h_prev), dim=-1)).chunk(4, -1)
        c = torch.sigmoid(f + 1) * c_prev + torch.sigmoid(i) * torch.tanh(g)
        h = torch.sigmoid(o) * torch.tanh(c)
        return h, (h, c)


class VeLORNN(nn.Module, HubMixin, **HUB_KW):
    def __init__(self, input_size=30, lstm_hidden_size=512, param_inits=256, mix_layers=True):
        super().__init__()
        self.mix_layers = mix_layers
        self.mix_layer1 = nn.Linear(input_size, lstm_hidden_size)
        self.mix_layer2 = nn.Linear(input_size, lstm_hidden_size)
        self.final_mix_layer = nn.Linear(input_size, lstm_hidden_size)
        self.lstm = LSTM(input_size=lstm_hidden_size, hidden_size=lstm_hidden_size)
        self.rnn_to_controls = nn.Linear(lstm_hidden_size, param_inits)
        self.step_size = nn.Linear(lstm_hidden_size, 1)
        self.lstm_init_state = nn.ParameterList(
            [nn.Parameter(torch.zeros(1, lstm_hidden_size)), nn.Parameter(torch.zeros(1, lstm_hidden_size))]
        )

    def forward(self, x, state):
        if self.mix_layers:
            pooled = F.relu(self.mix_layer2(x)).max(dim=0, keepdim=True).values
            x = self.final_mix_layer(x) + pooled
        out, state = self.lstm(x, state)
        return self.rnn_to_controls(out), self.step_size(out).squeeze(-1), state
