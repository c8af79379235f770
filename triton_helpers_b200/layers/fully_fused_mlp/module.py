r"""``nn.Module`` around the fused MLP; drop-in for ``triton_helpers/layers/fully_fused_mlp/module.py:9-53``.

Parameters are created from ``nn.Linear`` layers in the order input, hidden..., output, so the
RNG stream and the parameter names (``w_in, b_in, w_hid, b_hid, w_out, b_out``) match the
reference and its ``state_dict``.
"""
import torch
import torch.nn as nn
from torch import Tensor

from .kernel import fully_fused_mlp


class FullyFusedMLP(nn.Module):

    def __init__(
        self,
        d_in: int,
        d_hidden: int,
        d_out: int,
        depth: int,
        activation: str = "relu",
        fp16_acc: bool = False,
        bias: bool = True,
    ):
        # ``bias=False`` (an extension; the reference always has biases) builds a bias-free network
        super().__init__()
        first = nn.Linear(d_in, d_hidden, bias=bias)
        self.w_in = first.weight
        self.b_in = first.bias

        if depth > 1:
            hidden = [nn.Linear(d_hidden, d_hidden, bias=bias) for _ in range(depth - 1)]
            self.w_hid = nn.Parameter(torch.cat([layer.weight for layer in hidden], 0))
            self.b_hid = nn.Parameter(torch.stack([layer.bias for layer in hidden], 0)) if bias else None
        else:
            self.w_hid = self.b_hid = None

        last = nn.Linear(d_hidden, d_out, bias=bias)
        self.w_out = last.weight
        self.b_out = last.bias

        self.activation = activation
        self.fp16_acc = fp16_acc

    def forward(self, x: Tensor) -> Tensor:
        return fully_fused_mlp(
            x,
            self.w_in,
            self.b_in,
            self.w_out,
            self.b_out,
            self.w_hid,
            self.b_hid,
            self.activation,
            fp16_acc=self.fp16_acc,
        )
