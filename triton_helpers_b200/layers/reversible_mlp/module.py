r"""``nn.Module`` around the reversible fused MLP, in the style of ``FullyFusedMLP``
(``triton_helpers/layers/fully_fused_mlp/module.py:9-53``): parameters come from ``nn.Linear``
initialisation, stacked along dim 0, created block by block in the order f1, f2, g1, g2."""
import torch
import torch.nn as nn
from torch import Tensor

from .kernel import reversible_mlp


class ReversibleMLP(nn.Module):

    def __init__(
        self,
        d_model: int = 128,
        blocks: int = 8,
        d_hidden: int = 64,
        activation: str = "relu",
        bias: bool = False,
    ):
        super().__init__()
        assert d_model % 2 == 0, "Model dimension must be even"
        half = d_model // 2
        layers = [
            [nn.Linear(half, d_hidden, bias=bias), nn.Linear(d_hidden, half, bias=bias),
             nn.Linear(half, d_hidden, bias=bias), nn.Linear(d_hidden, half, bias=bias)]
            for _ in range(blocks)
        ]  # fmt: skip
        for i, name in enumerate(("f1", "f2", "g1", "g2")):
            setattr(self, f"w_{name}", nn.Parameter(torch.cat([blk[i].weight for blk in layers], 0)))
            if bias:
                setattr(self, f"b_{name}", nn.Parameter(torch.stack([blk[i].bias for blk in layers], 0)))
            else:
                setattr(self, f"b_{name}", None)
        self.activation = activation

    def forward(self, x: Tensor) -> Tensor:
        return reversible_mlp(
            x, self.w_f1, self.w_f2, self.w_g1, self.w_g2, self.b_f1, self.b_f2, self.b_g1, self.b_g2, self.activation
        )
