r"""CPU port of the neural-field training step.  TEST INFRASTRUCTURE / CPU BASELINE ONLY.

Composes the oracles of the two layers the way benchmark configuration 3 describes: hash
encoding (``oracle.hash_encoding.encode``, the restatement of the reference's
``_cpu_hash_encoding``, ``triton_helpers/layers/hash_encoding/kernel.py:482-502``) -> float32 MLP
(``oracle.fused_mlp.forward``, the reference's test MLP,
``tests/test_layers/test_fully_fused_mlp.py:21-35``) -> MSE -> torch autograd -> ``torch.optim.Adam``.
Everything is float32 on the host (the 16-bit storage of the GPU configuration has no fast CPU
equivalent); it is timed beside the CUDA path as the "reference's torch CPU path".
"""
from typing import Dict, Tuple

import torch
from torch import Tensor

from . import fused_mlp, hash_encoding


class CpuNeuralField:

    def __init__(self, levels=16, table_cap=2**19, n_min=16, n_max=2048, feats=2, d_hidden=64, d_out=16, depth=2,
                 lr=1e-2, betas=(0.9, 0.99), eps=1e-15, seed=0):  # fmt: skip
        g = torch.Generator().manual_seed(seed)
        self.geo = dict(table_cap=table_cap, levels=levels, n_min=n_min, n_max=n_max)
        rows = sum(hash_encoding.level_rows(levels, table_cap, 3, n_min, n_max))
        uni = lambda *shape, bound: ((torch.rand(*shape, generator=g) * 2 - 1) * bound).requires_grad_(True)  # noqa: E731
        d_in = levels * feats
        self.params: Dict[str, Tensor] = dict(
            table=uni(rows, feats, bound=1e-4),
            w_in=uni(d_hidden, d_in, bound=d_in**-0.5),
            w_hid=uni((depth - 1) * d_hidden, d_hidden, bound=d_hidden**-0.5),
            w_out=uni(d_out, d_hidden, bound=d_hidden**-0.5),
        )
        self.optimizer = torch.optim.Adam(self.params.values(), lr=lr, betas=betas, eps=eps)

    def predict(self, coords: Tensor) -> Tensor:
        p = self.params
        enc = hash_encoding.encode(coords, p["table"], **self.geo)
        return fused_mlp.forward(enc, p["w_in"], None, p["w_out"], None, p["w_hid"], None)

    def step(self, coords: Tensor, targets: Tensor) -> float:
        self.optimizer.zero_grad(set_to_none=True)
        loss = torch.nn.functional.mse_loss(self.predict(coords), targets)
        loss.backward()
        self.optimizer.step()
        return float(loss.detach())


def make_batch(n_points: int, d_out: int = 16, seed: int = 0) -> Tuple[Tensor, Tensor]:
    g = torch.Generator().manual_seed(seed)
    return torch.rand(n_points, 3, generator=g), torch.rand(n_points, d_out, generator=g)
