r"""CPU oracle of the reversible (additive-coupling) fused MLP.  TEST INFRASTRUCTURE ONLY.

PARITY UNPINNED BY THE REFERENCE: triton_helpers ships no reversible operator, no test
and no vector for one.  This file is the definition the CUDA kernels are held to: the
stack evaluated in float32 with torch autograd and stored activations.

The input ``x (N, 2*H)`` is split into halves ``x1 = x[:, :H]`` and ``x2 = x[:, H:]``.  Block ``k`` is

    y1 = x1 + F_k(x2)        F_k(u) = act(u @ w_f1[k].T + b_f1[k]) @ w_f2[k].T + b_f2[k]
    y2 = x2 + G_k(y1)        G_k(u) = act(u @ w_g1[k].T + b_g1[k]) @ w_g2[k].T + b_g2[k]

and the output of the last block is ``cat(y1, y2)``.  Weights are stacked along dim 0 the way
``fully_fused_mlp`` stacks its hidden layers
(``triton_helpers/layers/fully_fused_mlp/kernel.py:534-537``): ``w_*1`` is ``(blocks * D_hidden, H)``,
``w_*2`` is ``(blocks * H, D_hidden)``, biases ``(blocks, D_hidden)`` / ``(blocks, H)`` or ``None``.

``reconstruct`` inverts the stack from its output (what the fused backward does instead of
storing activations): ``x2 = y2 - G(y1)``, ``x1 = y1 - F(x2)``, last block first.
"""
from typing import Optional, Sequence, Tuple

import torch
import torch.nn.functional as F
from torch import Tensor

from .fused_mlp import activation_fn


def _branch(u: Tensor, w1: Tensor, b1: Optional[Tensor], w2: Tensor, b2: Optional[Tensor], activation: str) -> Tensor:
    return F.linear(activation_fn(activation, F.linear(u, w1, b1)), w2, b2)


def _split(params: Sequence[Optional[Tensor]], k: int, half: int, hidden: int):
    w_f1, w_f2, w_g1, w_g2, b_f1, b_f2, b_g1, b_g2 = params
    sl = lambda w, rows: w[k * rows : (k + 1) * rows]  # noqa: E731
    bi = lambda b: None if b is None else b[k]  # noqa: E731
    return (
        (sl(w_f1, hidden), bi(b_f1), sl(w_f2, half), bi(b_f2)),
        (sl(w_g1, hidden), bi(b_g1), sl(w_g2, half), bi(b_g2)),
    )


def _to_f32(params: Sequence[Optional[Tensor]]):
    return [None if p is None else p.to(torch.float32) for p in params]


def forward(
    x: Tensor,
    w_f1: Tensor,
    w_f2: Tensor,
    w_g1: Tensor,
    w_g2: Tensor,
    b_f1: Optional[Tensor] = None,
    b_f2: Optional[Tensor] = None,
    b_g1: Optional[Tensor] = None,
    b_g2: Optional[Tensor] = None,
    activation: str = "relu",
) -> Tensor:
    r"""float32, differentiable forward of the whole stack."""
    params = _to_f32((w_f1, w_f2, w_g1, w_g2, b_f1, b_f2, b_g1, b_g2))
    half = x.shape[-1] // 2
    hidden = w_f2.shape[-1]
    blocks = w_f1.shape[0] // hidden
    x = x.to(torch.float32)
    x1, x2 = x[..., :half], x[..., half:]
    for k in range(blocks):
        f, g = _split(params, k, half, hidden)
        x1 = x1 + _branch(x2, *f, activation)
        x2 = x2 + _branch(x1, *g, activation)
    return torch.cat([x1, x2], dim=-1)


@torch.no_grad()
def reconstruct(
    y: Tensor,
    w_f1: Tensor,
    w_f2: Tensor,
    w_g1: Tensor,
    w_g2: Tensor,
    b_f1: Optional[Tensor] = None,
    b_f2: Optional[Tensor] = None,
    b_g1: Optional[Tensor] = None,
    b_g2: Optional[Tensor] = None,
    activation: str = "relu",
) -> Tensor:
    r"""Inverse of ``forward`` in float32: the input recovered from the output."""
    params = _to_f32((w_f1, w_f2, w_g1, w_g2, b_f1, b_f2, b_g1, b_g2))
    half = y.shape[-1] // 2
    hidden = w_f2.shape[-1]
    blocks = w_f1.shape[0] // hidden
    y = y.to(torch.float32)
    y1, y2 = y[..., :half], y[..., half:]
    for k in reversed(range(blocks)):
        f, g = _split(params, k, half, hidden)
        y2 = y2 - _branch(y1, *g, activation)
        y1 = y1 - _branch(y2, *f, activation)
    return torch.cat([y1, y2], dim=-1)


def forward_backward(
    x: Tensor,
    weights: Sequence[Tensor],
    biases: Sequence[Optional[Tensor]],
    grad_out: Tensor,
    activation: str = "relu",
) -> Tuple[Tensor, Tensor, Tuple[Optional[Tensor], ...]]:
    r"""Stored-activation autograd: returns ``(y, dx, (dw_f1, dw_f2, dw_g1, dw_g2, db_f1, db_f2, db_g1, db_g2))`` in float32."""
    leaves = [x.detach().to(torch.float32).requires_grad_(True)]
    for p in (*weights, *biases):
        leaves.append(None if p is None else p.detach().to(torch.float32).requires_grad_(True))
    y = forward(*leaves, activation=activation)
    y.backward(grad_out.to(torch.float32))
    grads = tuple(None if p is None else p.grad for p in leaves[1:])
    return y.detach(), leaves[0].grad, grads
