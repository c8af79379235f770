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


@torch.no_grad()
def forward_backward_storage_rounded(
    x: Tensor,
    weights: Sequence[Tensor],
    biases: Sequence[Optional[Tensor]],
    grad_out: Tensor,
    activation: str = "relu",
    y_saved: Optional[Tensor] = None,
):
    r"""The stack with the fused kernels' rounding points and the reconstructing backward.

    ``y_saved`` (optional) replaces the forward result as the tensor the backward pass starts
    from: pass the output another implementation produced to check its backward in isolation.

    Arithmetic being restated (float32 everywhere except where noted): the residual stream stays
    float32 inside a pass; each branch input, hidden activation and pre-activation is rounded to
    the storage dtype before it is used as a matrix operand; the output of the forward pass is
    rounded to the storage dtype (it is what gets saved); the backward pass starts from that
    rounded output, reconstructs ``x2 = y2 - G(y1)`` and ``x1 = y1 - F(x2)`` block by block,
    and rounds the branch-output gradient and ``dz`` to the storage dtype before they are used as
    matrix operands.  Returns ``(y, dx, grads(8), x_reconstructed)`` in float32.
    """
    from .fused_mlp import activation_grad

    dtype = x.dtype
    rnd = lambda t: t.to(dtype).to(torch.float32)  # noqa: E731
    params = _to_f32((*weights, *biases))
    half = x.shape[-1] // 2
    hidden = weights[1].shape[-1]
    blocks = weights[0].shape[0] // hidden
    lead = x.shape[:-1]
    xf = x.to(torch.float32).reshape(-1, 2 * half)

    def branch(u, w1, b1, w2, b2):
        z = F.linear(rnd(u), w1, b1)
        h = rnd(activation_fn(activation, z))
        return F.linear(h, w2, b2), rnd(z), h

    s1, s2 = xf[:, :half].clone(), xf[:, half:].clone()
    for k in range(blocks):
        f, g = _split(params, k, half, hidden)
        s1 = s1 + branch(s2, *f)[0]
        s2 = s2 + branch(s1, *g)[0]
    y = rnd(torch.cat([s1, s2], -1))

    if y_saved is not None:
        y = y_saved.to(torch.float32).reshape(-1, 2 * half)
    s1, s2 = y[:, :half].clone(), y[:, half:].clone()
    go = rnd(grad_out.to(torch.float32).reshape(-1, 2 * half))
    d1, d2 = go[:, :half].clone(), go[:, half:].clone()
    has_bias = biases[0] is not None
    dw = [torch.zeros_like(p) for p in params[:4]]
    db = [torch.zeros_like(p) if has_bias else None for p in (params[4:] if has_bias else [None] * 4)]
    for k in reversed(range(blocks)):
        f, g = _split(params, k, half, hidden)
        for (w1, b1, w2, b2), m1, in_is_first in ((g, 2, True), (f, 0, False)):
            in_s, out_d = (s1, d2) if in_is_first else (s2, d1)
            out, z, h = branch(in_s, w1, b1, w2, b2)
            if in_is_first:
                s2 = s2 - out
            else:
                s1 = s1 - out
            dy = rnd(out_d)
            dz = rnd(activation_grad(activation, z, dy @ w2))
            dw[m1 + 1][k * half : (k + 1) * half] = dy.t() @ h
            dw[m1][k * hidden : (k + 1) * hidden] = dz.t() @ rnd(in_s)
            if has_bias:
                db[m1 + 1][k] = dy.sum(0)
                db[m1][k] = dz.sum(0)
            if in_is_first:
                d1 = d1 + dz @ w1
            else:
                d2 = d2 + dz @ w1
    dx = rnd(torch.cat([d1, d2], -1)).reshape(*lead, -1)
    x_rec = rnd(torch.cat([s1, s2], -1)).reshape(*lead, -1)
    return y.reshape(*lead, -1), dx, (*dw, *db), x_rec
