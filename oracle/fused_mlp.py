r"""CPU oracle of the fully fused MLP.  TEST INFRASTRUCTURE ONLY.

The reference package has no CPU function for this operator; what its tests and
benchmark compare the fused kernel with is a plain chain of ``F.linear`` + activation
(``tests/test_layers/test_fully_fused_mlp.py:21-35``,
``triton_helpers/layers/fully_fused_mlp/__main__.py:40-62``).  This file restates that
chain with the stacked-weight calling convention of ``fully_fused_mlp``
(``triton_helpers/layers/fully_fused_mlp/kernel.py:640-686``): ``w_hid`` is
``((depth - 1) * D_hidden, D_hidden)``, ``b_hid`` is ``(depth - 1, D_hidden)``, the output
layer is never activated (kernel.py:250).

Activations follow ``triton_helpers/ops.py:38-66``: ``relu``, ``silu``, ``relu2(z) = max(z, 0) * z``
and ``none``.  Everything is evaluated in float32 from the (possibly fp16/bf16-valued)
inputs, which is the comparison BASELINE configuration 1 asks for.
"""
from typing import Optional, Tuple

import torch
import torch.nn.functional as F
from torch import Tensor


def activation_fn(name: str, z: Tensor) -> Tensor:
    if name == "relu":
        return F.relu(z)
    if name == "silu":
        return F.silu(z)
    if name == "relu2":
        return F.relu(z) * z
    if name == "none":
        return z
    raise ValueError(f"unknown activation {name}")


def forward(
    x: Tensor,
    w_in: Tensor,
    b_in: Optional[Tensor],
    w_out: Tensor,
    b_out: Optional[Tensor],
    w_hid: Optional[Tensor] = None,
    b_hid: Optional[Tensor] = None,
    activation: str = "relu",
) -> Tensor:
    r"""float32 forward; differentiable, so ``backward`` below is just autograd."""
    f32 = lambda t: None if t is None else t.to(torch.float32)  # noqa: E731
    h = activation_fn(activation, F.linear(f32(x), f32(w_in), f32(b_in)))
    if w_hid is not None:
        d_hidden = w_in.shape[0]
        for i in range(w_hid.shape[0] // d_hidden):
            w = w_hid[i * d_hidden : (i + 1) * d_hidden]
            b = None if b_hid is None else b_hid[i]
            h = activation_fn(activation, F.linear(h, f32(w), f32(b)))
    return F.linear(h, f32(w_out), f32(b_out))


def forward_backward(
    x: Tensor,
    w_in: Tensor,
    b_in: Optional[Tensor],
    w_out: Tensor,
    b_out: Optional[Tensor],
    w_hid: Optional[Tensor],
    b_hid: Optional[Tensor],
    grad_out: Tensor,
    activation: str = "relu",
) -> Tuple[Tensor, ...]:
    r"""Returns ``(y, dx, dw_in, db_in, dw_out, db_out, dw_hid, db_hid)`` in float32 (None where the input was None)."""
    leaves = []
    for t in (x, w_in, b_in, w_out, b_out, w_hid, b_hid):
        leaves.append(None if t is None else t.detach().to(torch.float32).requires_grad_(True))
    y = forward(*leaves, activation=activation)
    y.backward(grad_out.to(torch.float32))
    grads = [None if t is None else t.grad for t in leaves]
    return (y.detach(), *grads)
