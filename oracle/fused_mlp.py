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
inputs, which is the comparison benchmark configuration 1 asks for.
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


def activation_grad(name: str, z: Tensor, grad: Tensor) -> Tensor:
    r"""``d act(z) / dz * grad`` with the formulas of ``triton_helpers/ops.py:43-66``."""
    if name == "relu":
        return torch.where(z > 0, grad, torch.zeros_like(grad))
    if name == "silu":
        s = torch.sigmoid(z)
        return grad * s * (z * (1 - s) + 1)
    if name == "relu2":
        return torch.where(z > 0, grad * (2 * z), torch.zeros_like(grad))
    if name == "none":
        return grad
    raise ValueError(f"unknown activation {name}")


@torch.no_grad()
def forward_backward_storage_rounded(
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
    r"""The same network with the fused kernels' rounding points, evaluated in float32 in between.

    What the reference's fused kernels do and plain float32 autograd does not: every layer's
    output is rounded to the storage dtype (``fully_fused_mlp/kernel.py:47``), the backward pass
    evaluates ``act'`` on the dtype-rounded pre-activation (:278-281) and rounds ``dz`` and ``dx``
    to the gradient dtype between layers (:64, :74).  A ReLU whose pre-activation is within
    rounding noise of zero can therefore switch differently than in float32, which changes single
    rows of ``dx`` by far more than 1e-2; this function is the oracle for that arithmetic, so the
    CUDA path can be held to a tight tolerance, while ``forward_backward`` above stays the float32
    yardstick for outputs and for gradients summed over many rows.

    Returns ``(y, dx, dw_in, db_in, dw_out, db_out, dw_hid, db_hid)`` in float32 (weight and bias
    gradients are float32 sums, not rounded).
    """
    dtype = x.dtype
    rnd = lambda t: t.to(dtype).to(torch.float32)  # noqa: E731
    f32 = lambda t: None if t is None else t.to(torch.float32)  # noqa: E731
    d_hidden = w_in.shape[0]
    n_hid = 0 if w_hid is None else w_hid.shape[0] // d_hidden
    weights = [f32(w_in)] + [f32(w_hid[i * d_hidden : (i + 1) * d_hidden]) for i in range(n_hid)] + [f32(w_out)]
    if b_in is None:
        biases = [None] * (n_hid + 2)
    else:
        biases = [f32(b_in)] + [f32(b_hid[i]) for i in range(n_hid)] + [f32(b_out)]
    lead = x.shape[:-1]
    acts = [f32(x).reshape(-1, x.shape[-1])]
    pre = []
    for w, b in zip(weights[:-1], biases[:-1]):
        z = F.linear(acts[-1], w, b)
        pre.append(rnd(z))
        acts.append(rnd(activation_fn(activation, z)))
    y = rnd(F.linear(acts[-1], weights[-1], biases[-1]))

    dy = rnd(f32(grad_out).reshape(-1, grad_out.shape[-1]))
    dws, dbs = [None] * len(weights), [None] * len(weights)
    for l in range(len(weights) - 1, -1, -1):
        dz = dy if l == len(weights) - 1 else rnd(activation_grad(activation, pre[l], dy))
        dws[l] = dz.t() @ acts[l]
        dbs[l] = dz.sum(0)
        dy = rnd(dz @ weights[l])
    has_bias = b_in is not None
    dw_hid = torch.cat(dws[1:-1], 0) if n_hid else None
    db_hid = torch.stack(dbs[1:-1], 0) if n_hid and has_bias else None
    return (
        y.reshape(*lead, -1),
        dy.reshape(*lead, -1),
        dws[0],
        dbs[0] if has_bias else None,
        dws[-1],
        dbs[-1] if has_bias else None,
        dw_hid,
        db_hid,
    )
