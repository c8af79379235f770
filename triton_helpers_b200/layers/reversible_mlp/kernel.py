r"""Reversible (additive coupling) fused MLP on hand-written sm_100a kernels.

There is no such operator in triton_helpers; this module follows the conventions of its fused
MLP (``triton_helpers/layers/fully_fused_mlp/kernel.py:503-686``): a ``torch.autograd.Function``
plus a functional wrapper, stacked ``(out, in)`` weights, 16-bit tensors, fp32 accumulation,
autocast to float16.

    x = [x1 | x2]                      halves of width H = d_model / 2
    y1 = x1 + F_k(x2)                  F_k(u) = act(u @ w_f1[k].T + b_f1[k]) @ w_f2[k].T + b_f2[k]
    y2 = x2 + G_k(y1)                  G_k(u) = act(u @ w_g1[k].T + b_g1[k]) @ w_g2[k].T + b_g2[k]

for ``k = 0 .. blocks-1``; the output is ``[y1 | y2]`` of the last block.  The backward pass keeps
no activations: it starts from the saved OUTPUT and reconstructs every block's input
(``x2 = y2 - G(y1)``, ``x1 = y1 - F(x2)``) while forming the gradients.
"""
from typing import Final, NamedTuple, Optional, Tuple

import torch
from torch import Tensor
from torch.autograd import Function

from ... import _lib
from ...ops import ensure_str

ACTIVATIONS: Final = ("relu", "relu2", "silu", "none")


class ReversibleGrads(NamedTuple):
    dx: Tensor
    dw_f1: Tensor
    dw_f2: Tensor
    dw_g1: Tensor
    dw_g2: Tensor
    db_f1: Optional[Tensor]
    db_f2: Optional[Tensor]
    db_g1: Optional[Tensor]
    db_g2: Optional[Tensor]
    x_reconstructed: Optional[Tensor]


def _rows2d(t: Tensor, width: int) -> Tensor:
    t = t.reshape(-1, width)
    if t.stride(1) != 1 or (t.shape[0] > 1 and (t.stride(0) < width or t.stride(0) % 2)) or t.data_ptr() % 4:
        t = t.contiguous()
    return t


def _validate(x: Tensor, weights: Tuple[Tensor, ...], biases: Tuple[Optional[Tensor], ...], activation: str):
    w_f1, w_f2, w_g1, w_g2 = weights
    d_model = x.shape[-1]
    assert d_model % 2 == 0, "Model dimension must be even"
    half = d_model // 2
    d_hidden = w_f2.shape[-1]
    assert w_f1.shape[0] % d_hidden == 0, "Stacked weight shape mismatch"
    blocks = w_f1.shape[0] // d_hidden
    assert blocks >= 1, "At least one coupling block is required"
    assert w_f1.shape == (blocks * d_hidden, half) and w_g1.shape == w_f1.shape, "First-layer weight shape mismatch"
    assert w_f2.shape == (blocks * half, d_hidden) and w_g2.shape == w_f2.shape, "Second-layer weight shape mismatch"
    assert half <= 64 and half % 16 == 0, f"Half width {half} must be a multiple of 16 up to 64"
    assert d_hidden <= 64 and d_hidden % 16 == 0, f"Hidden dimension {d_hidden} must be a multiple of 16 up to 64"
    has_bias = biases[0] is not None
    assert all((b is not None) == has_bias for b in biases), "Biases must be given for every layer or for none"
    if has_bias:
        assert biases[0].shape == (blocks, d_hidden) and biases[2].shape == (blocks, d_hidden), "Bias shape mismatch"
        assert biases[1].shape == (blocks, half) and biases[3].shape == (blocks, half), "Bias shape mismatch"
    assert activation in ACTIVATIONS, f"Invalid activation function: {activation}"
    dtypes = {t.dtype for t in (x, *weights, *biases) if t is not None}
    if len(dtypes) != 1 or next(iter(dtypes)) not in (torch.float16, torch.bfloat16):
        raise TypeError(f"reversible MLP kernels take float16 or bfloat16 tensors of one dtype, got {dtypes}")
    return d_model, d_hidden, blocks


def _contiguous(ts):
    return tuple(None if t is None else t.contiguous() for t in ts)


@torch.no_grad()
def reversible_mlp_forward(x, weights, biases, activation: str = "relu") -> Tensor:
    r"""Raw forward launch (no autograd): ``x (..., d_model)`` -> ``y`` of the same shape."""
    d_model, d_hidden, blocks = _validate(x, weights, biases, activation)
    device = _lib.require_cuda(x, *weights, *biases)
    weights, biases = _contiguous(weights), _contiguous(biases)
    x2d = _rows2d(x, d_model)
    y = torch.empty((x2d.shape[0], d_model), dtype=x.dtype, device=device)
    with torch.cuda.device(device):
        _lib.check(
            _lib.lib().th_rev_fwd(
                x2d.data_ptr(), x2d.stride(0) if x2d.shape[0] > 1 else d_model,
                *(w.data_ptr() for w in weights), *(_lib.ptr(b) for b in biases),
                y.data_ptr(), d_model, x2d.shape[0], d_model, d_hidden, blocks,
                _lib.ACTIVATION_CODE[activation], _lib.DTYPE_CODE[x.dtype], _lib.stream_ptr(device),
            ),
            "th_rev_fwd",
        )  # fmt: skip
    return y.view(x.shape)


@torch.no_grad()
def reversible_mlp_backward(
    y: Tensor, grad_out: Tensor, weights, biases, activation: str = "relu", reconstruct: bool = False
) -> ReversibleGrads:
    r"""Raw backward launch from the stack's output ``y``; optionally also returns the reconstructed input."""
    d_model, d_hidden, blocks = _validate(y, weights, biases, activation)
    device = _lib.require_cuda(y, grad_out, *weights, *biases)
    weights, biases = _contiguous(weights), _contiguous(biases)
    y2d = _rows2d(y, d_model)
    go = _rows2d(grad_out.to(y.dtype), d_model)
    rows = y2d.shape[0]
    dx = torch.empty((rows, d_model), dtype=y.dtype, device=device)
    x_rec = torch.empty_like(dx) if reconstruct else None
    dws = tuple(torch.empty_like(w) for w in weights)
    dbs = tuple(None if b is None else torch.empty_like(b) for b in biases)
    with torch.cuda.device(device):  # the size depends on the SM count of the tensors' device, which must be current
        ws_bytes = _lib.lib().th_rev_workspace_bytes(rows, d_model, d_hidden, blocks)
    workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=device)
    stride = lambda t: t.stride(0) if t.shape[0] > 1 else d_model  # noqa: E731
    with torch.cuda.device(device):
        _lib.check(
            _lib.lib().th_rev_bwd(
                y2d.data_ptr(), stride(y2d), *(w.data_ptr() for w in weights), *(_lib.ptr(b) for b in biases),
                go.data_ptr(), stride(go), dx.data_ptr(), d_model, _lib.ptr(x_rec), d_model,
                *(w.data_ptr() for w in dws), *(_lib.ptr(b) for b in dbs),
                workspace.data_ptr(), ws_bytes, rows, d_model, d_hidden, blocks,
                _lib.ACTIVATION_CODE[activation], _lib.DTYPE_CODE[y.dtype], _lib.stream_ptr(device),
            ),
            "th_rev_bwd",
        )  # fmt: skip
    view = lambda t: None if t is None else t.view(y.shape)  # noqa: E731
    return ReversibleGrads(view(dx), *dws, *dbs, view(x_rec))


class _reversible_mlp(Function):

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.float16)
    def forward(ctx, x, w_f1, w_f2, w_g1, w_g2, b_f1, b_f2, b_g1, b_g2, activation="relu"):
        weights, biases = (w_f1, w_f2, w_g1, w_g2), (b_f1, b_f2, b_g1, b_g2)
        y = reversible_mlp_forward(x, weights, biases, activation)
        # the OUTPUT is saved, not the input: backward reconstructs every intermediate from it
        ctx.save_for_backward(y, *weights, *(b for b in biases if b is not None))
        ctx.has_bias = b_f1 is not None
        ctx.activation = activation
        return y

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    @torch.no_grad()
    def backward(ctx, do: Tensor):
        y, *params = ctx.saved_tensors
        weights = tuple(params[:4])
        biases = tuple(params[4:]) if ctx.has_bias else (None, None, None, None)
        g = reversible_mlp_backward(y, do, weights, biases, ctx.activation)
        return (g.dx, g.dw_f1, g.dw_f2, g.dw_g1, g.dw_g2, g.db_f1, g.db_f2, g.db_g1, g.db_g2, None)


def reversible_mlp(
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
    r"""Stack of additive coupling blocks evaluated in one kernel, with a backward that stores no activations.

    Shapes:
        - x, output: :math:`(..., 2H)`
        - w_f1, w_g1: :math:`(blocks \cdot D_{hidden}, H)`; w_f2, w_g2: :math:`(blocks \cdot H, D_{hidden})`
        - b_f1, b_g1: :math:`(blocks, D_{hidden})`; b_f2, b_g2: :math:`(blocks, H)`; all or none
    """
    activation = ensure_str(activation)
    return _reversible_mlp.apply(x, w_f1, w_f2, w_g1, w_g2, b_f1, b_f2, b_g1, b_g2, activation)
