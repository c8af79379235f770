r"""Fully fused small MLP on hand-written sm_100a kernels.

Drop-in for ``triton_helpers/layers/fully_fused_mlp/kernel.py``: ``_fully_fused_mlp`` is the
``torch.autograd.Function`` (reference :503-637) and ``fully_fused_mlp`` the functional wrapper
(reference :640-686) with the same argument order, assertions and 9-tuple of gradients.  The
Triton launches are replaced by ``th_mlp_fwd`` / ``th_mlp_bwd`` of ``libth_b200.so``.

Differences a caller can observe:

* float32 tensors are accepted like in the reference, whose ``tl.dot`` then runs in TF32 (10-bit
  operand mantissa, float32 accumulation).  Here they are rounded to float16 (the same 10-bit
  mantissa, float32 accumulation) for the tensor cores and the results are returned in float32;
  values beyond the float16 range (|v| > 65504) overflow, which TF32 would not.  Setting the
  environment variable ``TH_MLP_F32_OPERANDS=bf16`` before the first call rounds float32 tensors to
  bfloat16 instead (TF32's exponent range, 8 instead of 10 mantissa bits) for data that needs the range.
  As in the reference, a float32 backward pass is refused for depth >= 4 (reference :576).
* ``fp16_acc=True`` is accepted (the reference's callers and benchmarks pass it) but changes nothing:
  accumulation is always float32, which is at least as accurate as what was asked for.  The first
  such call emits a ``UserWarning`` saying so.
* biases may be ``None`` (all of them) for a bias-free network; the reference requires tensors.
* the Triton device functions the reference re-exports (``feedforward`` ...) do not exist.
"""
import warnings
from typing import Final, Optional

import torch
from torch import Tensor
from torch.autograd import Function

from ... import _lib
from ...ops import ensure_str

# Above this size the weights no longer stay on chip (reference :13-14)
FULLY_FUSED_MAX_DIM: Final = 64
ACTIVATIONS: Final = ("relu", "relu2", "silu", "none")


_F32_OPERANDS: Optional[torch.dtype] = None


def _f32_operand_dtype() -> torch.dtype:
    r"""The 16-bit type float32 tensors are rounded to for the tensor cores: float16 (TF32's mantissa) unless
    ``TH_MLP_F32_OPERANDS=bf16`` asks for bfloat16 (TF32's range).  Read once per process."""
    global _F32_OPERANDS
    if _F32_OPERANDS is None:
        import os

        choice = os.environ.get("TH_MLP_F32_OPERANDS", "fp16").lower()
        if choice not in ("fp16", "float16", "bf16", "bfloat16"):
            raise ValueError(f"TH_MLP_F32_OPERANDS must be fp16 or bf16, got {choice!r}")
        _F32_OPERANDS = torch.bfloat16 if choice.startswith("b") else torch.float16
    return _F32_OPERANDS


_FP16_ACC_WARNED = False


def _warn_fp16_acc() -> None:
    global _FP16_ACC_WARNED
    if not _FP16_ACC_WARNED:
        _FP16_ACC_WARNED = True
        warnings.warn("fp16_acc=True is accepted for compatibility; these kernels always accumulate in float32", UserWarning, stacklevel=3)


def _rows_view(t: Tensor) -> Tensor:
    r"""``(B, L, D)`` tensor whose ``B * L`` rows are evenly strided with unit stride inside a row."""
    B, L, _ = t.shape
    if t.stride(2) != 1 or (B > 1 and t.stride(0) != L * t.stride(1)) or t.stride(1) < t.shape[2]:
        t = t.contiguous()
    return t


def _check_dtype(*tensors: Optional[Tensor]) -> torch.dtype:
    dtypes = {t.dtype for t in tensors if t is not None}
    if len(dtypes) != 1:
        raise TypeError(f"input and parameters must share one dtype, got {dtypes}")
    (dtype,) = dtypes
    if dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise TypeError(f"fused MLP kernels take float16, bfloat16 or float32 tensors, got {dtype}")
    return dtype


class _fully_fused_mlp(Function):

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.float16)
    @torch.no_grad()
    def forward(
        ctx,
        x: Tensor,
        w_in: Tensor,
        b_in: Optional[Tensor],
        w_out: Tensor,
        b_out: Optional[Tensor],
        w_hid: Optional[Tensor],
        b_hid: Optional[Tensor],
        activation: str = "relu",
        fp16_acc: bool = False,
    ) -> Tensor:
        B, L, D = x.shape
        D_hidden, D_in = w_in.shape
        D_out, _ = w_out.shape
        assert D_in == D, "Input dimension mismatch"
        assert D_hidden == w_out.shape[-1], "Hidden dimension mismatch"

        assert D_in <= FULLY_FUSED_MAX_DIM, f"Input dimension {D_in} too large for full fusion"
        assert D_hidden <= FULLY_FUSED_MAX_DIM, f"Hidden dimension {D_hidden} too large for full fusion"
        assert D_out <= FULLY_FUSED_MAX_DIM, f"Output dimension {D_out} too large for full fusion"
        assert D_hidden & (D_hidden - 1) == 0, "Hidden dimension must be a power of 2"
        assert D_hidden >= 16, "Hidden dimension must be at least 16"

        if w_hid is not None and w_hid.numel() > 0:
            depth = w_hid.shape[0] // D_hidden
            assert w_hid.shape == (depth * D_hidden, D_hidden), "Hidden weight shape mismatch"
            assert b_hid is None or b_hid.shape == (depth, D_hidden), "Hidden bias shape mismatch"
            depth += 1
        else:
            depth = 1
            w_hid = b_hid = None
        assert activation in ACTIVATIONS, f"Invalid activation function: {activation}"
        if fp16_acc:
            _warn_fp16_acc()
        has_bias = b_in is not None
        assert (b_out is not None) == has_bias and (depth == 1 or (b_hid is not None) == has_bias), (
            "Biases must be given for every layer or for none"
        )

        device = _lib.require_cuda(x, w_in, b_in, w_out, b_out, w_hid, b_hid)
        io_dtype = _check_dtype(x, w_in, b_in, w_out, b_out, w_hid, b_hid)
        dtype = _f32_operand_dtype() if io_dtype == torch.float32 else io_dtype  # float32: 16-bit operands, fp32 accumulate
        if io_dtype == torch.float32:
            x, w_in, w_out = x.to(dtype), w_in.to(dtype), w_out.to(dtype)
            w_hid = None if w_hid is None else w_hid.to(dtype)
            b_in, b_out, b_hid = (None if b is None else b.to(dtype) for b in (b_in, b_out, b_hid))
        x = _rows_view(x)
        w_in, w_out = w_in.contiguous(), w_out.contiguous()
        w_hid = None if w_hid is None else w_hid.contiguous()
        b_in, b_out, b_hid = (None if b is None else b.contiguous() for b in (b_in, b_out, b_hid))

        o = x.new_empty((B, L, D_out))
        with torch.cuda.device(device):
            _lib.check(
                _lib.lib().th_mlp_fwd(
                    x.data_ptr(), x.stride(1), w_in.data_ptr(), _lib.ptr(b_in), _lib.ptr(w_hid), _lib.ptr(b_hid),
                    w_out.data_ptr(), _lib.ptr(b_out), o.data_ptr(), D_out, B * L, D_in, D_hidden, D_out, depth,
                    _lib.ACTIVATION_CODE[activation], _lib.DTYPE_CODE[dtype], int(fp16_acc), _lib.stream_ptr(device),
                ),
                "th_mlp_fwd",
            )  # fmt: skip

        ctx.save_for_backward(x, w_in, b_in, w_out, b_out, w_hid, b_hid)
        ctx.activation = activation
        ctx.fp16_acc = fp16_acc
        ctx.depth = depth
        ctx.io_dtype = io_dtype
        return o if io_dtype == dtype else o.to(io_dtype)

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    @torch.no_grad()
    def backward(ctx, do: Tensor):
        x, w_in, b_in, w_out, b_out, w_hid, b_hid = ctx.saved_tensors
        assert ctx.io_dtype != torch.float32 or ctx.depth < 4, "FP32 backward not supported for depth >= 4"
        B, L, D_in = x.shape
        D_hidden, _ = w_in.shape
        D_out, _ = w_out.shape
        depth = ctx.depth
        device, dtype = x.device, x.dtype

        if do.dtype != dtype:
            do = do.to(dtype)
        do = _rows_view(do)

        dx = x.new_empty((B, L, D_in))
        dw_in, dw_out = torch.empty_like(w_in), torch.empty_like(w_out)
        dw_hid = None if w_hid is None else torch.empty_like(w_hid)
        db_in, db_out, db_hid = (None if b is None else torch.empty_like(b) for b in (b_in, b_out, b_hid))
        ws_bytes = _lib.lib().th_mlp_workspace_bytes(D_in, D_hidden, D_out, depth)
        workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=device)
        with torch.cuda.device(device):
            _lib.check(
                _lib.lib().th_mlp_bwd(
                    x.data_ptr(), x.stride(1), w_in.data_ptr(), _lib.ptr(b_in), _lib.ptr(w_hid), _lib.ptr(b_hid),
                    w_out.data_ptr(), _lib.ptr(b_out), do.data_ptr(), do.stride(1), dx.data_ptr(), D_in,
                    dw_in.data_ptr(), _lib.ptr(db_in), _lib.ptr(dw_hid), _lib.ptr(db_hid), dw_out.data_ptr(),
                    _lib.ptr(db_out), workspace.data_ptr(), ws_bytes, B * L, D_in, D_hidden, D_out, depth,
                    _lib.ACTIVATION_CODE[ctx.activation], _lib.DTYPE_CODE[dtype], int(ctx.fp16_acc),
                    _lib.stream_ptr(device),
                ),
                "th_mlp_bwd",
            )  # fmt: skip
        if ctx.io_dtype != dtype:
            cast = lambda t: None if t is None else t.to(ctx.io_dtype)  # noqa: E731
            dx, dw_in, db_in, dw_out, db_out, dw_hid, db_hid = map(cast, (dx, dw_in, db_in, dw_out, db_out, dw_hid, db_hid))
        return dx, dw_in, db_in, dw_out, db_out, dw_hid, db_hid, None, None


def fully_fused_mlp(
    x: Tensor,
    w_in: Tensor,
    b_in: Optional[Tensor],
    w_out: Tensor,
    b_out: Optional[Tensor],
    w_hid: Optional[Tensor] = None,
    b_hid: Optional[Tensor] = None,
    activation: str = "relu",
    fp16_acc: bool = False,
) -> Tensor:
    r"""Forward pass of a multi-layer perceptron in a single kernel (Mueller et al., arXiv:2106.12372).

    Args:
        x: Input tensor
        w_in, b_in: Weight and bias of the input layer
        w_out, b_out: Weight and bias of the (never activated) output layer
        w_hid, b_hid: Stacked weights and biases of the hidden layers, or ``None`` for a single layer
        activation: ``"relu"``, ``"relu2"``, ``"silu"`` or ``"none"``
        fp16_acc: accepted for compatibility; accumulation is always float32

    Shapes:
        - x: :math:`(B, L, D_{in})`, output :math:`(B, L, D_{out})`
        - w_in: :math:`(D_{hidden}, D_{in})`, b_in: :math:`(D_{hidden},)`
        - w_out: :math:`(D_{out}, D_{hidden})`, b_out: :math:`(D_{out},)`
        - w_hid: :math:`(depth \cdot D_{hidden}, D_{hidden})`, b_hid: :math:`(depth, D_{hidden})`
    """
    activation = ensure_str(activation)
    return _fully_fused_mlp.apply(x, w_in, b_in, w_out, b_out, w_hid, b_hid, activation, fp16_acc)


class _fully_fused_mlp_mse(torch.autograd.Function):
    r"""Forward pass and squared-error loss in one kernel; see ``fully_fused_mlp_mse``."""

    @staticmethod
    def forward(ctx, x, w_in, w_out, w_hid, target, grad_scale, activation):
        B, L, D_in = x.shape
        D_hidden, D_out = w_in.shape[0], w_out.shape[0]
        depth = 1 if w_hid is None else w_hid.shape[0] // D_hidden + 1
        device = _lib.require_cuda(x, w_in, w_out, w_hid, target)
        dtype = x.dtype
        assert dtype in (torch.float16, torch.bfloat16) and all(
            t is None or t.dtype == dtype for t in (w_in, w_out, w_hid, target)
        ), "fused forward + MSE takes float16 or bfloat16 tensors of one dtype"
        assert target.shape == (B, L, D_out), "target shape mismatch"
        x, target = _rows_view(x), _rows_view(target)
        w_in, w_out = w_in.contiguous(), w_out.contiguous()
        w_hid = None if w_hid is None else w_hid.contiguous()
        grad = x.new_empty((B, L, D_out))
        loss_sum = torch.zeros(1, dtype=torch.float32, device=device)
        lib = _lib.lib()
        with torch.cuda.device(device):
            code = lib.th_mlp_fwd_mse(
                x.data_ptr(), x.stride(1), w_in.data_ptr(), None, _lib.ptr(w_hid), None, w_out.data_ptr(), None,
                None, D_out, target.data_ptr(), target.stride(1), grad.data_ptr(), D_out, loss_sum.data_ptr(),
                grad_scale, B * L, D_in, D_hidden, D_out, depth, _lib.ACTIVATION_CODE[activation],
                _lib.DTYPE_CODE[dtype], _lib.stream_ptr(device),
            )  # fmt: skip
            if code == _lib.TH_ERR_UNSUPPORTED:
                # shapes the fused kernel does not take: the two kernels it stands for
                o = x.new_empty((B, L, D_out))
                _lib.check(
                    lib.th_mlp_fwd(
                        x.data_ptr(), x.stride(1), w_in.data_ptr(), None, _lib.ptr(w_hid), None, w_out.data_ptr(), None,
                        o.data_ptr(), D_out, B * L, D_in, D_hidden, D_out, depth, _lib.ACTIVATION_CODE[activation],
                        _lib.DTYPE_CODE[dtype], 0, _lib.stream_ptr(device),
                    ),
                    "th_mlp_fwd",
                )  # fmt: skip
                target_c = target.contiguous()
                _lib.check(
                    lib.th_mse_grad(
                        o.data_ptr(), target_c.data_ptr(), grad.data_ptr(), loss_sum.data_ptr(), o.numel(), grad_scale,
                        _lib.DTYPE_CODE[dtype], _lib.stream_ptr(device),
                    ),
                    "th_mse_grad",
                )  # fmt: skip
            else:
                _lib.check(code, "th_mlp_fwd_mse")
        ctx.save_for_backward(x, w_in, w_out, w_hid, grad)
        ctx.activation, ctx.depth = activation, depth
        return loss_sum

    @staticmethod
    @torch.no_grad()
    def backward(ctx, d_loss: Tensor):
        # The gradients of (grad_scale / 2) * loss_sum; the incoming gradient is taken to be one.
        x, w_in, w_out, w_hid, grad = ctx.saved_tensors
        B, L, D_in = x.shape
        D_hidden, D_out = w_in.shape[0], w_out.shape[0]
        device, dtype = x.device, x.dtype
        dx = x.new_empty((B, L, D_in)) if ctx.needs_input_grad[0] else None
        dw_in, dw_out = torch.empty_like(w_in), torch.empty_like(w_out)
        dw_hid = None if w_hid is None else torch.empty_like(w_hid)
        ws_bytes = _lib.lib().th_mlp_workspace_bytes(D_in, D_hidden, D_out, ctx.depth)
        workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=device)
        with torch.cuda.device(device):
            _lib.check(
                _lib.lib().th_mlp_bwd(
                    x.data_ptr(), x.stride(1), w_in.data_ptr(), None, _lib.ptr(w_hid), None, w_out.data_ptr(), None,
                    grad.data_ptr(), D_out, _lib.ptr(dx), D_in, dw_in.data_ptr(), None, _lib.ptr(dw_hid), None,
                    dw_out.data_ptr(), None, workspace.data_ptr(), ws_bytes, B * L, D_in, D_hidden, D_out, ctx.depth,
                    _lib.ACTIVATION_CODE[ctx.activation], _lib.DTYPE_CODE[dtype], 0, _lib.stream_ptr(device),
                ),
                "th_mlp_bwd",
            )  # fmt: skip
        return dx, dw_in, dw_out, dw_hid, None, None, None


def fully_fused_mlp_mse(
    x: Tensor,
    w_in: Tensor,
    w_out: Tensor,
    w_hid: Optional[Tensor],
    target: Tensor,
    grad_scale: float = 1.0,
    activation: str = "relu",
) -> Tensor:
    r"""Bias-free MLP forward with the squared-error loss fused into its output layer.

    Returns ``loss_sum = sum((mlp(x) - target) ** 2)`` as a one-element float32 tensor; the prediction
    is never written to memory.  What the kernel does write is ``(mlp(x) - target) * grad_scale`` in
    the 16-bit dtype, and ``loss_sum.backward()`` back-propagates exactly that tensor: the gradients
    it leaves are those of ``grad_scale / 2 * loss_sum`` (a training loop folds the factor into its
    optimiser step, as ``training.NeuralFieldTrainer`` does, so that 16-bit gradients neither
    underflow nor overflow).  The incoming gradient of ``loss_sum`` is taken to be one.
    triton_helpers has no such function; it is the fusion of ``fully_fused_mlp`` with the loss
    that follows it in a regression loop.

    Shapes:
        - x: :math:`(B, L, D_{in})`, target: :math:`(B, L, D_{out})`, weights as in ``fully_fused_mlp``.
    """
    activation = ensure_str(activation)
    assert activation in ACTIVATIONS, f"Invalid activation function: {activation}"
    return _fully_fused_mlp_mse.apply(x, w_in, w_out, w_hid, target, float(grad_scale), activation)
