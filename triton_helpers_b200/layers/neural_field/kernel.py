r"""Hash encoding and fused MLP in one kernel per direction (``th_field_fwd`` / ``th_field_bwd``).

triton_helpers has no such operator: it launches ``hash_encoding`` and ``fully_fused_mlp`` one after the
other and notes that the encoding is meant to feed a fully fused MLP with its ``L * F`` columns staying on
chip (``triton_helpers/layers/hash_encoding/kernel.py:241-243``).  ``hash_encoded_mlp(coords, embeddings,
w_in, w_out, w_hid, ...)`` computes ``fully_fused_mlp(hash_encoding(coords, embeddings, ...), w_in, None,
w_out, None, w_hid, None, activation)`` - same arguments, same values, same gradients - without the
encoding making a round trip through memory between the two.

Covered by the fused kernels: one 16-bit dtype for table and weights, 2 or 3 coordinate dimensions, 2 or 4
features per level, ``levels * features`` a multiple of 16, ReLU or no activation, no biases.  Other
configurations raise ``FieldUnsupported``; callers fall back to the two separate layers.
"""
from typing import Optional, Tuple

import torch
from torch import Tensor

from ... import _lib
from ...ops import ensure_str
from ..hash_encoding.kernel import _default_pi, _Launch


class FieldUnsupported(RuntimeError):
    r"""The configuration is outside what the fused kernels are built for."""


def _check(code: int, what: str) -> None:
    if code == _lib.TH_ERR_UNSUPPORTED:
        raise FieldUnsupported(_lib.lib().th_last_error_string().decode(errors="replace"))
    _lib.check(code, what)


def _mlp_dims(w_in: Tensor, w_out: Tensor, w_hid: Optional[Tensor]) -> Tuple[int, int, int, int]:
    d_hidden, d_in = w_in.shape
    d_out = w_out.shape[0]
    depth = 1 if w_hid is None or w_hid.numel() == 0 else w_hid.shape[0] // d_hidden + 1
    return d_in, d_hidden, d_out, depth


@torch.no_grad()
def field_forward(
    launch: _Launch,
    table: Tensor,
    w_in: Tensor,
    w_out: Tensor,
    w_hid: Optional[Tensor],
    activation: str,
    levels: int,
    feats_out: Optional[Tensor] = None,
    out: Optional[Tensor] = None,
    target: Optional[Tensor] = None,
    grad_out: Optional[Tensor] = None,
    loss_sum: Optional[Tensor] = None,
    grad_scale: float = 1.0,
    biases: Tuple[Optional[Tensor], Optional[Tensor], Optional[Tensor]] = (None, None, None),
) -> None:
    r"""One ``th_field_fwd`` launch on caller-owned buffers (all contiguous, on ``table``'s device).

    ``launch`` carries the coordinates and level geometry (``hash_encoding.kernel._Launch``).  Writes
    ``feats_out (N, L*F)`` when given, ``out (N, d_out)`` when given, and - when ``target`` is given -
    ``grad_out = (prediction - target) * grad_scale`` and adds the squared error to ``loss_sum``.
    ``biases = (b_in, b_hid, b_out)``.
    """
    d_in, d_hidden, d_out, depth = _mlp_dims(w_in, w_out, w_hid)
    device = _lib.require_cuda(table, w_in, w_out, w_hid, feats_out, out, target, grad_out, loss_sum, *biases)
    D, F = launch.coords2d.shape[1], table.shape[1]
    assert d_in == levels * F, "the MLP's input width must be levels * features"
    with torch.cuda.device(device):
        _check(
            _lib.lib().th_field_fwd(
                *launch.coord_args, table.data_ptr(), D, F, levels, launch.res, launch.rows, launch.offsets, launch.primes,
                launch.scale, w_in.data_ptr(), _lib.ptr(biases[0]), _lib.ptr(w_hid), _lib.ptr(biases[1]), w_out.data_ptr(),
                _lib.ptr(biases[2]), d_hidden, d_out, depth, _lib.ACTIVATION_CODE[activation],
                _lib.ptr(feats_out), d_in if feats_out is None else feats_out.stride(0),
                _lib.ptr(out), d_out if out is None else out.stride(0),
                _lib.ptr(target), d_out if target is None else target.stride(0),
                _lib.ptr(grad_out), d_out if grad_out is None else grad_out.stride(0),
                _lib.ptr(loss_sum), grad_scale, launch.n, _lib.dtype_code(table), _lib.stream_ptr(device),
            ),
            "th_field_fwd",
        )  # fmt: skip


@torch.no_grad()
def field_backward(
    launch: _Launch,
    feats: Tensor,
    grad_out: Tensor,
    w_in: Tensor,
    w_out: Tensor,
    w_hid: Optional[Tensor],
    activation: str,
    levels: int,
    grad_table: Tensor,
    workspace: Tensor,
    grad_feats: Optional[Tensor] = None,
) -> None:
    r"""One ``th_field_bwd`` launch: adds the table gradient into ``grad_table`` (zero-initialised by the
    caller, shaped and typed like the table), leaves the float32 weight-gradient sums in ``workspace``
    (``[w_in | w_hid | w_out]``, zero-filled by the call) and, when given, writes the feature gradient."""
    d_in, d_hidden, d_out, depth = _mlp_dims(w_in, w_out, w_hid)
    device = _lib.require_cuda(feats, grad_out, w_in, w_out, w_hid, grad_table, workspace, grad_feats)
    D, F = launch.coords2d.shape[1], grad_table.shape[1]
    with torch.cuda.device(device):
        _check(
            _lib.lib().th_field_bwd(
                *launch.coord_args, D, F, levels, launch.res, launch.rows, launch.offsets, launch.primes, launch.scale,
                w_in.data_ptr(), _lib.ptr(w_hid), w_out.data_ptr(), d_hidden, d_out, depth, _lib.ACTIVATION_CODE[activation],
                feats.data_ptr(), feats.stride(0), grad_out.data_ptr(), grad_out.stride(0), grad_table.data_ptr(),
                _lib.ptr(grad_feats), d_in if grad_feats is None else grad_feats.stride(0), workspace.data_ptr(),
                workspace.numel() * workspace.element_size(), launch.n, _lib.dtype_code(grad_table), _lib.stream_ptr(device),
            ),
            "th_field_bwd",
        )  # fmt: skip


class HashEncodedMLP(torch.autograd.Function):

    @staticmethod
    def forward(ctx, coords, embeddings, w_in, w_out, w_hid, pi, max_entries_per_level, min_res, max_res, levels, activation, scale):
        D = coords.shape[-1]
        if pi is None:
            pi = _default_pi(coords.device)
        assert not coords.requires_grad, "Gradients not supported for coords"
        dtype = embeddings.dtype
        assert all(t is None or t.dtype == dtype for t in (w_in, w_out, w_hid)), "table and weights must share one dtype"
        launch = _Launch(coords, pi, D, max_entries_per_level, levels, min_res, max_res, scale)
        table = embeddings if embeddings.is_contiguous() else embeddings.contiguous()
        w_in, w_out = w_in.contiguous(), w_out.contiguous()
        w_hid = None if w_hid is None or w_hid.numel() == 0 else w_hid.contiguous()
        d_in, _, d_out, _ = _mlp_dims(w_in, w_out, w_hid)
        needs_grad = any(ctx.needs_input_grad)
        feats = embeddings.new_empty(launch.n, d_in) if needs_grad else None
        out = embeddings.new_empty(launch.n, d_out)
        field_forward(launch, table, w_in, w_out, w_hid, activation, levels, feats_out=feats, out=out)
        ctx.save_for_backward(coords, embeddings, w_in, w_out, w_hid, feats)
        ctx.geometry = (launch.prime_values, max_entries_per_level, min_res, max_res, levels, activation, scale)
        return out.view(*coords.shape[:-1], d_out)

    @staticmethod
    @torch.no_grad()
    def backward(ctx, do: Tensor):
        coords, embeddings, w_in, w_out, w_hid, feats = ctx.saved_tensors
        primes, cap, min_res, max_res, levels, activation, scale = ctx.geometry
        launch = _Launch(coords, primes, coords.shape[-1], cap, levels, min_res, max_res, scale)
        d_in, d_hidden, d_out, depth = _mlp_dims(w_in, w_out, w_hid)
        go = do.reshape(-1, d_out).to(embeddings.dtype)
        if go.stride(-1) != 1 or (go.shape[0] > 1 and go.stride(0) < d_out):
            go = go.contiguous()
        de = torch.zeros(embeddings.shape, dtype=embeddings.dtype, device=embeddings.device)
        ws_bytes = _lib.lib().th_field_workspace_bytes(levels, embeddings.shape[1], d_hidden, d_out, depth)
        workspace = torch.empty(ws_bytes // 4, dtype=torch.float32, device=embeddings.device)
        field_backward(launch, feats, go, w_in, w_out, w_hid, activation, levels, de, workspace)
        # float32 sums -> gradients in the parameter dtype, as the separate layers return them
        sizes = [w_in.numel(), 0 if w_hid is None else w_hid.numel(), w_out.numel()]
        parts = torch.split(workspace[: sum(sizes)], sizes)
        dw_in = parts[0].view_as(w_in).to(w_in.dtype)
        dw_hid = None if w_hid is None else parts[1].view_as(w_hid).to(w_hid.dtype)
        dw_out = parts[2].view_as(w_out).to(w_out.dtype)
        return None, de, dw_in, dw_out, dw_hid, None, None, None, None, None, None, None


def hash_encoded_mlp(
    coord: Tensor,
    embeddings: Tensor,
    w_in: Tensor,
    w_out: Tensor,
    w_hid: Optional[Tensor] = None,
    pi: Optional[Tensor] = None,
    max_entries_per_level: int = 2**14,
    min_res: int = 16,
    max_res: int = 512,
    levels: int = 16,
    activation: str = "relu",
    scale: float = 1.0,
) -> Tensor:
    r"""``fully_fused_mlp(hash_encoding(coord, embeddings, ...), w_in, None, w_out, None, w_hid, None, activation)``
    in one kernel per direction.  Arguments are those of the two functions (bias-free network); output
    ``(..., D_out)``.  Raises ``FieldUnsupported`` for configurations the fused kernels do not cover."""
    return HashEncodedMLP.apply(
        coord, embeddings, w_in, w_out, w_hid, pi, max_entries_per_level, min_res, max_res, levels, ensure_str(activation), scale
    )
