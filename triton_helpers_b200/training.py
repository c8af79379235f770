r"""Neural-field training step: hash encoding -> fused MLP -> MSE -> backward -> gradient sum -> Adam.

The step benchmark configuration 3 describes, built only from this package's operators.  It
has no counterpart in triton_helpers (which stops at the two layers); the layers it drives are
the drop-in ``HashEncoding`` and ``FullyFusedMLP`` modules, so everything between the coordinates
and the parameter update runs in the hand-written kernels: ``th_hash_fwd``, ``th_mlp_fwd``,
``th_mse_grad``, ``th_mlp_bwd``, ``th_hash_bwd``, ``th_adam_step``.  With more than one process
the point batch is split across ranks, parameters are replicated and their gradients summed once
per step (``parallel.allreduce_gradients``).
"""
from typing import Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn
from torch import Tensor

from . import _lib
from .layers.fully_fused_mlp import FullyFusedMLP, fully_fused_mlp_mse
from .layers.hash_encoding import HashEncoding
from .layers.hash_encoding.helpers import level_geometry
from .layers.hash_encoding.kernel import hash_encoding_backward_levels
from .optim import FusedAdam
from .parallel import PendingReduce, allreduce_gradients, level_passes


@torch.no_grad()
def mse_grad(pred: Tensor, target: Tensor, grad_scale: float) -> Tuple[Tensor, Tensor]:
    r"""``(grad, loss_sum)``: ``grad = (pred - target) * grad_scale`` in ``pred``'s dtype and the
    float32 sum of squared differences (a one-element device tensor), in one kernel."""
    assert pred.shape == target.shape and pred.dtype == target.dtype, "Prediction / target mismatch"
    device = _lib.require_cuda(pred, target)
    pred, target = pred.contiguous(), target.contiguous()
    grad = torch.empty_like(pred)
    loss_sum = torch.zeros(1, dtype=torch.float32, device=device)
    with torch.cuda.device(device):
        _lib.check(
            _lib.lib().th_mse_grad(
                pred.data_ptr(), target.data_ptr(), grad.data_ptr(), loss_sum.data_ptr(), pred.numel(), grad_scale,
                _lib.dtype_code(pred), _lib.stream_ptr(device),
            ),
            "th_mse_grad",
        )  # fmt: skip
    return grad, loss_sum


class NeuralFieldTrainer(nn.Module):
    r"""Hash-encoded MLP regressed on targets with MSE and Adam.

    Args:
        encoding, mlp: the two layers (moved to the device and dtype the caller wants; float16
            tables and weights for benchmark configuration 3).
        lr, betas, eps: Adam hyper-parameters.
        grad_out_scale: the MLP receives ``(pred - target) * grad_out_scale`` as its output
            gradient, i.e. the loss is scaled so 16-bit gradients neither underflow nor overflow;
            Adam undoes the scale exactly.
        group: process group for data parallelism (``None``: the default group, if initialised).
        backward_passes: ``None`` (default): one backward through autograd, then one gradient sum over
            the ranks.  An integer n: the encoding backward runs in n level ranges, finest first; the
            gradient rows of a finished range are summed over the ranks (NCCL, asynchronously) while
            the kernels of the next range run, and the MLP gradients are summed under the whole
            encoding backward.  Measured on 2 B200 with the cfg 3 step: 2.08 ms per step with n = 2
            against 2.07 ms without - the sum of 24 MB over NVLink takes about as long as the second
            pass over the points costs extra - so overlapping is left to the caller to switch on
            (slower interconnects, larger tables).
    """

    def __init__(
        self,
        encoding: HashEncoding,
        mlp: FullyFusedMLP,
        lr: float = 1e-2,
        betas: Tuple[float, float] = (0.9, 0.99),
        eps: float = 1e-15,
        grad_out_scale: float = 1.0 / 16.0,
        group: Optional[dist.ProcessGroup] = None,
        backward_passes: Optional[int] = None,
    ):
        super().__init__()
        self.encoding = encoding
        self.mlp = mlp
        self.grad_out_scale = grad_out_scale
        self.group = group
        self.backward_passes = backward_passes
        self.optimizer = FusedAdam(self.parameters(), lr=lr, betas=betas, eps=eps)

    def world_size(self) -> int:
        return dist.get_world_size(self.group) if dist.is_available() and dist.is_initialized() else 1

    def forward(self, coords: Tensor) -> Tensor:
        r"""Prediction ``(N, d_out)`` for coordinates ``(N, D)``."""
        return self.mlp(self.encoding(coords).unsqueeze(0)).squeeze(0)

    def step(self, coords: Tensor, targets: Tensor) -> Tensor:
        r"""One optimisation step on this rank's points; returns the local mean squared error
        (float32, on the device, not synchronised)."""
        world = self.world_size()
        passes = self.backward_passes
        if passes is None:
            n_values, loss_sum = self._backward_through_autograd(coords, targets)
        else:
            n_values, loss_sum = self._backward_in_level_passes(coords, targets, passes)
        # d(mean over the global batch)/d pred = 2 (pred - target) / (N_global * C)
        true_over_stored = 2.0 / (n_values * world * self.grad_out_scale)
        self.optimizer.step(grad_scale=true_over_stored)
        for p in self.parameters():
            p.grad = None
        return loss_sum / n_values

    def _fusable(self) -> bool:
        r"""Whether the MLP's last layer and the loss can share a kernel (bias-free 16-bit network)."""
        mlp = self.mlp
        return mlp.b_in is None and mlp.w_in.dtype in (torch.float16, torch.bfloat16)

    def _loss_backward(self, feats: Tensor, targets: Tensor) -> Tuple[int, Tensor]:
        r"""MLP forward, squared error and the whole backward below ``feats``' producer.  Returns the
        number of predicted values and the float32 sum of squared errors."""
        mlp = self.mlp
        if self._fusable():
            loss_sum = fully_fused_mlp_mse(
                feats.unsqueeze(0), mlp.w_in, mlp.w_out, mlp.w_hid, targets.to(feats.dtype).unsqueeze(0),
                self.grad_out_scale, mlp.activation,
            )  # fmt: skip
            loss_sum.backward()
            return targets.numel(), loss_sum.detach()
        pred = mlp(feats.unsqueeze(0)).squeeze(0)
        grad_out, loss_sum = mse_grad(pred, targets.to(pred.dtype), self.grad_out_scale)
        pred.backward(grad_out)
        return pred.numel(), loss_sum

    def _backward_through_autograd(self, coords: Tensor, targets: Tensor) -> Tuple[int, Tensor]:
        n_values, loss_sum = self._loss_backward(self.encoding(coords), targets)
        allreduce_gradients([p.grad for p in self.parameters() if p.grad is not None], self.group)
        return n_values, loss_sum

    def _backward_in_level_passes(self, coords: Tensor, targets: Tensor, n_passes: int) -> Tuple[int, Tensor]:
        r"""The same gradients with the exchange overlapped: autograd covers the MLP only; the encoding
        backward is launched range by range (finest levels first) and each finished range of table
        rows goes to an asynchronous all-reduce while the next range is computed."""
        enc = self.encoding
        with torch.no_grad():
            feats = enc(coords)
        feats.requires_grad_(True)
        n_values, loss_sum = self._loss_backward(feats, targets)
        pending = PendingReduce(self.group)
        pending.start([p.grad for p in self.mlp.parameters() if p.grad is not None])
        table = enc.embeddings
        geo = level_geometry(enc.num_levels, enc.max_entries_per_level, coords.shape[-1], enc.min_res, enc.max_res)
        grad_table = torch.zeros_like(table)
        for begin, end in level_passes(geo.rows, n_passes):
            hash_encoding_backward_levels(
                coords, feats.grad, grad_table, enc.pi, enc.max_entries_per_level, enc.min_res, enc.max_res,
                enc.num_levels, begin, end,
            )  # fmt: skip
            first_row = geo.offsets[begin]
            last_row = geo.offsets[end - 1] + geo.rows[end - 1]
            pending.start([grad_table[first_row:last_row]])
        pending.finish()
        table.grad = grad_table
        return n_values, loss_sum
