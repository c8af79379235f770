r"""Neural-field training step: hash encoding -> fused MLP -> MSE -> backward -> gradient sum -> Adam.

The step benchmark configuration 3 describes, built only from this package's operators.  It
has no counterpart in triton_helpers (which stops at the two layers); the layers it drives are
the drop-in ``HashEncoding`` and ``FullyFusedMLP`` modules.

Two ways through the step:

* **direct** (table and MLP share one 16-bit dtype): the trainer calls the C ABI itself on buffers it
  keeps from step to step - by default the fused pair ``th_field_fwd`` (encoding + MLP + loss) and
  ``th_field_bwd`` (MLP backward + encoding backward), else ``th_hash_fwd``, ``th_mlp_fwd_mse``,
  ``th_mlp_bwd``, ``th_hash_bwd``; then ``th_scale_cast`` and ``th_adam_step``.  All gradients live in ONE flat 16-bit
  buffer ``[table gradient | MLP gradients]`` so that a step costs one all-reduce:

  - the table part holds ``grad_out_scale * sum over the local batch`` (the encoding backward adds
    into it with 16-bit reductions; Adam clears it in the pass that consumes it);
  - the MLP part holds the MEAN over the local batch of the unscaled gradient: the float32 sums
    ``th_mlp_bwd`` leaves in its workspace are divided by ``rows * grad_out_scale`` before they are
    rounded.  A sum over 2^21 rows reaches 1e4..1e5 and four ranks of that exceed float16's 65504;
    means stay below one at any batch size and world size.

* **autograd** (float32 parameters): forward and backward through the layers' autograd functions,
  ``parallel.allreduce_gradients`` on the float32 gradients.

With more than one process the point batch is split across ranks (every rank passes the same
number of points), parameters are replicated and their gradients summed once per step.
"""
import math
from typing import List, Optional, Tuple, Union

import torch
import torch.distributed as dist
import torch.nn as nn
from torch import Tensor

from . import _lib
from .layers.fully_fused_mlp import FullyFusedMLP
from .layers.hash_encoding import HashEncoding
from .layers.hash_encoding.kernel import _Launch
from .layers.neural_field.kernel import FieldUnsupported, field_backward, field_forward
from .optim import FusedAdam, adam_update
from .parallel import PendingReduce, allreduce_gradients, gradient_scales, level_passes


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


def default_grad_out_scale(global_points: int) -> float:
    r"""Loss scale for 16-bit table gradients: the power of two nearest below ``2^18 / global_points``,
    kept within ``[2^-8, 1]``.  A row of the coarsest level collects a share of EVERY point of every
    rank, so its 16-bit sum grows with the global batch (measured on the float32 CPU port of
    configuration 3: max |row sum| = 260 per 2^19 points at unit scale); dividing the scale by the
    batch keeps that sum near 130 whatever the number of ranks, two orders of magnitude inside
    float16's range, while single contributions on the fine levels (1e-4 .. 1 at unit scale) stay
    representable."""
    scale = 2.0 ** math.floor(math.log2(max(2.0**18 / max(global_points, 1), 2.0**-8)))
    return min(scale, 1.0)


class NeuralFieldTrainer(nn.Module):
    r"""Hash-encoded MLP regressed on targets with MSE and Adam.

    Args:
        encoding, mlp: the two layers (moved to the device and dtype the caller wants; float16
            tables and weights for benchmark configuration 3).  In direct mode the MLP's parameters
            are re-pointed into one flat buffer (their values, names and shapes are unchanged).
        lr, betas, eps: Adam hyper-parameters.
        grad_out_scale: the MLP receives ``(pred - target) * grad_out_scale`` as its output
            gradient, i.e. the loss is scaled so 16-bit table gradients neither underflow nor
            overflow; Adam undoes the scale exactly.  ``None``: ``default_grad_out_scale`` of the
            global batch of the first step.
        group: process group for data parallelism (``None``: the default group, if initialised).
        fused: direct mode only; which steps run in the kernels that fuse the encoding with the MLP.
            ``None`` (default): the backward pass when the fused kernel covers the configuration (measured
            at benchmark configuration 3 on a B200: fused backward 1.04 ms against 0.36 + 0.78 ms for MLP
            backward + encoding backward; fused forward 0.71 ms against 0.55 + 0.12 ms, so the forward stays
            separate); ``"backward"``: the same, but raise if it is not covered; ``True``: forward and
            backward fused, raise if not covered; ``False``: always the separate operators.
        backward_passes: ``None`` (default): one encoding backward, then one gradient sum over the
            ranks.  An integer n (direct mode): the encoding backward runs in n level ranges, finest
            first; the gradient rows of a finished range are summed over the ranks (NCCL,
            asynchronously) while the kernels of the next range run, and the MLP gradients travel
            with the first range.  Measured on 2 and 8 B200 with the cfg 3 step it gains nothing -
            the sum of 24 MB over NVLink takes about as long as the second pass over the points
            costs extra - so it is left to the caller to switch on (slower interconnects, larger tables).
    """

    def __init__(
        self,
        encoding: HashEncoding,
        mlp: FullyFusedMLP,
        lr: float = 1e-2,
        betas: Tuple[float, float] = (0.9, 0.99),
        eps: float = 1e-15,
        grad_out_scale: Optional[float] = None,
        group: Optional[dist.ProcessGroup] = None,
        backward_passes: Optional[int] = None,
        fused: Union[None, bool, str] = None,
    ):
        super().__init__()
        self.fused = fused
        self._no_fused_forward = self._no_fused_backward = False
        self.encoding = encoding
        self.mlp = mlp
        self.grad_out_scale = grad_out_scale
        self.group = group
        self.backward_passes = backward_passes
        self.lr, self.betas, self.eps = lr, betas, eps
        table_dtype, mlp_dtype = encoding.embeddings.dtype, mlp.w_in.dtype
        sixteen = (torch.float16, torch.bfloat16)
        if table_dtype == mlp_dtype and table_dtype in sixteen:
            self.direct = True
        elif table_dtype in sixteen or mlp_dtype in sixteen:
            raise ValueError(
                "NeuralFieldTrainer takes a table and an MLP of one 16-bit dtype, or float32 for both "
                f"(got {table_dtype} and {mlp_dtype}): unnormalised 16-bit MLP gradients cannot be summed over ranks"
            )
        else:
            self.direct = False
        self.optimizer = None if self.direct else FusedAdam(self.parameters(), lr=lr, betas=betas, eps=eps)
        self._state = None  # direct mode: buffers, created on the first step
        self._steps = 0

    def world_size(self) -> int:
        return dist.get_world_size(self.group) if dist.is_available() and dist.is_initialized() else 1

    def forward(self, coords: Tensor) -> Tensor:
        r"""Prediction ``(N, d_out)`` for coordinates ``(N, D)``."""
        return self.mlp(self.encoding(coords).unsqueeze(0)).squeeze(0)

    def skipped_elements(self) -> int:
        r"""Parameter elements Adam has passed over so far because their gradient was not finite
        (reads the device: synchronises).  Zero in a healthy run."""
        if self.direct:
            return 0 if self._state is None else int(self._state.skipped.item())
        return self.optimizer.skipped_elements()

    def step(self, coords: Tensor, targets: Tensor) -> Tensor:
        r"""One optimisation step on this rank's points; returns the local mean squared error
        (float32, on the device, not synchronised)."""
        if self.grad_out_scale is None:
            self.grad_out_scale = default_grad_out_scale(coords.shape[0] * self.world_size())
        self._steps += 1
        return self._step_direct(coords, targets) if self.direct else self._step_autograd(coords, targets)

    # ---- autograd mode (float32 parameters) --------------------------------------------------------

    def _step_autograd(self, coords: Tensor, targets: Tensor) -> Tensor:
        world = self.world_size()
        pred = self.mlp(self.encoding(coords).unsqueeze(0)).squeeze(0)
        grad_out, loss_sum = mse_grad(pred, targets.to(pred.dtype), self.grad_out_scale)
        pred.backward(grad_out)
        allreduce_gradients([p.grad for p in self.parameters() if p.grad is not None], self.group)
        # d(mean over the global batch)/d pred = 2 (pred - target) / (N_global * C)
        self.optimizer.step(grad_scale=2.0 / (pred.numel() * world * self.grad_out_scale))
        for p in self.parameters():
            p.grad = None
        return loss_sum / pred.numel()

    # ---- direct mode (one 16-bit dtype) ------------------------------------------------------------

    def _step_direct(self, coords: Tensor, targets: Tensor) -> Tensor:
        st = self._prepare(coords)
        enc, mlp, lib = self.encoding, self.mlp, _lib.lib()
        device, dtype = st.device, st.dtype
        n, world, scale = coords.shape[0], self.world_size(), float(self.grad_out_scale)
        targets = targets.to(dtype)
        if targets.stride(-1) != 1:
            targets = targets.contiguous()
        d_coord = coords.shape[1]
        launch = _Launch(coords, st.primes, d_coord, enc.max_entries_per_level, enc.num_levels, enc.min_res, enc.max_res, 1.0)
        cast_scale, table_adam_scale, mlp_adam_scale = gradient_scales(n, world, st.d_out, scale)
        code, act = _lib.dtype_code(st.flat_grad), _lib.ACTIVATION_CODE[mlp.activation]
        mlp_ptrs = (st.w_in.data_ptr(), _lib.ptr(st.b_in), _lib.ptr(st.w_hid), _lib.ptr(st.b_hid), st.w_out.data_ptr(), _lib.ptr(st.b_out))
        dims = (st.d_feat, st.d_hidden, st.d_out, st.depth)
        fuse_fwd, fuse_bwd = self._fusion_plan(st)
        with torch.cuda.device(device):
            stream = _lib.stream_ptr(device)
            st.loss_sum.zero_()
            geometry = (launch.n, d_coord, st.n_feats, enc.num_levels, launch.res, launch.rows, launch.offsets, launch.primes, launch.scale)
            weights = (st.w_in, st.w_out, st.w_hid)
            # ---- forward: encoding, MLP, loss ----
            if fuse_fwd:
                try:
                    field_forward(launch, enc.embeddings.data, *weights, mlp.activation, enc.num_levels, feats_out=st.feats,
                                  target=targets, grad_out=st.grad_pred, loss_sum=st.loss_sum, grad_scale=scale,
                                  biases=(st.b_in, st.b_hid, st.b_out))  # fmt: skip
                except FieldUnsupported:
                    if self.fused is True:
                        raise
                    self._no_fused_forward = True  # nothing was launched: the separate operators from now on
                    fuse_fwd = False
            if not fuse_fwd:
                _lib.check(
                    lib.th_hash_fwd(*launch.coord_args, enc.embeddings.data_ptr(), code, st.feats.data_ptr(), st.d_feat,
                                    *geometry, 0, enc.num_levels, stream),
                    "th_hash_fwd",
                )  # fmt: skip
                rc = lib.th_mlp_fwd_mse(
                    st.feats.data_ptr(), st.d_feat, *mlp_ptrs, None, st.d_out, targets.data_ptr(), targets.stride(0),
                    st.grad_pred.data_ptr(), st.d_out, st.loss_sum.data_ptr(), scale, n, *dims, act, code, stream,
                )  # fmt: skip
                if rc == _lib.TH_ERR_UNSUPPORTED:  # shapes the fused forward + loss does not take: the two kernels it stands for
                    _lib.check(lib.th_mlp_fwd(st.feats.data_ptr(), st.d_feat, *mlp_ptrs, st.pred.data_ptr(), st.d_out, n, *dims, act, code, 0, stream), "th_mlp_fwd")
                    t = targets.contiguous()
                    _lib.check(lib.th_mse_grad(st.pred.data_ptr(), t.data_ptr(), st.grad_pred.data_ptr(), st.loss_sum.data_ptr(), n * st.d_out, scale, code, stream), "th_mse_grad")
                else:
                    _lib.check(rc, "th_mlp_fwd_mse")
            # ---- backward: MLP, then the encoding's table gradient into the flat buffer ----
            if fuse_bwd:
                try:
                    field_backward(launch, st.feats, st.grad_pred, *weights, mlp.activation, enc.num_levels, st.table_grad, st.workspace)
                except FieldUnsupported:
                    if self.fused in (True, "backward"):
                        raise
                    self._no_fused_backward = True
                    fuse_bwd = False
            if not fuse_bwd:
                _lib.check(
                    lib.th_mlp_bwd(st.feats.data_ptr(), st.d_feat, *mlp_ptrs, st.grad_pred.data_ptr(), st.d_out, st.grad_feats.data_ptr(),
                                   st.d_feat, None, None, None, None, None, None, st.workspace.data_ptr(), st.workspace.numel() * 4,
                                   n, *dims, act, code, 0, stream),
                    "th_mlp_bwd",
                )  # fmt: skip
            # float32 sums over this rank's rows -> mean of the unscaled gradient, rounded into the flat buffer's tail
            _lib.check(lib.th_scale_cast(st.workspace.data_ptr(), st.mlp_grad.data_ptr(), st.mlp_grad.numel(), cast_scale, code, stream), "th_scale_cast")
            pending = PendingReduce(self.group, bucket_bytes=0)
            if fuse_bwd:
                pending.start([st.flat_grad])
            else:
                passes = [(0, enc.num_levels)] if not self.backward_passes else level_passes(launch.geo.rows, self.backward_passes)
                for i, (begin, end) in enumerate(passes):  # finest first
                    _lib.check(
                        lib.th_hash_bwd(*launch.coord_args, st.grad_feats.data_ptr(), st.d_feat, st.table_grad.data_ptr(), code,
                                        *geometry, begin, end, stream),
                        "th_hash_bwd",
                    )  # fmt: skip
                    first = launch.geo.offsets[begin] * st.n_feats
                    last = st.flat_grad.numel() if i == 0 else (launch.geo.offsets[end - 1] + launch.geo.rows[end - 1]) * st.n_feats
                    pending.start([st.flat_grad[first:last]])  # one collective per range; the first carries the MLP gradients
            pending.finish()
        adam_update(enc.embeddings.data.view(-1), st.table_grad.view(-1), st.table_m, st.table_v, self._steps, self.lr, self.betas,
                    self.eps, table_adam_scale, True, st.skipped)  # fmt: skip
        adam_update(st.mlp_flat, st.mlp_grad, st.mlp_m, st.mlp_v, self._steps, self.lr, self.betas, self.eps, mlp_adam_scale, False, st.skipped)
        return st.loss_sum / (n * st.d_out)

    def _fusion_plan(self, st: "_DirectState") -> Tuple[bool, bool]:
        r"""(fused forward?, fused backward?) for this step; see ``fused`` in the class docstring."""
        mode = self.fused
        if mode is False:
            return False, False
        want_fwd = mode is True
        want_bwd = mode in (None, True, "backward")
        if st.b_in is not None or self.backward_passes:
            # the fused backward is built for bias-free networks; level-range passes need the separate encoding backward
            if mode in (True, "backward"):
                raise FieldUnsupported("the fused backward takes bias-free networks and one pass over all levels")
            want_bwd = False
        return want_fwd and not self._no_fused_forward, want_bwd and not self._no_fused_backward

    def _prepare(self, coords: Tensor) -> "_DirectState":
        st = self._state
        if st is None:
            st = self._state = _DirectState(self.encoding, self.mlp)
        assert coords.ndim == 2 and 1 <= coords.shape[1] <= 3, "coordinates must be (N, D) with D in 1..3"
        st.resize(coords.shape[0])
        return st


class _DirectState:
    r"""Buffers the direct step keeps: the flat gradient, Adam moments, the MLP's flat parameter
    buffer, per-batch intermediates."""

    def __init__(self, enc: HashEncoding, mlp: FullyFusedMLP):
        table = enc.embeddings
        self.device, self.dtype = table.device, table.dtype
        _lib.require_cuda(table, mlp.w_in)
        assert table.is_contiguous(), "the embedding table must be contiguous"
        self.n_feats = table.shape[1]
        self.primes = enc.pi
        self.d_hidden, self.d_feat = mlp.w_in.shape
        self.d_out = mlp.w_out.shape[0]
        self.depth = 1 if mlp.w_hid is None else mlp.w_hid.shape[0] // self.d_hidden + 1
        assert self.d_feat == enc.num_levels * self.n_feats, "the MLP's input width must be levels * features"

        # MLP parameters in one flat buffer, in the order of th_mlp_bwd's workspace
        has_bias = mlp.b_in is not None
        ordered: List[Tuple[str, Optional[nn.Parameter]]] = [("w_in", mlp.w_in), ("w_hid", mlp.w_hid), ("w_out", mlp.w_out)]
        if has_bias:
            ordered += [("b_in", mlp.b_in), ("b_hid", mlp.b_hid), ("b_out", mlp.b_out)]
        total = _lib.lib().th_mlp_workspace_bytes(self.d_feat, self.d_hidden, self.d_out, self.depth) // 4
        self.mlp_flat = torch.zeros(total, dtype=self.dtype, device=self.device)
        table_elems = table.numel()
        tail = (table_elems + 15) // 16 * 16  # 32-byte aligned start of the MLP part
        self.flat_grad = torch.zeros(tail + total, dtype=self.dtype, device=self.device)
        self.table_grad = self.flat_grad[:table_elems].view_as(table)
        self.mlp_grad = self.flat_grad[tail:]
        offset = 0
        for name, p in ordered:
            setattr(self, name, None)
            if p is None:
                continue
            view = self.mlp_flat[offset : offset + p.numel()].view_as(p)
            view.copy_(p.data)
            p.data = view
            p.grad = self.mlp_grad[offset : offset + p.numel()].view_as(p)
            setattr(self, name, view)
            offset += p.numel()
        if not has_bias:
            self.b_in = self.b_hid = self.b_out = None
        table.grad = self.table_grad
        f32 = dict(dtype=torch.float32, device=self.device)
        self.table_m, self.table_v = torch.zeros(table_elems, **f32), torch.zeros(table_elems, **f32)
        self.mlp_m, self.mlp_v = torch.zeros(total, **f32), torch.zeros(total, **f32)
        self.workspace = torch.zeros(total, **f32)
        self.loss_sum = torch.zeros(1, **f32)
        self.skipped = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.rows = -1

    def resize(self, n: int) -> None:
        if n == self.rows:
            return
        kw = dict(dtype=self.dtype, device=self.device)
        self.feats = torch.empty(n, self.d_feat, **kw)
        self.grad_feats = torch.empty(n, self.d_feat, **kw)
        self.grad_pred = torch.empty(n, self.d_out, **kw)
        self.pred = torch.empty(n, self.d_out, **kw)
        self.rows = n
