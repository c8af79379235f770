r"""Multiresolution hash encoding (Instant-NGP) on hand-written sm_100a kernels.

Drop-in for ``triton_helpers/layers/hash_encoding/kernel.py``: ``HashEncoding`` is the
``torch.autograd.Function`` (reference :509-675) and ``hash_encoding`` the functional
wrapper (reference :678-728), with the same positional arguments, defaults, assertions
and gradient tuple.  The Triton launches are replaced by ``th_hash_fwd`` / ``th_hash_bwd``
of ``libth_b200.so``; nothing here falls back to PyTorch or the CPU.

Differences a caller can observe:

* ``divider`` / ``bwd_divider`` are honoured as the number of levels per kernel pass when
  given, but nothing is autotuned: the default is one pass over all levels (the reference
  times every power-of-two divider with ``do_bench`` on first use, :600-607).
* Index arithmetic follows the reference's CPU path bit for bit (one float32 multiply
  per level); the Triton kernel multiplies the coordinate incrementally level to level
  (:253-256) and so differs from its own CPU path in the last bit of some coordinates.
"""
import math
import weakref
from typing import Final, Optional, Sequence, Tuple

import torch
from torch import Tensor

from ... import _lib
from .helpers import (  # noqa: F401  (re-exported like the reference module does)
    compute_b,
    compute_embedding_counts,
    compute_level_embedding_offset,
    compute_resolutions,
    get_first_hash_level,
    level_geometry,
    seek_to_level_embeddings,
)

# One prime per spatial dimension, as in the Instant-NGP paper (reference :24-27)
PI_1: Final = 1
PI_2: Final = 2_654_435_761
PI_3: Final = 805_459_861

SUPPORTED_FEATURES: Final = (1, 2, 4, 8)


def _flatten_rows(t: Tensor, width: int) -> Tensor:
    r"""``(..., width)`` -> ``(N, width)`` without copying when the layout allows it."""
    return t.reshape(-1, width)


def _check_divider(divider: int, levels: int) -> None:
    assert 1 <= divider <= levels, f"Divider must be between 1 and {levels}"
    assert divider & (divider - 1) == 0, "Divider must be a power of 2"


_DEFAULT_PI: dict = {}


def _default_pi(device: torch.device) -> Tensor:
    r"""The built-in primes as an int64 tensor on ``device``, created once per device."""
    pi = _DEFAULT_PI.get(device)
    if pi is None:
        pi = torch.tensor([PI_1, PI_2, PI_3], dtype=torch.int64, device=device)
        _DEFAULT_PI[device] = pi
    return pi


_PRIMES_SEEN: dict = {}


def host_primes(pi, D: int) -> Tuple[int, ...]:
    r"""The first ``D`` hash primes as Python ints.  ``pi`` is a tensor (the module's buffer, usually
    on the GPU) or an already extracted tuple.  Reading a device tensor synchronises the stream, which
    would stall every forward and backward call behind the GPU, so the values are read once per tensor
    object and version and remembered."""
    if not isinstance(pi, Tensor):
        return tuple(int(v) for v in pi[:D])
    key = id(pi)
    hit = _PRIMES_SEEN.get(key)
    if hit is not None and hit[0]() is pi and hit[1] == pi._version and len(hit[2]) >= D:
        return hit[2][:D]
    values = tuple(int(v) for v in pi.tolist())
    if len(_PRIMES_SEEN) > 256:
        _PRIMES_SEEN.clear()
    _PRIMES_SEEN[key] = (weakref.ref(pi, lambda _ref, key=key: _PRIMES_SEEN.pop(key, None)), pi._version, values)
    return values[:D]


class _Launch:
    r"""Host-side arguments shared by the forward, backward and debug entry points."""

    def __init__(self, coords: Tensor, pi, D: int, T: int, levels: int, min_res: int, max_res: int, scale: float):
        geo = level_geometry(levels, T, D, min_res, max_res)
        self.geo = geo
        self._fill(coords, pi, D, geo.resolutions, geo.rows, geo.offsets, scale)

    @classmethod
    def from_levels(cls, coords: Tensor, pi, D: int, resolutions, rows, scale: float) -> "_Launch":
        self = cls.__new__(cls)
        self.geo = None
        offsets = [sum(rows[:i]) for i in range(len(rows))]
        self._fill(coords, pi, D, resolutions, rows, offsets, scale)
        return self

    def _fill(self, coords: Tensor, pi, D: int, resolutions, rows, offsets, scale: float) -> None:
        self.coords2d = _flatten_rows(coords, D)
        self.n = self.coords2d.shape[0]
        self.res = _lib.i32_array(list(resolutions))
        self.rows = _lib.i64_array(list(rows))
        self.offsets = _lib.i64_array(list(offsets))
        self.prime_values = host_primes(pi, D)
        self.primes = _lib.i64_array(list(self.prime_values))
        self.scale = float(scale)
        self.coord_args = (
            self.coords2d.data_ptr(),
            self.coords2d.stride(0) if self.n > 1 else D,
            self.coords2d.stride(1),
            _lib.dtype_code(self.coords2d),
        )


def _launch_backward(launch: "_Launch", do: Tensor, de: Tensor, D_in: int, D_embed: int, levels: int, begin: int, end: int):
    r"""``th_hash_bwd`` for levels ``[begin, end)``: adds into the (zero-initialised) table gradient ``de``."""
    D_out = do.shape[-1]
    go = _flatten_rows(do, D_out)
    if go.dtype != de.dtype:
        go = go.to(de.dtype)
    if go.stride(-1) != 1 or (go.shape[0] > 1 and go.stride(0) < D_out):
        go = go.contiguous()  # e.g. the stride-0 gradient of ``o.sum()``
    go_stride = go.stride(0) if go.shape[0] > 1 else D_out
    device = de.device
    with torch.cuda.device(device):
        _lib.check(
            _lib.lib().th_hash_bwd(
                *launch.coord_args, go.data_ptr(), go_stride, de.data_ptr(), _lib.dtype_code(de),
                launch.n, D_in, D_embed, levels, launch.res, launch.rows, launch.offsets, launch.primes,
                launch.scale, begin, end, _lib.stream_ptr(device),
            ),
            "th_hash_bwd",
        )  # fmt: skip


@torch.no_grad()
def hash_encoding_backward_levels(
    coord: Tensor,
    grad_out: Tensor,
    grad_embeddings: Tensor,
    pi: Optional[Tensor],
    max_entries_per_level: int,
    min_res: int,
    max_res: int,
    levels: int,
    level_begin: int,
    level_end: int,
    scale: float = 1.0,
) -> None:
    r"""Adds the table gradient of levels ``[level_begin, level_end)`` into ``grad_embeddings``.

    The piece of ``HashEncoding.backward`` that a caller needs when it wants the gradient level range
    by level range, e.g. to start summing the finished rows over ranks while the other levels are
    still being computed (``training.NeuralFieldTrainer``).  ``grad_out`` is the gradient of the
    encoding's output (its first ``levels * F`` columns are read), ``grad_embeddings`` a tensor shaped
    and typed like the table that starts at zero.  triton_helpers has no such entry: its backward
    always returns the whole table gradient (hash_encoding/kernel.py:636-671).
    """
    D_in, D_embed = coord.shape[-1], grad_embeddings.shape[-1]
    if pi is None:
        pi = _default_pi(coord.device)
    _lib.require_cuda(coord, grad_out, grad_embeddings, pi)
    assert 0 <= level_begin < level_end <= levels, "level range out of bounds"
    assert grad_embeddings.is_contiguous(), "the table gradient must be contiguous"
    launch = _Launch(coord, pi, D_in, max_entries_per_level, levels, min_res, max_res, scale)
    assert grad_embeddings.shape[0] >= launch.geo.total_rows
    _launch_backward(launch, grad_out, grad_embeddings, D_in, D_embed, levels, level_begin, level_end)


class HashEncoding(torch.autograd.Function):

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.float16)
    def forward(
        ctx,
        coords: Tensor,
        embeddings: Tensor,
        pi: Optional[Tensor],
        features: Optional[Tensor],
        max_entries_per_level: int,
        min_res: int,
        max_res: int,
        levels: int,
        divider: Optional[int] = None,
        bwd_divider: Optional[int] = None,
        scale: float = 1.0,
    ) -> Tensor:
        D_in = coords.shape[-1]
        D_feature = features.shape[-1] if features is not None else 0
        D_embed = embeddings.shape[-1]

        assert coords.is_floating_point(), "Coords must be float"
        if pi is None:
            if D_in > 3:
                raise ValueError("Pi must be provided for more than 3 dimensions")
            pi = _default_pi(coords.device)
        assert isinstance(pi, Tensor)
        assert pi.ndim == 1, "Pi must be a 1-dimensional tensor"
        assert pi.numel() >= D_in, "Pi must have at least D_in elements"
        if features is not None:
            assert isinstance(features, Tensor)
            assert (
                features.shape[:-1] == coords.shape[:-1]
            ), "Features must have the same shape as coords, except for the last dimension"

        # only the table receives a gradient
        assert not coords.requires_grad, "Gradients not supported for coords"
        assert features is None or not features.requires_grad, "Gradients not supported for features"
        assert not pi.requires_grad, "Gradients not supported for pi"
        device = _lib.require_cuda(coords, embeddings, pi, features)

        assert levels & (levels - 1) == 0, "Levels must be a power of 2"
        if D_in > 3:
            raise ValueError(f"coordinate dimension {D_in} is not supported by the CUDA kernels (1..3)")
        if D_embed not in SUPPORTED_FEATURES:
            raise ValueError(f"embedding width {D_embed} is not supported by the CUDA kernels {SUPPORTED_FEATURES}")
        if divider is not None:
            _check_divider(divider, levels)

        launch = _Launch(coords, pi, D_in, max_entries_per_level, levels, min_res, max_res, scale)
        assert embeddings.ndim == 2 and embeddings.shape[0] >= launch.geo.total_rows, (
            f"Embedding table has {tuple(embeddings.shape)} rows, the level layout needs {launch.geo.total_rows}"
        )
        table = embeddings if embeddings.is_contiguous() else embeddings.contiguous()

        D_out = D_embed * levels + D_feature
        o = embeddings.new_empty(*coords.shape[:-1], D_out)
        step = divider if divider is not None else levels
        with torch.cuda.device(device):
            stream = _lib.stream_ptr(device)
            for begin in range(0, levels, step):
                _lib.check(
                    _lib.lib().th_hash_fwd(
                        *launch.coord_args, table.data_ptr(), _lib.dtype_code(table), o.data_ptr(), D_out,
                        launch.n, D_in, D_embed, levels, launch.res, launch.rows, launch.offsets, launch.primes,
                        launch.scale, begin, begin + step, stream,
                    ),
                    "th_hash_fwd",
                )  # fmt: skip
        if features is not None:
            o[..., D_embed * levels :] = features

        ctx.save_for_backward(coords, embeddings, pi)
        ctx.prime_values = launch.prime_values  # the backward pass needs no second look at `pi`
        ctx.max_entries_per_level = max_entries_per_level
        ctx.min_res = min_res
        ctx.max_res = max_res
        ctx.levels = levels
        ctx.scale = scale
        ctx.bwd_divider = bwd_divider
        return o

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    @torch.no_grad()
    def backward(ctx, do: Tensor):
        coords, embeddings, pi = ctx.saved_tensors
        D_in = coords.shape[-1]
        D_embed = embeddings.shape[-1]
        levels = ctx.levels
        if ctx.bwd_divider is not None:
            _check_divider(ctx.bwd_divider, levels)

        launch = _Launch(coords, ctx.prime_values, D_in, ctx.max_entries_per_level, levels, ctx.min_res, ctx.max_res, ctx.scale)
        de = torch.zeros(embeddings.shape, dtype=embeddings.dtype, device=embeddings.device)
        step = ctx.bwd_divider if ctx.bwd_divider is not None else levels
        for begin in range(0, levels, step):
            _launch_backward(launch, do, de, D_in, D_embed, levels, begin, begin + step)
        return None, de, None, None, None, None, None, None, None, None, None

    @staticmethod
    def _possible_dividers(levels: int) -> Tuple[int, ...]:
        return tuple(2**i for i in range(int(math.log2(levels)) + 1))


def hash_encoding(
    coord: Tensor,
    embeddings: Tensor,
    features: Optional[Tensor] = None,
    pi: Optional[Tensor] = None,
    max_entries_per_level: int = 2**14,
    min_res: int = 16,
    max_res: int = 512,
    levels: int = 16,
    divider: Optional[int] = None,
    bwd_divider: Optional[int] = None,
    scale: float = 1.0,
) -> Tensor:
    r"""Multi-resolution hash encoding as defined in Instant NGP.

    Args:
        coord: Coordinates on the range :math:`[0, scale]`.
        embeddings: Embedding table, all levels concatenated.
        features: Optional features to concatenate to the output.
        pi: Hashing primes. Built in for up to ``D=3`` if not provided.
        max_entries_per_level: Maximum number of rows per level.
        min_res: Resolution of the coarsest level.
        max_res: Resolution of the finest level.
        levels: Number of levels (a power of two).
        divider: Levels per forward kernel pass; all levels in one pass when ``None``.
        bwd_divider: Levels per backward kernel pass; all levels in one pass when ``None``.
        scale: Upper end of the coordinate range.

    Shapes:
        ``coord`` - :math:`(..., D)`, ``embeddings`` - :math:`(E, D_e)`, ``features`` - :math:`(..., D_f)`,
        ``pi`` - :math:`(D,)`, output - :math:`(..., L \times D_e + D_f)`.
    """
    return HashEncoding.apply(
        coord, embeddings, pi, features, max_entries_per_level, min_res, max_res, levels, divider, bwd_divider, scale
    )


@torch.no_grad()
def hash_corner_indices(
    coord: Tensor,
    resolutions: Sequence[int],
    rows: Sequence[int],
    pi: Optional[Tensor] = None,
    scale: float = 1.0,
) -> Tuple[Tensor, Tensor]:
    r"""Row index (relative to its level) and interpolation weight of every corner, from the CUDA path.

    ``resolutions[l]`` / ``rows[l]`` describe level ``l`` (a level is dense when
    ``(res + 1)**D <= rows``).  Returns ``(indices int64 (N, levels, 2**D), weights float32
    (N, levels, 2**D))``.  This is the hook of the bit-exact index tests; it runs the same
    device functions as the forward and backward kernels.
    """
    D = coord.shape[-1]
    levels = len(resolutions)
    if pi is None:
        pi = torch.tensor([PI_1, PI_2, PI_3], dtype=torch.int64, device=coord.device)
    device = _lib.require_cuda(coord, pi)
    launch = _Launch.from_levels(coord, pi, D, resolutions, rows, scale)
    idx = torch.empty(launch.n, levels, 2**D, dtype=torch.int64, device=device)
    w = torch.empty(launch.n, levels, 2**D, dtype=torch.float32, device=device)
    with torch.cuda.device(device):
        _lib.check(
            _lib.lib().th_hash_debug_indices(
                *launch.coord_args, idx.data_ptr(), w.data_ptr(), launch.n, D, levels, launch.res, launch.rows,
                launch.primes, launch.scale, _lib.stream_ptr(device),
            ),
            "th_hash_debug_indices",
        )  # fmt: skip
    return idx, w
