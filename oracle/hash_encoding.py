r"""CPU oracle of the multiresolution hash encoding.  TEST INFRASTRUCTURE ONLY.

A restatement of the reference's CPU path, function by function:

================================  =====================================================
here                              follows (``triton_helpers/layers/hash_encoding/``)
================================  =====================================================
``growth_factor``                 ``helpers.py:12-23``  ``compute_b``
``level_resolutions``             ``helpers.py:26-39``  ``compute_resolutions``
``level_rows``                    ``helpers.py:42-57``  ``compute_embedding_counts``
``first_hash_level``              ``helpers.py:60-73``  ``get_first_hash_level``
``level_offsets``                 ``helpers.py:101-115`` ``compute_level_embedding_offset``
``corner_offsets``                ``kernel.py:443-445`` ``_cpu_create_corner_offsets``
``corner_indices``                ``kernel.py:448-462`` ``_cpu_embedding_lookup``
``corner_weights``                ``kernel.py:465-477`` weights of ``_cpu_interpolate``
``interpolate``                   ``kernel.py:465-479`` ``_cpu_interpolate``
``encode``                        ``kernel.py:482-502`` ``_cpu_hash_encoding``
``encode_backward``               torch autograd through ``_cpu_hash_encoding`` as used
                                  by ``tests/test_layers/test_hash_encoding.py:468-476``
================================  =====================================================

Parity is pinned by ``tests/test_oracle_hash.py`` against the golden index tables of the
reference's tests and against fixtures produced by running the reference's own
``_cpu_*`` functions (``tests/golden/make_golden.py``).

Arithmetic contract (this is what the CUDA kernels must reproduce):

* ``cell = floor(x * res)`` with ONE float32 multiply per level, then integer;
* dense level (``(res + 1)**D <= T``): ``index = sum_d corner_d * res**d`` (stride ``res``,
  not ``res + 1``: distinct corners can alias, the reference does the same);
* hashed level: ``index = xor_d(corner_d * pi_d) mod rows`` in int64, ``pi = (1, 2654435761, 805459861)``;
* ``t = x * res - cell`` in float32; corner weight ``prod_d (bit_d ? t_d : 1 - t_d)``
  multiplied in axis order 0, 1, 2; corner ``c`` has bit ``d`` as its offset on axis ``d``;
* output feature = float32 sum over the corners of ``weight * table[index]`` rounded once
  to the table dtype.
"""
import math
import sys
from typing import List, Sequence

import torch
from torch import Tensor


PRIMES = (1, 2_654_435_761, 805_459_861)
GROWTH_EPS = 1e-5


def growth_factor(n_min: int, n_max: int, levels: int) -> float:
    return float(math.exp((math.log(n_max) - math.log(n_min)) / (levels - 1))) + GROWTH_EPS


def level_resolutions(levels: int, n_min: int, n_max: int) -> List[int]:
    # float32 pow, float32 multiply, floor: the reference evaluates this with a float32 tensor
    base = torch.tensor(growth_factor(n_min, n_max, levels), dtype=torch.float32)
    steps = torch.arange(levels, dtype=torch.int64)
    return torch.floor(base.pow(steps) * n_min).to(torch.int64).tolist()


def level_rows(levels: int, table_cap: int, dims: int, n_min: int, n_max: int) -> List[int]:
    return [min((r + 1) ** dims, table_cap) for r in level_resolutions(levels, n_min, n_max)]


def first_hash_level(n_min: int, n_max: int, levels: int, table_cap: int, dims: int) -> int:
    uncapped = level_rows(levels, sys.maxsize, dims, n_min, n_max)
    hashed = [rows > table_cap for rows in uncapped]
    return hashed.index(True) if any(hashed) else levels + 1


def level_offsets(levels: int, table_cap: int, dims: int, n_min: int, n_max: int) -> List[int]:
    out, running = [], 0
    for rows in level_rows(levels, table_cap, dims, n_min, n_max):
        out.append(running)
        running += rows
    return out


def corner_offsets(dims: int) -> Tensor:
    r"""``(2**dims, dims)`` int64; bit ``d`` of the corner number is the step along axis ``d``."""
    corner = torch.arange(2**dims, dtype=torch.int64).unsqueeze(1)
    axis = torch.arange(dims, dtype=torch.int64).unsqueeze(0)
    return (corner >> axis) & 1


@torch.no_grad()
def corner_indices(x: Tensor, pi: Sequence[int] | Tensor, dims: int, rows: int, res: int) -> Tensor:
    r"""Row index of every corner of the cell containing ``x`` at one level: ``(N, 2**dims)`` int64.

    ``x`` is float32 in ``[0, 1]``, shape ``(N, dims)``.  ``rows`` is the level's row count
    (already capped), ``res`` its resolution.
    """
    x = x.to(torch.float32)
    cell = torch.floor(x * res).to(torch.int64)
    corners = cell.unsqueeze(1) + corner_offsets(dims).unsqueeze(0)
    if (res + 1) ** dims <= rows:
        stride = torch.tensor([res**d for d in range(dims)], dtype=torch.int64)
        return (corners * stride).sum(-1)
    primes = torch.as_tensor(pi, dtype=torch.int64)[:dims]
    prod = corners * primes
    h = prod[..., 0]
    for d in range(1, dims):
        h = torch.bitwise_xor(h, prod[..., d])
    return h % rows


def corner_weights(x: Tensor, dims: int, res: int) -> Tensor:
    r"""Linear-interpolation weight of every corner: ``(N, 2**dims)`` float32."""
    x = x.to(torch.float32)
    scaled = x * res
    cell = torch.floor(scaled).to(torch.int64)
    t = (scaled - cell).unsqueeze(1)
    per_axis = torch.where(corner_offsets(dims).unsqueeze(0) == 0, 1 - t, t)
    return per_axis.prod(-1)


def interpolate(x: Tensor, e: Tensor, dims: int, res: int) -> Tensor:
    r"""``(N, F)`` = sum over corners of weight * ``e`` where ``e`` is ``(N, 2**dims, F)``."""
    return (corner_weights(x, dims, res).unsqueeze(-1) * e).sum(1)


def encode(
    x: Tensor,
    table: Tensor,
    pi: Sequence[int] | Tensor = PRIMES,
    *,
    table_cap: int,
    levels: int,
    n_min: int,
    n_max: int,
) -> Tensor:
    r"""Forward pass: ``(N, levels * F)`` in the table's dtype.  ``x`` in ``[0, 1]``, ``(N, D)`` with ``D <= 3``."""
    n, dims = x.shape
    assert 1 <= dims <= 3
    feats = table.shape[-1]
    res = level_resolutions(levels, n_min, n_max)
    rows = level_rows(levels, table_cap, dims, n_min, n_max)
    offs = level_offsets(levels, table_cap, dims, n_min, n_max)
    out = table.new_zeros(n, levels * feats)
    for lvl in range(levels):
        idx = corner_indices(x, pi, dims, rows[lvl], res[lvl])
        gathered = table[offs[lvl] : offs[lvl] + rows[lvl]][idx]
        out[:, lvl * feats : (lvl + 1) * feats] = interpolate(x, gathered, dims, res[lvl])
    return out


@torch.no_grad()
def encode_backward(
    x: Tensor,
    grad_out: Tensor,
    table_like: Tensor,
    pi: Sequence[int] | Tensor = PRIMES,
    *,
    table_cap: int,
    levels: int,
    n_min: int,
    n_max: int,
    accumulate_dtype: torch.dtype = torch.float32,
) -> Tensor:
    r"""Gradient of ``sum(encode(x, table) * grad_out)`` with respect to the table.

    Explicit scatter-add, equal to what autograd produces for ``encode``: every corner
    receives ``weight * grad_out`` for its level's feature columns.  The sum is formed in
    ``accumulate_dtype`` and rounded once to the table dtype at the end.
    """
    n, dims = x.shape
    feats = table_like.shape[-1]
    res = level_resolutions(levels, n_min, n_max)
    rows = level_rows(levels, table_cap, dims, n_min, n_max)
    offs = level_offsets(levels, table_cap, dims, n_min, n_max)
    grad = torch.zeros(table_like.shape, dtype=accumulate_dtype)
    go = grad_out.to(accumulate_dtype)
    for lvl in range(levels):
        idx = corner_indices(x, pi, dims, rows[lvl], res[lvl]) + offs[lvl]
        w = corner_weights(x, dims, res[lvl]).to(accumulate_dtype)
        contrib = w.unsqueeze(-1) * go[:, None, lvl * feats : (lvl + 1) * feats]
        grad.index_add_(0, idx.reshape(-1), contrib.reshape(-1, feats))
    return grad.to(table_like.dtype)
