r"""Level geometry of the multiresolution hash table.

Host-side arithmetic that fixes the table layout: growth factor, per-level grid
resolutions, rows per level, the first level that needs the spatial hash, and the
row offset of each level inside the single concatenated table.  Function names,
argument order and results match ``triton_helpers/layers/hash_encoding/helpers.py:12-115``
so code written against the reference keeps working; the results are what the CUDA
kernels receive as their per-level parameter block.

The resolutions deliberately go through a float32 ``torch.pow`` followed by ``floor``:
that is what the reference does (helpers.py:37-39) and a float64 evaluation gives a
different integer for some levels.
"""
import math
import sys
from functools import lru_cache
from typing import Final, List, NamedTuple, Tuple

import torch
from torch import Tensor


EPS: Final = 1e-5


def compute_b(N_min: int, N_max: int, L: int) -> float:
    r"""Per-level growth factor ``exp((ln N_max - ln N_min) / (L - 1)) + EPS`` (helpers.py:12-23)."""
    return float(math.exp((math.log(N_max) - math.log(N_min)) / (L - 1))) + EPS


def compute_resolutions(num_levels: int, N_min: int, N_max: int) -> List[int]:
    r"""Grid resolution of every level: ``floor(N_min * b**l)`` evaluated in float32 (helpers.py:26-39)."""
    growth = torch.tensor(compute_b(N_min, N_max, num_levels))
    exponent = torch.arange(0, num_levels)
    scaled = torch.pow(growth, exponent) * N_min
    return [int(v) for v in torch.floor(scaled).to(torch.int64)]


def compute_embedding_counts(L: int, T: int, D: int, N_min: int, N_max: int) -> List[int]:
    r"""Rows stored for every level: ``min((res + 1)**D, T)`` (helpers.py:42-57)."""
    return [min((res + 1) ** D, T) for res in compute_resolutions(L, N_min, N_max)]


def get_first_hash_level(N_min: int, N_max: int, L: int, T: int, D: int) -> int:
    r"""Index of the first level whose dense grid exceeds ``T`` rows, ``L + 1`` if none does (helpers.py:60-73)."""
    for level, rows in enumerate(compute_embedding_counts(L, sys.maxsize, D, N_min, N_max)):
        if rows > T:
            return level
    return L + 1


def _level_starts(L: int, T: int, D: int, N_min: int, N_max: int) -> List[int]:
    starts = [0]
    for rows in compute_embedding_counts(L, T, D, N_min, N_max):
        starts.append(starts[-1] + rows)
    return starts


def seek_to_level_embeddings(e: Tensor, l_i: int, L: int, T: int, D: int, N_min: int, N_max: int) -> Tensor:
    r"""View of the rows of level ``l_i`` inside the concatenated table ``(*, E, F)`` (helpers.py:76-98)."""
    starts = _level_starts(L, T, D, N_min, N_max)
    return e[..., starts[l_i] : starts[l_i + 1], :]


def compute_level_embedding_offset(l_i: int, L: int, T: int, D: int, N_min: int, N_max: int) -> int:
    r"""First row of level ``l_i`` inside the concatenated table (helpers.py:101-115)."""
    return _level_starts(L, T, D, N_min, N_max)[l_i]


class LevelGeometry(NamedTuple):
    r"""Everything the kernels need to know about the table, one entry per level."""

    resolutions: Tuple[int, ...]
    rows: Tuple[int, ...]
    offsets: Tuple[int, ...]
    first_hash_level: int
    total_rows: int


@lru_cache(maxsize=256)
def level_geometry(L: int, T: int, D: int, N_min: int, N_max: int) -> LevelGeometry:
    r"""Cached per-configuration geometry passed to the C ABI as three ``L``-long integer arrays."""
    res = compute_resolutions(L, N_min, N_max)
    rows = compute_embedding_counts(L, T, D, N_min, N_max)
    starts = _level_starts(L, T, D, N_min, N_max)
    return LevelGeometry(
        tuple(res),
        tuple(rows),
        tuple(starts[:-1]),
        get_first_hash_level(N_min, N_max, L, T, D),
        starts[-1],
    )
