r"""``nn.Module`` owning a hash table; drop-in for ``triton_helpers/layers/hash_encoding/module.py:8-39``.

Parameter and buffer names, shapes and initialisation order match the reference, so a
``state_dict`` saved from the reference module loads here and vice versa.
"""
from typing import Optional

import torch
import torch.nn as nn
from torch import Tensor

from .helpers import compute_embedding_counts
from .kernel import PI_1, PI_2, PI_3, hash_encoding


class HashEncoding(nn.Module):

    def __init__(
        self,
        max_entries_per_level: int = 2**14,
        num_levels: int = 16,
        d_in: int = 3,
        d_embed: int = 2,
        min_res: int = 16,
        max_res: int = 512,
    ):
        super().__init__()
        rows = compute_embedding_counts(num_levels, max_entries_per_level, d_in, min_res, max_res)
        # one randn block per level, concatenated: the reference consumes the RNG in this order
        self.embeddings = nn.Parameter(torch.cat([torch.randn(int(r), d_embed) for r in rows], dim=0))
        self.register_buffer("pi", torch.tensor([PI_1, PI_2, PI_3], dtype=torch.int64))
        self.max_entries_per_level = max_entries_per_level
        self.num_levels = num_levels
        self.min_res = min_res
        self.max_res = max_res

    def forward(self, coords: Tensor, features: Optional[Tensor] = None, scale: float = 1.0) -> Tensor:
        return hash_encoding(
            coords,
            self.embeddings,
            features,
            self.pi,
            self.max_entries_per_level,
            self.min_res,
            self.max_res,
            self.num_levels,
            scale=scale,
        )
