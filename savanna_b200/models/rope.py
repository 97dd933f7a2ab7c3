"""Rotary position embeddings (rotate-half convention).

`RotaryEmbedding` covers the reference's `rotary`, `rotary_linear_scaled` (position interpolation:
positions divided by the scaling factor, optionally with a larger base) and `rotary_ntk_scaled`
(base stretched by factor^(d/(d-2))) variants (savanna/model/operators/positional_embeddings.py:28-234).
Positions are always passed explicitly, so zigzag context-parallel shards get the right angles for
every variant (the reference's plain variant overwrites them with arange, :74).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..ops import reference as ref


class RotaryEmbedding(nn.Module):
    def __init__(self, dim: int, base: float = 10000.0, scaling_factor: float = 1.0, kind: str = "rotary",
                 max_unscaled_len: int = 8192, device=None):
        super().__init__()
        self.dim, self.kind = dim, kind
        if kind == "rotary_ntk_scaled" and scaling_factor > 1.0:
            base = base * scaling_factor ** (dim / (dim - 2))
            scaling_factor = 1.0
        if kind == "rotary":
            scaling_factor = 1.0
        self.base, self.scaling_factor = float(base), float(scaling_factor)
        inv = 1.0 / (self.base ** (torch.arange(0, dim, 2, dtype=torch.float32, device=device) / dim))
        self.register_buffer("inv_freq", inv, persistent=True)
        self._cache = None

    def forward(self, positions: torch.Tensor):
        """positions [L] (global token positions) -> (cos, sin) each [L, dim] fp32."""
        key = (positions.data_ptr(), positions.shape[0], positions.device)
        if self._cache is not None and self._cache[0] == key:
            return self._cache[1], self._cache[2]
        cos, sin = ref.rope_tables(positions, self.dim, self.base, self.scaling_factor)
        self._cache = (key, cos, sin)
        return cos, sin


class AliBi(nn.Module):
    """Attention-with-linear-biases slopes (positional_embeddings.py:262-339); used by the oracle
    attention path only."""

    def __init__(self, num_heads: int, mp_size: int = 1, mp_rank: int = 0):
        super().__init__()
        import math

        def slopes(n):
            if math.log2(n).is_integer():
                start = 2 ** (-(2 ** -(math.log2(n) - 3)))
                return [start * start ** i for i in range(n)]
            c = 2 ** math.floor(math.log2(n))
            return slopes(c) + slopes(2 * c)[0::2][: n - c]
        per = num_heads // mp_size
        self.register_buffer("slopes", torch.tensor(slopes(num_heads))[mp_rank * per:(mp_rank + 1) * per])

    def bias(self, q_pos, k_pos):
        rel = (k_pos[None, :] - q_pos[:, None]).float()
        return self.slopes.view(-1, 1, 1) * rel[None]
