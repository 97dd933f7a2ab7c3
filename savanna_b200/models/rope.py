"""Rotary position embeddings (rotate-half convention).

`RotaryEmbedding` covers the reference's `rotary`, `rotary_linear_scaled` (position interpolation:
positions divided by the scaling factor, optionally with a larger base) and `rotary_ntk_scaled`
(dynamic NTK: beyond the unscaled length the base grows with the sequence length) variants (savanna/model/operators/positional_embeddings.py:28-234).
Positions are always passed explicitly, so zigzag context-parallel shards get the right angles for
every variant (the reference's plain variant overwrites them with arange, :74).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..ops import reference as ref
from ..parallel import state


class RotaryEmbedding(nn.Module):
    def __init__(self, dim: int, base: float = 10000.0, scaling_factor: float = 1.0, kind: str = "rotary",
                 max_unscaled_len: int = 8192, device=None):
        super().__init__()
        self.dim, self.kind = dim, kind
        # "rotary_ntk_scaled": the base grows with the sequence length once it exceeds `max_unscaled_len` (dynamic NTK
        # scaling, positional_embeddings.py:194-237); "rotary_linear_scaled": positions are divided by the factor
        self.ntk_factor = float(scaling_factor) if kind == "rotary_ntk_scaled" else 1.0
        self.max_unscaled_len = int(max_unscaled_len or 2048)
        if kind in ("rotary", "rotary_ntk_scaled"):
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
        base = self.base
        if self.kind == "rotary_ntk_scaled":
            seq_len = positions.shape[0] * state.get_context_parallel_world_size()
            if seq_len > self.max_unscaled_len:
                base = base * ((self.ntk_factor * seq_len / self.max_unscaled_len) - (self.ntk_factor - 1)) \
                    ** (self.dim / (self.dim - 2))
        cos, sin = ref.rope_tables(positions, self.dim, base, self.scaling_factor)
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


class RelativePositionBias(nn.Module):
    """T5-style bucketed relative-position bias: a table [num_buckets, heads / tp] indexed by the bucket of
    (key position - query position); half of the buckets are exact small distances, the rest grow logarithmically up
    to `max_distance`.  `bias(q_pos, k_pos)` -> [heads / tp, Lq, Lk] * scale, added to the attention scores
    (reference: savanna/mpu/layers.py:194-349 `ParallelRelativePositionBias`, heads split over tensor-parallel ranks)."""

    def __init__(self, scale: float, causal: bool = True, num_buckets: int = 32, max_distance: int = 128, heads: int = 8,
                 mp_size: int = 1, mp_rank: int = 0, init_method=None, dtype=None, device=None):
        super().__init__()
        import math
        self.scale, self.causal, self.num_buckets, self.max_distance = scale, causal, num_buckets, max_distance
        per = heads // mp_size
        full = torch.empty(num_buckets, heads, dtype=torch.float32)
        (init_method or nn.init.xavier_normal_)(full)              # the whole table, then this rank's head columns
        self.weight = nn.Parameter(full[:, mp_rank * per:(mp_rank + 1) * per].to(dtype=dtype, device=device).contiguous())
        self._log_ratio = math.log

    def bucket(self, relative_position: torch.Tensor) -> torch.Tensor:
        import math
        nb = self.num_buckets
        n = -relative_position
        ret = torch.zeros_like(n)
        if not self.causal:
            nb //= 2
            ret = ret + (n < 0).long() * nb
            n = n.abs()
        else:
            n = n.clamp_min(0)
        max_exact = nb // 2
        large = max_exact + (torch.log(n.float().clamp_min(1) / max_exact) / math.log(self.max_distance / max_exact)
                             * (nb - max_exact)).long()
        large = large.clamp_max(nb - 1)
        return ret + torch.where(n < max_exact, n, large)

    def bias(self, q_pos: torch.Tensor, k_pos: torch.Tensor) -> torch.Tensor:
        rel = k_pos[None, :].long() - q_pos[:, None].long()
        values = nn.functional.embedding(self.bucket(rel), self.weight)          # [Lq, Lk, heads]
        return values.permute(2, 0, 1) * self.scale

    def forward(self, q_len: int, k_len: int) -> torch.Tensor:
        dev = self.weight.device
        return self.bias(torch.arange(q_len, device=dev) + (k_len - q_len), torch.arange(k_len, device=dev))
