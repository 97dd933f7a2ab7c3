"""Zigzag context-parallel sharding of the sequence.

The global sequence is cut into 2*cp equal chunks c_0..c_{2cp-1}; rank r holds [c_r ; c_{2cp-1-r}],
which balances causal work (reference: savanna/mpu/data.py:123-206).
"""
from __future__ import annotations

from typing import List

import torch
import torch.distributed as dist

from . import state


def zigzag_chunk_ids(cp: int, rank: int) -> tuple:
    return rank, 2 * cp - 1 - rank


def zigzag_indices(seq_len: int, cp: int, rank: int, device=None) -> torch.Tensor:
    """Global positions held by `rank`, in local order."""
    if seq_len % (2 * cp):
        raise ValueError(f"sequence length {seq_len} is not divisible by 2*cp={2 * cp}")
    c = seq_len // (2 * cp)
    a, b = zigzag_chunk_ids(cp, rank)
    return torch.cat([torch.arange(a * c, (a + 1) * c, device=device), torch.arange(b * c, (b + 1) * c, device=device)])


def inverse_zigzag_permutation(seq_len: int, cp: int, device=None) -> torch.Tensor:
    """Index p such that cat_over_ranks(local)[..., p] is the sequence in natural order."""
    order = torch.cat([zigzag_indices(seq_len, cp, r, device) for r in range(cp)])
    inv = torch.empty_like(order)
    inv[order] = torch.arange(seq_len, device=device)
    return inv


def zigzag_split(x: torch.Tensor, cp: int, rank: int, seq_dim: int = 1) -> torch.Tensor:
    if cp == 1:
        return x
    idx = zigzag_indices(x.shape[seq_dim], cp, rank, x.device)
    return x.index_select(seq_dim, idx)


def zigzag_split_across_cp_ranks(x: torch.Tensor, seq_dim: int = 1) -> torch.Tensor:
    return zigzag_split(x, state.get_context_parallel_world_size(), state.get_context_parallel_rank(), seq_dim)


def zigzag_merge(parts: List[torch.Tensor], seq_dim: int = 1) -> torch.Tensor:
    """Inverse of zigzag_split given every rank's shard (in rank order)."""
    cp = len(parts)
    if cp == 1:
        return parts[0]
    full = torch.cat(parts, dim=seq_dim)
    inv = inverse_zigzag_permutation(full.shape[seq_dim], cp, full.device)
    return full.index_select(seq_dim, inv)


class _ZigzagGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, seq_dim):
        group = state.get_context_parallel_group()
        cp = state.get_context_parallel_world_size()
        ctx.seq_dim, ctx.cp = seq_dim, cp
        parts = [torch.empty_like(x) for _ in range(cp)]
        dist.all_gather(parts, x.contiguous(), group=group)
        return zigzag_merge(parts, seq_dim)

    @staticmethod
    def backward(ctx, g):
        return zigzag_split(g, ctx.cp, state.get_context_parallel_rank(), ctx.seq_dim).contiguous(), None


def zigzag_gather_from_cp_ranks(x: torch.Tensor, seq_dim: int = 1) -> torch.Tensor:
    if state.get_context_parallel_world_size() == 1:
        return x
    return _ZigzagGather.apply(x, seq_dim)
