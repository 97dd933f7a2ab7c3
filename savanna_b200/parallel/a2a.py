"""Context-parallel all-to-all between the sequence-sharded and the channel-sharded layout.

    split_to_full : [B, L/cp (zigzag shard), D]  ->  [B, L (natural order), D/cp]
    full_to_split : the inverse

This is the channel-last restatement of the reference's AllToAllSingleFunction
(savanna/model/operators/hyena/distributed_a2a.py:45-168).  The collective itself is NCCL/gloo
here; the fused CUDA long-convolution path pulls the peer slices itself.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import state
from .zigzag import inverse_zigzag_permutation, zigzag_indices


def _all_to_all(out: torch.Tensor, inp: torch.Tensor, group) -> None:
    try:
        dist.all_to_all_single(out, inp, group=group)
        return
    except (RuntimeError, NotImplementedError):
        pass
    # backends without all-to-all: pairwise exchange
    ranks = state.get_context_parallel_ranks()
    me = state.get_context_parallel_rank()
    reqs = []
    for i, r in enumerate(ranks):
        if i == me:
            out[i].copy_(inp[i])
        else:
            reqs.append(dist.P2POp(dist.isend, inp[i].contiguous(), r, group))
            reqs.append(dist.P2POp(dist.irecv, out[i], r, group))
    if reqs:
        for q in dist.batch_isend_irecv(reqs):
            q.wait()


def _split_to_full(x: torch.Tensor, zigzag: bool) -> torch.Tensor:
    group, cp = state.get_context_parallel_group(), state.get_context_parallel_world_size()
    B, l, D = x.shape
    d = D // cp
    send = x.view(B, l, cp, d).permute(2, 0, 1, 3).contiguous()          # [cp(dst), B, l, d]
    recv = torch.empty_like(send)                                          # [cp(src), B, l, d]
    _all_to_all(recv, send, group)
    full = recv.permute(1, 0, 2, 3).reshape(B, cp * l, d)
    if zigzag:
        full = full.index_select(1, inverse_zigzag_permutation(cp * l, cp, x.device))
    return full.contiguous()


def _full_to_split(x: torch.Tensor, zigzag: bool) -> torch.Tensor:
    group, cp = state.get_context_parallel_group(), state.get_context_parallel_world_size()
    B, L, d = x.shape
    l = L // cp
    if zigzag:
        order = torch.cat([zigzag_indices(L, cp, r, x.device) for r in range(cp)])
        x = x.index_select(1, order)
    send = x.view(B, cp, l, d).permute(1, 0, 2, 3).contiguous()          # [cp(dst), B, l, d]
    recv = torch.empty_like(send)                                          # [cp(src = channel block), B, l, d]
    _all_to_all(recv, send, group)
    return recv.permute(1, 2, 0, 3).reshape(B, l, cp * d).contiguous()


class AllToAllSingle(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, direction, zigzag):
        ctx.direction, ctx.zigzag = direction, zigzag
        return _split_to_full(x, zigzag) if direction == "split_to_full" else _full_to_split(x, zigzag)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        out = _full_to_split(g, ctx.zigzag) if ctx.direction == "split_to_full" else _split_to_full(g, ctx.zigzag)
        return out, None, None


def split_to_full(x, zigzag: bool = True):
    if state.get_context_parallel_world_size() == 1:
        return x
    return AllToAllSingle.apply(x, "split_to_full", zigzag)


def full_to_split(x, zigzag: bool = True):
    if state.get_context_parallel_world_size() == 1:
        return x
    return AllToAllSingle.apply(x, "full_to_split", zigzag)
