"""Context-parallel halo exchange for causal FIR operators under zigzag sharding.

Rank r holds chunks (c_r, c_{2cp-1-r}).  A causal filter of length k needs the k-1 samples that
precede each chunk:
    first chunk  c_r          <- tail of c_{r-1}, which is the first chunk of rank r-1 (zeros on rank 0)
    second chunk c_{2cp-1-r}  <- tail of c_{2cp-2-r}, the second chunk of rank r+1; on the last rank
                                 it is the rank's own first chunk.
Backward sends the halo gradients the opposite way.  (Reference algorithm:
savanna/model/operators/hyena/p2p_cp_conv.py:6-164.)  This module is the NCCL/gloo form; the CUDA
convolution kernels can instead read the neighbour's tail straight from peer memory.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import state


def _exchange(send_fwd, send_bwd, group, ranks, me):
    """send_fwd goes to rank+1 (if any), send_bwd to rank-1 (if any).  Returns (from rank-1, from rank+1)."""
    cp = len(ranks)
    ops, recv_prev, recv_next = [], None, None
    if me + 1 < cp:
        ops.append(dist.P2POp(dist.isend, send_fwd.contiguous(), ranks[me + 1], group))
        recv_next = torch.empty_like(send_bwd)
        ops.append(dist.P2POp(dist.irecv, recv_next, ranks[me + 1], group))
    if me > 0:
        ops.append(dist.P2POp(dist.isend, send_bwd.contiguous(), ranks[me - 1], group))
        recv_prev = torch.empty_like(send_fwd)
        ops.append(dist.P2POp(dist.irecv, recv_prev, ranks[me - 1], group))
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()
    return recv_prev, recv_next


class _ZigzagHalo(torch.autograd.Function):
    """x [B, L_local, C] (two zigzag chunks back to back) -> halo [B, 2, H, C]."""

    @staticmethod
    def forward(ctx, x, H):
        group, ranks, me = state.get_context_parallel_group(), state.get_context_parallel_ranks(), state.get_context_parallel_rank()
        B, L, C = x.shape
        half = L // 2
        if H > half:
            raise ValueError(f"halo {H} exceeds the chunk length {half}")
        tail_a = x[:, half - H:half]
        tail_b = x[:, L - H:]
        prev, nxt = _exchange(tail_a, tail_b, group, ranks, me)
        halo_a = prev if prev is not None else torch.zeros_like(tail_a)
        halo_b = nxt if nxt is not None else tail_a
        ctx.meta = (H, half, L, me, len(ranks))
        return torch.stack([halo_a, halo_b], dim=1)

    @staticmethod
    def backward(ctx, g):
        H, half, L, me, cp = ctx.meta
        group, ranks = state.get_context_parallel_group(), state.get_context_parallel_ranks()
        g_a, g_b = g[:, 0].contiguous(), g[:, 1].contiguous()
        # g_a belongs to the first-chunk tail of rank-1; g_b to the second-chunk tail of rank+1
        # (or to the own first-chunk tail on the last rank)
        from_prev, from_next = _exchange(g_b, g_a, group, ranks, me)
        # what arrives from rank+1 is its g_a (for my first-chunk tail); from rank-1 its g_b (my second-chunk tail)
        gx = torch.zeros((g.shape[0], L, g.shape[-1]), dtype=g.dtype, device=g.device)
        if from_next is not None:
            gx[:, half - H:half] += from_next
        if me == cp - 1:
            gx[:, half - H:half] += g_b
        if from_prev is not None:
            gx[:, L - H:] += from_prev
        return gx, None


def zigzag_halo(x: torch.Tensor, H: int) -> torch.Tensor:
    """Halo rows for both chunks of a zigzag shard: [B, 2, H, C]."""
    return _ZigzagHalo.apply(x, H)
