"""Context parallelism of Hyena-LI by modal-state hand-off.

The implicit modal filter is an order-O diagonal recurrence, so a sequence shard only needs the O
states per channel left by everything before it.  Each rank (1) runs its two zigzag chunks with a
zero initial state and keeps their end states, (2) all-gathers the end states of all 2*cp chunks
(B*D*O floats each — kilobytes, against the megabytes of activations an all-to-all moves),
(3) combines them into the state entering each of its chunks,
        s_in(c_j) = sum_{i<j} lam^{(j-1-i) * len} s_end0(c_i),
and (4) adds the state's response to its outputs.  Steps 1 and 4 are one operator call each.
The reference has no counterpart (it always uses the all-to-all, hyena.py:451-467); the algebra is
the chunked-scan identity of the same filter (implicit_modal.py:265-274).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import ops
from . import state


class _AllGatherStates(torch.autograd.Function):
    @staticmethod
    def forward(ctx, s):
        group, cp = state.get_context_parallel_group(), state.get_context_parallel_world_size()
        parts = [torch.empty_like(s) for _ in range(cp)]
        dist.all_gather(parts, s.contiguous(), group=group)
        return torch.stack(parts, 0)

    @staticmethod
    def backward(ctx, g):
        group = state.get_context_parallel_group()
        g = g.contiguous()
        dist.all_reduce(g, group=group)
        return g[state.get_context_parallel_rank()]


def hyena_li_modal_state_cp(feat, gamma, R, p, bias):
    cp, r = state.get_context_parallel_world_size(), state.get_context_parallel_rank()
    B, L, C = feat.shape
    half = L // 2
    two = feat.reshape(B * 2, half, C)
    # pass 1: zero-state run, only the end states are needed
    _, s_end = ops.hyena_li_modal(two, gamma, R, p, bias, None, True)
    s_end = s_end.reshape(B, 2, *s_end.shape[1:])                      # [B, 2, D, O]
    alls = _AllGatherStates.apply(s_end)                               # [cp, B, 2, D, O]
    # chunk id of (rank q, slot s): s == 0 -> q ; s == 1 -> 2cp-1-q
    logp = -torch.exp(p.float()) * torch.exp(gamma.float())            # [D, O]
    step = torch.exp(logp * half)                                      # lam^len
    n = 2 * cp
    chunk_states = [None] * n
    for q in range(cp):
        chunk_states[q] = alls[q, :, 0]
        chunk_states[n - 1 - q] = alls[q, :, 1]
    ins = []
    for cid in (r, n - 1 - r):
        s = torch.zeros_like(chunk_states[0])
        for i in range(cid):
            s = s * step + chunk_states[i]
        ins.append(s)
    s_in = torch.stack(ins, 1).reshape(B * 2, *ins[0].shape[1:])
    z = ops.hyena_li_modal(two, gamma, R, p, bias, s_in, False)
    return z.reshape(B, L, -1)
