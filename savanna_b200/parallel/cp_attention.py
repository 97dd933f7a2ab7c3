"""Context-parallel attention by head exchange ("a2a", DeepSpeed-Ulysses style) and by key/value all-gather.

The reference reaches these through TransformerEngine's DotProductAttention (`operator: flash_te` with
`flash_te_comm_type` in {"p2p", "all_gather", "a2a"}, savanna/model/block.py:483-514); "p2p" is the ring
(parallel/ring_attention.py).  Both forms here work on zigzag shards q, k, v [B, l, H, hd] (rank r holds chunks r and
2cp-1-r of the sequence, rotary embedding already applied with the tokens' true positions):

    a2a         one all-to-all turns (q, k, v) from sequence-sharded / all heads into head-sharded / whole sequence in
                natural order, plain causal attention runs on H/cp heads, a second all-to-all brings the result back.
                Needs H divisible by cp.  The exchanges go through parallel/a2a.py (peer-memory pulls on B200, NCCL or gloo
                elsewhere), so a rank moves (cp-1)/cp of its q, k, v and output once each.
    all_gather  every rank gathers the whole K and V (natural order), and each of its two query chunks attends to the
                keys before it without a mask plus its own chunk causally; the two partial results are merged by their
                log-sum-exp.  K/V gradients return by reduce-scatter.  Communication grows with cp (every rank receives
                all of K and V), so this form is for small cp or short key/value rows.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import ops
from . import a2a, state
from .ring_attention import _merge_all


def ulysses_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True) -> torch.Tensor:
    cp = state.get_context_parallel_world_size()
    if cp == 1:
        return ops.attention(q, k, v, causal=causal)
    B, l, H, hd = q.shape
    if H % cp:
        raise ValueError(f"a2a context-parallel attention needs the head count ({H}) divisible by the context-parallel size ({cp})")
    packed = torch.cat([q, k, v], dim=-1).reshape(B, l, H * 3 * hd)          # heads stay contiguous: a channel block = H/cp heads
    full = a2a.split_to_full(packed).view(B, l * cp, H // cp, 3 * hd)
    qf, kf, vf = full[..., :hd], full[..., hd:2 * hd], full[..., 2 * hd:]
    o = ops.attention(qf, kf, vf, causal=causal)                             # natural order: the plain causal kernel applies
    return a2a.full_to_split(o.reshape(B, l * cp, (H // cp) * hd).contiguous()).view(B, l, H, hd)


class _GatherKV(torch.autograd.Function):
    """[2, B, l, H, hd] zigzag shards -> [2, B, L, H, hd] in natural order; backward reduce-scatters."""

    @staticmethod
    def forward(ctx, kv):
        group, cp = state.get_context_parallel_group(), state.get_context_parallel_world_size()
        parts = [torch.empty_like(kv) for _ in range(cp)]
        dist.all_gather(parts, kv.contiguous(), group=group)
        c = kv.shape[2] // 2
        chunks = [None] * (2 * cp)
        for r, p in enumerate(parts):
            chunks[r], chunks[2 * cp - 1 - r] = p[:, :, :c], p[:, :, c:]
        return torch.cat(chunks, dim=2)

    @staticmethod
    def backward(ctx, g):
        group, cp = state.get_context_parallel_group(), state.get_context_parallel_world_size()
        me = state.get_context_parallel_rank()
        c = g.shape[2] // (2 * cp)
        shards = [torch.cat([g[:, :, r * c:(r + 1) * c], g[:, :, (2 * cp - 1 - r) * c:(2 * cp - r) * c]], dim=2).contiguous()
                  for r in range(cp)]
        out = torch.empty_like(shards[me])
        if dist.get_backend(group) == "gloo":
            stacked = torch.stack(shards)
            dist.all_reduce(stacked, group=group)
            out = stacked[me].clone()
        else:
            dist.reduce_scatter(out, shards, group=group)
        return out


def allgather_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True) -> torch.Tensor:
    cp, r = state.get_context_parallel_world_size(), state.get_context_parallel_rank()
    if cp == 1:
        return ops.attention(q, k, v, causal=causal)
    B, l, H, hd = q.shape
    c = l // 2
    kv = _GatherKV.apply(torch.stack([k, v], 0))
    kf, vf = kv[0], kv[1]
    if not causal:
        return ops.attention(q, kf, vf, causal=False)
    outs = []
    for half, chunk in ((0, r), (1, 2 * cp - 1 - r)):
        qc = q[:, half * c:(half + 1) * c]
        lo = chunk * c
        parts = [ops.attention(qc, kf[:, lo:lo + c], vf[:, lo:lo + c], causal=True, return_lse=True)]
        if lo > 0:
            parts.append(ops.attention(qc, kf[:, :lo], vf[:, :lo], causal=False, return_lse=True))
        outs.append(_merge_all(parts) if len(parts) > 1 else parts[0][0])
    return torch.cat([o.to(q.dtype) for o in outs], dim=1)
