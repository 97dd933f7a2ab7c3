"""Context-parallel causal attention over zigzag shards (ring of KV blocks, log-sum-exp merge).

Rank r holds query/key/value rows of chunks (c_r, c_{2cp-1-r}).  In step s it attends to the KV shard of
rank (r - s) mod cp; partial outputs are merged with their log-sum-exp.  Because of the zigzag layout
every (query half, KV half) pair is either fully visible, causal-diagonal (same chunk) or fully masked,
so each step is expressed with plain `causal` in {True, False} attention calls and no masks
(reference: operators/attention/flash.py:523-597 via ring_flash_attn's zigzag variant).
The KV exchange is a differentiable ring shift (send/recv on the context-parallel group).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import ops
from . import state


def _acc(t):
    return t.float() if t.dtype in (torch.bfloat16, torch.float16) else t


def _merge(o_acc, lse_acc, o, lse):
    """Merge two partial attention results (o [B,L,H,hd], lse [B,H,L]); accumulation in fp32 or wider."""
    if o_acc is None:
        return _acc(o), _acc(lse)
    lse = _acc(lse).to(lse_acc.dtype)
    new = torch.logaddexp(lse_acc, lse)
    wa = torch.exp(lse_acc - new).transpose(1, 2).unsqueeze(-1)
    wb = torch.exp(lse - new).transpose(1, 2).unsqueeze(-1)
    return o_acc * wa + _acc(o) * wb, new


def _exchange(t: torch.Tensor, dst: int, src: int, group) -> torch.Tensor:
    out = torch.empty_like(t)
    for req in dist.batch_isend_irecv([dist.P2POp(dist.isend, t.contiguous(), dst, group),
                                       dist.P2POp(dist.irecv, out, src, group)]):
        req.wait()
    return out


class _RingShift(torch.autograd.Function):
    """Pass a tensor to the next rank of the ring and receive the previous rank's; the gradient travels
    the other way, so KV gradients produced on other ranks come home."""

    @staticmethod
    def forward(ctx, t):
        group, ranks, r = state.get_context_parallel_group(), state.get_context_parallel_ranks(), state.get_context_parallel_rank()
        cp = len(ranks)
        return _exchange(t, ranks[(r + 1) % cp], ranks[(r - 1) % cp], group)

    @staticmethod
    def backward(ctx, g):
        group, ranks, r = state.get_context_parallel_group(), state.get_context_parallel_ranks(), state.get_context_parallel_rank()
        cp = len(ranks)
        return _exchange(g.contiguous(), ranks[(r - 1) % cp], ranks[(r + 1) % cp], group)


def ring_attention(q, k, v, positions, causal: bool = True):
    group, ranks, r = state.get_context_parallel_group(), state.get_context_parallel_ranks(), state.get_context_parallel_rank()
    cp = len(ranks)
    if cp == 1:
        return ops.attention(q, k, v, causal=causal)
    B, L, H, hd = q.shape
    half = L // 2
    q0, q1 = q[:, :half], q[:, half:]
    kv = torch.stack([k, v], 0).contiguous()
    o0 = l0 = o1 = l1 = None
    for s in range(cp):
        src = (r - s) % cp                      # owner of the KV shard used in this step
        ks, vs = kv[0], kv[1]
        k0, k1, v0, v1 = ks[:, :half], ks[:, half:], vs[:, :half], vs[:, half:]
        if not causal:
            o, l = ops.attention(q, ks, vs, causal=False, return_lse=True)
            oa, la = _merge(None if o0 is None else torch.cat([o0, o1], 1), None if l0 is None else torch.cat([l0, l1], 2), o, l)
            o0, o1, l0, l1 = oa[:, :half], oa[:, half:], la[..., :half], la[..., half:]
        elif src == r:
            # own shard: first half causal on itself; second half sees the whole first half and itself causally
            o, l = ops.attention(q0, k0, v0, causal=True, return_lse=True)
            o0, l0 = _merge(o0, l0, o, l)
            o, l = ops.attention(q1, k0, v0, causal=False, return_lse=True)
            o1, l1 = _merge(o1, l1, o, l)
            o, l = ops.attention(q1, k1, v1, causal=True, return_lse=True)
            o1, l1 = _merge(o1, l1, o, l)
        elif src < r:
            # chunks (src, 2cp-1-src): chunk src precedes both of my chunks; chunk 2cp-1-src follows both -> only k0
            o, l = ops.attention(q, k0, v0, causal=False, return_lse=True)
            o0, l0 = _merge(o0, l0, o[:, :half], l[..., :half])
            o1, l1 = _merge(o1, l1, o[:, half:], l[..., half:])
        else:
            # src > r: chunk src follows my first chunk and precedes my second; so does chunk 2cp-1-src
            o, l = ops.attention(q1, ks, vs, causal=False, return_lse=True)
            o1, l1 = _merge(o1, l1, o, l)
        if s + 1 < cp:
            kv = _RingShift.apply(kv)
    return torch.cat([o0, o1], dim=1).to(q.dtype)
