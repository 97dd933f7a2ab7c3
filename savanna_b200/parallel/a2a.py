"""Context-parallel all-to-all between the sequence-sharded and the channel-sharded layout.

    split_to_full : [B, L/cp (zigzag shard), D]  ->  [B, L (natural order), D/cp]
    full_to_split : the inverse

This is the channel-last restatement of the reference's AllToAllSingleFunction
(savanna/model/operators/hyena/distributed_a2a.py:45-168).  Two forms: NCCL/gloo all_to_all_single with the
permutes around it, and (CUDA bf16 with the context-parallel peer workspace up) a pull over NVSwitch peer memory: the
tensor is staged once in a symmetric buffer and every rank copies its blocks from their owners straight into the final
layout with this framework's pitched-copy kernel, zigzag addressing included.
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


# ------------------------------------------------------------------------------------------ peer-memory form
def _peer_ws(x: torch.Tensor, zigzag: bool):
    """The context-parallel peer workspace when this tensor can take the pull path (CUDA bf16, zigzag, 16-byte rows)."""
    from . import halo
    ws = halo._PEER_WS
    if ws is None or not zigzag or not x.is_cuda or x.dtype != torch.bfloat16 or x.dim() != 3:
        return None
    return ws if ws.world == state.get_context_parallel_world_size() else None


def _pull(ws, dst, dst_pitch, src_ptr, src_off, src_pitch, row_bytes, rows):
    rc = ws.lib.sb_peer_copy_2d(dst, dst_pitch, src_ptr + src_off, src_pitch, row_bytes, rows, 0,
                                torch.cuda.current_stream().cuda_stream)
    if rc != 0:
        raise RuntimeError(f"sb_peer_copy_2d failed ({rc})")


def _split_to_full_peer(ws, x: torch.Tensor) -> torch.Tensor:
    """[B, l (zigzag shard), D] -> [B, l*cp (natural order), D/cp]: stage x in symmetric memory, one device barrier, then
    pull this rank's channel block of every sequence chunk from its owner straight into its natural position."""
    cp, me = ws.world, ws.rank
    B, l, D = x.shape
    d, c = D // cp, l // 2
    stage, ptrs = ws.symm_buffer("a2a_s2f", x.numel())
    stage.view(B, l, D).copy_(x)
    ws.barrier()
    full = torch.empty((B, cp * l, d), dtype=x.dtype, device=x.device)
    for j in range(2 * cp):                               # natural chunk j lives on rank j (first half) or 2cp-1-j
        owner, loc = (j, 0) if j < cp else (2 * cp - 1 - j, c)
        for b in range(B):
            _pull(ws, full[b, j * c].data_ptr(), d * 2, ptrs[owner], ((b * l + loc) * D + me * d) * 2, D * 2, d * 2, c)
    ws.cuda_ops._count(2 * cp * B)
    return full


def _full_to_split_peer(ws, x: torch.Tensor) -> torch.Tensor:
    """[B, L (natural order), d] -> [B, L/cp (zigzag shard), d*cp]: the inverse pull."""
    cp, me = ws.world, ws.rank
    B, L, d = x.shape
    l = L // cp
    c = l // 2
    stage, ptrs = ws.symm_buffer("a2a_f2s", x.numel())
    stage.view(B, L, d).copy_(x)
    ws.barrier()
    out = torch.empty((B, l, cp * d), dtype=x.dtype, device=x.device)
    for r in range(cp):                                   # channel block r comes from rank r
        for loc, j in ((0, me), (c, 2 * cp - 1 - me)):
            for b in range(B):
                _pull(ws, out[b, loc, r * d:].data_ptr(), cp * d * 2, ptrs[r], ((b * L + j * c) * d) * 2, d * 2, d * 2, c)
    ws.cuda_ops._count(2 * cp * B)
    return out


def _peer_shapes_ok(x, direction, cp) -> bool:
    if direction == "split_to_full":
        B, l, D = x.shape
        return D % cp == 0 and l % 2 == 0 and ((D // cp) * 2) % 16 == 0
    B, L, d = x.shape
    return L % (2 * cp) == 0 and (d * 2) % 16 == 0


class AllToAllSingle(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, direction, zigzag):
        ctx.direction, ctx.zigzag = direction, zigzag
        return _run(x, direction, zigzag)

    @staticmethod
    def backward(ctx, g):
        inverse = "full_to_split" if ctx.direction == "split_to_full" else "split_to_full"
        return _run(g.contiguous(), inverse, ctx.zigzag), None, None


PEER_CALLS = 0        # number of all-to-alls that took the peer-memory pull path (tests read it)


def _run(x, direction, zigzag):
    global PEER_CALLS
    ws = _peer_ws(x, zigzag)
    if ws is not None and _peer_shapes_ok(x, direction, ws.world):
        PEER_CALLS += 1
        x = x.contiguous()
        return _split_to_full_peer(ws, x) if direction == "split_to_full" else _full_to_split_peer(ws, x)
    return _split_to_full(x, zigzag) if direction == "split_to_full" else _full_to_split(x, zigzag)


def split_to_full(x, zigzag: bool = True):
    if state.get_context_parallel_world_size() == 1:
        return x
    return AllToAllSingle.apply(x, "split_to_full", zigzag)


def full_to_split(x, zigzag: bool = True):
    if state.get_context_parallel_world_size() == 1:
        return x
    return AllToAllSingle.apply(x, "full_to_split", zigzag)
