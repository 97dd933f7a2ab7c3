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


# ------------------------------------------------------------------------------------------ peer-memory form
_PEER_WS = None


def setup_peer(group=None, ranks=None) -> bool:
    """Collective over the context-parallel group: symmetric staging buffers and the device barrier for the
    peer-memory halo exchange (csrc/halo_peer.cu).  Returns False (on every rank) if it cannot be brought up."""
    global _PEER_WS
    import ctypes
    from . import fused_tp
    group = group if group is not None else state.get_context_parallel_group()
    ranks = ranks or state.get_context_parallel_ranks()
    ok, ws = 1, None
    try:
        ws = fused_tp.TPWorkspace(group, ranks)
        P, I = ctypes.c_void_p, ctypes.c_int
        ws.lib.sb_halo_pull.restype = I
        ws.lib.sb_halo_pull.argtypes = [P, P, P, P, I, I, I, P]
        ws.lib.sb_halo_push_add.restype = I
        ws.lib.sb_halo_push_add.argtypes = [P, P, P, P, I, I, I, I, P]
        LL = ctypes.c_longlong
        ws.lib.sb_peer_copy.restype = I
        ws.lib.sb_peer_copy.argtypes = [P, P, LL, I, P]
        ws.lib.sb_peer_copy_2d.restype = I
        ws.lib.sb_peer_copy_2d.argtypes = [P, LL, P, LL, LL, LL, I, P]
        ws.lib.sb_zero_reduce_scatter.restype = I
        ws.lib.sb_zero_reduce_scatter.argtypes = [P, I, I, LL, LL, P, P, P, P]
    except Exception as exc:  # noqa: BLE001
        print(f"[rank {dist.get_rank()}] peer-memory halo set-up failed: {exc}", flush=True)
        ok = 0
    flag = torch.tensor([ok], dtype=torch.int32, device=torch.device("cuda", torch.cuda.current_device()))
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    _PEER_WS = ws if int(flag.item()) == 1 else None
    return _PEER_WS is not None


def teardown_peer() -> None:
    global _PEER_WS
    _PEER_WS = None


def _peer_ptr(ptrs, idx, cp):
    return ptrs[idx] if 0 <= idx < cp else None


class _ZigzagHaloPeer(torch.autograd.Function):
    """Same contract as _ZigzagHalo, with the neighbours' tails read from their symmetric buffers by this framework's
    own kernels: stage the two tails -> device barrier -> pull; backward: stage the halo gradients -> device barrier ->
    add the neighbours' parts onto the tail rows.  Staging buffers alternate between two slots, so one barrier per
    exchange suffices (a slot is rewritten only after the barrier of the following exchange)."""

    @staticmethod
    def forward(ctx, x, H):
        ws = _PEER_WS
        B, L, C = x.shape
        half = L // 2
        if H > half:
            raise ValueError(f"halo {H} exceeds the chunk length {half}")
        me, cp = ws.rank, ws.world
        stage, ptrs = ws.symm_buffer("halo_fwd", B * 2 * H * C)
        sv = stage.view(B, 2, H, C)
        sv[:, 0].copy_(x[:, half - H:half])
        sv[:, 1].copy_(x[:, L - H:])
        ws.barrier()
        halo = torch.empty((B, 2, H, C), dtype=x.dtype, device=x.device)
        rc = ws.lib.sb_halo_pull(halo.data_ptr(), _peer_ptr(ptrs, me - 1, cp), _peer_ptr(ptrs, me + 1, cp), stage.data_ptr(),
                                 B, H, C, torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise RuntimeError(f"sb_halo_pull failed ({rc})")
        ws.cuda_ops._count()
        ctx.meta = (H, L, C, B)
        return halo

    @staticmethod
    def backward(ctx, g):
        ws = _PEER_WS
        H, L, C, B = ctx.meta
        me, cp = ws.rank, ws.world
        stage, ptrs = ws.symm_buffer("halo_bwd", B * 2 * H * C)
        stage.view(B, 2, H, C).copy_(g)
        ws.barrier()
        gx = torch.zeros((B, L, C), dtype=g.dtype, device=g.device)
        rc = ws.lib.sb_halo_push_add(gx.data_ptr(), _peer_ptr(ptrs, me - 1, cp), _peer_ptr(ptrs, me + 1, cp), stage.data_ptr(),
                                     B, L, C, H, torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise RuntimeError(f"sb_halo_push_add failed ({rc})")
        ws.cuda_ops._count()
        return gx, None


def zigzag_halo(x: torch.Tensor, H: int) -> torch.Tensor:
    """Halo rows for both chunks of a zigzag shard: [B, 2, H, C]."""
    if (_PEER_WS is not None and x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0
            and x.shape[1] % 2 == 0):
        return _ZigzagHaloPeer.apply(x, H)
    return _ZigzagHalo.apply(x, H)
