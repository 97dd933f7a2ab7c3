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
    if _peer_ring_ok(q, k, v):
        return _RingAttentionPeer.apply(q.contiguous(), k.contiguous(), v.contiguous(), causal)
    B, L, H, hd = q.shape
    half = L // 2
    q0, q1 = q[:, :half], q[:, half:]
    kv = torch.stack([k, v], 0).contiguous()
    # partial results per half of the local queries: (output, lse) pairs over disjoint key sets, merged once at the end
    parts0, parts1 = [], []
    for s in range(cp):
        src = (r - s) % cp                      # owner of the KV shard used in this step
        ks, vs = kv[0], kv[1]
        k0, k1, v0, v1 = ks[:, :half], ks[:, half:], vs[:, :half], vs[:, half:]
        if not causal:
            o, l = ops.attention(q, ks, vs, causal=False, return_lse=True)
            parts0.append((o[:, :half], l[..., :half]))
            parts1.append((o[:, half:], l[..., half:]))
        elif src == r:
            # own shard: first half causal on itself; second half sees the whole first half and itself causally
            parts0.append(ops.attention(q0, k0, v0, causal=True, return_lse=True))
            parts1.append(ops.attention(q1, k0, v0, causal=False, return_lse=True))
            parts1.append(ops.attention(q1, k1, v1, causal=True, return_lse=True))
        elif src < r:
            # chunks (src, 2cp-1-src): chunk src precedes both of my chunks; chunk 2cp-1-src follows both -> only k0
            o, l = ops.attention(q, k0, v0, causal=False, return_lse=True)
            parts0.append((o[:, :half], l[..., :half]))
            parts1.append((o[:, half:], l[..., half:]))
        else:
            # src > r: chunk src follows my first chunk and precedes my second; so does chunk 2cp-1-src
            parts1.append(ops.attention(q1, ks, vs, causal=False, return_lse=True))
        if s + 1 < cp:
            kv = _RingShift.apply(kv)
    return torch.cat([_merge_all(parts0), _merge_all(parts1)], dim=1).to(q.dtype)


# ------------------------------------------------------------------------------------------ peer-memory form
_SIDE = {}


def _side_stream(dev):
    if dev not in _SIDE:
        _SIDE[dev] = torch.cuda.Stream(device=dev)
    return _SIDE[dev]


def _block_plan(me: int, src: int, causal: bool):
    """The attention calls of one ring step as (query part, key part, causal) with parts 'lo' / 'hi' / 'all' (halves of
    the local zigzag shard): rank r holds chunks (r, 2cp-1-r), so a key shard of an earlier rank contributes only its
    first chunk (to all local queries), one of a later rank contributes both chunks to the second half only."""
    if not causal:
        return [("all", "all", False)]
    if src == me:
        return [("lo", "lo", True), ("hi", "lo", False), ("hi", "hi", True)]
    if src < me:
        return [("all", "lo", False)]
    return [("hi", "all", False)]


def _part(t, which, half):
    return t if which == "all" else (t[:, :half] if which == "lo" else t[:, half:])


class _RingAttentionPeer(torch.autograd.Function):
    """Zigzag ring attention over NVSwitch peer memory, one autograd node (B = 1, bf16, 128-wide heads).

    Forward: every rank stages its K/V shard in a symmetric buffer; after one device barrier each step copies the shard
    it needs from its owner with this framework's copy kernel on a side stream, one step ahead of the tcgen05 attention
    kernels working on the previous shard, so the transfers hide behind the math.  The partial results of a query half
    are combined by the fused merge kernel.
    Backward: the block gradients are computed against the merged output and log-sum-exp (then every block's softmax is
    the global one, no merge backward is needed); dq accumulates in one fp32 buffer across the steps; the K/V gradients
    of every shard are written into a per-owner slot of a symmetric buffer and, after a barrier, each owner sums its
    slot over all ranks with peer loads.  Replaces the NCCL send/recv ring (reference: ring_flash_attn zigzag, called
    from savanna/model/operators/attention/flash.py:523-597)."""

    @staticmethod
    def forward(ctx, q, k, v, causal):
        from ..ops import cuda_ops, flash_sm100
        from . import halo
        ws = halo._PEER_WS
        me, cp = ws.rank, ws.world
        B, L, H, hd = q.shape
        half, n = L // 2, q.numel()
        dev, scale = q.device, hd ** -0.5
        main, side = torch.cuda.current_stream(), _side_stream(dev)
        stage, ptrs = ws.symm_buffer("ring_kv", 2 * n)
        sv = stage.view(2, B, L, H, hd)
        sv[0].copy_(k)
        sv[1].copy_(v)
        ws.barrier()
        ready = torch.cuda.Event()
        ready.record(main)
        side.wait_event(ready)
        bufs = [torch.empty(2 * n, dtype=q.dtype, device=dev) for _ in range(min(2, cp - 1))]
        free = [None, None]

        def prefetch(step):
            b = step % len(bufs)
            if free[b] is not None:
                side.wait_event(free[b])
            src = (me - step) % cp
            rc = ws.lib.sb_peer_copy(bufs[b].data_ptr(), ptrs[src], 2 * n * 2, 64, side.cuda_stream)
            if rc != 0:
                raise RuntimeError(f"sb_peer_copy failed ({rc})")
            ev = torch.cuda.Event()
            ev.record(side)
            return ev

        parts = {"lo": [], "hi": []}
        nxt = prefetch(1) if cp > 1 else None
        for s in range(cp):
            src = (me - s) % cp
            if s == 0:
                ks, vs = k, v
            else:
                main.wait_event(nxt)
                kvb = bufs[s % len(bufs)].view(2, B, L, H, hd)
                ks, vs = kvb[0], kvb[1]
                nxt = prefetch(s + 1) if s + 1 < cp else None
            for qp, kp, cz in _block_plan(me, src, causal):
                o, l = flash_sm100.forward(_part(q, qp, half), _part(ks, kp, half), _part(vs, kp, half), cz, scale)
                if qp == "all":
                    parts["lo"].append((o[:, :half], l[..., :half]))
                    parts["hi"].append((o[:, half:], l[..., half:]))
                else:
                    parts[qp].append((o, l))
            if s > 0:
                ev = torch.cuda.Event()
                ev.record(main)
                free[s % len(bufs)] = ev
        cuda_ops._count(max(cp - 1, 0))
        o_lo, l_lo = flash_sm100.merge_forward([p[0] for p in parts["lo"]], [p[1] for p in parts["lo"]])
        o_hi, l_hi = flash_sm100.merge_forward([p[0] for p in parts["hi"]], [p[1] for p in parts["hi"]])
        out = torch.cat([o_lo, o_hi], dim=1)
        lse = torch.cat([l_lo, l_hi], dim=2)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.causal = causal
        return out

    @staticmethod
    def backward(ctx, go):
        from ..ops import cuda_ops, flash_sm100
        from . import halo
        q, k, v, out, lse = ctx.saved_tensors
        causal = ctx.causal
        ws = halo._PEER_WS
        me, cp = ws.rank, ws.world
        B, L, H, hd = q.shape
        half, n = L // 2, q.numel()
        dev, scale = q.device, hd ** -0.5
        main, side = torch.cuda.current_stream(), _side_stream(dev)
        go = go.contiguous()
        stage, ptrs = ws.symm_buffer("ring_kv", 2 * n)
        sv = stage.view(2, B, L, H, hd)
        sv[0].copy_(k)
        sv[1].copy_(v)
        dstage, dptrs = ws.symm_buffer("ring_dkv", cp * 2 * n)
        dstage.zero_()
        dsv = dstage.view(cp, 2, B, L, H, hd)
        ws.barrier()
        ready = torch.cuda.Event()
        ready.record(main)
        side.wait_event(ready)
        bufs = [torch.empty(2 * n, dtype=q.dtype, device=dev) for _ in range(min(2, cp - 1))]
        free = [None, None]

        def prefetch(step):
            b = step % len(bufs)
            if free[b] is not None:
                side.wait_event(free[b])
            src = (me - step) % cp
            rc = ws.lib.sb_peer_copy(bufs[b].data_ptr(), ptrs[src], 2 * n * 2, 64, side.cuda_stream)
            if rc != 0:
                raise RuntimeError(f"sb_peer_copy failed ({rc})")
            ev = torch.cuda.Event()
            ev.record(side)
            return ev

        dq_acc = torch.zeros((B, L, H, hd), dtype=torch.float32, device=dev)
        lse_parts = {"all": lse, "lo": lse[..., :half].contiguous(), "hi": lse[..., half:].contiguous()}
        nxt = prefetch(1) if cp > 1 else None
        for s in range(cp):
            src = (me - s) % cp
            if s == 0:
                ks, vs = k, v
            else:
                main.wait_event(nxt)
                kvb = bufs[s % len(bufs)].view(2, B, L, H, hd)
                ks, vs = kvb[0], kvb[1]
                nxt = prefetch(s + 1) if s + 1 < cp else None
            written = set()
            for qp, kp, cz in _block_plan(me, src, causal):
                dk_dst, dv_dst = _part(dsv[src, 0], kp, half), _part(dsv[src, 1], kp, half)
                first = kp not in written
                dk_t = dk_dst if first else None
                dv_t = dv_dst if first else None
                _, dk_o, dv_o = flash_sm100.backward(_part(go, qp, half), _part(q, qp, half), _part(ks, kp, half),
                                                     _part(vs, kp, half), _part(out, qp, half), lse_parts[qp], cz, scale,
                                                     dq_acc=_part(dq_acc, qp, half), dk=dk_t, dv=dv_t)
                if not first:                      # a second block on the same keys (own shard): add to the slot
                    dk_dst += dk_o
                    dv_dst += dv_o
                written.add(kp)
            if s > 0:
                ev = torch.cuda.Event()
                ev.record(main)
                free[s % len(bufs)] = ev
        cuda_ops._count(max(cp - 1, 0))
        ws.barrier()
        # every owner sums its slot over all ranks (fp32 accumulation, peer loads)
        dkv = torch.empty(2 * n, dtype=q.dtype, device=dev)
        sq = torch.zeros((), dtype=torch.float32, device=dev)
        rc = ws.lib.sb_zero_reduce_scatter(dptrs, cp, me, me * 2 * n, 2 * n, dkv.data_ptr(), None, sq.data_ptr(),
                                           main.cuda_stream)
        if rc != 0:
            raise RuntimeError(f"slot reduction failed ({rc})")
        cuda_ops._count()
        dkv = dkv.view(2, B, L, H, hd)
        return dq_acc.to(q.dtype), dkv[0], dkv[1], None


def _peer_ring_ok(q, k, v) -> bool:
    from . import halo
    ws = halo._PEER_WS
    return (ws is not None and q.is_cuda and q.dtype == torch.bfloat16 and q.shape[0] == 1 and q.shape[-1] == 128
            and q.shape[1] % 2 == 0 and k.shape == q.shape and v.shape == q.shape and (q.numel() * 2) % 16 == 0
            and ws.world == state.get_context_parallel_world_size())


def _merge_all(parts):
    """Combine the partial results of one query block.  CUDA bf16 with 128-wide heads: one fused kernel (forward and
    backward); otherwise the pairwise log-sum-exp merge in PyTorch."""
    os_, lses = [p[0] for p in parts], [p[1] for p in parts]
    if os_[0].is_cuda:
        from ..ops import flash_sm100
        if flash_sm100.merge_supported(os_, lses):
            return flash_sm100.merge_partials(os_, lses)[0]
    o_acc = l_acc = None
    for o, l in parts:
        o_acc, l_acc = _merge(o_acc, l_acc, o, l)
    return o_acc
