"""Tensor/sequence-parallel projections fused with their collective over NVSwitch peer memory.

    linear_allgather     Y = allgather_seq(X) W^T     one kernel: copy CTAs pull the peers' sequence shards while the
                                                      tcgen05 GEMM CTAs already work on the local shard
    linear_reducescatter Y = reduce_scatter_seq(X W^T)  the GEMM epilogue stores tiles into the owner rank's memory,
                                                      a small owner-side kernel sums the partials
(kernels: csrc/gemm_tp_sm100.cu).  Backward passes use the same two kernels with the roles swapped (the gradient of an
all-gather is a reduce-scatter and vice versa); weight gradients gather their sharded operand with a peer-copy kernel
and run the plain GEMM.  Reference call sites replaced: savanna/mpu/mappings.py:84-157 around
savanna/mpu/layers.py:525-560 and :746-786 (NCCL all-gather / reduce-scatter next to cuBLAS GEMMs).

Both entry points return None when the fused path does not apply (workspace not set up, tensor-parallel size 1,
shard not a multiple of 128 rows, non-bf16): the caller then runs the NCCL collective and the GEMM separately.  A
micro-batch of several sequences is one launch.  With `fp8` the operands are e4m3 / e5m2 bytes (per-tensor scaling;
an operand that is sharded over the group is quantised with the group-wide amax so that all shards share one scale).  Cross-GPU ordering uses stream-ordered device barriers (csrc/peer_barrier.cu, bounded waits); symmetric staging buffers are
double-buffered so that a rank can stage its next operand while a peer still reads the previous one.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from . import state

_WS: Optional["TPWorkspace"] = None
bf16 = torch.bfloat16
FP8_CALLS = 0               # fused projections that ran on fp8 operands
_SEEN_FP8_REQUEST = False   # a layer asked for fp8 on the fused path
E4M3, E5M2 = 0, 1


class TPWorkspace:
    def __init__(self, group, ranks):
        from . import symm
        from ..ops import cuda_ops
        symm_mem = symm.load()
        self.symm_mem, self.cuda_ops, self._symm_api = symm_mem, cuda_ops, symm
        self.lib = cuda_ops.require()
        P, I, LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        self.lib.sb_gemm_tp.restype = I
        self.lib.sb_gemm_tp.argtypes = [P, I, P, I, I, P, I, P, I, I, I, I, I, P, P, I, I, I, I, P, P, P, I, I, I, I, P, P, P]
        # CTA-pair variant of the fused kernels (cta_group::2, 256 x 256 tiles per SM pair) where the shapes allow it
        # (rows a multiple of 256); SAVANNA_B200_TP_PAIR=0 selects the single-CTA kernel (A/B measurements)
        self.lib.sb_gemm_tp_set_pair.restype = I
        self.lib.sb_gemm_tp_set_pair.argtypes = [I]
        self.pair = os.environ.get("SAVANNA_B200_TP_PAIR", "1") == "1"
        self.lib.sb_gemm_tp_set_pair(int(self.pair))
        self.lib.sb_rs_reduce.restype = I
        self.lib.sb_rs_reduce.argtypes = [P, P, P, P, I, LL, I, P]
        self.lib.sb_gather_rows.restype = I
        self.lib.sb_gather_rows.argtypes = [P, I, P, I, I, I, I, I, P]
        LLc = ctypes.c_longlong
        self.lib.sb_amax_bf16.restype = I
        self.lib.sb_amax_bf16.argtypes = [P, P, LLc, P]
        self.lib.sb_quantize_fp8_with_amax.restype = I
        self.lib.sb_quantize_fp8_with_amax.argtypes = [P, P, P, P, LLc, I, P]
        self.group = group if group is not None else dist.group.WORLD
        self.world = len(ranks)
        self.rank = ranks.index(dist.get_rank())
        self.dev = torch.device("cuda", torch.cuda.current_device())
        self.token = torch.zeros(1, device=self.dev)
        self.flags = torch.zeros(8192, dtype=torch.int32, device=self.dev)
        self.epoch = 0
        self.lib.sb_peer_barrier.restype = I
        self.lib.sb_peer_barrier.argtypes = [P, I, I, I, P, P]
        # signal words of the device-side barrier (int32[world] per rank, zeroed before anyone signals)
        self.sig = symm_mem.empty(32, dtype=torch.int32, device=self.dev)
        self.sig.zero_()
        hs = symm_mem.rendezvous(self.sig, self.group)
        self.sig_ptrs = (ctypes.c_void_p * self.world)(*symm.peer_pointers(hs, self.world))
        self.bar_epoch = 0
        torch.cuda.synchronize()
        dist.barrier(group=self.group)               # every rank's signal words are zero before the first device barrier
        self.symm: Dict[Tuple[str, int, int], Tuple[torch.Tensor, object]] = {}
        self.local: Dict[Tuple[str, int], torch.Tensor] = {}
        self.parity: Dict[str, int] = {}

    def barrier(self) -> None:
        """Stream-ordered barrier over the group: one small kernel with bounded peer waits (csrc/peer_barrier.cu)."""
        self.bar_epoch += 1
        rc = self.lib.sb_peer_barrier(self.sig_ptrs, self.rank, self.world, self.bar_epoch,
                                      self.cuda_ops.status_word(self.dev).data_ptr(), torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise RuntimeError(f"sb_peer_barrier failed ({rc})")
        self.cuda_ops._count()

    def symm_buffer(self, name: str, numel: int):
        """Next slot (of two) of a symmetric bf16 buffer; allocation + rendezvous happen once per (name, size, slot)."""
        slot = self.parity.get(name, 0)
        self.parity[name] = slot ^ 1
        key = (name, numel, slot)
        if key not in self.symm:
            t = self.symm_mem.empty(numel, dtype=bf16, device=self.dev)
            h = self.symm_mem.rendezvous(t, self.group)
            ptrs = (ctypes.c_void_p * self.world)(*self._symm_api.peer_pointers(h, self.world))
            self.symm[key] = (t, ptrs)
        return self.symm[key]

    def local_buffer(self, name: str, numel: int) -> torch.Tensor:
        key = (name, numel)
        if key not in self.local:
            self.local[key] = torch.empty(numel, dtype=bf16, device=self.dev)
        return self.local[key]

    def next_epoch(self) -> int:
        self.epoch = self.epoch % 2000000000 + 1
        return self.epoch

    # ---- kernel launchers -------------------------------------------------------------------------------
    def gemm_tp(self, a, w, b_mn, out, M, N, K, ag=None, rs=None, bias=None, batch=1, fp8=None):
        """ag = (src_ptrs, gather, flags_epoch) or None; rs = staging ptr array or None; fp8 = (alpha, alpha2, a_fmt,
        b_fmt) for one-byte operands (a / w / gather are uint8 tensors then) or None for bf16."""
        st = torch.cuda.current_stream().cuda_stream
        ag_world, ag_src, gather, epoch = (self.world, ag[0], ag[1].data_ptr(), ag[2]) if ag else (0, None, None, 0)
        al, al2, afmt, bfmt = (fp8[0].data_ptr(), fp8[1].data_ptr(), fp8[2], fp8[3]) if fp8 else (None, None, 0, 0)
        rc = self.lib.sb_gemm_tp(a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), int(b_mn),
                                 None if out is None else out.data_ptr(), 0 if out is None else out.stride(0),
                                 None if bias is None else bias.data_ptr(), M, N, K, batch, 1 if fp8 else 2, al, al2, afmt, bfmt,
                                 ag_world, self.rank, ag_src, gather,
                                 self.flags.data_ptr(), epoch, 16, self.world if rs is not None else 0, self.rank, rs,
                                 self.cuda_ops.status_word(self.dev).data_ptr(), st)
        if rc != 0:
            raise RuntimeError(f"sb_gemm_tp failed ({rc}) M={M} N={N} K={K} batch={batch} fp8={fp8 is not None}")
        self.cuda_ops._count()

    def rs_reduce(self, staging, out, rows, N, bias=None, residual=None):
        st = torch.cuda.current_stream().cuda_stream
        rc = self.lib.sb_rs_reduce(staging.data_ptr(), None if bias is None else bias.data_ptr(),
                                   None if residual is None else residual.data_ptr(), out.data_ptr(), self.world, rows, N, st)
        if rc != 0:
            raise RuntimeError(f"sb_rs_reduce failed ({rc})")
        self.cuda_ops._count()

    def gather_rows(self, src_ptrs, gather, M, K, ld, batch=1, elem_bytes=2):
        st = torch.cuda.current_stream().cuda_stream
        rc = self.lib.sb_gather_rows(src_ptrs, self.world, gather.data_ptr(), M, K, ld, batch, elem_bytes, st)
        if rc != 0:
            raise RuntimeError(f"sb_gather_rows failed ({rc})")
        self.cuda_ops._count()

    # ---- fp8 operands sharded over the group: one scale for all ranks ------------------------------------
    def quantize_shared(self, x2: torch.Tensor, fmt: int, name: str):
        """Quantise this rank's shard x2 [rows, K] (bf16) into the next slot of the symmetric byte buffer `name` with
        the scale of the whole gathered operand: local amax, maximum over the group (one small NCCL all-reduce on the
        compute stream), quantise.  Returns (staged uint8 view, peers' pointers, de-quantisation factor)."""
        lib, st = self.lib, torch.cuda.current_stream().cuda_stream
        amax = torch.empty(1, dtype=torch.float32, device=self.dev)
        if lib.sb_amax_bf16(x2.data_ptr(), amax.data_ptr(), x2.numel(), st) != 0:
            raise RuntimeError("sb_amax_bf16 failed")
        dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=self.group)
        stage, ptrs = self.symm_buffer(name, (x2.numel() + 1) // 2)          # bytes = numel: half as many bf16 slots
        q = stage.view(torch.uint8)[: x2.numel()].view(x2.shape)
        sinv = torch.empty(1, dtype=torch.float32, device=self.dev)
        if lib.sb_quantize_fp8_with_amax(x2.data_ptr(), q.data_ptr(), amax.data_ptr(), sinv.data_ptr(), x2.numel(), fmt, st) != 0:
            raise RuntimeError("sb_quantize_fp8_with_amax failed")
        self.cuda_ops._count(2)
        return q, ptrs, sinv

    def local_bytes(self, name: str, nbytes: int) -> torch.Tensor:
        return self.local_buffer(name, (nbytes + 1) // 2).view(torch.uint8)[:nbytes]


def setup(group=None, ranks=None) -> bool:
    """Collective over the tensor-parallel group: bring up the workspace (or agree not to)."""
    global _WS
    group = group if group is not None else state.get_model_parallel_group()
    ranks = ranks or state.get_group_ranks("model")
    ok, ws = 1, None
    try:
        ws = TPWorkspace(group, ranks)
    except Exception as exc:  # noqa: BLE001
        print(f"[rank {dist.get_rank()}] fused tensor-parallel set-up failed: {exc}", flush=True)
        ok = 0
    flag = torch.tensor([ok], dtype=torch.int32, device=torch.device("cuda", torch.cuda.current_device()))
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    _WS = ws if int(flag.item()) == 1 else None
    return _WS is not None


def teardown() -> None:
    global _WS
    _WS = None


def fp8_active():
    """None: the fused projections are off, or no layer has asked them for fp8.  True: fp8 requests ran on fp8 operands.
    False: a layer asked for fp8 and got bf16 (shape not a multiple of 16; bench.py reports it next to the dtype)."""
    if _WS is None:
        return None
    if not _SEEN_FP8_REQUEST:
        return None
    return FP8_CALLS > 0


def _eligible(x, w, rows_per_rank: int) -> bool:
    return (_WS is not None and x.is_cuda and x.dtype == bf16 and w.dtype == bf16 and rows_per_rank % 128 == 0
            and w.shape[0] % 8 == 0 and w.shape[1] % 8 == 0)


def _accumulate_wgrad(ctx_w, g2, x2, a_mn=True):
    """dW = g2^T x2 (both [T, .] row-major): into the flat gradient buffer when the parameter has one."""
    from ..ops.cuda_ops import gemm
    tgt = ctx_w.grad if getattr(ctx_w, "_fuse_grad_accum", False) else None
    if tgt is not None and tgt.dtype == bf16 and tgt.is_contiguous() and tgt.shape == ctx_w.shape:
        gemm(g2, x2, tgt, a_mn=True, b_mn=True, accumulate=True)
        return None
    gw = torch.empty_like(ctx_w)
    gemm(g2, x2, gw, a_mn=True, b_mn=True)
    return gw


class _LinearAllGather(torch.autograd.Function):
    """x [B, l, K] sequence shard -> y [B, l*tp, N] (bf16 operands)."""

    @staticmethod
    def forward(ctx, x, w, bias):
        ws = _WS
        Bn, l, K = x.shape
        N, M = w.shape[0], Bn * l * ws.world
        x2 = x.reshape(Bn * l, K)
        xs, ptrs = ws.symm_buffer("ag_x", Bn * l * K)
        xs.view(Bn * l, K).copy_(x2)
        ws.barrier()
        gather = ws.local_buffer("gather", M * K)
        out = torch.empty((M, N), dtype=bf16, device=x.device)
        ws.gemm_tp(xs.view(Bn * l, K), w, False, out, M, N, K, ag=(ptrs, gather, ws.next_epoch()), bias=bias, batch=Bn)
        ctx.save_for_backward(x2.contiguous() if not x2.is_contiguous() else x2, w)
        ctx.wref, ctx.has_bias, ctx.Bn = w, bias is not None, Bn
        return out.view(Bn, l * ws.world, N)

    @staticmethod
    def backward(ctx, gy):
        ws = _WS
        x2, w = ctx.saved_tensors
        Bn = ctx.Bn
        rows, K = x2.shape                       # rows = Bn * l
        N, M = w.shape[0], rows * ws.world
        g2 = gy.reshape(M, N)
        if not g2.is_contiguous():
            g2 = g2.contiguous()
        gx = gw = gb = None
        # stage the operand of the weight gradient for the peers, then one barrier serves both products
        xs, ptrs = ws.symm_buffer("ag_x", rows * K)
        xs.view(rows, K).copy_(x2)
        stage, sptrs = ws.symm_buffer("rs_stage", ws.world * rows * K)
        ws.barrier()
        if ctx.needs_input_grad[0]:
            # dX = reduce_scatter(dY W): epilogue stores into the owners' staging buffers
            ws.gemm_tp(g2, w, True, None, M, K, N, rs=sptrs, batch=Bn)
        if ctx.needs_input_grad[1]:
            gather = ws.local_buffer("gather", M * K)
            ws.gather_rows(ptrs, gather, M, K, K, batch=Bn)
            gw = _accumulate_wgrad(ctx.wref, g2, gather.view(M, K))
        if ctx.has_bias and ctx.needs_input_grad[2]:
            from ..ops.cuda_ops import colsum
            gb = colsum(g2).to(gy.dtype)
        if ctx.needs_input_grad[0]:
            ws.barrier()
            gx = torch.empty((rows, K), dtype=bf16, device=gy.device)
            ws.rs_reduce(stage, gx, rows, K)
            gx = gx.view(Bn, rows // Bn, K)
        return gx, gw, gb


class _LinearReduceScatter(torch.autograd.Function):
    """x [B, L, K_local] -> y [B, L/tp, N] = reduce_scatter(x w^T) (+ bias + residual on the owner), bf16 operands."""

    @staticmethod
    def forward(ctx, x, w, bias, residual):
        ws = _WS
        Bn, L, K = x.shape
        M = Bn * L
        N, rows = w.shape[0], M // ws.world          # rows = Bn * l owned by this rank
        x2 = x.reshape(M, K)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        stage, sptrs = ws.symm_buffer("rs_stage", ws.world * rows * N)
        ws.barrier()
        ws.gemm_tp(x2, w, False, None, M, N, K, rs=sptrs, batch=Bn)
        ws.barrier()
        y = torch.empty((rows, N), dtype=bf16, device=x.device)
        r2 = residual.reshape(rows, N).contiguous() if residual is not None else None
        ws.rs_reduce(stage, y, rows, N, bias=bias, residual=r2)
        ctx.save_for_backward(x2, w)
        ctx.wref, ctx.has_bias, ctx.has_res, ctx.Bn = w, bias is not None, residual is not None, Bn
        return y.view(Bn, rows // Bn, N)

    @staticmethod
    def backward(ctx, gy):
        ws = _WS
        x2, w = ctx.saved_tensors
        Bn = ctx.Bn
        M, K = x2.shape
        N, rows = w.shape[0], M // ws.world
        g2 = gy.reshape(rows, N)
        gs, ptrs = ws.symm_buffer("ag_x", rows * N)
        gs.view(rows, N).copy_(g2)
        ws.barrier()
        gather = ws.local_buffer("gather", M * N)
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            # dX = allgather(dY) W : fused pull + GEMM, W [N, K] read as the [K_red = N, N_out = K] operand
            gx = torch.empty((M, K), dtype=bf16, device=gy.device)
            ws.gemm_tp(gs.view(rows, N), w, True, gx, M, K, N, ag=(ptrs, gather, ws.next_epoch()), batch=Bn)
            gx = gx.view(Bn, M // Bn, K)
        if ctx.needs_input_grad[1]:
            if ctx.needs_input_grad[0]:
                # the fused kernel filled every remote tile of the gather buffer; add the local blocks
                gather.view(Bn, ws.world, rows // Bn, N)[:, ws.rank].copy_(g2.view(Bn, rows // Bn, N))
            else:
                ws.gather_rows(ptrs, gather, M, N, N, batch=Bn)
            gw = _accumulate_wgrad(ctx.wref, gather.view(M, N), x2)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            from ..ops.cuda_ops import colsum
            gb = colsum(g2.contiguous()).to(gy.dtype)       # bias is added once, on the owner: local column sums
        gr = gy if (ctx.has_res and ctx.needs_input_grad[3]) else None
        return gx, gw, gb, gr


# ------------------------------------------------------------------------------------------ fp8 operands
def _wgrad_fp8(wref, gq, sg, xq, sx):
    """dW = (gq^T xq) * sg * sx, into the flat gradient buffer when the parameter has one; gq [T, N] e5m2, xq [T, K] e4m3."""
    from ..ops.cuda_ops import gemm_fp8
    tgt = wref.grad if getattr(wref, "_fuse_grad_accum", False) else None
    if tgt is not None and tgt.dtype == bf16 and tgt.is_contiguous() and tgt.shape == wref.shape:
        gemm_fp8(gq, xq, tgt, sg, a_mn=True, b_mn=True, a_fmt=E5M2, b_fmt=E4M3, accumulate=True, alpha2=sx)
        return None
    gw = torch.empty(wref.shape, dtype=bf16, device=gq.device)
    gemm_fp8(gq, xq, gw, sg, a_mn=True, b_mn=True, a_fmt=E5M2, b_fmt=E4M3, alpha2=sx)
    return gw


class _LinearAllGatherFP8(torch.autograd.Function):
    """Column projection of a sequence-sharded activation with fp8 tensor-core operands: the shard is quantised to e4m3
    with the scale of the whole gathered activation (group-wide amax) straight into the symmetric staging buffer, so
    half the bytes of the bf16 path cross NVLink; weights are the cached e4m3 copy; gradients are e5m2."""

    @staticmethod
    def forward(ctx, x, w, bias):
        global FP8_CALLS
        from ..ops.cuda_ops import _fp8_weight
        ws = _WS
        Bn, l, K = x.shape
        N, M = w.shape[0], Bn * l * ws.world
        x2 = x.reshape(Bn * l, K)
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        xq, ptrs, sx = ws.quantize_shared(x2, E4M3, "ag_q")
        wq, sw = _fp8_weight(w)
        ws.barrier()
        gather = ws.local_bytes("gather", M * K)
        out = torch.empty((M, N), dtype=bf16, device=x.device)
        ws.gemm_tp(xq, wq, False, out, M, N, K, ag=(ptrs, gather, ws.next_epoch()), bias=bias, batch=Bn,
                   fp8=(sx, sw, E4M3, E4M3))
        FP8_CALLS += 1
        ctx.save_for_backward(xq.clone(), sx, wq, sw)
        ctx.wref, ctx.has_bias, ctx.Bn = w, bias is not None, Bn
        return out.view(Bn, l * ws.world, N)

    @staticmethod
    def backward(ctx, gy):
        from ..ops.cuda_ops import colsum, quantize_fp8_site
        ws = _WS
        xq, sx, wq, sw = ctx.saved_tensors
        Bn = ctx.Bn
        rows, K = xq.shape
        N, M = wq.shape[0], rows * ws.world
        g2 = gy.reshape(M, N)
        g2 = g2 if g2.is_contiguous() else g2.contiguous()
        gq, sg = quantize_fp8_site(g2, E5M2, ctx.wref, "g")            # dY is whole on every rank: local scale
        gx = gw = gb = None
        # stage the quantised shard again for the weight gradient's gather; one barrier serves both products
        stage, ptrs = ws.symm_buffer("ag_q", (rows * K + 1) // 2)
        stage.view(torch.uint8)[: rows * K].view(rows, K).copy_(xq)
        rstage, sptrs = ws.symm_buffer("rs_stage", ws.world * rows * K)
        ws.barrier()
        if ctx.needs_input_grad[0]:
            ws.gemm_tp(gq, wq, True, None, M, K, N, rs=sptrs, batch=Bn, fp8=(sg, sw, E5M2, E4M3))
        if ctx.needs_input_grad[1]:
            gather = ws.local_bytes("gather", M * K)
            ws.gather_rows(ptrs, gather, M, K, K, batch=Bn, elem_bytes=1)
            gw = _wgrad_fp8(ctx.wref, gq, sg, gather.view(M, K), sx)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            gb = colsum(g2).to(gy.dtype)
        if ctx.needs_input_grad[0]:
            ws.barrier()
            gx = torch.empty((rows, K), dtype=bf16, device=gy.device)
            ws.rs_reduce(rstage, gx, rows, K)
            gx = gx.view(Bn, rows // Bn, K)
        return gx, gw, gb


class _LinearReduceScatterFP8(torch.autograd.Function):
    """Row projection with fp8 operands followed by the reduce-scatter along the sequence (partial sums travel as bf16).
    Backward: the sharded output gradient is quantised to e5m2 with the group-wide scale and gathered inside the GEMM."""

    @staticmethod
    def forward(ctx, x, w, bias, residual):
        global FP8_CALLS
        from ..ops.cuda_ops import _fp8_weight, quantize_fp8_site
        ws = _WS
        Bn, L, K = x.shape
        M = Bn * L
        N, rows = w.shape[0], M // ws.world
        x2 = x.reshape(M, K)
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        xq, sx = quantize_fp8_site(x2, E4M3, w, "x")                   # x is whole on this rank: local (delayed) scale
        wq, sw = _fp8_weight(w)
        stage, sptrs = ws.symm_buffer("rs_stage", ws.world * rows * N)
        ws.barrier()
        ws.gemm_tp(xq, wq, False, None, M, N, K, rs=sptrs, batch=Bn, fp8=(sx, sw, E4M3, E4M3))
        ws.barrier()
        y = torch.empty((rows, N), dtype=bf16, device=x.device)
        r2 = residual.reshape(rows, N).contiguous() if residual is not None else None
        ws.rs_reduce(stage, y, rows, N, bias=bias, residual=r2)
        FP8_CALLS += 1
        ctx.save_for_backward(xq, sx, wq, sw)
        ctx.wref, ctx.has_bias, ctx.has_res, ctx.Bn = w, bias is not None, residual is not None, Bn
        return y.view(Bn, rows // Bn, N)

    @staticmethod
    def backward(ctx, gy):
        from ..ops.cuda_ops import colsum
        ws = _WS
        xq, sx, wq, sw = ctx.saved_tensors
        Bn = ctx.Bn
        M, K = xq.shape
        N, rows = wq.shape[0], M // ws.world
        g2 = gy.reshape(rows, N)
        g2 = g2 if g2.is_contiguous() else g2.contiguous()
        gq, ptrs, sg = ws.quantize_shared(g2, E5M2, "ag_q")
        ws.barrier()
        gather = ws.local_bytes("gather", M * N)
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            gx = torch.empty((M, K), dtype=bf16, device=gy.device)
            ws.gemm_tp(gq, wq, True, gx, M, K, N, ag=(ptrs, gather, ws.next_epoch()), batch=Bn, fp8=(sg, sw, E5M2, E4M3))
            gx = gx.view(Bn, M // Bn, K)
        if ctx.needs_input_grad[1]:
            if ctx.needs_input_grad[0]:
                gather.view(Bn, ws.world, rows // Bn, N)[:, ws.rank].copy_(gq.view(Bn, rows // Bn, N))
            else:
                ws.gather_rows(ptrs, gather, M, N, N, batch=Bn, elem_bytes=1)
            gw = _wgrad_fp8(ctx.wref, gather.view(M, N), sg, xq, sx)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            gb = colsum(g2).to(gy.dtype)
        gr = gy if (ctx.has_res and ctx.needs_input_grad[3]) else None
        return gx, gw, gb, gr


def _fp8_ok(x, w) -> bool:
    return w.shape[0] % 16 == 0 and w.shape[1] % 16 == 0


def linear_allgather(x, w, bias, seq_dim, fp8: bool = False):
    global _SEEN_FP8_REQUEST
    if _WS is None or seq_dim != 1 or x.dim() != 3 or not _eligible(x, w, x.shape[1]):
        return None
    if fp8:
        _SEEN_FP8_REQUEST = True
        if _fp8_ok(x, w):
            return _LinearAllGatherFP8.apply(x, w, bias)
    return _LinearAllGather.apply(x, w, bias)


def linear_reducescatter(x, w, seq_dim, bias=None, residual=None, fp8: bool = False):
    global _SEEN_FP8_REQUEST
    if _WS is None or seq_dim != 1 or x.dim() != 3:
        return None
    if x.shape[1] % _WS.world or not _eligible(x, w, x.shape[1] // _WS.world):
        return None
    if fp8:
        _SEEN_FP8_REQUEST = True
        if _fp8_ok(x, w):
            return _LinearReduceScatterFP8.apply(x, w, bias, residual)
    return _LinearReduceScatter.apply(x, w, bias, residual)
