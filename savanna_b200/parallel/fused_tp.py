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
shard not a multiple of 128 rows, non-bf16; a micro-batch > 1 runs one sequence at a time): the caller then runs the NCCL collective and the GEMM
separately.  Cross-GPU ordering uses stream-ordered device barriers (csrc/peer_barrier.cu, bounded waits); symmetric staging buffers are
double-buffered so that a rank can stage its next operand while a peer still reads the previous one.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from . import state

_WS: Optional["TPWorkspace"] = None
bf16 = torch.bfloat16


class TPWorkspace:
    def __init__(self, group, ranks):
        import torch.distributed._symmetric_memory as symm_mem
        from ..ops import cuda_ops
        self.symm_mem, self.cuda_ops = symm_mem, cuda_ops
        self.lib = cuda_ops.require()
        P, I, LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        self.lib.sb_gemm_tp.restype = I
        self.lib.sb_gemm_tp.argtypes = [P, I, P, I, I, P, I, P, I, I, I, I, I, P, P, P, I, I, I, I, P, P, P]
        self.lib.sb_rs_reduce.restype = I
        self.lib.sb_rs_reduce.argtypes = [P, P, P, P, I, LL, I, P]
        self.lib.sb_gather_rows.restype = I
        self.lib.sb_gather_rows.argtypes = [P, I, P, I, I, I, P]
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
        self.sig_ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in hs.buffer_ptrs])
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
            ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in h.buffer_ptrs])
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
    def gemm_tp(self, a, w, b_mn, out, M, N, K, ag=None, rs=None, bias=None):
        """ag = (src_ptrs, gather, flags_epoch) or None; rs = staging ptr array or None."""
        st = torch.cuda.current_stream().cuda_stream
        ag_world, ag_src, gather, epoch = (self.world, ag[0], ag[1].data_ptr(), ag[2]) if ag else (0, None, None, 0)
        rc = self.lib.sb_gemm_tp(a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), int(b_mn),
                                 None if out is None else out.data_ptr(), 0 if out is None else out.stride(0),
                                 None if bias is None else bias.data_ptr(), M, N, K, ag_world, self.rank, ag_src, gather,
                                 self.flags.data_ptr(), epoch, 16, self.world if rs is not None else 0, self.rank, rs,
                                 self.cuda_ops.status_word(self.dev).data_ptr(), st)
        if rc != 0:
            raise RuntimeError(f"sb_gemm_tp failed ({rc}) M={M} N={N} K={K}")
        self.cuda_ops._count()

    def rs_reduce(self, staging, out, rows, N, bias=None, residual=None):
        st = torch.cuda.current_stream().cuda_stream
        rc = self.lib.sb_rs_reduce(staging.data_ptr(), None if bias is None else bias.data_ptr(),
                                   None if residual is None else residual.data_ptr(), out.data_ptr(), self.world, rows, N, st)
        if rc != 0:
            raise RuntimeError(f"sb_rs_reduce failed ({rc})")
        self.cuda_ops._count()

    def gather_rows(self, src_ptrs, gather, M, K, ld):
        st = torch.cuda.current_stream().cuda_stream
        rc = self.lib.sb_gather_rows(src_ptrs, self.world, gather.data_ptr(), M, K, ld, st)
        if rc != 0:
            raise RuntimeError(f"sb_gather_rows failed ({rc})")
        self.cuda_ops._count()


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
    """None: the fused projections are off.  False: they are on and run bf16 GEMMs even where the layer asks for fp8
    (reported by bench.py next to the dtype).  True: they run fp8 operands."""
    if _WS is None:
        return None
    return False


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
    """x [1, l, K] sequence shard -> y [1, l*tp, N]."""

    @staticmethod
    def forward(ctx, x, w, bias):
        ws = _WS
        l, K = x.shape[1], x.shape[2]
        N, M = w.shape[0], l * ws.world
        x2 = x.reshape(l, K)
        xs, ptrs = ws.symm_buffer("ag_x", l * K)
        xs.view(l, K).copy_(x2)
        ws.barrier()
        gather = ws.local_buffer("gather", M * K)
        out = torch.empty((M, N), dtype=bf16, device=x.device)
        ws.gemm_tp(xs.view(l, K), w, False, out, M, N, K, ag=(ptrs, gather, ws.next_epoch()), bias=bias)
        ctx.save_for_backward(x2.contiguous() if not x2.is_contiguous() else x2, w)
        ctx.wref, ctx.has_bias = w, bias is not None
        return out.view(1, M, N)

    @staticmethod
    def backward(ctx, gy):
        ws = _WS
        x2, w = ctx.saved_tensors
        l, K = x2.shape
        N, M = w.shape[0], l * ws.world
        g2 = gy.reshape(M, N)
        if not g2.is_contiguous():
            g2 = g2.contiguous()
        gx = gw = gb = None
        # stage the operand of the weight gradient for the peers, then one barrier serves both products
        xs, ptrs = ws.symm_buffer("ag_x", l * K)
        xs.view(l, K).copy_(x2)
        stage, sptrs = ws.symm_buffer("rs_stage", ws.world * l * K)
        ws.barrier()
        if ctx.needs_input_grad[0]:
            # dX = reduce_scatter(dY W): epilogue stores into the owners' staging buffers
            ws.gemm_tp(g2, w, True, None, M, K, N, rs=sptrs)
        if ctx.needs_input_grad[1]:
            gather = ws.local_buffer("gather", M * K)
            ws.gather_rows(ptrs, gather, M, K, K)
            gw = _accumulate_wgrad(ctx.wref, g2, gather.view(M, K))
        if ctx.has_bias and ctx.needs_input_grad[2]:
            from ..ops.cuda_ops import colsum
            gb = colsum(g2).to(gy.dtype)
        if ctx.needs_input_grad[0]:
            ws.barrier()
            gx = torch.empty((l, K), dtype=bf16, device=gy.device)
            ws.rs_reduce(stage, gx, l, K)
            gx = gx.view(1, l, K)
        return gx, gw, gb


class _LinearReduceScatter(torch.autograd.Function):
    """x [1, L, K_local] -> y [1, L/tp, N] = reduce_scatter(x w^T) (+ bias + residual on the owner)."""

    @staticmethod
    def forward(ctx, x, w, bias, residual):
        ws = _WS
        M, K = x.shape[1], x.shape[2]
        N, l = w.shape[0], x.shape[1] // ws.world
        x2 = x.reshape(M, K)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        stage, sptrs = ws.symm_buffer("rs_stage", ws.world * l * N)
        ws.barrier()
        ws.gemm_tp(x2, w, False, None, M, N, K, rs=sptrs)
        ws.barrier()
        y = torch.empty((l, N), dtype=bf16, device=x.device)
        r2 = residual.reshape(l, N).contiguous() if residual is not None else None
        ws.rs_reduce(stage, y, l, N, bias=bias, residual=r2)
        ctx.save_for_backward(x2, w)
        ctx.wref, ctx.has_bias, ctx.has_res = w, bias is not None, residual is not None
        return y.view(1, l, N)

    @staticmethod
    def backward(ctx, gy):
        ws = _WS
        x2, w = ctx.saved_tensors
        M, K = x2.shape
        N, l = w.shape[0], M // ws.world
        g2 = gy.reshape(l, N)
        gs, ptrs = ws.symm_buffer("ag_x", l * N)
        gs.view(l, N).copy_(g2)
        ws.barrier()
        gather = ws.local_buffer("gather", M * N)
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            # dX = allgather(dY) W : fused pull + GEMM, W [N, K] read as the [K_red = N, N_out = K] operand
            gx = torch.empty((M, K), dtype=bf16, device=gy.device)
            ws.gemm_tp(gs.view(l, N), w, True, gx, M, K, N, ag=(ptrs, gather, ws.next_epoch()))
            gx = gx.view(1, M, K)
        if ctx.needs_input_grad[1]:
            if ctx.needs_input_grad[0]:
                # the fused kernel filled every remote tile of the gather buffer; add the local shard
                gather.view(M, N)[ws.rank * l:(ws.rank + 1) * l].copy_(g2)
            else:
                ws.gather_rows(ptrs, gather, M, N, N)
            gw = _accumulate_wgrad(ctx.wref, gather.view(M, N), x2)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            from ..ops.cuda_ops import colsum
            gb = colsum(g2.contiguous()).to(gy.dtype)       # bias is added once, on the owner: local column sums
        gr = gy if (ctx.has_res and ctx.needs_input_grad[3]) else None
        return gx, gw, gb, gr


def linear_allgather(x, w, bias, seq_dim):
    if _WS is None or seq_dim != 1 or x.dim() != 3 or not _eligible(x, w, x.shape[1]):
        return None
    if x.shape[0] == 1:
        return _LinearAllGather.apply(x, w, bias)
    # the kernels take one sequence at a time (a rank's shard must be one block of rows): loop over the micro-batch
    return torch.cat([_LinearAllGather.apply(x[b:b + 1], w, bias) for b in range(x.shape[0])], dim=0)


def linear_reducescatter(x, w, seq_dim, bias=None, residual=None):
    if _WS is None or seq_dim != 1 or x.dim() != 3:
        return None
    if x.shape[1] % _WS.world or not _eligible(x, w, x.shape[1] // _WS.world):
        return None
    if x.shape[0] == 1:
        return _LinearReduceScatter.apply(x, w, bias, residual)
    return torch.cat([_LinearReduceScatter.apply(x[b:b + 1], w, bias, None if residual is None else residual[b:b + 1])
                      for b in range(x.shape[0])], dim=0)
