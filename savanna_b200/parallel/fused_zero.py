"""ZeRO-1 step over NVLink peer memory (the "symm" communication path).

The flat bf16 gradient and parameter buffers of every rank are allocated in symmetric memory
(torch.distributed._symmetric_memory: each rank maps all peers' buffers).  One optimizer step is then

    barrier (stream-ordered)                         every rank's backward has finished writing gradients
    zero_rs_kernel      per flat group               peer loads -> fp32 sum -> own shard + squared-norm partial
    all-reduce of one scalar                         global gradient norm (also orders the ranks)
    zero_adam_kernel    per flat group               Adam on the shard + peer stores of the new bf16 params
    barrier (stream-ordered)                         all parameter stores have landed before the next forward

(csrc/zero_fused.cu).  Barriers are tiny NCCL all-reduces on the compute stream, so the kernels themselves
never wait on a peer.

Overlap with backward (`overlap_comm`, the reference's `zero_optimization.overlap_comm`): during the LAST micro-batch's
backward the model reports, block by block, which parameters' gradients are final (models/backbone.py:
`grad_boundary_callback`).  For every report the side stream waits for the compute stream's position, runs a device
barrier (all ranks have finished those blocks) and reduce-scatters the newly final range of each flat group - the part
of it that lies in this rank's shard - while the compute stream carries on with the earlier blocks' backward.  The
optimizer step then only reduces what is left (the first block and the embedding) before Adam.  When the symmetric buffers carry an NVLink multicast mapping (`use_nvls`), the reduce-scatter
reads the in-switch sum with multimem.ld_reduce and the parameter all-gather is one multimem.st per 16 bytes.  fp32 flat groups (filter parameters, a few MB) stay on the NCCL path.
Reference behaviour replaced: DeepSpeed stage-1 reduce-scatter, fused Adam and all-gather
(savanna/training.py:1329-1337, 1391-1400, 1497).
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import print_rank_0
from . import state, symm


class SymmAllocator:
    """Allocates flat buffers in symmetric memory and remembers the handles for the later rendezvous."""

    def __init__(self, group):
        from . import symm
        self.symm_mem = symm.load()
        self.group = group
        self.tensors: List[torch.Tensor] = []

    def __call__(self, n: int, dtype: torch.dtype) -> torch.Tensor:
        dev = torch.device("cuda", torch.cuda.current_device())
        if dtype != torch.bfloat16:
            return torch.zeros(n, dtype=dtype, device=dev)
        t = self.symm_mem.empty(n, dtype=dtype, device=dev)
        t.zero_()
        self.tensors.append(t)
        return t

    def rendezvous(self, t: torch.Tensor):
        group = self.group if self.group is not None else dist.group.WORLD
        return self.symm_mem.rendezvous(t, group)


class FusedZeroStep:
    def __init__(self, opt, allocator: SymmAllocator, use_nvls: bool = True):
        from ..ops import cuda_ops
        self.lib = cuda_ops.require()
        self.cuda_ops = cuda_ops
        P, I, LL, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
        self.lib.sb_zero_reduce_scatter.restype = I
        self.lib.sb_zero_reduce_scatter.argtypes = [P, I, I, LL, LL, P, P, P, P]
        self.lib.sb_zero_adam_allgather.restype = I
        self.lib.sb_zero_adam_allgather.argtypes = [P, P, P, P, P, P, I, I, LL, LL, F, F, F, F, F, F, F, I, P, P]
        self.lib.sb_zero_reduce_scatter_mm.restype = I
        self.lib.sb_zero_reduce_scatter_mm.argtypes = [P, LL, LL, P, P, P, P]
        self.world, self.rank = opt.world, opt.rank
        self.handles = {}
        for g in opt.groups:
            if g.flat_param.dtype != torch.bfloat16:
                continue
            hg = allocator.rendezvous(g.flat_grad)
            hp = allocator.rendezvous(g.flat_param)
            gp = (ctypes.c_void_p * self.world)(*symm.peer_pointers(hg, self.world))
            pp = (ctypes.c_void_p * self.world)(*symm.peer_pointers(hp, self.world))
            # NVLS: the buffers' multicast addresses (0 when the fabric offers none)
            mcg = symm.multicast_pointer(hg) if use_nvls else 0
            mcp = symm.multicast_pointer(hp) if use_nvls else 0
            self.handles[id(g)] = (hg, hp, gp, pp, mcg, mcp)
        self.nvls = bool(self.handles) and all(h[4] and h[5] for h in self.handles.values())
        dev = opt.groups[0].flat_param.device
        self.dev = dev
        self._token = torch.zeros(1, device=dev)
        self._sq = torch.zeros((), dtype=torch.float32, device=dev)
        # ---- overlap of the reduce-scatter with the last micro-batch's backward
        self.overlap = False                 # armed by begin_overlap(), consumed by step()
        self.overlap_launches = 0            # reduce-scatter kernels launched from the backward (tests / bench read it)
        self.overlap_rounds = 0              # barriers issued from the backward (same on every rank)
        self._watermark = {}                 # id(group) -> start of the range already handed to the side stream
        self._block_start = None             # per group: flat offset of the first parameter of every block
        self._side = None
        self._sig = None
        if self.handles:
            self.lib.sb_peer_barrier.restype = I
            self.lib.sb_peer_barrier.argtypes = [P, I, I, I, P, P]
            self._sig = allocator.symm_mem.empty(32, dtype=torch.int32, device=dev)
            self._sig.zero_()
            hs = allocator.rendezvous(self._sig)
            self._sig_ptrs = (ctypes.c_void_p * self.world)(*symm.peer_pointers(hs, self.world))
            self._bar_epoch = 0
            torch.cuda.synchronize()
            dist.barrier(group=opt.group)    # every rank's signal words are zero before the first device barrier

    def _barrier(self, group) -> None:
        dist.all_reduce(self._token, group=group)          # stream-ordered: completes once every rank has arrived

    # ------------------------------------------------------------------ overlap with backward
    def index_blocks(self, opt, block_params) -> None:
        """`block_params[i]`: the parameters of block i, in model order.  Records, per flat group, the offset at which
        each block's parameters start (groups are flattened in model order, so 'blocks >= i are final' is a suffix)."""
        self._block_start = {}
        for g in opt.groups:
            off_of = {id(p): o for p, o in zip(g.params, g.offsets)}
            starts, nxt = [], g.numel
            for params in reversed(block_params):
                offs = [off_of[id(p)] for p in params if id(p) in off_of]
                if offs:
                    nxt = min(min(offs), nxt)
                starts.append(nxt)
            self._block_start[id(g)] = list(reversed(starts))

    def begin_overlap(self, opt) -> bool:
        """Arm the overlap for the backward that follows (the last micro-batch of the step)."""
        if self._block_start is None or not self.handles:
            return False
        if self._side is None:
            self._side = torch.cuda.Stream(device=self.dev)
        self._sq.zero_()
        for g in opt.groups:
            self._watermark[id(g)] = g.padded
        self.overlap = True
        return True

    def _reduce_range(self, opt, g, lo: int, hi: int, stream) -> None:
        """Reduce-scatter the part of [lo, hi) that lies in this rank's shard of flat group g, on `stream`."""
        s_lo, s_hi = g.rank * g.shard, (g.rank + 1) * g.shard
        a, b = max(lo, s_lo), min(hi, s_hi)
        if a >= b:
            return
        h = self.handles[id(g)]
        out = g.flat_grad[a:b]
        nw = None if g.norm_weight is None else g.norm_weight[a - s_lo:].data_ptr()
        if self.nvls:
            rc = self.lib.sb_zero_reduce_scatter_mm(h[4], a, b - a, out.data_ptr(), nw, self._sq.data_ptr(), stream)
        else:
            rc = self.lib.sb_zero_reduce_scatter(h[2], self.world, self.rank, a, b - a, out.data_ptr(), nw,
                                                 self._sq.data_ptr(), stream)
        if rc != 0:
            raise RuntimeError(f"zero_reduce_scatter failed ({rc})")
        self.cuda_ops._count()

    def grads_final_from(self, opt, first_final_block: int) -> None:
        """Called from the backward: every parameter of blocks >= `first_final_block` has its final gradient on this
        rank.  Hands the newly final range of every flat group to the side stream."""
        if not self.overlap:
            return
        todo = []
        for g in opt.groups:
            if id(g) not in self.handles:
                continue
            starts = self._block_start[id(g)]
            if first_final_block >= len(starts):
                continue
            new = -(-starts[first_final_block] // 256) * 256          # round up: 512-byte aligned ranges
            old = self._watermark[id(g)]
            if new < old:
                todo.append((g, new, old))
                self._watermark[id(g)] = new
        if not todo:
            return
        side = self._side
        self.overlap_rounds += 1
        side.wait_stream(torch.cuda.current_stream())
        # all ranks have finished these blocks' backward (every rank issues the same barriers in the same order)
        self._bar_epoch += 1
        rc = self.lib.sb_peer_barrier(self._sig_ptrs, self.rank, self.world, self._bar_epoch,
                                      self.cuda_ops.status_word(self.dev).data_ptr(), side.cuda_stream)
        if rc != 0:
            raise RuntimeError(f"sb_peer_barrier failed ({rc})")
        self.cuda_ops._count()
        for g, lo, hi in todo:
            before = self.cuda_ops.launch_count()
            self._reduce_range(opt, g, lo, hi, side.cuda_stream)
            self.overlap_launches += self.cuda_ops.launch_count() - before

    @torch.no_grad()
    def step(self, opt) -> torch.Tensor:
        opt.step_count += 1
        st = torch.cuda.current_stream().cuda_stream
        self._barrier(opt.group)
        overlapped = self.overlap
        self.overlap = False
        if overlapped:
            # ranges reduced from the backward have accumulated into _sq on the side stream; join it
            torch.cuda.current_stream().wait_stream(self._side)
        else:
            self._sq.zero_()
        shards = []
        for g in opt.groups:
            h = self.handles.get(id(g))
            if h is None:
                s = opt._reduce_scatter(g)
                self._sq += self.cuda_ops.sq_norm(s, g.norm_weight) if s.is_cuda else (s.float() ** 2).sum()
                shards.append(s)
                continue
            # whatever the backward has not handed over yet (everything, without overlap)
            self._reduce_range(opt, g, 0, self._watermark.get(id(g), g.padded) if overlapped else g.padded, st)
            shards.append(g.shard_slice(g.flat_grad))
        inv = opt.grad_scale()                      # mean over data-parallel replicas, sum over context-parallel ranks
        if opt.grad_divisor:
            inv = inv / opt.grad_divisor
        sq = self._sq * (inv * inv)
        dist.all_reduce(sq, group=opt.group)
        tp = state.get_model_parallel_world_size()
        if tp > 1:
            dist.all_reduce(sq, group=state.get_model_parallel_group())
        if state.get_pipe_parallel_world_size() > 1:
            dist.all_reduce(sq, group=state.get_pipe_parallel_group())
        norm = sq.sqrt()
        opt.last_grad_norm = norm
        if opt.clip_grad > 0.0:
            coef = (torch.clamp(opt.clip_grad / (norm + 1e-6), max=1.0) * inv).reshape(1).float()
        else:
            coef = torch.full((1,), inv, dtype=torch.float32, device=norm.device)
        b1, b2 = opt.betas
        bc1, bc2 = 1.0 - b1 ** opt.step_count, 1.0 - b2 ** opt.step_count
        for g, s in zip(opt.groups, shards):
            h = self.handles.get(id(g))
            if h is None:
                from .. import ops
                ops.adam_step(g.master, g.exp_avg, g.exp_avg_sq, s, g.hyper["lr"], b1, b2, opt.eps, g.hyper["weight_decay"],
                              opt.step_count, opt.adamw, coef, None if g.master_is_view else g.shard_slice(g.flat_param))
                opt._all_gather(g)
                continue
            pp, mcp = h[3], h[5]
            rc = self.lib.sb_zero_adam_allgather(g.master.data_ptr(), g.exp_avg.data_ptr(), g.exp_avg_sq.data_ptr(),
                                                 s.data_ptr(), pp, mcp if self.nvls else None, self.world, self.rank,
                                                 g.rank * g.shard, g.shard,
                                                 g.hyper["lr"], b1, b2, opt.eps, g.hyper["weight_decay"], bc1, bc2,
                                                 int(opt.adamw), coef.data_ptr(), st)
            if rc != 0:
                raise RuntimeError(f"zero_adam_allgather failed ({rc})")
            self.cuda_ops._count()
        self._barrier(opt.group)
        return norm


def make_allocator(group) -> Optional[SymmAllocator]:
    try:
        return SymmAllocator(group)
    except Exception as exc:  # noqa: BLE001
        print_rank_0(f"symmetric memory unavailable ({exc}); ZeRO uses the NCCL path")
        return None


def attach(opt, allocator: Optional[SymmAllocator], use_nvls: bool = True) -> bool:
    """Switch `opt.step` to the fused path.  Every rank must reach the same decision: the outcome of the
    rendezvous is agreed on with an all-reduce, and a failure anywhere keeps everyone on the NCCL path."""
    ok = 1
    fused = None
    if allocator is None or opt.world > 16 or not opt.partition:
        ok = 0
    else:
        try:
            fused = FusedZeroStep(opt, allocator, use_nvls)
        except Exception as exc:  # noqa: BLE001
            print(f"[rank {dist.get_rank()}] fused ZeRO set-up failed: {exc}", flush=True)
            ok = 0
    nv = 1 if (fused is not None and fused.nvls) else 0
    flag = torch.tensor([ok, nv], device=opt.groups[0].flat_param.device, dtype=torch.int32)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=opt.group)
    if int(flag[0].item()) == 1:
        fused.nvls = bool(int(flag[1].item()))           # multimem only if every rank has the multicast mapping
        opt.fused = fused
        print_rank_0(" > ZeRO-1 step: fused peer-memory kernels (reduce-scatter + Adam + all-gather)"
                     + (", NVLS multimem.ld_reduce / multimem.st" if fused.nvls else ", plain peer loads / stores"))
        return True
    print_rank_0(" > ZeRO-1 step: NCCL reduce-scatter / all-gather path")
    return False
