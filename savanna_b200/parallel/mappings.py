"""Autograd-aware tensor/sequence-parallel communication ops.

Pairs (forward <-> backward), as in the reference (savanna/mpu/mappings.py:179-334):
  copy_to_model_parallel_region          identity      <-> all-reduce
  reduce_from_model_parallel_region      all-reduce    <-> identity
  scatter_to_model_parallel_region       split lastdim <-> all-gather lastdim
  gather_from_model_parallel_region      all-gather    <-> split lastdim
  reduce_scatter_to_sequence_parallel_region   reduce-scatter(seq) <-> all-gather(seq)
  gather_from_sequence_parallel_region         all-gather(seq)     <-> reduce-scatter(seq) | split
  scatter_to_sequence_parallel_region          split(seq)          <-> all-gather(seq)

These are the NCCL (or gloo) forms.  On B200 the all-gather->GEMM and GEMM->reduce-scatter pairs
around the projections are replaced by fused kernels (parallel/fused_tp.py); the ops here remain the
baseline and the CPU path.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import state


def _tp():
    return state.get_model_parallel_group(), state.get_model_parallel_world_size(), state.get_model_parallel_rank()


def _all_reduce(x: torch.Tensor) -> torch.Tensor:
    group, n, _ = _tp()
    if n == 1:
        return x
    if state.get_fp32_allreduce() and x.dtype != torch.float32:
        y = x.float()
        dist.all_reduce(y, group=group)
        return y.to(x.dtype)
    x = x.contiguous()
    dist.all_reduce(x, group=group)
    return x


def _split_last(x):
    _, n, r = _tp()
    if n == 1:
        return x
    return x.chunk(n, dim=-1)[r].contiguous()


def _gather_last(x):
    group, n, _ = _tp()
    if n == 1:
        return x
    parts = [torch.empty_like(x) for _ in range(n)]
    dist.all_gather(parts, x.contiguous(), group=group)
    return torch.cat(parts, dim=-1)


def _split_seq(x, seq_dim):
    _, n, r = _tp()
    if n == 1:
        return x
    if x.shape[seq_dim] % n:
        raise ValueError(f"sequence dim {x.shape[seq_dim]} not divisible by tensor-parallel size {n}")
    return x.chunk(n, dim=seq_dim)[r].contiguous()


def _gather_seq(x, seq_dim):
    group, n, _ = _tp()
    if n == 1:
        return x
    if seq_dim == 0:
        out = torch.empty((x.shape[0] * n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out
    parts = [torch.empty_like(x) for _ in range(n)]
    dist.all_gather(parts, x.contiguous(), group=group)
    return torch.cat(parts, dim=seq_dim)


def _reduce_scatter_seq(x, seq_dim):
    group, n, _ = _tp()
    if n == 1:
        return x
    orig = x.dtype
    if state.get_fp32_allreduce():
        x = x.float()
    if seq_dim != 0:
        x = x.transpose(0, seq_dim)
    x = x.contiguous()
    out = torch.empty((x.shape[0] // n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    if dist.get_backend(group) == "gloo":
        # gloo has no reduce_scatter_tensor: all-reduce and keep the own slice
        dist.all_reduce(x, group=group)
        out = x.chunk(n, dim=0)[state.get_model_parallel_rank()].contiguous()
    else:
        dist.reduce_scatter_tensor(out, x, group=group)
    if seq_dim != 0:
        out = out.transpose(0, seq_dim).contiguous()
    return out.to(orig)


class _Copy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return x

    @staticmethod
    def backward(ctx, g):
        return _all_reduce(g.clone())


class _Reduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return _all_reduce(x.clone())

    @staticmethod
    def backward(ctx, g):
        return g


class _Scatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return _split_last(x)

    @staticmethod
    def backward(ctx, g):
        return _gather_last(g)


class _Gather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return _gather_last(x)

    @staticmethod
    def backward(ctx, g):
        return _split_last(g)


class _ReduceScatterSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, seq_dim):
        ctx.seq_dim = seq_dim
        return _reduce_scatter_seq(x, seq_dim)

    @staticmethod
    def backward(ctx, g):
        return _gather_seq(g, ctx.seq_dim), None


class _GatherSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, seq_dim, reduce_scatter_grad):
        ctx.seq_dim, ctx.rs = seq_dim, reduce_scatter_grad
        return _gather_seq(x, seq_dim)

    @staticmethod
    def backward(ctx, g):
        if ctx.rs:
            return _reduce_scatter_seq(g, ctx.seq_dim), None, None
        return _split_seq(g, ctx.seq_dim), None, None


class _ScatterSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, seq_dim):
        ctx.seq_dim = seq_dim
        return _split_seq(x, seq_dim)

    @staticmethod
    def backward(ctx, g):
        return _gather_seq(g, ctx.seq_dim), None


def copy_to_model_parallel_region(x):
    return _Copy.apply(x)


def reduce_from_model_parallel_region(x):
    return _Reduce.apply(x)


def scatter_to_model_parallel_region(x):
    return _Scatter.apply(x)


def gather_from_model_parallel_region(x):
    return _Gather.apply(x)


def reduce_scatter_to_sequence_parallel_region(x, seq_dim: int = 1):
    return _ReduceScatterSeq.apply(x, seq_dim)


def gather_from_sequence_parallel_region(x, seq_dim: int = 1, reduce_scatter_grad: bool = True):
    return _GatherSeq.apply(x, seq_dim, reduce_scatter_grad)


def scatter_to_sequence_parallel_region(x, seq_dim: int = 1):
    return _ScatterSeq.apply(x, seq_dim)
