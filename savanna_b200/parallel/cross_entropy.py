"""Vocabulary-parallel cross-entropy (reference: savanna/mpu/cross_entropy.py:8-94): the logits'
last dim is sharded over the tensor-parallel group; three small all-reduces (max, target logit,
sum-exp) produce the per-token loss; backward is softmax minus one-hot, computed locally."""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import state


class _VocabParallelCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, target):
        group = state.get_model_parallel_group()
        tp, rank = state.get_model_parallel_world_size(), state.get_model_parallel_rank()
        x = logits.float()
        m = x.max(dim=-1)[0]
        if tp > 1:
            dist.all_reduce(m, op=dist.ReduceOp.MAX, group=group)
        x = x - m.unsqueeze(-1)
        per = x.shape[-1]
        lo = rank * per
        mask = (target < lo) | (target >= lo + per)
        local_t = (target - lo).masked_fill(mask, 0)
        tl = x.gather(-1, local_t.unsqueeze(-1)).squeeze(-1).masked_fill(mask, 0.0)
        ex = x.exp()
        se = ex.sum(-1)
        if tp > 1:
            dist.all_reduce(tl, group=group)
            dist.all_reduce(se, group=group)
        loss = se.log() - tl
        ctx.save_for_backward(ex / se.unsqueeze(-1), mask, local_t)
        ctx.in_dtype = logits.dtype
        return loss

    @staticmethod
    def backward(ctx, g):
        sm, mask, local_t = ctx.saved_tensors
        grad = sm.clone()
        upd = (~mask).to(grad.dtype)
        grad.scatter_add_(-1, local_t.unsqueeze(-1), -upd.unsqueeze(-1))
        grad.mul_(g.unsqueeze(-1))
        return grad.to(ctx.in_dtype), None


def vocab_parallel_cross_entropy(logits: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
    return _VocabParallelCE.apply(logits, target)
