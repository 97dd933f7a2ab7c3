"""Causal attention on CUDA tensors.

q [B, Lq, H, hd], k/v [B, Lk, H, hd] (bf16).  Plain causal self-attention (Lq == Lk, positions in natural
order) is the training hot path.  Shards with explicit positions (context-parallel ring steps) are
expressed as (full | causal-diagonal | skip) block cases by the caller (parallel/ring_attention.py), so
this entry only needs `causal` in {True, False} plus the log-sum-exp output used to merge partial results.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from . import reference as ref


class _SdpaWithLse(torch.autograd.Function):
    """Attention that also returns the log-sum-exp, through the flash kernels shipped with PyTorch."""

    @staticmethod
    def forward(ctx, q, k, v, causal):
        scale = 1.0 / math.sqrt(q.shape[-1])
        qt, kt, vt = (t.transpose(1, 2) for t in (q, k, v))
        out, lse, cum_q, cum_k, max_q, max_k, seed, offset, _ = torch.ops.aten._scaled_dot_product_flash_attention(
            qt, kt, vt, 0.0, causal, False, scale=scale)
        ctx.save_for_backward(qt, kt, vt, out, lse, cum_q, cum_k, seed, offset)
        ctx.meta = (max_q, max_k, causal, scale)
        return out.transpose(1, 2), lse

    @staticmethod
    def backward(ctx, go, glse):
        qt, kt, vt, out, lse, cum_q, cum_k, seed, offset = ctx.saved_tensors
        max_q, max_k, causal, scale = ctx.meta
        gq, gk, gv = torch.ops.aten._scaled_dot_product_flash_attention_backward(
            go.transpose(1, 2), qt, kt, vt, out, lse, cum_q, cum_k, max_q, max_k, 0.0, causal, seed, offset, scale=scale)
        return gq.transpose(1, 2), gk.transpose(1, 2), gv.transpose(1, 2), None


_OWN = True


def set_own_kernels(on: bool) -> None:
    """Debug switch: False routes every call to the flash kernels shipped with PyTorch (the library baseline)."""
    global _OWN
    _OWN = bool(on)


_ALLOW_LIBRARY = False


def set_allow_library(on: bool) -> None:
    """Policy for shapes the tcgen05 kernels do not cover (head size other than 128, odd layouts): False (default)
    raises, True runs them on the flash kernels shipped with PyTorch (config key `allow_library_attention`)."""
    global _ALLOW_LIBRARY
    _ALLOW_LIBRARY = bool(on)


def attention(q, k, v, causal=True, q_pos=None, k_pos=None, return_lse=False, own_kernels=True):
    if q_pos is not None or k_pos is not None or q.dtype != torch.bfloat16:
        # explicit positions (partial blocks of the NCCL ring) and fp32 inputs: the fp32 statement of the operator
        return ref.attention(q, k, v, causal, q_pos, k_pos, return_lse)
    from . import flash_sm100
    if _OWN and own_kernels:
        if flash_sm100.supported(q, k, v, causal):
            return flash_sm100.attention(q, k, v, causal, return_lse)
        if not _ALLOW_LIBRARY:
            raise RuntimeError(
                f"attention shape q{tuple(q.shape)} k{tuple(k.shape)} (strides {q.stride()}) is not covered by the "
                "tcgen05 kernels (head size 128, bf16, unit inner stride); set `allow_library_attention: true` to run "
                "it on PyTorch's flash kernels instead")
    if return_lse:
        return _SdpaWithLse.apply(q, k, v, causal)
    o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=causal)
    return o.transpose(1, 2)
