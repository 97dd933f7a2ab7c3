"""Operator front-end.

Every hot operator of the model goes through a function of this module.  A CUDA tensor runs the
hand-written sm_100a kernel (ops/cuda_ops.py over the in-tree extension `savanna_b200._C`); a CPU
tensor runs the fp32-capable PyTorch statement in ops/reference.py, which is also the oracle of the
kernel tests.  `set_backend("torch")` (or SAVANNA_B200_BACKEND=torch) forces the PyTorch statement
for CUDA tensors too: the comparison arm of tests and benchmarks, never the default.  There is no
silent fallback: a CUDA tensor without the built extension raises.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import reference as ref

_BACKEND = os.environ.get("SAVANNA_B200_BACKEND", "auto")
_LAUNCHES = 0


def set_backend(name: str) -> None:
    global _BACKEND
    if name not in ("auto", "torch"):
        raise ValueError("backend is 'auto' (kernels on CUDA tensors) or 'torch' (oracle everywhere)")
    _BACKEND = name


def get_backend() -> str:
    return _BACKEND


def kernel_launch_count() -> int:
    """Number of launches of this package's own kernels since import (counted at the call sites)."""
    from . import cuda_ops
    return cuda_ops.launch_count()


def _k(x: torch.Tensor) -> bool:
    if not x.is_cuda or _BACKEND == "torch":
        return False
    from . import cuda_ops  # raises with a clear message when the extension is not built
    cuda_ops.require()
    return True


def _co():
    from . import cuda_ops
    return cuda_ops


# ----------------------------------------------------------------------------- dense


def rmsnorm(x, weight, eps: float, form: str = "te"):
    return _co().rmsnorm(x, weight, eps, form) if _k(x) else ref.rmsnorm(x, weight, eps, form)


def norm_linear(x, norm_weight, eps: float, form: str, w, bias=None, fp8: bool = False):
    """(linear(rmsnorm(x)), x for the residual branch)."""
    if _k(x):
        return _co().norm_linear(x, norm_weight, eps, form, w, bias, fp8)
    return linear(ref.rmsnorm(x, norm_weight, eps, form), w, bias, fp8), x


def glu_linear(ab, act: str, w, bias=None, residual=None, fp8: bool = False):
    """linear(act(a) * b) (+ bias) (+ residual) for the packed gate input ab = [a | b]."""
    if _k(ab):
        return _co().glu_linear(ab, act, w, bias, residual, fp8)
    return linear(glu_act_packed(ab, act), w, bias, fp8, residual)


def mlp_gated(x, norm_weight, eps: float, form: str, w12, w3, b3=None, act: str = "silu", fp8: bool = False):
    """x + w3(act(a) * b) + b3 with [a | b] = w12(rmsnorm(x)) on one tensor-parallel rank."""
    if _k(x):
        return _co().mlp_gated(x, norm_weight, eps, form, w12, w3, b3, act, fp8)
    ab = linear(ref.rmsnorm(x, norm_weight, eps, form), w12, None, fp8)
    return linear(glu_act_packed(ab, act), w3, b3, fp8, x)


def rmsnorm_residual(x, weight, eps: float, form: str = "te"):
    """(rmsnorm(x), x): the second value is x as it continues down the residual branch.  On the kernel path the
    gradient that comes back along that branch is added inside the norm's backward kernel."""
    if _k(x):
        return _co().rmsnorm_residual(x, weight, eps, form)
    return ref.rmsnorm(x, weight, eps, form), x


def linear(x, w, bias=None, fp8: bool = False, residual=None):
    """x w^T (+ bias) (+ residual).  On CUDA bias and residual are added in the GEMM epilogue."""
    if _k(x):
        return _co().linear(x, w, bias, fp8, residual)
    y = ref.linear(x, w, bias)
    return y if residual is None else y + residual


def linear_allgather(x, w, bias=None, seq_dim: int = 1, fp8: bool = False):
    """Sequence-parallel column projection: all-gather x along `seq_dim` over the tensor-parallel group,
    then x w^T.  CUDA: one fused peer-memory kernel when the symmetric workspace is up."""
    if _k(x):
        y = _co().linear_allgather(x, w, bias, seq_dim, fp8)
        if y is not None:
            return y
    from ..parallel import mappings
    xg = mappings.gather_from_sequence_parallel_region(x, seq_dim, True)
    return linear(xg, w, bias, fp8)


def linear_reducescatter(x, w, seq_dim: int = 1, fp8: bool = False):
    """Sequence-parallel row projection: x w^T, partial sums reduce-scattered along `seq_dim`."""
    if _k(x):
        y = _co().linear_reducescatter(x, w, seq_dim, fp8)
        if y is not None:
            return y
    from ..parallel import mappings
    return mappings.reduce_scatter_to_sequence_parallel_region(linear(x, w, None, fp8), seq_dim)


def glu_act(a, b, act: str = "silu"):
    return _co().glu_act(a, b, act) if _k(a) else ref.glu_act(a, b, act)


def glu_act_packed(ab, act: str = "silu"):
    """ab [..., 2F] = [a | b] (w1 and w2 outputs side by side) -> act(a) * b."""
    if _k(ab):
        return _co().glu_act_packed(ab, act)
    a, b = ab.chunk(2, dim=-1)
    return ref.glu_act(a, b, act)


# ----------------------------------------------------------------------------- hyena


def causal_conv1d(x, w, halo=None):
    return _co().causal_conv1d(x, w, halo) if _k(x) else ref.causal_conv1d(x, w, halo)


def hyena_se_inner(feat, w, halo=None, pregate=True, postgate=True):
    if _k(feat):
        return _co().hyena_se_inner(feat, w, halo, pregate, postgate)
    return ref.hyena_se_inner(feat, w, halo, pregate, postgate)


def hyena_mr_inner(feat, h, bias, halo=None):
    return _co().hyena_mr_inner(feat, h, bias, halo) if _k(feat) else ref.hyena_mr_inner(feat, h, bias, halo)


def hyena_li_modal(feat, gamma, R, p, bias, state_in=None, return_state=False):
    if _k(feat):
        return _co().hyena_li_modal(feat, gamma, R, p, bias, state_in, return_state)
    return ref.hyena_li_modal(feat, gamma, R, p, bias, state_in, return_state)


def hyena_long_fft(feat, h, bias):
    # explicit long filters (non-modal filter classes) use the FFT statement on every device
    return ref.hyena_long_fft(feat, h, bias)


def hyena_long_fft_bidirectional(feat, h, bias):
    return ref.hyena_long_fft_bidirectional(feat, h, bias)


def hyena_multihead(feat, h, bias):
    return ref.hyena_multihead(feat, h, bias)


# ----------------------------------------------------------------------------- attention


def apply_rope(x, cos, sin):
    return _co().apply_rope(x, cos, sin) if _k(x) else ref.apply_rope(x, cos, sin)


def attention(q, k, v, causal=True, q_pos=None, k_pos=None, return_lse=False):
    if q.is_cuda:
        # CUDA tensors never materialise the score matrix: own flash kernel, or (backend "torch") PyTorch's
        from . import attention_cuda
        return attention_cuda.attention(q, k, v, causal, q_pos, k_pos, return_lse, own_kernels=_k(q))
    return ref.attention(q, k, v, causal, q_pos, k_pos, return_lse)


def attention_packed(qkv, cos, sin, causal=True):
    """Self-attention on the packed projection qkv [B, L, H, 3*hd] with rotary embedding of q and k (cos / sin [L, rd] or
    None).  Returns [B, L, H, hd], or None when the fused function does not cover the case (the caller then slices,
    rotates and calls `attention`)."""
    if not (qkv.is_cuda and _k(qkv)):
        return None
    from . import attention_cuda, flash_sm100
    if not attention_cuda._OWN or not flash_sm100.packed_supported(qkv):
        return None
    if cos is not None and (cos.shape[-1] % 16 or cos.shape[-1] > 128 or cos.shape[0] != qkv.shape[1]):
        return None
    return flash_sm100.attention_packed(qkv, cos, sin, causal)


# ----------------------------------------------------------------------------- loss / optimizer


def cross_entropy(logits, labels):
    return _co().cross_entropy(logits, labels) if _k(logits) else ref.cross_entropy(logits, labels)


def adam_step(master, exp_avg, exp_avg_sq, grad, lr, beta1, beta2, eps, weight_decay, step, adamw=True,
              grad_scale=1.0, param_out=None):
    if _k(master):
        return _co().adam_step(master, exp_avg, exp_avg_sq, grad, lr, beta1, beta2, eps, weight_decay, step, adamw,
                               grad_scale, param_out)
    return ref.adam_step(master, exp_avg, exp_avg_sq, grad, lr, beta1, beta2, eps, weight_decay, step, adamw,
                         grad_scale, param_out)


def sq_norm(x, weight=None):
    """Sum of squares in fp32 as a 0-dim tensor (optionally element-weighted), without a fp32 copy of x."""
    if _k(x):
        return _co().sq_norm(x, weight)
    xf = x.float()
    return (xf * xf * weight).sum() if weight is not None else (xf * xf).sum()
