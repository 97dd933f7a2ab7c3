"""tcgen05 flash attention front-end (kernels: csrc/attn_sm100.cu).

q [B, Lq, H, 128], k/v [B, Lk, H, 128] in bf16 with a contiguous head dimension; the other strides are free (multiples
of 8 elements), so slices of a fused QKV projection are consumed in place.  `causal` means row i attends keys 0..i
and needs Lq == Lk; the non-causal form takes any Lq, Lk (the off-diagonal steps of ring attention).  The log-sum-exp
output [B, H, Lq] lets partial results be merged.  Covers the role of the reference's FlashAttention-2 calls
(savanna/model/operators/attention/flash.py:462-597).
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import cuda_ops

_SIGS_SET = False
_LL3 = ctypes.c_longlong * 3


def _lib():
    global _SIGS_SET
    lib = cuda_ops.require()
    if not _SIGS_SET:
        P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        lib.sb_attn_fwd.restype = I
        lib.sb_attn_fwd.argtypes = [P, P, P, P, P, I, I, I, I, P, P, P, P, I, F, P, P]
        lib.sb_attn_bwd.restype = I
        lib.sb_attn_bwd.argtypes = [P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, P, P, P, P, P, P, P, I, F, P, P]
        lib.sb_attn_last_encode_result.restype = I
        lib.sb_attn_last_encode_result.argtypes = []
        lib.sb_attn_set_bwd_variant.restype = I
        lib.sb_attn_set_bwd_variant.argtypes = [I]
        _SIGS_SET = True
    return lib


def set_backward_variant(p_in_tmem: bool) -> None:
    """Backward kernel variant: P^T as the tensor-memory operand of the dV product with three Q/dO stages (default),
    or P^T through shared memory with two stages."""
    _lib().sb_attn_set_bwd_variant(int(bool(p_in_tmem)))


def _ok_layout(t) -> bool:
    return (t.dim() == 4 and t.dtype == torch.bfloat16 and t.is_cuda and t.shape[-1] == 128 and t.stride(-1) == 1
            and all(s % 8 == 0 for s in t.stride()[:3]) and t.data_ptr() % 16 == 0)


def supported(q, k, v, causal) -> bool:
    if not (_ok_layout(q) and _ok_layout(k) and _ok_layout(v)):
        return False
    if q.shape[0] != k.shape[0] or q.shape[2] != k.shape[2] or k.shape != v.shape:
        return False
    return (not causal) or q.shape[1] == k.shape[1]


def _str3(t):
    return _LL3(t.stride(0), t.stride(1), t.stride(2))


def forward(q, k, v, causal: bool, scale: float):
    """Returns (out [B, Lq, H, 128] bf16, lse [B, H, Lq] fp32)."""
    lib = _lib()
    B, Lq, H, _ = q.shape
    Lk = k.shape[1]
    out = torch.empty((B, Lq, H, 128), dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((B, H, Lq), dtype=torch.float32, device=q.device)
    rc = lib.sb_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), B, H, Lq, Lk,
                         _str3(q), _str3(k), _str3(v), _str3(out), int(causal), float(scale),
                         cuda_ops.status_word(q.device).data_ptr(), cuda_ops._stream())
    if rc != 0:
        raise RuntimeError(f"attention forward failed (code {rc}, encode {lib.sb_attn_last_encode_result()}): "
                           f"q{tuple(q.shape)}{q.stride()} k{tuple(k.shape)}{k.stride()}")
    cuda_ops._count()
    return out, lse


def backward(go, q, k, v, out, lse, causal: bool, scale: float, glse=None):
    """Gradients (dq, dk, dv) in bf16.  `glse` [B, H, Lq] is the gradient that arrived at the log-sum-exp output (the
    merge step of ring attention differentiates through it); it enters as a shift of the row term delta."""
    lib = _lib()
    B, Lq, H, _ = q.shape
    Lk = k.shape[1]
    go = go if _ok_layout(go) else go.contiguous()
    dq_acc = torch.zeros((B, Lq, H, 128), dtype=torch.float32, device=q.device)
    stats = torch.empty(2 * B * H * ((Lq + 63) // 64 * 64), dtype=torch.float32, device=q.device)
    dq = torch.empty((B, Lq, H, 128), dtype=torch.bfloat16, device=q.device)
    dk = torch.empty((B, Lk, H, 128), dtype=torch.bfloat16, device=q.device)
    dv = torch.empty((B, Lk, H, 128), dtype=torch.bfloat16, device=q.device)
    if glse is not None:
        glse = glse.contiguous().float()
    rc = lib.sb_attn_bwd(go.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(),
                         cuda_ops._ptr(glse), stats.data_ptr(), dq_acc.data_ptr(), dq.data_ptr(), dk.data_ptr(),
                         B, H, Lq, Lk, dv.data_ptr(), _str3(go), _str3(q), _str3(k), _str3(v), _str3(out),
                         _str3(dq), int(causal), float(scale), cuda_ops.status_word(q.device).data_ptr(),
                         cuda_ops._stream())
    if rc != 0:
        raise RuntimeError(f"attention backward failed (code {rc}, encode {lib.sb_attn_last_encode_result()})")
    cuda_ops._count(3)
    return dq, dk, dv


class _Flash(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal):
        scale = 1.0 / math.sqrt(q.shape[-1])
        out, lse = forward(q, k, v, causal, scale)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.causal, ctx.scale = causal, scale
        ctx.set_materialize_grads(False)
        return out, lse

    @staticmethod
    def backward(ctx, go, glse):
        q, k, v, out, lse = ctx.saved_tensors
        if go is None:
            go = torch.zeros_like(out)
        dq, dk, dv = backward(go, q, k, v, out, lse, ctx.causal, ctx.scale, glse)
        return dq, dk, dv, None


def attention(q, k, v, causal, return_lse=False):
    out, lse = _Flash.apply(q, k, v, causal)
    if return_lse:
        return out, lse
    return out
