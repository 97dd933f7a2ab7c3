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
from .cuda_ops import _alloc, _alloc_like, _zeros, _zeros_like

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
        lib.sb_attn_bwd.argtypes = [P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, P, P, P, P, P, P, P, P, P, I, F, P, P]
        lib.sb_attn_last_encode_result.restype = I
        lib.sb_attn_last_encode_result.argtypes = []
        lib.sb_attn_set_bwd_variant.restype = I
        lib.sb_attn_set_bwd_variant.argtypes = [I]
        lib.sb_attn_set_fwd_variant.restype = I
        lib.sb_attn_set_fwd_variant.argtypes = [I]
        lib.sb_attn_set_fwd_p_tmem.restype = I
        lib.sb_attn_set_fwd_p_tmem.argtypes = [I]
        lib.sb_attn_merge_fwd.restype = I
        lib.sb_attn_merge_fwd.argtypes = [P, P, P, P, I, I, I, I, P, P, P]
        lib.sb_attn_merge_bwd.restype = I
        lib.sb_attn_merge_bwd.argtypes = [P, P, P, P, I, I, I, I, P, P, P, P, P, P, P]
        _SIGS_SET = True
    return lib


def set_backward_variant(p_in_tmem: bool) -> None:
    """Backward kernel variant: P^T as the tensor-memory operand of the dV product with three Q/dO stages (default),
    or P^T through shared memory with two stages."""
    _lib().sb_attn_set_bwd_variant(int(bool(p_in_tmem)))


def set_forward_variant(pingpong: bool) -> None:
    """Forward kernel variant: the two softmax warpgroups of a CTA take turns on the exponentials (default), or run
    without coordination."""
    _lib().sb_attn_set_fwd_variant(int(bool(pingpong)))


def set_forward_p_in_tmem(on: bool) -> None:
    """Forward kernel variant: the probabilities as the tensor-memory operand of the P V product (packed bf16 over the
    score columns; default), or through shared memory."""
    _lib().sb_attn_set_fwd_p_tmem(int(bool(on)))


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
    out = _alloc((B, Lq, H, 128), dtype=torch.bfloat16, device=q.device)
    lse = _alloc((B, H, Lq), dtype=torch.float32, device=q.device)
    rc = lib.sb_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), B, H, Lq, Lk,
                         _str3(q), _str3(k), _str3(v), _str3(out), int(causal), float(scale),
                         cuda_ops.status_word(q.device).data_ptr(), cuda_ops._stream())
    if rc != 0:
        raise RuntimeError(f"attention forward failed (code {rc}, encode {lib.sb_attn_last_encode_result()}): "
                           f"q{tuple(q.shape)}{q.stride()} k{tuple(k.shape)}{k.stride()}")
    cuda_ops._count()
    return out, lse


def backward(go, q, k, v, out, lse, causal: bool, scale: float, glse=None, dq_acc=None, dk=None, dv=None, dq=None):
    """Gradients (dq, dk, dv) in bf16.  `glse` [B, H, Lq] is the gradient that arrived at the log-sum-exp output (the
    merge step of ring attention differentiates through it); it enters as a shift of the row term delta.
    With `dq_acc` (fp32, contiguous [B, Lq, H, 128]) the query gradient is ADDED into that accumulator and no bf16 dq is
    produced (returned as None): several calls over different key blocks share one accumulator.  `dq` / `dk` / `dv`
    may be given as bf16 destinations [B, L, H, 128] with a unit inner stride and the other strides multiples of 8
    elements (slices of a packed gradient buffer)."""
    lib = _lib()
    B, Lq, H, _ = q.shape
    Lk = k.shape[1]
    go = go if _ok_layout(go) else go.contiguous()
    shared = dq_acc is not None
    if not shared:
        dq_acc = _zeros((B, Lq, H, 128), dtype=torch.float32, device=q.device)
    stats = _alloc(2 * B * H * ((Lq + 63) // 64 * 64), dtype=torch.float32, device=q.device)
    if shared:
        dq = None
    elif dq is None:
        dq = _alloc((B, Lq, H, 128), dtype=torch.bfloat16, device=q.device)
    for t in (dq, dk, dv):
        if t is not None and not _ok_layout(t):
            raise ValueError(f"attention backward: destination layout {tuple(t.shape)} {t.stride()} is not supported")
    if dk is None:
        dk = _alloc((B, Lk, H, 128), dtype=torch.bfloat16, device=q.device)
    if dv is None:
        dv = _alloc((B, Lk, H, 128), dtype=torch.bfloat16, device=q.device)
    if glse is not None:
        glse = glse.contiguous().float()
    rc = lib.sb_attn_bwd(go.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(),
                         cuda_ops._ptr(glse), stats.data_ptr(), dq_acc.data_ptr(), cuda_ops._ptr(dq), dk.data_ptr(),
                         B, H, Lq, Lk, dv.data_ptr(), _str3(go), _str3(q), _str3(k), _str3(v), _str3(out),
                         _str3(dq if dq is not None else out), _str3(dk), _str3(dv), int(causal), float(scale),
                         cuda_ops.status_word(q.device).data_ptr(), cuda_ops._stream())
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
            go = _zeros_like(out)
        dq, dk, dv = backward(go, q, k, v, out, lse, ctx.causal, ctx.scale, glse)
        return dq, dk, dv, None


class _FlashPacked(torch.autograd.Function):
    """Attention on the packed projection qkv [B, L, H, 3*128] (per head: q, k, v) with rotary embedding of q and k inside
    the function.  The backward writes dq, dk, dv straight into one packed gradient buffer: the slice / concatenate
    bookkeeping of autograd (a zero fill, a strided copy and an add per slice) does not run."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, causal):
        B, L, H, _ = qkv.shape
        q, k, v = qkv[..., :128], qkv[..., 128:256], qkv[..., 256:]
        if cos is not None:
            q = cuda_ops._rope_launch(q, cos, sin, 0)
            k = cuda_ops._rope_launch(k, cos, sin, 0)
        scale = 1.0 / math.sqrt(128)
        out, lse = forward(q, k, v, causal, scale)
        ctx.save_for_backward(qkv, q if cos is not None else None, k if cos is not None else None, out, lse, cos, sin)
        ctx.causal, ctx.scale = causal, scale
        return out

    @staticmethod
    def backward(ctx, go):
        qkv, q, k, out, lse, cos, sin = ctx.saved_tensors
        rot = cos is not None
        if not rot:
            q, k = qkv[..., :128], qkv[..., 128:256]
        v = qkv[..., 256:]
        dqkv = _alloc(tuple(qkv.shape), dtype=torch.bfloat16, device=qkv.device)
        dq_dst, dk_dst, dv_dst = dqkv[..., :128], dqkv[..., 128:256], dqkv[..., 256:]
        if rot:
            dq, dk, _ = backward(go, q, k, v, out, lse, ctx.causal, ctx.scale, dv=dv_dst)
            cuda_ops._rope_launch(dq, cos, sin, 1, out=dq_dst)
            cuda_ops._rope_launch(dk, cos, sin, 1, out=dk_dst)
        else:
            backward(go, q, k, v, out, lse, ctx.causal, ctx.scale, dq=dq_dst, dk=dk_dst, dv=dv_dst)
        return dqkv, None, None, None


def packed_supported(qkv) -> bool:
    return (qkv.dim() == 4 and qkv.dtype == torch.bfloat16 and qkv.is_cuda and qkv.shape[-1] == 384 and qkv.is_contiguous()
            and qkv.data_ptr() % 16 == 0)


def attention_packed(qkv, cos, sin, causal):
    """qkv [B, L, H, 384] bf16 contiguous; cos / sin [L, rd] fp32 (or None for no rotary embedding) -> [B, L, H, 128]."""
    if cos is not None:
        cos, sin = cos.float().contiguous(), sin.float().contiguous()
    return _FlashPacked.apply(qkv, cos, sin, causal)


def attention(q, k, v, causal, return_lse=False):
    out, lse = _Flash.apply(q, k, v, causal)
    if return_lse:
        return out, lse
    return out


# ------------------------------------------------------------------------------------------ merging partial results
MERGE_MAX = 16


def _merge_args(os_, lses):
    S = len(os_)
    optr = (ctypes.c_void_p * S)(*[t.data_ptr() for t in os_])
    lptr = (ctypes.c_void_p * S)(*[t.data_ptr() for t in lses])
    ostr = (ctypes.c_longlong * (3 * S))(*[v for t in os_ for v in (t.stride(0), t.stride(1), t.stride(2))])
    lstr = (ctypes.c_longlong * (3 * S))(*[v for t in lses for v in (t.stride(0), t.stride(1), t.stride(2))])
    return optr, lptr, ostr, lstr


def merge_supported(os_, lses) -> bool:
    if not (1 <= len(os_) <= MERGE_MAX and len(os_) == len(lses)):
        return False
    shp = os_[0].shape
    for o, l in zip(os_, lses):
        if not (o.is_cuda and o.dtype == torch.bfloat16 and o.dim() == 4 and o.shape == shp and o.shape[-1] == 128
                and o.stride(-1) == 1 and all(st % 4 == 0 for st in o.stride()[:3]) and o.data_ptr() % 8 == 0):
            return False
        if not (l.dtype == torch.float32 and l.shape == (shp[0], shp[2], shp[1])):
            return False
    return True


def merge_forward(os_, lses):
    """The merge without autograd: (o [B, L, H, 128] bf16, lse [B, H, L] fp32)."""
    lib = _lib()
    S = len(os_)
    B, L, H, _ = os_[0].shape
    out = _alloc((B, L, H, 128), dtype=torch.bfloat16, device=os_[0].device)
    lse = _alloc((B, H, L), dtype=torch.float32, device=os_[0].device)
    optr, lptr, ostr, lstr = _merge_args(os_, lses)
    rc = lib.sb_attn_merge_fwd(optr, lptr, ostr, lstr, S, B, L, H, out.data_ptr(), lse.data_ptr(), cuda_ops._stream())
    if rc != 0:
        raise RuntimeError(f"attention merge failed ({rc})")
    cuda_ops._count()
    return out, lse


class _Merge(torch.autograd.Function):
    """Combine partial attention results over disjoint key sets: o = sum_s exp(lse_s - lse) o_s, lse = logsumexp_s lse_s
    (one kernel forward, one backward; csrc/attn_sm100.cu)."""

    @staticmethod
    def forward(ctx, S, *ts):
        os_, lses = ts[:S], ts[S:]
        lib = _lib()
        B, L, H, _ = os_[0].shape
        out = _alloc((B, L, H, 128), dtype=torch.bfloat16, device=os_[0].device)
        lse = _alloc((B, H, L), dtype=torch.float32, device=os_[0].device)
        optr, lptr, ostr, lstr = _merge_args(os_, lses)
        rc = lib.sb_attn_merge_fwd(optr, lptr, ostr, lstr, S, B, L, H, out.data_ptr(), lse.data_ptr(), cuda_ops._stream())
        if rc != 0:
            raise RuntimeError(f"attention merge failed ({rc})")
        cuda_ops._count()
        ctx.save_for_backward(out, lse, *ts)
        ctx.S = S
        ctx.mark_non_differentiable(lse)
        return out, lse

    @staticmethod
    def backward(ctx, gout, _glse):
        S = ctx.S
        saved = ctx.saved_tensors              # one access only (activation checkpointing unpacks on access)
        out, lse = saved[:2]
        ts = saved[2:]
        os_, lses = ts[:S], ts[S:]
        lib = _lib()
        B, L, H, _ = out.shape
        if gout.stride(-1) != 1 or any(st % 4 for st in gout.stride()[:3]) or gout.data_ptr() % 8:
            gout = gout.contiguous()
        gos = [_alloc((B, L, H, 128), dtype=torch.bfloat16, device=out.device) for _ in range(S)]
        gls = [_alloc((B, H, L), dtype=torch.float32, device=out.device) for _ in range(S)]
        optr, lptr, ostr, lstr = _merge_args(os_, lses)
        gstr = _LL3(gout.stride(0), gout.stride(1), gout.stride(2))
        goptr = (ctypes.c_void_p * S)(*[t.data_ptr() for t in gos])
        glptr = (ctypes.c_void_p * S)(*[t.data_ptr() for t in gls])
        rc = lib.sb_attn_merge_bwd(optr, lptr, ostr, lstr, S, B, L, H, out.data_ptr(), lse.data_ptr(), gout.data_ptr(), gstr,
                                   goptr, glptr, cuda_ops._stream())
        if rc != 0:
            raise RuntimeError(f"attention merge backward failed ({rc})")
        cuda_ops._count()
        return (None, *gos, *gls)


def merge_partials(os_, lses):
    """os_: list of [B, L, H, 128] bf16 partial outputs (views allowed), lses: list of [B, H, L] fp32 -> (o, lse)."""
    return _Merge.apply(len(os_), *os_, *lses)
