"""Context-parallel causal convolutions whose kernels read the neighbouring chunks' edge rows from peer memory.

Under zigzag sharding rank r holds chunks (r, 2cp-1-r) of every sequence back to back.  A causal FIR filter of K taps
needs the K-1 rows before each chunk in the forward pass, and its backward pass needs the K-1 rows of the upstream
gradient (times the post-gate, for the gated operators) that FOLLOW each chunk: with them the input gradient of the
chunk's last rows is complete on the rank that owns those rows, so no halo gradient has to travel back.

    forward    stage the two chunk tails [B, 2, K-1, W] in a symmetric buffer -> stream-ordered device barrier ->
               convolution kernel, whose tile loader fetches the rows before a chunk straight from the staging
               buffer of the rank that owns them (plain loads over NVLink)
    backward   stage tails of the input and heads of (input, upstream gradient) -> barrier -> backward kernel, whose
               loader fetches history rows and look-ahead rows from the neighbours the same way

No copy kernel runs between the barrier and the convolution, no halo tensor and no halo-gradient tensor exist, and the
input gradient is written once (the NCCL form, parallel/halo.py, sends halo gradients back and adds them to the tail
rows in a second pass).  Kernels: csrc/conv.cu (`sb_dwconv_*_cp`, `sb_se_*_cp`), csrc/mr_conv_tc.cu
(`sb_mr_tc_*_cp`); addressing of the staged edges: csrc/halo_src.cuh.  Reference algorithm replaced:
savanna/model/operators/hyena/p2p_cp_conv.py:50-164 (send/recv of the overlap region around a local convolution).

Every entry point returns None when this path does not apply (no peer workspace, non-bf16, a shape without a tiled
kernel); the caller then uses the halo-tensor path.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import halo as halo_mod

bf16 = torch.bfloat16
CALLS = 0                      # number of convolutions that went through this path (tests and bench read it)


class HaloSrc(ctypes.Structure):
    """Mirror of `sb::HaloSrc` (csrc/halo_src.cuh)."""
    _fields_ = [("p0", ctypes.c_void_p), ("p1", ctypes.c_void_p), ("slot0", ctypes.c_int), ("slot1", ctypes.c_int),
                ("chunked", ctypes.c_int)]


def before_src(ptrs, me: int, cp: int) -> HaloSrc:
    """Rows preceding each chunk, out of staged tails [B, 2, H, W]: chunk 0 <- rank-1's chunk-0 tail (none on rank 0);
    chunk 1 <- rank+1's chunk-1 tail, on the last rank its own chunk-0 tail."""
    p0 = ptrs[me - 1] if me > 0 else None
    if me + 1 < cp:
        p1, s1 = ptrs[me + 1], 1
    else:
        p1, s1 = ptrs[me], 0
    return HaloSrc(p0, p1, 0, s1, 1)


def ahead_src(ptrs, me: int, cp: int) -> HaloSrc:
    """Rows following each chunk, out of staged heads [B, 2, H, W]: chunk 0 <- rank+1's chunk-0 head, on the last rank
    its own chunk-1 head; chunk 1 <- rank-1's chunk-1 head (none on rank 0: the sequence ends there)."""
    if me + 1 < cp:
        p0, s0 = ptrs[me + 1], 0
    else:
        p0, s0 = ptrs[me], 1
    p1 = ptrs[me - 1] if me > 0 else None
    return HaloSrc(p0, p1, s0, 1, 1)


_BOUND = False


def _lib(ws):
    global _BOUND
    lib = ws.lib
    if not _BOUND:
        P, I = ctypes.c_void_p, ctypes.c_int
        H = ctypes.POINTER(HaloSrc)
        lib.sb_dwconv_fwd_cp.restype = I
        lib.sb_dwconv_fwd_cp.argtypes = [P, H, P, P, I, I, I, I, P]
        lib.sb_dwconv_bwd_cp.restype = I
        lib.sb_dwconv_bwd_cp.argtypes = [P, H, P, P, H, P, P, I, I, I, I, P]
        lib.sb_se_fwd_cp.restype = I
        lib.sb_se_fwd_cp.argtypes = [P, H, P, P, I, I, I, I, I, I, I, P]
        lib.sb_se_bwd_cp.restype = I
        lib.sb_se_bwd_cp.argtypes = [P, H, P, P, H, H, P, P, I, I, I, I, I, I, I, P]
        lib.sb_mr_tc_fwd_cp.restype = I
        lib.sb_mr_tc_fwd_cp.argtypes = [P, H, P, P, P, I, I, I, I, I, P]
        lib.sb_mr_tc_bwd_cp.restype = I
        lib.sb_mr_tc_bwd_cp.argtypes = [P, H, P, P, P, H, H, P, P, P, I, I, I, I, I, P]
        lib.sb_mr_tc_supported.restype = I
        lib.sb_mr_tc_supported.argtypes = [I, I, I]
        _BOUND = True
    return lib


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _stage(ws, name: str, x: torch.Tensor, H: int, heads: bool):
    """Copy the H first (heads) or last (tails) rows of both chunks of x [B, L, W] into the next slot of the symmetric
    buffer `name`; returns the peers' pointers to that slot."""
    B, L, W = x.shape
    half = L // 2
    stage, ptrs = ws.symm_buffer(name, B * 2 * H * W)
    sv = stage.view(B, 2, H, W)
    if heads:
        sv[:, 0].copy_(x[:, :H])
        sv[:, 1].copy_(x[:, half:half + H])
    else:
        sv[:, 0].copy_(x[:, half - H:half])
        sv[:, 1].copy_(x[:, L - H:])
    return ptrs


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed ({rc})")


def _f32c(t):
    return t.detach().float().contiguous()


def _usable(x: torch.Tensor, H: int) -> bool:
    ws = halo_mod._PEER_WS
    return (ws is not None and x.is_cuda and x.dtype == bf16 and x.dim() == 3 and x.shape[1] % 2 == 0
            and 0 < H <= x.shape[1] // 2)


class _DwConvCP(torch.autograd.Function):
    """Depthwise causal conv (the featuriser) on a zigzag shard x [B, L_local, C]; w [C, K]."""

    @staticmethod
    def forward(ctx, x, w):
        global CALLS
        ws = halo_mod._PEER_WS
        lib = _lib(ws)
        B, L, C = x.shape
        K = w.shape[-1]
        xc = x.contiguous()
        wf = _f32c(w)
        tails = _stage(ws, "cpconv_tail", xc, K - 1, heads=False)
        ws.barrier()
        y = torch.empty_like(xc)
        src = before_src(tails, ws.rank, ws.world)
        _check(lib.sb_dwconv_fwd_cp(xc.data_ptr(), ctypes.byref(src), wf.data_ptr(), y.data_ptr(), 2 * B, L // 2, C, K, _stream()),
               "dwconv_fwd_cp")
        ws.cuda_ops._count()
        CALLS += 1
        ctx.save_for_backward(xc, wf)
        ctx.wdtype = w.dtype
        return y

    @staticmethod
    def backward(ctx, gy):
        ws = halo_mod._PEER_WS
        lib = _lib(ws)
        xc, wf = ctx.saved_tensors
        B, L, C = xc.shape
        K = wf.shape[-1]
        g = gy.contiguous()
        tails = _stage(ws, "cpconv_tail", xc, K - 1, heads=False)
        heads = _stage(ws, "cpconv_head_g", g, K - 1, heads=True)
        ws.barrier()
        dx = torch.empty_like(xc)
        dw = torch.zeros_like(wf)
        before, ahead = before_src(tails, ws.rank, ws.world), ahead_src(heads, ws.rank, ws.world)
        _check(lib.sb_dwconv_bwd_cp(xc.data_ptr(), ctypes.byref(before), wf.data_ptr(), g.data_ptr(), ctypes.byref(ahead),
                                    dx.data_ptr(), dw.data_ptr(), 2 * B, L // 2, C, K, _stream()), "dwconv_bwd_cp")
        ws.cuda_ops._count()
        return dx, dw.to(ctx.wdtype)


class _HyenaSeCP(torch.autograd.Function):
    """Hyena-SE z = x1 * conv_K(x2 * v) on a zigzag shard feat [B, L_local, 3D]; w [G, K]."""

    @staticmethod
    def forward(ctx, feat, w, pregate, postgate):
        global CALLS
        ws = halo_mod._PEER_WS
        lib = _lib(ws)
        B, L, C3 = feat.shape
        D = C3 // 3
        G, K = w.shape
        fc = feat.contiguous()
        wf = _f32c(w)
        tails = _stage(ws, "cpconv_tail", fc, K - 1, heads=False)
        ws.barrier()
        z = torch.empty((B, L, D), dtype=bf16, device=feat.device)
        src = before_src(tails, ws.rank, ws.world)
        _check(lib.sb_se_fwd_cp(fc.data_ptr(), ctypes.byref(src), wf.data_ptr(), z.data_ptr(), 2 * B, L // 2, D, G, K,
                                int(pregate), int(postgate), _stream()), "se_fwd_cp")
        ws.cuda_ops._count()
        CALLS += 1
        ctx.save_for_backward(fc, wf)
        ctx.meta = (w.dtype, pregate, postgate)
        return z

    @staticmethod
    def backward(ctx, gz):
        ws = halo_mod._PEER_WS
        lib = _lib(ws)
        fc, wf = ctx.saved_tensors
        wdtype, pregate, postgate = ctx.meta
        B, L, C3 = fc.shape
        D = C3 // 3
        G, K = wf.shape
        g = gz.contiguous()
        tails = _stage(ws, "cpconv_tail", fc, K - 1, heads=False)
        heads_f = _stage(ws, "cpconv_head_f", fc, K - 1, heads=True)
        heads_g = _stage(ws, "cpconv_head_g", g, K - 1, heads=True)
        ws.barrier()
        df = torch.empty_like(fc)
        dw = torch.zeros_like(wf)
        me, cp = ws.rank, ws.world
        before, af, ag = before_src(tails, me, cp), ahead_src(heads_f, me, cp), ahead_src(heads_g, me, cp)
        _check(lib.sb_se_bwd_cp(fc.data_ptr(), ctypes.byref(before), wf.data_ptr(), g.data_ptr(), ctypes.byref(af),
                                ctypes.byref(ag), df.data_ptr(), dw.data_ptr(), 2 * B, L // 2, D, G, K, int(pregate),
                                int(postgate), _stream()), "se_bwd_cp")
        ws.cuda_ops._count()
        return df, dw.to(wdtype), None, None


class _HyenaMrCP(torch.autograd.Function):
    """Hyena-MR z = x1 * (h * (x2 v) + bias * (x2 v)) on a zigzag shard feat [B, L_local, 3D]; h [G, K]."""

    @staticmethod
    def forward(ctx, feat, h, bias):
        global CALLS
        ws = halo_mod._PEER_WS
        lib = _lib(ws)
        B, L, C3 = feat.shape
        D = C3 // 3
        G, K = h.shape
        fc = feat.contiguous()
        hf, bf = _f32c(h), _f32c(bias)
        tails = _stage(ws, "cpconv_tail", fc, K - 1, heads=False)
        ws.barrier()
        z = torch.empty((B, L, D), dtype=bf16, device=feat.device)
        src = before_src(tails, ws.rank, ws.world)
        _check(lib.sb_mr_tc_fwd_cp(fc.data_ptr(), ctypes.byref(src), hf.data_ptr(), bf.data_ptr(), z.data_ptr(), 2 * B, L // 2,
                                   D, G, K, _stream()), "mr_tc_fwd_cp")
        ws.cuda_ops._count()
        CALLS += 1
        ctx.save_for_backward(fc, hf, bf)
        ctx.meta = (h.dtype, bias.dtype)
        return z

    @staticmethod
    def backward(ctx, gz):
        ws = halo_mod._PEER_WS
        lib = _lib(ws)
        fc, hf, bf = ctx.saved_tensors
        hdtype, bdtype = ctx.meta
        B, L, C3 = fc.shape
        D = C3 // 3
        G, K = hf.shape
        g = gz.contiguous()
        tails = _stage(ws, "cpconv_tail", fc, K - 1, heads=False)
        heads_f = _stage(ws, "cpconv_head_f", fc, K - 1, heads=True)
        heads_g = _stage(ws, "cpconv_head_g", g, K - 1, heads=True)
        ws.barrier()
        df = torch.empty_like(fc)
        dh = torch.zeros_like(hf)
        db = torch.zeros_like(bf)
        me, cp = ws.rank, ws.world
        before, af, ag = before_src(tails, me, cp), ahead_src(heads_f, me, cp), ahead_src(heads_g, me, cp)
        _check(lib.sb_mr_tc_bwd_cp(fc.data_ptr(), ctypes.byref(before), hf.data_ptr(), bf.data_ptr(), g.data_ptr(),
                                   ctypes.byref(af), ctypes.byref(ag), df.data_ptr(), dh.data_ptr(), db.data_ptr(), 2 * B,
                                   L // 2, D, G, K, _stream()), "mr_tc_bwd_cp")
        ws.cuda_ops._count()
        return df, dh.to(hdtype), db.to(bdtype)


def causal_conv1d_cp(x: torch.Tensor, w: torch.Tensor) -> Optional[torch.Tensor]:
    """x [B, L_local, C] (two zigzag chunks), w [C, K] -> y, or None when the fused path does not apply."""
    K = w.shape[-1]
    if not _usable(x, K - 1) or not 2 <= K <= 8 or x.shape[-1] % 64:
        return None
    return _DwConvCP.apply(x, w)


def hyena_se_inner_cp(feat: torch.Tensor, w: torch.Tensor, pregate: bool = True, postgate: bool = True):
    G, K = w.shape
    D = feat.shape[-1] // 3
    if not _usable(feat, K - 1) or not 2 <= K <= 8 or D % 32 or D % G:
        return None
    return _HyenaSeCP.apply(feat, w, pregate, postgate)


def hyena_mr_inner_cp(feat: torch.Tensor, h: torch.Tensor, bias: torch.Tensor):
    G, K = h.shape
    D = feat.shape[-1] // 3
    if not _usable(feat, K - 1) or (feat.shape[1] // 2) % 64:
        return None
    if not _lib(halo_mod._PEER_WS).sb_mr_tc_supported(D, G, K):
        return None
    return _HyenaMrCP.apply(feat, h, bias)
