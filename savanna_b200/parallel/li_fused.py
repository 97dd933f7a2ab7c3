"""Context-parallel Hyena-LI whose scan kernels perform the all-to-all themselves.

The long (sequence-length) modal filter needs the whole sequence per channel, so the ranks switch from the
sequence-sharded layout [B, l, D] (zigzag shard) to a channel-sharded one [B, l*cp, D/cp] and back.  The reference does
this with two NCCL all-to-alls around an FFT convolution (savanna/model/operators/hyena/distributed_a2a.py:45-168,
hyena.py:451-467) and ships the three feature streams (x1, x2, v) in and z out.  Here

    forward    u = x2 v written into a symmetric staging buffer            (local gate kernel)
               barrier
               scan pass 1 reads this rank's channel block of every chunk straight from its owner's staging buffer
               (peer loads, zigzag addressing in the kernel) and keeps a local copy; scan pass 2 stores y straight
               into the owner's staging buffer (peer stores)
               barrier
               z = x1 y                                                    (local gate kernel, ordinary output tensor)
    backward   dy = dz x1 staged -> barrier -> the backward scans read dy from the owners, recompute y, and store y and
               du into the owners' staging buffers -> barrier -> (dz y, du v, du x2) locally

so only the pre-gated signal and the un-gated result cross NVLink (one third of the forward bytes of the reference
scheme), no tensor is permuted or copied by a kernel of its own, and the local copy of u is what the backward keeps.
Kernels: csrc/li_scan.cu (`sb_li_cp_*`).  Returns None when the path does not apply (the caller then uses the
all-to-all module, parallel/a2a.py).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import halo as halo_mod

bf16 = torch.bfloat16
LO = 16
CALLS = 0


class LiCpMap(ctypes.Structure):
    """Mirror of `sb::LiCpMap` (csrc/li_scan.cu)."""
    _fields_ = [("base", ctypes.c_void_p * 32), ("batch_stride", ctypes.c_longlong), ("row_stride", ctypes.c_int),
                ("chunk_len", ctypes.c_int), ("n_chunks", ctypes.c_int)]


def make_map(ptrs, me: int, cp: int, l: int, Dtot: int) -> LiCpMap:
    """Addresses of natural chunk j = 0..2cp-1 inside the ranks' staging buffers [B, l, Dtot] (bf16), offset to the
    channel block of rank `me`: chunk j lives on rank j (as its first chunk) for j < cp, else on rank 2cp-1-j (second)."""
    c, d = l // 2, Dtot // cp
    m = LiCpMap()
    for j in range(2 * cp):
        owner, loc = (j, 0) if j < cp else (2 * cp - 1 - j, c)
        m.base[j] = int(ptrs[owner]) + 2 * (loc * Dtot + me * d)
    m.batch_stride, m.row_stride, m.chunk_len, m.n_chunks = l * Dtot, Dtot, c, 2 * cp
    return m


_BOUND = False


def _lib(ws):
    global _BOUND
    lib = ws.lib
    if not _BOUND:
        P, I, LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        M = ctypes.POINTER(LiCpMap)
        lib.sb_li_cp_gate.restype = I
        lib.sb_li_cp_gate.argtypes = [P, P, P, LL, I, I, P]
        lib.sb_li_cp_finalize_bwd.restype = I
        lib.sb_li_cp_finalize_bwd.argtypes = [P, P, P, P, P, LL, I, P]
        lib.sb_li_cp_fwd.restype = I
        lib.sb_li_cp_fwd.argtypes = [M, M, P, P, P, P, P, I, I, I, I, P]
        lib.sb_li_cp_bwd.restype = I
        lib.sb_li_cp_bwd.argtypes = [M, M, M, P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, P]
        _BOUND = True
    return lib


def scan_chunk(c: int, B: int, d: int, L: int) -> int:
    """Scan chunk length: the largest power of two <= 1024 that divides the natural chunk length c (so a scan chunk
    has one owner) while the chunk grid still oversubscribes the GPU."""
    tc = 1024
    while tc > 64 and (c % tc or B * ((d + 127) // 128) * (L // tc) < 2048):
        tc //= 2
    return tc if c % tc == 0 else 0


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _check(rc, what):
    if rc != 0:
        raise RuntimeError(f"{what} failed ({rc})")


def _pad_order(t, fill):
    D, O = t.shape
    if O == LO:
        return t.contiguous()
    out = torch.full((D, LO), fill, dtype=torch.float32, device=t.device)
    out[:, :O] = t
    return out


class _HyenaLiCP(torch.autograd.Function):
    """feat [B, l, 3D] zigzag shard; gamma, R, p [d, O] and bias [d] are this rank's channel block of the filter."""

    @staticmethod
    def forward(ctx, feat, gamma, R, p, bias):
        global CALLS
        ws = halo_mod._PEER_WS
        lib = _lib(ws)
        me, cp = ws.rank, ws.world
        B, l, C3 = feat.shape
        D = C3 // 3
        d, L = D // cp, l * cp
        O = gamma.shape[1]
        fc = feat.contiguous()
        dev = feat.device
        loglam = -torch.exp(p.detach().float()) * torch.exp(gamma.detach().float())
        ll = _pad_order(loglam, -1.0e30)
        Rp = _pad_order(R.detach().float(), 0.0)
        bfv = bias.detach().float().contiguous()
        tc = scan_chunk(l // 2, B, d, L)
        NC = L // tc
        # u = x2 v into this rank's staging buffer
        ustage, uptrs = ws.symm_buffer("li_u", B * l * D)
        _check(lib.sb_li_cp_gate(fc.data_ptr(), None, ustage.data_ptr(), B * l, D, 0, _stream()), "li_cp_gate(u)")
        ystage, yptrs = ws.symm_buffer("li_y", B * l * D)
        ws.barrier()
        S = torch.empty((B, NC, d, LO), dtype=torch.float32, device=dev)
        ufull = torch.empty((B, L, d), dtype=bf16, device=dev)
        umap, ymap = make_map(uptrs, me, cp, l, D), make_map(yptrs, me, cp, l, D)
        _check(lib.sb_li_cp_fwd(ctypes.byref(umap), ctypes.byref(ymap), ll.data_ptr(), Rp.data_ptr(), bfv.data_ptr(),
                                S.data_ptr(), ufull.data_ptr(), B, L, d, tc, _stream()), "li_cp_fwd")
        ws.barrier()
        z = torch.empty((B, l, D), dtype=bf16, device=dev)
        _check(lib.sb_li_cp_gate(fc.data_ptr(), ystage.data_ptr(), z.data_ptr(), B * l, D, 1, _stream()), "li_cp_gate(z)")
        ws.cuda_ops._count(5)
        CALLS += 1
        ctx.save_for_backward(fc, ufull, ll, Rp, bfv)
        ctx.meta = (O, tc, gamma.dtype, R.dtype, p.dtype, bias.dtype)
        return z

    @staticmethod
    def backward(ctx, gz):
        ws = halo_mod._PEER_WS
        lib = _lib(ws)
        me, cp = ws.rank, ws.world
        fc, ufull, ll, Rp, bfv = ctx.saved_tensors
        O, tc, gdt, rdt, pdt, bdt = ctx.meta
        B, l, C3 = fc.shape
        D = C3 // 3
        d, L = D // cp, l * cp
        NC = L // tc
        dev = fc.device
        g = gz.contiguous()
        gstage, gptrs = ws.symm_buffer("li_dy", B * l * D)
        _check(lib.sb_li_cp_gate(fc.data_ptr(), g.data_ptr(), gstage.data_ptr(), B * l, D, 1, _stream()), "li_cp_gate(dy)")
        ystage, yptrs = ws.symm_buffer("li_y", B * l * D)
        dustage, duptrs = ws.symm_buffer("li_du", B * l * D)
        ws.barrier()
        shape = (B, NC, d, LO)
        S, W, A, dRp, dLp = (torch.empty(shape, dtype=torch.float32, device=dev) for _ in range(5))
        dBp = torch.empty((B, NC, d), dtype=torch.float32, device=dev)
        dyfull = torch.empty((B, L, d), dtype=bf16, device=dev)
        gmap, ymap, dumap = (make_map(x, me, cp, l, D) for x in (gptrs, yptrs, duptrs))
        _check(lib.sb_li_cp_bwd(ctypes.byref(gmap), ctypes.byref(ymap), ctypes.byref(dumap), ufull.data_ptr(), dyfull.data_ptr(),
                                ll.data_ptr(), Rp.data_ptr(), bfv.data_ptr(), S.data_ptr(), W.data_ptr(), A.data_ptr(),
                                dRp.data_ptr(), dLp.data_ptr(), dBp.data_ptr(), B, L, d, tc, _stream()), "li_cp_bwd")
        ws.barrier()
        df = torch.empty_like(fc)
        _check(lib.sb_li_cp_finalize_bwd(fc.data_ptr(), g.data_ptr(), ystage.data_ptr(), dustage.data_ptr(), df.data_ptr(),
                                         B * l, D, _stream()), "li_cp_finalize_bwd")
        ws.cuda_ops._count(6)
        dR = dRp.sum((0, 1))[:, :O]
        dlam = dLp.sum((0, 1))
        lam = torch.exp(ll)
        dll = (dlam * lam * ll)[:, :O]          # d/dp = d/dgamma = dloglam * loglam
        dll = torch.nan_to_num(dll, nan=0.0, posinf=0.0, neginf=0.0)
        db = dBp.sum((0, 1))
        return df, dll.to(gdt), dR.to(rdt), dll.to(pdt), db.to(bdt)


def hyena_li_modal_cp(feat: torch.Tensor, gamma, R, p, bias) -> Optional[torch.Tensor]:
    """feat [B, l, 3D] (zigzag shard, all channels); gamma / R / p [D/cp, O] and bias [D/cp]: the filter parameters of
    this rank's channel block.  Returns z [B, l, D], or None when the fused path does not apply."""
    ws = halo_mod._PEER_WS
    if ws is None or not feat.is_cuda or feat.dtype != bf16 or feat.dim() != 3:
        return None
    cp = ws.world
    B, l, C3 = feat.shape
    D = C3 // 3
    if C3 % 3 or D % (8 * cp) or l % 2 or 2 * cp > 32 or gamma.shape[1] > LO or gamma.shape[0] != D // cp:
        return None
    if scan_chunk(l // 2, B, D // cp, l * cp) == 0:
        return None
    return _HyenaLiCP.apply(feat, gamma, R, p, bias)
