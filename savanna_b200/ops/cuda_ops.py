"""CUDA operator implementations: autograd Functions over the in-tree sm_100a library.

The library (`savanna_b200/libsavanna_b200.so`, built by `python -m savanna_b200.csrc.build`) exposes C
symbols; they are called through ctypes with raw device pointers and the current CUDA stream, so the
kernels run in PyTorch's stream order and under its caching allocator.  All kernels take bf16
activations and accumulate in fp32.  Tensors of another dtype run the PyTorch statement of the op
(reference.py) — a debugging configuration, not a performance path.

`launch_count()` counts launches of this library's kernels (incremented at every call site by the
number of kernels the C entry point launches).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import reference as ref

_LIB = None
_LIB_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "libsavanna_b200.so")
_LAUNCHES = 0
_STATUS = {}

_ACT = {"silu": 0, "swish": 0, "gelu": 1, "relu": 2, "identity": 3}
bf16 = torch.bfloat16

c_void_p, c_int, c_float, c_ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong


def require():
    """Load the native library; raise if it is missing (never fall back silently on a GPU)."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if not os.path.exists(_LIB_PATH):
        raise RuntimeError(
            f"{_LIB_PATH} is missing: build the CUDA kernels with `python -m savanna_b200.csrc.build` "
            "(CUDA tensors never fall back to PyTorch ops silently; set SAVANNA_B200_BACKEND=torch to ask for that)")
    raw = ctypes.CDLL(_LIB_PATH)
    for name in dir(_Sig):
        if name.startswith("sb_"):
            fn = getattr(raw, name)
            fn.restype = c_int
            fn.argtypes = getattr(_Sig, name)
    _LIB = _Library(raw)
    return _LIB


NVTX = False        # one NVTX range per native entry point (named after it) while True; the capture-range profiler turns it on


def set_nvtx(on: bool) -> None:
    global NVTX
    NVTX = bool(on)


class _Library:
    """The loaded native library.  Attribute access returns the C entry points unchanged (their `argtypes` / `restype` are
    set on those objects); while `NVTX` is on, calls go through a wrapper that opens an NVTX range named after the entry
    point, so that every kernel launcher shows up by name in an Nsight Systems timeline next to the step marks."""

    def __init__(self, raw):
        object.__setattr__(self, "_raw", raw)
        object.__setattr__(self, "_wrapped", {})

    def __getattr__(self, name):
        fn = getattr(self._raw, name)
        if not NVTX or not name.startswith("sb_"):
            return fn
        w = self._wrapped.get(name)
        if w is None:
            def w(*args, _fn=fn, _name=name):
                torch.cuda.nvtx.range_push(_name)
                try:
                    return _fn(*args)
                finally:
                    torch.cuda.nvtx.range_pop()
            self._wrapped[name] = w
        return w

    def __setattr__(self, name, value):
        setattr(self._raw, name, value)


class _Sig:
    P, I, F, LL = c_void_p, c_int, c_float, c_ll
    sb_gemm_bf16 = [P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, P, I, P]
    sb_colsum = [P, P, I, I, P]
    sb_gemm_set_pair_mode = [I]
    sb_gemm_fp8 = [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, I, P, P]
    sb_quantize_fp8 = [P, P, P, P, LL, I, P]
    sb_quantize_fp8_delayed = [P, P, P, I, I, P, LL, I, P]
    sb_rmsnorm_fwd = [P, P, P, P, I, I, F, I, P]
    sb_rmsnorm_fwd_fp8 = [P, P, P, P, I, I, F, I, P, I, I, P, P]
    sb_glu_fwd_fp8 = [P, P, LL, I, I, P, I, I, P, P]
    sb_glu_bwd_fp8 = [P, P, P, LL, I, I, P, I, I, P, P]
    sb_rmsnorm_bwd = [P, P, P, P, P, P, P, P, I, I, F, I, P]
    sb_rmsnorm_bwd_blocks = [I]
    sb_glu_fwd = [P, P, LL, I, I, P]
    sb_glu_bwd = [P, P, P, LL, I, I, P]
    sb_rope = [P, P, P, P, I, I, I, I, I, LL, LL, I, P]
    sb_ce_fwd = [P, P, P, P, LL, I, P]
    sb_ce_bwd = [P, P, P, P, P, LL, I, P]
    sb_sqnorm = [P, P, P, LL, I, P]
    sb_adam = [P, P, P, P, P, LL, F, F, F, F, F, F, F, I, P, F, I, P]
    sb_dwconv_fwd = [P, P, P, P, I, I, I, I, P]
    sb_dwconv_bwd = [P, P, P, P, P, P, P, I, I, I, I, P]
    sb_se_fwd = [P, P, P, P, I, I, I, I, I, I, I, P]
    sb_se_bwd = [P, P, P, P, P, P, P, I, I, I, I, I, I, I, P]
    sb_mr_fwd = [P, P, P, P, P, P, I, I, I, I, I, P]
    sb_mr_bwd = [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, P]
    sb_mr_tc_fwd = [P, P, P, P, P, I, I, I, I, I, P]
    sb_mr_tc_set_bwd_variant = [I]
    sb_se_set_bwd_variant = [I]
    sb_conv_set_fwd_variant = [I]
    sb_mr_tc_bwd = [P, P, P, P, P, P, P, P, P, I, I, I, I, I, P]
    sb_li_fwd = [P, P, P, P, P, P, P, P, I, I, I, I, P]
    sb_li_set_variant = [I]
    sb_li_bwd_chunk = [I, I]
    sb_li_bwd = [P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, P]


def launch_count() -> int:
    return _LAUNCHES


# ----------------------------------------------------------------------------- guarded allocation (debug aid)
# Every buffer a kernel of this library writes (outputs, gradients, scratch) is allocated through the four helpers
# below.  Normally they are torch.empty / zeros.  Inside `guarded_allocations()` each buffer is instead a window into a
# larger one whose margins (GUARD elements on either side) hold a byte pattern; `check_guards()` verifies the margins
# after the kernels have run, so a kernel that stores outside its output - a wrong tile bound, a bad leading
# dimension - is caught even when the stray store lands in memory the process owns (where no fault would show it).
GUARD = 256                 # elements on each side; keeps the window 256-byte aligned for every dtype
_GUARD_BYTE = 0x5B
_GUARDED = None             # None = off; else list of (whole buffer, window numel, tag)


def _numel(shape) -> int:
    n = 1
    for d in (shape if isinstance(shape, (tuple, list, torch.Size)) else (shape,)):
        n *= int(d)
    return n


def _alloc(*shape, dtype=None, device=None):
    if len(shape) == 1 and isinstance(shape[0], (tuple, list, torch.Size)):
        shape = tuple(shape[0])
    if _GUARDED is None or (device is not None and torch.device(device).type != "cuda"):
        return torch.empty(shape, dtype=dtype, device=device)
    dtype = dtype or torch.get_default_dtype()
    n = _numel(shape)
    whole = torch.empty(n + 2 * GUARD, dtype=dtype, device=device)
    whole.view(torch.uint8).fill_(_GUARD_BYTE)
    _GUARDED.append((whole, n, f"{tuple(shape)} {dtype}"))
    return whole[GUARD:GUARD + n].view(shape)


def _alloc_like(t):
    if _GUARDED is None or not t.is_cuda:
        return torch.empty_like(t)
    return _alloc(tuple(t.shape), dtype=t.dtype, device=t.device)


def _zeros(*shape, dtype=None, device=None):
    if len(shape) == 1 and isinstance(shape[0], (tuple, list, torch.Size)):
        shape = tuple(shape[0])
    if _GUARDED is None or (device is not None and torch.device(device).type != "cuda"):
        return torch.zeros(shape, dtype=dtype, device=device)
    return _alloc(shape, dtype=dtype, device=device).zero_()


def _zeros_like(t):
    if _GUARDED is None or not t.is_cuda:
        return torch.zeros_like(t)
    return _alloc(tuple(t.shape), dtype=t.dtype, device=t.device).zero_()


class guarded_allocations:
    """Context manager: allocate this library's kernel outputs with guard margins (see above)."""

    def __enter__(self):
        global _GUARDED
        self.prev, _GUARDED = _GUARDED, []
        return self

    def __exit__(self, *exc):
        global _GUARDED
        _GUARDED = self.prev
        return False


def check_guards() -> int:
    """Verify the margins of every buffer allocated under `guarded_allocations()` so far; raises on the first damaged
    one, naming its shape.  Returns the number of buffers checked."""
    if _GUARDED is None:
        return 0
    torch.cuda.synchronize()
    for whole, n, tag in _GUARDED:
        b = whole.view(torch.uint8)
        item = whole.element_size()
        lo, hi = b[: GUARD * item], b[(GUARD + n) * item:]
        if bool((lo != _GUARD_BYTE).any()) or bool((hi != _GUARD_BYTE).any()):
            side = "before" if bool((lo != _GUARD_BYTE).any()) else "after"
            raise RuntimeError(f"a kernel wrote outside its output buffer {tag} ({side} it)")
    return len(_GUARDED)


def _count(n: int = 1) -> None:
    global _LAUNCHES
    _LAUNCHES += n


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"savanna_b200 kernel `{what}` rejected its arguments or failed to launch (code {rc})")


def status_word(device) -> torch.Tensor:
    """Per-device uint32 word the bounded waits of the kernels write when they give up."""
    key = torch.device(device).index or 0
    if key not in _STATUS:
        _STATUS[key] = _zeros(1, dtype=torch.int32, device=device)
    return _STATUS[key]


def check_status(device=None) -> int:
    """Read (and clear) the status word; raises if a kernel recorded a timed-out wait.  Synchronises."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    w = status_word(device)
    v = int(w.item())
    if v != 0:
        w.zero_()
        raise RuntimeError(f"a kernel gave up on a bounded wait: code {(v >> 24) & 0xff}, detail {v & 0xffffff}")
    return v


def _is_bf16(*ts) -> bool:
    return all(t is None or t.dtype == bf16 for t in ts)


# ----------------------------------------------------------------------------- GEMM


def gemm(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, a_mn: bool = False, b_mn: bool = False,
         bias: Optional[torch.Tensor] = None, accumulate: bool = False, max_ctas: int = 0,
         residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[M,N] = A * B^T (+bias) (+residual) (+out).  `a` is [M,K] (a_mn False) or the transposed storage [K,M]
    (a_mn True); `b` is [N,K] or [K,N].  2-D tensors with unit inner stride."""
    lib = require()
    M, N = out.shape
    K = a.shape[0] if a_mn else a.shape[1]
    for t in (a, b, out):
        if t.dim() != 2 or t.stride(1) != 1 or t.dtype != bf16:
            raise ValueError("gemm operands must be 2-D bf16 with unit inner stride")
    if residual is not None and (residual.dim() != 2 or residual.stride(1) != 1 or residual.dtype != bf16
                                 or tuple(residual.shape) != (M, N)):
        raise ValueError("gemm residual must be a [M, N] bf16 matrix with unit inner stride")
    rc = lib.sb_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), _ptr(bias), _ptr(residual), M, N, K, a.stride(0),
                          b.stride(0), out.stride(0), residual.stride(0) if residual is not None else 0, int(a_mn),
                          int(b_mn), int(accumulate), status_word(out.device).data_ptr(), max_ctas, _stream())
    if rc != 0:
        detail = lib.sb_gemm_last_error_detail()
        raise RuntimeError(f"gemm_bf16 failed (code {rc}, operand {detail >> 16}, driver result {detail & 0xffff}): "
                           f"M={M} N={N} K={K} a{tuple(a.shape)}/{a.stride()} b{tuple(b.shape)}/{b.stride()} "
                           f"out{tuple(out.shape)}/{out.stride()} a_mn={a_mn} b_mn={b_mn} "
                           f"ptrs {a.data_ptr():#x} {b.data_ptr():#x} {out.data_ptr():#x}")
    _count()
    return out


def set_mr_backward_variant(streaming: bool) -> None:
    """Hyena-MR tensor-core backward: the streaming kernel (rings of u and g rows, one filter-gradient flush per CTA;
    default) or one independent CTA per 64-row tile."""
    require().sb_mr_tc_set_bwd_variant(int(bool(streaming)))


def set_se_backward_variant(tiled: bool) -> None:
    """Hyena-SE backward: tiles staged through shared memory (default), or one run per thread reading global memory."""
    require().sb_se_set_bwd_variant(int(bool(tiled)))


def set_conv_forward_variant(tiled: bool) -> None:
    """Depthwise (featuriser) convolution forward: tiles staged through shared memory, or one run per thread."""
    require().sb_conv_set_fwd_variant(int(bool(tiled)))


_PAIR_MODE = 2


def set_gemm_pair_mode(mode: int) -> None:
    """0: one CTA per 128 x 256 tile; 1: CTA pairs (cta_group::2, 256 x 256 tiles) for fp8 operands; 2: for bf16 too."""
    global _PAIR_MODE
    require().sb_gemm_set_pair_mode(int(mode))
    _PAIR_MODE = int(mode)


def colsum(x2: torch.Tensor) -> torch.Tensor:
    """fp32 column sums of a [T, N] bf16 matrix (bias gradients) without an fp32 copy of the matrix."""
    lib = require()
    T, N = x2.shape
    out = _zeros(N, dtype=torch.float32, device=x2.device)
    _check(lib.sb_colsum(x2.data_ptr(), out.data_ptr(), T, N, _stream()), "colsum")
    _count()
    return out


def _rows(x):
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(1) != 1 or (x2.stride(0) % 8) or (x2.data_ptr() % 16):
        x2 = x2.contiguous()
    return x2


class _Linear(torch.autograd.Function):
    """y = x w^T (+ bias) (+ residual).  The weight gradient is accumulated by the GEMM epilogue directly into
    `w.grad` when the parameter lives in a persistent flat gradient buffer (marked `_fuse_grad_accum` by the
    ZeRO optimizer): no temporary gradient, no separate accumulation pass."""

    @staticmethod
    def forward(ctx, x, w, bias, residual):
        x2 = _rows(x)
        out = _alloc((x2.shape[0], w.shape[0]), dtype=bf16, device=x.device)
        r2 = _rows(residual) if residual is not None else None
        gemm(x2, w, out, bias=bias, residual=r2)
        ctx.save_for_backward(x2, w)
        ctx.has_bias = bias is not None
        ctx.has_res = residual is not None
        ctx.xshape = x.shape
        ctx.wref = w
        return out.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, gy):
        x2, w = ctx.saved_tensors
        g2 = _rows(gy)
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            gx = _alloc_like(x2)
            gemm(g2, w, gx, a_mn=False, b_mn=True)                 # dX[T,K] = dY[T,N] . W[N,K]
            gx = gx.view(ctx.xshape)
        if ctx.needs_input_grad[1]:
            wp = ctx.wref
            tgt = wp.grad if getattr(wp, "_fuse_grad_accum", False) else None
            if tgt is not None and tgt.dtype == bf16 and tgt.is_contiguous() and tgt.shape == w.shape:
                gemm(g2, x2, tgt, a_mn=True, b_mn=True, accumulate=True)   # dW += dY^T X, straight into the flat buffer
            else:
                gw = _alloc_like(w)
                gemm(g2, x2, gw, a_mn=True, b_mn=True)             # dW[N,K] = dY^T[N,T] . X[T,K]
        if ctx.has_bias and ctx.needs_input_grad[2]:
            gb = colsum(g2).to(gy.dtype) if g2.shape[1] % 8 == 0 else g2.float().sum(0).to(gy.dtype)
        gr = gy if (ctx.has_res and ctx.needs_input_grad[3]) else None
        return gx, gw, gb, gr


# ----------------------------------------------------------------------------- fp8 projections (per-tensor scaling)

E4M3, E5M2 = 0, 1
PARAM_EPOCH = 0          # bumped by the optimizer after every parameter update: invalidates cached fp8 weights


def bump_param_epoch() -> None:
    global PARAM_EPOCH
    PARAM_EPOCH += 1


def quantize_fp8(x2: torch.Tensor, fmt: int):
    """Per-tensor current scaling: q = sat(x * fmax / amax(x)) as bytes, plus the de-quantisation factor (device scalar)."""
    lib = require()
    q = _alloc(x2.shape, dtype=torch.uint8, device=x2.device)
    amax = _alloc(1, dtype=torch.float32, device=x2.device)
    sinv = _alloc(1, dtype=torch.float32, device=x2.device)
    _check(lib.sb_quantize_fp8(x2.data_ptr(), q.data_ptr(), amax.data_ptr(), sinv.data_ptr(), x2.numel(), fmt, _stream()),
           "quantize_fp8")
    _count(2)
    return q, sinv


class Fp8History:
    """Amax ring of one quantisation site for delayed scaling (the recipe of the reference's TransformerEngine layers:
    amax_history_len=16, amax_compute_algo="max", savanna/model/tengine.py:19).  The ring has two slots more than the
    history: the one that collects the running call's amax and the one being cleared for the call after it."""

    __slots__ = ("buf", "cur", "primed")

    def __init__(self, device, history: int):
        self.buf = _zeros(history + 2, dtype=torch.float32, device=device)
        self.cur = 0
        self.primed = False


FP8_HISTORY = 16         # amax history length of the activation/gradient sites; 0 = current scaling (two passes)


def set_fp8_history(n: int) -> None:
    global FP8_HISTORY
    FP8_HISTORY = int(n)


def _site(owner, role: str, device) -> Fp8History:
    sites = owner.__dict__.setdefault("_fp8_sites", {})
    h = sites.get(role)
    if h is None or h.buf.numel() != FP8_HISTORY + 2 or h.buf.device != device:
        h = sites[role] = Fp8History(device, FP8_HISTORY)
    return h


def quantize_fp8_site(x2: torch.Tensor, fmt: int, owner, role: str):
    """Quantise at a named site of `owner` (a parameter): delayed scaling from the site's amax history in one pass over
    the data; the first call at a site has no history and uses current scaling."""
    if FP8_HISTORY <= 0 or owner is None:
        return quantize_fp8(x2, fmt)
    h = _site(owner, role, x2.device)
    lib = require()
    q = _alloc(x2.shape, dtype=torch.uint8, device=x2.device)
    sinv = _alloc(1, dtype=torch.float32, device=x2.device)
    if not h.primed:
        _check(lib.sb_quantize_fp8(x2.data_ptr(), q.data_ptr(), h.buf.data_ptr(), sinv.data_ptr(), x2.numel(), fmt, _stream()),
               "quantize_fp8")
        _count(2)
        h.primed, h.cur = True, 1
        return q, sinv
    _check(lib.sb_quantize_fp8_delayed(x2.data_ptr(), q.data_ptr(), h.buf.data_ptr(), h.buf.numel(), h.cur, sinv.data_ptr(),
                                       x2.numel(), fmt, _stream()), "quantize_fp8_delayed")
    _count()
    h.cur = (h.cur + 1) % h.buf.numel()
    return q, sinv


def gemm_fp8(a, b, out, alpha, a_mn=False, b_mn=False, a_fmt=E4M3, b_fmt=E4M3, bias=None, residual=None, accumulate=False,
             alpha2=None):
    lib = require()
    M, N = out.shape
    K = a.shape[0] if a_mn else a.shape[1]
    rc = lib.sb_gemm_fp8(a.data_ptr(), b.data_ptr(), out.data_ptr(), _ptr(bias), _ptr(residual), alpha.data_ptr(),
                         _ptr(alpha2), M, N, K,
                         a.stride(0), b.stride(0), out.stride(0), residual.stride(0) if residual is not None else 0,
                         int(a_mn), int(b_mn), a_fmt, b_fmt, int(accumulate), status_word(out.device).data_ptr(), _stream())
    if rc != 0:
        raise RuntimeError(f"gemm_fp8 failed (code {rc}): M={M} N={N} K={K} a{tuple(a.shape)} b{tuple(b.shape)} a_mn={a_mn} b_mn={b_mn}")
    _count()
    return out


# gated MLP: apply the gate in the epilogue of the w1|w2 projection (CTA-pair fp8 kernel); SAVANNA_B200_GLU_EPILOGUE=0
# selects the separate gate kernel (A/B measurements)
GLU_EPILOGUE = os.environ.get("SAVANNA_B200_GLU_EPILOGUE", "1") != "0"


GLU_BWD_EPILOGUE = os.environ.get("SAVANNA_B200_GLU_BWD_EPILOGUE", "0") != "0"    # likewise for the gate backward (w3 dgrad)


def set_glu_epilogue(on: bool, backward=None) -> None:
    global GLU_EPILOGUE, GLU_BWD_EPILOGUE
    GLU_EPILOGUE = bool(on)
    if backward is not None:
        GLU_BWD_EPILOGUE = bool(backward)


def gemm_fp8_glu(xq, w12q, ab, hq, sx, s12, site, sh):
    """ab [T, 2F] = (x w12^T) de-quantised, hq [T, F] = e4m3(silu(a) * b) under the delayed scaling of `site` (advances
    its ring); sh receives hq's de-quantisation factor."""
    lib = require()
    if not getattr(lib, "_sb_glu_ready", False):
        P, I = ctypes.c_void_p, ctypes.c_int
        lib.sb_gemm_fp8_glu.restype = I
        lib.sb_gemm_fp8_glu.argtypes = [P, P, P, P, P, P, I, I, I, I, I, I, P, I, I, P, P, P]
        lib._sb_glu_ready = True
    T, K = xq.shape
    F = hq.shape[1]
    rc = lib.sb_gemm_fp8_glu(xq.data_ptr(), w12q.data_ptr(), ab.data_ptr(), hq.data_ptr(), sx.data_ptr(), s12.data_ptr(), T, F, K,
                             xq.stride(0), w12q.stride(0), ab.stride(0), site.buf.data_ptr(), site.buf.numel(), site.cur,
                             sh.data_ptr(), status_word(ab.device).data_ptr(), _stream())
    if rc != 0:
        raise RuntimeError(f"gemm_fp8_glu failed (code {rc}): T={T} F={F} K={K}")
    _count()
    site.cur = (site.cur + 1) % site.buf.numel()


def gemm_fp8_glu_bwd(gq, w3q, ab, dq, sg, s3, site, sd):
    """dq [T, 2F] = e5m2 gate gradients of [a | b] from g = (gq w3q) de-quantised, under the delayed scaling of `site`
    (advances its ring); sd receives dq's de-quantisation factor.  g itself is not stored."""
    lib = require()
    if not getattr(lib, "_sb_glu_bwd_ready", False):
        P, I = ctypes.c_void_p, ctypes.c_int
        lib.sb_gemm_fp8_glu_bwd.restype = I
        lib.sb_gemm_fp8_glu_bwd.argtypes = [P, P, P, P, P, P, I, I, I, I, I, I, P, I, I, P, P, P]
        lib._sb_glu_bwd_ready = True
    T, D = gq.shape
    F = w3q.shape[1]
    rc = lib.sb_gemm_fp8_glu_bwd(gq.data_ptr(), w3q.data_ptr(), ab.data_ptr(), dq.data_ptr(), sg.data_ptr(), s3.data_ptr(), T, F, D,
                                 gq.stride(0), w3q.stride(0), ab.stride(0), site.buf.data_ptr(), site.buf.numel(), site.cur,
                                 sd.data_ptr(), status_word(ab.device).data_ptr(), _stream())
    if rc != 0:
        raise RuntimeError(f"gemm_fp8_glu_bwd failed (code {rc}): T={T} F={F} D={D}")
    _count()
    site.cur = (site.cur + 1) % site.buf.numel()


def _fp8_weight(w):
    cache = getattr(w, "_fp8_cache", None)
    if cache is None or cache[0] != PARAM_EPOCH:
        wq, sw = quantize_fp8(w.detach(), E4M3)
        cache = (PARAM_EPOCH, wq, sw)
        w._fp8_cache = cache
    return cache[1], cache[2]


class _LinearFP8(torch.autograd.Function):
    """Projection with fp8 tensor-core operands (e4m3 activations and weights, e5m2 output gradients — the HYBRID
    recipe of the reference's TransformerEngine layers, savanna/model/tengine.py:17-20), per-tensor scaling (delayed
    for activations and gradients, current for the weights), fp32 accumulation, bf16 results.  The quantised
    activation is reused by the weight-gradient GEMM; quantised weights are cached until the optimizer updates the
    parameters."""

    @staticmethod
    def forward(ctx, x, w, bias, residual):
        x2 = _rows(x)
        xq, sx = quantize_fp8_site(x2, E4M3, w, "x")
        wq, sw = _fp8_weight(w)
        out = _alloc((x2.shape[0], w.shape[0]), dtype=bf16, device=x.device)
        r2 = _rows(residual) if residual is not None else None
        gemm_fp8(xq, wq, out, sx, bias=bias, residual=r2, alpha2=sw)
        ctx.save_for_backward(xq, sx, wq, sw)
        ctx.has_bias, ctx.has_res, ctx.xshape, ctx.wref = bias is not None, residual is not None, x.shape, w
        return out.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, gy):
        xq, sx, wq, sw = ctx.saved_tensors
        g2 = _rows(gy)
        gq, sg = quantize_fp8_site(g2, E5M2, ctx.wref, "g")
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            gx = _alloc((g2.shape[0], wq.shape[1]), dtype=bf16, device=gy.device)
            gemm_fp8(gq, wq, gx, sg, b_mn=True, a_fmt=E5M2, b_fmt=E4M3, alpha2=sw)
            gx = gx.view(ctx.xshape)
        if ctx.needs_input_grad[1]:
            wp = ctx.wref
            tgt = wp.grad if getattr(wp, "_fuse_grad_accum", False) else None
            if tgt is not None and tgt.dtype == bf16 and tgt.is_contiguous() and tgt.shape == wp.shape:
                gemm_fp8(gq, xq, tgt, sg, a_mn=True, b_mn=True, a_fmt=E5M2, b_fmt=E4M3, accumulate=True, alpha2=sx)
            else:
                gw = _alloc(wp.shape, dtype=bf16, device=gy.device)
                gemm_fp8(gq, xq, gw, sg, a_mn=True, b_mn=True, a_fmt=E5M2, b_fmt=E4M3, alpha2=sx)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            gb = colsum(g2).to(gy.dtype)
        gr = gy if (ctx.has_res and ctx.needs_input_grad[3]) else None
        return gx, gw, gb, gr


# ----------------------------------------------------------------------------- block-scaled fp8 (MXFP8)
FP8_RECIPE = "delayed"      # "delayed": per-tensor scaling (default); "mxfp8": one E8M0 scale per 32 elements of the contraction


def set_fp8_recipe(name: str) -> None:
    global FP8_RECIPE
    if name not in ("delayed", "mxfp8"):
        raise ValueError(f"unknown fp8 recipe {name!r}")
    FP8_RECIPE = name


def _mx_sigs(lib):
    if getattr(lib, "_sb_mx_ready", False):
        return
    P, I, LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    lib.sb_mx_sf_bytes.restype = LL
    lib.sb_mx_sf_bytes.argtypes = [LL, LL]
    lib.sb_mx_quantize.restype = I
    lib.sb_mx_quantize.argtypes = [P, P, P, LL, I, LL, I, P]
    lib.sb_gemm_mx.restype = I
    lib.sb_gemm_mx.argtypes = [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, P, P]
    lib._sb_mx_ready = True


def mx_quantize(x2: torch.Tensor, transposed: bool = False):
    """x2 [R, C] bf16 -> (q, sf): e4m3 bytes and E8M0 block scales (one per 32 elements of the contraction dimension) in
    the layout the block-scaled tensor-core instruction reads.  transposed=False: q [R, C], scales along C (C % 32 == 0).
    transposed=True: q [C, R], scales along R (R % 32 == 0): the operand form of a product contracted over the rows."""
    lib = require()
    _mx_sigs(lib)
    R, C = x2.shape
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    rows, k = (C, R) if transposed else (R, C)
    q = _alloc((rows, k), dtype=torch.uint8, device=x2.device)
    sf = _zeros(lib.sb_mx_sf_bytes(rows, k), dtype=torch.uint8, device=x2.device)
    _check(lib.sb_mx_quantize(x2.data_ptr(), q.data_ptr(), sf.data_ptr(), R, C, x2.stride(0), int(transposed), _stream()),
           "mx_quantize")
    _count(2)
    return q, sf


def gemm_mx(a, sfa, b, sfb, out, bias=None, residual=None, accumulate=False):
    """out [M, N] bf16 (+)= a [M, K] b [N, K]^T with e4m3 operands and their block scales."""
    lib = require()
    _mx_sigs(lib)
    M, K = a.shape
    N = b.shape[0]
    rc = lib.sb_gemm_mx(a.data_ptr(), sfa.data_ptr(), b.data_ptr(), sfb.data_ptr(), out.data_ptr(), _ptr(bias), _ptr(residual),
                        M, N, K, a.stride(0), b.stride(0), out.stride(0), residual.stride(0) if residual is not None else 0,
                        int(accumulate), status_word(out.device).data_ptr(), _stream())
    if rc != 0:
        raise RuntimeError(f"gemm_mx failed (code {rc}): M={M} N={N} K={K}")
    _count()
    return out


def _mx_weight(w):
    """(row-wise quantised w [N, K], its scales, row-wise quantised w^T [K, N], its scales), cached per parameter update:
    the forward contracts over K, the input-gradient product over N."""
    cache = getattr(w, "_mx_cache", None)
    if cache is None or cache[0] != PARAM_EPOCH:
        wd = w.detach()
        cache = (PARAM_EPOCH,) + mx_quantize(wd) + mx_quantize(wd, transposed=True)
        w._mx_cache = cache
    return cache[1:]


class _LinearMX(torch.autograd.Function):
    """Projection with block-scaled fp8 operands (MXFP8: e4m3 data, one power-of-two scale per 32 elements of the
    contraction, applied inside `tcgen05.mma.kind::mxf8f6f4.block_scale`): every product gets operands quantised along
    its own contraction dimension, so activations and output gradients are quantised twice (row-wise for the forward /
    input-gradient products, transposed for the weight-gradient product) and weights twice per optimizer step.  No amax
    history and no global scale: outliers only cost the 32 values that share their block."""

    @staticmethod
    def forward(ctx, x, w, bias, residual):
        x2 = _rows(x)
        xq, sx = mx_quantize(x2)
        wq, sw, wtq, swt = _mx_weight(w)
        out = _alloc((x2.shape[0], w.shape[0]), dtype=bf16, device=x.device)
        r2 = _rows(residual) if residual is not None else None
        gemm_mx(xq, sx, wq, sw, out, bias=bias, residual=r2)
        xtq, sxt = mx_quantize(x2, transposed=True) if w.requires_grad else (None, None)
        ctx.save_for_backward(xtq, sxt, wtq, swt)
        ctx.has_bias, ctx.has_res, ctx.xshape, ctx.wref = bias is not None, residual is not None, x.shape, w
        return out.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, gy):
        xtq, sxt, wtq, swt = ctx.saved_tensors
        g2 = _rows(gy)
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            gq, sg = mx_quantize(g2)
            gx = _alloc((g2.shape[0], wtq.shape[0]), dtype=bf16, device=gy.device)
            gemm_mx(gq, sg, wtq, swt, gx)                                   # dX = dY W: contraction over the outputs
            gx = gx.view(ctx.xshape)
        if ctx.needs_input_grad[1]:
            gtq, sgt = mx_quantize(g2, transposed=True)
            wp = ctx.wref
            tgt = wp.grad if getattr(wp, "_fuse_grad_accum", False) else None
            if tgt is not None and tgt.dtype == bf16 and tgt.is_contiguous() and tgt.shape == wp.shape:
                gemm_mx(gtq, sgt, xtq, sxt, tgt, accumulate=True)           # dW += dY^T X: contraction over the rows
            else:
                gw = _alloc(wp.shape, dtype=bf16, device=gy.device)
                gemm_mx(gtq, sgt, xtq, sxt, gw)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            gb = colsum(g2).to(gy.dtype)
        gr = gy if (ctx.has_res and ctx.needs_input_grad[3]) else None
        return gx, gw, gb, gr


def linear(x, w, bias=None, fp8: bool = False, residual=None):
    if fp8 and FP8_RECIPE == "mxfp8" and _is_bf16(x, w, bias, residual) and w.shape[0] % 32 == 0 and w.shape[1] % 32 == 0 \
            and (x.numel() // x.shape[-1]) % 32 == 0:
        return _LinearMX.apply(x, w, bias, residual)
    if fp8 and _is_bf16(x, w, bias, residual) and w.shape[0] % 16 == 0 and w.shape[1] % 16 == 0:
        return _LinearFP8.apply(x, w, bias, residual)
    if not _is_bf16(x, w, bias, residual) or (w.shape[0] % 8) or (w.shape[1] % 8):
        y = ref.linear(x, w, bias)
        return y if residual is None else y + residual
    return _Linear.apply(x, w, bias, residual)


def linear_allgather(x, w, bias, seq_dim, fp8):
    from ..parallel import fused_tp
    if fp8 and FP8_RECIPE == "mxfp8":
        return None                 # block-scaled operands: the caller gathers with NCCL and runs the MXFP8 projection
    return fused_tp.linear_allgather(x, w, bias, seq_dim, fp8=bool(fp8) and _is_bf16(x, w, bias))


def linear_reducescatter(x, w, seq_dim, fp8):
    from ..parallel import fused_tp
    if fp8 and FP8_RECIPE == "mxfp8":
        return None                 # as above: MXFP8 projection, then an NCCL reduce-scatter
    return fused_tp.linear_reducescatter(x, w, seq_dim, fp8=bool(fp8) and _is_bf16(x, w))


# ----------------------------------------------------------------------------- RMSNorm


def _rmsnorm_fwd(x, w, eps, form):
    lib = require()
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    T, D = x2.shape
    y = _alloc_like(x2)
    a = _alloc(T, dtype=torch.float32, device=x.device)
    wc = w.contiguous()
    _check(lib.sb_rmsnorm_fwd(x2.data_ptr(), wc.data_ptr(), y.data_ptr(), a.data_ptr(), T, D, eps, form, _stream()),
           "rmsnorm_fwd")
    _count()
    return x2, wc, a, y


def _rmsnorm_bwd(x2, w, a, gy, gres, eps, form):
    lib = require()
    T, D = x2.shape
    g2 = gy.reshape(T, D).contiguous()
    r2 = gres.reshape(T, D).contiguous() if gres is not None else None
    dx = _alloc_like(x2)
    dw = _alloc(D, dtype=bf16, device=x2.device)
    partial = _alloc(lib.sb_rmsnorm_bwd_blocks(T) * D, dtype=torch.float32, device=x2.device)
    _check(lib.sb_rmsnorm_bwd(x2.data_ptr(), w.data_ptr(), g2.data_ptr(), a.data_ptr(), _ptr(r2), dx.data_ptr(),
                              dw.data_ptr(), partial.data_ptr(), T, D, eps, form, _stream()), "rmsnorm_bwd")
    _count(2)
    return dx, dw


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps, form):
        x2, wc, a, y = _rmsnorm_fwd(x, w, eps, form)
        ctx.save_for_backward(x2, wc, a)
        ctx.meta = (eps, form, x.shape)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, gy):
        x2, w, a = ctx.saved_tensors
        eps, form, shape = ctx.meta
        dx, dw = _rmsnorm_bwd(x2, w, a, gy, None, eps, form)
        return dx.view(shape), dw, None, None


class _RMSNormResidual(torch.autograd.Function):
    """(norm(x), x): the second output carries x down the residual branch; the gradient arriving there is added inside
    the norm's backward kernel instead of by a separate accumulation kernel."""

    @staticmethod
    def forward(ctx, x, w, eps, form):
        x2, wc, a, y = _rmsnorm_fwd(x, w, eps, form)
        ctx.save_for_backward(x2, wc, a)
        ctx.meta = (eps, form, x.shape)
        ctx.set_materialize_grads(False)
        return y.view(x.shape), x.view_as(x)

    @staticmethod
    def backward(ctx, gy, gres):
        x2, w, a = ctx.saved_tensors
        eps, form, shape = ctx.meta
        if gy is None:
            return gres, None, None, None
        dx, dw = _rmsnorm_bwd(x2, w, a, gy, gres, eps, form)
        return dx.view(shape), dw, None, None


def _fp8_backward_gemms(ctx_w, gy2, xq, sx, wq, sw, need_gx, need_gw, quantised=None):
    """Shared by the fp8 projections: quantise the output gradient (e5m2), then dgrad and (in-place) wgrad.
    `quantised` = (gq, sg) when the caller has already quantised the gradient."""
    gq, sg = quantised if quantised is not None else quantize_fp8_site(gy2, E5M2, ctx_w, "g")
    gx = gw = None
    if need_gx:
        gx = _alloc((gy2.shape[0], wq.shape[1]), dtype=bf16, device=gy2.device)
        gemm_fp8(gq, wq, gx, sg, b_mn=True, a_fmt=E5M2, b_fmt=E4M3, alpha2=sw)
    if need_gw:
        tgt = ctx_w.grad if getattr(ctx_w, "_fuse_grad_accum", False) else None
        if tgt is not None and tgt.dtype == bf16 and tgt.is_contiguous() and tgt.shape == ctx_w.shape:
            gemm_fp8(gq, xq, tgt, sg, a_mn=True, b_mn=True, a_fmt=E5M2, b_fmt=E4M3, accumulate=True, alpha2=sx)
        else:
            gw = _alloc(ctx_w.shape, dtype=bf16, device=gy2.device)
            gemm_fp8(gq, xq, gw, sg, a_mn=True, b_mn=True, a_fmt=E5M2, b_fmt=E4M3, alpha2=sx)
    return gx, gw


class _NormLinearFP8(torch.autograd.Function):
    """(linear(rmsnorm(x)), x): the norm kernel emits the e4m3 operand of the projection directly (delayed scaling: the
    scale is known before the tensor exists), so the normalised activations never exist in bf16; the second output
    carries x down the residual branch and its gradient is added inside the norm's backward kernel."""

    @staticmethod
    def forward(ctx, x, wn, eps, form, w, bias):
        lib = require()
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        T, D = x2.shape
        h = _site(w, "x", x.device)
        wnc = wn.contiguous()
        if not h.primed:
            _, _, a, y = _rmsnorm_fwd(x, wn, eps, form)
            xq, sx = quantize_fp8_site(y, E4M3, w, "x")
        else:
            xq = _alloc((T, D), dtype=torch.uint8, device=x.device)
            a = _alloc(T, dtype=torch.float32, device=x.device)
            sx = _alloc(1, dtype=torch.float32, device=x.device)
            _check(lib.sb_rmsnorm_fwd_fp8(x2.data_ptr(), wnc.data_ptr(), xq.data_ptr(), a.data_ptr(), T, D, eps, form,
                                          h.buf.data_ptr(), h.buf.numel(), h.cur, sx.data_ptr(), _stream()), "rmsnorm_fwd_fp8")
            _count()
            h.cur = (h.cur + 1) % h.buf.numel()
        wq, sw = _fp8_weight(w)
        out = _alloc((T, w.shape[0]), dtype=bf16, device=x.device)
        gemm_fp8(xq, wq, out, sx, bias=bias, alpha2=sw)
        ctx.save_for_backward(x2, wnc, a, xq, sx, wq, sw)
        ctx.meta = (eps, form, x.shape, bias is not None)
        ctx.wref = w
        ctx.set_materialize_grads(False)
        return out.view(*x.shape[:-1], w.shape[0]), x.view_as(x)

    @staticmethod
    def backward(ctx, gy, gres):
        x2, wn, a, xq, sx, wq, sw = ctx.saved_tensors
        eps, form, shape, has_bias = ctx.meta
        if gy is None:
            return gres, None, None, None, None, None
        g2 = _rows(gy)
        gxn, gw = _fp8_backward_gemms(ctx.wref, g2, xq, sx, wq, sw, True, ctx.needs_input_grad[4])
        gb = colsum(g2).to(gy.dtype) if (has_bias and ctx.needs_input_grad[5]) else None
        dx, dwn = _rmsnorm_bwd(x2, wn, a, gxn, gres, eps, form)
        return dx.view(shape), dwn, None, None, gw, gb


class _GluLinearFP8(torch.autograd.Function):
    """linear(act(a) * b) (+ bias, + residual) for ab = [a | b]: the gate kernel emits the e4m3 operand directly."""

    @staticmethod
    def forward(ctx, ab, act, w, bias, residual):
        lib = require()
        ab2 = ab.reshape(-1, ab.shape[-1]).contiguous()
        T, F2 = ab2.shape
        Fh = F2 // 2
        h = _site(w, "x", ab.device)
        if not h.primed:
            hb = _alloc((T, Fh), dtype=bf16, device=ab.device)
            _check(lib.sb_glu_fwd(ab2.data_ptr(), hb.data_ptr(), T, Fh, act, _stream()), "glu_fwd")
            _count()
            xq, sx = quantize_fp8_site(hb, E4M3, w, "x")
        else:
            xq = _alloc((T, Fh), dtype=torch.uint8, device=ab.device)
            sx = _alloc(1, dtype=torch.float32, device=ab.device)
            _check(lib.sb_glu_fwd_fp8(ab2.data_ptr(), xq.data_ptr(), T, Fh, act, h.buf.data_ptr(), h.buf.numel(), h.cur,
                                      sx.data_ptr(), _stream()), "glu_fwd_fp8")
            _count()
            h.cur = (h.cur + 1) % h.buf.numel()
        wq, sw = _fp8_weight(w)
        out = _alloc((T, w.shape[0]), dtype=bf16, device=ab.device)
        r2 = _rows(residual) if residual is not None else None
        gemm_fp8(xq, wq, out, sx, bias=bias, residual=r2, alpha2=sw)
        ctx.save_for_backward(ab2, xq, sx, wq, sw)
        ctx.meta = (act, ab.shape, bias is not None, residual is not None)
        ctx.wref = w
        return out.view(*ab.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, gy):
        lib = require()
        ab2, xq, sx, wq, sw = ctx.saved_tensors
        act, shape, has_bias, has_res = ctx.meta
        g2 = _rows(gy)
        gh, gw = _fp8_backward_gemms(ctx.wref, g2, xq, sx, wq, sw, True, ctx.needs_input_grad[2])
        gb = colsum(g2).to(gy.dtype) if (has_bias and ctx.needs_input_grad[3]) else None
        T, F2 = ab2.shape
        dab = _alloc_like(ab2)
        _check(lib.sb_glu_bwd(ab2.data_ptr(), gh.data_ptr(), dab.data_ptr(), T, F2 // 2, act, _stream()), "glu_bwd")
        _count()
        gr = gy if (has_res and ctx.needs_input_grad[4]) else None
        return dab.view(shape), None, gw, gb, gr


class _MlpFP8(torch.autograd.Function):
    """x + w3(act(a) * b) + b3 with [a | b] = w12(rmsnorm(x)): the whole gated MLP of a block as one autograd node, all
    three GEMMs on fp8 operands.  Every fp8 operand is written by the kernel that produces the tensor (norm, gate, gate
    backward), so neither the normalised input, nor the gated activation, nor the gradient of [a | b] exists in bf16."""

    @staticmethod
    def forward(ctx, x, wn, eps, form, w12, w3, b3, act):
        lib = require()
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        T, D = x2.shape
        F2 = w12.shape[0]
        Fh = F2 // 2
        dev = x.device
        wnc = wn.contiguous()
        hx, hh = _site(w12, "x", dev), _site(w3, "x", dev)
        if not (hx.primed and hh.primed):
            # first call: no amax history yet, take the separate kernels (they prime the sites)
            _, _, a, y = _rmsnorm_fwd(x, wn, eps, form)
            xq, sx = quantize_fp8_site(y, E4M3, w12, "x")
        else:
            xq = _alloc((T, D), dtype=torch.uint8, device=dev)
            a = _alloc(T, dtype=torch.float32, device=dev)
            sx = _alloc(1, dtype=torch.float32, device=dev)
            _check(lib.sb_rmsnorm_fwd_fp8(x2.data_ptr(), wnc.data_ptr(), xq.data_ptr(), a.data_ptr(), T, D, eps, form,
                                          hx.buf.data_ptr(), hx.buf.numel(), hx.cur, sx.data_ptr(), _stream()), "rmsnorm_fwd_fp8")
            _count()
            hx.cur = (hx.cur + 1) % hx.buf.numel()
        w12q, s12 = _fp8_weight(w12)
        ab = _alloc((T, F2), dtype=bf16, device=dev)
        fuse_gate = hh.primed and act == 0 and Fh % 128 == 0 and GLU_EPILOGUE and _PAIR_MODE >= 1
        if fuse_gate:
            # the gate runs in the epilogue of the w1|w2 projection: [a | b] and the e4m3 operand of w3 from one kernel
            hq = _alloc((T, Fh), dtype=torch.uint8, device=dev)
            sh = _alloc(1, dtype=torch.float32, device=dev)
            gemm_fp8_glu(xq, w12q, ab, hq, sx, s12, hh, sh)
        else:
            gemm_fp8(xq, w12q, ab, sx, alpha2=s12)
        if fuse_gate:
            pass
        elif not hh.primed:
            hb = _alloc((T, Fh), dtype=bf16, device=dev)
            _check(lib.sb_glu_fwd(ab.data_ptr(), hb.data_ptr(), T, Fh, act, _stream()), "glu_fwd")
            _count()
            hq, sh = quantize_fp8_site(hb, E4M3, w3, "x")
        else:
            hq = _alloc((T, Fh), dtype=torch.uint8, device=dev)
            sh = _alloc(1, dtype=torch.float32, device=dev)
            _check(lib.sb_glu_fwd_fp8(ab.data_ptr(), hq.data_ptr(), T, Fh, act, hh.buf.data_ptr(), hh.buf.numel(), hh.cur,
                                      sh.data_ptr(), _stream()), "glu_fwd_fp8")
            _count()
            hh.cur = (hh.cur + 1) % hh.buf.numel()
        w3q, s3 = _fp8_weight(w3)
        out = _alloc((T, w3.shape[0]), dtype=bf16, device=dev)
        gemm_fp8(hq, w3q, out, sh, bias=b3, residual=x2, alpha2=s3)
        ctx.save_for_backward(x2, wnc, a, xq, sx, w12q, s12, ab, hq, sh, w3q, s3)
        ctx.meta = (eps, form, x.shape, act, b3 is not None)
        ctx.w12, ctx.w3 = w12, w3
        return out.view(x.shape)

    @staticmethod
    def backward(ctx, gy):
        lib = require()
        x2, wn, a, xq, sx, w12q, s12, ab, hq, sh, w3q, s3 = ctx.saved_tensors
        eps, form, shape, act, has_b3 = ctx.meta
        w12, w3 = ctx.w12, ctx.w3
        g2 = _rows(gy)
        T, F2 = ab.shape
        dev = gy.device
        hg = _site(w12, "g", dev)
        Fh = F2 // 2
        fuse_gate = hg.primed and act == 0 and Fh % 32 == 0 and GLU_EPILOGUE and GLU_BWD_EPILOGUE and _PAIR_MODE >= 1
        if fuse_gate:
            # the gate backward runs in the epilogue of the w3 input-gradient product: its result [T, F] never exists
            gq3, sg3 = quantize_fp8_site(g2, E5M2, w3, "g")
            dq = _alloc((T, F2), dtype=torch.uint8, device=dev)
            sd = _alloc(1, dtype=torch.float32, device=dev)
            gemm_fp8_glu_bwd(gq3, w3q, ab, dq, sg3, s3, hg, sd)
            _, gw3 = _fp8_backward_gemms(w3, g2, hq, sh, w3q, s3, False, ctx.needs_input_grad[5], quantised=(gq3, sg3))
        else:
            gh, gw3 = _fp8_backward_gemms(w3, g2, hq, sh, w3q, s3, True, ctx.needs_input_grad[5])
        gb3 = colsum(g2).to(gy.dtype) if (has_b3 and ctx.needs_input_grad[6]) else None
        if fuse_gate:
            pass
        elif not hg.primed:
            dab = _alloc_like(ab)
            _check(lib.sb_glu_bwd(ab.data_ptr(), gh.data_ptr(), dab.data_ptr(), T, F2 // 2, act, _stream()), "glu_bwd")
            _count()
            dq, sd = quantize_fp8_site(dab, E5M2, w12, "g")
        else:
            dq = _alloc((T, F2), dtype=torch.uint8, device=dev)
            sd = _alloc(1, dtype=torch.float32, device=dev)
            _check(lib.sb_glu_bwd_fp8(ab.data_ptr(), gh.data_ptr(), dq.data_ptr(), T, F2 // 2, act, hg.buf.data_ptr(),
                                      hg.buf.numel(), hg.cur, sd.data_ptr(), _stream()), "glu_bwd_fp8")
            _count()
            hg.cur = (hg.cur + 1) % hg.buf.numel()
        gxn = _alloc((T, x2.shape[1]), dtype=bf16, device=dev)
        gemm_fp8(dq, w12q, gxn, sd, b_mn=True, a_fmt=E5M2, b_fmt=E4M3, alpha2=s12)
        gw12 = None
        if ctx.needs_input_grad[4]:
            tgt = w12.grad if getattr(w12, "_fuse_grad_accum", False) else None
            if tgt is not None and tgt.dtype == bf16 and tgt.is_contiguous() and tgt.shape == w12.shape:
                gemm_fp8(dq, xq, tgt, sd, a_mn=True, b_mn=True, a_fmt=E5M2, b_fmt=E4M3, accumulate=True, alpha2=sx)
            else:
                gw12 = _alloc(w12.shape, dtype=bf16, device=dev)
                gemm_fp8(dq, xq, gw12, sd, a_mn=True, b_mn=True, a_fmt=E5M2, b_fmt=E4M3, alpha2=sx)
        # the residual branch's gradient (gy itself) is added inside the norm's backward kernel
        dx, dwn = _rmsnorm_bwd(x2, wn, a, gxn, g2, eps, form)
        return dx.view(shape), dwn, None, None, gw12, gw3, gb3, None


def mlp_gated(x, norm_weight, eps, form, w12, w3, b3, act, fp8):
    """x + w3(act(a) * b) + b3, [a | b] = w12(rmsnorm(x)): one node on the fp8 path, the composed ops otherwise."""
    if (fp8 and act in _ACT and _fp8_fusable(x, w12, norm_weight, b3) and _is_bf16(w3) and 64 <= x.shape[-1] <= 16384
            and w3.shape[0] % 16 == 0 and w3.shape[1] % 16 == 0 and (w12.shape[0] // 2) % 16 == 0):
        return _MlpFP8.apply(x, norm_weight, float(eps), 0 if form == "te" else 1, w12, w3, b3, _ACT[act])
    ab, res = norm_linear(x, norm_weight, eps, form, w12, None, fp8)
    return glu_linear(ab, act, w3, b3, res, fp8)


def _fp8_fusable(x, w, *others) -> bool:
    # the norm / gate kernels write per-tensor (delayed-scaling) fp8 operands: not with the block-scaled recipe
    return (FP8_HISTORY > 0 and FP8_RECIPE == "delayed" and _is_bf16(x, w, *others) and w.shape[0] % 16 == 0 and w.shape[1] % 16 == 0
            and x.shape[-1] % 16 == 0)


def norm_linear(x, norm_weight, eps, form, w, bias, fp8):
    """(linear(rmsnorm(x)), x).  With fp8 projections and delayed scaling the norm emits the fp8 operand itself."""
    if fp8 and _fp8_fusable(x, w, norm_weight, bias) and 64 <= x.shape[-1] <= 16384:
        return _NormLinearFP8.apply(x, norm_weight, float(eps), 0 if form == "te" else 1, w, bias)
    y, res = rmsnorm_residual(x, norm_weight, eps, form)
    return linear(y, w, bias, fp8), res


def glu_linear(ab, act, w, bias, residual, fp8):
    """linear(act(a) * b) + bias + residual for ab = [a | b]."""
    if fp8 and act in _ACT and _fp8_fusable(ab, w, bias, residual) and (ab.shape[-1] // 2) % 16 == 0:
        return _GluLinearFP8.apply(ab, _ACT[act], w, bias, residual)
    return linear(glu_act_packed(ab, act), w, bias, fp8, residual)


def rmsnorm_residual(x, weight, eps, form="te"):
    """(rmsnorm(x), x) with the two gradients combined in one backward kernel."""
    if not _is_bf16(x, weight) or x.shape[-1] % 8 or x.shape[-1] > 16384 or x.shape[-1] < 64:
        return ref.rmsnorm(x, weight, eps, form), x
    return _RMSNormResidual.apply(x, weight, float(eps), 0 if form == "te" else 1)


def rmsnorm(x, weight, eps, form="te"):
    if not _is_bf16(x, weight) or x.shape[-1] % 8 or x.shape[-1] > 16384 or x.shape[-1] < 64:
        return ref.rmsnorm(x, weight, eps, form)
    return _RMSNorm.apply(x, weight, float(eps), 0 if form == "te" else 1)


# ----------------------------------------------------------------------------- gated activation


class _GluPacked(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ab, act):
        lib = require()
        ab2 = ab.reshape(-1, ab.shape[-1]).contiguous()
        T, F2 = ab2.shape
        Fh = F2 // 2
        h = _alloc((T, Fh), dtype=bf16, device=ab.device)
        _check(lib.sb_glu_fwd(ab2.data_ptr(), h.data_ptr(), T, Fh, act, _stream()), "glu_fwd")
        _count()
        ctx.save_for_backward(ab2)
        ctx.meta = (act, ab.shape)
        return h.view(*ab.shape[:-1], Fh)

    @staticmethod
    def backward(ctx, gh):
        lib = require()
        (ab2,) = ctx.saved_tensors
        act, shape = ctx.meta
        T, F2 = ab2.shape
        g2 = gh.reshape(T, F2 // 2).contiguous()
        dab = _alloc_like(ab2)
        _check(lib.sb_glu_bwd(ab2.data_ptr(), g2.data_ptr(), dab.data_ptr(), T, F2 // 2, act, _stream()), "glu_bwd")
        _count()
        return dab.view(shape), None


def glu_act_packed(ab, act="silu"):
    if not _is_bf16(ab) or (ab.shape[-1] // 2) % 8 or act not in _ACT:
        a, b = ab.chunk(2, dim=-1)
        return ref.glu_act(a, b, act)
    return _GluPacked.apply(ab, _ACT[act])


def glu_act(a, b, act="silu"):
    return glu_act_packed(torch.cat([a, b], dim=-1), act)


# ----------------------------------------------------------------------------- RoPE


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin):
        y = _rope_launch(x, cos, sin, 0)
        ctx.save_for_backward(cos, sin)
        return y

    @staticmethod
    def backward(ctx, gy):
        cos, sin = ctx.saved_tensors
        return _rope_launch(gy, cos, sin, 1), None, None


def _one_row_stride(t, L, H):
    rs = t.stride(2)
    return t.stride(3) == 1 and t.stride(1) == H * rs and t.stride(0) == L * H * rs and rs % 8 == 0 and t.data_ptr() % 16 == 0


def _rope_launch(x, cos, sin, inverse, out=None):
    """`out`: a destination [B, L, H, hd] whose rows (b, l, h) are one stride apart (a slice of a packed buffer)."""
    lib = require()
    B, L, H, hd = x.shape
    # rows (b,l,h) must be addressable with one stride: true for a slice of the packed [B,L,H,3*hd] projection
    rs = x.stride(2)
    if x.stride(3) != 1 or x.stride(1) != H * rs or x.stride(0) != L * H * rs or rs % 8 or x.data_ptr() % 16:
        x = x.contiguous()
        rs = hd
    if out is None:
        y, ys = _alloc((B, L, H, hd), dtype=bf16, device=x.device), hd
    else:
        if not _one_row_stride(out, L, H):
            raise ValueError("rope: destination rows must be one stride apart")
        y, ys = out, out.stride(2)
    _check(lib.sb_rope(x.data_ptr(), y.data_ptr(), cos.data_ptr(), sin.data_ptr(), B, L, H, hd, cos.shape[-1], rs, ys,
                       inverse, _stream()), "rope")
    _count()
    return y


def apply_rope(x, cos, sin):
    if not _is_bf16(x) or x.shape[-1] % 8 or cos.shape[-1] % 16:
        return ref.apply_rope(x, cos, sin)
    return _Rope.apply(x, cos.float().contiguous(), sin.float().contiguous())


# ----------------------------------------------------------------------------- attention




# ----------------------------------------------------------------------------- cross entropy


class _CrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, labels):
        lib = require()
        V = logits.shape[-1]
        l2 = logits.reshape(-1, V).contiguous()
        lab = labels.reshape(-1).contiguous()
        T = l2.shape[0]
        loss = _alloc(T, dtype=torch.float32, device=logits.device)
        lse = _alloc(T, dtype=torch.float32, device=logits.device)
        _check(lib.sb_ce_fwd(l2.data_ptr(), lab.data_ptr(), loss.data_ptr(), lse.data_ptr(), T, V, _stream()), "ce_fwd")
        _count()
        ctx.save_for_backward(l2, lab, lse)
        ctx.shape = logits.shape
        return loss.view(labels.shape)

    @staticmethod
    def backward(ctx, g):
        lib = require()
        l2, lab, lse = ctx.saved_tensors
        T, V = l2.shape
        gc = g.reshape(-1).float().contiguous()
        dl = _alloc_like(l2)
        _check(lib.sb_ce_bwd(l2.data_ptr(), lab.data_ptr(), lse.data_ptr(), gc.data_ptr(), dl.data_ptr(), T, V, _stream()),
               "ce_bwd")
        _count()
        return dl.view(ctx.shape), None


def cross_entropy(logits, labels):
    if not _is_bf16(logits) or logits.shape[-1] % 8 or labels.dtype != torch.int64:
        return ref.cross_entropy(logits, labels)
    return _CrossEntropy.apply(logits, labels)


# ----------------------------------------------------------------------------- optimizer pieces


def sq_norm(x, weight=None):
    if x.dtype not in (bf16, torch.float32) or not x.is_contiguous():
        xf = x.float()
        return (xf * xf * weight).sum() if weight is not None else (xf * xf).sum()
    lib = require()
    out = _zeros((), dtype=torch.float32, device=x.device)
    _check(lib.sb_sqnorm(x.data_ptr(), _ptr(weight), out.data_ptr(), x.numel(), int(x.dtype == bf16), _stream()), "sqnorm")
    _count()
    return out


def adam_step(master, exp_avg, exp_avg_sq, grad, lr, beta1, beta2, eps, weight_decay, step, adamw=True, grad_scale=1.0,
              param_out=None):
    ok = (master.dtype == torch.float32 and grad.dtype in (bf16, torch.float32) and grad.is_contiguous()
          and (param_out is None or param_out.dtype == bf16))
    if not ok:
        return ref.adam_step(master, exp_avg, exp_avg_sq, grad, lr, beta1, beta2, eps, weight_decay, step, adamw,
                             grad_scale, param_out)
    lib = require()
    if isinstance(grad_scale, torch.Tensor):
        sp, sh = grad_scale.float().reshape(1), 1.0
    else:
        sp, sh = None, float(grad_scale)
    bc1, bc2 = 1.0 - beta1 ** step, 1.0 - beta2 ** step
    _check(lib.sb_adam(master.data_ptr(), exp_avg.data_ptr(), exp_avg_sq.data_ptr(), grad.data_ptr(), _ptr(param_out),
                       master.numel(), lr, beta1, beta2, eps, weight_decay, bc1, bc2, int(adamw), _ptr(sp), sh,
                       int(grad.dtype == bf16), _stream()), "adam")
    _count()


# ----------------------------------------------------------------------------- short convolutions


def _f32c(t):
    return t.detach().float().contiguous()


class _DwConv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, halo):
        lib = require()
        B, L, C = x.shape
        K = w.shape[-1]
        xc = x.contiguous()
        hc = halo.contiguous() if halo is not None else None
        wf = _f32c(w)
        y = _alloc_like(xc)
        _check(lib.sb_dwconv_fwd(xc.data_ptr(), _ptr(hc), wf.data_ptr(), y.data_ptr(), B, L, C, K, _stream()), "dwconv_fwd")
        _count()
        ctx.save_for_backward(xc, wf, hc if hc is not None else _alloc(0, device=x.device))
        ctx.meta = (halo is not None, w.dtype)
        return y

    @staticmethod
    def backward(ctx, gy):
        lib = require()
        xc, wf, hc = ctx.saved_tensors
        has_halo, wdtype = ctx.meta
        B, L, C = xc.shape
        K = wf.shape[-1]
        g = gy.contiguous()
        dx = _alloc_like(xc)
        dh = _alloc_like(hc) if has_halo else None
        dw = _zeros_like(wf)
        _check(lib.sb_dwconv_bwd(xc.data_ptr(), hc.data_ptr() if has_halo else None, wf.data_ptr(), g.data_ptr(),
                                 dx.data_ptr(), _ptr(dh), dw.data_ptr(), B, L, C, K, _stream()), "dwconv_bwd")
        _count()
        return dx, dw.to(wdtype), dh


def causal_conv1d(x, w, halo=None):
    K = w.shape[-1]
    if not _is_bf16(x, halo) or x.shape[-1] % 8 or not 2 <= K <= 8:
        return ref.causal_conv1d(x, w, halo)
    return _DwConv.apply(x, w, halo)


class _HyenaSE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, feat, w, halo, pregate, postgate):
        lib = require()
        B, L, C3 = feat.shape
        D = C3 // 3
        G, K = w.shape
        fc = feat.contiguous()
        hc = halo.contiguous() if halo is not None else None
        wf = _f32c(w)
        z = _alloc((B, L, D), dtype=bf16, device=feat.device)
        _check(lib.sb_se_fwd(fc.data_ptr(), _ptr(hc), wf.data_ptr(), z.data_ptr(), B, L, D, G, K, int(pregate),
                             int(postgate), _stream()), "se_fwd")
        _count()
        ctx.save_for_backward(fc, wf, hc if hc is not None else _alloc(0, device=feat.device))
        ctx.meta = (halo is not None, w.dtype, pregate, postgate)
        return z

    @staticmethod
    def backward(ctx, gz):
        lib = require()
        fc, wf, hc = ctx.saved_tensors
        has_halo, wdtype, pregate, postgate = ctx.meta
        B, L, C3 = fc.shape
        D = C3 // 3
        G, K = wf.shape
        g = gz.contiguous()
        df = _alloc_like(fc)
        dh = _alloc_like(hc) if has_halo else None
        dw = _zeros_like(wf)
        _check(lib.sb_se_bwd(fc.data_ptr(), hc.data_ptr() if has_halo else None, wf.data_ptr(), g.data_ptr(), df.data_ptr(),
                             _ptr(dh), dw.data_ptr(), B, L, D, G, K, int(pregate), int(postgate), _stream()), "se_bwd")
        _count()
        return df, dw.to(wdtype), dh, None, None


def hyena_se_inner(feat, w, halo=None, pregate=True, postgate=True):
    K = w.shape[-1]
    D = feat.shape[-1] // 3
    if not _is_bf16(feat, halo) or D % 8 or not 2 <= K <= 8:
        return ref.hyena_se_inner(feat, w, halo, pregate, postgate)
    return _HyenaSE.apply(feat, w, halo, pregate, postgate)


class _HyenaMR(torch.autograd.Function):
    """Tensor-core kernels (csrc/mr_conv_tc.cu) when a 16-channel slab shares one filter (dg % 16 == 0), else the
    CUDA-core kernels (csrc/mr_conv.cu)."""

    @staticmethod
    def forward(ctx, feat, h, bias, halo):
        lib = require()
        B, L, C3 = feat.shape
        D = C3 // 3
        G, K = h.shape
        fc = feat.contiguous()
        hc = halo.contiguous() if halo is not None else None
        hf, bf = _f32c(h), _f32c(bias)
        z = _alloc((B, L, D), dtype=bf16, device=feat.device)
        tc = (D // G) % 16 == 0 and D % 8 == 0
        y = None
        if tc:
            _check(lib.sb_mr_tc_fwd(fc.data_ptr(), _ptr(hc), hf.data_ptr(), bf.data_ptr(), z.data_ptr(), B, L, D, G, K,
                                    _stream()), "mr_tc_fwd")
        else:
            y = _alloc_like(z) if any(ctx.needs_input_grad) else None
            _check(lib.sb_mr_fwd(fc.data_ptr(), _ptr(hc), hf.data_ptr(), bf.data_ptr(), z.data_ptr(), _ptr(y), B, L, D, G, K,
                                 _stream()), "mr_fwd")
        _count()
        empty = _alloc(0, device=feat.device)
        ctx.save_for_backward(fc, hf, bf, y if y is not None else empty, hc if hc is not None else empty)
        ctx.meta = (halo is not None, h.dtype, bias.dtype, tc)
        return z

    @staticmethod
    def backward(ctx, gz):
        lib = require()
        fc, hf, bf, y, hc = ctx.saved_tensors
        has_halo, hdtype, bdtype, tc = ctx.meta
        B, L, C3 = fc.shape
        D = C3 // 3
        G, K = hf.shape
        g = gz.contiguous()
        df = _alloc_like(fc)
        dhalo = _zeros_like(hc) if has_halo else None
        dh = _zeros_like(hf)
        db = _zeros_like(bf)
        hp = hc.data_ptr() if has_halo else None
        if tc:
            _check(lib.sb_mr_tc_bwd(fc.data_ptr(), hp, hf.data_ptr(), bf.data_ptr(), g.data_ptr(), df.data_ptr(), _ptr(dhalo),
                                    dh.data_ptr(), db.data_ptr(), B, L, D, G, K, _stream()), "mr_tc_bwd")
            _count()
        else:
            _check(lib.sb_mr_bwd(fc.data_ptr(), hp, hf.data_ptr(), bf.data_ptr(), g.data_ptr(), y.data_ptr(), df.data_ptr(),
                                 _ptr(dhalo), dh.data_ptr(), db.data_ptr(), B, L, D, G, K, _stream()), "mr_bwd")
            _count(2)
        return df, dh.to(hdtype), db.to(bdtype), dhalo


def hyena_mr_inner(feat, h, bias, halo=None):
    G, K = h.shape
    D = feat.shape[-1] // 3
    dg = D // G
    if not _is_bf16(feat, halo) or K > 128 or D % G or ((64 % dg) and (dg % 64)):
        return ref.hyena_mr_inner(feat, h, bias, halo)
    return _HyenaMR.apply(feat, h, bias, halo)


# ----------------------------------------------------------------------------- Hyena-LI (modal scan)

LI_ORDER = 16


LI_CHUNK_OVERRIDE = None      # tests set this to exercise a chunk length that their small shapes would not select
LI_TILED = True


def set_li_variant(tiled: bool) -> None:
    """True (default): shared-memory tiled scan kernels; False: the per-thread streaming kernels (A/B measurements, tests)."""
    global LI_TILED
    LI_TILED = bool(tiled)
    require().sb_li_set_variant(int(LI_TILED))


def _li_chunk(B: int, L: int, D: int) -> int:
    """Chunk length of the scan: as long as possible (the pass over the chunk states is serial in the number of
    chunks) while the chunk grid still oversubscribes the GPU (>= 2048 blocks of 128 channels; with fewer blocks the
    chunk kernels lose more than the shorter chunk-state pass gains: 0.37 ms against 0.28 ms forward at L = 8192)."""
    if LI_CHUNK_OVERRIDE:
        return int(LI_CHUNK_OVERRIDE)
    tc = 1024
    while tc > 128 and B * ((D + 127) // 128) * ((L + tc - 1) // tc) < 2048:
        tc //= 2
    return tc


def _pad_order(t, fill):
    D, O = t.shape
    if O == LI_ORDER:
        return t.contiguous()
    out = torch.full((D, LI_ORDER), fill, dtype=torch.float32, device=t.device)
    out[:, :O] = t
    return out


class _HyenaLI(torch.autograd.Function):
    @staticmethod
    def forward(ctx, feat, gamma, R, p, bias, state_in, want_state):
        lib = require()
        B, L, C3 = feat.shape
        D = C3 // 3
        O = gamma.shape[1]
        fc = feat.contiguous()
        loglam = -torch.exp(p.detach().float()) * torch.exp(gamma.detach().float())
        ll = _pad_order(loglam, -1.0e30)
        Rp = _pad_order(R.detach().float(), 0.0)
        bf = _f32c(bias)
        sin = None
        if state_in is not None:
            sin = _zeros((B, D, LI_ORDER), dtype=torch.float32, device=feat.device)
            sin[..., :O] = state_in.detach().float()
        tc = _li_chunk(B, L, D)
        NC = (L + tc - 1) // tc
        S = _alloc((B, NC, D, LI_ORDER), dtype=torch.float32, device=feat.device)
        sout = _alloc((B, D, LI_ORDER), dtype=torch.float32, device=feat.device) if want_state else None
        z = _alloc((B, L, D), dtype=bf16, device=feat.device)
        _check(lib.sb_li_fwd(fc.data_ptr(), ll.data_ptr(), Rp.data_ptr(), bf.data_ptr(), _ptr(sin), _ptr(sout), S.data_ptr(),
                             z.data_ptr(), B, L, D, tc, _stream()), "li_fwd")
        _count(3)
        ctx.save_for_backward(fc, ll, Rp, bf, sin if sin is not None else _alloc(0, device=feat.device))
        ctx.meta = (O, state_in is not None, gamma.dtype, R.dtype, p.dtype, bias.dtype, want_state)
        if want_state:
            return z, sout[..., :O].contiguous()
        return z, None

    @staticmethod
    def backward(ctx, gz, gstate):
        lib = require()
        fc, ll, Rp, bf, sin = ctx.saved_tensors
        O, has_sin, gdt, rdt, pdt, bdt, want_state = ctx.meta
        B, L, C3 = fc.shape
        D = C3 // 3
        dev = fc.device
        # the shared-memory tiled backward keeps a whole chunk on chip and fixes the chunk length itself
        tc_fwd = _li_chunk(B, L, D)
        tc = int(lib.sb_li_bwd_chunk(D, tc_fwd))
        NC = (L + tc - 1) // tc
        g = gz.contiguous()
        shape = (B, NC, D, LI_ORDER)
        S, W, A, dRp, dLp = (_alloc(shape, dtype=torch.float32, device=dev) for _ in range(5))
        dBp = _alloc((B, NC, D), dtype=torch.float32, device=dev)
        tiled = tc != tc_fwd
        tmp = None if tiled else _alloc((B, L, D), dtype=bf16, device=dev)     # dx1 round trip of the streaming kernels only
        df = _alloc_like(fc)
        dso = None
        if want_state and gstate is not None:
            dso = _zeros((B, D, LI_ORDER), dtype=torch.float32, device=dev)
            dso[..., :O] = gstate.float()
        w_end = _alloc((B, D, LI_ORDER), dtype=torch.float32, device=dev) if dso is not None else None
        dsi = _alloc((B, D, LI_ORDER), dtype=torch.float32, device=dev) if has_sin else None
        _check(lib.sb_li_bwd(fc.data_ptr(), g.data_ptr(), ll.data_ptr(), Rp.data_ptr(), bf.data_ptr(),
                             sin.data_ptr() if has_sin else None, _ptr(dso), S.data_ptr(), W.data_ptr(), A.data_ptr(),
                             dRp.data_ptr(), dLp.data_ptr(), dBp.data_ptr(), _ptr(tmp), df.data_ptr(), _ptr(w_end),
                             _ptr(dsi), B, L, D, tc, _stream()), "li_bwd")
        _count(4)
        dR = dRp.sum((0, 1))[:, :O]
        dlam = dLp.sum((0, 1))
        if dso is not None:
            dlam = dlam + (dso * w_end).sum(0)
        lam = torch.exp(ll)
        dll = (dlam * lam * ll)[:, :O]          # d/dp = d/dgamma = dloglam * loglam
        dll = torch.nan_to_num(dll, nan=0.0, posinf=0.0, neginf=0.0)
        db = dBp.sum((0, 1))
        return (df, dll.to(gdt), dR.to(rdt), dll.to(pdt), db.to(bdt), dsi[..., :O].contiguous() if has_sin else None, None)


def hyena_li_modal(feat, gamma, R, p, bias, state_in=None, return_state=False):
    if not _is_bf16(feat) or gamma.shape[1] > LI_ORDER:
        return ref.hyena_li_modal(feat, gamma, R, p, bias, state_in, return_state)
    z, s = _HyenaLI.apply(feat, gamma, R, p, bias, state_in, return_state)
    return (z, s) if return_state else z
