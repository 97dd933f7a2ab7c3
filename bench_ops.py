"""Operator benchmark and per-kernel roofline table: times this framework's CUDA kernels and, beside each, the
PyTorch/library statement of the same operator, on the Evo-2-7B shapes (hidden 4096, 256 groups of 16 channels, filter
lengths 3 / 7 / 128, modal order 16).

    python bench_ops.py [--seq 8192] [--ops gemm,dwconv,se,mr,li,norm,glu,ce,adam] [--iters 10]

Context-parallel operator sweep (one Hyena-MR block and one Hyena-LI block, batch 1, hidden 4096, forward and
backward, the sequence split over the GPUs of the job; N(0,1) activations, seeded filters):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 bench_ops.py --cp-sweep \
        [--seqs 8192,32768,131072,1048576]

  MR block = featuriser conv (k = 3) + gated FIR (k = 128), halo rows read from the neighbour ranks inside the kernels;
  LI block = featuriser conv + modal scan (order 16) with the all-to-all inside the scan kernels.
Every row is device-timed (CUDA events, max over ranks) and carries the achieved fraction of its roofline, the slower of
the algorithmic HBM bytes over the measured copy bandwidth and the bytes that must cross NVLink over 770 GB/s.

Timing: CUDA events on the launching stream, 3 warm-up launches, an L2 flush (a 256 MB buffer write)
between timed launches.  Rooflines use MEASURED_PEAKS.json (copy bandwidth, cuBLAS bf16 throughput) when
present, else the fallback figures 6.65 TB/s / 1.59 PFLOP/s.  One JSON line per measurement.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

from savanna_b200 import ops  # noqa: E402
from savanna_b200.ops import reference as ref  # noqa: E402
from savanna_b200.utils.mfu import measured_peaks  # noqa: E402

BF = torch.bfloat16


def peaks():
    m = measured_peaks() or {}
    return float(m.get("hbm_gbs", 6650.0)) * 1e9, float(m.get("bf16_tflops", 1590.0)) * 1e12, ("measured" if m else "fallback")


_FLUSH = None


def flush_l2():
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _FLUSH.zero_()


def timeit(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def report(name, ms, flops=None, bytes_=None, **kw):
    bw, tf, src = peaks()
    rec = {"op": name, "ms": round(ms, 4)}
    if flops:
        rec["tflops"] = round(flops / ms / 1e9, 1)
        rec["frac_of_gemm_peak"] = round(flops / (ms / 1e3) / tf, 3)
    if bytes_:
        rec["gbs"] = round(bytes_ / ms / 1e6, 1)
        rec["frac_of_copy_bw"] = round(bytes_ / (ms / 1e3) / bw, 3)
    rec["peaks"] = src
    rec.update(kw)
    print(json.dumps(rec), flush=True)


def bench_gemm(T, iters):
    from savanna_b200.ops import cuda_ops
    D, F = 4096, 11264
    shapes = [("in_proj", T, 3 * D, D), ("out_proj", T, D, D), ("mlp_w12", T, 2 * F, D), ("mlp_w3", T, D, F), ("logits", T, 512, D)]
    for name, M, N, K in shapes:
        x = torch.randn(M, K, device="cuda", dtype=BF)
        w = torch.randn(N, K, device="cuda", dtype=BF) * 0.02
        gy = torch.randn(M, N, device="cuda", dtype=BF)
        out = torch.empty(M, N, device="cuda", dtype=BF)
        gx, gw = torch.empty_like(x), torch.empty_like(w)
        fl = 2.0 * M * N * K
        cuda_ops.set_gemm_pair_mode(0)
        report(f"gemm.{name}.fwd.ours", timeit(lambda: cuda_ops.gemm(x, w, out), iters), fl, M=M, N=N, K=K)
        report(f"gemm.{name}.fwd.cublas", timeit(lambda: torch.matmul(x, w.t(), out=out), iters), fl)
        report(f"gemm.{name}.dgrad.ours", timeit(lambda: cuda_ops.gemm(gy, w, gx, b_mn=True), iters), fl)
        report(f"gemm.{name}.dgrad.cublas", timeit(lambda: torch.matmul(gy, w, out=gx), iters), fl)
        report(f"gemm.{name}.wgrad.ours", timeit(lambda: cuda_ops.gemm(gy, x, gw, a_mn=True, b_mn=True), iters), fl)
        report(f"gemm.{name}.wgrad.cublas", timeit(lambda: torch.matmul(gy.t(), x, out=gw), iters), fl)
        # fp8 operands (quantisation excluded: it is timed separately below)
        xq, sx = cuda_ops.quantize_fp8(x, 0); wq, sw = cuda_ops.quantize_fp8(w, 0); gq, sg = cuda_ops.quantize_fp8(gy, 1)
        al = sx * sw
        report(f"gemm.{name}.fwd.ours_fp8", timeit(lambda: cuda_ops.gemm_fp8(xq, wq, out, al), iters), fl)
        report(f"gemm.{name}.dgrad.ours_fp8", timeit(lambda: cuda_ops.gemm_fp8(gq, wq, gx, al, b_mn=True, a_fmt=1), iters), fl)
        report(f"gemm.{name}.wgrad.ours_fp8", timeit(lambda: cuda_ops.gemm_fp8(gq, xq, gw, al, a_mn=True, b_mn=True, a_fmt=1), iters), fl)
        cuda_ops.set_gemm_pair_mode(2)
        report(f"gemm.{name}.fwd.ours_pair", timeit(lambda: cuda_ops.gemm(x, w, out), iters), fl)
        report(f"gemm.{name}.dgrad.ours_pair", timeit(lambda: cuda_ops.gemm(gy, w, gx, b_mn=True), iters), fl)
        report(f"gemm.{name}.wgrad.ours_pair", timeit(lambda: cuda_ops.gemm(gy, x, gw, a_mn=True, b_mn=True), iters), fl)
        report(f"gemm.{name}.fwd.ours_fp8_pair", timeit(lambda: cuda_ops.gemm_fp8(xq, wq, out, al), iters), fl)
        report(f"gemm.{name}.dgrad.ours_fp8_pair", timeit(lambda: cuda_ops.gemm_fp8(gq, wq, gx, al, b_mn=True, a_fmt=1), iters), fl)
        report(f"gemm.{name}.wgrad.ours_fp8_pair", timeit(lambda: cuda_ops.gemm_fp8(gq, xq, gw, al, a_mn=True, b_mn=True, a_fmt=1), iters), fl)
        if N % 32 == 0 and K % 32 == 0 and M % 32 == 0:
            # block-scaled fp8: the three products of a projection on operands quantised along their own contraction
            xm, sxm = cuda_ops.mx_quantize(x); wm, swm = cuda_ops.mx_quantize(w); gm, sgm = cuda_ops.mx_quantize(gy)
            wtm, swtm = cuda_ops.mx_quantize(w, True); xtm, sxtm = cuda_ops.mx_quantize(x, True); gtm, sgtm = cuda_ops.mx_quantize(gy, True)
            report(f"gemm.{name}.fwd.ours_mxfp8", timeit(lambda: cuda_ops.gemm_mx(xm, sxm, wm, swm, out), iters), fl)
            report(f"gemm.{name}.dgrad.ours_mxfp8", timeit(lambda: cuda_ops.gemm_mx(gm, sgm, wtm, swtm, gx), iters), fl)
            report(f"gemm.{name}.wgrad.ours_mxfp8", timeit(lambda: cuda_ops.gemm_mx(gtm, sgtm, xtm, sxtm, gw), iters), fl)
            report(f"quantize_mxfp8.{name}.x.rowwise", timeit(lambda: cuda_ops.mx_quantize(x), iters), None, M * K * 3)
            report(f"quantize_mxfp8.{name}.x.transposed", timeit(lambda: cuda_ops.mx_quantize(x, True), iters), None, M * K * 3)
        report(f"quantize_fp8.{name}.x.current", timeit(lambda: cuda_ops.quantize_fp8(x, 0), iters), None, M * K * 5)
        site = torch.nn.Parameter(torch.zeros(1, device=x.device))
        report(f"quantize_fp8.{name}.x.delayed", timeit(lambda: cuda_ops.quantize_fp8_site(x, 0, site, "x"), iters), None, M * K * 3)
        cuda_ops.check_status()


def _fwd_bwd(fn, inputs, iters):
    outs = fn(*inputs)
    out = outs[0] if isinstance(outs, tuple) else outs
    g = torch.randn_like(out)
    f_ms = timeit(lambda: fn(*inputs), iters)

    def fb():
        for t in inputs:
            if isinstance(t, torch.Tensor) and t.grad is not None:
                t.grad = None
        o = fn(*inputs)
        o = o[0] if isinstance(o, tuple) else o
        o.backward(g)
    fb_ms = timeit(fb, iters)
    return f_ms, fb_ms - f_ms


FWD_TILED_DEFAULT = True
TILED_DEFAULT = True      # which short-convolution backward variant the library starts with


def bench_convs(L, iters, which):
    from savanna_b200.ops import cuda_ops
    D, G = 4096, 256
    B = 1
    feat = torch.randn(B, L, 3 * D, device="cuda", dtype=BF, requires_grad=True)
    proj = torch.randn(B, L, 3 * D, device="cuda", dtype=BF, requires_grad=True)
    nb = B * L * D * 2
    for backend in ("auto", "torch"):
        ops.set_backend(backend)
        tag = "ours" if backend == "auto" else "torch"
        if backend == "torch" and L > 32768:
            continue
        if "dwconv" in which:
            w = torch.randn(3 * D, 3, device="cuda", requires_grad=True)
            f, b = _fwd_bwd(lambda x, w_: ops.causal_conv1d(x, w_), (proj, w), iters)
            report(f"featurizer_conv3.fwd.{tag}", f, None, 6 * nb, L=L)
            report(f"featurizer_conv3.bwd.{tag}", b, None, 9 * nb, L=L)
            if backend == "auto":
                cuda_ops.set_conv_forward_variant(not FWD_TILED_DEFAULT)
                f2, _ = _fwd_bwd(lambda x, w_: ops.causal_conv1d(x, w_), (proj, w), iters)
                report("featurizer_conv3.fwd.ours_other_variant", f2, None, 6 * nb, L=L, tiled=not FWD_TILED_DEFAULT)
                cuda_ops.set_conv_forward_variant(FWD_TILED_DEFAULT)
                cuda_ops.set_se_backward_variant(not TILED_DEFAULT)
                _, b2 = _fwd_bwd(lambda x, w_: ops.causal_conv1d(x, w_), (proj, w), iters)
                report("featurizer_conv3.bwd.ours_other_variant", b2, None, 9 * nb, L=L, tiled=not TILED_DEFAULT)
                cuda_ops.set_se_backward_variant(TILED_DEFAULT)
        if "se" in which:
            w = torch.randn(G, 7, device="cuda", requires_grad=True)
            f, b = _fwd_bwd(lambda x, w_: ops.hyena_se_inner(x, w_), (feat, w), iters)
            report(f"hyena_se_k7.fwd.{tag}", f, None, 4 * nb, L=L)
            report(f"hyena_se_k7.bwd.{tag}", b, None, 7 * nb, L=L)
            if backend == "auto":
                cuda_ops.set_conv_forward_variant(not FWD_TILED_DEFAULT)
                f2, _ = _fwd_bwd(lambda x, w_: ops.hyena_se_inner(x, w_), (feat, w), iters)
                report("hyena_se_k7.fwd.ours_other_variant", f2, None, 4 * nb, L=L, tiled=not FWD_TILED_DEFAULT)
                cuda_ops.set_conv_forward_variant(FWD_TILED_DEFAULT)
                cuda_ops.set_se_backward_variant(not TILED_DEFAULT)
                _, b2 = _fwd_bwd(lambda x, w_: ops.hyena_se_inner(x, w_), (feat, w), iters)
                report("hyena_se_k7.bwd.ours_other_variant", b2, None, 7 * nb, L=L, tiled=not TILED_DEFAULT)
                cuda_ops.set_se_backward_variant(TILED_DEFAULT)
        if "mr" in which:
            h = (torch.randn(G, 128, device="cuda") / 11.3).requires_grad_()
            bias = torch.randn(D, device="cuda", requires_grad=True)
            f, b = _fwd_bwd(lambda x, h_, b_: ops.hyena_mr_inner(x, h_, b_), (feat, h, bias), iters)
            fl = 2.0 * 128 * B * L * D
            report(f"hyena_mr_k128.fwd.{tag}", f, fl, 4 * nb, L=L)
            report(f"hyena_mr_k128.bwd.{tag}", b, 2 * fl, 8 * nb, L=L)
        if "li" in which:
            O = 16
            gamma = (torch.rand(D, O, device="cuda") * 0.09 + 0.01).log().requires_grad_()
            R = (0.1 * torch.randn(D, O, device="cuda") / 4).requires_grad_()
            p = (-torch.ones(D, O, device="cuda")).requires_grad_()
            bias = torch.randn(D, device="cuda", requires_grad=True)
            f, b = _fwd_bwd(lambda x, g_, r_, p_, b_: ops.hyena_li_modal(x, g_, r_, p_, b_), (feat, gamma, R, p, bias), iters)
            report(f"hyena_li_modal16.fwd.{tag}", f, None, 7 * nb, L=L)
            report(f"hyena_li_modal16.bwd.{tag}", b, None, 17 * nb, L=L)
    ops.set_backend("auto")


def bench_elementwise(T, iters, which):
    D, F = 4096, 11264
    for backend in ("auto", "torch"):
        ops.set_backend(backend)
        tag = "ours" if backend == "auto" else "torch"
        if "norm" in which:
            x = torch.randn(T, D, device="cuda", dtype=BF, requires_grad=True)
            w = torch.ones(D, device="cuda", dtype=BF, requires_grad=True)
            f, b = _fwd_bwd(lambda x_, w_: ops.rmsnorm(x_, w_, 1e-6, "te"), (x, w), iters)
            report(f"rmsnorm.fwd.{tag}", f, None, 2 * T * D * 2)
            report(f"rmsnorm.bwd.{tag}", b, None, 3 * T * D * 2)
        if "glu" in which:
            ab = torch.randn(T, 2 * F, device="cuda", dtype=BF, requires_grad=True)
            f, b = _fwd_bwd(lambda t: ops.glu_act_packed(t, "silu"), (ab,), iters)
            report(f"swiglu.fwd.{tag}", f, None, 3 * T * F * 2)
            report(f"swiglu.bwd.{tag}", b, None, 5 * T * F * 2)
        if "ce" in which:
            lg = torch.randn(T, 512, device="cuda", dtype=BF, requires_grad=True)
            lab = torch.randint(0, 512, (T,), device="cuda")
            f, b = _fwd_bwd(lambda t: ops.cross_entropy(t, lab), (lg,), iters)
            report(f"cross_entropy.fwd.{tag}", f, None, T * 512 * 2)
            report(f"cross_entropy.bwd.{tag}", b, None, 2 * T * 512 * 2)
    ops.set_backend("auto")
    if "adam" in which:
        n = 256 * 1024 * 1024
        master, m, v = (torch.zeros(n, device="cuda") for _ in range(3))
        g = torch.randn(n, device="cuda", dtype=BF)
        p = torch.empty(n, device="cuda", dtype=BF)
        ms = timeit(lambda: ops.adam_step(master, m, v, g, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1, True, 1.0, p), iters)
        report("adam.ours", ms, None, n * 28, n=n)


def cuda_ops_status():
    from savanna_b200.ops import cuda_ops
    cuda_ops.check_status()


def bench_attention(L, iters, heads=32, small=False):
    """Causal attention of one 7B layer (32 heads x 128): this framework's tcgen05 kernels and the flash kernels that
    ship with PyTorch (library baseline).  FLOPs: 4 L^2 hd H / 2 forward, 2.5x that backward."""
    from savanna_b200.ops import attention_cuda, flash_sm100
    B, H, hd = 1, heads, 128
    qkv = torch.randn(B, L, 3, H, hd, device="cuda", dtype=BF)
    q, k, v = (qkv[:, :, i].detach().requires_grad_() for i in range(3))
    fl = 4.0 * L * L * hd * H / 2 * B
    o, lse = flash_sm100.forward(q, k, v, True, hd ** -0.5)
    go = torch.randn_like(o)
    report("attention.fwd.ours", timeit(lambda: flash_sm100.forward(q, k, v, True, hd ** -0.5), iters), fl, L=L, H=H)
    qn, kn, vn = (torch.randn(B, L, H, hd, device="cuda", dtype=BF) for _ in range(3))
    report("attention.fwd.ours_noncausal", timeit(lambda: flash_sm100.forward(qn, kn, vn, False, hd ** -0.5), iters), 2 * fl)
    flash_sm100.set_forward_variant(True)
    report("attention.fwd.ours_pingpong", timeit(lambda: flash_sm100.forward(q, k, v, True, hd ** -0.5), iters), fl)
    report("attention.fwd.ours_pingpong_noncausal", timeit(lambda: flash_sm100.forward(qn, kn, vn, False, hd ** -0.5), iters), 2 * fl)
    flash_sm100.set_forward_variant(False)
    flash_sm100.set_forward_p_in_tmem(False)
    report("attention.fwd.ours_p_in_smem", timeit(lambda: flash_sm100.forward(q, k, v, True, hd ** -0.5), iters), fl)
    report("attention.fwd.ours_p_in_smem_noncausal", timeit(lambda: flash_sm100.forward(qn, kn, vn, False, hd ** -0.5), iters), 2 * fl)
    flash_sm100.set_forward_p_in_tmem(True)
    cuda_ops_status()
    report("attention.bwd.ours", timeit(lambda: flash_sm100.backward(go, q, k, v, o, lse, True, hd ** -0.5), iters), 2.5 * fl)
    flash_sm100.set_backward_variant(False)
    report("attention.bwd.ours_p_in_smem", timeit(lambda: flash_sm100.backward(go, q, k, v, o, lse, True, hd ** -0.5), iters), 2.5 * fl)
    flash_sm100.set_backward_variant(True)
    if small:
        return

    def lib_fwd():
        return attention_cuda._SdpaWithLse.apply(q, k, v, True)
    report("attention.fwd.torch_flash", timeit(lib_fwd, iters), fl)
    o2, _ = lib_fwd()
    fwd_ms = timeit(lib_fwd, iters)

    def lib_fb():
        oo, _ = lib_fwd()
        oo.backward(go)
        q.grad = k.grad = v.grad = None
    report("attention.bwd.torch_flash", timeit(lib_fb, iters) - fwd_ms, 2.5 * fl)
    import torch.nn.functional as F
    qt, kt, vt = (t.detach().transpose(1, 2).requires_grad_() for t in (q, k, v))
    sd = lambda: F.scaled_dot_product_attention(qt, kt, vt, is_causal=True)
    sd_f = timeit(sd, iters)
    report("attention.fwd.torch_sdpa", sd_f, fl)

    def sd_fb():
        sd().backward(go.transpose(1, 2))
        qt.grad = kt.grad = vt.grad = None
    report("attention.bwd.torch_sdpa", timeit(sd_fb, iters) - sd_f, 2.5 * fl)
    from savanna_b200.ops import cuda_ops
    cuda_ops.check_status()


NVLINK_BW = 770e9          # measured peer-copy bandwidth per direction per GPU on this pool (nominal 900e9)


def cp_sweep(seqs, iters):
    """One Hyena-MR block and one Hyena-LI block under context parallelism over all ranks of the job."""
    import torch.distributed as dist
    from savanna_b200.parallel import halo, halo_fused, li_fused, state
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dev = torch.device("cuda", torch.cuda.current_device())
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        state.initialize_model_parallel(1, world, 1)
        if not halo.setup_peer():
            raise RuntimeError("context-parallel peer workspace did not come up")
    D, G, O = 4096, 256, 16
    bw, _, src = peaks()
    torch.manual_seed(1234)
    w3 = torch.randn(3 * D, 3, device=dev, requires_grad=True)
    h = (torch.randn(G, 128, device=dev) / 11.3 * torch.exp(-torch.linspace(0, 4, 128, device=dev))).requires_grad_()
    bias = torch.randn(D, device=dev, requires_grad=True)
    d = D // world
    sl = slice(rank * d, (rank + 1) * d)
    gamma = (torch.rand(D, O, device=dev) * 0.09 + 0.01).log()
    Rm = 0.1 * torch.randn(D, O, device=dev) / 4
    pm = -torch.ones(D, O, device=dev)
    gam_l, R_l, p_l, b_l = (t[sl].clone().requires_grad_() for t in (gamma, Rm, pm, bias.detach()))

    def mr_block(x):
        if world > 1:
            f = halo_fused.causal_conv1d_cp(x, w3)
            return halo_fused.hyena_mr_inner_cp(f, h, bias)
        return ops.hyena_mr_inner(ops.causal_conv1d(x, w3), h, bias)

    def li_block(x):
        if world > 1:
            f = halo_fused.causal_conv1d_cp(x, w3)
            return li_fused.hyena_li_modal_cp(f, gam_l, R_l, p_l, b_l)
        return ops.hyena_li_modal(ops.causal_conv1d(x, w3), gam_l, R_l, p_l, b_l)

    def timed(fn):
        ms = timeit(fn, iters)
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for L in seqs:
        l = L // world
        if L % (2 * world) or (l // 2) % 64:
            continue
        need = l * 3 * D * 2 * 14                     # rough per-rank working set of a forward + backward, bytes
        if need > 150e9:
            if rank == 0:
                print(json.dumps({"op": "skipped", "L": L, "cp": world, "why": "working set exceeds the GPU's memory"}), flush=True)
            continue
        torch.manual_seed(99 + rank)
        x = torch.randn(1, l, 3 * D, device=dev, dtype=BF, requires_grad=True)
        tok = l * D * 2                               # bytes of one [l, D] bf16 tensor on this rank
        for name, blk, hbm_f, hbm_b, nv_f, nv_b in (
                # MR: conv reads/writes 3D each way; FIR reads 3D writes D (+ bwd: reads 3D + D, writes 3D).  Halo rows only.
                ("hyena_mr_block", mr_block, (6 + 4) * tok, (9 + 7) * tok, 0.0, 0.0),
                # LI: conv; gate u (3D in, D out); scan pulls u and stores y (each D over NVLink, share (cp-1)/cp); gate z
                ("hyena_li_block", li_block, (6 + 4 + 4 + 5) * tok, (9 + 5 + 8 + 9) * tok,
                 2 * tok * (world - 1) / world, 3 * tok * (world - 1) / world)):
            out = blk(x)
            g = torch.randn_like(out)
            f_ms = timed(lambda: blk(x))

            def fb():
                for t in (x, w3, h, bias, gam_l, R_l, p_l, b_l):
                    t.grad = None
                blk(x).backward(g)
            b_ms = timed(fb) - f_ms
            if rank == 0:
                for tag, ms, hb, nb in (("fwd", f_ms, hbm_f, nv_f), ("bwd", b_ms, hbm_b, nv_b)):
                    t_hbm, t_nv = hb / bw, nb / NVLINK_BW
                    roof = max(t_hbm, t_nv)
                    print(json.dumps({"op": f"{name}.{tag}", "L": L, "cp": world, "tokens_per_gpu": l, "ms": round(ms, 3),
                                      "roofline_ms": round(roof * 1e3, 3), "bound": "nvlink" if t_nv > t_hbm else "hbm",
                                      "frac_of_roofline": round(roof * 1e3 / ms, 3), "hbm_bytes": hb, "nvlink_bytes": nb,
                                      "peaks": src}), flush=True)
            del out, g
        del x
        torch.cuda.empty_cache()
    from savanna_b200.ops import cuda_ops
    torch.cuda.synchronize()
    cuda_ops.check_status()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--cp-sweep", action="store_true", help="context-parallel operator sweep over the ranks of the job")
    ap.add_argument("--seqs", type=str, default="8192,32768,131072,1048576")
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--ops", type=str, default="gemm,dwconv,se,mr,li,norm,glu,ce,adam,attention")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--own-only", action="store_true", help="attention: time only this framework's kernels")
    a = ap.parse_args()
    if a.cp_sweep:
        return cp_sweep([int(v) for v in a.seqs.split(",")], a.iters)
    which = set(a.ops.split(","))
    torch.cuda.set_device(0)
    if "gemm" in which:
        bench_gemm(a.seq, a.iters)
    if which & {"dwconv", "se", "mr", "li"}:
        bench_convs(a.seq, a.iters, which)
    if which & {"norm", "glu", "ce", "adam"}:
        bench_elementwise(a.seq, a.iters, which)
    if "attention" in which:
        bench_attention(a.seq, a.iters, a.heads, a.own_only)


if __name__ == "__main__":
    main()
