"""Context-parallel convolution kernels that read the neighbouring chunks' edge rows in place (csrc/conv.cu `*_cp`,
csrc/mr_conv_tc.cu `*_cp`), checked on ONE GPU: the `cp` ranks are emulated as separate calls whose "peer" staging
buffers are ordinary tensors of the same device (the kernels only dereference the pointers they are given).  The full
sequence is cut into 2*cp zigzag chunks; every virtual rank runs the kernel on its two chunks with the staged tails /
heads of its neighbours; outputs and gradients, re-assembled, must equal the fp32 PyTorch statement of the operator on
the whole sequence (ops/reference.py + autograd)."""
import ctypes

import pytest
import torch

from savanna_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF = torch.bfloat16


class _WS:
    def __init__(self):
        from savanna_b200.ops import cuda_ops
        self.lib = cuda_ops.require()


def _chunks(cp, r):
    return r, 2 * cp - 1 - r


def _shard(full, cp, r):
    """[B, Lfull, W] -> this virtual rank's two zigzag chunks back to back [B, 2c, W]."""
    c = full.shape[1] // (2 * cp)
    a, b = _chunks(cp, r)
    return torch.cat([full[:, a * c:(a + 1) * c], full[:, b * c:(b + 1) * c]], dim=1).contiguous()


def _unshard(parts, cp):
    c = parts[0].shape[1] // 2
    out = [None] * (2 * cp)
    for r, p in enumerate(parts):
        a, b = _chunks(cp, r)
        out[a], out[b] = p[:, :c], p[:, c:]
    return torch.cat(out, dim=1)


def _stage(x, H, heads):
    B, L, W = x.shape
    half = L // 2
    s = torch.empty((B, 2, H, W), dtype=x.dtype, device=x.device)
    if heads:
        s[:, 0], s[:, 1] = x[:, :H], x[:, half:half + H]
    else:
        s[:, 0], s[:, 1] = x[:, half - H:half], x[:, L - H:]
    return s


def _close(a, b, tol, what):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    bound = tol * (1.0 + b.abs())
    assert bool((err <= bound).all()), f"{what}: max excess {(err - bound).max().item():.4g} (max err {err.max().item():.4g})"


def _rel(a, b, tol, what):
    r = (a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-12)
    assert r <= tol, f"{what}: relative L2 error {r.item():.4g} > {tol}"


def _ptrs(bufs):
    return [b.data_ptr() for b in bufs]


@pytest.mark.parametrize("cp", [2, 3])
@pytest.mark.parametrize("K", [3, 4])
def test_dwconv_cp_matches_full_sequence(cp, K):
    from savanna_b200.parallel import halo_fused as hf
    lib = hf._lib(_WS())
    torch.manual_seed(0)
    B, C, c = 2, 192, 160
    L = 2 * cp * c
    x = torch.randn(B, L, C, device=DEV, dtype=BF)
    w = (torch.randn(C, K, device=DEV) * 0.5)
    gy = torch.randn(B, L, C, device=DEV, dtype=BF)
    xr = x.float().requires_grad_()
    wr = w.clone().requires_grad_()
    y_ref = ref.causal_conv1d(xr, wr)
    y_ref.backward(gy.float())
    xs = [_shard(x, cp, r) for r in range(cp)]
    gs = [_shard(gy, cp, r) for r in range(cp)]
    tails = [_stage(s, K - 1, False) for s in xs]
    heads = [_stage(g, K - 1, True) for g in gs]
    st = torch.cuda.current_stream().cuda_stream
    ys, dxs, dw = [], [], torch.zeros_like(w)
    for r in range(cp):
        y = torch.full_like(xs[r], float("nan"))
        before = hf.before_src(_ptrs(tails), r, cp)
        assert lib.sb_dwconv_fwd_cp(xs[r].data_ptr(), ctypes.byref(before), w.data_ptr(), y.data_ptr(), 2 * B, c, C, K, st) == 0
        dx = torch.full_like(xs[r], float("nan"))
        ahead = hf.ahead_src(_ptrs(heads), r, cp)
        assert lib.sb_dwconv_bwd_cp(xs[r].data_ptr(), ctypes.byref(before), w.data_ptr(), gs[r].data_ptr(), ctypes.byref(ahead),
                                    dx.data_ptr(), dw.data_ptr(), 2 * B, c, C, K, st) == 0
        ys.append(y); dxs.append(dx)
    torch.cuda.synchronize()
    _close(_unshard(ys, cp), y_ref, 2e-2, "dwconv cp y")
    _close(_unshard(dxs, cp), xr.grad, 2e-2, "dwconv cp dx")
    _rel(dw, wr.grad, 1e-2, "dwconv cp dw")


@pytest.mark.parametrize("cp", [2, 3])
@pytest.mark.parametrize("gates", [(True, True), (False, True)])
def test_hyena_se_cp_matches_full_sequence(cp, gates):
    from savanna_b200.parallel import halo_fused as hf
    lib = hf._lib(_WS())
    torch.manual_seed(1)
    pre, post = gates
    B, D, G, K, c = 1, 128, 8, 7, 192
    L = 2 * cp * c
    feat = torch.randn(B, L, 3 * D, device=DEV, dtype=BF)
    w = torch.randn(G, K, device=DEV) * 0.4
    gz = torch.randn(B, L, D, device=DEV, dtype=BF)
    fr = feat.float().requires_grad_()
    wr = w.clone().requires_grad_()
    z_ref = ref.hyena_se_inner(fr, wr, None, pre, post)
    z_ref.backward(gz.float())
    fs = [_shard(feat, cp, r) for r in range(cp)]
    gs = [_shard(gz, cp, r) for r in range(cp)]
    tails = [_stage(f, K - 1, False) for f in fs]
    heads_f = [_stage(f, K - 1, True) for f in fs]
    heads_g = [_stage(g, K - 1, True) for g in gs]
    st = torch.cuda.current_stream().cuda_stream
    zs, dfs, dw = [], [], torch.zeros_like(w)
    for r in range(cp):
        z = torch.full((B, 2 * c, D), float("nan"), device=DEV, dtype=BF)
        before = hf.before_src(_ptrs(tails), r, cp)
        assert lib.sb_se_fwd_cp(fs[r].data_ptr(), ctypes.byref(before), w.data_ptr(), z.data_ptr(), 2 * B, c, D, G, K,
                                int(pre), int(post), st) == 0
        df = torch.full_like(fs[r], float("nan"))
        af, ag = hf.ahead_src(_ptrs(heads_f), r, cp), hf.ahead_src(_ptrs(heads_g), r, cp)
        assert lib.sb_se_bwd_cp(fs[r].data_ptr(), ctypes.byref(before), w.data_ptr(), gs[r].data_ptr(), ctypes.byref(af),
                                ctypes.byref(ag), df.data_ptr(), dw.data_ptr(), 2 * B, c, D, G, K, int(pre), int(post), st) == 0
        zs.append(z); dfs.append(df)
    torch.cuda.synchronize()
    _close(_unshard(zs, cp), z_ref, 3e-2, "se cp z")
    _close(_unshard(dfs, cp), fr.grad, 4e-2, "se cp dfeat")
    _rel(dw, wr.grad, 1e-2, "se cp dw")


@pytest.mark.parametrize("cp,K", [(2, 128), (3, 37)])
def test_hyena_mr_cp_matches_full_sequence(cp, K):
    from savanna_b200.parallel import halo_fused as hf
    lib = hf._lib(_WS())
    torch.manual_seed(2)
    B, D, G, c = 1, 128, 8, 256
    L = 2 * cp * c
    feat = torch.randn(B, L, 3 * D, device=DEV, dtype=BF)
    decay = torch.exp(-0.05 * torch.arange(K, device=DEV))
    h = torch.randn(G, K, device=DEV) * 0.3 * decay
    bias = torch.randn(D, device=DEV) * 0.5
    gz = torch.randn(B, L, D, device=DEV, dtype=BF)
    fr = feat.float().requires_grad_()
    hr, br = h.clone().requires_grad_(), bias.clone().requires_grad_()
    z_ref = ref.hyena_mr_inner(fr, hr, br)
    z_ref.backward(gz.float())
    fs = [_shard(feat, cp, r) for r in range(cp)]
    gs = [_shard(gz, cp, r) for r in range(cp)]
    tails = [_stage(f, K - 1, False) for f in fs]
    heads_f = [_stage(f, K - 1, True) for f in fs]
    heads_g = [_stage(g, K - 1, True) for g in gs]
    st = torch.cuda.current_stream().cuda_stream
    zs, dfs, dh, db = [], [], torch.zeros_like(h), torch.zeros_like(bias)
    for r in range(cp):
        z = torch.full((B, 2 * c, D), float("nan"), device=DEV, dtype=BF)
        before = hf.before_src(_ptrs(tails), r, cp)
        assert lib.sb_mr_tc_fwd_cp(fs[r].data_ptr(), ctypes.byref(before), h.data_ptr(), bias.data_ptr(), z.data_ptr(), 2 * B, c,
                                   D, G, K, st) == 0
        df = torch.full_like(fs[r], float("nan"))
        af, ag = hf.ahead_src(_ptrs(heads_f), r, cp), hf.ahead_src(_ptrs(heads_g), r, cp)
        assert lib.sb_mr_tc_bwd_cp(fs[r].data_ptr(), ctypes.byref(before), h.data_ptr(), bias.data_ptr(), gs[r].data_ptr(),
                                   ctypes.byref(af), ctypes.byref(ag), df.data_ptr(), dh.data_ptr(), db.data_ptr(), 2 * B, c,
                                   D, G, K, st) == 0
        zs.append(z); dfs.append(df)
    torch.cuda.synchronize()
    scale = float(z_ref.detach().abs().max())
    _close(_unshard(zs, cp) / scale, z_ref / scale, 2e-2, "mr cp z")
    gscale = float(fr.grad.abs().max())
    _close(_unshard(dfs, cp) / gscale, fr.grad / gscale, 2e-2, "mr cp dfeat")
    _rel(dh, hr.grad, 2e-2, "mr cp dh")
    _rel(db, br.grad, 2e-2, "mr cp dbias")


@pytest.mark.parametrize("cp", [2, 3])
def test_hyena_li_cp_scan_with_exchange_inside(cp):
    """Hyena-LI with the all-to-all inside the scan kernels (csrc/li_scan.cu `sb_li_cp_*`), virtual ranks on one GPU:
    every rank stages u = x2 v of its zigzag shard, the channel-sharded scans read it from the owners' staging buffers
    and store y back; z and all gradients equal the fp32 statement of the operator on the unsplit sequence."""
    from savanna_b200.parallel import li_fused as lf
    ws = _WS()
    lib = lf._lib(ws)
    torch.manual_seed(3)
    B, D, O, c = 1, 64 * cp, 8, 256
    d, l, L = D // cp, 2 * c, 2 * cp * c
    feat = (torch.randn(B, L, 3 * D, device=DEV) * 0.7).to(BF)
    gamma = torch.randn(D, O, device=DEV) * 0.3 - 1.0
    p = torch.randn(D, O, device=DEV) * 0.2 - 1.0
    R = torch.randn(D, O, device=DEV) * 0.3
    bias = torch.randn(D, device=DEV) * 0.5
    gz = torch.randn(B, L, D, device=DEV, dtype=BF)
    fr = feat.float().requires_grad_()
    gr, Rr, pr, br = (t.clone().requires_grad_() for t in (gamma, R, p, bias))
    z_ref = ref.hyena_li_modal(fr, gr, Rr, pr, br)
    z_ref.backward(gz.float())
    st = torch.cuda.current_stream().cuda_stream
    fs = [_shard(feat, cp, r) for r in range(cp)]
    gs = [_shard(gz, cp, r) for r in range(cp)]
    tc = lf.scan_chunk(c, B, d, L)
    assert tc > 0 and c % tc == 0
    NC = L // tc
    ll_all = lf._pad_order(-torch.exp(p) * torch.exp(gamma), -1.0e30)
    R_all = lf._pad_order(R, 0.0)
    ustage = [torch.empty(B, l, D, device=DEV, dtype=BF) for _ in range(cp)]
    ystage = [torch.full((B, l, D), float("nan"), device=DEV, dtype=BF) for _ in range(cp)]
    for r in range(cp):
        assert lib.sb_li_cp_gate(fs[r].data_ptr(), None, ustage[r].data_ptr(), B * l, D, 0, st) == 0
    ufull = []
    for r in range(cp):
        sl = slice(r * d, (r + 1) * d)
        ll, Rp, bf = ll_all[sl].contiguous(), R_all[sl].contiguous(), bias[sl].contiguous()
        S = torch.empty(B, NC, d, 16, device=DEV)
        uf = torch.empty(B, L, d, device=DEV, dtype=BF)
        um, ym = lf.make_map(_ptrs(ustage), r, cp, l, D), lf.make_map(_ptrs(ystage), r, cp, l, D)
        assert lib.sb_li_cp_fwd(ctypes.byref(um), ctypes.byref(ym), ll.data_ptr(), Rp.data_ptr(), bf.data_ptr(), S.data_ptr(),
                                uf.data_ptr(), B, L, d, tc, st) == 0
        ufull.append(uf)
    zs = []
    for r in range(cp):
        z = torch.empty(B, l, D, device=DEV, dtype=BF)
        assert lib.sb_li_cp_gate(fs[r].data_ptr(), ystage[r].data_ptr(), z.data_ptr(), B * l, D, 1, st) == 0
        zs.append(z)
    torch.cuda.synchronize()
    scale = float(z_ref.detach().abs().max())
    _close(_unshard(zs, cp) / scale, z_ref.detach() / scale, 2e-2, "li cp z")
    # backward
    gstage = [torch.empty(B, l, D, device=DEV, dtype=BF) for _ in range(cp)]
    ystage = [torch.full((B, l, D), float("nan"), device=DEV, dtype=BF) for _ in range(cp)]
    dustage = [torch.full((B, l, D), float("nan"), device=DEV, dtype=BF) for _ in range(cp)]
    for r in range(cp):
        assert lib.sb_li_cp_gate(fs[r].data_ptr(), gs[r].data_ptr(), gstage[r].data_ptr(), B * l, D, 1, st) == 0
    dR, dll, db = torch.zeros(D, O, device=DEV), torch.zeros(D, O, device=DEV), torch.zeros(D, device=DEV)
    for r in range(cp):
        sl = slice(r * d, (r + 1) * d)
        ll, Rp, bf = ll_all[sl].contiguous(), R_all[sl].contiguous(), bias[sl].contiguous()
        S, W, A, dRp, dLp = (torch.empty(B, NC, d, 16, device=DEV) for _ in range(5))
        dBp = torch.empty(B, NC, d, device=DEV)
        dyf = torch.empty(B, L, d, device=DEV, dtype=BF)
        gm, ym, dm = (lf.make_map(_ptrs(x), r, cp, l, D) for x in (gstage, ystage, dustage))
        assert lib.sb_li_cp_bwd(ctypes.byref(gm), ctypes.byref(ym), ctypes.byref(dm), ufull[r].data_ptr(), dyf.data_ptr(),
                                ll.data_ptr(), Rp.data_ptr(), bf.data_ptr(), S.data_ptr(), W.data_ptr(), A.data_ptr(),
                                dRp.data_ptr(), dLp.data_ptr(), dBp.data_ptr(), B, L, d, tc, st) == 0
        dR[sl] = dRp.sum((0, 1))[:, :O]
        dll[sl] = (dLp.sum((0, 1)) * torch.exp(ll) * ll)[:, :O]
        db[sl] = dBp.sum((0, 1))
    dfs = []
    for r in range(cp):
        df = torch.empty_like(fs[r])
        assert lib.sb_li_cp_finalize_bwd(fs[r].data_ptr(), gs[r].data_ptr(), ystage[r].data_ptr(), dustage[r].data_ptr(),
                                         df.data_ptr(), B * l, D, st) == 0
        dfs.append(df)
    torch.cuda.synchronize()
    gscale = float(fr.grad.abs().max())
    _close(_unshard(dfs, cp) / gscale, fr.grad / gscale, 2e-2, "li cp dfeat")
    _rel(dR, Rr.grad, 3e-2, "li cp dR")
    _rel(dll, gr.grad, 3e-2, "li cp dgamma")
    _rel(dll, pr.grad, 3e-2, "li cp dp")
    _rel(db, br.grad, 3e-2, "li cp dbias")
