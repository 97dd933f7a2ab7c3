"""CUDA kernels against the fp32 PyTorch statement of the same operator (ops/reference.py).

Tolerances: bf16 tensors are compared element by element, |got - want| <= atol * rms(want) + rtol * |want|, with
atol = rtol = 2e-2 by default: a few bf16 ulps (2^-8 relative) on the element itself plus a floor of 2 % of the tensor's
typical magnitude for elements that are small because their terms cancel.  (The reference's kernel tests use 1e-3 on
bf16 intermediates that are compared before the final rounding; outputs that are themselves rounded to bf16 cannot meet
that.)  fp32 quantities (filter gradients, norms) are compared in relative L2 norm."""
import math

import pytest
import torch

from savanna_b200 import ops
from savanna_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF = torch.bfloat16


def _close(a, b, rtol=2e-2, atol=2e-2, what=""):
    a, b = a.float(), b.float()
    rms = b.pow(2).mean().sqrt().clamp(min=1e-12)
    err = (a - b).abs()
    bound = atol * rms + rtol * b.abs()
    bad = err > bound
    assert not bool(bad.any()), (f"{what}: {int(bad.sum())} of {bad.numel()} elements outside atol*rms + rtol*|ref| "
                                 f"(worst excess {(err - bound).max().item():.4g}, rms {rms.item():.4g})")


def _rel(a, b, tol, what=""):
    a, b = a.float(), b.float()
    denom = b.norm().clamp(min=1e-12)
    r = (a - b).norm() / denom
    assert r <= tol, f"{what}: relative L2 error {r.item():.4g} > {tol}"


def _status_ok():
    from savanna_b200.ops import cuda_ops
    cuda_ops.check_status()


@pytest.fixture(params=[0, 2], ids=["one_cta", "cta_pair"])
def pair_mode(request):
    """Runs a GEMM test with the single-CTA kernel and with the cta_group::2 kernel."""
    from savanna_b200.ops import cuda_ops
    cuda_ops.set_gemm_pair_mode(request.param)
    yield request.param
    cuda_ops.set_gemm_pair_mode(2)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (300, 264, 136), (1024, 768, 512), (8192, 512, 1024)])
def test_gemm_tn(M, N, K, pair_mode):
    from savanna_b200.ops import cuda_ops
    torch.manual_seed(0)
    a = torch.randn(M, K, device=DEV, dtype=BF)
    b = torch.randn(N, K, device=DEV, dtype=BF)
    out = torch.full((M, N), float("nan"), device=DEV, dtype=BF)
    cuda_ops.gemm(a, b, out)
    _status_ok()
    _rel(out, a.float() @ b.float().t(), 1e-2, "gemm TN")


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (384, 520, 200)])
def test_gemm_bias_accumulate(M, N, K, pair_mode):
    from savanna_b200.ops import cuda_ops
    torch.manual_seed(1)
    a = torch.randn(M, K, device=DEV, dtype=BF)
    b = torch.randn(N, K, device=DEV, dtype=BF)
    bias = torch.randn(N, device=DEV, dtype=BF)
    c0 = torch.randn(M, N, device=DEV, dtype=BF)
    out = c0.clone()
    cuda_ops.gemm(a, b, out, bias=bias, accumulate=True)
    _status_ok()
    _rel(out, a.float() @ b.float().t() + bias.float() + c0.float(), 1e-2, "gemm bias+acc")


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (512, 384, 320), (264, 136, 520)])
def test_gemm_dgrad_layout(M, N, K, pair_mode):
    """B given as its transpose storage [K, N] (weights in dgrad)."""
    from savanna_b200.ops import cuda_ops
    torch.manual_seed(2)
    a = torch.randn(M, K, device=DEV, dtype=BF)
    bt = torch.randn(K, N, device=DEV, dtype=BF)
    out = torch.empty(M, N, device=DEV, dtype=BF)
    cuda_ops.gemm(a, bt, out, b_mn=True)
    _status_ok()
    _rel(out, a.float() @ bt.float(), 1e-2, "gemm A K-major, B MN-major")


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (512, 384, 1000), (136, 264, 4096)])
def test_gemm_wgrad_layout(M, N, K, pair_mode):
    """Both operands stored with the reduction dim as the row index."""
    from savanna_b200.ops import cuda_ops
    torch.manual_seed(3)
    at = torch.randn(K, M, device=DEV, dtype=BF)
    bt = torch.randn(K, N, device=DEV, dtype=BF)
    out = torch.empty(M, N, device=DEV, dtype=BF)
    cuda_ops.gemm(at, bt, out, a_mn=True, b_mn=True)
    _status_ok()
    _rel(out, at.float().t() @ bt.float(), 1e-2, "gemm both MN-major")


def test_linear_autograd():
    torch.manual_seed(4)
    x = torch.randn(2, 96, 256, device=DEV, dtype=BF, requires_grad=True)
    w = (torch.randn(384, 256, device=DEV) * 0.05).to(BF).requires_grad_()
    b = torch.randn(384, device=DEV, dtype=BF, requires_grad=True)
    y = ops.linear(x, w, b)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = ref.linear(xr, wr, br)
    yr.backward(g.float())
    _status_ok()
    _rel(y, yr, 1e-2, "linear fwd")
    _rel(x.grad, xr.grad, 1e-2, "linear dx")
    _rel(w.grad, wr.grad, 1e-2, "linear dw")
    _rel(b.grad, br.grad, 1e-2, "linear db")


@pytest.mark.parametrize("form", ["te", "classic"])
@pytest.mark.parametrize("D", [256, 4096])
def test_rmsnorm(form, D):
    torch.manual_seed(5)
    x = torch.randn(3, 50, D, device=DEV, dtype=BF, requires_grad=True)
    w = (1 + 0.1 * torch.randn(D, device=DEV)).to(BF).requires_grad_()
    y = ops.rmsnorm(x, w, 1e-6, form)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = ref.rmsnorm(xr, wr, 1e-6, form)
    yr.backward(g.float())
    _close(y, yr, what="rmsnorm fwd")
    _close(x.grad, xr.grad, what="rmsnorm dx")
    _rel(w.grad, wr.grad, 2e-2, "rmsnorm dw")


def test_rmsnorm_residual_branch():
    """(norm(x), x): the gradient of the residual branch is added inside the norm's backward kernel."""
    torch.manual_seed(50)
    x = torch.randn(3, 70, 4096, device=DEV, dtype=BF, requires_grad=True)
    w = (1 + 0.1 * torch.randn(4096, device=DEV)).to(BF).requires_grad_()
    y, r = ops.rmsnorm_residual(x, w, 1e-6, "te")
    g1, g2 = torch.randn_like(y), torch.randn_like(y)
    ((y.float() * g1.float()).sum() + (r.float() * g2.float()).sum()).backward()
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = ref.rmsnorm(xr, wr, 1e-6, "te")
    ((yr * g1.float()).sum() + (xr * g2.float()).sum()).backward()
    _rel(y, yr, 1e-2, "y")
    assert torch.equal(r, x)
    _rel(x.grad, xr.grad, 1e-2, "dx with residual gradient")
    _rel(w.grad, wr.grad, 2e-2, "dw")
    # only the residual branch used: the gradient passes through unchanged
    x2 = x.detach().clone().requires_grad_()
    _, r2 = ops.rmsnorm_residual(x2, w, 1e-6, "te")
    (r2.float() * g2.float()).sum().backward()
    _rel(x2.grad, g2, 1e-3, "pass-through")


@pytest.mark.parametrize("act", ["silu", "gelu", "identity"])
def test_glu(act):
    torch.manual_seed(6)
    ab = torch.randn(4, 33, 2 * 688, device=DEV, dtype=BF, requires_grad=True)
    h = ops.glu_act_packed(ab, act)
    g = torch.randn_like(h)
    h.backward(g)
    abr = ab.detach().float().requires_grad_()
    a, b = abr.chunk(2, -1)
    hr = ref.glu_act(a, b, act)
    hr.backward(g.float())
    _close(h, hr, what="glu fwd")
    _close(ab.grad, abr.grad, what="glu bwd")


def test_rope():
    torch.manual_seed(7)
    B, L, H, hd = 2, 64, 4, 64
    qkv = torch.randn(B, L, H, 3 * hd, device=DEV, dtype=BF, requires_grad=True)
    pos = torch.arange(L, device=DEV)
    cos, sin = ref.rope_tables(pos, hd)
    q = qkv[..., :hd]
    y = ops.apply_rope(q, cos, sin)
    g = torch.randn_like(y)
    y.backward(g)
    qr = qkv.detach().float().requires_grad_()
    yr = ref.apply_rope(qr[..., :hd], cos, sin)
    yr.backward(g.float())
    _close(y, yr, what="rope fwd")
    _close(qkv.grad, qr.grad, what="rope bwd")


def test_cross_entropy():
    torch.manual_seed(8)
    logits = (torch.randn(2, 100, 512, device=DEV) * 3).to(BF).requires_grad_()
    labels = torch.randint(0, 512, (2, 100), device=DEV)
    l = ops.cross_entropy(logits, labels)
    w = torch.rand_like(l)
    (l * w).sum().backward()
    lr_ = logits.detach().float().requires_grad_()
    lref = ref.cross_entropy(lr_, labels)
    (lref * w).sum().backward()
    _rel(l, lref, 1e-3, "ce fwd")
    _close(logits.grad, lr_.grad, what="ce bwd")


def test_sqnorm_adam():
    torch.manual_seed(9)
    n = 100_003
    g = torch.randn(n, device=DEV).to(BF)
    wgt = torch.rand(n, device=DEV)
    _rel(ops.sq_norm(g), (g.float() ** 2).sum(), 1e-4, "sqnorm")
    _rel(ops.sq_norm(g, wgt), (g.float() ** 2 * wgt).sum(), 1e-4, "weighted sqnorm")
    master = torch.randn(n, device=DEV)
    m, v = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    p = torch.empty(n, device=DEV, dtype=BF)
    mr, mm, vv = master.clone(), m.clone(), v.clone()
    pr = torch.empty(n, device=DEV, dtype=BF)
    scale = torch.tensor(0.5, device=DEV)
    for step in (1, 2, 3):
        ops.adam_step(master, m, v, g, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, True, scale, p)
        ref.adam_step(mr, mm, vv, g, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, True, 0.5, pr)
    _rel(master, mr, 1e-5, "adam master")
    _rel(v, vv, 1e-5, "adam v")
    assert torch.equal(p, master.to(BF))


@pytest.fixture(params=[(True, True), (False, False)], ids=["tiled", "per_thread_run"])
def conv_variant(request):
    from savanna_b200.ops import cuda_ops
    cuda_ops.set_conv_forward_variant(request.param[0])
    cuda_ops.set_se_backward_variant(request.param[1])
    yield request.param
    cuda_ops.set_conv_forward_variant(True)
    cuda_ops.set_se_backward_variant(True)


@pytest.mark.parametrize("K", [3, 4, 7])
@pytest.mark.parametrize("halo", [False, True])
@pytest.mark.parametrize("C,L", [(96, 300), (192, 300), (128, 128), (64, 517)])
def test_dwconv(K, halo, C, L, conv_variant):
    torch.manual_seed(10)
    B = 2
    x = torch.randn(B, L, C, device=DEV, dtype=BF, requires_grad=True)
    w = (torch.randn(C, K, device=DEV) * 0.5).requires_grad_()
    h = torch.randn(B, K - 1, C, device=DEV, dtype=BF, requires_grad=True) if halo else None
    y = ops.causal_conv1d(x, w, h)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(), w.detach().clone().requires_grad_()
    hr = h.detach().float().requires_grad_() if halo else None
    yr = ref.causal_conv1d(xr, wr, hr)
    yr.backward(g.float())
    _close(y, yr, what="dwconv fwd")
    _close(x.grad, xr.grad, what="dwconv dx")
    _rel(w.grad, wr.grad, 2e-2, "dwconv dw")
    if halo:
        _close(h.grad, hr.grad, what="dwconv dhalo")


@pytest.fixture(params=[True, False], ids=["tiled", "per_thread_run"])
def se_bwd_variant(request):
    from savanna_b200.ops import cuda_ops
    cuda_ops.set_se_backward_variant(request.param)
    cuda_ops.set_conv_forward_variant(request.param)
    yield request.param
    cuda_ops.set_se_backward_variant(True)
    cuda_ops.set_conv_forward_variant(True)


@pytest.mark.parametrize("K,G,L", [(7, 16, 200), (3, 64, 200), (7, 256, 200), (7, 8, 515), (4, 4, 128), (7, 2, 130)])
@pytest.mark.parametrize("halo", [False, True])
def test_hyena_se(K, G, L, halo, se_bwd_variant):
    torch.manual_seed(11)
    B, D = 2, 256
    feat = torch.randn(B, L, 3 * D, device=DEV, dtype=BF, requires_grad=True)
    w = (torch.randn(G, K, device=DEV) * 0.4).requires_grad_()
    h = torch.randn(B, K - 1, 3 * D, device=DEV, dtype=BF, requires_grad=True) if halo else None
    z = ops.hyena_se_inner(feat, w, h)
    g = torch.randn_like(z)
    z.backward(g)
    fr, wr = feat.detach().float().requires_grad_(), w.detach().clone().requires_grad_()
    hr = h.detach().float().requires_grad_() if halo else None
    zr = ref.hyena_se_inner(fr, wr, hr)
    zr.backward(g.float())
    _close(z, zr, what="se fwd")
    _close(feat.grad, fr.grad, what="se dfeat")
    _rel(w.grad, wr.grad, 2e-2, "se dw")
    if halo:
        _close(h.grad, hr.grad, what="se dhalo")


@pytest.fixture(params=[True, False], ids=["streaming", "per_tile"])
def mr_bwd_variant(request):
    from savanna_b200.ops import cuda_ops
    cuda_ops.set_mr_backward_variant(request.param)
    yield request.param
    cuda_ops.set_mr_backward_variant(True)


@pytest.mark.parametrize("K,G,L", [(128, 16, 400), (32, 16, 130), (128, 4, 256), (128, 32, 200), (100, 16, 333), (128, 16, 2100)])
@pytest.mark.parametrize("halo", [False, True])
def test_hyena_mr(K, G, L, halo, mr_bwd_variant):
    torch.manual_seed(12)
    B, D = 2, 256
    feat = torch.randn(B, L, 3 * D, device=DEV, dtype=BF, requires_grad=True)
    hflt = (torch.randn(G, K, device=DEV) * (1.0 / math.sqrt(K))).requires_grad_()
    bias = torch.randn(D, device=DEV).requires_grad_()
    h = torch.randn(B, K - 1, 3 * D, device=DEV, dtype=BF, requires_grad=True) if halo else None
    z = ops.hyena_mr_inner(feat, hflt, bias, h)
    g = torch.randn_like(z)
    z.backward(g)
    fr, hr_, br = feat.detach().float().requires_grad_(), hflt.detach().clone().requires_grad_(), bias.detach().clone().requires_grad_()
    hh = h.detach().float().requires_grad_() if halo else None
    zr = ref.hyena_mr_inner(fr, hr_, br, hh)
    zr.backward(g.float())
    # the Toeplitz products run on bf16 tensor-core operands (u = x2 v, the taps, and in the backward y and du are
    # rounded to bf16 before the MMAs), one rounding more than the element-wise kernels: 3 % instead of 2 %
    _close(z, zr, rtol=3e-2, atol=3e-2, what="mr fwd")
    _close(feat.grad, fr.grad, rtol=3e-2, atol=3e-2, what="mr dfeat")
    _rel(hflt.grad, hr_.grad, 2e-2, "mr dh")
    _rel(bias.grad, br.grad, 2e-2, "mr dbias")
    if halo:
        _close(h.grad, hh.grad, rtol=3e-2, atol=3e-2, what="mr dhalo")


@pytest.fixture(params=[None, 512], ids=["chunk_auto", "chunk_512"])
def li_chunk(request):
    """Chunk length of the scan: the automatic choice (128 at these sizes) and the 512 that the 7B shapes select."""
    from savanna_b200.ops import cuda_ops
    cuda_ops.LI_CHUNK_OVERRIDE = request.param
    yield request.param
    cuda_ops.LI_CHUNK_OVERRIDE = None


@pytest.fixture(params=[True, False], ids=["tiled", "streaming"])
def li_variant(request):
    from savanna_b200.ops import cuda_ops
    cuda_ops.set_li_variant(request.param)
    yield request.param
    cuda_ops.set_li_variant(True)


@pytest.mark.parametrize("L,O,state", [(512, 16, False), (300, 8, False), (384, 16, True), (1300, 16, True)])
def test_hyena_li(L, O, state, li_chunk, li_variant):
    torch.manual_seed(13)
    B, D = 2, 128
    feat = (torch.randn(B, L, 3 * D, device=DEV) * 0.7).to(BF).requires_grad_()
    gamma = (torch.rand(D, O, device=DEV) * 0.09 + 0.01).log().requires_grad_()
    R = (0.1 * torch.randn(D, O, device=DEV) / math.sqrt(O)).requires_grad_()
    p = (-torch.ones(D, O, device=DEV)).requires_grad_()
    bias = torch.randn(D, device=DEV).requires_grad_()
    s_in = torch.randn(B, D, O, device=DEV).requires_grad_() if state else None
    out = ops.hyena_li_modal(feat, gamma, R, p, bias, s_in, state)
    z, s_out = out if state else (out, None)
    g = torch.randn_like(z)
    gs = torch.randn_like(s_out) if state else None
    loss = (z.float() * g.float()).sum() + ((s_out * gs).sum() if state else 0.0)
    loss.backward()
    leaves = [t.detach().float().requires_grad_() for t in (feat, gamma, R, p, bias)]
    sr = s_in.detach().clone().requires_grad_() if state else None
    outr = ref.hyena_li_modal(*leaves, sr, state)
    zr, sor = outr if state else (outr, None)
    lossr = (zr.float() * g.float()).sum() + ((sor * gs).sum() if state else 0.0)
    lossr.backward()
    _close(z, zr, what="li fwd")
    _close(feat.grad, leaves[0].grad, rtol=3e-2, atol=3e-2, what="li dfeat")
    _rel(R.grad, leaves[2].grad, 3e-2, "li dR")
    _rel(gamma.grad, leaves[1].grad, 3e-2, "li dgamma")
    _rel(p.grad, leaves[3].grad, 3e-2, "li dp")
    _rel(bias.grad, leaves[4].grad, 3e-2, "li dbias")
    if state:
        _rel(s_out, sor, 1e-3, "li state_out")
        _rel(s_in.grad, sr.grad, 3e-2, "li dstate_in")


def test_linear_residual_epilogue_and_inplace_grad_accumulation():
    torch.manual_seed(20)
    x = torch.randn(3, 100, 256, device=DEV, dtype=BF, requires_grad=True)
    res = torch.randn(3, 100, 384, device=DEV, dtype=BF, requires_grad=True)
    w = torch.nn.Parameter((torch.randn(384, 256, device=DEV) * 0.05).to(BF))
    b = torch.nn.Parameter(torch.randn(384, device=DEV, dtype=BF))
    w.grad = torch.zeros_like(w)
    w._fuse_grad_accum = True                       # what the ZeRO flat buffer sets
    grad_buffer = w.grad
    g1, g2 = torch.randn(3, 100, 384, device=DEV, dtype=BF), torch.randn(3, 100, 384, device=DEV, dtype=BF)
    for g in (g1, g2):                              # two micro-steps accumulate into the same buffer
        y = ops.linear(x, w, b, residual=res)
        y.backward(g)
    _status_ok()
    assert w.grad is grad_buffer
    xr, rr = x.detach().float().requires_grad_(), res.detach().float().requires_grad_()
    wr, br = w.detach().float().requires_grad_(), b.detach().float().requires_grad_()
    for g in (g1, g2):
        yr = ref.linear(xr, wr, br) + rr
        yr.backward(g.float())
    _rel(y, yr, 1e-2, "linear+residual fwd")
    _rel(w.grad, wr.grad, 2e-2, "in-place accumulated dW")
    _rel(b.grad, br.grad, 1e-2, "bias grad (colsum)")
    _rel(x.grad, xr.grad, 1e-2, "dx")
    _rel(res.grad, rr.grad, 1e-2, "dresidual")


@pytest.mark.parametrize("layout", ["tn", "dgrad", "wgrad"])
def test_gemm_fp8_layouts(layout, pair_mode):
    """fp8 operands, per-tensor scales: compare against the product of the DE-QUANTISED operands (exact fp32 math),
    so only accumulation order and the bf16 output rounding remain."""
    from savanna_b200.ops import cuda_ops
    torch.manual_seed(30)
    M, N, K = 384, 512, 640

    def deq(q, sinv, fmt):
        dt = torch.float8_e4m3fn if fmt == 0 else torch.float8_e5m2
        return q.view(dt).float() * sinv
    if layout == "tn":
        a = torch.randn(M, K, device=DEV, dtype=BF); b = torch.randn(N, K, device=DEV, dtype=BF)
        aq, sa = cuda_ops.quantize_fp8(a, 0); bq, sb_ = cuda_ops.quantize_fp8(b, 0)
        out = torch.empty(M, N, device=DEV, dtype=BF)
        cuda_ops.gemm_fp8(aq, bq, out, sa, alpha2=sb_)
        want = deq(aq, sa, 0) @ deq(bq, sb_, 0).t()
    elif layout == "dgrad":
        a = torch.randn(M, K, device=DEV, dtype=BF); bt = torch.randn(K, N, device=DEV, dtype=BF)
        aq, sa = cuda_ops.quantize_fp8(a, 1); bq, sb_ = cuda_ops.quantize_fp8(bt, 0)
        out = torch.empty(M, N, device=DEV, dtype=BF)
        cuda_ops.gemm_fp8(aq, bq, out, sa * sb_, b_mn=True, a_fmt=1, b_fmt=0)
        want = deq(aq, sa, 1) @ deq(bq, sb_, 0)
    else:
        at = torch.randn(K, M, device=DEV, dtype=BF); bt = torch.randn(K, N, device=DEV, dtype=BF)
        aq, sa = cuda_ops.quantize_fp8(at, 1); bq, sb_ = cuda_ops.quantize_fp8(bt, 0)
        out = torch.empty(M, N, device=DEV, dtype=BF)
        cuda_ops.gemm_fp8(aq, bq, out, sa * sb_, a_mn=True, b_mn=True, a_fmt=1, b_fmt=0)
        want = deq(aq, sa, 1).t() @ deq(bq, sb_, 0)
    _status_ok()
    _rel(out, want, 1e-2, f"fp8 gemm {layout}")


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (512, 768, 640), (384, 264, 200), (1000, 520, 1032), (2048, 1024, 4096)])
def test_gemm_cta_pair_bf16(M, N, K):
    """cta_group::2 kernel (two CTAs per 256 x 256 tile): every operand layout, bias / residual / accumulate epilogue."""
    from savanna_b200.ops import cuda_ops
    torch.manual_seed(40)
    cuda_ops.set_gemm_pair_mode(2)
    try:
        a = torch.randn(M, K, device=DEV, dtype=BF); b = torch.randn(N, K, device=DEV, dtype=BF)
        at, bt = a.t().contiguous(), b.t().contiguous()
        want = a.float() @ b.float().t()
        out = torch.full((M, N), float("nan"), device=DEV, dtype=BF)
        cuda_ops.gemm(a, b, out)
        _status_ok(); _rel(out, want, 1e-2, "pair TN")
        out.fill_(float("nan")); cuda_ops.gemm(a, bt, out, b_mn=True)
        _status_ok(); _rel(out, want, 1e-2, "pair dgrad layout")
        out.fill_(float("nan")); cuda_ops.gemm(at, bt, out, a_mn=True, b_mn=True)
        _status_ok(); _rel(out, want, 1e-2, "pair wgrad layout")
        out.fill_(float("nan")); cuda_ops.gemm(at, b, out, a_mn=True)
        _status_ok(); _rel(out, want, 1e-2, "pair A MN-major, B K-major")
        bias = torch.randn(N, device=DEV, dtype=BF); res = torch.randn(M, N, device=DEV, dtype=BF)
        c0 = torch.randn(M, N, device=DEV, dtype=BF); out = c0.clone()
        cuda_ops.gemm(a, b, out, bias=bias, residual=res, accumulate=True)
        _status_ok(); _rel(out, want + bias.float() + res.float() + c0.float(), 1e-2, "pair epilogue")
    finally:
        cuda_ops.set_gemm_pair_mode(2)


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (384, 512, 640), (1008, 528, 1040)])
def test_gemm_cta_pair_fp8(M, N, K):
    from savanna_b200.ops import cuda_ops
    torch.manual_seed(41)

    def deq(q, sinv, fmt):
        return q.view(torch.float8_e4m3fn if fmt == 0 else torch.float8_e5m2).float() * sinv
    cuda_ops.set_gemm_pair_mode(1)
    try:
        a = torch.randn(M, K, device=DEV, dtype=BF); b = torch.randn(N, K, device=DEV, dtype=BF)
        aq, sa = cuda_ops.quantize_fp8(a, 1); bq, sb_ = cuda_ops.quantize_fp8(b, 0)
        atq, sat = cuda_ops.quantize_fp8(a.t().contiguous(), 1); btq, sbt = cuda_ops.quantize_fp8(b.t().contiguous(), 0)
        out = torch.full((M, N), float("nan"), device=DEV, dtype=BF)
        cuda_ops.gemm_fp8(aq, bq, out, sa, alpha2=sb_, a_fmt=1, b_fmt=0)
        _status_ok(); _rel(out, deq(aq, sa, 1) @ deq(bq, sb_, 0).t(), 1e-2, "pair fp8 TN")
        out.fill_(float("nan")); cuda_ops.gemm_fp8(aq, btq, out, sa, alpha2=sbt, b_mn=True, a_fmt=1, b_fmt=0)
        _status_ok(); _rel(out, deq(aq, sa, 1) @ deq(btq, sbt, 0), 1e-2, "pair fp8 dgrad layout")
        out.fill_(float("nan")); cuda_ops.gemm_fp8(atq, btq, out, sat, alpha2=sbt, a_mn=True, b_mn=True, a_fmt=1, b_fmt=0)
        _status_ok(); _rel(out, deq(atq, sat, 1).t() @ deq(btq, sbt, 0), 1e-2, "pair fp8 wgrad layout")
    finally:
        cuda_ops.set_gemm_pair_mode(2)


def test_quantize_fp8_matches_torch():
    from savanna_b200.ops import cuda_ops
    torch.manual_seed(31)
    x = (torch.randn(256, 512, device=DEV) * 3).to(BF)
    q, sinv = cuda_ops.quantize_fp8(x, 0)
    amax = x.float().abs().max()
    assert abs(float(sinv) - float(amax) / 448.0) < 1e-6 * float(amax)
    want = (x.float() * (448.0 / amax)).to(torch.float8_e4m3fn)
    same = (q.view(torch.float8_e4m3fn).float() == want.float()).float().mean()
    assert same > 0.999, f"only {same.item():.4f} of the fp8 codes agree"


def test_quantize_fp8_delayed_scaling():
    """One-pass quantiser: the scale comes from the amax history (max over the last `history` calls), the running amax
    lands in the ring, values beyond the stale range saturate, and the ring forgets after `history` calls."""
    from savanna_b200.ops import cuda_ops
    torch.manual_seed(33)
    old = cuda_ops.FP8_HISTORY
    cuda_ops.set_fp8_history(3)
    try:
        owner = torch.nn.Parameter(torch.zeros(1, device=DEV))
        amaxes, f8 = [], torch.float8_e4m3fn
        for call, gain in enumerate([1.0, 4.0, 0.5, 0.5, 0.5, 0.5]):
            x = (torch.randn(128, 512, device=DEV) * gain).to(BF)
            q, sinv = cuda_ops.quantize_fp8_site(x, 0, owner, "x")
            amaxes.append(float(x.float().abs().max()))
            used = amaxes[0] if call == 0 else max(amaxes[max(0, call - 3):call])
            assert abs(float(sinv) * 448.0 - used) < 1e-5 * used, (call, float(sinv) * 448.0, used)
            want = (x.float() * (448.0 / used)).clamp(-448.0, 448.0).to(f8)
            same = (q.view(f8).float() == want.float()).float().mean()
            assert same > 0.999, (call, same.item())
        hist = owner._fp8_sites["x"].buf
        assert abs(float(hist.max()) - max(amaxes[-3:])) < 1e-6          # the gain-4 call has left the ring
        _status_ok()
    finally:
        cuda_ops.set_fp8_history(old)


def test_linear_fp8_autograd():
    torch.manual_seed(32)
    x = torch.randn(2, 128, 512, device=DEV, dtype=BF, requires_grad=True)
    w = (torch.randn(768, 512, device=DEV) * 0.05).to(BF).requires_grad_()
    y = ops.linear(x, w, None, fp8=True)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = ref.linear(xr, wr)
    yr.backward(g.float())
    _status_ok()
    _rel(y, yr, 6e-2, "fp8 linear fwd")          # e4m3 has 3 mantissa bits: a few percent relative error is the format
    _rel(x.grad, xr.grad, 8e-2, "fp8 linear dx")
    _rel(w.grad, wr.grad, 8e-2, "fp8 linear dw")


def test_fused_fp8_producers_match_unfused():
    """RMSNorm -> fp8 projection and gate -> fp8 projection with the producing kernel writing the fp8 operand: from the
    second call at a site on (the first call has no amax history) outputs and gradients equal those of the separate
    norm / gate, quantise and GEMM kernels, which see the same scale."""
    from savanna_b200.ops import cuda_ops
    torch.manual_seed(60)
    T, D, N, Fh = 384, 512, 768, 640
    wn = (1 + 0.1 * torch.randn(D, device=DEV)).to(BF)
    w0 = (torch.randn(N, D, device=DEV) * 0.05).to(BF)
    w3_0 = (torch.randn(D, Fh, device=DEV) * 0.05).to(BF)
    b3_0 = torch.randn(D, device=DEV, dtype=BF)
    results = []
    for fused in (True, False):
        w, w3, b3 = (torch.nn.Parameter(t.clone()) for t in (w0, w3_0, b3_0))
        wnp = torch.nn.Parameter(wn.clone())
        outs = None
        for call in range(3):
            torch.manual_seed(100 + call)
            x = torch.randn(2, T // 2, D, device=DEV, dtype=BF, requires_grad=True)
            ab = torch.randn(2, T // 2, 2 * Fh, device=DEV, dtype=BF, requires_grad=True)
            res = torch.randn(2, T // 2, D, device=DEV, dtype=BF, requires_grad=True)
            for p in (w, w3, b3, wnp):
                p.grad = None
            if fused:
                y, r = cuda_ops.norm_linear(x, wnp, 1e-6, "te", w, None, True)
                z = cuda_ops.glu_linear(ab, "silu", w3, b3, res, True)
            else:
                u, r = cuda_ops.rmsnorm_residual(x, wnp, 1e-6, "te")
                y = cuda_ops.linear(u, w, None, True)
                z = cuda_ops.linear(cuda_ops.glu_act_packed(ab, "silu"), w3, b3, True, res)
            g1, g2, g3 = torch.randn_like(y), torch.randn_like(z), torch.randn_like(r)
            ((y.float() * g1.float()).sum() + (z.float() * g2.float()).sum() + (r.float() * g3.float()).sum()).backward()
            outs = [t.detach().float().clone() for t in (y, z, x.grad, ab.grad, res.grad, w.grad, w3.grad, b3.grad, wnp.grad)]
        results.append(outs)
        _status_ok()
    names = ["y", "z", "dx", "dab", "dres", "dw", "dw3", "db3", "dwn"]
    for name, a, b in zip(names, *results):
        _rel(a, b, 2e-3, f"fused vs unfused {name}")


def test_mlp_fp8_single_node_matches_composed_ops():
    """The whole gated MLP as one autograd node (fp8 operands written by the norm, gate and gate-backward kernels) against
    the composition of the separate ops, from the third call on (amax histories primed on both sides)."""
    from savanna_b200.ops import cuda_ops
    torch.manual_seed(61)
    T, D, Fh = 256, 512, 640
    wn0 = (1 + 0.1 * torch.randn(D, device=DEV)).to(BF)
    w12_0 = (torch.randn(2 * Fh, D, device=DEV) * 0.05).to(BF)
    w3_0 = (torch.randn(D, Fh, device=DEV) * 0.05).to(BF)
    b3_0 = torch.randn(D, device=DEV, dtype=BF)
    results = []
    for fused in (True, False):
        wn, w12, w3, b3 = (torch.nn.Parameter(t.clone()) for t in (wn0, w12_0, w3_0, b3_0))
        for call in range(3):
            torch.manual_seed(200 + call)
            x = torch.randn(2, T // 2, D, device=DEV, dtype=BF, requires_grad=True)
            for p in (wn, w12, w3, b3):
                p.grad = None
            if fused:
                y = cuda_ops.mlp_gated(x, wn, 1e-6, "te", w12, w3, b3, "silu", True)
            else:
                u, r = cuda_ops.rmsnorm_residual(x, wn, 1e-6, "te")
                ab = cuda_ops.linear(u, w12, None, True)
                y = cuda_ops.linear(cuda_ops.glu_act_packed(ab, "silu"), w3, b3, True, r)
            g = torch.randn_like(y)
            (y.float() * g.float()).sum().backward()
            outs = [t.detach().float().clone() for t in (y, x.grad, wn.grad, w12.grad, w3.grad, b3.grad)]
        results.append(outs)
        _status_ok()
    for name, a, b in zip(["y", "dx", "dwn", "dw12", "dw3", "db3"], *results):
        _rel(a, b, 2e-3, f"mlp node vs composed {name}")


def test_fp8_training_tracks_bf16():
    """Same tiny model, same data: the loss trace with fp8 projections stays close to the bf16 one."""
    import os
    from savanna_b200.config import GlobalConfig
    from savanna_b200.data.synthetic import acgt_batch
    from savanna_b200.parallel import state
    from savanna_b200.train.trainer import Trainer
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    traces = []
    for fp8 in (False, True):
        over = {"global_num_gpus": 1}
        if fp8:
            over.update({"use_fp8_linears": True, "use_fp8_input_projections": True, "use_fp8_output_projections": True,
                         "use_fp8_mlp_projections": True})
        cfg = GlobalConfig.from_ymls([os.path.join(root, "configs", "baseline", "tiny_sh2_gpu.yml")], over)
        tr = Trainer(cfg, load=False)
        batches = iter([{"text": acgt_batch(cfg.train_micro_batch_size_per_gpu, cfg.seq_length, seed=i).cuda()} for i in range(30)])
        traces.append([float(tr.train_step(batches)) for _ in range(30)])
        state.destroy_model_parallel()
    a, b = traces
    assert b[-1] < b[0] - 1.5, b
    assert abs(a[-1] - b[-1]) < 0.08 * a[-1], (a[-1], b[-1])
    assert max(abs(x - y) for x, y in zip(a, b)) < 0.25, (a, b)


def test_peer_barrier_wait_runs_out_and_reports():
    """A bounded device-side wait that nothing satisfies: the barrier kernel of "rank 0 of 2" waits for a signal word
    that no one writes, gives up after its budget (30 ms here), records the time-out code with the missing rank in the
    status word and returns by itself; the host turns the word into an exception and the context stays usable."""
    import ctypes
    import time
    from savanna_b200.ops import cuda_ops
    lib = cuda_ops.require()
    P, I = ctypes.c_void_p, ctypes.c_int
    lib.sb_peer_barrier_budget.restype = I
    lib.sb_peer_barrier_budget.argtypes = [P, I, I, I, P, ctypes.c_ulonglong, P]
    cuda_ops.check_status()
    sig = [torch.zeros(32, dtype=torch.int32, device=DEV) for _ in range(2)]        # both ranks' signal arrays, local
    ptrs = (ctypes.c_void_p * 2)(sig[0].data_ptr(), sig[1].data_ptr())
    dev = torch.device("cuda", torch.cuda.current_device())
    torch.cuda.synchronize()
    t0 = time.time()
    rc = lib.sb_peer_barrier_budget(ptrs, 0, 2, 1, cuda_ops.status_word(dev).data_ptr(), 30_000_000,
                                    torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert time.time() - t0 < 1.0                       # the kernel ended on its own, well inside the default 1.5 s
    assert int(sig[1][0]) == 1                          # rank 0 did signal its (absent) peer
    with pytest.raises(RuntimeError, match="bounded wait: code 5"):
        cuda_ops.check_status()
    cuda_ops.check_status()                             # the word was cleared; the context still works
    a = torch.ones(8, device=DEV)
    assert float((a + a).sum()) == 16.0


# ----------------------------------------------------------------------------- block-scaled fp8 (MXFP8)
from savanna_b200.ops import cuda_ops  # noqa: E402


def _done():
    torch.cuda.synchronize()
    cuda_ops.check_status()


def _mx_reference_quantize(x, transposed=False):
    """PyTorch statement of the MXFP8 quantiser: per 32 elements of the contraction e = ceil(log2(amax / 448)),
    q = e4m3(x / 2^e).  Returns (q as float, e as int tensor, the de-quantised tensor) in operand orientation [rows, K]."""
    xf = x.float().t().contiguous() if transposed else x.float()
    R, K = xf.shape
    blocks = xf.view(R, K // 32, 32)
    amax = blocks.abs().amax(-1)
    e = torch.where(amax > 0, torch.ceil(torch.log2(amax / 448.0)), torch.full_like(amax, -127.0)).clamp(-127, 127)
    scale = torch.exp2(e)[..., None]
    q = (blocks / scale).to(torch.float8_e4m3fn).float()
    return q.view(R, K), e.to(torch.int32), (q * scale).view(R, K)


def _mx_unpack_scales(sf, rows, k):
    """E8M0 bytes of the kernel's atom layout -> [rows, k / 32] exponents."""
    kb = (k + 127) // 128
    atoms = sf.view((rows + 127) // 128, kb, 32, 4, 4)          # [row tile, k-block, r % 32, r // 32, k4]
    full = atoms.permute(0, 3, 2, 1, 4).reshape(-1, kb * 4)      # rows = tile * 128 + (r // 32) * 32 + r % 32
    return full[:rows, : k // 32].to(torch.int32) - 127


@pytest.mark.parametrize("shape", [(256, 256), (192, 416), (64, 4096)])
@pytest.mark.parametrize("transposed", [False, True])
def test_mx_quantize_matches_the_block_scaling_rule(shape, transposed):
    torch.manual_seed(41)
    R, C = shape
    x = (torch.randn(R, C, device=DEV) * torch.exp(torch.randn(R, 1, device=DEV) * 2)).to(BF)
    x[3, :40] = 0
    q, sf = cuda_ops.mx_quantize(x, transposed)
    _done()
    qr, er, _ = _mx_reference_quantize(x, transposed)
    rows, k = (C, R) if transposed else (R, C)
    assert q.shape == (rows, k)
    e = _mx_unpack_scales(sf, rows, k)
    assert torch.equal(e, er), (e - er).abs().max()
    assert torch.equal(q.view(torch.float8_e4m3fn).float(), qr)


@pytest.mark.parametrize("shape", [(128, 256, 128), (256, 512, 1024), (200, 328, 416), (1024, 4096, 4096)])
def test_mx_gemm_against_dequantised_fp32(shape):
    """The block-scaled tensor-core product against fp32 matmul of the de-quantised operands: only the summation order
    differs, so the tolerance is tight."""
    torch.manual_seed(42)
    M, N, K = shape
    a = (torch.randn(M, K, device=DEV) * torch.exp(torch.randn(M, 1, device=DEV))).to(BF)
    b = (torch.randn(N, K, device=DEV) * 0.05 * torch.exp(torch.randn(1, K, device=DEV))).to(BF)
    aq, sa = cuda_ops.mx_quantize(a)
    bq, sb_ = cuda_ops.mx_quantize(b)
    bias = torch.randn(N, device=DEV, dtype=BF)
    res = torch.randn(M, N, device=DEV, dtype=BF)
    out = torch.empty(M, N, device=DEV, dtype=BF)
    cuda_ops.gemm_mx(aq, sa, bq, sb_, out, bias=bias, residual=res)
    _done()
    _, _, ad = _mx_reference_quantize(a)
    _, _, bd = _mx_reference_quantize(b)
    want = ad @ bd.t() + bias.float() + res.float()
    _close(out, want, rtol=1e-2, atol=5e-3, what="mx gemm")
    acc = out.clone()
    cuda_ops.gemm_mx(aq, sa, bq, sb_, acc, accumulate=True)
    _done()
    _close(acc, out.float() + ad @ bd.t(), rtol=1e-2, atol=1e-2, what="mx gemm accumulate")


def test_mx_linear_forward_and_gradients_track_bf16():
    """`fp8_recipe: mxfp8` projection: output and all gradients against the fp32 statement, at the accuracy of e4m3
    operands with per-32 scales (a few percent of the rms, no dependence on outliers elsewhere in the tensor)."""
    torch.manual_seed(43)
    T, K, N = 512, 1024, 768
    x = torch.randn(2, T // 2, K, device=DEV, dtype=BF, requires_grad=True)
    x.data[0, 0, 0] = 300.0                                      # an outlier only costs its own block
    w = (torch.randn(N, K, device=DEV) * 0.03).to(BF).requires_grad_()
    b = torch.randn(N, device=DEV, dtype=BF, requires_grad=True)
    cuda_ops.set_fp8_recipe("mxfp8")
    try:
        y = cuda_ops.linear(x, w, b, fp8=True)
        g = torch.randn_like(y)
        y.backward(g)
    finally:
        cuda_ops.set_fp8_recipe("delayed")
    _done()
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(g.float())
    _rel(y, yr, 4e-2, "mx linear fwd")
    _rel(x.grad, xr.grad, 4e-2, "mx linear dx")
    _rel(w.grad, wr.grad, 4e-2, "mx linear dw")
    _rel(b.grad, br.grad, 1e-2, "mx linear db")


def test_mxfp8_training_tracks_bf16():
    """Same tiny model, same data: the loss trace with block-scaled fp8 projections (`fp8_recipe: mxfp8`) stays close to
    the bf16 one, and the block-scaled function is what ran."""
    import os
    from savanna_b200.config import GlobalConfig
    from savanna_b200.data.synthetic import acgt_batch
    from savanna_b200.parallel import state
    from savanna_b200.train.trainer import Trainer
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    traces = []
    calls = {"n": 0}
    orig = cuda_ops.gemm_mx

    def counting(*a, **k):
        calls["n"] += 1
        return orig(*a, **k)
    try:
        for mx in (False, True):
            over = {"global_num_gpus": 1}
            if mx:
                over.update({"use_fp8_linears": True, "use_fp8_input_projections": True, "use_fp8_output_projections": True,
                             "use_fp8_mlp_projections": True, "fp8_recipe": "mxfp8"})
                cuda_ops.gemm_mx = counting
            cfg = GlobalConfig.from_ymls([os.path.join(root, "configs", "baseline", "tiny_sh2_gpu.yml")], over)
            tr = Trainer(cfg, load=False)
            batches = iter([{"text": acgt_batch(cfg.train_micro_batch_size_per_gpu, cfg.seq_length, seed=i).cuda()} for i in range(30)])
            traces.append([float(tr.train_step(batches)) for _ in range(30)])
            state.destroy_model_parallel()
    finally:
        cuda_ops.gemm_mx = orig
        cuda_ops.set_fp8_recipe("delayed")
    a, b = traces
    assert calls["n"] > 0
    assert b[-1] < b[0] - 1.5, b
    assert abs(a[-1] - b[-1]) < 0.06 * a[-1], (a[-1], b[-1])
    assert max(abs(x - y) for x, y in zip(a, b)) < 0.2, (a, b)


GLU_BWD_DEFAULT = cuda_ops.GLU_BWD_EPILOGUE


def test_gate_in_the_projection_epilogue_matches_the_separate_gate_kernel():
    """The gated MLP with the gate applied in the epilogue of the w1|w2 projection and the gate backward in the epilogue of
    the w3 input-gradient product (CTA-pair fp8 kernel, GLU modes 1 and 2) against the same function with the separate gate
    kernels: identical [a | b], identical e4m3 operand of w3 and e5m2 gradient of [a | b] (same scales, same rounding),
    same amax history, same output and gradients, bit for bit."""
    torch.manual_seed(51)
    T, D, F = 384, 512, 1024
    x = torch.randn(1, T, D, device=DEV, dtype=BF)
    wn = (1 + 0.1 * torch.randn(D, device=DEV)).to(BF)
    w12 = (torch.randn(2 * F, D, device=DEV) * 0.05).to(BF)
    w3 = (torch.randn(D, F, device=DEV) * 0.05).to(BF)
    b3 = torch.randn(D, device=DEV, dtype=BF)
    outs = []
    for fused in (False, True):
        cuda_ops.set_glu_epilogue(fused, backward=fused)
        ps = [t.clone().requires_grad_() for t in (x, wn, w12, w3, b3)]
        try:
            for _ in range(3):                                   # the third call runs on primed amax histories
                for t in ps:
                    t.grad = None
                before = cuda_ops.launch_count()
                y = cuda_ops.mlp_gated(ps[0], ps[1], 1e-5, "te", ps[2], ps[3], ps[4], "silu", True)
                launches = cuda_ops.launch_count() - before
                y.backward(torch.ones_like(y) * 0.01)
        finally:
            cuda_ops.set_glu_epilogue(True, backward=GLU_BWD_DEFAULT)
        _done()
        outs.append((y.detach().float(), [t.grad.float() for t in ps], launches,
                     ps[3]._fp8_sites["x"].buf.clone()))
    (y0, g0, n0, h0), (y1, g1, n1, h1) = outs
    assert n1 == n0 - 1, (n0, n1)                                 # one kernel fewer in the forward
    assert torch.equal(h0, h1), (h0, h1)                          # same amax history of the gated activation
    assert torch.equal(y0, y1)
    for a, b, name in zip(g0, g1, ("dx", "dwn", "dw12", "dw3", "db3")):
        assert torch.equal(a, b), name
