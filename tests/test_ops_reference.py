"""Algebraic checks of the oracle operators themselves (the kernels are tested against these)."""
import math

import pytest

import torch

from savanna_b200.ops import reference as ref


def test_causal_conv_matches_explicit_sum():
    torch.manual_seed(0)
    x = torch.randn(2, 20, 3, dtype=torch.float64)
    w = torch.randn(3, 4, dtype=torch.float64)
    y = ref.causal_conv1d(x, w)
    t, c = 7, 1
    exp = sum(w[c, j] * x[0, t - 3 + j, c] for j in range(4))
    assert abs(y[0, t, c] - exp) < 1e-6
    # halo == explicit left context
    y2 = ref.causal_conv1d(x[:, 5:], w, x[:, 2:5])
    assert torch.allclose(y2, y[:, 5:], atol=1e-6)


def test_fft_conv_equals_direct():
    torch.manual_seed(1)
    u = torch.randn(1, 64, 4)
    h = torch.randn(4, 64)
    y = ref.fft_causal_conv(u, h)
    yd = ref.fir_causal(u, h)
    assert torch.allclose(y, yd, atol=1e-4)


def test_modal_state_splits_sequence():
    """Running two halves with the state hand-off equals running the whole sequence."""
    torch.manual_seed(2)
    B, L, D, O = 2, 64, 6, 4
    feat = torch.randn(B, L, 3 * D)
    gamma = (torch.rand(D, O) * 0.09 + 0.01).log()
    R = torch.randn(D, O) * 0.1
    p = -torch.ones(D, O)
    bias = torch.randn(D)
    full = ref.hyena_li_modal(feat, gamma, R, p, bias)
    a, s = ref.hyena_li_modal(feat[:, :32], gamma, R, p, bias, None, True)
    b = ref.hyena_li_modal(feat[:, 32:], gamma, R, p, bias, s)
    assert torch.allclose(torch.cat([a, b], 1), full, atol=1e-4)


def test_rope_is_rotation():
    pos = torch.arange(16)
    cos, sin = ref.rope_tables(pos, 8)
    x = torch.randn(1, 16, 2, 8)
    y = ref.apply_rope(x, cos, sin)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)
    back = ref.apply_rope(y, cos, -sin)
    assert torch.allclose(back, x, atol=1e-5)


def test_attention_matches_sdpa():
    torch.manual_seed(3)
    q, k, v = (torch.randn(2, 12, 3, 8) for _ in range(3))
    o = ref.attention(q, k, v, causal=True)
    exp = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
    assert torch.allclose(o, exp.transpose(1, 2), atol=1e-5)


def test_rmsnorm_forms():
    x = torch.randn(4, 32)
    w = torch.rand(32) + 0.5
    a = ref.rmsnorm(x, w, 1e-6, "te")
    b = ref.rmsnorm(x, w, 1e-6, "classic")
    assert torch.allclose(a, b, atol=1e-4)      # the forms differ only in where eps enters
    assert torch.allclose(a, w * x / x.pow(2).mean(-1, keepdim=True).sqrt(), atol=1e-4)


def test_adam_matches_torch():
    torch.manual_seed(4)
    p0 = torch.randn(100)
    g = torch.randn(100)
    q = torch.nn.Parameter(p0.clone())
    opt = torch.optim.AdamW([q], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m, v, master = torch.zeros(100), torch.zeros(100), p0.clone()
    for step in (1, 2, 3):
        q.grad = g.clone()
        opt.step()
        ref.adam_step(master, m, v, g, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, True)
    assert torch.allclose(master, q.detach(), atol=1e-6)


def test_hippo_nplr_and_dplr_initialisers():
    """HiPPO matrices: A + P^T P is normal for every measure; the kept half of the spectrum with its conjugate rebuilds
    the matrix; LegS has the known diagonal; the DPLR layouts have the documented poles."""
    from savanna_b200.models import ssm_init as si
    N = 16
    for measure in ("legs", "legt", "lagt", "fourier"):
        A, B = si.transition(measure, N)
        P = si.rank_correction(measure, N, rank=2 if measure == "legt" else 1)
        AP = A + (P[:, :, None] * P[:, None, :]).sum(0)
        assert torch.allclose(AP @ AP.t(), AP.t() @ AP, atol=1e-8), measure
        w, Pc, Bc, V = si.nplr(measure, N, rank=P.shape[0], dtype=torch.float64)
        assert w.shape == (N // 2,) and (w.imag >= -1e-9).all()
        full = (V * w) @ V.conj().t()
        rebuilt = 2 * full.real if measure != "lagt" else None
        if rebuilt is not None and (w.imag.abs() > 1e-6).all():
            assert torch.allclose(rebuilt, AP, atol=1e-6), measure
    A, _ = si.transition("legs", 4)
    assert torch.allclose(torch.diagonal(A), -torch.arange(1, 5, dtype=torch.float64))
    assert float(A[2, 1]) == pytest.approx(-(5 ** 0.5) * (3 ** 0.5))
    w, P, B, V = si.dplr("linear", N=8, H=3)
    assert w.shape == (3, 4) and torch.allclose(w.real, torch.full((3, 4), -0.5))
    assert torch.allclose(w.imag[0], math.pi * torch.arange(4.0))
    assert float(P.abs().sum()) == 0.0 and V.shape == (3, 8, 4)
    w2, *_ = si.ssm("diag-inv", 8, 1, 2)
    assert w2.shape == (2, 4)
    wc, Pc, Bc, Vc = si.combination("diag", 8, 1, 4)
    assert wc.shape == (4, 4) and Pc.shape == (1, 4, 4) and Vc.shape == (4, 8, 4)
    E = si.embed_c2r(torch.tensor([[1 + 2j]]))
    assert torch.equal(E, torch.tensor([[1.0, -2.0], [2.0, 1.0]]))


def test_bidirectional_long_convolution_matches_its_time_domain_statement():
    """y[t] = sum_{j<=t} h1[t-j] u[j] + c2[(2L - t) mod 2L], c2 the linear convolution of u with the second half."""
    import torch
    from savanna_b200.ops import reference as ref
    torch.manual_seed(0)
    B, L, D = 2, 12, 4
    feat = torch.randn(B, L, 3 * D, dtype=torch.float64)
    h = torch.randn(2 * D, L, dtype=torch.float64)
    bias = torch.randn(D, dtype=torch.float64)
    got = ref.hyena_long_fft_bidirectional(feat, h, bias).double()
    x1, x2, v = ref.split_features(feat)
    u = x2 * v
    want = torch.zeros(B, L, D, dtype=torch.float64)
    for d in range(D):
        for b in range(B):
            c1 = torch.zeros(2 * L, dtype=torch.float64)
            c2 = torch.zeros(2 * L, dtype=torch.float64)
            for j in range(L):
                for k in range(L):
                    c1[j + k] += u[b, j, d] * h[d, k]
                    c2[j + k] += u[b, j, d] * h[D + d, k]
            for t in range(L):
                want[b, t, d] = c1[t] + c2[(2 * L - t) % (2 * L)]
    want = x1 * (want + bias * u)
    assert torch.allclose(got, want, atol=1e-4), (got - want).abs().max()


def test_multihead_hyena_matches_its_time_domain_statement():
    import torch
    from savanna_b200.ops import reference as ref
    torch.manual_seed(1)
    B, L, H, d = 2, 10, 3, 2
    D = H * d
    feat = torch.randn(B, L, 3 * D, dtype=torch.float64)
    h = torch.randn(H, L, dtype=torch.float64)
    bias = torch.randn(H, dtype=torch.float64)
    got = ref.hyena_multihead(feat, h, bias).double()
    x1, x2, v = ref.split_features(feat)
    want = torch.zeros(B, L, D, dtype=torch.float64)
    for hd in range(H):
        for i in range(d):
            for j in range(d):
                kv = x2[:, :, hd * d + i] * v[:, :, hd * d + j]              # [B, L]
                o = bias[hd] * kv
                for t in range(L):
                    for s in range(t + 1):
                        o[:, t] = o[:, t] + h[hd, t - s] * kv[:, s]
                want[:, :, hd * d + j] += x1[:, :, hd * d + i] * o
    assert torch.allclose(got, want, atol=1e-4), (got - want).abs().max()


def test_freeform_filter_position_embeddings_and_normalisation():
    import torch
    from savanna_b200.models.filters import ParallelImplicitFreeformFilter
    torch.manual_seed(0)
    f = ParallelImplicitFreeformFilter(6, emb_dim=8, order=16, L_cache=64, pos_emb="random_fourier", omega_0=2.0,
                                       normalized=True)
    h = f(48)
    assert h.shape == (6, 48)
    assert torch.allclose(h.mean(0), torch.zeros(48), atol=1e-5)              # LayerNorm over the channels
    names = dict(f.named_parameters())
    assert "pos_emb.linear.weight" in names and "post_modulation_norm.weight" in names
    assert 2.0 < float(names["pos_emb.linear.weight"].std()) < 40.0           # drawn at scale 2 pi omega_0
    h.sum().backward()
    assert names["pos_emb.linear.weight"].grad is not None
    import pytest
    with pytest.raises(ValueError):
        ParallelImplicitFreeformFilter(6, emb_dim=9, pos_emb="random_fourier")
    g = ParallelImplicitFreeformFilter(6, emb_dim=9, order=16, L_cache=64)(32)
    assert g.shape == (6, 32) and float(g[:, -1].abs().max()) < float(g[:, 0].abs().max()) + 1.0


def test_losses_match_their_plain_statements():
    """Lower-case reweighting (target upper-cased, weight from the case), diffusion reweighting and the preference loss's
    per-row log-probability, each against a few lines of plain PyTorch."""
    import torch
    import torch.nn.functional as F
    from savanna_b200.models import losses
    torch.manual_seed(0)
    B, L, V = 3, 12, 128
    logits = torch.randn(B, L, V)
    labels = torch.randint(65, 91, (B, L))
    lower = torch.rand(B, L) < 0.4
    labels = torch.where(lower, labels + 32, labels)
    mask = (torch.rand(B, L) < 0.8).float()
    upper = torch.where(lower, labels - 32, labels)
    ce = F.cross_entropy(logits.view(-1, V), upper.view(-1), reduction="none").view(B, L)
    w = torch.where(lower, 0.1, 1.0) * mask
    got = losses.reweighted_cross_entropy(logits, labels, mask, 0.1, normalize_per_batch=False)
    assert torch.allclose(got, (ce * w).sum() / mask.sum(), atol=1e-6)
    wn = mask.sum() * w / w.sum()
    got = losses.reweighted_cross_entropy(logits, labels, mask, 0.1, normalize_per_batch=True)
    assert torch.allclose(got, (ce * wn).sum() / mask.sum(), atol=1e-6)
    ce_plain = F.cross_entropy(logits.view(-1, V), labels.view(-1), reduction="none").view(B, L)
    labels_p = labels.clone()
    labels_p[0, -3:] = 1                                                  # pad tokens shorten row 0
    ce_p = F.cross_entropy(logits.view(-1, V), labels_p.view(-1), reduction="none").view(B, L)
    want = sum((labels_p[b] != 1).sum() / mask[b].sum() * (ce_p[b] * mask[b]).sum() for b in range(B)) / mask.sum()
    assert torch.allclose(losses.oadm_loss(logits, labels_p, mask), want, atol=1e-5)
    lp = losses.sequence_logps(logits, labels, mask)
    assert torch.allclose(lp, -(ce_plain * mask).mean(-1), atol=1e-6)
    loss, _, _ = losses.dpo_loss(lp[:1], lp[1:2], torch.tensor([-1.0]), torch.tensor([-2.0]), beta=0.5)
    assert torch.allclose(loss, -F.logsigmoid(0.5 * ((lp[0] + 1.0) - (lp[1] + 2.0))), atol=1e-6)
