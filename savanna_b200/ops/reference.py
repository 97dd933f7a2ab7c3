"""fp32-capable PyTorch statements of every operator: the numerical oracle of the CUDA kernels and the
implementation used on CPU tensors.

Layout convention of the whole framework: activations are channel-last `[B, L, C]`; the Hyena
projections are one `[B, L, 3*D]` tensor whose channels are interleaved `(d, p)` with p in
(x1, x2, v), i.e. x1 = feat[..., 0::3], x2 = feat[..., 1::3], v = feat[..., 2::3]
(reference split: savanna/model/block.py:879-888).

Math sources in the reference: RMSNorm savanna/model/operators/local/norms.py:68-88; depthwise causal
conv savanna/model/operators/hyena/hyena.py:136-181; Hyena-SE hyena.py:845-852; Hyena-MR / -LI
hyena.py:536-555 with savanna/ops/fftconv.py:11-60; modal filter
savanna/model/operators/hyena/parametrization/implicit_modal.py:265-274; explicit decay filter
parametrization/explicit.py:40-75; RoPE savanna/model/operators/positional_embeddings.py:240-259.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


# ----------------------------------------------------------------------------- norms


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, form: str = "te") -> torch.Tensor:
    xf = x.float()
    if form == "te":
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    else:  # eps added to the rms, outside the square root
        rms = xf.norm(2, dim=-1, keepdim=True) * (x.shape[-1] ** -0.5)
        y = xf / (rms + eps)
    return (y * weight.float()).to(x.dtype)


def layernorm(x, weight, bias, eps):
    return F.layer_norm(x.float(), (x.shape[-1],), weight.float(), None if bias is None else bias.float(), eps).to(x.dtype)


# ----------------------------------------------------------------------------- linear


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    return F.linear(x, w, bias)


# ----------------------------------------------------------------------------- short convs


def causal_conv1d(x: torch.Tensor, w: torch.Tensor, halo: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Depthwise causal correlation, channel-last.

    x [B, L, C]; w [C, k] in `F.conv1d` tap order (w[:, k-1] multiplies the current sample);
    halo [B, k-1, C] holds the samples preceding x (zeros when None).  Returns [B, L, C].
    """
    B, L, C = x.shape
    k = w.shape[-1]
    xt = x.transpose(1, 2)
    if halo is None:
        xt = F.pad(xt, (k - 1, 0))
    else:
        xt = torch.cat([halo.transpose(1, 2).to(x.dtype), xt], dim=-1)
    y = F.conv1d(xt.float(), w.float().unsqueeze(1), groups=C)
    return y.transpose(1, 2).to(x.dtype)


def split_features(feat: torch.Tensor, interleaved: bool = True):
    if interleaved:
        return feat[..., 0::3], feat[..., 1::3], feat[..., 2::3]
    return feat.chunk(3, dim=-1)


def hyena_se_inner(feat: torch.Tensor, w: torch.Tensor, halo: Optional[torch.Tensor] = None,
                   pregate: bool = True, postgate: bool = True) -> torch.Tensor:
    """z = x1 * conv_k(x2 * v); w [G, k] shared by the D/G channels of a group (conv1d tap order).
    halo [B, k-1, 3D] = the features preceding `feat`."""
    x1, x2, v = split_features(feat)
    D = x1.shape[-1]
    G = w.shape[0]
    wc = w.repeat_interleave(D // G, dim=0)
    z = x2 * v if pregate else v
    hz = None
    if halo is not None:
        h1, h2, hv = split_features(halo)
        hz = h2 * hv if pregate else hv
    z = causal_conv1d(z, wc, hz)
    return x1 * z if postgate else z


def fir_causal(u: torch.Tensor, h: torch.Tensor, halo: Optional[torch.Tensor] = None) -> torch.Tensor:
    """True causal convolution y[t] = sum_s h[c, s] u[t-s, c]; u [B, L, C], h [C, k]."""
    return causal_conv1d(u, h.flip(-1), halo)


def hyena_mr_inner(feat: torch.Tensor, h: torch.Tensor, bias: torch.Tensor,
                   halo: Optional[torch.Tensor] = None) -> torch.Tensor:
    """z = x1 * ( (h * (x2 v))_causal + bias * (x2 v) ); h [G, k] convolution-order taps, bias [D]."""
    x1, x2, v = split_features(feat)
    D = x1.shape[-1]
    G = h.shape[0]
    hc = h.repeat_interleave(D // G, dim=0)
    u = (x2 * v)
    hu = None
    if halo is not None:
        _, h2, hv = split_features(halo)
        hu = h2 * hv
    y = fir_causal(u.float(), hc.float(), None if hu is None else hu.float())
    y = y + bias.float() * u.float()
    return (x1.float() * y).to(feat.dtype)


def fft_causal_conv(u: torch.Tensor, h: torch.Tensor) -> torch.Tensor:
    """u [B, L, C] fp32, h [C, Lh] fp32 -> causal convolution via a size-2L real FFT (fftconv.py:42-52)."""
    L = u.shape[1]
    n = 2 * L
    uf = torch.fft.rfft(u.float().transpose(1, 2), n=n)
    hf = torch.fft.rfft(h.float()[..., :L], n=n)
    y = torch.fft.irfft(uf * hf, n=n)[..., :L]
    return y.transpose(1, 2)


def fft_bidirectional_conv(u: torch.Tensor, h_fwd: torch.Tensor, h_bwd: torch.Tensor) -> torch.Tensor:
    """The reference's `bidirectional` long convolution (fftconv.py:19-38), stated as it computes it: with U, K1, K2 the
    size-2L real FFTs of the input and of the two filter halves,  y = irfft(U K1 + conj(U K2))[:L].  The first term is
    the causal convolution with h_fwd; conjugating a spectrum reverses the (circular, length 2L) signal in time, so the
    second term is c[(2L - t) mod 2L] with c the linear convolution of u and h_bwd: positions t >= 1 see c[2L - t], the
    part of that convolution that extends past the end of the sequence.  u [B, L, C], filters [C, Lh]."""
    L = u.shape[1]
    n = 2 * L
    uf = torch.fft.rfft(u.float().transpose(1, 2), n=n)
    k1 = torch.fft.rfft(h_fwd.float()[..., :L], n=n)
    k2 = torch.fft.rfft(h_bwd.float()[..., :L], n=n)
    y = torch.fft.irfft(uf * k1 + (uf * k2).conj(), n=n)[..., :L]
    return y.transpose(1, 2)


def hyena_long_fft_bidirectional(feat: torch.Tensor, h: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """Hyena long convolution with a two-sided filter h [2*G, L]: rows [:G] act forward, rows [G:] through the
    conjugate term of `fft_bidirectional_conv`."""
    x1, x2, v = split_features(feat)
    D = x1.shape[-1]
    G = h.shape[0] // 2
    hf, hb = h[:G], h[G:]
    if G != D:
        hf, hb = hf.repeat_interleave(D // G, dim=0), hb.repeat_interleave(D // G, dim=0)
    u = (x2 * v).float()
    y = fft_bidirectional_conv(u, hf, hb) + bias.float() * u
    return (x1.float() * y).to(feat.dtype)


def hyena_multihead(feat: torch.Tensor, h: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """Outer-product ("slow") heads of the Hyena operator (reference: operators/hyena/hyena.py:361-406).  The width D is
    H heads of d channels (channel = head * d + i), one filter h [H, L] and one bias [H] per head:
        kv[i, j] = x2[head, i] * v[head, j]                      (d x d per head and position)
        o[i, j]  = causal_conv(kv[i, j], h[head]) + bias[head] * kv[i, j]
        z[head, j] = sum_i x1[head, i] * o[i, j]
    feat [B, L, 3D] interleaved -> [B, L, D]."""
    x1, x2, v = split_features(feat)
    B, L, D = x1.shape
    H = h.shape[0]
    d = D // H
    q = x1.float().reshape(B, L, H, d)
    k = x2.float().reshape(B, L, H, d)
    vv = v.float().reshape(B, L, H, d)
    kv = k.unsqueeze(-1) * vv.unsqueeze(-2)                                   # [B, L, H, d(i), d(j)]
    hc = h.float().repeat_interleave(d * d, dim=0)                            # one filter row per (head, i, j)
    o = fft_causal_conv(kv.reshape(B, L, H * d * d), hc).reshape(B, L, H, d, d)
    o = o + bias.float().view(1, 1, H, 1, 1) * kv
    z = (q.unsqueeze(-1) * o).sum(-2)                                         # [B, L, H, d(j)]
    return z.reshape(B, L, D).to(feat.dtype)


def modal_filter(gamma: torch.Tensor, R: torch.Tensor, p: torch.Tensor, L: int, t0: int = 0) -> torch.Tensor:
    """h[d, t] = sum_o R[d,o] exp(-exp(p[d,o]) exp(gamma[d,o]) t), t = t0..t0+L-1 (fp32) -> [D, L]."""
    t = torch.arange(t0, t0 + L, device=gamma.device, dtype=torch.float32)
    logp = -torch.exp(p.float()) * torch.exp(gamma.float())           # [D, O], log of the pole
    return (R.float().unsqueeze(-1) * torch.exp(logp.unsqueeze(-1) * t)).sum(1)


def hyena_long_fft(feat: torch.Tensor, h: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """Hyena long convolution with an explicit filter h [D or G, L]."""
    x1, x2, v = split_features(feat)
    D = x1.shape[-1]
    if h.shape[0] != D:
        h = h.repeat_interleave(D // h.shape[0], dim=0)
    u = (x2 * v).float()
    y = fft_causal_conv(u, h) + bias.float() * u
    return (x1.float() * y).to(feat.dtype)


def hyena_li_modal(feat: torch.Tensor, gamma: torch.Tensor, R: torch.Tensor, p: torch.Tensor,
                   bias: torch.Tensor, state_in: Optional[torch.Tensor] = None,
                   return_state: bool = False):
    """Hyena-LI with the implicit modal filter, evaluated through the filter's FFT form.

    With `state_in` [B, D, O] (the modal state left by the preceding part of the sequence, s_o =
    sum_{j<0} lam_o^{-1-j} u[j]) the contribution lam_o^{t+1} R_o s_o is added, which makes the op
    exact on a sequence shard.  `return_state` also returns the state after the last sample.
    """
    x1, x2, v = split_features(feat)
    B, L, D = x1.shape
    u = (x2 * v).float()
    h = modal_filter(gamma, R, p, L)
    y = fft_causal_conv(u, h) + bias.float() * u
    logp = -torch.exp(p.float()) * torch.exp(gamma.float())           # [D, O]
    t = torch.arange(1, L + 1, device=feat.device, dtype=torch.float32)
    if state_in is not None:
        # y[t] += sum_o R_o lam_o^{t+1} s_o
        decay = torch.exp(logp.unsqueeze(0) * t.view(L, 1, 1))         # [L, D, O]
        y = y + torch.einsum("ldo,bdo->bld", decay * R.float().unsqueeze(0), state_in.float())
    out = (x1.float() * y).to(feat.dtype)
    if not return_state:
        return out
    # s_out[o] = lam^L s_in + sum_j lam^{L-1-j} u[j]
    w = torch.exp(logp.unsqueeze(0) * (L - t).view(L, 1, 1))           # lam^{L-1-j}, j = 0..L-1
    s_out = torch.einsum("ldo,bld->bdo", w, u)
    if state_in is not None:
        s_out = s_out + torch.exp(logp * L).unsqueeze(0) * state_in.float()
    return out, s_out


# ----------------------------------------------------------------------------- attention / rope


def rope_tables(positions: torch.Tensor, dim: int, base: float = 10000.0, scaling: float = 1.0):
    """cos/sin tables [L, dim] for rotate-half RoPE; `scaling` divides positions (linear interpolation)."""
    inv = 1.0 / (base ** (torch.arange(0, dim, 2, device=positions.device, dtype=torch.float32) / dim))
    ang = torch.outer(positions.float() / scaling, inv)
    emb = torch.cat([ang, ang], dim=-1)
    return emb.cos(), emb.sin()


def rotate_half(x):
    a, b = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat([-b, a], dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [B, L, H, hd]; cos/sin [L, rd] with rd <= hd (partial rotary leaves the tail untouched)."""
    rd = cos.shape[-1]
    xr, xp = x[..., :rd], x[..., rd:]
    c, s = cos[None, :, None, :].to(torch.float32), sin[None, :, None, :].to(torch.float32)
    y = xr.float() * c + rotate_half(xr.float()) * s
    return torch.cat([y.to(x.dtype), xp], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True,
              q_pos: Optional[torch.Tensor] = None, k_pos: Optional[torch.Tensor] = None,
              return_lse: bool = False, bias: Optional[torch.Tensor] = None):
    """softmax(q k^T / sqrt(hd) + bias) v; q [B, Lq, H, hd], k/v [B, Lk, H, hd], bias [H, Lq, Lk] (ALiBi or a
    relative-position table).  With q_pos/k_pos (global positions) the causal mask is q_pos >= k_pos, which covers
    zigzag shards."""
    B, Lq, H, hd = q.shape
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) / math.sqrt(hd)
    if bias is not None:
        s = s + bias.float()[None]
    if causal:
        if q_pos is None:
            q_pos = torch.arange(Lq, device=q.device) + (k.shape[1] - Lq)
        if k_pos is None:
            k_pos = torch.arange(k.shape[1], device=q.device)
        mask = q_pos[:, None] >= k_pos[None, :]
        s = s.masked_fill(~mask[None, None], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    pr = torch.exp(s - lse.unsqueeze(-1))
    pr = torch.nan_to_num(pr, nan=0.0)
    o = torch.einsum("bhqk,bkhd->bqhd", pr, v.float()).to(q.dtype)
    if return_lse:
        return o, lse
    return o


# ----------------------------------------------------------------------------- mlp / loss


def glu_act(a: torch.Tensor, b: torch.Tensor, act: str = "silu") -> torch.Tensor:
    af = a.float()
    if act == "silu" or act == "swish":
        g = F.silu(af)
    elif act == "gelu":
        g = F.gelu(af)
    elif act == "relu":
        g = F.relu(af)
    elif act == "identity":
        g = af
    else:
        raise ValueError(f"unknown gate activation {act!r}")
    return (g * b.float()).to(a.dtype)


def cross_entropy(logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    """Per-token CE in fp32; logits [..., V], labels [...]."""
    return F.cross_entropy(logits.float().reshape(-1, logits.shape[-1]), labels.reshape(-1), reduction="none").view(labels.shape)


def adam_step(master, exp_avg, exp_avg_sq, grad, lr, beta1, beta2, eps, weight_decay, step, adamw=True,
              grad_scale: float = 1.0, param_out: Optional[torch.Tensor] = None):
    """One Adam(W) step on fp32 flat tensors; writes the low-precision copy into `param_out`."""
    g = grad.float() * grad_scale
    if weight_decay != 0.0 and not adamw:
        g = g + weight_decay * master
    exp_avg.mul_(beta1).add_(g, alpha=1 - beta1)
    exp_avg_sq.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    denom = (exp_avg_sq / bc2).sqrt_().add_(eps)
    upd = (exp_avg / bc1) / denom
    if weight_decay != 0.0 and adamw:
        upd = upd + weight_decay * master
    master.add_(upd, alpha=-lr)
    if param_out is not None:
        param_out.copy_(master)
