"""Hyena filter parametrisations.

ExplicitSingleDecayFilter (Hyena-MR): h[g,t] = h_hat[g,t] * exp(-alpha_g * t/(L_cache-1)),
alpha = logspace(r_min, r_max, G_global) sliced by tensor-parallel rank
(reference: parametrization/explicit.py:15-75).
ImplicitModalFilter (Hyena-LI): h[d,t] = sum_o R[d,o] exp(-exp(p) exp(gamma) t)
(parametrization/implicit_modal.py:220-282).  The modal form is an order-`order` diagonal linear
recurrence, which is what the CUDA kernel evaluates; `forward(L)` materialises h only for the oracle,
for filter inspection and for checkpoint tools.
Other classes of the reference (real modal, complex modal, free-form sine MLP) are provided for
configuration parity and evaluate through the generic FFT long-convolution path.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from ..ops import reference as ref
from ..parallel import state

_PRESETS = {"strong": (0, 2), "normal": (-1, 2), "weak": (-2, 2)}


def _tp_slice(full: torch.Tensor) -> torch.Tensor:
    """Rows of a tensor drawn at the global (all tensor-parallel ranks) size that belong to this rank.
    Drawing globally and slicing keeps the initial model identical for every tensor-parallel size."""
    tp, rank = state.get_model_parallel_world_size(), state.get_model_parallel_rank()
    return full.chunk(tp, dim=0)[rank].contiguous() if tp > 1 else full


class ExplicitSingleDecayFilter(nn.Module):
    def __init__(self, d_model: int, L_cache: int, decay_preset: str = "strong", num_decay_repeats: int = 1,
                 small_init: bool = True, unit_passthrough: bool = False, device=None):
        super().__init__()
        if decay_preset not in _PRESETS:
            raise ValueError(f"decay preset {decay_preset!r} unknown")
        r_min, r_max = _PRESETS[decay_preset]
        tp_ = state.get_model_parallel_world_size()
        h = _tp_slice(torch.randn(d_model * tp_, L_cache, device=device)) / math.sqrt(L_cache)
        if small_init:
            h = h * 1e-5
        if unit_passthrough:
            h[:, :1] = 1.0
        self.h = nn.Parameter(h)
        self.h.is_filter_param = True
        tp, rank = state.get_model_parallel_world_size(), state.get_model_parallel_rank()
        global_d = d_model * tp // num_decay_repeats
        alpha = torch.logspace(r_min, r_max, global_d)[:, None].repeat(num_decay_repeats, 1)
        alpha = alpha[rank * d_model:(rank + 1) * d_model]
        t = torch.linspace(0, 1, L_cache)[None]
        self.register_buffer("decay", torch.exp(-alpha * t).to(device))

    def forward(self, L: int):
        return self.h[:, :L] * self.decay[:, :L]

    filter = forward


class ImplicitModalFilter(nn.Module):
    def __init__(self, d_model: int, order: int = 64, L_cache: int = None, gamma_min: float = 0.01,
                 gamma_max: float = 0.1, device=None):
        super().__init__()
        self.order, self.d_model = order, d_model
        self.register_buffer("t", torch.arange(L_cache or 1, dtype=torch.float32, device=device).view(1, 1, -1))
        tp_ = state.get_model_parallel_world_size()
        gamma = _tp_slice(torch.rand(d_model * tp_, order, dtype=torch.float32, device=device)) * (gamma_max - gamma_min) + gamma_min
        self.gamma = nn.Parameter(gamma.log())
        self.R = nn.Parameter(1e-1 * _tp_slice(torch.randn(d_model * tp_, order, dtype=torch.float32, device=device)) / math.sqrt(order))
        self.p = nn.Parameter(-torch.ones(d_model, order, dtype=torch.float32, device=device))
        for q in (self.gamma, self.R, self.p):
            q.is_filter_param = True

    def forward(self, L: int):
        return ref.modal_filter(self.gamma, self.R, self.p, L)

    filter = forward


def _tp_slice_dim(full: torch.Tensor, dim: int) -> torch.Tensor:
    """As `_tp_slice`, along another dimension."""
    tp, rank = state.get_model_parallel_world_size(), state.get_model_parallel_rank()
    return full.chunk(tp, dim=dim)[rank].contiguous() if tp > 1 else full


class ImplicitRealModalFilter(nn.Module):
    """Real decaying modes with factored poles and residues (reference: parametrization/implicit_modal.py:11-83):

        h[d, t] = sum_o (prod_f R[o, d, f]) * pole[o, d] ^ (dt[o, d] * t),   pole = exp(-exp(prod_f p[o, d, f]))

    with dt clamped to [dt_min, dt_max] and t = linspace(0, L, L) (L points from 0 to L inclusive, the reference's time
    grid).  Parameters as in the reference: `dt` [order, d], `p` [order, d, pole_factors] (one draw per mode, shared by
    the channels at start), `R` [order, d, residue_factors] ~ N(0, 1 / order), and the unused `residues_norm`."""

    def __init__(self, d_model, order=64, L_cache=None, dt_min=0.001, dt_max=0.1, residue_factors=4, pole_factors=4,
                 device=None):
        super().__init__()
        self.order, self.d_model, self.dt_min, self.dt_max = order, d_model, dt_min, dt_max
        tp_ = state.get_model_parallel_world_size()
        dt = torch.rand(order, d_model * tp_, device=device) * (dt_max - dt_min) + dt_min
        self.dt = nn.Parameter(_tp_slice_dim(dt, 1))
        start = torch.randn(order, pole_factors, device=device)
        self.p = nn.Parameter(start[:, None, :].repeat(1, d_model, 1))
        R = torch.randn(order, d_model * tp_, residue_factors, device=device) / math.sqrt(order)
        self.R = nn.Parameter(_tp_slice_dim(R, 1))
        self.residues_norm = nn.LayerNorm(d_model, device=device)
        for q in self.parameters():
            q.is_filter_param = True

    def forward(self, L: int):
        R = self.R.float().prod(dim=-1)
        dt = torch.clamp(self.dt.float(), min=self.dt_min, max=self.dt_max)[..., None]
        log_pole = -torch.exp(self.p.float().prod(dim=-1))          # log of the pole, without forming a pole that underflows
        t = torch.linspace(0, L, L, device=R.device)[None, None]
        return torch.sum(R.unsqueeze(-1) * torch.exp(t * dt * log_pole.unsqueeze(-1)), dim=0)

    filter = forward


class _ComplexModalParameters(nn.Module):
    """Holder of the complex modal filter's parameters under the reference's names (`inner_cls.*`,
    parametrization/implicit_complex.py:11-30): C and B as real views of complex tensors, A = -exp(inv_A_real) + i A_imag."""

    def __init__(self, A, B, C, log_dt):
        super().__init__()
        self.C = nn.Parameter(torch.view_as_real(C.conj().resolve_conj()))
        self.log_dt = nn.Parameter(log_dt)
        self.inv_A_real = nn.Parameter(torch.log(-A.real))
        self.A_imag = nn.Parameter(A.imag)
        self.B = nn.Parameter(torch.view_as_real(B.conj().resolve_conj()))


class ParallelComplexModalFilter(nn.Module):
    """Complex diagonal modes (reference: parametrization/implicit_complex.py:35-97):

        h[d, t] = 2 Re sum_n C[d, n] exp(dt[d] * A[d, n] * t),   A = -exp(inv_A_real) + i A_imag

    started at A = -1/2 + i pi n, dt log-uniform in [dt_min, dt_max], C complex normal; B is carried (all ones) and, as
    in the reference, does not enter the filter."""

    def __init__(self, d_model, order=64, dt_min=0.001, dt_max=0.1, device=None):
        super().__init__()
        self.d_model, self.order = d_model, order
        half = max(1, order // 2)
        tp_ = state.get_model_parallel_world_size()
        log_dt = _tp_slice(torch.rand(d_model * tp_, device=device)) * (math.log(dt_max) - math.log(dt_min)) + math.log(dt_min)
        A = -0.5 * torch.ones(d_model, half, device=device) + 1j * math.pi * torch.arange(half, device=device).repeat(d_model, 1)
        B = torch.ones(d_model, half, dtype=torch.cfloat, device=device)
        C = _tp_slice_dim(torch.randn(1, d_model * tp_, half, dtype=torch.cfloat, device=device), 1)
        self.inner_cls = _ComplexModalParameters(A, B, C, log_dt)
        for q in self.parameters():
            q.is_filter_param = True

    def forward(self, L: int):
        m = self.inner_cls
        dt = torch.exp(m.log_dt.float())
        C = torch.view_as_complex(m.C.float().contiguous())[0]                     # [d, n]
        A = -torch.exp(m.inv_A_real.float()) + 1j * m.A_imag.float()
        dtA = A * dt.unsqueeze(-1)
        t = torch.arange(L, device=dt.device)
        return 2 * torch.einsum("dn,dnl->dl", C, torch.exp(dtA.unsqueeze(-1) * t)).real

    filter = forward


class _Sin(nn.Module):
    """sin(freq * x) with one trainable frequency per feature (reference: savanna/model/activations.py:12-19)."""

    def __init__(self, dim, w, device=None):
        super().__init__()
        self.freq = nn.Parameter(w * torch.ones(1, dim, device=device))

    def forward(self, x):
        return torch.sin(self.freq * x)


class _FixedFourierEmbedding(nn.Module):
    """Buffers `z` [1, L, emb_dim] = [t, Re e^{-i f w}, Im e^{-i f w}] and `t` [1, L, 1] in [0, 1]
    (implicit_utils.py:12-38); w = 2 pi n / L, f = `bands` frequencies from 1e-4 to bands - 1."""

    def __init__(self, emb_dim, seq_len, device=None):
        super().__init__()
        if emb_dim % 2 == 0 or emb_dim < 3:
            raise ValueError("emb_dim must be odd and >= 3 (time + sine/cosine pairs)")
        bands = (emb_dim - 1) // 2
        t = torch.linspace(0, 1, seq_len, device=device)[None, :, None]
        w = 2 * math.pi * torch.linspace(0, seq_len - 1, seq_len, device=device)[None, :, None] / seq_len
        f = torch.linspace(1e-4, bands - 1, bands, device=device)[None, None]
        self.register_buffer("t", t)
        self.register_buffer("z", torch.cat([t, torch.cos(f * w), -torch.sin(f * w)], dim=-1))

    def forward(self, L):
        return self.z[:, :L], self.t[:, :L]


class _RandomFourierEmbedding(nn.Module):
    """Learned frequencies drawn from N(0, 2 pi omega_0): features [cos(w t), sin(w t)] on t in [-1, 1]; the decay
    window sees (t + 1) / 2 (implicit_utils.py:39-67)."""

    def __init__(self, emb_dim, seq_len, omega_0, device=None):
        super().__init__()
        if emb_dim % 2:
            raise ValueError(f"emb_dim must be even for the random Fourier embedding (got {emb_dim})")
        self.linear = nn.Linear(1, emb_dim // 2, bias=False, device=device)
        with torch.no_grad():
            self.linear.weight.normal_(0.0, 2 * math.pi * omega_0)
        self.register_buffer("t", torch.linspace(-1, 1, seq_len, device=device)[None, :, None])

    def forward(self, L):
        out = self.linear(self.t[:, :L])
        return torch.cat([torch.cos(out), torch.sin(out)], dim=-1), (self.t[:, :L] + 1) / 2


class _ExponentialModulation(nn.Module):
    """h * exp(-t |weight|): per-channel decay rates, spread linearly between a slow and a fast one that reach 1e-2 at
    `slow_decay` / `fast_decay` of the sequence; trainable, as in the reference (implicit_utils.py:70-111)."""

    def __init__(self, d_model, fast_decay=0.3, slow_decay=1.5, target=1e-2, device=None):
        super().__init__()
        max_decay, min_decay = math.log(target) / fast_decay, math.log(target) / slow_decay
        self.weight = nn.Parameter(torch.linspace(min_decay, max_decay, d_model, device=device)[None, None])

    def forward(self, t, x):
        return x * torch.exp(-t * self.weight.abs())


class ParallelImplicitFreeformFilter(nn.Module):
    """Sine-activated MLP over a positional embedding, modulated by an exponential decay window
    (parametrization/implicit_freeform.py:15-122).  Sub-module and parameter names are the reference's, so its
    checkpoints load: `pos_emb.{z,t}` (or `pos_emb.linear.weight`), `act.freq`, `implicit_filter.<2i>.{weight,bias}`
    (the shared activation sits at the odd positions), `final_filter.weight`, `modulation.weight`,
    `post_modulation_norm.*`.

    pos_emb "fourier_fixed": fixed complex-exponential features (emb_dim odd); "random_fourier": learned frequencies
    (emb_dim even, scale `omega_0`).  `normalized` applies a LayerNorm over the channels after the decay window."""

    def __init__(self, d_model, emb_dim=33, order=64, num_inner_mlps=2, w=14, L_cache=8192, fast_decay=0.3,
                 slow_decay=1.2, modulate=True, pos_emb="fourier_fixed", omega_0=1.0, normalized=False, device=None):
        super().__init__()
        self.w, self.modulate, self.pos_emb_type = w, modulate, pos_emb
        if pos_emb == "fourier_fixed":
            self.pos_emb = _FixedFourierEmbedding(emb_dim, L_cache, device=device)
        elif pos_emb == "random_fourier":
            self.pos_emb = _RandomFourierEmbedding(emb_dim, L_cache, omega_0, device=device)
        else:
            raise ValueError(f"hyena_pos_emb {pos_emb!r} unknown (fourier_fixed | random_fourier)")
        self.act = _Sin(order, w, device=device)
        layers = [nn.Linear(emb_dim, order, device=device), self.act]
        for _ in range(num_inner_mlps):
            layers += [nn.Linear(order, order, device=device), self.act]
        self.implicit_filter = nn.Sequential(*layers)
        self.final_filter = nn.Linear(order, d_model, bias=False, device=device)
        nn.init.xavier_normal_(self.final_filter.weight, gain=1)
        self.modulation = _ExponentialModulation(d_model, fast_decay, slow_decay, device=device)
        self.post_modulation_norm = nn.LayerNorm(d_model, device=device) if normalized else None
        for q in self.parameters():
            q.is_filter_param = True

    def forward(self, L: int):
        z, t = self.pos_emb(L)
        h = self.final_filter(self.implicit_filter(z))
        if self.modulate:
            h = self.modulation(t, h)
        if self.post_modulation_norm is not None:
            h = self.post_modulation_norm(h)
        return h[0].transpose(0, 1).float()

    filter = forward


def build_filter(cfg, operator_type: str, num_groups: int, device=None) -> nn.Module:
    cls = cfg.hyena_filter_cls
    if operator_type == "hyena_mr" and cfg.hyena_medium_filter_cls is not None:
        cls = cfg.hyena_medium_filter_cls
    if cls == "explicit_single_decay":
        return ExplicitSingleDecayFilter(num_groups, cfg.seq_length, decay_preset=cfg.explicit_filter_decay_preset,
                                         num_decay_repeats=cfg.explicit_filter_num_decay_repeats, device=device)
    if cls == "implicit_modal":
        return ImplicitModalFilter(num_groups, cfg.hyena_filter_order, cfg.seq_length, cfg.modal_gamma_min,
                                   cfg.modal_gamma_max, device=device)
    if cls == "implicit_real_modal":
        return ImplicitRealModalFilter(num_groups, cfg.hyena_filter_order, cfg.seq_length,
                                       residue_factors=cfg.modal_residue_factors, pole_factors=cfg.modal_pole_factors,
                                       device=device)
    # a two-sided (`bidirectional`) operator asks its filter for a forward and a backward half: twice the rows
    two_sided = 2 if cfg.bidirectional and operator_type == "hyena" else 1
    if two_sided == 2 and cls not in ("implicit_complex_modal", "implicit", "implicit_freeform"):
        raise ValueError(f"bidirectional needs an implicit free-form or complex modal filter (got {cls!r})")
    if cls == "implicit_complex_modal":
        return ParallelComplexModalFilter(num_groups * two_sided, cfg.hyena_filter_order, device=device)
    if cls in ("implicit", "implicit_freeform"):
        return ParallelImplicitFreeformFilter(num_groups * two_sided, cfg.hyena_filter_emb_dim, cfg.hyena_filter_order,
                                              cfg.hyena_filter_num_inner_mlps, cfg.hyena_filter_w, cfg.seq_length,
                                              cfg.hyena_filter_fast_decay, cfg.hyena_filter_slow_decay,
                                              pos_emb=cfg.hyena_pos_emb, omega_0=cfg.hyena_filter_omega_0,
                                              normalized=cfg.normalize_hyena_filters, device=device)
    raise ValueError(f"hyena filter class {cls!r} unknown")
