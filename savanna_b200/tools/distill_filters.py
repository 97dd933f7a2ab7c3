"""Modal distillation of long convolution filters: fit a low-order sum of decaying modes to given filters.

A long filter h [N, L] (one row per channel, e.g. the materialised taps of a trained explicit or free-form Hyena-LI
filter) is approximated by

    complex form   h[0] kept as a pass-through tap;  h[t] = Re( sum_o R_o * lam_o^(t-1) ),  lam_o = r_o e^{i theta_o}, t >= 1
    real form      h[t] = sum_o R_o * exp(-exp(p_o) exp(gamma_o) t),                                                   t >= 0

and the parameters are found by AdamW with a cosine schedule on the mean squared error.  The complex form is the
constant-memory recurrent ("Laughing Hyena") parametrisation; the real form is exactly this framework's
`ImplicitModalFilter`, so `export_implicit_modal` turns a distilled filter into (gamma, R, p) tensors that the
Hyena-LI scan kernels and the cached decoder consume directly: a model trained with an explicit long filter can be
served with the O(order) recurrence.

Role of the reference's notebooks/distill.ipynb (cells 3-5: `LaughingHyenaFilter`, `fit`, `distill_hyena`); here a
module with a command line instead of a notebook, without plots (the per-step loss and the final relative error are
returned and printed).
"""
from __future__ import annotations

import argparse
import math
from typing import Dict, List, Tuple

import torch
from torch import nn


class ComplexModalFilter(nn.Module):
    """order complex poles on a ring r in [r_min, r_max], phase in [0, theta_max]; residues R = R_re + i R_im."""

    def __init__(self, order: int, num_filters: int, r_min: float = 0.9, r_max: float = 0.99, theta_max: float = 2 * math.pi):
        super().__init__()
        self.order, self.num_filters = order, num_filters
        u1, u2 = torch.rand(order, num_filters), torch.rand(order, num_filters)
        self.r = nn.Parameter(r_min + (r_max - r_min) * u1)
        self.theta = nn.Parameter(theta_max * u2)
        self.R_re = nn.Parameter(torch.randn(order, num_filters) * math.sqrt(1.0 / order))
        self.R_im = nn.Parameter(torch.randn(order, num_filters) * math.sqrt(1.0 / order))
        self.register_buffer("h_0", torch.zeros(num_filters, 1))

    def forward(self, L: int) -> torch.Tensor:
        """[num_filters, L - 1]: taps 1 .. L-1 (tap 0 is `h_0`)."""
        t = torch.arange(L - 1, device=self.r.device, dtype=torch.float32)                   # exponent t - 1 = 0 .. L-2
        logmag = torch.log(self.r.clamp_min(1e-8))[..., None] * t                             # [O, N, L-1]
        phase = self.theta[..., None] * t
        mag = torch.exp(logmag)
        re = mag * (self.R_re[..., None] * torch.cos(phase) - self.R_im[..., None] * torch.sin(phase))
        return re.sum(0)

    def filter(self, L: int) -> torch.Tensor:
        return torch.cat([self.h_0.to(self.r.device), self.forward(L)], dim=1)

    @torch.no_grad()
    def step_matrices(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """(lam, R) as complex [N, O] tensors for a recurrent evaluation s <- lam s + u, y = h_0 u + Re(R . s_prev)."""
        lam = torch.polar(self.r, self.theta).t().contiguous()
        return lam, torch.complex(self.R_re, self.R_im).t().contiguous()


class RealModalFilter(nn.Module):
    """Real decaying modes in the parametrisation of `ImplicitModalFilter`: h[t] = sum_o R exp(-exp(p) exp(gamma) t)."""

    def __init__(self, order: int, num_filters: int, gamma_min: float = 0.01, gamma_max: float = 0.1):
        super().__init__()
        self.order, self.num_filters = order, num_filters
        g = torch.rand(num_filters, order) * (gamma_max - gamma_min) + gamma_min
        self.gamma = nn.Parameter(g.log())
        self.R = nn.Parameter(1e-1 * torch.randn(num_filters, order) / math.sqrt(order))
        self.p = nn.Parameter(-torch.ones(num_filters, order))

    def forward(self, L: int) -> torch.Tensor:
        t = torch.arange(L, device=self.R.device, dtype=torch.float32)
        rate = torch.exp(self.p) * torch.exp(self.gamma)                                      # [N, O]
        return (self.R[..., None] * torch.exp(-rate[..., None] * t)).sum(1)

    filter = forward


def fit(target: torch.Tensor, model: nn.Module, epochs: int = 3000, lr: float = 6e-4, log_interval: int = 0,
        device: str = "cpu") -> List[float]:
    """Fit `model` to `target` [N, L]; returns the loss per step."""
    target = target.detach().float().to(device)
    model.to(device)
    L = target.shape[1]
    if isinstance(model, ComplexModalFilter):
        model.h_0 = target[:, :1].clone()
        goal = target[:, 1:]
    else:
        goal = target
    opt = torch.optim.AdamW(model.parameters(), lr=lr, weight_decay=0.0, betas=(0.9, 0.99))
    sched = torch.optim.lr_scheduler.CosineAnnealingWarmRestarts(opt, T_0=max(epochs, 1), T_mult=1, eta_min=1e-6)
    log = []
    for i in range(epochs):
        opt.zero_grad()
        loss = (model(L) - goal).pow(2).mean()
        loss.backward()
        opt.step()
        sched.step()
        log.append(float(loss.detach()))
        if log_interval and i % log_interval == 0:
            print(f"step {i}: loss {log[-1]:.4e}")
    return log


def distill(filters: torch.Tensor, order: int = 16, form: str = "complex", **fit_kw) -> Tuple[List[nn.Module], List[List[float]]]:
    """filters [layers, N, L] (or [N, L]) -> one fitted module per layer and its loss log."""
    if filters.dim() == 2:
        filters = filters[None]
    models, logs = [], []
    for k in range(filters.shape[0]):
        m = ComplexModalFilter(order, filters.shape[1]) if form == "complex" else RealModalFilter(order, filters.shape[1])
        logs.append(fit(filters[k], m, **fit_kw))
        models.append(m)
    return models, logs


@torch.no_grad()
def relative_error(model: nn.Module, target: torch.Tensor) -> float:
    got = model.filter(target.shape[1]).to(target.device)
    return float((got - target.float()).norm() / target.float().norm().clamp_min(1e-12))


@torch.no_grad()
def export_implicit_modal(model: RealModalFilter) -> Dict[str, torch.Tensor]:
    """State-dict entries of `ImplicitModalFilter` (`gamma`, `R`, `p`, each [N, order])."""
    return {"gamma": model.gamma.detach().clone(), "R": model.R.detach().clone(), "p": model.p.detach().clone()}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("filters", help=".pt file holding a tensor [layers, N, L] or [N, L]")
    ap.add_argument("output", help=".pt file to write: per layer the fitted parameters and the relative error")
    ap.add_argument("--order", type=int, default=16)
    ap.add_argument("--form", choices=["complex", "real"], default="complex")
    ap.add_argument("--epochs", type=int, default=30000)
    ap.add_argument("--lr", type=float, default=6e-4)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--log-interval", type=int, default=10000)
    a = ap.parse_args(argv)
    filt = torch.load(a.filters, map_location="cpu")
    if filt.dim() == 2:
        filt = filt[None]
    models, logs = distill(filt, a.order, a.form, epochs=a.epochs, lr=a.lr, device=a.device, log_interval=a.log_interval)
    out = []
    for k, m in enumerate(models):
        err = relative_error(m, filt[k].to(a.device))
        print(f"layer {k}: final loss {logs[k][-1]:.4e}, relative error {err:.4f}")
        out.append({"state": {n: v.detach().cpu() for n, v in m.state_dict().items()}, "form": a.form, "order": a.order,
                    "relative_error": err, "final_loss": logs[k][-1]})
    torch.save(out, a.output)


if __name__ == "__main__":
    main()
