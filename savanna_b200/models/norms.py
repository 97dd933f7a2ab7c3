"""Normalisation layers.

`RMSNorm` has two forms.  "te": y = w * x * rsqrt(mean(x^2)+eps), parameter `weight` (what the
reference runs when `use_fp8_norm` selects TransformerEngine's RMSNorm, local/norms.py:22-34).
"classic": y = scale * x / (rms + eps) with eps outside the square root, parameter `scale`
(local/norms.py:68-88).  Both run the same fused kernel on CUDA.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-8, form: str = "te", dtype=None, device=None):
        super().__init__()
        self.eps, self.form, self.dim = eps, form, dim
        w = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))
        if form == "te":
            self.weight = w
        else:
            self.scale = w
        w.is_norm_param = True

    @property
    def gain(self):
        return self.weight if self.form == "te" else self.scale

    def forward(self, x):
        return ops.rmsnorm(x, self.gain, self.eps, self.form)

    def forward_with_residual(self, x):
        """(norm(x), x for the residual branch)."""
        return ops.rmsnorm_residual(x, self.gain, self.eps, self.form)


class ScaleNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5, dtype=None, device=None):
        super().__init__()
        self.g = nn.Parameter(torch.ones(1, dtype=dtype, device=device))
        self.g.is_norm_param = True
        self.eps = eps

    def forward(self, x):
        n = torch.norm(x.float(), dim=-1, keepdim=True).clamp(min=self.eps)
        return (x.float() * (self.g.float() / n)).to(x.dtype)


class LayerNorm(nn.LayerNorm):
    def __init__(self, dim, eps=1e-5, dtype=None, device=None):
        super().__init__(dim, eps=eps, dtype=dtype, device=device)
        self.weight.is_norm_param = True
        self.bias.is_norm_param = True


def get_norm(cfg, dtype=None, device=None) -> nn.Module:
    if cfg.norm == "rmsnorm":
        return RMSNorm(cfg.hidden_size, cfg.rms_norm_epsilon, cfg.rmsnorm_form, dtype, device)
    if cfg.norm == "layernorm":
        return LayerNorm(cfg.hidden_size, cfg.layernorm_epsilon, dtype, device)
    if cfg.norm == "scalenorm":
        return ScaleNorm(cfg.hidden_size, cfg.scalenorm_epsilon, dtype, device)
    raise ValueError(f"norm {cfg.norm!r} not recognised")
