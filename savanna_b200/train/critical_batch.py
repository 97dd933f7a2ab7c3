"""Gradient-noise-scale (critical batch size) estimator, B_simple = tr(Sigma) / |G|^2, from gradient norms at a
small and a large batch size with exponential moving averages (reference: savanna/scaling/critical_batch.py:12-195;
McCandlish et al. 2018, appendix A)."""
from __future__ import annotations

from typing import Optional

import torch


class CriticalBatchEstimator:
    def __init__(self, batch_size_small: int, n_batches: int = 5, beta: float = 0.99, cpu_offload: bool = False):
        self.b_small, self.n_batches, self.beta, self.cpu = batch_size_small, n_batches, beta, cpu_offload
        self.b_big = batch_size_small * n_batches
        self.buffer = None
        self.count = 0
        self.ema_scale: Optional[float] = None
        self.ema_noise: Optional[float] = None
        self.n_updates = 0
        self.noise_scale: Optional[float] = None

    @staticmethod
    def _flat_grad(params) -> torch.Tensor:
        return torch.cat([p.grad.detach().float().reshape(-1) for p in params if p.grad is not None])

    def _ema(self, avg, x):
        if avg is None:
            avg = 0.0
        avg = self.beta * avg + (1 - self.beta) * x
        return avg

    def update(self, params) -> Optional[float]:
        """Call once per small batch, after backward and before the gradients are zeroed."""
        g = self._flat_grad(params)
        if self.cpu:
            g = g.cpu()
        g_small_sq = float(g.pow(2).sum())
        self.buffer = g.clone() if self.buffer is None else self.buffer + g
        self.count += 1
        if self.count < self.n_batches:
            return self.noise_scale
        g_big_sq = float((self.buffer / self.n_batches).pow(2).sum())
        self.buffer, self.count = None, 0
        bs, bb = self.b_small, self.b_big
        g2 = (bb * g_big_sq - bs * g_small_sq) / (bb - bs)           # unbiased |G|^2
        s = (g_small_sq - g_big_sq) / (1 / bs - 1 / bb)              # unbiased tr(Sigma)
        self.n_updates += 1
        self.ema_scale = self._ema(self.ema_scale, g2)
        self.ema_noise = self._ema(self.ema_noise, s)
        corr = 1 - self.beta ** self.n_updates
        scale, noise = self.ema_scale / corr, self.ema_noise / corr
        self.noise_scale = noise / scale if scale != 0 else None
        return self.noise_scale
