"""Hyena operators and the depthwise causal convolution module.

Parameter names and shapes follow the reference so its checkpoints load
(savanna/model/operators/hyena/hyena.py:76-181, 191-565, 568-852):
  CausalDepthwiseConv1d.short_conv_weight   [groups, 1, k]  (or [groups, k] with the "fast" flag)
  HyenaOperator.conv_bias [D/tp], .filter.{h,decay} (MR) / .filter.{gamma,R,p,t} (LI)
  ShortHyenaOperator.short_conv.short_conv_weight [G/tp, 1, k]
All operators take the featurised projections `feat [B, L, 3*D/tp]` (interleaved x1,x2,v) and return
`[B, L, D/tp]`; nothing is permuted to channel-first.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn

from .. import ops
from ..parallel import a2a, halo as halo_mod, halo_fused, li_fused, state
from .filters import ExplicitSingleDecayFilter, ImplicitModalFilter, build_filter


def groups_per_rank(hidden: int, num_groups: Optional[int], tp: int, expansion: float = 1.0):
    """(width, filter groups, channels per group) on one tensor-parallel rank.  `hidden` is the operator's width, already
    expanded by the mixer; the group count is scaled by `expansion` here, as the reference does
    (operators/hyena/hyena.py:184-188: groups per rank = int(groups / tp * hyena_width_expansion))."""
    if num_groups is None:
        num_groups = hidden
    if hidden % tp or num_groups % tp:
        raise ValueError("hyena width and group count must be divisible by the tensor-parallel size")
    w, g = hidden // tp, int(num_groups // tp * expansion)
    if g <= 0 or w % g:
        raise ValueError(f"hyena width per rank {w} must be divisible by the groups per rank {g}")
    return w, g, w // g


def _as_two_chunks(x):
    """[B, L, C] zigzag shard -> [(B 2), L/2, C] view (each chunk becomes a batch row)."""
    B, L, C = x.shape
    return x.reshape(B * 2, L // 2, C)


class CausalDepthwiseConv1d(nn.Module):
    def __init__(self, channels: int, cfg, kernel_size: int, num_groups: Optional[int] = None, fast: bool = False,
                 dtype=None, device=None):
        super().__init__()
        self.channels, self.kernel_size = channels, kernel_size
        self.num_groups = num_groups or channels
        self.group_dim = channels // self.num_groups
        shape = (self.num_groups, kernel_size) if fast else (self.num_groups, 1, kernel_size)
        bound = math.sqrt(1.0 / cfg.short_conv_L)
        tp, rank = state.get_model_parallel_world_size(), state.get_model_parallel_rank()
        full = torch.empty((self.num_groups * tp,) + shape[1:], dtype=torch.float32, device=device).uniform_(-bound, bound)
        self.short_conv_weight = nn.Parameter(full.chunk(tp, 0)[rank].to(dtype).contiguous())
        self.short_conv_weight.model_parallel = True
        self.short_conv_weight.partition_dim = 0
        self.short_conv_weight.is_filter_param = True

    def taps(self) -> torch.Tensor:
        """[groups, k] view of the weight."""
        return self.short_conv_weight.reshape(self.num_groups, self.kernel_size)

    def forward(self, x: torch.Tensor, halo: Optional[torch.Tensor] = None) -> torch.Tensor:
        w = self.taps()
        if self.group_dim > 1:
            w = w.repeat_interleave(self.group_dim, dim=0)
        return ops.causal_conv1d(x, w, halo)

    def forward_cp(self, x: torch.Tensor) -> torch.Tensor:
        """x [B, L_local, C] holding two zigzag chunks of a context-parallel shard.  The kernel reads the rows before
        each chunk from the neighbour ranks' memory itself when the peer workspace is up; otherwise the halo rows are
        exchanged first (NCCL or a pull kernel) and passed as a tensor."""
        w = self.taps()
        if self.group_dim > 1:
            w = w.repeat_interleave(self.group_dim, dim=0)
        y = halo_fused.causal_conv1d_cp(x, w)
        if y is not None:
            return y
        B, L, C = x.shape
        k = self.kernel_size
        h = halo_mod.zigzag_halo(x, k - 1)
        return ops.causal_conv1d(_as_two_chunks(x), w, h.reshape(B * 2, k - 1, C)).reshape(B, L, C)


class ShortHyenaOperator(nn.Module):
    """Hyena-SE: z = x1 * conv_k(x2 * v); also the `short_hyena` MLP replacement."""

    def __init__(self, hidden_size: int, cfg, is_mlp: bool = False, dtype=None, device=None):
        super().__init__()
        tp = state.get_model_parallel_world_size()
        if is_mlp:
            k = cfg.hyena_mlp_len if cfg.hyena_mlp_len is not None else cfg.hyena_se_len
            self.pregate, self.postgate = cfg.hyena_mlp_pregate, cfg.hyena_mlp_postgate
            g = cfg.num_groups_hyena_mlp if cfg.num_groups_hyena_mlp is not None else cfg.num_groups_hyena
            g = int((g or cfg.hidden_size) * cfg.hyena_mlp_expansion_factor)
            fast = cfg.fast_hyena_mlp_conv
        else:
            k = cfg.hyena_se_len
            self.pregate, self.postgate = cfg.hyena_se_pregate, cfg.hyena_se_postgate
            g = cfg.num_groups_hyena_short if cfg.num_groups_hyena_short is not None else cfg.num_groups_hyena
            g = int((g or cfg.hidden_size) * cfg.hyena_width_expansion)
            fast = cfg.fast_conv_mixer
        self.kernel_size = k
        self.width, self.num_groups, self.group_dim = groups_per_rank(hidden_size, g, tp, cfg.hyena_width_expansion)
        self.short_conv = CausalDepthwiseConv1d(self.width, cfg, k, num_groups=self.num_groups, fast=fast, dtype=dtype,
                                                device=device)
        self.use_cp = cfg.use_cp_hyena

    def forward(self, feat: torch.Tensor) -> torch.Tensor:
        w = self.short_conv.taps()
        if self.use_cp and state.get_context_parallel_world_size() > 1:
            z = halo_fused.hyena_se_inner_cp(feat, w, self.pregate, self.postgate)
            if z is not None:
                return z
            h = halo_mod.zigzag_halo(feat, self.kernel_size - 1)
            B, L, C = feat.shape
            z = ops.hyena_se_inner(_as_two_chunks(feat), w, h.reshape(B * 2, self.kernel_size - 1, C), self.pregate,
                                   self.postgate)
            return z.reshape(B, L, -1)
        return ops.hyena_se_inner(feat, w, None, self.pregate, self.postgate)


class HyenaOperator(nn.Module):
    """Hyena-MR (`hyena_mr`, explicit decaying filter of `hyena_mr_len` taps) and Hyena-LI (`hyena`,
    implicit filter as long as the sequence):  z = x1 * ( h * (x2 v) + conv_bias * (x2 v) )."""

    def __init__(self, hidden_size: int, cfg, layer_number: int, operator_type: str, dtype=None, device=None):
        super().__init__()
        self.cfg, self.operator_type = cfg, operator_type
        self.is_mr = operator_type == "hyena_mr"
        tp = state.get_model_parallel_world_size()
        g = cfg.num_groups_hyena
        if self.is_mr and cfg.num_groups_hyena_medium is not None:
            g = cfg.num_groups_hyena_medium
        self.width, self.num_groups, self.group_dim = groups_per_rank(hidden_size, g, tp, cfg.hyena_width_expansion)
        self.hyena_mr_len = cfg.hyena_mr_len
        self.use_cp = cfg.use_cp_hyena
        # the two PyTorch-level variants of the long operator: a two-sided filter, and outer-product heads with one
        # filter and one bias per group.  They apply to the `hyena` (long) layers; hyena_mr layers of the same model keep
        # their causal finite filter
        self.bidirectional = bool(cfg.bidirectional) and not self.is_mr
        self.slow_heads = bool(cfg.use_slow_heads) and not self.is_mr
        if self.bidirectional and self.slow_heads:
            raise ValueError("bidirectional and use_slow_heads exclude each other")
        self.filter = build_filter(cfg, operator_type, self.num_groups, device=device)
        bias_len = self.num_groups if self.slow_heads else self.width
        self.conv_bias = nn.Parameter(torch.full((bias_len,), float(cfg.conv_bias_init), dtype=torch.float32, device=device))
        self.conv_bias.model_parallel = True
        self.conv_bias.partition_dim = 0
        self.conv_bias.is_filter_param = True

    # -- Hyena-MR ---------------------------------------------------------------
    def _forward_mr(self, feat, cp):
        B, L, C = feat.shape
        k = min(self.hyena_mr_len, L * cp)
        h = self.filter(k)
        if cp > 1 and self.cfg.cp_hyena_mr_algo == "p2p":
            z = halo_fused.hyena_mr_inner_cp(feat, h, self.conv_bias)
            if z is not None:
                return z
            hal = halo_mod.zigzag_halo(feat, k - 1)
            z = ops.hyena_mr_inner(_as_two_chunks(feat), h, self.conv_bias, hal.reshape(B * 2, k - 1, C))
            return z.reshape(B, L, -1)
        if cp > 1:
            r = state.get_context_parallel_rank()
            full = a2a.split_to_full(feat)                           # [B, L*cp, 3*width/cp]
            wl = self.width // cp
            gl = max(1, self.num_groups // cp)
            if self.num_groups % cp:
                hc = h.repeat_interleave(self.group_dim, 0)[r * wl:(r + 1) * wl]
            else:
                hc = h[r * gl:(r + 1) * gl]
            z = ops.hyena_mr_inner(full, hc, self.conv_bias[r * wl:(r + 1) * wl])
            return a2a.full_to_split(z)
        return ops.hyena_mr_inner(feat, h, self.conv_bias)

    # -- Hyena-LI ---------------------------------------------------------------
    def _modal(self):
        f = self.filter
        if not isinstance(f, ImplicitModalFilter):
            return None
        g, R, p = f.gamma, f.R, f.p
        if self.group_dim > 1:
            g, R, p = (t.repeat_interleave(self.group_dim, 0) for t in (g, R, p))
        return g, R, p

    def _forward_li(self, feat, cp):
        B, L, C = feat.shape
        if self.bidirectional or self.slow_heads:
            if cp > 1:
                raise NotImplementedError("bidirectional / use_slow_heads do not run under context parallelism")
            h = self.filter(L)
            fn = ops.hyena_long_fft_bidirectional if self.bidirectional else ops.hyena_multihead
            return fn(feat, h, self.conv_bias)
        modal = self._modal()
        if cp == 1:
            if modal is not None:
                return ops.hyena_li_modal(feat, *modal, self.conv_bias)
            return ops.hyena_long_fft(feat, self.filter(L), self.conv_bias)
        r = state.get_context_parallel_rank()
        if modal is not None and self.cfg.cp_hyena_li_algo == "state":
            from ..parallel.modal_cp import hyena_li_modal_state_cp
            return hyena_li_modal_state_cp(feat, *modal, self.conv_bias)
        wl = self.width // cp
        sl = slice(r * wl, (r + 1) * wl)
        if modal is not None:
            # scan kernels that read / write the other ranks' staging buffers themselves (the all-to-all inside the scan)
            z = li_fused.hyena_li_modal_cp(feat, modal[0][sl], modal[1][sl], modal[2][sl], self.conv_bias[sl])
            if z is not None:
                return z
        full = a2a.split_to_full(feat)
        if modal is not None:
            z = ops.hyena_li_modal(full, modal[0][sl], modal[1][sl], modal[2][sl], self.conv_bias[sl])
        else:
            h = self.filter(L * cp)
            if h.shape[0] != self.width:
                h = h.repeat_interleave(self.group_dim, 0)
            z = ops.hyena_long_fft(full, h[sl], self.conv_bias[sl])
        return a2a.full_to_split(z)

    def forward(self, feat: torch.Tensor) -> torch.Tensor:
        cp = state.get_context_parallel_world_size() if self.use_cp else 1
        return self._forward_mr(feat, cp) if self.is_mr else self._forward_li(feat, cp)
