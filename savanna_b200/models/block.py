"""Transformer-style block with a sequence mixer and an MLP.

Evo 2 layout (`prenorm`, `pre_mlp_norm`, dropout 0; reference: savanna/model/block.py:1113-1212):
    a = x + dropout(mixer(norm_in(x)) + out_bias)
    y = a + mlp(norm_premlp(a))
All four norms the reference allocates are created (two are unused there as well) so checkpoints keep
the same key set.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .mixer import ParallelSequenceMixer
from .mlp import ParallelGLU, ParallelMLP
from .norms import get_norm


def _norm_and_residual(norm, x):
    fn = getattr(norm, "forward_with_residual", None)
    return fn(x) if fn is not None else (norm(x), x)


class ParallelBlock(nn.Module):
    def __init__(self, cfg, init_method, output_layer_init_method, layer_number: int, dtype=None, device=None):
        super().__init__()
        self.cfg, self.layer_number = cfg, layer_number
        self.operator_type = cfg.operator_config[layer_number]
        self.prenorm, self.postnorm = cfg.prenorm, cfg.postnorm
        self.pre_mlp_norm, self.outer_mlp_norm = cfg.pre_mlp_norm, cfg.outer_mlp_norm
        self.gpt_j_residual = cfg.gpt_j_residual
        self.hidden_dropout = cfg.hidden_dropout
        self.input_layernorm = get_norm(cfg, dtype, device)
        self.post_attention_layernorm = get_norm(cfg, dtype, device)
        self.pre_mlp_layernorm = get_norm(cfg, dtype, device)
        self.outer_mlp_layernorm = get_norm(cfg, dtype, device)
        self.mixer = ParallelSequenceMixer(cfg, init_method, output_layer_init_method, layer_number, dtype=dtype,
                                           device=device)
        if cfg.identity_mlp:
            self.mlp = nn.Identity()
        elif cfg.mlp_type == "regular" or (cfg.safe and self.operator_type == "hyena"):
            # `safe`: Hyena-LI layers take the plain two-layer MLP whatever `mlp_type` says (block.py:1074)
            self.mlp = ParallelMLP(cfg, init_method, output_layer_init_method, dtype=dtype, device=device)
        elif cfg.mlp_type == "short_hyena":
            self.mlp = ParallelSequenceMixer(cfg, init_method, output_layer_init_method, layer_number,
                                             operator_type="hyena_se", is_mlp=True, dtype=dtype, device=device)
        else:
            self.mlp = ParallelGLU(cfg, init_method, output_layer_init_method, layer_number, dtype=dtype, device=device)

    def _drop(self, x):
        if self.hidden_dropout > 0.0 and self.training:
            return F.dropout(x, self.hidden_dropout, True)
        return x

    def _mlp(self, x, positions, residual=None):
        if isinstance(self.mlp, nn.Identity):
            return (x if residual is None else residual + x), None
        if isinstance(self.mlp, ParallelSequenceMixer):
            return self.mlp(x, positions, residual)
        if isinstance(self.mlp, ParallelGLU):
            return self.mlp(x, residual)
        y, b = self.mlp(x)
        if residual is not None:
            y = residual + (y + b if b is not None else y)
            b = None
        return y, b

    def forward(self, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        if self.gpt_j_residual:
            # parallel residual: x + mixer(ln1(x)) + mlp(ln2(x))
            m, mb = self.mixer(self.input_layernorm(x), positions)
            f, fb = self._mlp(self.post_attention_layernorm(x), positions)
            out = m + f
            for b in (mb, fb):
                if b is not None:
                    out = out + b
            return x + self._drop(out)
        residual = x
        no_drop = not (self.hidden_dropout > 0.0 and self.training)
        if no_drop and not self.postnorm and not self.outer_mlp_norm:
            # residual and bias additions ride in the epilogues of the out-projection and w3 GEMMs; the norms hand the
            # residual branch through so that its gradient is added inside their backward kernels
            if self.prenorm:
                a, _ = self.mixer(x, positions, None, pre_norm=self.input_layernorm)
            else:
                a, _ = self.mixer(x, positions, x)
            if self.pre_mlp_norm and isinstance(self.mlp, (ParallelGLU, ParallelSequenceMixer)):
                y, _ = (self.mlp(a, None, pre_norm=self.pre_mlp_layernorm) if isinstance(self.mlp, ParallelGLU)
                        else self.mlp(a, positions, None, pre_norm=self.pre_mlp_layernorm))
                return y
            u, a_res = _norm_and_residual(self.pre_mlp_layernorm, a) if self.pre_mlp_norm else (a, a)
            y, _ = self._mlp(u, positions, a_res)
            return y
        # the general order of the reference (savanna/model/block.py:1105-1212): the post-norm acts on the MLP output,
        # the outer norm on the sum of the gated MLP's output and its residual, and the gated MLP's branch has no dropout
        u = self.input_layernorm(x) if self.prenorm else x
        m, mb = self.mixer(u, positions)
        if mb is not None:
            m = m + mb
        a = residual + self._drop(m)
        if isinstance(self.mlp, nn.Identity):
            return a
        u = self.pre_mlp_layernorm(a) if self.pre_mlp_norm else a
        f, fb = self._mlp(u, positions)
        if self.postnorm:
            f = self.post_attention_layernorm(f)
        if isinstance(self.mlp, ParallelGLU):
            out = a + f
            return self.outer_mlp_layernorm(out) if self.outer_mlp_norm else out
        if fb is not None:
            f = f + fb
        return a + self._drop(f)
