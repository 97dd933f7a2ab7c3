"""MLPs: gated (`ParallelGLU`, the SwiGLU slot), plain (`ParallelMLP`) and the lm-head linear.

Gated MLP: w3( act(w1 x) * w2 x ), no biases, inner size from `cfg.ffn_size`
(reference: savanna/model/operators/local/base.py:83-220).  w1 and w2 are separate parameters (for
checkpoint parity) but run as ONE column GEMM over the concatenated weight followed by a fused
gate kernel.  The gate activation is an explicit per-layer decision (`gate_activation`) instead of
the reference's mutated global: "evo2_compat" reproduces what released Evo 2 checkpoints were
trained with (gelu in layer 0, identity afterwards).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops
from ..parallel import state
from ..parallel.layers import ColumnParallelLinear, RowParallelLinear


def gate_activation(cfg, layer_number: int) -> str:
    mode = cfg.mlp_activation
    if mode is None:
        mode = cfg.parallel_glu_activation_default or "evo2_compat"
    if mode == "evo2_compat":
        ops_before = cfg.operator_config[: layer_number + 1]
        hyena_seen = any(o in ("hyena", "hyena_mr") for o in ops_before)
        return "identity" if hyena_seen else cfg.activation
    return mode


class ParallelGLU(nn.Module):
    def __init__(self, cfg, init_method, output_layer_init_method, layer_number: int = 0, dtype=None, device=None):
        super().__init__()
        self.act = gate_activation(cfg, layer_number)
        D, Fh = cfg.hidden_size, cfg.ffn_size
        tp = state.get_model_parallel_world_size()
        if cfg.pad_mlp_weights:
            m = 16 * tp
            Fh = m * ((Fh + m - 1) // m)
        fp8 = cfg.use_fp8_linears or cfg.use_fp8_mlp_projections
        sp = cfg.sequence_parallel
        kw = dict(bias=False, gather_output=False, init_method=init_method, skip_bias_add=True,
                  sequence_parallel=sp, dtype=dtype, device=device, fp8=fp8)
        self.w1 = ColumnParallelLinear(D, Fh, **kw)
        self.w2 = ColumnParallelLinear(D, Fh, **kw)
        self.w3 = RowParallelLinear(Fh, D, bias=False, input_is_parallel=True, init_method=output_layer_init_method,
                                    skip_bias_add=True, sequence_parallel=sp, dtype=dtype, device=device,
                                    fp8=fp8 and not cfg.disable_fp8_w3)
        self.sequence_parallel = sp and tp > 1
        self._w12 = None

    def _packed_weight(self):
        # [2F/tp, D]: w1 rows then w2 rows.  Built by autograd-visible concatenation so both parameters get grads.
        return torch.cat([self.w1.weight, self.w2.weight], dim=0)

    def forward(self, x):
        w12 = self._packed_weight()
        if self.sequence_parallel:
            ab = ops.linear_allgather(x, w12, None, 1, fp8=self.w1.fp8)
        else:
            from ..parallel import mappings
            xin = mappings.copy_to_model_parallel_region(x) if state.get_model_parallel_world_size() > 1 else x
            ab = ops.linear(xin, w12, None, fp8=self.w1.fp8)
        h = ops.glu_act_packed(ab, self.act)
        return self.w3(h)


class ParallelMLP(nn.Module):
    """h -> 4h -> h with the configured activation (base.py:18-80)."""

    def __init__(self, cfg, init_method, output_layer_init_method, dtype=None, device=None):
        super().__init__()
        D = cfg.hidden_size
        ff = 4 * D
        self.act = cfg.activation
        self.dense_h_to_4h = ColumnParallelLinear(D, ff, bias=True, init_method=init_method, skip_bias_add=False,
                                                  sequence_parallel=cfg.sequence_parallel, dtype=dtype, device=device)
        self.dense_4h_to_h = RowParallelLinear(ff, D, bias=True, init_method=output_layer_init_method, skip_bias_add=True,
                                               sequence_parallel=cfg.sequence_parallel, dtype=dtype, device=device)

    def forward(self, x):
        from ..models.activations import get_activation
        h, _ = self.dense_h_to_4h(x)
        h = get_activation(self.act)(h)
        return self.dense_4h_to_h(h)


class ParallelLinear(nn.Module):
    """Untied lm head (base.py:223-268)."""

    def __init__(self, cfg, init_method, parallel_output=True, dtype=None, device=None):
        super().__init__()
        if cfg.output_layer_parallelism == "column":
            self.final_linear = ColumnParallelLinear(cfg.hidden_size, cfg.padded_vocab_size, bias=False,
                                                     init_method=init_method, gather_output=not parallel_output,
                                                     skip_bias_add=False, sequence_parallel=cfg.sequence_parallel,
                                                     dtype=dtype, device=device)
        else:
            self.final_linear = RowParallelLinear(cfg.hidden_size, cfg.padded_vocab_size, bias=False,
                                                  input_is_parallel=False, init_method=init_method,
                                                  parallel_output=False, skip_bias_add=False, dtype=dtype, device=device)

    def forward(self, x):
        return self.final_linear(x)
