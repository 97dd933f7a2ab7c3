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
    """Gated MLP.  `w12` stacks the local rows of w1 and w2 ([2F/tp, D]) so both run as one GEMM; state
    dicts still carry `w1.weight` and `w2.weight` (hooks below), which keeps checkpoints and the
    tensor-parallel reshard tools unchanged."""

    def __init__(self, cfg, init_method, output_layer_init_method, layer_number: int = 0, dtype=None, device=None):
        super().__init__()
        from ..parallel.layers import _master_init, mark_tp
        self.act = gate_activation(cfg, layer_number)
        D, Fh = cfg.hidden_size, cfg.ffn_size
        tp = state.get_model_parallel_world_size()
        if cfg.pad_mlp_weights:
            m = 16 * tp
            Fh = m * ((Fh + m - 1) // m)
        if Fh % tp:
            raise ValueError(f"MLP inner size {Fh} not divisible by the tensor-parallel size {tp}")
        self.ffn_local = Fh // tp
        self.fp8 = bool(cfg.use_fp8_linears or cfg.use_fp8_mlp_projections)
        sp = cfg.sequence_parallel
        w1 = _master_init((Fh, D), init_method, 0, dtype, device)
        w2 = _master_init((Fh, D), init_method, 0, dtype, device)
        self.w12 = nn.Parameter(torch.cat([w1, w2], dim=0))
        mark_tp(self.w12, True, 0)
        self.w12.glu_packed = True
        self.w3 = RowParallelLinear(Fh, D, bias=False, input_is_parallel=True, init_method=output_layer_init_method,
                                    skip_bias_add=True, sequence_parallel=sp, dtype=dtype, device=device,
                                    fp8=self.fp8 and not cfg.disable_fp8_w3)
        self.sequence_parallel = sp and tp > 1
        self._register_state_dict_hook(self._split_hook)
        self._register_load_state_dict_pre_hook(self._merge_hook)

    @staticmethod
    def _split_hook(module, sd, prefix, local_metadata):
        w = sd.pop(prefix + "w12")
        sd[prefix + "w1.weight"], sd[prefix + "w2.weight"] = w[: module.ffn_local], w[module.ffn_local:]
        # keep the reference's key order: w1, w2, w3
        w3 = {k: sd.pop(k) for k in [k for k in sd if k.startswith(prefix + "w3.")]}
        sd.update(w3)
        return sd

    def _merge_hook(self, sd, prefix, local_metadata, strict, missing, unexpected, errors):
        k1, k2 = prefix + "w1.weight", prefix + "w2.weight"
        if k1 in sd and k2 in sd:
            sd[prefix + "w12"] = torch.cat([sd.pop(k1), sd.pop(k2)], dim=0)

    @property
    def w1_weight(self):
        return self.w12[: self.ffn_local]

    @property
    def w2_weight(self):
        return self.w12[self.ffn_local:]

    def forward(self, x, residual=None, pre_norm=None):
        """With `pre_norm` (the block's pre-MLP norm) x is the un-normalised stream: the norm is applied here so that
        it can be fused with the w1|w2 projection, and x itself becomes the residual."""
        tp = state.get_model_parallel_world_size()
        if pre_norm is not None:
            gain = getattr(pre_norm, "gain", None)
            if gain is not None and tp == 1:
                w3 = self.w3
                if w3.input_is_parallel and w3.fp8 == self.fp8:
                    return ops.mlp_gated(x, gain, pre_norm.eps, pre_norm.form, self.w12, w3.weight, w3.bias, self.act,
                                         fp8=self.fp8), None
                ab, residual = ops.norm_linear(x, gain, pre_norm.eps, pre_norm.form, self.w12, None, fp8=self.fp8)
                return self.w3.forward_glu(ab, self.act, residual)
            fn = getattr(pre_norm, "forward_with_residual", None)
            x, residual = fn(x) if fn is not None else (pre_norm(x), x)
        if self.sequence_parallel:
            ab = ops.linear_allgather(x, self.w12, None, 1, fp8=self.fp8)
        else:
            from ..parallel import mappings
            xin = mappings.copy_to_model_parallel_region(x) if tp > 1 else x
            ab = ops.linear(xin, self.w12, None, fp8=self.fp8)
        return self.w3.forward_glu(ab, self.act, residual)


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
