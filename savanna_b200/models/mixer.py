"""Sequence mixer: projection -> (Hyena featuriser conv + Hyena operator | attention) -> out-projection.

Reference: savanna/model/block.py:82-1003.  Parameter names: `dense_projection`, `hyena_proj_conv`,
`mixer`, `rotary_emb`, `dense`.  The out-projection returns its bias un-added (the block fuses it
into bias-dropout-add).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn

from .. import ops
from ..parallel import halo as halo_mod, state
from ..parallel.layers import ColumnParallelLinear, RowParallelLinear
from .hyena import CausalDepthwiseConv1d, HyenaOperator, ShortHyenaOperator, _as_two_chunks
from .rope import RotaryEmbedding

HYENA_OPS = ("hyena", "hyena_mr", "hyena_se")
ATTENTION_OPS = ("flash_v2", "flash", "global", "ring", "flash_te", "local", "sparse_fixed", "sparse_variable", "bigbird",
                 "bslongformer")


class SelfAttention(nn.Module):
    """Causal multi-head attention on [B, L, heads/tp, 3*hd] projections with rotate-half RoPE.

    Context parallelism: `ring` / `flash_te` operators run the zigzag ring algorithm
    (parallel/ring_attention.py): KV shards travel around the context-parallel group and partial
    outputs are merged by log-sum-exp (reference: operators/attention/flash.py:523-597).
    """

    def __init__(self, cfg, operator_type: str, device=None):
        super().__init__()
        tp = state.get_model_parallel_world_size()
        self.heads = cfg.num_attention_heads // tp
        self.hd = cfg.hidden_size // cfg.num_attention_heads
        self.causal = cfg.causal
        self.operator_type = operator_type
        # context-parallel exchange of `flash_te` layers: "p2p" = ring of K/V shards, "a2a" = head exchange, "all_gather"
        self.cp_comm_type = cfg.flash_te_comm_type or "p2p"
        # legacy block-sparse operators: a layout mask over materialised scores (models/sparse_layouts.py)
        from .sparse_layouts import SPARSE_OPERATORS
        self.sparse = operator_type in SPARSE_OPERATORS
        self.sparsity_config = dict(cfg.sparsity_config or {})
        self._sparse_masks = {}
        if self.sparse and not cfg.causal:
            raise NotImplementedError("block-sparse attention operators are built for causal models (unidirectional layouts)")
        # dropout on the attention probabilities (0 in every Evo 2 configuration): the own kernels have none, so a
        # training step with a non-zero rate runs PyTorch's fused attention, which has
        self.attn_dropout = float(cfg.attention_dropout or 0.0)
        self._rotary = []          # the module itself is registered by the owning mixer as `rotary_emb`
        if cfg.pos_emb in ("rotary", "rotary_linear_scaled", "rotary_ntk_scaled", "rotary2"):
            rd = int(self.hd * cfg.rotary_pct)
            self._rotary.append(RotaryEmbedding(rd, cfg.rotary_emb_base, cfg.rotary_emb_scaling_factor,
                                                "rotary" if cfg.pos_emb == "rotary2" else cfg.pos_emb,
                                                cfg.rotary_emb_max_unscaled_seq_len, device=device))
        # score biases (ALiBi slopes, bucketed relative positions): only the legacy `global` operator takes them; its
        # scores are materialised (the flash kernels have no bias input), as in the reference's non-flash attention
        self.score_bias = None
        if cfg.pos_emb in ("alibi", "rpe"):
            if operator_type != "global":
                raise NotImplementedError(f"pos_emb={cfg.pos_emb!r} needs the `global` attention operator "
                                          f"(got {operator_type!r}): the flash kernels take no score bias")
            from .rope import AliBi, RelativePositionBias
            rank = state.get_model_parallel_rank()
            if cfg.pos_emb == "alibi":
                self.score_bias = AliBi(cfg.num_attention_heads, tp, rank).to(device)
            else:
                self.score_bias = RelativePositionBias(math.sqrt(self.hd), self.causal,
                                                       cfg.rpe_num_buckets, cfg.rpe_max_distance, cfg.num_attention_heads,
                                                       tp, rank, dtype=torch.float32, device=device)

    def _sparse_mask(self, L: int, device) -> torch.Tensor:
        m = self._sparse_masks.get(L)
        if m is None or m.device != device:
            from .sparse_layouts import additive_mask
            tp, r = state.get_model_parallel_world_size(), state.get_model_parallel_rank()
            m = additive_mask(self.operator_type, self.heads * tp, L, self.sparsity_config)      # layouts of all heads ...
            m = m[r * self.heads:(r + 1) * self.heads].to(device)                                 # ... this rank's slice
            self._sparse_masks = {L: m}                 # one length at a time: the mask is [heads, L, L]
        return m

    def forward(self, qkv: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        B, L, _ = qkv.shape
        qkv = qkv.view(B, L, self.heads, 3 * self.hd)
        cp = state.get_context_parallel_world_size()
        if self.sparse:
            if cp > 1:
                raise NotImplementedError("block-sparse attention operators do not run under context parallelism")
            from ..ops import reference as ref
            q, k, v = qkv[..., : self.hd], qkv[..., self.hd: 2 * self.hd], qkv[..., 2 * self.hd:]
            if self._rotary:
                cos, sin = self._rotary[0](positions)
                q, k = ops.apply_rope(q, cos, sin), ops.apply_rope(k, cos, sin)
            o = ref.attention(q, k, v, True, positions, positions, bias=self._sparse_mask(L, qkv.device))
            return o.reshape(B, L, self.heads * self.hd)
        if self.score_bias is not None:
            if cp > 1:
                raise NotImplementedError("score-bias attention (alibi / rpe) does not run under context parallelism")
            from ..ops import reference as ref
            q, k, v = qkv[..., : self.hd], qkv[..., self.hd: 2 * self.hd], qkv[..., 2 * self.hd:]
            o = ref.attention(q, k, v, self.causal, positions, positions, bias=self.score_bias.bias(positions, positions))
            return o.reshape(B, L, self.heads * self.hd)
        cos = sin = None
        if self._rotary:
            cos, sin = self._rotary[0](positions)
        if self.attn_dropout > 0.0 and self.training:
            if cp > 1:
                raise NotImplementedError("attention_dropout does not run under context parallelism")
            import torch.nn.functional as F
            q, k, v = qkv[..., : self.hd], qkv[..., self.hd: 2 * self.hd], qkv[..., 2 * self.hd:]
            if self._rotary:
                q, k = ops.apply_rope(q, cos, sin), ops.apply_rope(k, cos, sin)
            o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                               dropout_p=self.attn_dropout, is_causal=self.causal)
            return o.transpose(1, 2).reshape(B, L, self.heads * self.hd)
        if cp == 1 or self.operator_type not in ("ring", "flash_te"):
            o = ops.attention_packed(qkv, cos, sin, self.causal)      # one function: no slice / concatenate in autograd
            if o is not None:
                return o.reshape(B, L, self.heads * self.hd)
        q, k, v = qkv[..., : self.hd], qkv[..., self.hd: 2 * self.hd], qkv[..., 2 * self.hd:]
        if self._rotary:
            q, k = ops.apply_rope(q, cos, sin), ops.apply_rope(k, cos, sin)
        comm = self.cp_comm_type if self.operator_type == "flash_te" else "p2p"
        if cp > 1 and self.operator_type in ("ring", "flash_te") and comm == "a2a":
            from ..parallel.cp_attention import ulysses_attention
            o = ulysses_attention(q, k, v, causal=self.causal)
        elif cp > 1 and self.operator_type in ("ring", "flash_te") and comm == "all_gather":
            from ..parallel.cp_attention import allgather_attention
            o = allgather_attention(q, k, v, causal=self.causal)
        elif cp > 1 and self.operator_type in ("ring", "flash_te"):
            from ..parallel.ring_attention import ring_attention
            o = ring_attention(q, k, v, positions, causal=self.causal)
        else:
            o = ops.attention(q, k, v, causal=self.causal)
        return o.reshape(B, L, self.heads * self.hd)


class ParallelSequenceMixer(nn.Module):
    def __init__(self, cfg, init_method, output_layer_init_method, layer_number: int,
                 operator_type: Optional[str] = None, is_mlp: bool = False, dtype=None, device=None):
        super().__init__()
        self.cfg, self.layer_number, self.is_mlp = cfg, layer_number, is_mlp
        self.operator_type = operator_type or cfg.operator_config[layer_number]
        D = cfg.hidden_size
        tp = state.get_model_parallel_world_size()
        sp = cfg.sequence_parallel
        # Hyena layers may run wider than the residual stream (`hyena_width_expansion`, or `hyena_mlp_expansion_factor`
        # for the short-Hyena MLP): projections go D -> 3 H and H -> D, H rounded up to a multiple of 32 when expanded
        # (reference: savanna/model/block.py:178-201)
        H = D
        if self.operator_type in HYENA_OPS:
            e = float(cfg.hyena_mlp_expansion_factor if is_mlp else cfg.hyena_width_expansion)
            H = int(D * e)
            if e > 1:
                H = 32 * ((H + 31) // 32)
        self.inner_size = H
        if is_mlp:
            fp8_in = cfg.use_fp8_linears and cfg.use_fp8_hyena_mlp_input_projections
            fp8_out = cfg.use_fp8_linears and cfg.use_fp8_hyena_mlp_output_projections
        else:
            fp8_in = cfg.use_fp8_linears and cfg.use_fp8_input_projections
            fp8_out = cfg.use_fp8_linears and cfg.use_fp8_output_projections
        # width of the in-projection: 3 D, or D when one projection serves as all three streams
        # (`tie_projection_weights`), or D + 2 D / proj_groups for attention layers whose second and third stream are
        # produced for one group of channels and repeated over the `proj_groups` groups
        # (reference: savanna/model/block.py:213-236, 773-800)
        self.tie_projections = bool(cfg.tie_projection_weights)
        self.proj_groups = int(cfg.proj_groups or 1) if self.operator_type in ATTENTION_OPS else 1
        if self.tie_projections:
            proj_out = H
        elif self.proj_groups > 1:
            if (2 * D) % (self.proj_groups * tp):
                raise ValueError(f"proj_groups={self.proj_groups}: 2 * hidden_size must divide by proj_groups * tensor-parallel size")
            proj_out = D + 2 * D // self.proj_groups
        else:
            proj_out = 3 * H
        self.dense_projection = ColumnParallelLinear(D, proj_out, bias=False, gather_output=False, init_method=init_method,
                                                     skip_bias_add=True, sequence_parallel=sp, dtype=dtype, device=device,
                                                     fp8=fp8_in)
        if self.operator_type in HYENA_OPS:
            width = 3 * H // tp
            self.short_conv_L = cfg.short_conv_L
            self.hyena_proj_conv = CausalDepthwiseConv1d(width, cfg, cfg.short_conv_L, num_groups=width,
                                                         fast=cfg.fast_conv_proj, dtype=dtype, device=device)
            if self.operator_type == "hyena_se":
                self.mixer = ShortHyenaOperator(H, cfg, is_mlp=is_mlp, dtype=dtype, device=device)
            else:
                self.mixer = HyenaOperator(H, cfg, layer_number, self.operator_type, dtype=dtype, device=device)
            if not cfg.interleave_projections:
                raise NotImplementedError("non-interleaved projections: convert the checkpoint with "
                                          "tools/interleave_model_states.py and set interleave_projections")
        elif self.operator_type in ATTENTION_OPS:
            self.mixer = SelfAttention(cfg, self.operator_type, device=device)
            if self.mixer._rotary:
                self.rotary_emb = self.mixer._rotary[0]
        else:
            raise NotImplementedError(f"operator {self.operator_type!r} has no implementation in this framework")
        self.dense = RowParallelLinear(H, D, bias=True, input_is_parallel=True, init_method=output_layer_init_method,
                                       skip_bias_add=True, sequence_parallel=sp, dtype=dtype, device=device, fp8=fp8_out)

    def forward(self, x: torch.Tensor, positions: torch.Tensor, residual: Optional[torch.Tensor] = None, pre_norm=None):
        """Returns (output, out-projection bias to be added by the caller).  With `residual` the
        out-projection adds bias and residual itself and the bias slot is None.  With `pre_norm` (the block's input
        norm) x is the un-normalised stream: the norm is fused with the in-projection and x becomes the residual."""
        if pre_norm is not None:
            proj, _, residual = self.dense_projection.forward_normed(x, pre_norm)
        else:
            proj, _ = self.dense_projection(x)
        if self.tie_projections:
            proj = proj.repeat_interleave(3, dim=-1)              # every channel three times: its three streams are equal
        elif self.proj_groups > 1:
            own = proj.shape[-1] * self.proj_groups // (self.proj_groups + 2)          # this rank's D / tp first-stream columns
            proj = torch.cat([proj[..., :own], proj[..., own:].repeat(1, 1, self.proj_groups)], dim=-1)
        if self.operator_type in HYENA_OPS:
            cp = state.get_context_parallel_world_size() if self.cfg.use_cp_hyena else 1
            if cp > 1:
                feat = self.hyena_proj_conv.forward_cp(proj)
            else:
                feat = self.hyena_proj_conv(proj)
            z = self.mixer(feat)
        else:
            z = self.mixer(proj, positions)
        return self.dense(z, residual)
