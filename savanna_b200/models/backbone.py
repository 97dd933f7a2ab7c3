"""Whole model: embedding -> N blocks -> final norm -> (tied) logits.

Module indices reproduce the reference's sequential layout so state-dict keys match its checkpoints
(savanna/model/backbone.py:312-434): `sequential.0` embedding, `.1` placeholder, layer i at
`.{i+2}`, placeholder, final norm at `.{N+3}`, and (untied only) the lm head at `.{N+4}`.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.utils.checkpoint as ckpt

from .. import ops
from ..parallel import mappings, state
from .block import ParallelBlock
from .embedding import Embedding
from .init_functions import get_init_methods
from .mlp import ParallelLinear
from .norms import get_norm


class _Placeholder(nn.Module):
    """Parameter-free slot (the reference puts layout lambdas here)."""

    def forward(self, x, *a):
        return x


class NormPipe(nn.Module):
    def __init__(self, cfg, dtype=None, device=None):
        super().__init__()
        self.norm = get_norm(cfg, dtype, device)

    def forward(self, x):
        return self.norm(x)


class Backbone(nn.Module):
    def __init__(self, cfg, device=None, dtype=None, layer_range: Optional[range] = None):
        super().__init__()
        self.cfg = cfg
        dtype = dtype or cfg.params_dtype
        init_m, out_init_m = get_init_methods(cfg)
        N = cfg.num_layers
        self.num_layers = N
        self.layer_range = layer_range if layer_range is not None else range(N)
        first = self.layer_range.start == 0
        last = self.layer_range.stop == N
        self.has_embedding, self.has_head = first or not cfg.no_weight_tying and last, last
        # Every component draws its initial weights from its own seeded stream (seed + component index), so a
        # layer is initialised identically whichever pipeline stage builds it and whatever else that stage holds.
        def seeded(idx):
            s = (cfg.seed or 0) + 7919 * (idx + 1)
            torch.manual_seed(s)
            if torch.cuda.is_available():
                torch.cuda.manual_seed(s)
        cpu_state = torch.get_rng_state()
        cuda_state = torch.cuda.get_rng_state() if torch.cuda.is_available() else None
        mods: List[nn.Module] = []
        seeded(0)
        mods.append(Embedding(cfg, init_m, dtype, device) if self.has_embedding else _Placeholder())
        mods.append(_Placeholder())
        for i in range(N):
            if i in self.layer_range:
                seeded(i + 1)
                mods.append(ParallelBlock(cfg, init_m, out_init_m, i, dtype, device))
            else:
                mods.append(_Placeholder())
        mods.append(_Placeholder())
        mods.append(NormPipe(cfg, dtype, device) if last else _Placeholder())
        if cfg.no_weight_tying and last:
            seeded(N + 1)
            mods.append(ParallelLinear(cfg, init_m, parallel_output=True, dtype=dtype, device=device))
        torch.set_rng_state(cpu_state)
        if cuda_state is not None:
            torch.cuda.set_rng_state(cuda_state)
        self.sequential = nn.ModuleList(mods)
        self.checkpoint_activations = cfg.checkpoint_activations
        self.checkpoint_num_layers = max(1, cfg.checkpoint_num_layers)
        self.sequence_parallel = cfg.sequence_parallel and state.get_model_parallel_world_size() > 1
        self.mup_output_mult = (1.0 / cfg.mup_width_scale * cfg.mup_output_temp) if cfg.use_mup else 1.0
        # Set by the trainer around the last micro-batch of a step: called as fn(i) from the backward pass once every
        # parameter of the blocks with local index >= i has its final gradient (ZeRO reduce-scatter overlap).
        self.grad_boundary_callback = None

    # -- pieces -------------------------------------------------------------------
    @property
    def embedding(self) -> Embedding:
        return self.sequential[0]

    def blocks(self):
        return [self.sequential[i + 2] for i in self.layer_range]

    @property
    def final_norm(self):
        return self.sequential[self.num_layers + 3]

    def _watch(self, x, first_final_block: int):
        """Report from the backward when the gradient of x (the input of block `first_final_block - 1`) is complete.
        Autograd runs the nodes of later blocks first (they were created later), so at that moment every node of the
        blocks >= `first_final_block` has run and their parameter gradients are final."""
        cb = self.grad_boundary_callback
        if cb is not None and x.requires_grad:
            x.register_hook(lambda g, i=first_final_block: cb(i))
        return x

    def _run_blocks(self, x, positions):
        blocks = self.blocks()
        if not (self.checkpoint_activations and self.training):
            for i, b in enumerate(blocks):
                x = b(self._watch(x, i + 1), positions)
            return x
        n = self.checkpoint_num_layers

        def chunk_fn(start, end):
            def fn(h, pos):
                for b in blocks[start:end]:
                    h = b(h, pos)
                return h
            return fn
        for s in range(0, len(blocks), n):
            e = min(s + n, len(blocks))
            store = self._checkpoint_storage()
            if store is None:
                x = ckpt.checkpoint(chunk_fn(s, e), self._watch(x, e), positions, use_reentrant=False)
            else:
                with store:
                    x = ckpt.checkpoint(chunk_fn(s, e), self._watch(x, e), positions, use_reentrant=True)
        return x

    def _checkpoint_storage(self):
        """Where the inputs of a checkpointed chunk live until its backward (the options of DeepSpeed's activation
        checkpointing, reference: savanna/initialize.py:63-90): `checkpoint_in_cpu` moves them to pinned host memory and
        back for the recomputation; `partition_activations` keeps 1 / tp of a tensor that is replicated over the
        tensor-parallel group (no sequence parallelism) and all-gathers it for the recomputation.  Both are saved-tensor
        hooks, so the chunk then runs through the re-entrant checkpoint, which hands its inputs to `save_for_backward`
        (the non-re-entrant one keeps them in a closure that no hook sees).  None when neither option is on."""
        cfg = self.cfg
        if cfg.checkpoint_in_cpu:
            return torch.autograd.graph.save_on_cpu(pin_memory=torch.cuda.is_available())
        tp = state.get_model_parallel_world_size()
        if cfg.partition_activations and tp > 1 and not self.sequence_parallel:
            return _partitioned_saved_tensors(tp, state.get_model_parallel_rank(), state.get_model_parallel_group())
        return None

    def logits(self, h: torch.Tensor) -> torch.Tensor:
        h = self.final_norm(h)
        if self.cfg.no_weight_tying:
            out, _ = self.sequential[self.num_layers + 4](h)
            return out
        w = self.embedding.word_embeddings.weight
        if self.sequence_parallel:
            h = mappings.gather_from_sequence_parallel_region(h, 1, True)
        elif state.get_model_parallel_world_size() > 1:
            h = mappings.copy_to_model_parallel_region(h)
        out = ops.linear(h, w)
        if self.mup_output_mult != 1.0:
            out = out * self.mup_output_mult
        return out

    def forward(self, tokens: torch.Tensor, positions: Optional[torch.Tensor] = None,
                hidden_in: Optional[torch.Tensor] = None, return_hidden: bool = False) -> torch.Tensor:
        """tokens [B, L_local] -> logits [B, L_local, V/tp] (vocab-parallel when tp > 1).
        Pipeline stages pass `hidden_in` instead of tokens and set `return_hidden`."""
        if positions is None:
            ref_t = tokens if tokens is not None else hidden_in
            positions = torch.arange(ref_t.shape[1], device=ref_t.device)
        x = self.embedding(tokens, positions) if hidden_in is None else hidden_in
        x = self._run_blocks(x, positions)
        if return_hidden or not self.has_head:
            return x
        return self.logits(x)


def build_model(cfg, device=None) -> Backbone:
    if cfg.padded_vocab_size is None:
        raise ValueError("padded_vocab_size is unset: build the tokenizer first (cfg.build_tokenizer())")
    model = Backbone(cfg, device=device)
    if cfg.use_mup and (device is None or torch.device(device).type != "meta"):
        # muP initialisation: tensors whose two dimensions grow with the width start 1 / sqrt(width multiplier) smaller
        # (what `mup.init.normal_` does in the reference's re-initialisation pass, savanna/training.py:1053-1056)
        ids, mult = _mup_matrix_like(model, cfg)
        if mult != 1.0:
            with torch.no_grad():
                for p in model.parameters():
                    if id(p) in ids:
                        p.mul_(mult ** -0.5)
    return model


def _partitioned_saved_tensors(tp: int, rank: int, group):
    """Saved-tensor hooks that store this rank's 1 / tp slice (along the sequence dimension) of every saved floating-point
    activation [B, L, D] whose length divides by tp, and rebuild the whole tensor with an all-gather when the backward
    asks for it.  Every tensor-parallel rank saves and restores the same tensors in the same order."""
    def pack(t):
        if t.dim() == 3 and t.is_floating_point() and t.shape[1] % tp == 0 and t.shape[1] >= tp and not isinstance(t, nn.Parameter):
            return ("part", t.chunk(tp, dim=1)[rank].contiguous(), t.shape)
        return ("whole", t, None)

    def unpack(packed):
        kind, t, shape = packed
        if kind == "whole":
            return t
        parts = [torch.empty_like(t) for _ in range(tp)]
        dist.all_gather(parts, t, group=group)
        return torch.cat(parts, dim=1).view(shape)
    return torch.autograd.graph.saved_tensors_hooks(pack, unpack)


def param_groups(model: nn.Module, cfg):
    """Weight-decay / no-weight-decay (+ optional per-group lr) parameter groups, decided module by module on each
    module's own parameters exactly as the reference decides them (savanna/model/utils.py:28-109):

      * norm layers: no decay (and everything when `weight_decay` is 0);
      * with `hyena_filter_wd` = 0, the own parameters of the free-form, complex modal and factored real modal filter
        modules and of the short Hyena operator: no decay; the explicit Hyena-MR filter `h`: no decay, in its own group
        when `lr_medium_hyena` differs from the learning rate;
      * every other module: parameters named `bias` are not decayed, all the others are.

    The last rule is what the reference applies to the modal Hyena-LI filter (`gamma`, `R`, `p`), to `conv_bias`, to
    the depthwise convolution weights and to the layers inside the free-form filter's MLP, whose classes its list does not
    name: they are decayed, and so they are here.  `wd_free_lr` gives the no-decay group its own learning rate."""
    from .filters import (ExplicitSingleDecayFilter, ImplicitRealModalFilter, ParallelComplexModalFilter,
                          ParallelImplicitFreeformFilter)
    from .hyena import ShortHyenaOperator
    from .norms import LayerNorm, RMSNorm, ScaleNorm
    decay, no_decay, medium = [], [], []
    seen = set()
    wd_off = cfg.weight_decay == 0.0
    filters_free = cfg.hyena_filter_wd == 0.0
    own_medium = cfg.lr_medium_hyena is not None and cfg.lr_medium_hyena != cfg.lr
    for module in model.modules():
        own = [(n, p) for n, p in module._parameters.items() if p is not None and p.requires_grad and id(p) not in seen]
        if not own:
            continue
        seen.update(id(p) for _, p in own)
        if isinstance(module, (LayerNorm, RMSNorm, ScaleNorm, nn.LayerNorm)) or wd_off:
            no_decay += [p for _, p in own]
        elif filters_free and isinstance(module, (ParallelImplicitFreeformFilter, ParallelComplexModalFilter,
                                                  ImplicitRealModalFilter, ShortHyenaOperator)):
            no_decay += [p for _, p in own]
        elif filters_free and isinstance(module, ExplicitSingleDecayFilter):
            (medium if own_medium else no_decay).extend(p for _, p in own)
        else:
            decay += [p for n, p in own if n != "bias"]
            no_decay += [p for n, p in own if n == "bias"]
    wd = cfg.weight_decay
    groups = [{"params": decay, "weight_decay": wd, "name": "decay"},
              {"params": no_decay, "weight_decay": 0.0, "name": "no_decay"}]
    if cfg.wd_free_lr is not None:
        groups[1]["lr"] = cfg.wd_free_lr
    if medium:
        groups.append({"params": medium, "weight_decay": 0.0, "lr": cfg.lr_medium_hyena, "name": "medium_hyena"})
    groups = [g for g in groups if g["params"]]
    if cfg.use_mup:
        groups = mup_param_groups(groups, model, cfg)
    return groups


def _mup_shapes_path(cfg):
    """`<base_shapes_file>.<rank>` (how the file is written) or the bare name, whichever exists; None without one."""
    import os
    base = cfg.base_shapes_file
    if not base:
        return None
    rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
    for cand in (f"{base}.{rank}", f"{base}.0", base):
        if os.path.exists(cand):
            return cand
    return None


def _mup_matrix_like(model: nn.Module, cfg):
    """(ids of the matrix-like parameters, width multiplier).  With a base-shapes file on disk both come from it: matrix-
    like = two dimensions that grow with the width, multiplier = how much wider this model is than the base
    (train/mup_shapes.py).  Without one: the projection and MLP weights by name, and `mup_width_scale`."""
    matrix_ids = set()
    mult = float(cfg.mup_width_scale)
    shapes_file = _mup_shapes_path(cfg)
    if shapes_file is not None:
        from ..train import mup_shapes
        widths = mup_shapes.width_multipliers(model, mup_shapes.load_base_shapes(shapes_file))
        mults = set()
        for name, p in model.named_parameters():
            n_inf, m = widths[name]
            if n_inf >= 2:
                matrix_ids.add(id(p))
                mults.add(round(m, 6))
        if len(mults) > 1:
            raise NotImplementedError(f"base shapes give different width multipliers for the matrix-like parameters ({sorted(mults)}); "
                                      "one multiplier per model is supported")
        if mults:
            mult = mults.pop()
    else:
        for name, p in model.named_parameters():
            if p.dim() == 2 and name.endswith(".weight") and any(k in name for k in (
                    "dense_projection.", "mixer.dense.", ".mlp.w1.", ".mlp.w2.", ".mlp.w3.", ".mlp.dense_", ".mlp.w12")):
                matrix_ids.add(id(p))
    return matrix_ids, mult


def mup_param_groups(groups, model: nn.Module, cfg):
    """Per-group learning rates of the maximal-update parametrisation (the reference's MuAdam / MuSGD,
    savanna/training.py:1065-1185 with the `mup` package): parameters whose two dimensions both grow with the model
    width ("matrix-like": the projection and MLP weights) are separated from the rest ("vector-like": embeddings,
    norms, biases, filters).  Adam-type optimizers divide the matrix-like learning rate by the width multiplier
    `mup_width_scale` (and multiply a coupled weight decay by it); SGD multiplies the vector-like learning rate by it.
    With a `base_shapes_file` on disk the classification and the multiplier come from that file instead of from
    parameter names and `mup_width_scale`.  A group that was split keeps its name with a `_matrix` suffix for the matrix-like half."""
    matrix_ids, mult = _mup_matrix_like(model, cfg)
    sgd = str(cfg.optimizer_type).lower() in ("sgd", "musgd")
    decoupled = bool(((cfg.optimizer or {}).get("params", {}) or {}).get("adam_w_mode", True))
    out = []
    for g in groups:
        base_lr = g.get("lr", cfg.lr)
        mat = [p for p in g["params"] if id(p) in matrix_ids]
        vec = [p for p in g["params"] if id(p) not in matrix_ids]
        if vec:
            gv = dict(g, params=vec)
            if sgd:
                gv["lr"] = base_lr * mult
                gv["weight_decay"] = g.get("weight_decay", 0.0) / mult
            out.append(gv)
        if mat:
            gm = dict(g, params=mat, name=g.get("name", "group") + "_matrix")
            if not sgd:
                gm["lr"] = base_lr / mult
                if not decoupled:
                    gm["weight_decay"] = g.get("weight_decay", 0.0) * mult
            out.append(gm)
    return out
