"""Module input/output dumps for offline comparison of parallel layouts (reference: savanna/debug.py:16-63):
forward hooks save every leaf module's inputs and outputs under `debug_dir`, tagged with the parallel layout,
so two runs (e.g. tensor-parallel 1 vs 2) can be diffed tensor by tensor."""
from __future__ import annotations

import os

import torch

from ..parallel import state


def layout_tag(cfg) -> str:
    return f"mp{state.get_model_parallel_world_size()}_cp{state.get_context_parallel_world_size()}_" \
           f"mpr{state.get_model_parallel_rank()}_cpr{state.get_context_parallel_rank()}"


def _detach(x):
    if isinstance(x, torch.Tensor):
        return x.detach().cpu()
    if isinstance(x, (tuple, list)):
        return [_detach(t) for t in x]
    return x


def register_debug_hooks(model: torch.nn.Module, cfg, max_calls: int = 1):
    root = os.path.join(cfg.debug_dir, layout_tag(cfg))
    os.makedirs(root, exist_ok=True)
    counts = {}
    handles = []

    def make(name):
        def hook(mod, inp, out):
            n = counts.get(name, 0)
            if n >= max_calls:
                return
            counts[name] = n + 1
            torch.save({"input": _detach(inp), "output": _detach(out)}, os.path.join(root, f"{name}.call{n}.pt"))
        return hook
    for name, mod in model.named_modules():
        if len(list(mod.children())) == 0:
            handles.append(mod.register_forward_hook(make(name or "root")))
    return handles
