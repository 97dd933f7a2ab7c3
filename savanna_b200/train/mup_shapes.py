"""Base shapes for the maximal-update parametrisation (muP).

muP's learning-rate and initialisation rules depend on how much wider a tensor is than in a small base model, per
dimension.  The reference obtains that from the `mup` package (savanna/training.py:217-266, 1040-1056): with
`save_base_shapes` it builds the model at `hidden_size` and at `hidden_size * mup_width_scale`, records which
dimensions differ ("infinite" dimensions) and writes `<base_shapes_file>.<rank>`, then exits; later runs read the file
and derive every parameter's width multiplier from it.  This module restates that with plain JSON and models built on
the meta device (no memory, no initialisation):

    {"<parameter name>": {"shape": [..base shape..], "infinite": [true / false per dimension]}, ...}

`width_multipliers` gives, for a model of any width, parameter name -> (number of infinite dimensions, fan-in
multiplier).  Two infinite dimensions make a parameter matrix-like (Adam learning rate divided by the multiplier), fewer
make it vector-like.  `models/backbone.py:mup_param_groups` uses these when the run names a base-shapes file, and the
single `mup_width_scale` otherwise.
"""
from __future__ import annotations

import copy
import json
from typing import Dict, Tuple

import torch


def _shapes_at_width(cfg, hidden_size: int) -> Dict[str, Tuple[int, ...]]:
    from ..models.backbone import build_model
    c = copy.copy(cfg)
    c.hidden_size = int(hidden_size)
    model = build_model(c, device=torch.device("meta"))
    return {n: tuple(p.shape) for n, p in model.named_parameters()}


def make_base_shapes(cfg) -> Dict[str, Dict]:
    """Shapes at `hidden_size` (base) against `hidden_size * mup_width_scale` (delta)."""
    scale = cfg.mup_width_scale
    if not scale or float(scale) == 1.0:
        raise ValueError("save_base_shapes: mup_width_scale must differ from 1 (the delta model has to be wider than the base)")
    base = _shapes_at_width(cfg, cfg.hidden_size)
    delta = _shapes_at_width(cfg, int(cfg.hidden_size * scale))
    out = {}
    for name, shape in base.items():
        other = delta.get(name)
        if other is None or len(other) != len(shape):
            raise ValueError(f"parameter {name} exists at one width only: the two models differ in structure")
        out[name] = {"shape": list(shape), "infinite": [a != b for a, b in zip(shape, other)]}
    return out


def save_base_shapes(cfg, path: str) -> Dict[str, Dict]:
    shapes = make_base_shapes(cfg)
    with open(path, "w") as fh:
        json.dump(shapes, fh, indent=1)
    return shapes


def load_base_shapes(path: str) -> Dict[str, Dict]:
    with open(path) as fh:
        return json.load(fh)


def width_multipliers(model: torch.nn.Module, base_shapes: Dict[str, Dict]) -> Dict[str, Tuple[int, float]]:
    """name -> (infinite dimensions, fan-in multiplier).  The fan-in multiplier is the ratio of the last infinite
    dimension to the base ([out, in] weights: the input width); parameters missing from the file count as finite."""
    out = {}
    for name, p in model.named_parameters():
        rec = base_shapes.get(name)
        if rec is None or len(rec["shape"]) != p.dim():
            out[name] = (0, 1.0)
            continue
        inf = [i for i, flag in enumerate(rec["infinite"]) if flag]
        mult = float(p.shape[inf[-1]]) / float(rec["shape"][inf[-1]]) if inf else 1.0
        out[name] = (len(inf), mult)
    return out
