"""Activation lookup (reference: savanna/model/activations.py:21-136) — a pure function of the name;
it never writes to the configuration."""
from __future__ import annotations

import torch
import torch.nn.functional as F


def _geglu(x):
    a, b = x.chunk(2, dim=-1)
    return a * F.gelu(b)


_ACTS = {
    "gelu": F.gelu,
    "geglu": _geglu,
    "relu": F.relu,
    "softsign": F.softsign,
    "swish": F.silu,
    "silu": F.silu,
    "mish": F.mish,
    "sin": torch.sin,
    "identity": lambda x: x,
}


def get_activation(name: str):
    try:
        return _ACTS[name]
    except KeyError:
        raise ValueError(f"activation {name!r} not recognised") from None
