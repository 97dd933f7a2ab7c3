"""Weight initialisers (reference: savanna/model/init_functions.py:10-189).

`get_init_methods(cfg)` returns (input-side init, output-side init) as the reference does:
Evo 2 uses `small_init` (sigma = sqrt(2/(5 D))) for in-projections / MLP-in / embedding and
`wang_init` (sigma = 2/(N_layers sqrt(D))) for out-projections and `w3`.
"""
from __future__ import annotations

import math

import torch


def _normal(std):
    def f(t):
        return torch.nn.init.normal_(t, mean=0.0, std=std)
    return f


def init_method_normal(sigma):
    return _normal(sigma)


def scaled_init_method_normal(sigma, num_layers):
    return _normal(sigma / math.sqrt(2.0 * num_layers))


def orthogonal_init_method(n_layers=1):
    def f(t):
        return torch.nn.init.orthogonal_(t, gain=math.sqrt(2.0 / n_layers))      # sqrt(2) for the unscaled method
    return f


def xavier_uniform_init_method():
    return lambda t: torch.nn.init.xavier_uniform_(t)


def xavier_normal_init_method():
    return lambda t: torch.nn.init.xavier_normal_(t)


def small_init_init_method(dim):
    return _normal(math.sqrt(2.0 / (5.0 * dim)))


def wang_init_method(n_layers, dim):
    return _normal(2.0 / n_layers / math.sqrt(dim))


def _pick(name, cfg):
    if name == "normal":
        return init_method_normal(cfg.init_method_std)
    if name == "scaled_normal":
        return scaled_init_method_normal(cfg.init_method_std, cfg.num_layers)
    if name == "orthogonal":
        return orthogonal_init_method()
    if name == "scaled_orthogonal":
        return orthogonal_init_method(cfg.num_layers)
    if name == "xavier_uniform":
        return xavier_uniform_init_method()
    if name == "xavier_normal":
        return xavier_normal_init_method()
    if name == "wang_init":
        return wang_init_method(cfg.num_layers, cfg.hidden_size)
    if name == "small_init":
        return small_init_init_method(cfg.hidden_size)
    raise NotImplementedError(f"unknown init method {name!r}")


def get_init_methods(cfg):
    if cfg.use_mup:
        base = _pick(cfg.init_method, cfg)
        scale = cfg.mup_init_scale

        def mup(t):
            base(t)
            return t.mul_(scale)
        return mup, _pick(cfg.output_layer_init_method, cfg)
    return _pick(cfg.init_method, cfg), _pick(cfg.output_layer_init_method, cfg)
