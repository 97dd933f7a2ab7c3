"""Convert Hyena projection weights from the blocked row order [x1 | x2 | v] to the interleaved order
(x1_0, x2_0, v_0, x1_1, ...) that keeps tensor-parallel splits consistent (`interleave_projections: true`;
reference: tools/7b/conversion/interleave_model_states.py:29-69, savanna/model/block.py:877-888).
Affects `mixer.dense_projection.weight` and `mixer.hyena_proj_conv.short_conv_weight` of Hyena layers.

    python -m savanna_b200.tools.interleave_model_states --input <file.pt> --output <file.pt>
"""
from __future__ import annotations

import argparse

import torch

KEYS = ("mixer.dense_projection.weight", "mixer.hyena_proj_conv.short_conv_weight")


def interleave_rows(w: torch.Tensor) -> torch.Tensor:
    n = w.shape[0]
    if n % 3:
        raise ValueError("projection rows must be divisible by 3")
    d = n // 3
    return w.reshape(3, d, *w.shape[1:]).transpose(0, 1).reshape(n, *w.shape[1:]).contiguous()


def deinterleave_rows(w: torch.Tensor) -> torch.Tensor:
    n = w.shape[0]
    d = n // 3
    return w.reshape(d, 3, *w.shape[1:]).transpose(0, 1).reshape(n, *w.shape[1:]).contiguous()


def convert_module(module: dict, hyena_layer_prefixes=None, inverse: bool = False) -> dict:
    out = dict(module)
    fn = deinterleave_rows if inverse else interleave_rows
    for k, v in module.items():
        if not k.endswith(KEYS):
            continue
        prefix = k.rsplit(".mixer.", 1)[0]
        # attention layers have a dense_projection too but no featuriser conv: only convert layers that have one
        if prefix + ".mixer.hyena_proj_conv.short_conv_weight" not in module:
            continue
        if hyena_layer_prefixes is not None and prefix not in hyena_layer_prefixes:
            continue
        out[k] = fn(v)
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--input", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--inverse", action="store_true")
    a = ap.parse_args(argv)
    sd = torch.load(a.input, map_location="cpu", weights_only=False)
    sd["module"] = convert_module(sd["module"], inverse=a.inverse)
    torch.save(sd, a.output)
    print(f"wrote {a.output}")


if __name__ == "__main__":
    main()
