"""Export model states to the flat key layout of the vortex inference project (`blocks.<i>....`), merging
tensor-parallel shards first (reference: tools/convert_checkpoint_to_vortex.py:32-157).

Key map (per block i, source prefix `sequential.<i+2>.`):
    input_layernorm.{weight|scale}          -> blocks.i.pre_norm.scale
    pre_mlp_layernorm.{weight|scale}        -> blocks.i.post_norm.scale
    mixer.dense_projection.weight           -> blocks.i.projections.weight          (attention: inner_mha_cls.Wqkv.weight)
    mixer.hyena_proj_conv.short_conv_weight -> blocks.i.filter.short_filter_weight
    mixer.mixer.conv_bias                   -> blocks.i.filter.D
    mixer.mixer.filter.{h,decay} (MR)       -> blocks.i.filter.h = h*decay (first hyena_mr_len taps)
    mixer.mixer.filter.{gamma,R,p} (LI)     -> blocks.i.filter.log_poles = -exp(p)exp(gamma), .residues = R
    mixer.mixer.short_conv.short_conv_weight (SE) -> blocks.i.filter.h
    mixer.dense.{weight,bias}               -> blocks.i.out_filter_dense.{weight,bias}  (attention: inner_mha_cls.out_proj)
    mlp.w1/w2/w3.weight                     -> blocks.i.mlp.l1/l2/l3.weight
    word_embeddings.weight                  -> embedding_layer.weight and unembed.weight;  final norm -> norm.scale

    python -m savanna_b200.tools.convert_checkpoint_to_vortex --input <stepdir> --output model.pt [--mr-len 128]
"""
from __future__ import annotations

import argparse
import re

import torch

from .reshard_model_parallel import load_shards, merge_module


def convert(module: dict, mr_len: int = 128) -> dict:
    out = {}
    layer_ids = sorted({int(m.group(1)) for k in module for m in [re.match(r"sequential\.(\d+)\.", k)] if m})
    blocks = [i for i in layer_ids if any(k.startswith(f"sequential.{i}.mixer.") for k in module)]
    for bi, li in enumerate(blocks):
        p = f"sequential.{li}."
        g = lambda name: module.get(p + name)          # noqa: E731
        def first(*names):
            for n in names:
                if g(n) is not None:
                    return g(n)
            return None
        dst = f"blocks.{bi}."
        out[dst + "pre_norm.scale"] = first("input_layernorm.weight", "input_layernorm.scale")
        out[dst + "post_norm.scale"] = first("pre_mlp_layernorm.weight", "pre_mlp_layernorm.scale")
        is_hyena = g("mixer.hyena_proj_conv.short_conv_weight") is not None
        if is_hyena:
            out[dst + "projections.weight"] = g("mixer.dense_projection.weight")
            w = g("mixer.hyena_proj_conv.short_conv_weight")
            out[dst + "filter.short_filter_weight"] = w.reshape(w.shape[0], 1, w.shape[-1])
            if g("mixer.mixer.conv_bias") is not None:
                out[dst + "filter.D"] = g("mixer.mixer.conv_bias")
            if g("mixer.mixer.filter.h") is not None:
                h, d = g("mixer.mixer.filter.h"), g("mixer.mixer.filter.decay")
                n = min(mr_len, h.shape[-1])
                out[dst + "filter.h"] = (h[:, :n].float() * d[:, :n].float()).unsqueeze(1)
            elif g("mixer.mixer.filter.gamma") is not None:
                gamma, R, pp = (g(f"mixer.mixer.filter.{n}").float() for n in ("gamma", "R", "p"))
                out[dst + "filter.log_poles"] = (-torch.exp(pp) * torch.exp(gamma)).unsqueeze(-1)
                out[dst + "filter.residues"] = R
            elif g("mixer.mixer.short_conv.short_conv_weight") is not None:
                w = g("mixer.mixer.short_conv.short_conv_weight")
                out[dst + "filter.h"] = w.reshape(w.shape[0], 1, w.shape[-1])
            out[dst + "out_filter_dense.weight"] = g("mixer.dense.weight")
            out[dst + "out_filter_dense.bias"] = g("mixer.dense.bias")
        else:
            out[dst + "inner_mha_cls.Wqkv.weight"] = g("mixer.dense_projection.weight")
            out[dst + "inner_mha_cls.out_proj.weight"] = g("mixer.dense.weight")
            out[dst + "inner_mha_cls.out_proj.bias"] = g("mixer.dense.bias")
            if g("mixer.rotary_emb.inv_freq") is not None:
                out[dst + "inner_mha_cls.rotary_emb.inv_freq"] = g("mixer.rotary_emb.inv_freq")
        for src, d2 in (("mlp.w1.weight", "mlp.l1.weight"), ("mlp.w2.weight", "mlp.l2.weight"), ("mlp.w3.weight", "mlp.l3.weight")):
            if g(src) is not None:
                out[dst + d2] = g(src)
    emb = module.get("sequential.0.word_embeddings.weight")
    if emb is not None:
        out["embedding_layer.weight"] = emb
        out["unembed.weight"] = emb
    for k, v in module.items():
        if re.match(r"sequential\.\d+\.norm\.(weight|scale)$", k):
            out["norm.scale"] = v
    return {k: v for k, v in out.items() if v is not None}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--input", required=True, help="global_step directory")
    ap.add_argument("--output", required=True)
    ap.add_argument("--mr-len", type=int, default=128)
    a = ap.parse_args(argv)
    module = merge_module([s["module"] for s in load_shards(a.input)])
    sd = convert(module, a.mr_len)
    torch.save(sd, a.output)
    print(f"wrote {len(sd)} tensors to {a.output}")


if __name__ == "__main__":
    main()
