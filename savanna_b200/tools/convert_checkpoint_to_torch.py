"""Checkpoint directory -> one plain PyTorch file for use outside the training framework (reference:
tools/convert_savanna_to_standalone.py, tools/checkpoint_conversion/convert_checkpoint_to_torch.py).

The tensor-parallel model-state shards of a `global_step<N>` directory are merged along their partition dimensions into a
single state dict.  Keys keep the `sequential.<i>.` layout by default; `--strip-prefix` drops `sequential.` and
renumbers the blocks from 0 (embedding and final norm get the names `embedding.*` and `final_norm.*`), which is what
a stand-alone re-implementation of the model usually expects.  `--fp32` takes the weights from the ZeRO optimizer
shards' fp32 master copies instead of the bf16 model states.

    python -m savanna_b200.tools.convert_checkpoint_to_torch <ckpt>/global_step100 out/model.pt [--strip-prefix] [--fp32]
"""
from __future__ import annotations

import argparse
import os
import re
from collections import OrderedDict

import torch

from .reshard_model_parallel import load_shards, merge_module


def standalone_names(full: "OrderedDict[str, torch.Tensor]") -> "OrderedDict[str, torch.Tensor]":
    idx = sorted({int(m.group(1)) for k in full for m in [re.match(r"sequential\.(\d+)\.", k)] if m})
    if not idx:
        return full
    first, last = idx[0], idx[-1]
    blocks = [i for i in idx if i not in (first, last)]
    renum = {i: n for n, i in enumerate(blocks)}
    out = OrderedDict()
    for k, v in full.items():
        m = re.match(r"sequential\.(\d+)\.(.*)", k)
        if not m:
            out[k] = v
            continue
        i, rest = int(m.group(1)), m.group(2)
        if i == first:
            out["embedding." + rest] = v
        elif i == last:
            out["final_norm." + rest.replace("norm.", "", 1)] = v
        else:
            out[f"blocks.{renum[i]}.{rest}"] = v
    return out


def convert(step_dir: str, out_file: str, strip_prefix: bool = False, fp32: bool = False) -> "OrderedDict[str, torch.Tensor]":
    shards = load_shards(step_dir)
    if fp32:
        from .zero_to_fp32 import consolidate
        modules = [consolidate(step_dir, mp_rank=r) for r in range(len(shards))]
    else:
        modules = [s["module"] for s in shards]
    full = merge_module(modules)
    if strip_prefix:
        full = standalone_names(full)
    os.makedirs(os.path.dirname(os.path.abspath(out_file)), exist_ok=True)
    torch.save(full, out_file)
    return full


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("step_dir")
    ap.add_argument("out_file")
    ap.add_argument("--strip-prefix", action="store_true")
    ap.add_argument("--fp32", action="store_true")
    a = ap.parse_args(argv)
    full = convert(a.step_dir, a.out_file, a.strip_prefix, a.fp32)
    n = sum(v.numel() for v in full.values() if torch.is_tensor(v))
    print(f"wrote {len(full)} tensors ({n:,} elements) to {a.out_file}")


if __name__ == "__main__":
    main()
