"""Change the tensor-parallel degree of a checkpoint's model states: gather every partitioned tensor along its
partition dim over the source ranks, re-chunk for the target ranks (any TP -> any TP).  Works on
`mp_rank_XX_model_states.pt` files (reference: tools/convert_checkpoint_model_parallel.py:28-178).

    python -m savanna_b200.tools.reshard_model_parallel --input <ckpt>/global_stepN --output <dir> --target-mp 4
"""
from __future__ import annotations

import argparse
import glob
import re
import os
import shutil
from typing import Dict, List

import torch

from .params import partition_dim


def load_shards(step_dir: str) -> List[Dict]:
    """One model-states dict per tensor-parallel rank.  Two layouts are read: `mp_rank_<TP>_model_states.pt` holding
    the whole module, and the pipeline engine's one file per layer slot, `layer_<IDX>-model_<TP>-model_states.pt`
    (role of the reference's savanna/loading.py raw per-layer load): the layer files are put back under
    `sequential.<IDX>.` keys, one assembled module per tensor-parallel rank, whatever the number of stages was."""
    layer_files = sorted(glob.glob(os.path.join(step_dir, "layer_*-model_*-model_states.pt")))
    files = sorted(glob.glob(os.path.join(step_dir, "mp_rank_*_model_states.pt")))
    if layer_files:
        by_tp: Dict[int, Dict[int, str]] = {}
        for f in layer_files:
            m = re.match(r"layer_(\d+)-model_(\d+)-model_states\.pt$", os.path.basename(f))
            by_tp.setdefault(int(m.group(2)), {})[int(m.group(1))] = f
        engine = torch.load(files[0], map_location="cpu", weights_only=False) if files else {}
        out = []
        for tp in sorted(by_tp):
            module = {}
            for idx in sorted(by_tp[tp]):
                for k, v in torch.load(by_tp[tp][idx], map_location="cpu", weights_only=False).items():
                    module[f"sequential.{idx}.{k}"] = v
            shard = {k: v for k, v in engine.items() if k != "module"}
            shard["module"] = module
            shard["mp_world_size"] = len(by_tp)
            out.append(shard)
        return out
    if not files:
        raise FileNotFoundError(f"no mp_rank_*_model_states.pt and no layer_*-model_*-model_states.pt in {step_dir}")
    return [torch.load(f, map_location="cpu", weights_only=False) for f in files]


def merge_module(shards: List[Dict[str, torch.Tensor]]) -> Dict[str, torch.Tensor]:
    out = {}
    for k in shards[0]:
        ts = [s[k] for s in shards]
        d = partition_dim(k, ts[0].dim() if isinstance(ts[0], torch.Tensor) else None)
        if d is None or not isinstance(ts[0], torch.Tensor) or ts[0].dim() == 0 or len(ts) == 1:
            out[k] = ts[0]
        else:
            out[k] = torch.cat(ts, dim=d)
    return out


def split_module(full: Dict[str, torch.Tensor], target_mp: int) -> List[Dict[str, torch.Tensor]]:
    outs = [dict() for _ in range(target_mp)]
    for k, t in full.items():
        d = partition_dim(k, t.dim() if isinstance(t, torch.Tensor) else None)
        if d is None or not isinstance(t, torch.Tensor) or t.dim() == 0 or target_mp == 1:
            for o in outs:
                o[k] = t
            continue
        if t.shape[d] % target_mp:
            raise ValueError(f"{k}: dim {d} of size {t.shape[d]} is not divisible by {target_mp}")
        for o, c in zip(outs, t.chunk(target_mp, dim=d)):
            o[k] = c.clone().contiguous()
    return outs


def reshard(step_dir: str, out_dir: str, target_mp: int) -> None:
    shards = load_shards(step_dir)
    full = merge_module([s["module"] for s in shards])
    parts = split_module(full, target_mp)
    os.makedirs(out_dir, exist_ok=True)
    for r, mod in enumerate(parts):
        sd = {k: v for k, v in shards[0].items() if k != "module"}
        sd["module"] = mod
        sd["mp_world_size"] = target_mp
        if "param_shapes" in sd and sd["param_shapes"] is not None:
            sd["param_shapes"] = None          # stale after resharding; rebuilt on the next save
        torch.save(sd, os.path.join(out_dir, f"mp_rank_{r:02d}_model_states.pt"))
    cdir = os.path.join(step_dir, "configs")
    if os.path.isdir(cdir):
        shutil.copytree(cdir, os.path.join(out_dir, "configs"), dirs_exist_ok=True)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--input", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--target-mp", type=int, required=True)
    a = ap.parse_args(argv)
    reshard(a.input, a.output, a.target_mp)
    print(f"wrote {a.target_mp} model-parallel shard(s) to {a.output}")


if __name__ == "__main__":
    main()
