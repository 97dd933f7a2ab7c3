"""Export a checkpoint to the "universal" per-parameter layout, which can be loaded under any data- / tensor-parallel
degree (role of DeepSpeed's ds_to_universal utility, vendored by the reference as tools/ds_to_universal.py).

Input : <ckpt>/global_step<N>/ with mp_rank_XX_model_states.pt and *zero_pp_rank_D_mp_rank_XX_optim_states.pt
Output: <out>/zero/<parameter name>/fp32.pt, exp_avg.pt, exp_avg_sq.pt, step.pt   one folder per parameter; every
              file is {"param": tensor} (+ "cat_dim" for tensor-parallel parameters, "vocab_tensor" for the embedding)
        <out>/zero/optimizer_state.pt                                                 the non-tensor optimizer state
        <out>/mp_rank_XX_model_states.pt                                              copied
        <ckpt>/latest_universal                                                       tag of the exported step

The flat fp32 partitions are concatenated over the data-parallel ranks and cut by `param_shapes`; tensor-parallel
slices are merged along the dimension the parameter is split on.

    python -m savanna_b200.tools.ds_to_universal --input_folder <ckpt>/global_stepN --output_folder <out>
"""
from __future__ import annotations

import argparse
import glob
import os
import re
import shutil
from collections import OrderedDict
from typing import Dict, List

import torch

from .params import partition_dim

STATES = ("fp32", "exp_avg", "exp_avg_sq")


def _per_param_states(step_dir: str, mp_rank: int) -> "OrderedDict[str, Dict[str, torch.Tensor]]":
    """{name: {fp32, exp_avg, exp_avg_sq, step}} of one tensor-parallel rank."""
    ms = torch.load(os.path.join(step_dir, f"mp_rank_{mp_rank:02d}_model_states.pt"), map_location="cpu", weights_only=False)
    shapes = ms["param_shapes"]
    if not shapes:
        raise ValueError("model states carry no param_shapes (written by a resharding tool?)")
    files = glob.glob(os.path.join(step_dir, f"*zero_pp_rank_*_mp_rank_{mp_rank:02d}_optim_states.pt"))
    if not files:
        raise FileNotFoundError(f"no optimizer state files for tensor-parallel rank {mp_rank} in {step_dir}")
    files.sort(key=lambda f: int(re.search(r"zero_pp_rank_(\d+)_", f).group(1)))
    parts = [torch.load(f, map_location="cpu", weights_only=False)["optimizer_state_dict"] for f in files]
    n_groups = len(parts[0]["single_partition_of_fp32_groups"])
    if n_groups != len(shapes):
        raise ValueError(f"{n_groups} flat groups in the optimizer state but {len(shapes)} shape groups in the model state")
    out: "OrderedDict[str, Dict[str, torch.Tensor]]" = OrderedDict()
    for gi in range(n_groups):
        flats = {
            "fp32": torch.cat([p["single_partition_of_fp32_groups"][gi].float().reshape(-1) for p in parts]),
            "exp_avg": torch.cat([p["base_optimizer_state"]["state"][gi]["exp_avg"].float().reshape(-1) for p in parts]),
            "exp_avg_sq": torch.cat([p["base_optimizer_state"]["state"][gi]["exp_avg_sq"].float().reshape(-1) for p in parts]),
        }
        step = parts[0]["base_optimizer_state"]["state"][gi]["step"]
        off = 0
        for name, shape in shapes[gi].items():
            n = int(torch.Size(shape).numel())
            out[name] = {k: v[off:off + n].view(shape).clone() for k, v in flats.items()}
            out[name]["step"] = step
            off += n
    return out


def convert(step_dir: str, out_dir: str, write_latest: bool = True) -> List[str]:
    model_files = sorted(glob.glob(os.path.join(step_dir, "mp_rank_*_model_states.pt")))
    if not model_files:
        raise FileNotFoundError(f"no mp_rank_*_model_states.pt in {step_dir}")
    tp = len(model_files)
    per_rank = [_per_param_states(step_dir, r) for r in range(tp)]
    zero_dir = os.path.join(out_dir, "zero")
    os.makedirs(zero_dir, exist_ok=True)
    names = list(per_rank[0])
    for name in names:
        d = partition_dim(name) if tp > 1 else None
        pdir = os.path.join(zero_dir, name)
        os.makedirs(pdir, exist_ok=True)
        for st in STATES:
            slices = [pr[name][st] for pr in per_rank]
            if d is None or slices[0].dim() == 0:
                obj = {"param": slices[0]}
            else:
                obj = {"param": torch.cat(slices, dim=d), "cat_dim": d}
            if "word_embeddings" in name:
                obj["vocab_tensor"] = True
            torch.save(obj, os.path.join(pdir, f"{st}.pt"))
        torch.save(torch.tensor(float(per_rank[0][name]["step"])), os.path.join(pdir, "step.pt"))
    first = glob.glob(os.path.join(step_dir, "*zero_pp_rank_0_mp_rank_00_optim_states.pt"))[0]
    osd = torch.load(first, map_location="cpu", weights_only=False)["optimizer_state_dict"]
    keep = {k: v for k, v in osd.items() if k != "single_partition_of_fp32_groups"}
    keep["base_optimizer_state"] = {"param_groups": osd["base_optimizer_state"]["param_groups"]}
    torch.save({"optimizer_state_dict": keep, "universal_checkpoint_info": {"universal_checkpoint_version": 0.2}},
               os.path.join(zero_dir, "optimizer_state.pt"))
    for f in model_files:
        shutil.copy2(f, os.path.join(out_dir, os.path.basename(f)))
    if write_latest:
        root = os.path.dirname(os.path.abspath(step_dir.rstrip("/")))
        with open(os.path.join(root, "latest_universal"), "w") as fh:
            fh.write(os.path.basename(os.path.abspath(out_dir.rstrip("/"))))
    return names


def load_universal_param(out_dir: str, name: str, state: str = "fp32") -> torch.Tensor:
    return torch.load(os.path.join(out_dir, "zero", name, f"{state}.pt"), map_location="cpu", weights_only=False)["param"]


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--input_folder", required=True)
    ap.add_argument("--output_folder", required=True)
    ap.add_argument("--no_latest", action="store_true", help="do not write <ckpt>/latest_universal")
    a = ap.parse_args(argv)
    names = convert(a.input_folder, a.output_folder, not a.no_latest)
    print(f"wrote {len(names)} parameters to {a.output_folder}/zero")


if __name__ == "__main__":
    main()
