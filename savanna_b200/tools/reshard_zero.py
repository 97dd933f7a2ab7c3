"""Re-partition ZeRO-1 optimizer states for a different data-parallel (x context-parallel) size: the flat fp32
master weights and Adam moments of each group are concatenated over the old ranks, the old padding is dropped,
and the result is re-padded and re-cut for the new rank count (role of the reference's repartition scripts under
tools/40b/zero3/, for stage-1 layouts).

    python -m savanna_b200.tools.reshard_zero --input <stepdir> --output <stepdir> --target-dp 4 [--mp-rank 0]
"""
from __future__ import annotations

import argparse
import glob
import os
import re
import shutil

import torch

ALIGN = 256


def _pad_to(n, m):
    return m * ((n + m - 1) // m)


def reshard(step_dir: str, out_dir: str, target_dp: int, mp_rank: int = 0) -> None:
    files = glob.glob(os.path.join(step_dir, f"*zero_pp_rank_*_mp_rank_{mp_rank:02d}_optim_states.pt"))
    files.sort(key=lambda f: int(re.search(r"zero_pp_rank_(\d+)_", f).group(1)))
    if not files:
        raise FileNotFoundError("no optimizer state files found")
    prefix = "bf16_" if os.path.basename(files[0]).startswith("bf16_") else ""
    olds = [torch.load(f, map_location="cpu", weights_only=False) for f in files]
    ms = torch.load(os.path.join(step_dir, f"mp_rank_{mp_rank:02d}_model_states.pt"), map_location="cpu", weights_only=False)
    numels = [sum(int(torch.Size(s).numel()) for s in grp.values()) for grp in ms["param_shapes"]]
    osd0 = olds[0]["optimizer_state_dict"]
    n_groups = len(osd0["single_partition_of_fp32_groups"])
    os.makedirs(out_dir, exist_ok=True)
    new = [{"optimizer_state_dict": {k: v for k, v in osd0.items() if k not in ("single_partition_of_fp32_groups", "base_optimizer_state", "partition_count", "group_paddings")},
            "ds_config": olds[0].get("ds_config"), "ds_version": olds[0].get("ds_version")} for _ in range(target_dp)]
    for r in range(target_dp):
        o = new[r]["optimizer_state_dict"]
        o["single_partition_of_fp32_groups"], o["partition_count"], o["group_paddings"] = [], [target_dp] * n_groups, []
        o["base_optimizer_state"] = {"state": {}, "param_groups": osd0["base_optimizer_state"]["param_groups"]}
    for gi in range(n_groups):
        def cat(getter):
            return torch.cat([getter(o["optimizer_state_dict"]).reshape(-1) for o in olds])[: numels[gi]]
        master = cat(lambda o: o["single_partition_of_fp32_groups"][gi])
        m = cat(lambda o: o["base_optimizer_state"]["state"][gi]["exp_avg"])
        v = cat(lambda o: o["base_optimizer_state"]["state"][gi]["exp_avg_sq"])
        padded = _pad_to(numels[gi], ALIGN * target_dp)
        shard = padded // target_dp

        def cut(t, r):
            full = torch.zeros(padded, dtype=t.dtype)
            full[: t.numel()] = t
            return full[r * shard:(r + 1) * shard].clone()
        step = osd0["base_optimizer_state"]["state"][gi]["step"]
        for r in range(target_dp):
            o = new[r]["optimizer_state_dict"]
            o["single_partition_of_fp32_groups"].append(cut(master, r))
            o["group_paddings"].append(padded - numels[gi] if r == target_dp - 1 else 0)
            o["base_optimizer_state"]["state"][gi] = {"step": step, "exp_avg": cut(m, r), "exp_avg_sq": cut(v, r)}
    for r in range(target_dp):
        torch.save(new[r], os.path.join(out_dir, f"{prefix}zero_pp_rank_{r}_mp_rank_{mp_rank:02d}_optim_states.pt"))
    ms["dp_world_size"] = target_dp
    torch.save(ms, os.path.join(out_dir, f"mp_rank_{mp_rank:02d}_model_states.pt"))
    cdir = os.path.join(step_dir, "configs")
    if os.path.isdir(cdir) and os.path.abspath(out_dir) != os.path.abspath(step_dir):
        shutil.copytree(cdir, os.path.join(out_dir, "configs"), dirs_exist_ok=True)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--input", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--target-dp", type=int, required=True)
    ap.add_argument("--mp-rank", type=int, default=0)
    a = ap.parse_args(argv)
    reshard(a.input, a.output, a.target_dp, a.mp_rank)
    print(f"wrote {a.target_dp} optimizer shard(s) to {a.output}")


if __name__ == "__main__":
    main()
