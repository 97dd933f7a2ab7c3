"""ZeRO stage-3 checkpoint layout: read it, write it, re-partition it, and convert it to and from the stage-1 layout.

DeepSpeed's stage 3 partitions EVERY parameter on its own over the data-parallel ranks: a parameter of n elements is
padded to a multiple of the partition count P and rank r keeps elements [r c, (r+1) c) with c = ceil(n / P); a rank's
flat fp32 group is the concatenation of its pieces in the group's parameter order.  On disk (per tensor-parallel rank mp
and data-parallel rank r):

    zero_pp_rank_<r>_mp_rank_<mp:02d>_model_states.pt           param_shapes (list of name -> shape per group), buffers,
                                                                engine state; parameters themselves are placeholders
    [bf16_]zero_pp_rank_<r>_mp_rank_<mp:02d>_optim_states.pt    optimizer_state_dict: zero_stage 3, partition_count,
                                                                fp32_flat_groups [one flat tensor per group],
                                                                optimizer_state_dict.state[g] = {exp_avg, exp_avg_sq, step}
                                                                partitioned the same way

The stage-1 layout used by this framework's trainer (ckpt/io.py) flattens a whole GROUP first and cuts that once
(`single_partition_of_fp32_groups`, `mp_rank_XX_model_states.pt` with the module).  Role of the reference's stage-3
surgery scripts (tools/40b/zero3/partition_param.py:42-410 `partition_param` / `create_dp_partition`,
convert_zero3_to_zero1.py, zero3_conversion_lib.py): a stage-3 run can be continued here and a checkpoint of this
framework can be handed to a stage-3 run, at any data-parallel size.

    python -m savanna_b200.tools.convert_zero3 to-zero1   --input <step dir (stage 3)> --output <step dir> [--target-dp 8]
    python -m savanna_b200.tools.convert_zero3 from-zero1 --input <step dir (stage 1)> --output <step dir> --target-dp 16
    python -m savanna_b200.tools.convert_zero3 repartition --input <step dir (stage 3)> --output <step dir> --target-dp 4
    python -m savanna_b200.tools.convert_zero3 to-fp32    --input <step dir (stage 3)> --output weights.pt
"""
from __future__ import annotations

import argparse
import glob
import os
import re
import shutil
from collections import OrderedDict
from typing import Dict, List, Tuple

import torch

ALIGN_ZERO1 = 256          # element alignment of a stage-1 shard (parallel/zero.py)
STATE_KEYS = ("exp_avg", "exp_avg_sq")


# ----------------------------------------------------------------------------- per-parameter partitioning


def partition_size(numel: int, count: int) -> int:
    return (numel + count - 1) // count


def partition_param(param: torch.Tensor, count: int, rank: int) -> torch.Tensor:
    """Rank `rank`'s piece of a parameter partitioned over `count` ranks (zero-padded at the end)."""
    flat = param.contiguous().view(-1)
    c = partition_size(flat.numel(), count)
    out = torch.zeros(c, dtype=param.dtype)
    lo = c * rank
    n = max(0, min(c, flat.numel() - lo))
    if n:
        out[:n] = flat[lo:lo + n]
    return out


def flat_groups_for_rank(tensors: Dict[str, torch.Tensor], shape_groups: List[Dict], count: int, rank: int) -> List[torch.Tensor]:
    return [torch.cat([partition_param(tensors[name], count, rank) for name in grp]) if grp else torch.zeros(0)
            for grp in shape_groups]


def merge_flat_groups(per_rank: List[List[torch.Tensor]], shape_groups: List[Dict]) -> Dict[str, torch.Tensor]:
    """Inverse of `flat_groups_for_rank` over all ranks: name -> whole tensor."""
    count = len(per_rank)
    out: Dict[str, torch.Tensor] = OrderedDict()
    for gi, grp in enumerate(shape_groups):
        offs = 0
        for name, shape in grp.items():
            n = int(torch.Size(shape).numel())
            c = partition_size(n, count)
            pieces = [per_rank[r][gi][offs:offs + c] for r in range(count)]
            out[name] = torch.cat(pieces)[:n].view(torch.Size(shape)).clone()
            offs += c
    return out


# ----------------------------------------------------------------------------- file helpers


def _dp_files(step_dir: str, kind: str, mp_rank: int) -> List[str]:
    fs = glob.glob(os.path.join(step_dir, f"*zero_pp_rank_*_mp_rank_{mp_rank:02d}_{kind}.pt"))
    fs.sort(key=lambda f: int(re.search(r"zero_pp_rank_(\d+)_", f).group(1)))
    return fs


def _mp_ranks(step_dir: str) -> List[int]:
    ranks = {int(m.group(1)) for f in os.listdir(step_dir) if (m := re.search(r"mp_rank_(\d+)_", f))}
    return sorted(ranks) or [0]


def _prefix(step_dir: str, mp_rank: int) -> str:
    fs = _dp_files(step_dir, "optim_states", mp_rank)
    return "bf16_" if fs and os.path.basename(fs[0]).startswith("bf16_") else ""


def read_zero3(step_dir: str, mp_rank: int = 0) -> Tuple[Dict, Dict[str, Dict[str, torch.Tensor]], Dict]:
    """(model-state dict of dp rank 0, {"param" | "exp_avg" | "exp_avg_sq": name -> whole fp32 tensor}, optimizer header)."""
    mfiles = _dp_files(step_dir, "model_states", mp_rank)
    ofiles = _dp_files(step_dir, "optim_states", mp_rank)
    if not mfiles or not ofiles:
        raise FileNotFoundError(f"no stage-3 files for mp rank {mp_rank} in {step_dir}")
    ms = torch.load(mfiles[0], map_location="cpu", weights_only=False)
    shapes = ms["param_shapes"]
    osds = [torch.load(f, map_location="cpu", weights_only=False)["optimizer_state_dict"] for f in ofiles]
    if len(osds) != int(osds[0].get("partition_count", len(osds)) if not isinstance(osds[0].get("partition_count"), list)
                       else osds[0]["partition_count"][0]):
        raise ValueError("number of optimizer files differs from the recorded partition count")
    whole = {"param": merge_flat_groups([o["fp32_flat_groups"] for o in osds], shapes)}
    base = [o["optimizer_state_dict"]["state"] for o in osds]
    for key in STATE_KEYS:
        whole[key] = merge_flat_groups([[st[g][key] for g in range(len(shapes))] for st in base], shapes)
    header = {k: v for k, v in osds[0].items() if k not in ("fp32_flat_groups", "optimizer_state_dict")}
    header["param_groups"] = osds[0]["optimizer_state_dict"].get("param_groups")
    header["step"] = [base[0][g].get("step", 0) for g in range(len(shapes))]
    return ms, whole, header


def write_zero3(out_dir: str, ms: Dict, whole: Dict[str, Dict[str, torch.Tensor]], header: Dict, target_dp: int, mp_rank: int,
                prefix: str = "bf16_") -> None:
    os.makedirs(out_dir, exist_ok=True)
    shapes = ms["param_shapes"]
    for r in range(target_dp):
        flat = flat_groups_for_rank(whole["param"], shapes, target_dp, r)
        state = {}
        for g in range(len(shapes)):
            state[g] = {"step": header["step"][g]}
        for key in STATE_KEYS:
            pieces = flat_groups_for_rank(whole[key], shapes, target_dp, r)
            for g in range(len(shapes)):
                state[g][key] = pieces[g]
        osd = {k: v for k, v in header.items() if k not in ("param_groups", "step")}
        osd.update({"zero_stage": 3, "partition_count": target_dp, "fp32_flat_groups": flat,
                    "optimizer_state_dict": {"state": state, "param_groups": header.get("param_groups")}})
        torch.save({"optimizer_state_dict": osd, "ds_config": ms.get("ds_config"), "ds_version": ms.get("ds_version")},
                   os.path.join(out_dir, f"{prefix}zero_pp_rank_{r}_mp_rank_{mp_rank:02d}_optim_states.pt"))
        m = dict(ms)
        m["dp_world_size"] = target_dp
        # stage 3 keeps no whole parameters in the model file: placeholders, as DeepSpeed writes them
        m["module"] = OrderedDict((k, (torch.empty(0, dtype=v.dtype) if k in whole["param"] else v))
                                  for k, v in (ms.get("module") or {}).items())
        torch.save(m, os.path.join(out_dir, f"zero_pp_rank_{r}_mp_rank_{mp_rank:02d}_model_states.pt"))


# ----------------------------------------------------------------------------- stage 1 <-> whole tensors


def _pad_to(n: int, m: int) -> int:
    return m * ((n + m - 1) // m)


def read_zero1(step_dir: str, mp_rank: int = 0):
    ms = torch.load(os.path.join(step_dir, f"mp_rank_{mp_rank:02d}_model_states.pt"), map_location="cpu", weights_only=False)
    shapes = ms["param_shapes"]
    osds = [torch.load(f, map_location="cpu", weights_only=False)["optimizer_state_dict"] for f in _dp_files(step_dir, "optim_states", mp_rank)]
    if not osds:
        raise FileNotFoundError(f"no optimizer state files for mp rank {mp_rank} in {step_dir}")

    def cut(flats: List[torch.Tensor], grp) -> Dict[str, torch.Tensor]:
        flat, off, out = torch.cat([f.float().reshape(-1) for f in flats]), 0, OrderedDict()
        for name, shape in grp.items():
            n = int(torch.Size(shape).numel())
            out[name] = flat[off:off + n].view(torch.Size(shape)).clone()
            off += n
        return out
    whole = {"param": OrderedDict(), "exp_avg": OrderedDict(), "exp_avg_sq": OrderedDict()}
    for g, grp in enumerate(shapes):
        whole["param"].update(cut([o["single_partition_of_fp32_groups"][g] for o in osds], grp))
        for key in STATE_KEYS:
            whole[key].update(cut([o["base_optimizer_state"]["state"][g][key] for o in osds], grp))
    o0 = osds[0]
    header = {k: v for k, v in o0.items() if k not in ("single_partition_of_fp32_groups", "base_optimizer_state", "partition_count",
                                                       "group_paddings", "zero_stage")}
    header["param_groups"] = o0["base_optimizer_state"].get("param_groups")
    header["step"] = [o0["base_optimizer_state"]["state"][g].get("step", 0) for g in range(len(shapes))]
    return ms, whole, header


def write_zero1(out_dir: str, ms: Dict, whole, header: Dict, target_dp: int, mp_rank: int, prefix: str = "bf16_") -> None:
    os.makedirs(out_dir, exist_ok=True)
    shapes = ms["param_shapes"]
    m = dict(ms)
    m["dp_world_size"] = target_dp
    module = OrderedDict(ms.get("module") or {})
    for name, t in whole["param"].items():
        ref_t = module.get(name)
        dtype = ref_t.dtype if isinstance(ref_t, torch.Tensor) and ref_t.numel() else (torch.bfloat16 if prefix else torch.float32)
        module[name] = t.to(dtype)
    # the gated MLP's stacked parameter is stored as w1 / w2 in module state dicts
    for name in [n for n in module if n.endswith(".mlp.w12")]:
        w = module.pop(name)
        half = w.shape[0] // 2
        module[name[:-3] + "w1.weight"], module[name[:-3] + "w2.weight"] = w[:half].clone(), w[half:].clone()
    m["module"] = module
    torch.save(m, os.path.join(out_dir, f"mp_rank_{mp_rank:02d}_model_states.pt"))
    for r in range(target_dp):
        masters, state, pads = [], {}, []
        for g, grp in enumerate(shapes):
            def shard(src):
                flat = torch.cat([src[name].float().reshape(-1) for name in grp]) if grp else torch.zeros(0)
                padded = _pad_to(flat.numel(), ALIGN_ZERO1 * target_dp)
                flat = torch.nn.functional.pad(flat, (0, padded - flat.numel()))
                c = padded // target_dp
                return flat[r * c:(r + 1) * c].clone(), padded - sum(int(torch.Size(s).numel()) for s in grp.values())
            mst, pad = shard(whole["param"])
            masters.append(mst)
            pads.append(pad if r == target_dp - 1 else 0)
            state[g] = {"step": header["step"][g]}
            for key in STATE_KEYS:
                state[g][key] = shard(whole[key])[0]
        osd = {k: v for k, v in header.items() if k not in ("param_groups", "step")}
        osd.update({"zero_stage": 1, "partition_count": [target_dp] * len(shapes), "single_partition_of_fp32_groups": masters,
                    "group_paddings": pads, "base_optimizer_state": {"state": state, "param_groups": header.get("param_groups")}})
        torch.save({"optimizer_state_dict": osd, "ds_config": ms.get("ds_config"), "ds_version": ms.get("ds_version")},
                   os.path.join(out_dir, f"{prefix}zero_pp_rank_{r}_mp_rank_{mp_rank:02d}_optim_states.pt"))


# ----------------------------------------------------------------------------- commands


def _copy_rest(src: str, dst: str) -> None:
    for name in os.listdir(src):
        p = os.path.join(src, name)
        if os.path.isdir(p) and not os.path.exists(os.path.join(dst, name)):
            shutil.copytree(p, os.path.join(dst, name))


def to_zero1(inp: str, out: str, target_dp: int = None) -> None:
    for mp in _mp_ranks(inp):
        ms, whole, header = read_zero3(inp, mp)
        dp = target_dp or len(_dp_files(inp, "optim_states", mp))
        write_zero1(out, ms, whole, header, dp, mp, _prefix(inp, mp))
    _copy_rest(inp, out)


def from_zero1(inp: str, out: str, target_dp: int) -> None:
    for mp in _mp_ranks(inp):
        ms, whole, header = read_zero1(inp, mp)
        write_zero3(out, ms, whole, header, target_dp, mp, _prefix(inp, mp))
    _copy_rest(inp, out)


def repartition(inp: str, out: str, target_dp: int) -> None:
    for mp in _mp_ranks(inp):
        ms, whole, header = read_zero3(inp, mp)
        write_zero3(out, ms, whole, header, target_dp, mp, _prefix(inp, mp))
    _copy_rest(inp, out)


def to_fp32(inp: str, out_file: str, mp_rank: int = 0) -> None:
    ms, whole, _ = read_zero3(inp, mp_rank)
    sd = OrderedDict(whole["param"])
    for k, v in (ms.get("module") or {}).items():
        if k not in sd and isinstance(v, torch.Tensor) and v.numel():
            sd[k] = v
    torch.save(sd, out_file)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("command", choices=["to-zero1", "from-zero1", "repartition", "to-fp32"])
    ap.add_argument("--input", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--target-dp", type=int, default=None)
    ap.add_argument("--mp-rank", type=int, default=0)
    a = ap.parse_args(argv)
    if a.command == "to-zero1":
        to_zero1(a.input, a.output, a.target_dp)
    elif a.command == "to-fp32":
        to_fp32(a.input, a.output, a.mp_rank)
    else:
        if not a.target_dp:
            ap.error("--target-dp is required")
        (from_zero1 if a.command == "from-zero1" else repartition)(a.input, a.output, a.target_dp)
    print(f"{a.command}: wrote {a.output}")


if __name__ == "__main__":
    main()
