"""Consolidate the fp32 master weights of a ZeRO-1 checkpoint into one state dict per tensor-parallel rank
(role of DeepSpeed's zero_to_fp32 utility, vendored by the reference as tools/zero_to_fp32.py).

The optimizer files hold, per flat parameter group, this rank's slice of the flattened fp32 parameters
(`single_partition_of_fp32_groups`); the model file's `param_shapes` lists the parameter names and shapes of each
group in flattening order.  Concatenating the slices over data-parallel ranks and cutting by shape restores
every tensor.

    python -m savanna_b200.tools.zero_to_fp32 <ckpt>/global_stepN <out.pt> [--mp-rank 0]
"""
from __future__ import annotations

import argparse
import glob
import os
import re
from collections import OrderedDict

import torch


def consolidate(step_dir: str, mp_rank: int = 0) -> "OrderedDict[str, torch.Tensor]":
    ms = torch.load(os.path.join(step_dir, f"mp_rank_{mp_rank:02d}_model_states.pt"), map_location="cpu", weights_only=False)
    shapes = ms["param_shapes"]
    if not shapes:
        raise ValueError("model states carry no param_shapes (written by a resharding tool?)")
    files = glob.glob(os.path.join(step_dir, f"*zero_pp_rank_*_mp_rank_{mp_rank:02d}_optim_states.pt"))
    if not files:
        raise FileNotFoundError("no optimizer state files found")
    files.sort(key=lambda f: int(re.search(r"zero_pp_rank_(\d+)_", f).group(1)))
    parts = [torch.load(f, map_location="cpu", weights_only=False)["optimizer_state_dict"] for f in files]
    n_groups = len(parts[0]["single_partition_of_fp32_groups"])
    if n_groups != len(shapes):
        raise ValueError(f"{n_groups} flat groups in the optimizer state but {len(shapes)} shape groups in the model state")
    out = OrderedDict()
    for gi in range(n_groups):
        flat = torch.cat([p["single_partition_of_fp32_groups"][gi].float().reshape(-1) for p in parts])
        off = 0
        for name, shape in shapes[gi].items():
            n = int(torch.Size(shape).numel())
            out[name] = flat[off:off + n].view(shape).clone()
            off += n
    # the gated MLP keeps w1 and w2 stacked in one parameter; state dicts carry them separately
    for name in [n for n in out if n.endswith(".mlp.w12")]:
        w = out.pop(name)
        half = w.shape[0] // 2
        base = name[: -len("w12")]
        out[base + "w1.weight"], out[base + "w2.weight"] = w[:half].clone(), w[half:].clone()
    # buffers are not part of the optimizer state
    for k, v in ms["module"].items():
        if k not in out:
            out[k] = v
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("checkpoint_dir")
    ap.add_argument("output_file")
    ap.add_argument("--mp-rank", type=int, default=0)
    a = ap.parse_args(argv)
    sd = consolidate(a.checkpoint_dir, a.mp_rank)
    torch.save(sd, a.output_file)
    print(f"wrote {len(sd)} tensors to {a.output_file}")


if __name__ == "__main__":
    main()
