"""Throughput tuner: generates the grid of (micro batch, accumulation, tensor / context parallel size,
activation-checkpoint interval, ZeRO stage) variants of a base config that fit a GPU count, with one SLURM
script per variant or ONE job-array script (`--array`: task i runs variant i, `--array-parallel` bounds how many run at
once), optionally wrapped in the Nsight Systems preset (`--nsys`), and collects the `tokens/s/gpu` lines of their logs
into a table (reference: tuner/tuner.py:34-340, tuner/utils.py:81-200).

    python -m tuner.tuner generate --base configs/baseline/evo2_7b_8k.yml --gpus 8 --out tuner_runs \
        --micro-batch 1 2 --tp 1 2 --checkpoint-num-layers 0 2 4
    python -m tuner.tuner collect --logs tuner_runs/logs
"""
from __future__ import annotations

import argparse
import glob
import itertools
import os
import re

import yaml


def variants(base: dict, gpus: int, micro_batches, tps, cps, ckpt_layers, zero_stages, global_batch=None):
    for mb, tp, cp, ck, zs in itertools.product(micro_batches, tps, cps, ckpt_layers, zero_stages):
        if gpus % (tp * cp):
            continue
        dp = gpus // (tp * cp)
        cfg = dict(base)
        cfg.update({"train_micro_batch_size_per_gpu": mb, "model_parallel_size": tp, "context_parallel_size": cp})
        cfg.pop("train-micro-batch-size-per-gpu", None)
        if global_batch:
            if global_batch % (mb * dp):
                continue
            cfg["gradient_accumulation_steps"] = global_batch // (mb * dp)
        cfg["checkpoint-activations"] = ck > 0
        if ck > 0:
            cfg["checkpoint-num-layers"] = ck
        z = dict(cfg.get("zero_optimization") or {})
        z["stage"] = zs
        cfg["zero_optimization"] = z
        if tp > 1:
            cfg["sequence_parallel"] = True
        if cp > 1:
            cfg.update({"use_cp_hyena": True, "use_cp_ring": True})
        yield f"mb{mb}_tp{tp}_cp{cp}_ac{ck}_z{zs}", cfg


def cmd_generate(a):
    base = yaml.load(open(a.base), Loader=yaml.FullLoader)
    os.makedirs(os.path.join(a.out, "configs"), exist_ok=True)
    names = []
    for tag, cfg in variants(base, a.gpus, a.micro_batch, a.tp, a.cp, a.checkpoint_num_layers, a.zero_stage, a.global_batch):
        cfg["train-iters"] = a.iters
        cfg["log-interval"] = 1
        path = os.path.join(a.out, "configs", f"{tag}.yml")
        with open(path, "w") as fh:
            yaml.safe_dump(cfg, fh, sort_keys=False)
        names.append(tag)
    from launcher.slurm import build_script, nsys_command
    nodes = max(1, a.gpus // a.gpus_per_node)
    logs = os.path.join(a.out, "logs")
    prof = nsys_command(os.path.join(logs, "nsys-$TAG"), a.nsys_warmup_steps, a.nsys_num_steps) if a.nsys else None
    if a.array and names:
        # one script for all variants: the array index selects the configuration file
        with open(os.path.join(a.out, "variants.txt"), "w") as fh:
            fh.write("\n".join(names) + "\n")
        script = build_script("tune", nodes, min(a.gpus, a.gpus_per_node), os.getcwd(), os.path.join(a.out, "configs"),
                              ["$TAG.yml"], output_dir=logs, time_limit=a.time, profile_cmd=prof)
        head, _, body = script.partition("\n\nset -euo pipefail")
        limit = f"%{a.array_parallel}" if a.array_parallel else ""
        head += f"\n#SBATCH --array=0-{len(names) - 1}{limit}"
        head = head.replace("%x-%j", "%x-%A_%a")
        pick = f'\nTAG=$(sed -n "$((SLURM_ARRAY_TASK_ID + 1))p" {os.path.join(a.out, "variants.txt")})\nexport TAG'
        body = body.replace("'$TAG.yml'", '"$TAG.yml"')
        with open(os.path.join(a.out, "array.sbatch"), "w") as fh:
            fh.write(head + "\n\nset -euo pipefail" + pick + body)
        with open(os.path.join(a.out, "submit_all.sh"), "w") as fh:
            fh.write(f"#!/bin/bash\nsbatch {os.path.join(a.out, 'array.sbatch')}\n")
        print(f"generated {len(names)} variants under {a.out} as one job array")
        return
    for tag in names:
        script = build_script(f"tune_{tag}", nodes, min(a.gpus, a.gpus_per_node), os.getcwd(), os.path.join(a.out, "configs"),
                              [f"{tag}.yml"], output_dir=logs, time_limit=a.time,
                              profile_cmd=prof.replace("$TAG", tag) if prof else None)
        with open(os.path.join(a.out, f"{tag}.sbatch"), "w") as fh:
            fh.write(script)
    with open(os.path.join(a.out, "submit_all.sh"), "w") as fh:
        fh.write("#!/bin/bash\n" + "\n".join(f"sbatch {os.path.join(a.out, t)}.sbatch" for t in names) + "\n")
    print(f"generated {len(names)} variants under {a.out}")


def cmd_collect(a):
    rows = []
    for f in sorted(glob.glob(os.path.join(a.logs, "*.out"))):
        vals = [float(m.group(1).replace(",", "")) for m in re.finditer(r"tokens/s/gpu: ([\d,\.]+)", open(f).read())]
        if vals:
            tail = vals[len(vals) // 2:]
            rows.append((os.path.basename(f), sum(tail) / len(tail), max(vals)))
    rows.sort(key=lambda r: -r[1])
    print(f"{'run':60s} {'mean tok/s/gpu (2nd half)':>26s} {'max':>12s}")
    for r in rows:
        print(f"{r[0]:60s} {r[1]:26,.0f} {r[2]:12,.0f}")


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("generate")
    g.add_argument("--base", required=True)
    g.add_argument("--gpus", type=int, required=True)
    g.add_argument("--gpus-per-node", type=int, default=8)
    g.add_argument("--out", required=True)
    g.add_argument("--micro-batch", type=int, nargs="+", default=[1])
    g.add_argument("--tp", type=int, nargs="+", default=[1])
    g.add_argument("--cp", type=int, nargs="+", default=[1])
    g.add_argument("--checkpoint-num-layers", type=int, nargs="+", default=[0])
    g.add_argument("--zero-stage", type=int, nargs="+", default=[1])
    g.add_argument("--global-batch", type=int, default=None)
    g.add_argument("--iters", type=int, default=20)
    g.add_argument("--time", default="00:30:00")
    g.add_argument("--array", action="store_true", help="one SLURM job array instead of one script per variant")
    g.add_argument("--array-parallel", type=int, default=0, help="at most this many array tasks at once (0 = no limit)")
    g.add_argument("--nsys", action="store_true", help="wrap the workers in the Nsight Systems preset")
    g.add_argument("--nsys-warmup-steps", type=int, default=3)
    g.add_argument("--nsys-num-steps", type=int, default=2)
    g.set_defaults(fn=cmd_generate)
    c = sub.add_parser("collect")
    c.add_argument("--logs", required=True)
    c.set_defaults(fn=cmd_collect)
    a = ap.parse_args(argv)
    a.fn(a)


if __name__ == "__main__":
    main()
