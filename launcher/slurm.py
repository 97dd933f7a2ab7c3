"""SLURM batch-script generator (no pdsh / ssh fan-out needed).

The generated script has two steps, as in the reference's launcher (launcher/README.md:18-34,
launcher/slurm_template.py:16-470, launcher/generate_distributed_launcher.py:35-122):
  1. on the first node, `launch.py --train-args-output` parses and validates the YAML files once and writes the
     encoded worker arguments to a file on the shared filesystem;
  2. `srun` starts one launcher per node — `torchrun` (default, with --max-restarts for relaunch after a failure),
     or one task per GPU with plain `srun` — which run `train.py` with those arguments.
Options cover NUMA / CPU binding, environment exports (allocator configuration, NCCL settings), an optional
profiler wrapper and automatic requeue (`--dependency=singleton` chains + relaunch loop).

    python -m launcher.slurm --job-name evo2 --nodes 2 --gpus-per-node 8 --config-dir configs model.yml data.yml \
        --output job.sbatch
"""
from __future__ import annotations

import argparse
import os
import shlex
from typing import Dict, List, Optional

DEFAULT_ENV = {
    "PYTORCH_CUDA_ALLOC_CONF": "expandable_segments:True",
    "NCCL_DEBUG": "WARN",
    "OMP_NUM_THREADS": "8",
}


def sbatch_header(job_name: str, nodes: int, gpus_per_node: int, time_limit: str, partition: Optional[str],
                  account: Optional[str], output_dir: str, singleton: bool, extra: Optional[List[str]] = None) -> List[str]:
    lines = ["#!/bin/bash", f"#SBATCH --job-name={job_name}", f"#SBATCH --nodes={nodes}", "#SBATCH --ntasks-per-node=1",
             f"#SBATCH --gpus-per-node={gpus_per_node}", f"#SBATCH --time={time_limit}", "#SBATCH --exclusive",
             f"#SBATCH --output={output_dir}/%x-%j.out", f"#SBATCH --error={output_dir}/%x-%j.err"]
    if partition:
        lines.append(f"#SBATCH --partition={partition}")
    if account:
        lines.append(f"#SBATCH --account={account}")
    if singleton:
        lines.append("#SBATCH --dependency=singleton")
    for e in extra or []:
        lines.append(f"#SBATCH {e}")
    return lines


def build_script(job_name: str, nodes: int, gpus_per_node: int, repo_dir: str, conf_dir: Optional[str], conf_files: List[str],
                 launcher: str = "torch", time_limit: str = "24:00:00", partition: Optional[str] = None,
                 account: Optional[str] = None, output_dir: str = "logs", env: Optional[Dict[str, str]] = None,
                 max_restarts: int = 0, numa_bind: bool = False, profile_cmd: Optional[str] = None, master_port: int = 29500,
                 singleton: bool = False, container: Optional[str] = None, python: str = "python") -> str:
    if launcher not in ("torch", "srun"):
        raise ValueError("launcher must be 'torch' (one torchrun per node) or 'srun' (one task per GPU)")
    lines = sbatch_header(job_name, nodes, gpus_per_node, time_limit, partition, account, output_dir, singleton)
    if launcher == "srun":
        lines = [ln.replace("--ntasks-per-node=1", f"--ntasks-per-node={gpus_per_node}") for ln in lines]
    lines += ["", "set -euo pipefail", f"mkdir -p {shlex.quote(output_dir)}", f"cd {shlex.quote(repo_dir)}", ""]
    envs = dict(DEFAULT_ENV)
    envs.update(env or {})
    for k, v in envs.items():
        lines.append(f"export {k}={shlex.quote(str(v))}")
    world = nodes * gpus_per_node
    lines += [f"export GLOBAL_NUM_GPUS={world}",
              'export MASTER_ADDR=$(scontrol show hostnames "$SLURM_JOB_NODELIST" | head -n 1)',
              f"export MASTER_PORT={master_port}", 'TRAIN_ARGS_FILE="$PWD/' + output_dir + '/train_args-$SLURM_JOB_ID.txt"', ""]
    conf = (f"-d {shlex.quote(conf_dir)} " if conf_dir else "") + " ".join(shlex.quote(c) for c in conf_files)
    srun_pre = f"srun --container-image={shlex.quote(container)} " if container else "srun "
    lines += ["# step 1: parse the configuration once, on the first node",
              f"{srun_pre}--nodes=1 --ntasks=1 -w \"$MASTER_ADDR\" {python} launch.py train.py {conf} "
              f"--num_gpus {world} --train-args-output \"$TRAIN_ARGS_FILE\"", ""]
    bind = "numactl --cpunodebind=$((SLURM_LOCALID / 4)) --membind=$((SLURM_LOCALID / 4)) " if numa_bind else ""
    prof = (profile_cmd + " ") if profile_cmd else ""
    lines.append("# step 2: start the workers")
    if launcher == "torch":
        lines.append(f"{srun_pre}--nodes={nodes} --ntasks-per-node=1 bash -c '{prof}{python} -m torch.distributed.run "
                     f"--nnodes={nodes} --nproc-per-node={gpus_per_node} --rdzv-backend=c10d --rdzv-endpoint=$MASTER_ADDR:$MASTER_PORT "
                     f"--max-restarts={max_restarts} train.py $(cat \"$TRAIN_ARGS_FILE\")'")
    else:
        lines.append(f"{srun_pre}--nodes={nodes} --ntasks-per-node={gpus_per_node} bash -c 'export RANK=$SLURM_PROCID "
                     f"LOCAL_RANK=$SLURM_LOCALID WORLD_SIZE=$SLURM_NTASKS; {bind}{prof}{python} train.py $(cat \"$TRAIN_ARGS_FILE\")'")
    return "\n".join(lines) + "\n"


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("conf_files", nargs="+")
    ap.add_argument("--config-dir", "-d", default=None)
    ap.add_argument("--job-name", default="savanna_b200")
    ap.add_argument("--nodes", type=int, default=1)
    ap.add_argument("--gpus-per-node", type=int, default=8)
    ap.add_argument("--launcher", default="torch", choices=["torch", "srun"])
    ap.add_argument("--time", default="24:00:00")
    ap.add_argument("--partition", default=None)
    ap.add_argument("--account", default=None)
    ap.add_argument("--output-dir", default="logs")
    ap.add_argument("--max-restarts", type=int, default=0)
    ap.add_argument("--numa-bind", action="store_true")
    ap.add_argument("--singleton", action="store_true")
    ap.add_argument("--container", default=None)
    ap.add_argument("--profile-cmd", default=None)
    ap.add_argument("--env", action="append", default=[], help="KEY=VALUE (repeatable)")
    ap.add_argument("--output", default=None)
    a = ap.parse_args(argv)
    env = dict(e.split("=", 1) for e in a.env)
    script = build_script(a.job_name, a.nodes, a.gpus_per_node, os.getcwd(), a.config_dir, a.conf_files, a.launcher, a.time,
                          a.partition, a.account, a.output_dir, env, a.max_restarts, a.numa_bind, a.profile_cmd,
                          singleton=a.singleton, container=a.container)
    if a.output:
        with open(a.output, "w") as fh:
            fh.write(script)
        print(f"wrote {a.output}")
    else:
        print(script)


if __name__ == "__main__":
    main()
