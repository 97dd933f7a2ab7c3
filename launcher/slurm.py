"""SLURM batch-script generator (no pdsh / ssh fan-out needed).

The generated script has two steps, as in the reference's launcher (launcher/README.md:18-34,
launcher/slurm_template.py:16-470, launcher/generate_distributed_launcher.py:35-122):
  1. on the first node, `launch.py --train-args-output` parses and validates the YAML files once and writes the
     encoded worker arguments to a file on the shared filesystem;
  2. `srun` starts one launcher per node — `torchrun` (default, with --max-restarts for relaunch after a failure),
     or one task per GPU with plain `srun` — which run `train.py` with those arguments.
Options cover NUMA / CPU binding, environment exports (allocator configuration, NCCL settings), an optional
profiler wrapper (free-form, or the Nsight Systems preset of the reference's tuner), automatic requeue
(`--dependency=singleton` chains + relaunch loop), configuration overrides written as an extra YAML file
(`--override KEY=VALUE`, the reference's launcher/utils.py:341-394), a per-run checkpoint directory used for both `save`
and `load` so that a requeued job resumes by itself (`--checkpoint-dir`), and the run-time health options
(`--straggler-interval` turns the straggler report on, `--watchdog-timeout` the per-step watchdog with its heartbeat
directory under the output directory).

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


def nsys_command(output: str, warmup_steps: int = 3, num_steps: int = 2, trace: str = "cuda,nvtx,osrt,cudnn,cublas",
                 gpu_metrics_device: str = "none", cuda_memory_usage: bool = True, capture_range: str = "cudaProfilerApi",
                 extra: str = "") -> str:
    """Nsight Systems wrapper in the shape of the reference's tuner preset (tuner/tuner.py:253-290): the capture is
    bounded by the profiler API range that the training loop opens after `warmup_steps` and closes `num_steps` later
    (config keys `nsys_warmup_steps` / `nsys_num_steps`)."""
    return (f"nsys profile -o {shlex.quote(output)}-%q{{SLURM_PROCID}} --trace={trace} --gpu-metrics-device={gpu_metrics_device} "
            f"--cuda-memory-usage={'true' if cuda_memory_usage else 'false'} --capture-range={capture_range} "
            f"--capture-range-end=stop --force-overwrite=true --sample=process-tree {extra}").strip()


def write_overrides(path: str, overrides: Dict[str, object]) -> str:
    """YAML file of configuration overrides, handed to launch.py with `--overrides` (it replaces values of the model / data
    files, which themselves may not set a key twice)."""
    import yaml
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w") as fh:
        yaml.safe_dump(overrides, fh, sort_keys=True)
    return path


def parse_override(kv: str):
    import yaml
    k, _, v = kv.partition("=")
    if not k or not _:
        raise ValueError(f"override {kv!r} is not KEY=VALUE")
    return k.strip(), yaml.safe_load(v)


def build_script(job_name: str, nodes: int, gpus_per_node: int, repo_dir: str, conf_dir: Optional[str], conf_files: List[str],
                 launcher: str = "torch", time_limit: str = "24:00:00", partition: Optional[str] = None,
                 account: Optional[str] = None, output_dir: str = "logs", env: Optional[Dict[str, str]] = None,
                 max_restarts: int = 0, numa_bind: bool = False, profile_cmd: Optional[str] = None, master_port: int = 29500,
                 singleton: bool = False, container: Optional[str] = None, python: str = "python",
                 overrides_file: Optional[str] = None) -> str:
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
    if overrides_file:
        conf += f" --overrides {shlex.quote(overrides_file)}"
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
    ap.add_argument("--override", action="append", default=[], metavar="KEY=VALUE", help="configuration override (repeatable)")
    ap.add_argument("--checkpoint-dir", default=None, help="run directory used as both `save` and `load` (self-resuming requeue)")
    ap.add_argument("--straggler-interval", type=int, default=0, help="report stragglers every N steps (0 = off)")
    ap.add_argument("--watchdog-timeout", type=float, default=0.0, help="per-step watchdog deadline in seconds (0 = off)")
    ap.add_argument("--nsys", action="store_true", help="wrap the workers in the Nsight Systems preset")
    ap.add_argument("--nsys-warmup-steps", type=int, default=3)
    ap.add_argument("--nsys-num-steps", type=int, default=2)
    ap.add_argument("--output", default=None)
    a = ap.parse_args(argv)
    env = dict(e.split("=", 1) for e in a.env)
    over = dict(parse_override(kv) for kv in a.override)
    if a.checkpoint_dir:
        over.update({"save": a.checkpoint_dir, "load": a.checkpoint_dir})
    if a.straggler_interval > 0:
        over.update({"heimdall_log_straggler": True, "heimdall_log_interval": a.straggler_interval})
    if a.watchdog_timeout > 0:
        over.update({"watchdog_step_timeout": a.watchdog_timeout,
                     "watchdog_heartbeat_dir": os.path.join(a.output_dir, f"heartbeat-{a.job_name}")})
    profile_cmd = a.profile_cmd
    if a.nsys:
        over.update({"nsys_warmup_steps": a.nsys_warmup_steps, "nsys_num_steps": a.nsys_num_steps})
        profile_cmd = nsys_command(os.path.join(a.output_dir, f"nsys-{a.job_name}"), a.nsys_warmup_steps, a.nsys_num_steps)
    overrides_file = None
    if over:
        overrides_file = f"overrides-{a.job_name}.yml"
        write_overrides(os.path.join(a.config_dir or ".", overrides_file), over)
    script = build_script(a.job_name, a.nodes, a.gpus_per_node, os.getcwd(), a.config_dir, a.conf_files, a.launcher, a.time,
                          a.partition, a.account, a.output_dir, env, a.max_restarts, a.numa_bind, profile_cmd,
                          singleton=a.singleton, container=a.container, overrides_file=overrides_file)
    if a.output:
        with open(a.output, "w") as fh:
            fh.write(script)
        print(f"wrote {a.output}")
    else:
        print(script)


if __name__ == "__main__":
    main()
