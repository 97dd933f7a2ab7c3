#!/usr/bin/env python
"""Launcher: `python launch.py train.py -d configs data/x.yml model/y.yml`.

Parses and validates the YAML files, then starts one worker per GPU of this node with
torch.distributed.run (the resolved configuration travels as base64 JSON in --megatron_config, the engine
sub-dictionary in --deepspeed_config).  Multi-node jobs use the SLURM generators under launcher/.
Same command line as the reference (launch.py:12-28, README.md:47-49).
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from savanna_b200.config import GlobalConfig  # noqa: E402


def build_command(cfg, nproc=None):
    args = cfg.get_deepspeed_main_args()
    script_idx = args.index(cfg.user_script)
    worker_args = args[script_idx + 1:]
    nproc = nproc or cfg.global_num_gpus
    rank_logs = []
    if cfg.enable_each_rank_log:
        # one stdout / stderr file per rank (and still on the terminal), under <log_dir or .>/rank_logs
        log_dir = os.path.join(cfg.log_dir or ".", "rank_logs")
        os.makedirs(log_dir, exist_ok=True)
        rank_logs = ["--log-dir", log_dir, "--redirects", "3", "--tee", "3"]
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
            "--master-addr", cfg.master_addr or "127.0.0.1", "--master-port", str(cfg.master_port)] + rank_logs + \
           [cfg.user_script] + worker_args


def main(argv=None):
    cfg = GlobalConfig.consume_deepy_args(argv)
    if cfg.use_wandb is not False and "WANDB_API_KEY" in os.environ:
        os.environ.setdefault("WANDB_API_KEY", os.environ["WANDB_API_KEY"])
    out = getattr(cfg, "_train_args_output", None)
    cmd = build_command(cfg)
    if out:
        with open(out, "w") as fh:
            fh.write(" ".join(cmd[cmd.index(cfg.user_script) + 1:]))
        return 0
    if cfg.global_num_gpus == 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", str(cfg.master_port))
        import runpy
        sys.argv = [cfg.user_script] + cmd[cmd.index(cfg.user_script) + 1:]
        runpy.run_path(cfg.user_script, run_name="__main__")
        return 0
    import subprocess
    return subprocess.call(cmd)


if __name__ == "__main__":
    sys.exit(main())
