"""Checks of the SLURM environment before the workers start, and the world description for launchers that want one.

Role of the reference's launcher/config_parser.py:12-100: the generated batch script calls `check_slurm_env` on the first
node so that a mis-sized allocation fails in seconds instead of at the first collective, and `world_info` encodes
{host: [gpu indices]} the way DeepSpeed-style launchers read it (base64 of JSON).

    python -m launcher.config_parser --hostfile hosts.txt          # prints MASTER_NODE, nodes, GPUs per node
"""
from __future__ import annotations

import argparse
import base64
import json
import os
from typing import Dict, List, Optional, Tuple


def read_hostfile(path: str) -> List[str]:
    return [ln.split()[0] for ln in open(path).read().splitlines() if ln.strip() and not ln.startswith("#")]


def check_slurm_env(hostfile: str, env: Optional[Dict[str, str]] = None) -> Tuple[str, int, int]:
    """Returns (master node, number of nodes, GPUs per node); raises with a precise message when the allocation and the
    hostfile disagree or a variable the launch needs is unset."""
    env = os.environ if env is None else env
    hosts = read_hostfile(hostfile)
    n = env.get("SLURM_JOB_NUM_NODES")
    if n is None:
        raise RuntimeError("SLURM_JOB_NUM_NODES is not set: not inside a SLURM allocation")
    if len(hosts) != int(n):
        raise RuntimeError(f"hostfile lists {len(hosts)} hosts but the allocation has {n} nodes: {hosts}")
    master = env.get("MASTER_NODE") or env.get("MASTER_ADDR")
    if master is None:
        raise RuntimeError("MASTER_NODE / MASTER_ADDR is not set")
    if master != hosts[0]:
        raise RuntimeError(f"the master node {master!r} is not the first host of the hostfile ({hosts[0]!r})")
    if env.get("MASTER_PORT") is None:
        raise RuntimeError("MASTER_PORT is not set")
    gpus = env.get("SLURM_GPUS_ON_NODE")
    if gpus is None:
        raise RuntimeError("SLURM_GPUS_ON_NODE is not set: request GPUs with --gpus-per-node")
    return master, int(n), int(gpus)


def world_info(hosts: List[str], gpus_per_node: int, save_path: Optional[str] = None) -> str:
    enc = base64.urlsafe_b64encode(json.dumps({h: list(range(gpus_per_node)) for h in hosts}).encode()).decode()
    if save_path:
        with open(save_path, "w") as fh:
            fh.write(enc)
    return enc


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--hostfile", required=True)
    ap.add_argument("--world-info-output", default=None)
    a = ap.parse_args(argv)
    master, nodes, gpus = check_slurm_env(a.hostfile)
    print(f"MASTER_NODE={master} NODES={nodes} GPUS_PER_NODE={gpus}")
    if a.world_info_output:
        world_info(read_hostfile(a.hostfile), gpus, a.world_info_output)


if __name__ == "__main__":
    main()
