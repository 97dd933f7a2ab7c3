"""Process groups of the parallel runtime.

Group families (reference: savanna/mpu/initialize.py:44-215): data, pipe, io, context (called the
"sequence parallel group" there), fp8-sync, model (tensor) and sequence-data (data x context ranks
that share a tensor-parallel index; the ZeRO partition group under context parallelism).

Every getter works without an initialised process group (sizes 1, ranks 0) so single-process CPU
runs need no rendezvous.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from .topology import ProcessTopology, build_topology

_G: Dict[str, object] = {}
_RANKS: Dict[str, List[int]] = {}
_TOPO: Optional[ProcessTopology] = None
_FP8_SYNC_IS_WORLD = True


def _is_dist() -> bool:
    return dist.is_available() and dist.is_initialized()


def initialize_model_parallel(model_parallel_size: int = 1, context_parallel_size: int = 1,
                              pipe_parallel_size: int = 1, topology: Optional[ProcessTopology] = None,
                              fp32_allreduce: bool = False) -> ProcessTopology:
    """Create all group families.  Every rank calls `new_group` for every group (collective call)."""
    global _TOPO, _FP8_SYNC_IS_WORLD
    destroy_model_parallel()
    world = dist.get_world_size() if _is_dist() else 1
    rank = dist.get_rank() if _is_dist() else 0
    pp = max(1, pipe_parallel_size)
    if pp > 1 and context_parallel_size > 1:
        raise ValueError("pipeline and context parallelism cannot be combined")
    topo = topology or build_topology(world, pp=pp, cp=context_parallel_size, tp=model_parallel_size)
    _TOPO = topo
    _G["fp32_allreduce"] = fp32_allreduce

    def make(name: str, lists: List[List[int]]):
        for ranks in lists:
            grp = dist.new_group(ranks) if _is_dist() and world > 1 else None
            if rank in ranks:
                _G[name] = grp
                _RANKS[name] = list(ranks)

    make("data", topo.get_axis_comm_lists("data"))
    make("pipe", topo.get_axis_comm_lists("pipe"))
    make("context", topo.get_axis_comm_lists("context"))
    make("model", topo.get_axis_comm_lists("model"))
    make("seq_data", topo.get_multi_axis_comm_lists(["data", "context"]))
    # io group: ranks that read data = model-rank 0 (and context-rank 0) of the first and last pipe stage
    io_ranks = sorted(set(topo.filter_match(pipe=0, model=0) + topo.filter_match(pipe=pp - 1, model=0)))
    make("io", [io_ranks])
    if pp > 1:
        make("fp8_sync", [topo.filter_match(pipe=s) for s in range(pp)])
        _FP8_SYNC_IS_WORLD = False
    else:
        _FP8_SYNC_IS_WORLD = True
        _RANKS["fp8_sync"] = list(range(world))
        _G["fp8_sync"] = None
    for name in ("data", "pipe", "context", "model", "seq_data"):
        _RANKS.setdefault(name, [rank])
        _G.setdefault(name, None)
    return topo


def model_parallel_is_initialized() -> bool:
    return _TOPO is not None


def destroy_model_parallel() -> None:
    global _TOPO
    _G.clear()
    _RANKS.clear()
    _TOPO = None


def get_topology() -> Optional[ProcessTopology]:
    return _TOPO


def _group(name):
    return _G.get(name)


def _size(name) -> int:
    return len(_RANKS.get(name, [0]))


def _rank_in(name) -> int:
    ranks = _RANKS.get(name)
    if not ranks:
        return 0
    me = dist.get_rank() if _is_dist() else 0
    return ranks.index(me)


def get_model_parallel_group():
    return _group("model")


def get_model_parallel_world_size() -> int:
    return _size("model")


def get_model_parallel_rank() -> int:
    return _rank_in("model")


def get_model_parallel_src_rank() -> int:
    return _RANKS.get("model", [0])[0]


def get_data_parallel_group():
    return _group("data")


def get_data_parallel_world_size() -> int:
    return _size("data")


def get_data_parallel_rank() -> int:
    return _rank_in("data")


def get_data_parallel_src_rank() -> int:
    return _RANKS.get("data", [0])[0]


def get_context_parallel_group():
    return _group("context")


# the reference calls the context-parallel group "sequence parallel group" (mpu/initialize.py:140-154)
get_sequence_parallel_group = get_context_parallel_group


def get_context_parallel_world_size() -> int:
    return _size("context")


get_sequence_parallel_world_size = get_context_parallel_world_size


def get_context_parallel_rank() -> int:
    return _rank_in("context")


get_sequence_parallel_rank = get_context_parallel_rank


def get_context_parallel_ranks() -> List[int]:
    return list(_RANKS.get("context", [0]))


def get_context_parallel_src_rank() -> int:
    return _RANKS.get("context", [0])[0]


def get_sequence_data_parallel_group():
    return _group("seq_data")


def get_sequence_data_parallel_world_size() -> int:
    return _size("seq_data")


def get_sequence_data_parallel_rank() -> int:
    return _rank_in("seq_data")


def get_sequence_data_parallel_ranks() -> List[int]:
    return list(_RANKS.get("seq_data", [0]))


def get_pipe_parallel_group():
    return _group("pipe")


def get_pipe_parallel_world_size() -> int:
    return _size("pipe")


def get_pipe_parallel_rank() -> int:
    return _rank_in("pipe")


def get_pipe_parallel_ranks() -> List[int]:
    return list(_RANKS.get("pipe", [0]))


def get_io_parallel_group():
    return _group("io")


def is_io_rank() -> bool:
    me = dist.get_rank() if _is_dist() else 0
    return me in _RANKS.get("io", [0])


def get_fp8_sync_group():
    """None means "the whole world" (pipe size 1), as in the reference (mpu/initialize.py:156-168)."""
    return None if _FP8_SYNC_IS_WORLD else _group("fp8_sync")


def get_fp32_allreduce() -> bool:
    return bool(_G.get("fp32_allreduce", False))


def get_group_ranks(name: str) -> List[int]:
    return list(_RANKS.get(name, [0]))


def device() -> torch.device:
    return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")


def create_mics_groups(shard_size: int):
    """Split the sequence-data-parallel group into contiguous sub-groups of `shard_size` ranks (state is partitioned
    inside a sub-group) and the transposed replica groups (ranks holding the same shard).  Every rank calls this (the
    group constructors are collective).  Returns (shard group, shard ranks, replica group, replica ranks) of this rank."""
    ranks = get_sequence_data_parallel_ranks()
    n = len(ranks)
    if shard_size <= 0 or n % shard_size:
        raise ValueError(f"mics_shard_size {shard_size} does not divide the data-parallel size {n}")
    me = dist.get_rank() if _is_dist() else 0
    mine = None
    for s0 in range(0, n, shard_size):
        rs = ranks[s0:s0 + shard_size]
        g = dist.new_group(rs) if _is_dist() else None
        if me in rs:
            mine = (g, rs)
    rep = None
    for off in range(shard_size):
        rs = ranks[off::shard_size]
        g = dist.new_group(rs) if _is_dist() else None
        if me in rs:
            rep = (g, rs)
    return mine[0], mine[1], rep[0], rep[1]
