"""Broadcast of a batch from the data-reading rank to its tensor- and context-parallel peers
(reference: savanna/mpu/data.py:37-120): sizes first, then one flattened payload."""
from __future__ import annotations

from typing import Dict, List

import torch
import torch.distributed as dist

from . import state

_MAX_DIM = 4


def _bcast(t, src, group):
    dist.broadcast(t, src, group=group)


def broadcast_data(keys: List[str], data: Dict[str, torch.Tensor], dtype: torch.dtype) -> Dict[str, torch.Tensor]:
    tp, cp = state.get_model_parallel_world_size(), state.get_context_parallel_world_size()
    if tp == 1 and cp == 1:
        dev = state.device()
        return {k: data[k].to(dev, non_blocking=True) for k in keys}
    dev = state.device()
    out = None
    for group, src, size in ((state.get_model_parallel_group(), state.get_model_parallel_src_rank(), tp),
                             (state.get_context_parallel_group(), state.get_context_parallel_src_rank(), cp)):
        if size == 1:
            continue
        have = out is not None or (data is not None and all(k in data for k in keys) and dist.get_rank() == src)
        src_dict = out if out is not None else data
        sizes = torch.zeros(len(keys) * _MAX_DIM, dtype=torch.int64, device=dev)
        if dist.get_rank() == src:
            if not have:
                raise RuntimeError("broadcast source rank has no data")
            for i, k in enumerate(keys):
                if src_dict[k].dim() > _MAX_DIM:
                    raise ValueError("broadcast_data supports at most 4 dims")
                for j, s in enumerate(src_dict[k].shape):
                    sizes[i * _MAX_DIM + j] = s
        _bcast(sizes, src, group)
        shapes = []
        for i in range(len(keys)):
            shp = [int(s) for s in sizes[i * _MAX_DIM:(i + 1) * _MAX_DIM].tolist() if s > 0]
            shapes.append(shp)
        numels = [int(torch.tensor(s).prod()) if s else 0 for s in shapes]
        if dist.get_rank() == src:
            flat = torch.cat([src_dict[k].to(dev, dtype).reshape(-1) for k in keys])
        else:
            flat = torch.empty(sum(numels), dtype=dtype, device=dev)
        _bcast(flat, src, group)
        out, off = {}, 0
        for k, shp, n in zip(keys, shapes, numels):
            out[k] = flat[off:off + n].view(shp)
            off += n
    return out
