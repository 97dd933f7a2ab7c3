"""Cartesian rank topology.

Ranks are laid out over the axes (pipe, data, context, model) with `model` varying fastest, then
context, then data, then pipe — the order the reference builds with DeepSpeed's ProcessTopology
(savanna/initialize.py:141-144).  On one NVSwitch box every axis has the same bandwidth, so the
order only matters for checkpoint file naming and for parity of data-parallel sample assignment.
"""
from __future__ import annotations

from itertools import product
from typing import Dict, List, Sequence


class ProcessTopology:
    def __init__(self, axes: Sequence[str], dims: Sequence[int]):
        if len(axes) != len(dims):
            raise ValueError("axes and dims differ in length")
        self.axes = list(axes)
        self.dims = [int(d) for d in dims]
        self._coord_of: List[Dict[str, int]] = []
        self._rank_of: Dict[tuple, int] = {}
        for rank, coord in enumerate(product(*[range(d) for d in self.dims])):
            self._coord_of.append(dict(zip(self.axes, coord)))
            self._rank_of[coord] = rank

    def world_size(self) -> int:
        n = 1
        for d in self.dims:
            n *= d
        return n

    def get_dim(self, axis: str) -> int:
        return self.dims[self.axes.index(axis)] if axis in self.axes else 1

    def get_coord(self, rank: int) -> Dict[str, int]:
        return dict(self._coord_of[rank])

    def get_rank(self, **coord) -> int:
        return self._rank_of[tuple(coord[a] for a in self.axes)]

    def get_axis_comm_lists(self, axis: str) -> List[List[int]]:
        """Rank lists of every group obtained by varying `axis` and fixing all other axes."""
        if axis not in self.axes:
            return []
        others = [a for a in self.axes if a != axis]
        lists = []
        for fixed in product(*[range(self.get_dim(a)) for a in others]):
            base = dict(zip(others, fixed))
            lists.append([self.get_rank(**{**base, axis: i}) for i in range(self.get_dim(axis))])
        return lists

    def get_multi_axis_comm_lists(self, axes: Sequence[str]) -> List[List[int]]:
        """Groups obtained by varying all of `axes` together (e.g. data x context for ZeRO)."""
        axes = [a for a in axes if a in self.axes]
        others = [a for a in self.axes if a not in axes]
        lists = []
        for fixed in product(*[range(self.get_dim(a)) for a in others]):
            base = dict(zip(others, fixed))
            ranks = []
            for var in product(*[range(self.get_dim(a)) for a in axes]):
                ranks.append(self.get_rank(**{**base, **dict(zip(axes, var))}))
            lists.append(sorted(ranks))
        return lists

    def filter_match(self, **coord) -> List[int]:
        return [r for r, c in enumerate(self._coord_of) if all(c[k] == v for k, v in coord.items())]

    def __repr__(self):
        return "ProcessTopology(" + ", ".join(f"{a}={d}" for a, d in zip(self.axes, self.dims)) + ")"


def build_topology(world_size: int, pp: int = 1, cp: int = 1, tp: int = 1) -> ProcessTopology:
    pp, cp, tp = max(1, pp), max(1, cp), max(1, tp)
    if world_size % (pp * cp * tp):
        raise ValueError(f"world size {world_size} is not divisible by pipe {pp} x context {cp} x model {tp}")
    dp = world_size // (pp * cp * tp)
    return ProcessTopology(["pipe", "data", "context", "model"], [pp, dp, cp, tp])
