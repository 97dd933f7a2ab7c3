"""Parallel runtime: topology, process groups, autograd collectives, tensor-parallel layers,
context-parallel algorithms and the ZeRO-1 optimizer."""
from . import state
from .state import *  # noqa: F401,F403  (group getters, reference-compatible names)
from .topology import ProcessTopology, build_topology
from .mappings import (copy_to_model_parallel_region, gather_from_model_parallel_region,
                       gather_from_sequence_parallel_region, reduce_from_model_parallel_region,
                       reduce_scatter_to_sequence_parallel_region, scatter_to_model_parallel_region,
                       scatter_to_sequence_parallel_region)
from .zigzag import (zigzag_split, zigzag_merge, zigzag_indices, zigzag_split_across_cp_ranks,
                     zigzag_gather_from_cp_ranks, inverse_zigzag_permutation)
from .data import broadcast_data
from .cross_entropy import vocab_parallel_cross_entropy
