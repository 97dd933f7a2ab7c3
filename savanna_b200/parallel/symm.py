"""One door to PyTorch's symmetric-memory module (`torch.distributed._symmetric_memory`, a private API).

Every peer mapping and NVLink multicast address of the fused paths (ZeRO step, tensor-parallel projections, halo /
all-to-all / ring exchanges) comes from three calls of that module: `empty`, `rendezvous` and the handle's
`buffer_ptrs` (+ optional `multicast_ptr`).  `load()` checks that surface once and raises `SymmetricMemoryUnavailable`
with the PyTorch version in the message when it is missing, so that an upgrade of PyTorch that moves the API turns
into one clear line and the NCCL forms of all paths (which every caller keeps) instead of attribute errors in the
middle of a step.  Role of the reference's process-group bootstrap for NCCL (savanna/initialize.py:120-125); the
reference itself has no peer-memory layer.
"""
from __future__ import annotations

import importlib

import torch

_REQUIRED = ("empty", "rendezvous")
_MODULE = "torch.distributed._symmetric_memory"


class SymmetricMemoryUnavailable(RuntimeError):
    pass


def load(module_name: str = _MODULE):
    """The symmetric-memory module, after a check of the calls this framework uses."""
    try:
        mod = importlib.import_module(module_name)
    except Exception as exc:  # noqa: BLE001
        raise SymmetricMemoryUnavailable(
            f"PyTorch {torch.__version__} has no importable {module_name} ({exc}); the NCCL forms of the fused paths run") from exc
    missing = [name for name in _REQUIRED if not callable(getattr(mod, name, None))]
    if missing:
        raise SymmetricMemoryUnavailable(
            f"{module_name} of PyTorch {torch.__version__} lacks {', '.join(missing)}: the private API has moved; "
            "the NCCL forms of the fused paths run")
    return mod


def peer_pointers(handle, world: int):
    """Device addresses of every rank's copy of a symmetric buffer (checked: one per rank, none null)."""
    ptrs = getattr(handle, "buffer_ptrs", None)
    if ptrs is None or len(ptrs) != world or any(int(p) == 0 for p in ptrs):
        raise SymmetricMemoryUnavailable(
            f"symmetric-memory handle of PyTorch {torch.__version__} gives no usable buffer_ptrs for {world} ranks")
    return [int(p) for p in ptrs]


def multicast_pointer(handle) -> int:
    """NVLink multicast address of the buffer, 0 when the fabric (or this PyTorch) offers none."""
    return int(getattr(handle, "multicast_ptr", 0) or 0)
