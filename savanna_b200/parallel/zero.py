"""ZeRO stage-1 optimizer: flat low-precision parameters and gradients, fp32 master weights and Adam
moments partitioned over the data-parallel (x context-parallel) group.

Step = gradient reduce-scatter -> global-norm clip -> Adam on the owned shard -> parameter
all-gather.  Layout follows DeepSpeed's stage-1 so checkpoints carry the same objects
(`single_partition_of_fp32_groups`, one flat partition per parameter group; reference usage:
savanna/training.py:1329-1337 and the `zero_optimization` block of its configs):
each parameter group is flattened in parameter order, padded so that every rank owns an equal,
aligned slice, and rank i of the partition group owns slice i.

Two communication paths: "nccl" issues reduce_scatter_tensor / all_gather_into_tensor on the flat
buffers; "symm" runs the fused peer-memory kernels (parallel/fused_zero.py) when the buffers live in
a symmetric-memory workspace.  With one rank both degenerate to the fused Adam kernel alone.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from .. import ops
from . import state

ALIGN = 256  # elements; keeps every shard 512-byte aligned for vector loads and bulk copies


def _pad_to(n: int, m: int) -> int:
    return m * ((n + m - 1) // m)


def _file_tensor(path: str, numel: int) -> torch.Tensor:
    """fp32 tensor of `numel` elements whose storage is the file `path` (created or resized, shared mapping: writes go
    to the file)."""
    import os
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "ab") as fh:
        fh.truncate(numel * 4)
    return torch.from_file(path, shared=True, size=numel, dtype=torch.float32)


class FlatGroup:
    """One parameter group flattened into a parameter buffer and a gradient buffer."""

    def __init__(self, params: List[torch.nn.Parameter], world: int, rank: int, hyper: Dict, allocator=None,
                 offload: bool = False, nvme_prefix: Optional[str] = None):
        self.params = params
        self.offload = bool(offload)
        self.nvme_prefix = nvme_prefix
        self.hyper = hyper
        dtype, device = params[0].dtype, params[0].device
        if any(p.dtype != dtype for p in params):
            raise ValueError("all parameters of a group must share a dtype")
        self.numel = sum(p.numel() for p in params)
        self.padded = _pad_to(self.numel, ALIGN * world)
        self.shard = self.padded // world
        self.world, self.rank = world, rank
        alloc = allocator or (lambda n, dt: torch.zeros(n, dtype=dt, device=device))
        self.flat_param = alloc(self.padded, dtype)
        self.flat_grad = alloc(self.padded, dtype)
        self.offsets = []
        off = 0
        with torch.no_grad():
            for p in params:
                n = p.numel()
                view = self.flat_param[off:off + n].view(p.shape)
                view.copy_(p.data)
                p.data = view
                p.grad = self.flat_grad[off:off + n].view(p.shape)
                p._fuse_grad_accum = True           # GEMM epilogues may accumulate weight gradients in place
                self.offsets.append(off)
                off += n
        lo, hi = rank * self.shard, (rank + 1) * self.shard
        # fp32 parameters are their own master copy (the shard view is updated in place)
        self.master = self.flat_param[lo:hi] if dtype == torch.float32 else self.flat_param[lo:hi].float().clone()
        self.master_is_view = dtype == torch.float32
        if self.offload:
            # optimizer state in (pinned) host memory: the fp32 master copy of this rank's shard and both Adam moments;
            # the step copies the reduced gradient shard to the host, updates there and copies the shard back
            pin = device.type == "cuda"
            self.master = self.flat_param[lo:hi].float().cpu()
            if pin:
                self.master = self.master.pin_memory()
            self.master_is_view = False
            self.host_grad = torch.zeros(self.shard, dtype=torch.float32, pin_memory=pin)
            self.host_param = torch.zeros(self.shard, dtype=dtype, pin_memory=pin)
        if self.offload and nvme_prefix:
            # `offload_optimizer.device: nvme`: the three fp32 state arrays are files under `nvme_path`, mapped into
            # the address space; the CPU update walks them in place and the kernel's page cache moves the pages
            # between the drive and memory, so resident host memory is bounded by what the update touches at a time
            init = self.master
            self.master = _file_tensor(nvme_prefix + "_master.bin", self.shard)
            self.master.copy_(init)
            self.exp_avg = _file_tensor(nvme_prefix + "_exp_avg.bin", self.shard)
            self.exp_avg_sq = _file_tensor(nvme_prefix + "_exp_avg_sq.bin", self.shard)
            self.exp_avg.zero_()
            self.exp_avg_sq.zero_()
        else:
            self.exp_avg = torch.zeros_like(self.master)
            self.exp_avg_sq = torch.zeros_like(self.master)
        self.norm_weight: Optional[torch.Tensor] = None

    def shard_slice(self, t: torch.Tensor) -> torch.Tensor:
        return t[self.rank * self.shard:(self.rank + 1) * self.shard]

    def build_norm_weight(self, tp: int) -> None:
        """Per-element weight of the squared-norm sum on this shard: replicated (non tensor-parallel)
        parameters count once over the tensor-parallel group."""
        if tp == 1 or all(getattr(p, "model_parallel", False) for p in self.params):
            return
        w = torch.ones(self.padded, dtype=torch.float32, device=self.flat_param.device)
        for p, off in zip(self.params, self.offsets):
            if not getattr(p, "model_parallel", False):
                w[off:off + p.numel()] = 1.0 / tp
        self.norm_weight = self.shard_slice(w).clone()


class ZeroOptimizer:
    """Adam(W) with ZeRO-1 partitioning.  `param_groups` as for torch optimizers (dicts with `params`,
    optional `lr`, `weight_decay`, `name`)."""

    def __init__(self, param_groups: List[Dict], lr: float, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.0, adamw: bool = True, clip_grad: float = 0.0,
                 group=None, group_ranks: Optional[List[int]] = None, comm_path: str = "nccl",
                 grad_divisor: Optional[float] = None, partition: bool = True, allocator=None,
                 sum_ranks: Optional[int] = None, offload_optimizer: bool = False, nvme_path: Optional[str] = None):
        self.group = group
        self.nvme_path = nvme_path                 # with offload_optimizer: directory of the file-backed state arrays
        # ZeRO-Offload (`zero_optimization.offload_optimizer.device: cpu`): master weights and Adam moments live in
        # host memory and the update runs on the CPU; HBM then holds parameters, gradients and activations only
        self.offload_optimizer = bool(offload_optimizer)
        ranks = group_ranks or [0]
        self.world = len(ranks) if partition else 1
        me = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
        self.rank = ranks.index(me) if (partition and me in ranks) else 0
        self.reduce_world = len(ranks)
        # The reduction group is data x context parallel.  The loss of a context-parallel rank is its local
        # numerator over the GLOBAL token count (models/losses.py), so the ranks of one replica hold partial
        # gradients that must be SUMMED; only the data-parallel replicas are averaged (DeepSpeed divides by
        # dp_world / sequence_parallel_size for the same reason).
        self.sum_ranks = int(sum_ranks) if sum_ranks else state.get_context_parallel_world_size()
        if self.reduce_world % max(1, self.sum_ranks) != 0:
            self.sum_ranks = 1
        self.partition = partition
        self.betas, self.eps, self.adamw = betas, eps, adamw
        self.clip_grad = clip_grad or 0.0
        self.comm_path = comm_path
        self.step_count = 0
        self.defaults = {"lr": lr, "weight_decay": weight_decay}
        self.groups: List[FlatGroup] = []
        self.param_groups: List[Dict] = []
        tp = state.get_model_parallel_world_size()
        for g in param_groups:
            params = [p for p in g["params"] if p.requires_grad]
            if not params:
                continue
            hyper = {"lr": g.get("lr", lr), "weight_decay": g.get("weight_decay", weight_decay),
                     "name": g.get("name", f"group{len(self.param_groups)}"), "lr_mult": g.get("lr", lr) / lr if lr else 1.0,
                     "fixed_lr": "lr" in g}
            self.param_groups.append(hyper)         # lr schedulers write `lr` here
            # one flat buffer per dtype (low-precision weights and fp32 filter parameters share hyper-parameters)
            by_dtype: Dict[torch.dtype, List] = {}
            for q in params:
                by_dtype.setdefault(q.dtype, []).append(q)
            for dt, plist in by_dtype.items():
                prefix = None
                if self.offload_optimizer and nvme_path:
                    import os
                    prefix = os.path.join(nvme_path, f"zero_state_rank{me}_buf{len(self.groups)}")
                fg = FlatGroup(plist, self.world, self.rank, hyper, allocator, offload=self.offload_optimizer,
                               nvme_prefix=prefix)
                fg.hyper = hyper                    # shared object: both flats follow the schedule
                fg.build_norm_weight(tp)
                self.groups.append(fg)
        self.grad_divisor = grad_divisor
        self.last_grad_norm: Optional[torch.Tensor] = None
        self.loss_scaler = None                    # train/loss_scaler.py scaler for fp16 runs (set by the trainer)
        self.overflow = False                      # the last step found inf / nan gradients and was skipped
        self.fused = None                          # set by parallel.fused_zero.attach() on CUDA with symmetric memory

    # ------------------------------------------------------------------ gradients
    def zero_grad(self, set_to_none: bool = False) -> None:
        for g in self.groups:
            g.flat_grad.zero_()

    def _reduce_scatter(self, g: FlatGroup) -> torch.Tensor:
        """Average gradients over the partition group; returns this rank's gradient shard."""
        shard = g.shard_slice(g.flat_grad)
        if self.reduce_world == 1:
            return shard
        if not self.partition:
            dist.all_reduce(g.flat_grad, group=self.group)
            g.flat_grad.mul_(self.grad_scale())
            return g.flat_grad
        backend = dist.get_backend(self.group)
        if backend == "gloo":
            dist.all_reduce(g.flat_grad, group=self.group)
        else:
            dist.reduce_scatter_tensor(shard, g.flat_grad, group=self.group)
        return shard

    def grad_scale(self) -> float:
        """Factor that turns the SUM over the reduction group into the step's gradient: mean over the
        data-parallel replicas, sum over the context-parallel ranks of a replica."""
        return float(self.sum_ranks) / float(self.reduce_world)

    def _all_gather(self, g: FlatGroup) -> None:
        if self.world == 1:
            return
        shard = g.shard_slice(g.flat_param)
        backend = dist.get_backend(self.group)
        if backend == "gloo":
            parts = [torch.empty_like(shard) for _ in range(self.world)]
            dist.all_gather(parts, shard.clone(), group=self.group)
            g.flat_param.copy_(torch.cat(parts))
        else:
            dist.all_gather_into_tensor(g.flat_param, shard, group=self.group)

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self) -> torch.Tensor:
        """Runs one optimizer step; returns the global gradient norm (0-dim fp32 tensor, on device)."""
        if self.groups and self.groups[0].flat_param.is_cuda:
            from ..ops import cuda_ops
            cuda_ops.bump_param_epoch()             # cached fp8 copies of the weights are stale after this step
        if self.fused is not None:
            return self.fused.step(self)
        self.step_count += 1
        shards = [self._reduce_scatter(g) for g in self.groups]
        inv = self.grad_scale() if (self.reduce_world > 1 and self.partition) else 1.0
        if self.grad_divisor:
            inv = inv / self.grad_divisor
        scaler = self.loss_scaler
        if scaler is not None:
            inv = inv / scaler.scale                # the backward ran on loss * scale (fp16 training)
        sq = None
        for g, s in zip(self.groups, shards):
            part = ops.sq_norm(s, g.norm_weight)
            sq = part if sq is None else sq + part
        sq = sq * (inv * inv)
        if self.world > 1:
            dist.all_reduce(sq, group=self.group)
        tp = state.get_model_parallel_world_size()
        if tp > 1:
            dist.all_reduce(sq, group=state.get_model_parallel_group())
        if state.get_pipe_parallel_world_size() > 1:
            dist.all_reduce(sq, group=state.get_pipe_parallel_group())
        norm = sq.sqrt()
        self.last_grad_norm = norm
        if scaler is not None:
            # every rank holds the same reduced norm, so every rank takes the same branch
            self.overflow = scaler.check(norm)
            if self.overflow:
                self.step_count -= 1                # inf / nan in the gradients: no update, the scaler has backed off
                return norm
        if self.clip_grad > 0.0:
            coef = torch.clamp(self.clip_grad / (norm + 1e-6), max=1.0) * inv
        else:
            coef = torch.full_like(norm, inv)
        b1, b2 = self.betas
        if self.offload_optimizer:
            from ..ops import reference as ref
            coef_host = float(coef)                 # one synchronisation per step: the clip coefficient
            for g, s in zip(self.groups, shards):
                own = s if s.numel() == g.shard else g.shard_slice(s)
                g.host_grad.copy_(own, non_blocking=True)
            if self.groups and self.groups[0].flat_param.is_cuda:
                torch.cuda.current_stream().synchronize()
            for g in self.groups:
                ref.adam_step(g.master, g.exp_avg, g.exp_avg_sq, g.host_grad, g.hyper["lr"], b1, b2, self.eps,
                              g.hyper["weight_decay"], self.step_count, self.adamw, coef_host, None)
                g.host_param.copy_(g.master)
                g.shard_slice(g.flat_param).copy_(g.host_param, non_blocking=True)
                self._all_gather(g)
            return norm
        for g, s in zip(self.groups, shards):
            ops.adam_step(g.master, g.exp_avg, g.exp_avg_sq, s, g.hyper["lr"], b1, b2, self.eps,
                          g.hyper["weight_decay"], self.step_count, self.adamw, coef,
                          None if g.master_is_view else g.shard_slice(g.flat_param))
            self._all_gather(g)
        return norm

    # ------------------------------------------------------------------ state
    def state_dict(self) -> Dict:
        """DeepSpeed stage-1 shaped state."""
        base_state = {}
        for i, g in enumerate(self.groups):
            base_state[i] = {"step": self.step_count, "exp_avg": g.exp_avg, "exp_avg_sq": g.exp_avg_sq}
        return {
            "zero_stage": 1,
            "partition_count": [self.world] * len(self.groups),
            "loss_scaler": self.loss_scaler.state_dict() if self.loss_scaler is not None else None,
            "dynamic_loss_scale": bool(self.loss_scaler is not None and self.loss_scaler.dynamic),
            "overflow": bool(self.overflow),
            "clip_grad": self.clip_grad,
            "single_partition_of_fp32_groups": [g.master for g in self.groups],
            "group_paddings": [g.padded - g.numel if self.rank == self.world - 1 else 0 for g in self.groups],
            "base_optimizer_state": {
                "state": base_state,
                "param_groups": [{"lr": g.hyper["lr"], "betas": list(self.betas), "eps": self.eps,
                                  "weight_decay": g.hyper["weight_decay"], "name": g.hyper["name"],
                                  "params": [i]} for i, g in enumerate(self.groups)],
            },
        }

    def load_state_dict(self, sd: Dict, load_master: bool = True) -> None:
        masters = sd["single_partition_of_fp32_groups"]
        if len(masters) != len(self.groups):
            raise ValueError("optimizer state has a different number of parameter groups")
        st = sd["base_optimizer_state"]["state"]
        for i, g in enumerate(self.groups):
            if masters[i].numel() != g.master.numel():
                raise ValueError(f"optimizer partition size mismatch in group {i}: checkpoint was written with a "
                                 "different partition count; reshard it with tools/reshard_zero.py")
            if load_master:
                g.master.copy_(masters[i])
            g.exp_avg.copy_(st[i]["exp_avg"])
            g.exp_avg_sq.copy_(st[i]["exp_avg_sq"])
            self.step_count = int(st[i]["step"])
            pg = sd["base_optimizer_state"]["param_groups"][i]
            g.hyper["lr"] = pg["lr"]
        if self.loss_scaler is not None and isinstance(sd.get("loss_scaler"), dict):
            self.loss_scaler.load_state_dict(sd["loss_scaler"])

    def refresh_master_from_params(self) -> None:
        for g in self.groups:
            if not g.master_is_view:
                g.master.copy_(g.shard_slice(g.flat_param))

    def sync_params_from_master(self) -> None:
        for g in self.groups:
            if not g.master_is_view:
                g.shard_slice(g.flat_param).copy_(g.master)
            self._all_gather(g)
