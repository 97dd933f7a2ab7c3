"""ZeRO stages 2 and 3: gradient (stage 2) and parameter (stage 3) partitioning on top of the stage-1 state layout.

The reference passes its `zero_optimization` block to DeepSpeed; its 40B pre-training configs run stage 3 with
`deepspeed.zero.Init` over the sequence-data-parallel group (savanna/training.py:1243-1314,
configs/40b/40b_train.yml `zero_optimization.stage: 3`).  What the stages mean here:

* the model is cut into UNITS: one per backbone block, plus a root unit (embedding, final norm, head).  Every unit's
  parameters of one optimizer group and dtype live in one flat buffer, padded so that each rank of the partition group
  owns an equal aligned slice, exactly like the stage-1 groups (parallel/zero.py);
* every rank permanently holds only its slice of a unit: low-precision parameter shard, fp32 master, Adam moments and an
  fp32 gradient accumulator;
* stage 3: a unit's full parameter buffer exists only while the unit runs.  A forward pre-hook all-gathers it (the next
  unit's all-gather is issued asynchronously at the same time, so it overlaps this unit's compute), a post-hook frees
  it; a hook on the unit's output gradient gathers it again before the unit's backward, with the previous unit
  prefetched.  The buffer is freed by shrinking its storage to zero bytes and re-grown in place, so every view taken of
  it (the module's parameters, tensors saved for backward) stays valid across the cycle;
* stages 2 and 3: a unit's full gradient buffer exists only during the unit's backward.  When the backward reaches the
  next unit, the finished unit's gradients are reduce-scattered (asynchronously) and added to the owners' fp32
  accumulators, and the buffer is freed.  Micro-batches accumulate in the partitioned fp32 form;
* the optimizer step touches shards only: global-norm clip over all shards, Adam on the fp32 masters, low-precision
  shard written by the same kernel.  Stage 2 all-gathers the parameters afterwards; stage 3 leaves that to the next
  forward.

The root unit is small (byte-level vocabulary) and is used at both ends of the model (tied embedding), so it stays
resident and is handled like a stage-1 group.
"""
from __future__ import annotations

import contextlib
import os
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from .. import ops
from . import state
from .zero import ALIGN, _pad_to


def _all_gather(full: torch.Tensor, shard: torch.Tensor, group, world: int, async_op: bool = False):
    if world == 1:
        full[:shard.numel()].copy_(shard)
        return None
    if dist.get_backend(group) == "gloo":
        parts = [torch.empty_like(shard) for _ in range(world)]
        dist.all_gather(parts, shard.clone(), group=group)
        full.copy_(torch.cat(parts))
        return None
    return dist.all_gather_into_tensor(full, shard, group=group, async_op=async_op)


class UnitFlat:
    """The parameters of one unit that share an optimizer group and a dtype, flattened and partitioned."""

    def __init__(self, params: List[torch.nn.Parameter], world: int, rank: int, hyper: Dict, name: str,
                 free_params: bool, free_grads: bool, tp: int, offload_param: bool = False,
                 offload_optimizer: bool = False, nvme_prefix: Optional[str] = None):
        self.params, self.hyper, self.name = params, hyper, name
        self.world, self.rank = world, rank
        self.free_params, self.free_grads = free_params, free_grads
        dtype, device = params[0].dtype, params[0].device
        self.numel = sum(p.numel() for p in params)
        self.padded = _pad_to(self.numel, ALIGN * world)
        self.shard = self.padded // world
        self.full = torch.zeros(self.padded, dtype=dtype, device=device)
        self.gfull = torch.zeros(self.padded, dtype=dtype, device=device)
        self.nbytes = self.full.untyped_storage().size()
        self.offsets: List[int] = []
        off = 0
        with torch.no_grad():
            for p in params:
                n = p.numel()
                view = self.full[off:off + n].view(p.shape)
                view.copy_(p.data)
                p.data = view
                p.grad = self.gfull[off:off + n].view(p.shape)
                p._fuse_grad_accum = True
                self.offsets.append(off)
                off += n
        lo, hi = rank * self.shard, (rank + 1) * self.shard
        self.param_shard = self.full[lo:hi].clone()
        self.master_is_view = dtype == torch.float32          # fp32 parameters are their own master copy
        self.master = self.param_shard if self.master_is_view else self.param_shard.float()
        # `offload_param`: between uses the low-precision shard of a unit whose whole parameters are released lives in
        # (pinned) host memory; gathers stage it to the device, the optimizer step writes it back
        self.param_offloaded = bool(offload_param) and free_params and not self.master_is_view
        if self.param_offloaded:
            host = self.param_shard.cpu()
            self.param_shard = host.pin_memory() if device.type == "cuda" else host
        # `offload_optimizer`: fp32 master copy and Adam moments of this rank's shard live in (pinned) host memory and the
        # update runs on the CPU; the reduced gradient shard is copied down, the new low-precision shard copied up
        self.optimizer_offloaded = bool(offload_optimizer)
        self.host_grad = None
        if self.optimizer_offloaded:
            pin = device.type == "cuda"
            host = self.master.detach().float().cpu().clone()
            self.master = host.pin_memory() if pin else host
            self.master_is_view = False
            self.host_grad = torch.zeros(self.shard, dtype=torch.float32, pin_memory=pin)
        if self.optimizer_offloaded and nvme_prefix:
            # `device: nvme`: the three state arrays are mapped files under `nvme_path` (see parallel/zero.py)
            from .zero import _file_tensor
            init = self.master
            self.master = _file_tensor(nvme_prefix + "_master.bin", self.shard)
            self.master.copy_(init)
            self.exp_avg = _file_tensor(nvme_prefix + "_exp_avg.bin", self.shard).zero_()
            self.exp_avg_sq = _file_tensor(nvme_prefix + "_exp_avg_sq.bin", self.shard).zero_()
        else:
            self.exp_avg = torch.zeros_like(self.master)
            self.exp_avg_sq = torch.zeros_like(self.master)
        self.grad_acc = torch.zeros(self.shard, dtype=torch.float32, device=device)
        self.norm_weight: Optional[torch.Tensor] = None
        if tp > 1 and not all(getattr(p, "model_parallel", False) for p in params):
            w = torch.ones(self.padded, dtype=torch.float32, device=device)
            for p, o in zip(params, self.offsets):
                if not getattr(p, "model_parallel", False):
                    w[o:o + p.numel()] = 1.0 / tp
            self.norm_weight = w[lo:hi].clone()
        self.replicated = [(o, p.numel()) for p, o in zip(params, self.offsets) if not getattr(p, "model_parallel", False)]
        self.resident = True
        self.grads_live = True
        self.gather_work = None
        # hpZ: a secondary copy of the parameters partitioned over a small sub-group (see the optimizer)
        self.hpz_world, self.hpz_rank, self.hpz_group = 1, 0, None
        self.hpz_shard: Optional[torch.Tensor] = None
        self.hpz_fresh = False
        self.hpz_gathers = 0

    def shard_slice(self, t: torch.Tensor) -> torch.Tensor:
        return t[self.rank * self.shard:(self.rank + 1) * self.shard]

    def shard_on_device(self) -> torch.Tensor:
        """This rank's parameter shard as a device tensor (a staged copy when the shard is kept on the host)."""
        if self.param_offloaded:
            return self.param_shard.to(self.full.device, non_blocking=True)
        return self.param_shard

    # -- parameters ----------------------------------------------------------------
    def start_gather(self, group, async_op: bool, secondary: bool = False) -> None:
        """`secondary`: gather from the hpZ copy over the sub-group when it is up to date (the backward pass)."""
        if self.resident or self.gather_work is not None:
            return
        self.full.untyped_storage().resize_(self.nbytes)
        if secondary and self.hpz_world > 1 and self.hpz_fresh:
            self.hpz_gathers += 1
            self.gather_work = _all_gather(self.full, self.hpz_shard, self.hpz_group, self.hpz_world, async_op) or True
        else:
            self.gather_work = _all_gather(self.full, self.shard_on_device(), group, self.world, async_op) or True

    def keep_secondary(self) -> None:
        """Before the whole parameters are released after the forward pass: keep this rank's 1 / hpz_world slice."""
        if self.hpz_world <= 1 or self.hpz_fresh or not self.resident or not self.free_params:
            return
        n = self.padded // self.hpz_world
        if self.hpz_shard is None:
            self.hpz_shard = torch.empty(n, dtype=self.full.dtype, device=self.full.device)
        self.hpz_shard.copy_(self.full[self.hpz_rank * n:(self.hpz_rank + 1) * n])
        self.hpz_fresh = True

    def wait_gather(self) -> None:
        if self.gather_work is not None:
            if self.gather_work is not True:
                self.gather_work.wait()
            self.gather_work = None
            self.resident = True

    def release_params(self) -> None:
        if not self.free_params or not self.resident:
            return
        self.full.untyped_storage().resize_(0)
        self.resident = False
        for p in self.params:                                  # quantised copies of the weights go with them
            if getattr(p, "_fp8_cache", None) is not None:
                p._fp8_cache = None
            if getattr(p, "_mx_cache", None) is not None:
                p._mx_cache = None

    # -- gradients -----------------------------------------------------------------
    def alloc_grads(self) -> None:
        if self.grads_live:
            return
        self.gfull.untyped_storage().resize_(self.nbytes)
        self.gfull.zero_()
        self.grads_live = True

    def free_grad_buffer(self) -> None:
        if self.free_grads and self.grads_live:
            self.gfull.untyped_storage().resize_(0)
            self.grads_live = False


class Unit:
    def __init__(self, name: str, module: Optional[torch.nn.Module], index: int):
        self.name, self.module, self.index = name, module, index
        self.flats: List[UnitFlat] = []
        self.in_backward = False


class PartitionedZeroOptimizer:
    """Adam(W) with ZeRO stage 2 or 3 partitioning.  Same surface as `ZeroOptimizer` (param_groups for the schedulers,
    zero_grad / step / state_dict / load_state_dict, `groups` of flat buffers) plus `finish_backward()`, which the
    training step calls after every backward pass, and `full_params()`, a context in which every parameter is whole
    (checkpoint save / load, export, evaluation code that walks the parameters)."""

    def __init__(self, param_groups: List[Dict], unit_modules: Sequence[torch.nn.Module], stage: int, lr: float,
                 betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0, adamw: bool = True,
                 clip_grad: float = 0.0, group=None, group_ranks: Optional[List[int]] = None,
                 grad_divisor: Optional[float] = None, sync_replicated: bool = False, prefetch: bool = True,
                 sum_ranks: Optional[int] = None, replica_group=None, replica_world: int = 1, replica_index: int = 0,
                 hpz_group=None, hpz_ranks: Optional[List[int]] = None, offload_param: bool = False,
                 offload_optimizer: bool = False, nvme_path: Optional[str] = None):
        if stage not in (2, 3):
            raise ValueError("PartitionedZeroOptimizer implements ZeRO stages 2 and 3")
        self.offload_optimizer = bool(offload_optimizer)
        self.stage = stage
        self.group = group
        ranks = group_ranks or [0]
        self.world = len(ranks)
        me = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
        self.rank = ranks.index(me) if me in ranks else 0
        # MiCS-style sharding (`zero_use_mics` + `mics_shard_size`): states are partitioned over a sub-group of the
        # replicas (`group`, e.g. the GPUs of one node) and replicated across `replica_group` (the ranks that hold the
        # same shard in the other sub-groups); a shard's gradient is reduce-scattered inside the sub-group and then
        # all-reduced over the replica group, parameters are gathered inside the sub-group only.
        self.replica_group, self.replica_world, self.replica_index = replica_group, max(1, replica_world), replica_index
        self.reduce_world = self.world * self.replica_world
        # context-parallel ranks hold partial gradients of one replica (summed); replicas are averaged
        self.sum_ranks = int(sum_ranks) if sum_ranks else state.get_context_parallel_world_size()
        if self.reduce_world % max(1, self.sum_ranks) != 0:
            self.sum_ranks = 1
        self.betas, self.eps, self.adamw = betas, eps, adamw
        self.clip_grad = clip_grad or 0.0
        self.grad_divisor = grad_divisor
        self.sync_replicated = sync_replicated
        self.prefetch = prefetch
        self.step_count = 0
        self.defaults = {"lr": lr, "weight_decay": weight_decay}
        self.loss_scaler = None                    # train/loss_scaler.py scaler for fp16 runs (set by the trainer)
        self.overflow = False
        self.fused = None
        self.last_grad_norm: Optional[torch.Tensor] = None
        tp = state.get_model_parallel_world_size()

        owner: Dict[int, int] = {}
        self.units: List[Unit] = [Unit("root", None, 0)]
        for i, m in enumerate(unit_modules):
            self.units.append(Unit(f"unit{i}", m, i + 1))
            for p in m.parameters():
                owner.setdefault(id(p), i + 1)
        self.param_groups: List[Dict] = []
        self.groups: List[UnitFlat] = []
        for g in param_groups:
            params = [p for p in g["params"] if p.requires_grad]
            if not params:
                continue
            hyper = {"lr": g.get("lr", lr), "weight_decay": g.get("weight_decay", weight_decay),
                     "name": g.get("name", f"group{len(self.param_groups)}"),
                     "lr_mult": g.get("lr", lr) / lr if lr else 1.0, "fixed_lr": "lr" in g}
            self.param_groups.append(hyper)
            buckets: Dict = {}
            for p in params:
                buckets.setdefault((owner.get(id(p), 0), p.dtype), []).append(p)
            for (ui, dt), plist in sorted(buckets.items(), key=lambda kv: (kv[0][0], str(kv[0][1]))):
                unit = self.units[ui]
                root = ui == 0
                f = UnitFlat(plist, self.world, self.rank, hyper, f"{unit.name}.{hyper['name']}.{dt}",
                             free_params=(stage == 3 and not root), free_grads=not root, tp=tp,
                             offload_param=offload_param, offload_optimizer=offload_optimizer,
                             nvme_prefix=(os.path.join(nvme_path, f"zero_state_rank{me}_buf{len(self.groups)}")
                                          if (offload_optimizer and nvme_path) else None))
                unit.flats.append(f)
                self.groups.append(f)
        # hpZ (`zero_hpz_partition_size`, stage 3): after a unit's forward all-gather over the whole group, every rank keeps
        # its 1 / hpz slice of the whole parameters, partitioned over a small sub-group (the GPUs of one node); the
        # backward (and recomputation) gathers then run inside the sub-group only.  Costs padded / hpz elements per rank
        # and unit; the copies go stale when the optimizer updates the parameters.
        self.hpz_world = len(hpz_ranks) if (hpz_ranks and stage == 3) else 1
        if self.hpz_world > 1:
            if self.world % self.hpz_world:
                raise ValueError(f"zero_hpz_partition_size {self.hpz_world} does not divide the partition group size {self.world}")
            for f in self.groups:
                f.hpz_world, f.hpz_rank, f.hpz_group = self.hpz_world, hpz_ranks.index(me), hpz_group
        self.backward_phase = False
        self.pending: List = []                     # (work, flat, shard view) reductions in flight
        self._handles = []
        for u in self.units[1:]:
            self._handles.append(u.module.register_forward_pre_hook(self._make_pre_forward(u)))
            self._handles.append(u.module.register_forward_hook(self._make_post_forward(u)))
        for u in self.units[1:]:
            for f in u.flats:
                f.free_grad_buffer()
                f.release_params()

    # ------------------------------------------------------------------ hooks
    def _async(self) -> bool:
        return self.prefetch and self.world > 1 and dist.get_backend(self.group) != "gloo"

    def _ensure_resident(self, u: Unit) -> None:
        for f in u.flats:
            f.start_gather(self.group, False, secondary=self.backward_phase)
        for f in u.flats:
            f.wait_gather()

    def _prefetch(self, idx: int) -> None:
        if self.stage != 3 or not self._async() or idx < 1 or idx >= len(self.units):
            return
        for f in self.units[idx].flats:
            f.start_gather(self.group, True, secondary=self.backward_phase)

    def _make_pre_forward(self, u: Unit):
        def hook(module, args):
            if self.stage == 3:
                self._ensure_resident(u)
                # the neighbour that runs next: the following unit in the forward pass, the preceding one when this
                # forward is a recomputation inside the backward pass
                self._prefetch(u.index - 1 if self.backward_phase else u.index + 1)
        return hook

    def _make_post_forward(self, u: Unit):
        def hook(module, args, output):
            if self.backward_phase:
                return None                          # recomputation: the unit's backward follows, keep it whole
            if torch.is_grad_enabled():
                outs = output if isinstance(output, (tuple, list)) else (output,)
                for o in outs:
                    if isinstance(o, torch.Tensor) and o.requires_grad:
                        o.register_hook(self._make_pre_backward(u))
                        break
            for f in u.flats:
                f.keep_secondary()
                f.release_params()
            return None
        return hook

    def _make_pre_backward(self, u: Unit):
        def hook(grad):
            self.backward_phase = True
            for other in self.units[1:]:
                if other.in_backward and other is not u:
                    self._finish_unit(other)
            self._drain(keep=1)
            if not u.in_backward:
                u.in_backward = True
                if self.stage == 3:
                    self._ensure_resident(u)
                    self._prefetch(u.index - 1)
                for f in u.flats:
                    f.alloc_grads()
            return None
        return hook

    def _sync_replicated(self, f: UnitFlat) -> None:
        """Sequence parallelism: parameters replicated over the tensor-parallel group see one sequence slice per rank;
        their gradients are summed over that group before the data-parallel reduction."""
        if not self.sync_replicated or not f.replicated or state.get_model_parallel_world_size() == 1:
            return
        flat = torch.cat([f.gfull[o:o + n] for o, n in f.replicated])
        dist.all_reduce(flat, group=state.get_model_parallel_group())
        off = 0
        for o, n in f.replicated:
            f.gfull[o:o + n].copy_(flat[off:off + n])
            off += n

    def _finish_unit(self, u: Unit) -> None:
        """The unit's backward is complete: start the reduction of its gradients, free its parameters."""
        for f in u.flats:
            if not f.grads_live:
                continue
            self._sync_replicated(f)
            self._start_reduce(f)
        for f in u.flats:
            f.release_params()
        u.in_backward = False

    def _start_reduce(self, f: UnitFlat) -> None:
        shard = f.shard_slice(f.gfull)
        work = None
        if self.world > 1:
            if dist.get_backend(self.group) == "gloo":
                dist.all_reduce(f.gfull, group=self.group)
            else:
                work = dist.reduce_scatter_tensor(shard, f.gfull, group=self.group, async_op=self._async())
        self.pending.append((work, f, shard))

    def _drain(self, keep: int = 0) -> None:
        """Complete reductions in flight (all but the newest `keep`): add the reduced shard to the fp32 accumulator
        and free the unit's gradient buffer."""
        while len(self.pending) > keep:
            work, f, shard = self.pending.pop(0)
            if work is not None:
                work.wait()
            if self.replica_world > 1:
                dist.all_reduce(shard, group=self.replica_group)      # the same shard of the other sub-groups
            f.grad_acc.add_(shard)
            if f.free_grads:
                f.free_grad_buffer()
            else:
                f.gfull.zero_()

    def finish_backward(self) -> None:
        """Called after each backward pass: reduce what is left, free the blocks' buffers."""
        for u in self.units[1:]:
            if u.in_backward:
                self._finish_unit(u)
        self._drain(0)
        for u in self.units[1:]:
            for f in u.flats:
                f.wait_gather()
                f.release_params()
        self.backward_phase = False

    # ------------------------------------------------------------------ gradients / step
    def zero_grad(self, set_to_none: bool = False) -> None:
        for f in self.groups:
            f.grad_acc.zero_()
            if f.grads_live:
                f.gfull.zero_()

    @torch.no_grad()
    def step(self) -> torch.Tensor:
        if self.groups and self.groups[0].master.is_cuda:
            from ..ops import cuda_ops
            cuda_ops.bump_param_epoch()
        self.finish_backward()
        for f in self.units[0].flats:               # the resident root unit reduces once per step
            self._sync_replicated(f)
            self._start_reduce(f)
        self._drain(0)
        self.step_count += 1
        inv = float(self.sum_ranks) / float(self.reduce_world)
        if self.grad_divisor:
            inv = inv / self.grad_divisor
        scaler = self.loss_scaler
        if scaler is not None:
            inv = inv / scaler.scale                # the backward ran on loss * scale (fp16 training)
        sq = None
        for f in self.groups:
            part = ops.sq_norm(f.grad_acc, f.norm_weight)
            sq = part if sq is None else sq + part
        sq = sq * (inv * inv)
        if self.world > 1:
            dist.all_reduce(sq, group=self.group)
        if state.get_model_parallel_world_size() > 1:
            dist.all_reduce(sq, group=state.get_model_parallel_group())
        norm = sq.sqrt()
        self.last_grad_norm = norm
        if scaler is not None:
            self.overflow = scaler.check(norm)      # the same reduced norm, hence the same branch, on every rank
            if self.overflow:
                self.step_count -= 1
                return norm
        if self.clip_grad > 0.0:
            coef = torch.clamp(self.clip_grad / (norm + 1e-6), max=1.0) * inv
        else:
            coef = torch.full_like(norm, inv)
        b1, b2 = self.betas
        if self.offload_optimizer:
            from ..ops import reference as ref
            coef_host = float(coef)                 # one synchronisation per step: the clip coefficient
            for f in self.groups:
                f.host_grad.copy_(f.grad_acc, non_blocking=True)
            if self.groups and self.groups[0].grad_acc.is_cuda:
                torch.cuda.current_stream().synchronize()
            for f in self.groups:
                ref.adam_step(f.master, f.exp_avg, f.exp_avg_sq, f.host_grad, f.hyper["lr"], b1, b2, self.eps,
                              f.hyper["weight_decay"], self.step_count, self.adamw, coef_host, None)
                f.param_shard.copy_(f.master, non_blocking=True)
                f.hpz_fresh = False
                if not f.free_params:
                    _all_gather(f.full, f.shard_on_device(), self.group, self.world)
            return norm
        for f in self.groups:
            low = None if f.master_is_view else f.param_shard
            if f.param_offloaded:
                low = torch.empty(f.shard, dtype=f.param_shard.dtype, device=f.master.device)
            ops.adam_step(f.master, f.exp_avg, f.exp_avg_sq, f.grad_acc, f.hyper["lr"], b1, b2, self.eps,
                          f.hyper["weight_decay"], self.step_count, self.adamw, coef, low)
            if f.param_offloaded:
                f.param_shard.copy_(low, non_blocking=True)         # back to the host copy
            f.hpz_fresh = False                       # the secondary copies hold the old parameters
            if not f.free_params:
                _all_gather(f.full, f.shard_on_device(), self.group, self.world)
        return norm

    # ------------------------------------------------------------------ whole parameters
    @contextlib.contextmanager
    def full_params(self, writeback: bool = False):
        """Every parameter whole inside the context.  With `writeback` the shards (and the fp32 masters) are rebuilt
        from the full buffers on exit — for code that loads or edits parameters."""
        for u in self.units[1:]:
            self._ensure_resident(u)
        try:
            yield
        finally:
            if writeback:
                self.refresh_master_from_params()
            for u in self.units[1:]:
                for f in u.flats:
                    f.release_params()

    def refresh_master_from_params(self) -> None:
        """Rebuild shards and fp32 masters from the parameters: from the full buffer where a unit is whole (inside
        `full_params`, and always for resident units), else from the low-precision shard."""
        with torch.no_grad():
            for f in self.groups:
                if f.resident:
                    f.param_shard.copy_(f.shard_slice(f.full))
                if not f.master_is_view:
                    f.master.copy_(f.param_shard)

    def sync_params_from_master(self) -> None:
        with torch.no_grad():
            for f in self.groups:
                if not f.master_is_view:
                    f.param_shard.copy_(f.master)
                if f.resident:
                    _all_gather(f.full, f.shard_on_device(), self.group, self.world)

    # ------------------------------------------------------------------ state
    def state_dict(self) -> Dict:
        """Stage-1 shaped state (one fp32 partition per flat buffer), tagged with the stage that wrote it."""
        base_state = {i: {"step": self.step_count, "exp_avg": f.exp_avg, "exp_avg_sq": f.exp_avg_sq}
                      for i, f in enumerate(self.groups)}
        return {
            "zero_stage": self.stage,
            "partition_count": [self.world] * len(self.groups),
            "loss_scaler": self.loss_scaler.state_dict() if self.loss_scaler is not None else None,
            "dynamic_loss_scale": bool(self.loss_scaler is not None and self.loss_scaler.dynamic),
            "overflow": bool(self.overflow),
            "clip_grad": self.clip_grad,
            "single_partition_of_fp32_groups": [f.master for f in self.groups],
            "group_paddings": [f.padded - f.numel if self.rank == self.world - 1 else 0 for f in self.groups],
            "flat_names": [f.name for f in self.groups],
            "base_optimizer_state": {
                "state": base_state,
                "param_groups": [{"lr": f.hyper["lr"], "betas": list(self.betas), "eps": self.eps,
                                  "weight_decay": f.hyper["weight_decay"], "name": f.hyper["name"],
                                  "params": [i]} for i, f in enumerate(self.groups)],
            },
        }

    def load_state_dict(self, sd: Dict, load_master: bool = True) -> None:
        masters = sd["single_partition_of_fp32_groups"]
        if len(masters) != len(self.groups):
            raise ValueError("optimizer state has a different number of flat buffers: it was written by another ZeRO "
                             "stage or model cut; load the module only and rebuild the optimizer state")
        st = sd["base_optimizer_state"]["state"]
        with torch.no_grad():
            for i, f in enumerate(self.groups):
                if masters[i].numel() != f.master.numel():
                    raise ValueError(f"optimizer partition size mismatch in buffer {i}: checkpoint was written with a "
                                     "different partition count")
                if load_master:
                    f.master.copy_(masters[i])
                    if not f.master_is_view:
                        f.param_shard.copy_(f.master)
                f.exp_avg.copy_(st[i]["exp_avg"])
                f.exp_avg_sq.copy_(st[i]["exp_avg_sq"])
                self.step_count = int(st[i]["step"])
                f.hyper["lr"] = sd["base_optimizer_state"]["param_groups"][i]["lr"]
                if load_master and f.resident:
                    _all_gather(f.full, f.shard_on_device(), self.group, self.world)
        if self.loss_scaler is not None and isinstance(sd.get("loss_scaler"), dict):
            self.loss_scaler.load_state_dict(sd["loss_scaler"])

    def memory_report(self) -> Dict[str, int]:
        """Bytes this rank holds persistently (shards and optimizer state) and transiently at most (one unit whole)."""
        persistent = sum((0 if f.param_offloaded else f.param_shard.numel() * f.param_shard.element_size()) + f.grad_acc.numel() * 4
                         + (0 if (f.master_is_view or f.optimizer_offloaded) else f.master.numel() * 4)
                         + (0 if f.optimizer_offloaded else 2 * f.exp_avg.numel() * 4)
                         for f in self.groups)
        root = sum(2 * f.nbytes for f in self.units[0].flats)
        unit = max((sum(f.nbytes for f in u.flats) for u in self.units[1:]), default=0)
        return {"persistent_bytes": persistent + root, "largest_unit_param_bytes": unit,
                "full_model_param_bytes": sum(f.nbytes for f in self.groups)}
