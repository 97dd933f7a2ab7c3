"""Training program: distributed set-up, model + optimizer construction, the step and the loop.

Role of the reference's savanna/training.py (pretrain :340, setup_model_and_optimizer :1243,
forward_step :930, train_step :1410, train :1549, evaluate :1801) and savanna/initialize.py, without
DeepSpeed: the engine pieces (ZeRO-1/2/3 optimizers, gradient accumulation, activation checkpointing,
checkpoint I/O) are this package's own.

Public API:
    trainer = Trainer(cfg)                      # builds groups, model, optimizer, scheduler; loads a checkpoint
    loss = trainer.train_step(data_iterator)    # one optimizer step (all accumulation micro-steps)
    trainer.train(train_iter, valid_iter)       # the full loop with logging / eval / checkpoints
    pretrain(cfg)                               # what train.py calls
"""
from __future__ import annotations

import gc
import math
import os
import random
import time
from typing import Dict, Iterator, Optional

import numpy as np
import torch
import torch.distributed as dist

from .. import print_rank_0
from ..models import build_model, losses, param_groups
from ..parallel import state
from ..parallel.zero import ZeroOptimizer
from . import batch as batch_mod
from .lr import build_lr_scheduler


# ----------------------------------------------------------------------------- distributed set-up


def check_distributed_vars() -> None:
    """Environment sanity of a multi-process launch (reference: savanna/distributed.py:6-30)."""
    need = ("MASTER_ADDR", "MASTER_PORT", "RANK", "LOCAL_RANK", "WORLD_SIZE")
    missing = [k for k in need if k not in os.environ]
    if missing:
        raise RuntimeError(f"distributed launch needs the environment variables {missing}")


def set_random_seed(seed: int) -> None:
    """Same seed on every rank for parameters (tensor-parallel weights are sliced from a master draw);
    dropout and data order are offset by the data-parallel rank where they are used."""
    if seed is None or seed < 0:
        raise ValueError(f"seed must be a non-negative integer, got {seed}")
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed(seed)


def initialize_distributed(cfg) -> torch.device:
    world = int(os.environ.get("WORLD_SIZE", "1"))
    use_cuda = torch.cuda.is_available() and cfg.distributed_backend != "gloo"
    if use_cuda:
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local % max(1, torch.cuda.device_count()))
        device = torch.device("cuda", torch.cuda.current_device())
    else:
        device = torch.device("cpu")
    if world > 1 and not dist.is_initialized():
        check_distributed_vars()
        backend = cfg.distributed_backend if use_cuda else "gloo"
        kw = {}
        if backend == "nccl":
            kw["device_id"] = device
        dist.init_process_group(backend=backend, **kw)
    if world > 1 or not state.model_parallel_is_initialized():
        state.initialize_model_parallel(cfg.model_parallel_size, cfg.context_parallel_size,
                                        max(1, cfg.pipe_parallel_size or 0), fp32_allreduce=cfg.fp32_allreduce)
    cfg.rank = dist.get_rank() if dist.is_initialized() else 0
    cfg.world_size = world
    set_random_seed(cfg.seed)
    return device


# ----------------------------------------------------------------------------- trainer


class Trainer:
    def __init__(self, cfg, device: Optional[torch.device] = None, load: bool = True):
        self.cfg = cfg
        self.device = device if device is not None else initialize_distributed(cfg)
        if cfg.tokenizer is None:
            cfg.build_tokenizer()
        if cfg.disable_gc:
            gc.disable()
        self.iteration = 0
        self.tokens_seen = 0
        if self.device.type == "cuda":
            from ..ops import cuda_ops
            cuda_ops.set_fp8_history(cfg.fp8_amax_history_len)
            cuda_ops.set_fp8_recipe(cfg.fp8_recipe)
            from ..ops import attention_cuda
            attention_cuda.set_allow_library(bool(cfg.allow_library_attention))
        if (self.device.type == "cuda" and cfg.comm_path == "symm" and cfg.sequence_parallel
                and state.get_model_parallel_world_size() > 1 and cfg.precision == "bfloat16"):
            from ..parallel import fused_tp
            on = fused_tp.setup()
            print_rank_0(" > tensor-parallel projections: " + (("fused all-gather->GEMM / GEMM->reduce-scatter kernels"
                                                                + (", fp8 operands" if cfg.use_fp8_linears else ""))
                                                               if on else "NCCL collectives + GEMM"))
        if (self.device.type == "cuda" and cfg.comm_path == "symm" and cfg.use_cp_hyena
                and state.get_context_parallel_world_size() > 1 and cfg.precision == "bfloat16"):
            from ..parallel import halo as halo_mod
            on = halo_mod.setup_peer()
            print_rank_0(" > context-parallel halos: " + ("peer-memory pull kernels" if on else "NCCL send/recv"))
        self.model, self.optimizer, self.lr_scheduler = self._setup_model_and_optimizer()
        self.partitioned = hasattr(self.optimizer, "finish_backward")      # ZeRO stage 2 / 3
        self._zero_overlap = self._setup_zero_overlap()
        self.gas = cfg.gradient_accumulation_steps
        self.micro_batch = cfg.train_micro_batch_size_per_gpu
        self.skipped_iters = 0
        self.nan_iters = 0
        self.noise_scale = None
        if cfg.log_gradient_noise_scale and not self.partitioned:
            from .critical_batch import CriticalBatchEstimator
            self.noise_scale = CriticalBatchEstimator(cfg.train_micro_batch_size_per_gpu * cfg.gradient_accumulation_steps,
                                                      cfg.gradient_noise_scale_n_batches,
                                                      cpu_offload=bool(cfg.gradient_noise_scale_cpu_offload))
        # fp16 runs scale the loss; the ZeRO optimizers unscale, look for inf / nan and skip the step when they find one
        from . import loss_scaler as loss_scaler_mod
        from ..utils.watchdog import OverflowMonitor
        self.loss_scaler = loss_scaler_mod.from_config(cfg)
        self.overflow_monitor = OverflowMonitor(50)
        if self.loss_scaler is not None:
            if not hasattr(self.optimizer, "loss_scaler"):
                raise NotImplementedError("fp16 loss scaling needs the Adam-family ZeRO optimizer (stages 0-3)")
            if getattr(self.model, "is_pipeline_stage", False):
                raise NotImplementedError("fp16 loss scaling is not wired into the pipeline schedule; use bf16")
            self.optimizer.loss_scaler = self.loss_scaler
        if cfg.debug_dir:
            # every leaf module's first inputs / outputs go to <debug_dir>/<layout tag>/ for an offline diff of two
            # parallel layouts (python -m savanna_b200.utils.debug <dir a> <dir b>)
            from ..utils.debug import register_debug_hooks
            self._debug_hooks = register_debug_hooks(self.model, cfg)
        from . import curriculum as curriculum_mod
        self.curriculum = curriculum_mod.from_config(cfg)          # sequence-length curriculum, or None
        self.profiler = None
        self.timers = None
        self.watchdog = None
        self.straggler = self.comms_logger = self.alloc_stats = self.mem_snapshots = None
        if load and cfg.load is not None:
            from ..ckpt import load_checkpoint
            self.iteration = load_checkpoint(self)

    # ------------------------------------------------------------------ construction
    def _setup_model_and_optimizer(self):
        cfg = self.cfg
        if (cfg.pipe_parallel_size or 0) > 1:
            from ..parallel.pipeline import build_pipeline_stage
            model = build_pipeline_stage(cfg, self.device)
        else:
            model = build_model(cfg, device=self.device)
        nparams = sum(p.numel() for p in model.parameters())
        total = torch.tensor([float(nparams)], device=self.device)
        if dist.is_initialized() and state.get_model_parallel_world_size() > 1:
            dist.all_reduce(total, group=state.get_model_parallel_group())
        print_rank_0(f" > parameters on tensor-parallel rank 0: {nparams:,} (model total ~{int(total.item()):,})")
        self.num_params = int(total.item())
        groups = param_groups(model, cfg)
        opt_cfg = cfg.optimizer or {"type": "Adam", "params": {}}
        p = dict(opt_cfg.get("params", {}))
        otype = cfg.optimizer_type
        if otype in ("adam", "cpu_adam", "cpu_torch_adam", "onebitadam"):
            zranks = state.get_sequence_data_parallel_ranks()
            off = (cfg.zero_optimization or {}).get("offload_optimizer") or {}
            off_dev = str(off.get("device", "none")).lower() if isinstance(off, dict) else "none"
            offload = off_dev in ("cpu", "nvme")
            nvme_path = None
            if off_dev == "nvme":
                nvme_path = off.get("nvme_path")
                if not nvme_path:
                    raise ValueError("offload_optimizer.device nvme needs offload_optimizer.nvme_path (a directory on the drive)")
            use_symm = (self.device.type == "cuda" and cfg.comm_path == "symm" and len(zranks) > 1
                        and cfg.zero_stage >= 1 and cfg.precision == "bfloat16" and not offload)
            allocator = None
            if use_symm:
                from ..parallel import fused_zero
                allocator = fused_zero.make_allocator(state.get_sequence_data_parallel_group())
            if cfg.zero_stage >= 2 and len(zranks) >= 1 and hasattr(model, "blocks") \
                    and not getattr(model, "is_pipeline_stage", False):
                from ..parallel.zero_partitioned import PartitionedZeroOptimizer
                zgroup, mics = state.get_sequence_data_parallel_group(), {}
                shard = int((cfg.zero_optimization or {}).get("mics_shard_size", 0) or 0)
                if cfg.zero_use_mics and 0 < shard < len(zranks):
                    zgroup, zranks, rgroup, rranks = state.create_mics_groups(shard)
                    me = dist.get_rank() if dist.is_initialized() else 0
                    mics = {"replica_group": rgroup, "replica_world": len(rranks), "replica_index": rranks.index(me)}
                    print_rank_0(f" > MiCS: optimizer state sharded over sub-groups of {shard} ranks, {len(rranks)} replicas")
                hpz = int((cfg.zero_optimization or {}).get("zero_hpz_partition_size", 1) or 1)
                if hpz > 1 and cfg.zero_stage >= 3 and not mics and len(zranks) % hpz == 0 and hpz < len(zranks):
                    hgroup, hranks, _, _ = state.create_mics_groups(hpz)
                    mics = {"hpz_group": hgroup, "hpz_ranks": hranks}
                    print_rank_0(f" > hpZ: secondary parameter partition over sub-groups of {hpz} ranks for the backward gathers")
                offp = (cfg.zero_optimization or {}).get("offload_param") or {}
                offload_param = isinstance(offp, dict) and str(offp.get("device", "none")).lower() == "cpu" and cfg.zero_stage >= 3
                if offload_param:
                    print_rank_0(" > ZeRO-3 parameter offload: released units keep their parameter shard in host memory")
                optimizer = PartitionedZeroOptimizer(
                    groups, model.blocks(), stage=min(3, cfg.zero_stage), lr=cfg.lr,
                    betas=tuple(p.get("betas", (0.9, 0.999))), eps=p.get("eps", 1e-8), weight_decay=cfg.weight_decay,
                    adamw=p.get("adam_w_mode", True), clip_grad=cfg.gradient_clipping or 0.0,
                    group=zgroup, group_ranks=zranks,
                    sync_replicated=bool(cfg.sequence_parallel), offload_param=offload_param, offload_optimizer=offload,
                    nvme_path=nvme_path, **mics)
                rep = optimizer.memory_report()
                print_rank_0(f" > ZeRO stage {optimizer.stage}: {rep['persistent_bytes'] / 2**20:.0f} MiB of shards and "
                             f"optimizer state per rank, largest unit {rep['largest_unit_param_bytes'] / 2**20:.0f} MiB "
                             f"of {rep['full_model_param_bytes'] / 2**20:.0f} MiB of parameters")
                return model, optimizer, build_lr_scheduler(optimizer, cfg)
            optimizer = ZeroOptimizer(
                groups, lr=cfg.lr, betas=tuple(p.get("betas", (0.9, 0.999))), eps=p.get("eps", 1e-8),
                weight_decay=cfg.weight_decay, adamw=p.get("adam_w_mode", True), clip_grad=cfg.gradient_clipping or 0.0,
                group=state.get_sequence_data_parallel_group(), group_ranks=zranks,
                comm_path=cfg.comm_path, partition=cfg.zero_stage >= 1, allocator=allocator, offload_optimizer=offload,
                nvme_path=nvme_path)
            if offload:
                where = f"files under {nvme_path}" if nvme_path else "host memory"
                print_rank_0(f" > ZeRO-Offload: master weights and Adam moments in {where}, update on the CPU")
            if use_symm:
                fused_zero.attach(optimizer, allocator, use_nvls=bool(cfg.use_nvls))
        else:
            from .optimizers import build_generic_optimizer
            optimizer = build_generic_optimizer(otype, groups, cfg, p)
        sched = build_lr_scheduler(optimizer, cfg)
        return model, optimizer, sched

    def _setup_zero_overlap(self):
        """ZeRO-1 reduce-scatter overlapped with the last micro-batch's backward (`zero_optimization.overlap_comm`).
        Needs the fused peer-memory step and gradients that are final when a block's backward ends: not with sequence
        parallelism (replicated parameters' gradients are summed over the tensor-parallel group after the backward),
        pipeline stages, or the gradient-noise-scale estimator (which reads the un-reduced gradients)."""
        cfg = self.cfg
        fused = getattr(self.optimizer, "fused", None)
        if fused is None or not cfg.zero_overlap_comm or getattr(self.model, "is_pipeline_stage", False):
            return None
        if cfg.sequence_parallel and state.get_model_parallel_world_size() > 1:
            return None
        if cfg.log_gradient_noise_scale or not hasattr(self.model, "blocks"):
            return None
        fused.index_blocks(self.optimizer, [list(b.parameters()) for b in self.model.blocks()])
        print_rank_0(" > ZeRO-1 reduce-scatter overlapped with the last micro-batch's backward")
        return fused

    # ------------------------------------------------------------------ forward
    def compute_loss(self, logits: torch.Tensor, b: Dict[str, torch.Tensor]) -> torch.Tensor:
        cfg = self.cfg
        vp = state.get_model_parallel_world_size() > 1
        labels, mask = b["labels"], b["loss_mask"]
        if cfg.to_upper == "upper":
            labels = batch_mod.to_upper_bytes(labels)
        if cfg.alignment_method == "dpo":
            # rows 0..B-1 are the accepted texts, B..2B-1 the rejected ones (train/batch.py:build_batch_dpo)
            lp = losses.sequence_logps(logits, labels, mask, positions=max(1, cfg.seq_length - 1))
            B = lp.shape[0] // 2
            ref = b["ref_logps"]
            loss, _, _ = losses.dpo_loss(lp[:B], lp[B:], ref[:B], ref[B:], beta=cfg.dpo_beta)
            return loss
        if cfg.pretraining_strategy == "OADM":
            return losses.oadm_loss(logits, labels, mask, None)
        if cfg.to_upper in ("weighted", "normalized_weighted"):
            return losses.reweighted_cross_entropy(logits, labels, mask, cfg.lowercase_loss_reweighting,
                                                   normalize_per_batch=cfg.to_upper == "normalized_weighted",
                                                   vocab_parallel=vp)
        return losses.cross_entropy(logits, labels, mask, vocab_parallel=vp)

    def forward_step(self, b: Dict[str, torch.Tensor], return_logits: bool = False):
        tokens = b["tokens"]
        if self.cfg.to_upper in ("upper", "weighted", "normalized_weighted"):
            tokens = batch_mod.to_upper_bytes(tokens)
        logits = self.model(tokens, b["positions"])
        loss = self.compute_loss(logits, b)
        return (loss, logits) if return_logits else loss

    # ------------------------------------------------------------------ step
    def _unwatched(self):
        """Context for host-side phases that are not steps (checkpoint save, evaluation): the watchdog's step
        deadline is suspended inside it."""
        import contextlib
        return self.watchdog.paused() if self.watchdog is not None else contextlib.nullcontext()

    def check_device_status(self) -> None:
        """Raise if a device-side bounded wait (peer barrier, mbarrier, fused tensor-parallel pull) gave up since
        the last check.  Those kernels record a code in a per-device status word and return instead of hanging; a
        step that continued after one has used stale or partial peer data, so the run must stop and relaunch from
        the last checkpoint.  Reading the word synchronises with the device, so this is called where the host
        synchronises anyway: at the logging interval and before a checkpoint is written."""
        reader = getattr(self, "status_reader", None)    # tests inject a host-side word here
        if reader is None:
            if self.device.type != "cuda":
                return
            from ..ops import cuda_ops
            cuda_ops.check_status()
            return
        v = int(reader())
        if v != 0:
            raise RuntimeError(f"a kernel gave up on a bounded wait: code {(v >> 24) & 0xff}, detail {v & 0xffffff}")

    def _mark(self, name: str):
        import contextlib
        det = getattr(self, "straggler", None)
        if self.profiler is None and det is None:
            return contextlib.nullcontext()
        stack = contextlib.ExitStack()
        if self.profiler is not None:
            stack.enter_context(self.profiler.mark(name))
        if det is not None:
            stack.enter_context(det.section(name))
        return stack

    def train_step(self, data_iterator: Iterator) -> torch.Tensor:
        """One optimizer step over `gradient_accumulation_steps` micro-batches.  Returns the mean loss
        (0-dim device tensor; no host synchronisation happens inside the step)."""
        cfg = self.cfg
        if getattr(self.model, "is_pipeline_stage", False):
            from ..parallel.pipeline import pipeline_train_step
            return pipeline_train_step(self, data_iterator)
        self.model.train()
        self.optimizer.zero_grad()
        total = None
        max_len = None
        if self.curriculum is not None:
            # iteration + 1: the length of the step that is about to run (a resumed run continues the schedule)
            max_len = cfg.curriculum_seqlen = self.curriculum.update_difficulty(self.iteration + 1)
            if max_len >= cfg.seq_length:
                max_len = None
        for micro in range(self.gas):
            # the last micro-batch's forward plants the hooks through which its backward reports finished blocks
            overlap = self._zero_overlap if micro == self.gas - 1 else None
            if overlap is not None:
                opt = self.optimizer
                self.model.grad_boundary_callback = lambda i: overlap.grads_final_from(opt, i)
            try:
                with self._mark("TRAIN_STEP_FORWARD"):
                    b = batch_mod.get_batch(cfg, data_iterator, self.device, max_len)
                    loss = self.forward_step(b)
                with self._mark("TRAIN_STEP_BACKWARD"):
                    if overlap is not None:
                        overlap.begin_overlap(self.optimizer)
                    if self.loss_scaler is not None:
                        (loss * (self.loss_scaler.scale / self.gas)).backward()
                    else:
                        (loss / self.gas).backward()
                    if self.partitioned:
                        self.optimizer.finish_backward()
            finally:
                self.model.grad_boundary_callback = None
            total = loss.detach() if total is None else total + loss.detach()
        if not self.partitioned:
            self._sync_replicated_grads()
        if self.noise_scale is not None:
            # this rank's accumulated gradient, before the data-parallel reduction, is the "small batch" sample
            self.noise_scale.update([p for p in self.model.parameters() if p.requires_grad])
        with self._mark("TRAIN_STEP_OPTIMIZER_STEP"):
            self.grad_norm = self.optimizer.step()
            if self.loss_scaler is not None and getattr(self.optimizer, "overflow", False):
                # fp16: inf / nan gradients, no update was made; the learning-rate schedule does not advance either
                self.skipped_iters += 1
                self.overflow_monitor.check(True)
            else:
                if self.loss_scaler is not None:
                    self.overflow_monitor.check(False)
                self.lr_scheduler.step()
        self.iteration += 1
        self.tokens_seen += cfg.train_batch_size * (max_len or cfg.seq_length)
        if self.watchdog is not None:
            self.watchdog.beat(self.iteration)
        return self._reduce_loss(total / self.gas)

    def _reduce_loss(self, loss: torch.Tensor) -> torch.Tensor:
        """Mean of the step's loss over the data-parallel replicas (what gets logged; the reference's
        `reduce_losses`, savanna/utils.py:47-52).  One scalar all-reduce, no host synchronisation."""
        dp = state.get_data_parallel_world_size()
        if dp == 1 or not dist.is_initialized():
            return loss
        loss = loss.clone()
        dist.all_reduce(loss, group=state.get_data_parallel_group())
        return loss / dp

    def _sync_replicated_grads(self) -> None:
        """Sequence parallelism: parameters replicated over the tensor-parallel group (norm gains, row
        biases) see only a sequence slice per rank, so their gradients are summed over the group in ONE
        flat all-reduce (the reference registers a hook per norm weight, model/utils.py:329-368)."""
        cfg = self.cfg
        tp = state.get_model_parallel_world_size()
        if tp == 1 or not cfg.sequence_parallel:
            return
        grads = [p.grad for p in self.model.parameters()
                 if p.grad is not None and not getattr(p, "model_parallel", False)]
        if not grads:
            return
        flat = torch.cat([g.reshape(-1) for g in grads])
        dist.all_reduce(flat, group=state.get_model_parallel_group())
        off = 0
        for g in grads:
            g.copy_(flat[off:off + g.numel()].view_as(g))
            off += g.numel()

    # ------------------------------------------------------------------ evaluation
    @torch.no_grad()
    def evaluate(self, data_iterator: Iterator, iters: Optional[int] = None) -> Dict[str, float]:
        cfg = self.cfg
        self.model.eval()
        n = iters if iters is not None else cfg.eval_iters
        acc = torch.zeros((), device=self.device)
        for _ in range(n):
            b = batch_mod.get_batch(cfg, data_iterator, self.device)
            acc += self.forward_step(b).float()
        self.model.train()
        acc = acc / max(1, n)
        if dist.is_initialized() and state.get_data_parallel_world_size() > 1:
            dist.all_reduce(acc, group=state.get_data_parallel_group())
            acc = acc / state.get_data_parallel_world_size()
        lm = float(acc)
        out = {"lm_loss": lm, "lm_loss_ppl": math.exp(min(20.0, lm))}
        if cfg.char_level_ppl:
            out["lm_loss_char_lvl_ppl"] = out["lm_loss_ppl"]
        return out

    def evaluate_per_dataset(self, iters: Optional[int] = None) -> Dict[str, Dict[str, float]]:
        """Validation loss of every data source on its own (reference: savanna/training.py:1897-1940); the iterators
        are built on first use and keep their position between calls."""
        from ..data.loaders import build_per_dataset_val_iterators
        if getattr(self, "_per_ds_iters", None) is None:
            self._per_ds_iters = build_per_dataset_val_iterators(self.cfg)
        n = iters if iters is not None else (self.cfg.eval_per_ds_iters or self.cfg.eval_iters)
        return {name: self.evaluate(it, n) for name, _path, it in self._per_ds_iters}

    # ------------------------------------------------------------------ loop
    def train(self, train_iter: Iterator, valid_iter: Optional[Iterator] = None) -> None:
        from ..ckpt import save_checkpoint
        from ..utils.logging import TrainingLogger
        from ..utils.profiler import setup_profiler
        from ..utils.watchdog import Watchdog
        cfg = self.cfg
        logger = TrainingLogger(cfg, self)
        self.profiler = setup_profiler(cfg)
        if cfg.watchdog_step_timeout and cfg.watchdog_step_timeout > 0:
            self.watchdog = Watchdog(cfg.watchdog_step_timeout, cfg.watchdog_heartbeat_dir, rank=cfg.rank or 0)
            self.watchdog.start()
        from ..utils import observability
        self.straggler, self.comms_logger, self.alloc_stats = observability.build_from_config(
            cfg, cfg.rank or 0, int(os.environ.get("WORLD_SIZE", "1")))
        from ..utils.memory_stats import MemorySnapshotter
        self.mem_snapshots = MemorySnapshotter.from_config(cfg, cfg.rank or 0, self.iteration)
        self.profiler.start()
        if cfg.save and self.iteration == 0 and cfg.save_iters and 0 in cfg.save_iters:
            with self._unwatched():
                save_checkpoint(self)
        try:
            while self.iteration < cfg.train_iters:
                t0 = time.time()
                try:
                    loss = self.train_step(train_iter)
                except torch.OutOfMemoryError:
                    if self.mem_snapshots is not None:
                        self.mem_snapshots.on_oom()      # the allocator history that led to the failure
                    raise
                self.profiler.step()
                if self.mem_snapshots is not None:
                    self.mem_snapshots.step()
                logger.log_step(loss, time.time() - t0)
                it = self.iteration
                if self.straggler is not None:
                    self.straggler.step()
                if self.alloc_stats is not None:
                    self.alloc_stats.step(it)
                if self.comms_logger is not None and it % max(1, cfg.deepspeed_comms_logging_interval or cfg.log_interval or 1) == 0:
                    if cfg.deepspeed_comms_print_summary and (cfg.rank or 0) == 0:
                        print_rank_0(f"comms summary at iteration {it}: {self.comms_logger.summary()}")
                    self.comms_logger.serialize(cfg.deepspeed_comms_ops_to_log)
                if cfg.async_save:
                    from ..ckpt.io import finalize_async_save
                    finalize_async_save(blocking=False)  # publishes `latest` once every rank's writer is done
                if it % max(1, cfg.log_interval or 1) == 0:
                    self.check_device_status()          # the logger has just read the loss: the device is idle
                if cfg.save and cfg.save_iters and it in cfg.save_iters:
                    self.check_device_status()          # never write a checkpoint of a corrupted run
                    with self._unwatched():
                        save_checkpoint(self)
                if valid_iter is not None and cfg.eval_interval and it % cfg.eval_interval == 0 and cfg.do_valid != 0:
                    with self._unwatched():
                        res = self.evaluate(valid_iter)
                    logger.log_eval(res, it)
                if cfg.do_per_ds_valid and cfg.eval_per_ds_interval and it % cfg.eval_per_ds_interval == 0:
                    with self._unwatched():
                        per_ds = self.evaluate_per_dataset()
                    for name, res in per_ds.items():
                        logger.log_eval(res, it, prefix=f"validation/{name}")
                if cfg.exit_interval and it % cfg.exit_interval == 0:
                    print_rank_0(f"exit_interval reached at iteration {it}")
                    break
                if cfg.disable_gc and it % 100 == 0:
                    gc.collect(cfg.gc_collect_generation)
        finally:
            self.profiler.stop()
            if self.mem_snapshots is not None:
                self.mem_snapshots.close()
            if self.watchdog is not None:
                self.watchdog.stop()
            if self.comms_logger is not None:
                self.comms_logger.uninstall()
            if cfg.async_save:
                from ..ckpt.io import finalize_async_save
                finalize_async_save(blocking=True)
        if cfg.save and self.iteration > 0 and (not cfg.save_iters or self.iteration not in cfg.save_iters):
            self.check_device_status()
            save_checkpoint(self)
        if cfg.async_save:
            from ..ckpt.io import finalize_async_save
            finalize_async_save(blocking=True)


# ----------------------------------------------------------------------------- entry


def pretrain(cfg) -> Trainer:
    """Entry used by train.py: set up, build data iterators, train, final evaluation."""
    from ..data.loaders import build_train_valid_test_data_iterators
    if cfg.use_mup and cfg.save_base_shapes:
        from . import mup_shapes
        rank = dist.get_rank() if dist.is_initialized() else 0
        path = f"{cfg.base_shapes_file or 'base-shapes'}.{rank}"
        if cfg.padded_vocab_size is None:
            cfg.build_tokenizer()
        mup_shapes.save_base_shapes(cfg, path)
        raise SystemExit(f"base shapes written to {path}; exiting (rerun without save_base_shapes to train)")
    if cfg.use_mup and cfg.coord_check:
        raise SystemExit("coord_check: run `python -m savanna_b200.train.mup_coord_check <model configs>`; it builds the "
                         "model at several widths itself (the reference also exits after its coordinate check)")
    trainer = Trainer(cfg)
    cfg.iteration = trainer.iteration
    train_it, valid_it, test_it = build_train_valid_test_data_iterators(cfg, trainer)
    if cfg.do_train is None or cfg.do_train:
        trainer.train(train_it, valid_it)
    if valid_it is not None and cfg.do_valid:
        res = trainer.evaluate(valid_it)
        print_rank_0(f"final validation: {res}")
    if test_it is not None and cfg.do_test:
        res = trainer.evaluate(test_it)
        print_rank_0(f"final test: {res}")
    return trainer
