"""Checkpoint save / load in the DeepSpeed directory layout the reference produces, so its tools
(tensor-parallel reshard, projection interleave, filter extension, zero_to_fp32, vortex export) keep
working on files written here and its checkpoints load here.

    <save>/latest                                   text: "global_step<N>"
    <save>/global_step<N>/mp_rank_<TP:02d>_model_states.pt
        module (state dict, keys `sequential.<i>...`), param_shapes, buffer_names, shared_params,
        frozen_param_shapes, ds_config, ds_version, dp_world_size, mp_world_size, lr_scheduler,
        + client state: iteration, args, data_loading, RNG states, optional validation logits
    <save>/global_step<N>/[bf16_]zero_pp_rank_<DP>_mp_rank_<TP:02d>_optim_states.pt
        optimizer_state_dict (ZeRO stage-1 shaped, see parallel/zero.py), ds_config, ds_version
    <save>/global_step<N>/configs/*.yml             the raw YAML files of the run

With pipeline stages (pipe_parallel_size > 1) the files follow DeepSpeed's pipeline engine: the module is written
as one file per layer slot, `layer_<IDX:02d>-model_<TP:02d>-model_states.pt` (keys without the `sequential.<IDX>.`
prefix; a tied embedding held by two stages is written by the first), and the `mp_rank_` number of the engine and
optimizer files is the combined model rank `pipe_stage * tp + tp_rank`, so no two stages share a path.

Behaviour (reference: savanna/checkpointing.py:153-571): tag `global_step<N>`; `latest` is reconciled
with the directories on disk (the older of the two wins, so a half-written newest checkpoint is
skipped); keep-last-N deletion; optional background (async) writing finalised at the next step;
finetune = module only and iteration 0; warmstart = everything but the iteration, data cursor and random streams;
`no_load_optim` / `no_load_rng`; strict toggle; optional
forward-pass logits validation; data cursor (`train_data_token_index`) and LR-scheduler restore.
"""
from __future__ import annotations

import glob
import contextlib
import os
import random
import re
import shutil
import threading
import time
from collections import OrderedDict
from typing import Dict, Optional

import numpy as np
import torch
import torch.distributed as dist

from .. import __version__, print_rank_0
from ..parallel import state

DS_VERSION = "0.14.0+savanna_b200." + __version__
_ASYNC: Dict[str, threading.Thread] = {}
_PENDING: list = []          # (cfg, root, dir, iteration) of background saves whose `latest` is not yet written

ARGS_TO_CHECK = ("num_layers", "hidden_size", "num_attention_heads", "max_position_embeddings", "make_vocab_size_divisible_by",
                 "padded_vocab_size", "tokenizer_type", "model_parallel_size")


def checkpoint_dir(root: str, iteration: int) -> str:
    return os.path.join(root, f"global_step{iteration}")


def model_states_name(tp_rank: int) -> str:
    return f"mp_rank_{tp_rank:02d}_model_states.pt"


def optim_states_name(dp_rank: int, tp_rank: int, bf16: bool) -> str:
    return f"{'bf16_' if bf16 else ''}zero_pp_rank_{dp_rank}_mp_rank_{tp_rank:02d}_optim_states.pt"


def layer_states_name(layer_idx: int, tp_rank: int) -> str:
    return f"layer_{layer_idx:02d}-model_{tp_rank:02d}-model_states.pt"


def _model_rank() -> int:
    """Rank in the `mp_rank_XX` file names: the tensor-parallel rank, or with pipeline stages the combined
    (stage, tensor-parallel) rank, as DeepSpeed's pipeline grid numbers its model-parallel ranks."""
    pp = state.get_pipe_parallel_world_size()
    tp_rank = state.get_model_parallel_rank()
    if pp <= 1:
        return tp_rank
    return state.get_pipe_parallel_rank() * state.get_model_parallel_world_size() + tp_rank


def _split_by_layer(module_sd: Dict) -> Dict[int, Dict]:
    out: Dict[int, Dict] = {}
    for k, v in module_sd.items():
        m = re.match(r"sequential\.(\d+)\.(.+)$", k)
        if m is None:
            raise KeyError(f"module key {k!r} does not belong to a layer slot")
        out.setdefault(int(m.group(1)), OrderedDict())[m.group(2)] = v
    return out


def _zero_rank(trainer) -> int:
    """Index of this rank's optimizer shard in the file names: its position in the partition group (with MiCS sharding
    that is the sub-group, whose replicas all hold the same shards)."""
    opt = trainer.optimizer
    if getattr(opt, "replica_world", 1) > 1:
        return opt.rank
    return state.get_sequence_data_parallel_rank()


def _writes_optimizer(trainer) -> bool:
    return getattr(trainer.optimizer, "replica_index", 0) == 0          # replicas of a MiCS sub-group hold identical shards


def _barrier():
    if dist.is_available() and dist.is_initialized():
        dist.barrier()


def _rank() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


# ----------------------------------------------------------------------------- global step resolution


def read_global_step(load_dir: str) -> Optional[int]:
    """Iteration to resume from: min(latest file, newest global_step directory), None if nothing usable."""
    latest = None
    p = os.path.join(load_dir, "latest")
    if os.path.isfile(p):
        m = re.match(r"global_step(\d+)", open(p).read().strip())
        if m:
            latest = int(m.group(1))
    on_disk = []
    for d in glob.glob(os.path.join(load_dir, "global_step*")):
        m = re.match(r"global_step(\d+)$", os.path.basename(d))
        if m and os.path.isdir(d):
            on_disk.append(int(m.group(1)))
    if latest is None and not on_disk:
        return None
    if latest is None:
        return max(on_disk)
    if not on_disk:
        return None
    newest = max(on_disk)
    step = min(latest, newest)
    if step not in on_disk:
        older = [s for s in on_disk if s <= step]
        return max(older) if older else None
    return step


# ----------------------------------------------------------------------------- save


def _client_state(trainer, validation_logits=None) -> Dict:
    cfg = trainer.cfg
    sd = {
        "iteration": trainer.iteration,
        "args": {k: getattr(cfg, k) for k in ARGS_TO_CHECK},
        "data_loading": {
            "train_data_token_index": trainer.tokens_seen,
            "train_val_test_num_samples": cfg.train_val_test_num_samples,
        },
    }
    if not cfg.no_save_rng:
        sd["random_rng_state"] = random.getstate()
        sd["np_rng_state"] = np.random.get_state()
        sd["torch_rng_state"] = torch.get_rng_state()
        sd["cuda_rng_state"] = torch.cuda.get_rng_state() if torch.cuda.is_available() else None
        from ..parallel.random import get_cuda_rng_tracker
        sd["rng_tracker_states"] = get_cuda_rng_tracker().get_states()
    if validation_logits is not None:
        sd["checkpoint_validation_logits"] = validation_logits
    return sd


@torch.no_grad()
def _validation_forward(trainer):
    """Logits [L, V] of a fixed input (token i = i modulo the vocabulary, one micro-batch; every row is the same, the
    first is kept) in evaluation mode: stored with the checkpoint and recomputed after loading
    (`checkpoint_validation_with_forward_pass`, reference: savanna/checkpointing.py:70-128).  None for layouts where one
    rank does not see whole rows (pipeline stages, context parallelism)."""
    cfg, model = trainer.cfg, trainer.model
    if getattr(model, "is_pipeline_stage", False) or state.get_context_parallel_world_size() > 1:
        return None
    vocab = cfg.padded_vocab_size or 512
    tokens = (torch.arange(cfg.seq_length, device=trainer.device) % vocab).repeat(cfg.train_micro_batch_size_per_gpu, 1)
    was_training = model.training
    model.eval()
    try:
        logits = model(tokens, torch.arange(cfg.seq_length, device=trainer.device))
    finally:
        if was_training:
            model.train()
    return logits[0].detach().float().cpu()


def _param_shapes(trainer):
    names = {id(p): n for n, p in trainer.model.named_parameters()}
    out = []
    opt = trainer.optimizer
    if hasattr(opt, "groups"):
        for g in opt.groups:
            out.append(OrderedDict((names[id(p)], p.shape) for p in g.params))
    else:
        out.append(OrderedDict((n, p.shape) for n, p in trainer.model.named_parameters()))
    return out


def _write(obj, path: str) -> None:
    tmp = path + ".tmp"
    torch.save(obj, tmp)
    os.replace(tmp, path)


def _to_cpu(obj):
    if isinstance(obj, torch.Tensor):
        return obj.detach().to("cpu", copy=True)
    if isinstance(obj, dict):
        return type(obj)((k, _to_cpu(v)) for k, v in obj.items())
    if isinstance(obj, (list, tuple)):
        return type(obj)(_to_cpu(v) for v in obj)
    return obj


def finalize_async_save(blocking: bool = True) -> bool:
    """Complete background checkpoint writes.  Non-blocking: returns False while any rank is still writing (the
    ranks agree through one small all-reduce, so either all publish or none).  Blocking: joins the writers.
    Returns True when nothing is pending any more."""
    if not _ASYNC and not _PENDING:
        return True
    busy = any(th.is_alive() for th in _ASYNC.values())
    if not blocking and dist.is_available() and dist.is_initialized():
        flag = torch.tensor([1.0 if busy else 0.0])
        if dist.get_backend() == "nccl":
            flag = flag.cuda()
        dist.all_reduce(flag, op=dist.ReduceOp.MAX)
        busy = bool(flag.item() > 0)
    if busy and not blocking:
        return False
    for tag, th in list(_ASYNC.items()):
        th.join()
        _ASYNC.pop(tag, None)
    pending = list(_PENDING)
    _PENDING.clear()
    for cfg, root, d, it in pending:
        _barrier()
        _publish(cfg, root, d, it)
    return True


def save_checkpoint(trainer, iteration: Optional[int] = None) -> str:
    cfg = trainer.cfg
    it = trainer.iteration if iteration is None else iteration
    root = cfg.save
    d = checkpoint_dir(root, it)
    tp_rank = state.get_model_parallel_rank()
    mp_rank = _model_rank()
    pp = state.get_pipe_parallel_world_size()
    zero_rank = _zero_rank(trainer)
    if not _writes_optimizer(trainer):
        zero_rank = -1 - zero_rank                # a replica of a MiCS sub-group: takes part in collectives, writes nothing
    bf16 = cfg.precision == "bfloat16"
    finalize_async_save(True)
    if _rank() == 0:
        os.makedirs(d, exist_ok=True)
    _barrier()
    files = {}
    # the validation pass is collective under tensor parallelism and ZeRO-3: every rank runs it, writers keep the result
    validation_logits = _validation_forward(trainer) if cfg.checkpoint_validation_with_forward_pass else None
    full = getattr(trainer.optimizer, "full_params", None)          # ZeRO-3: the gather is collective, all ranks enter
    with (full() if full is not None else contextlib.nullcontext()):
        module_sd = {k: v.detach().clone() for k, v in trainer.model.state_dict().items()} \
            if (full is not None and zero_rank == 0) else (trainer.model.state_dict() if zero_rank == 0 else None)
    if zero_rank == 0:
        if pp > 1:
            # one file per layer slot of this stage; a tied embedding copy on the last stage is not written again
            for idx, sd in _split_by_layer(module_sd).items():
                if idx == 0 and state.get_pipe_parallel_rank() != 0:
                    continue
                files[os.path.join(d, layer_states_name(idx, tp_rank))] = sd
            module_sd = None
        ms = {
            "module": module_sd,
            "buffer_names": [n for n, _ in trainer.model.named_buffers()],
            "param_shapes": _param_shapes(trainer),
            "frozen_param_shapes": None,
            "shared_params": {},
            "frozen_param_fragments": None,
            "lr_scheduler": trainer.lr_scheduler.state_dict() if trainer.lr_scheduler is not None else None,
            "optimizer": None,
            "sparse_tensor_module_names": [],
            "skipped_steps": trainer.skipped_iters,
            "global_steps": it,
            "global_samples": it * cfg.train_batch_size,
            "dp_world_size": state.get_sequence_data_parallel_world_size(),
            "mp_world_size": state.get_model_parallel_world_size(),
            "ds_config": cfg.engine_config,
            "ds_version": DS_VERSION,
        }
        ms.update(_client_state(trainer, validation_logits))
        files[os.path.join(d, model_states_name(mp_rank))] = ms
    if not cfg.no_save_optim and hasattr(trainer.optimizer, "state_dict") and _writes_optimizer(trainer):
        files[os.path.join(d, optim_states_name(zero_rank, mp_rank, bf16))] = {
            "optimizer_state_dict": trainer.optimizer.state_dict(),
            "ds_config": cfg.engine_config,
            "ds_version": DS_VERSION,
        }

    def write_all(objs):
        for path, obj in objs.items():
            _write(obj, path)

    if cfg.async_save:
        snap = {p: _to_cpu(o) for p, o in files.items()}
        th = threading.Thread(target=write_all, args=(snap,), daemon=False)
        th.start()
        _ASYNC[f"global_step{it}"] = th
    else:
        write_all(files)
    if _rank() == 0:
        if cfg.config_files:
            cdir = os.path.join(d, "configs")
            os.makedirs(cdir, exist_ok=True)
            for name, text in cfg.config_files.items():
                with open(os.path.join(cdir, name), "w") as fh:
                    fh.write(text)
    if cfg.async_save:
        # The writer threads keep running while training continues; `latest`, pruning and uploads wait until every
        # rank's files are complete: at the trainer's next step (`finalize_async_save(False)` polls), at the next
        # save, or at exit (`finalize_async_save(True)`).
        _PENDING.append((cfg, root, d, it))
        print_rank_0(f"  checkpoint at iteration {it}: writing {d} in the background")
        return d
    _barrier()
    _publish(cfg, root, d, it)
    return d


def _publish(cfg, root: str, d: str, it: int) -> None:
    """All ranks' files of checkpoint `d` are on disk: point `latest` at it, prune, upload."""
    if _rank() == 0:
        with open(os.path.join(root, "latest"), "w") as fh:
            fh.write(f"global_step{it}")
        if cfg.keep_last_n_checkpoints:
            _delete_old(root, cfg.keep_last_n_checkpoints)
        # only every `save_retain_interval`-th iteration goes to the long-term stores; the others live (and are
        # pruned) on the local disk alone (reference: savanna/checkpointing.py:338-346)
        if cfg.checkpoint_stores and it % max(1, int(cfg.save_retain_interval or 1)) == 0:
            _upload(cfg, d)
    _barrier()
    print_rank_0(f"  saved checkpoint at iteration {it} to {d}")


def _delete_old(root: str, keep: int) -> None:
    steps = sorted(int(re.match(r"global_step(\d+)$", os.path.basename(p)).group(1))
                   for p in glob.glob(os.path.join(root, "global_step*")) if re.match(r"global_step(\d+)$", os.path.basename(p)))
    for s in steps[:-keep] if keep > 0 else []:
        d = os.path.join(root, f"global_step{s}")
        if os.path.exists(os.path.join(d, ".uploading")):
            continue                                 # an upload of this directory has not finished: keep it
        shutil.rmtree(d, ignore_errors=True)


def _upload(cfg, ckpt_dir: str) -> None:
    """Copy a finished checkpoint to every configured store (ckpt/stores.py: posix directories, S3 buckets)."""
    from .stores import build_stores, upload_checkpoint
    upload_checkpoint(ckpt_dir, build_stores(cfg.checkpoint_stores))


# ----------------------------------------------------------------------------- load


def _check_args(cfg, saved: Dict) -> None:
    for k, v in (saved or {}).items():
        mine = getattr(cfg, k, None)
        if mine != v:
            print_rank_0(f"  WARNING: checkpoint was written with {k}={v!r}, current configuration has {mine!r}")


def load_checkpoint(trainer, iteration: Optional[int] = None) -> int:
    cfg = trainer.cfg
    load_dir = cfg.load
    it = iteration if iteration is not None else (cfg.iteration if cfg.iteration is not None else read_global_step(load_dir))
    if it is None:
        print_rank_0(f"  no checkpoint found in {load_dir}; starting from scratch")
        return 0
    d = checkpoint_dir(load_dir, it)
    tp_rank = state.get_model_parallel_rank()
    mp_rank = _model_rank()
    zero_rank = _zero_rank(trainer)
    path = os.path.join(d, model_states_name(mp_rank))
    if not os.path.isfile(path):
        raise FileNotFoundError(f"checkpoint file {path} not found")
    dev = trainer.device
    ms = torch.load(path, map_location="cpu", weights_only=False)
    _check_args(cfg, ms.get("args"))
    if ms.get("module") is None:
        # pipeline layout: collect this stage's layer slots from the per-layer files
        module = OrderedDict()
        slots = sorted({int(k.split(".")[1]) for k in trainer.model.state_dict().keys()})
        for idx in slots:
            lp = os.path.join(d, layer_states_name(idx, tp_rank))
            if not os.path.isfile(lp):
                raise FileNotFoundError(f"checkpoint file {lp} not found")
            for k, v in torch.load(lp, map_location="cpu", weights_only=False).items():
                module[f"sequential.{idx}.{k}"] = v
        ms["module"] = module
    full = getattr(trainer.optimizer, "full_params", None)          # ZeRO-3: load into whole parameters, re-shard after
    with (full(writeback=True) if full is not None else contextlib.nullcontext()):
        missing, unexpected = trainer.model.load_state_dict(ms["module"], strict=False)
    # buffers that are recomputed (rotary tables, filter time index) may be absent in foreign checkpoints
    missing = [k for k in missing if not k.endswith((".inv_freq", ".filter.t", ".decay"))]
    if cfg.checkpoint_strict_load and (missing or unexpected):
        raise RuntimeError(f"checkpoint does not match the model: missing {missing[:8]}, unexpected {unexpected[:8]}")
    module_only = cfg.finetune or cfg.no_load_optim
    opt = trainer.optimizer
    bf16 = cfg.precision == "bfloat16"
    if not module_only and hasattr(opt, "load_state_dict"):
        opath = os.path.join(d, optim_states_name(zero_rank, mp_rank, bf16))
        if os.path.isfile(opath):
            osd = torch.load(opath, map_location=dev, weights_only=False)
            opt.load_state_dict(osd["optimizer_state_dict"])
        else:
            print_rank_0(f"  optimizer state {opath} not found; master weights are rebuilt from the module")
            if hasattr(opt, "refresh_master_from_params"):
                opt.refresh_master_from_params()
    elif hasattr(opt, "refresh_master_from_params"):
        opt.refresh_master_from_params()
    if cfg.finetune:
        it_out = 0
    elif cfg.warmstart:
        # weights, optimizer state and LR schedule come from the checkpoint, but the run counts from iteration 0 with a
        # fresh data cursor and fresh random streams (reference: checkpointing.py:445, :495)
        it_out = 0
        if trainer.lr_scheduler is not None and ms.get("lr_scheduler") is not None and not cfg.no_load_optim:
            trainer.lr_scheduler.load_state_dict(ms["lr_scheduler"])
    else:
        it_out = int(ms.get("iteration", it))
        if trainer.lr_scheduler is not None and ms.get("lr_scheduler") is not None and not cfg.no_load_optim:
            trainer.lr_scheduler.load_state_dict(ms["lr_scheduler"])
        dl = ms.get("data_loading") or {}
        if dl.get("train_data_token_index") is not None:
            trainer.tokens_seen = int(dl["train_data_token_index"])
            cfg.train_data_token_index = trainer.tokens_seen
        if cfg.use_checkpoint_num_samples and dl.get("train_val_test_num_samples") is not None:
            cfg.train_val_test_num_samples = dl["train_val_test_num_samples"]
        if not cfg.no_load_rng and "torch_rng_state" in ms:
            random.setstate(ms["random_rng_state"])
            np.random.set_state(ms["np_rng_state"])
            torch.set_rng_state(ms["torch_rng_state"])
            if torch.cuda.is_available() and ms.get("cuda_rng_state") is not None and dev.type == "cuda":
                torch.cuda.set_rng_state(ms["cuda_rng_state"])
            if ms.get("rng_tracker_states"):
                from ..parallel.random import get_cuda_rng_tracker
                get_cuda_rng_tracker().set_states(ms["rng_tracker_states"])
    if cfg.checkpoint_validation_with_forward_pass and "checkpoint_validation_logits" in ms:
        _validate_logits(trainer, ms)
    _barrier()
    print_rank_0(f"  loaded checkpoint {d} (iteration {it_out})")
    return it_out


def _validate_logits(trainer, ms) -> None:
    want = ms["checkpoint_validation_logits"]
    got = _validation_forward(trainer)
    if got is None or want is None:
        return
    want = want.float().cpu()
    if got.shape != want.shape:
        raise RuntimeError(f"stored validation logits have shape {tuple(want.shape)}, this model produces {tuple(got.shape)}")
    if not torch.equal(got, want):
        if not torch.allclose(got, want, atol=1e-2, rtol=1e-2):
            raise RuntimeError("forward pass after loading does not reproduce the logits stored with the checkpoint")
        print_rank_0("  checkpoint validation: logits after loading are close to, not identical with, the stored ones")
