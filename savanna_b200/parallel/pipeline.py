"""Pipeline parallelism over point-to-point messages (NCCL on GPUs, gloo on CPU).

Each stage owns a contiguous range of blocks (`Backbone(layer_range=...)`); the first stage also owns the
embedding, the last stage the final norm and the logits (with tied embeddings it holds a copy of the
embedding whose gradient is all-reduced with the first stage's after every step).  One optimizer step runs
the `gradient_accumulation_steps` micro-batches through an all-forward / all-backward schedule; activations
and their gradients travel as [B, L, D] tensors.  Role of the reference's DeepSpeed PipelineModule /
PipelineEngine use (savanna/model/backbone.py:219-284, savanna/training.py:1517-1546).
"""
from __future__ import annotations

from typing import List, Tuple

import torch
import torch.distributed as dist

from ..train import batch as batch_mod
from . import state


def stage_layer_range(num_layers: int, pp: int, stage: int) -> range:
    base, rem = divmod(num_layers, pp)
    start = stage * base + min(stage, rem)
    return range(start, start + base + (1 if stage < rem else 0))


def build_pipeline_stage(cfg, device):
    from ..models.backbone import Backbone
    pp, stage = state.get_pipe_parallel_world_size(), state.get_pipe_parallel_rank()
    model = Backbone(cfg, device=device, layer_range=stage_layer_range(cfg.num_layers, pp, stage))
    model.is_pipeline_stage = True
    model.stage, model.num_stages = stage, pp
    return model


def _neighbours() -> Tuple[int, int]:
    ranks, s = state.get_pipe_parallel_ranks(), state.get_pipe_parallel_rank()
    prev = ranks[s - 1] if s > 0 else -1
    nxt = ranks[s + 1] if s + 1 < len(ranks) else -1
    return prev, nxt


def _sync_tied_embedding_grads(model) -> None:
    """First and last stage both hold the embedding matrix when it is tied: sum their gradients."""
    cfg = model.cfg
    if cfg.no_weight_tying or model.num_stages == 1:
        return
    if model.stage not in (0, model.num_stages - 1):
        return
    ranks = state.get_pipe_parallel_ranks()
    w = model.embedding.word_embeddings.weight
    peer = ranks[-1] if model.stage == 0 else ranks[0]
    mine = w.grad.detach().clone()
    other = torch.empty_like(mine)
    ops = [dist.P2POp(dist.isend, mine, peer), dist.P2POp(dist.irecv, other, peer)]
    for r in dist.batch_isend_irecv(ops):
        r.wait()
    w.grad.add_(other)


def pipeline_train_step(trainer, data_iterator) -> torch.Tensor:
    cfg, model, dev = trainer.cfg, trainer.model, trainer.device
    prev, nxt = _neighbours()
    first, last = prev < 0, nxt < 0
    B, L, D = cfg.train_micro_batch_size_per_gpu, cfg.seq_length, cfg.hidden_size
    if cfg.sequence_parallel and state.get_model_parallel_world_size() > 1:
        L = L // state.get_model_parallel_world_size()
    dtype = cfg.params_dtype
    model.train()
    trainer.optimizer.zero_grad()
    saved: List[Tuple[torch.Tensor, torch.Tensor]] = []
    total = torch.zeros((), device=dev)
    gas = trainer.gas
    for _ in range(gas):
        b = batch_mod.get_batch(cfg, data_iterator, dev) if (first or last) else None
        if first:
            tokens = b["tokens"]
            if cfg.to_upper in ("upper", "weighted", "normalized_weighted"):
                tokens = batch_mod.to_upper_bytes(tokens)
            x_in = None
            out = model(tokens, b["positions"], return_hidden=not last)
        else:
            x_in = torch.empty((B, L, D), dtype=dtype, device=dev)
            dist.recv(x_in, prev)
            x_in.requires_grad_()
            positions = b["positions"] if b is not None else torch.arange(cfg.seq_length, device=dev)
            out = model(None, positions, hidden_in=x_in, return_hidden=not last)
        if last:
            loss = trainer.compute_loss(out, b)
            total += loss.detach()
            out = loss / gas
        else:
            dist.send(out.detach().contiguous(), nxt)
        saved.append((x_in, out))
    for x_in, out in reversed(saved):
        if last:
            out.backward()
        else:
            g = torch.empty_like(out)
            dist.recv(g, nxt)
            out.backward(g)
        if not first:
            dist.send(x_in.grad.contiguous(), prev)
    _sync_tied_embedding_grads(model)
    trainer._sync_replicated_grads()
    trainer.grad_norm = trainer.optimizer.step()
    trainer.lr_scheduler.step()
    trainer.iteration += 1
    trainer.tokens_seen += cfg.train_batch_size * cfg.seq_length
    # everyone reports the last stage's loss
    loss = total / gas
    ranks = state.get_pipe_parallel_ranks()
    dist.broadcast(loss, ranks[-1], group=state.get_pipe_parallel_group())
    return trainer._reduce_loss(loss)
