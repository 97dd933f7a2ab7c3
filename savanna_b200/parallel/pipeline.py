"""Pipeline parallelism over point-to-point messages (NCCL on GPUs, gloo on CPU).

Each stage owns a contiguous range of blocks (`Backbone(layer_range=...)`); the first stage also owns the
embedding, the last stage the final norm and the logits (with tied embeddings it holds a copy of the
embedding whose gradient is all-reduced with the first stage's after every step).  One optimizer step runs
the `gradient_accumulation_steps` micro-batches through the one-forward-one-backward (1F1B) schedule, so a stage
holds the activations of at most `stages - stage` micro-batches; activations and their gradients travel as
[B, L, D] tensors, the two directions of a steady-state exchange posted together.  Role of the reference's DeepSpeed PipelineModule /
PipelineEngine use (savanna/model/backbone.py:219-284, savanna/training.py:1517-1546).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ..train import batch as batch_mod
from . import state


def stage_layer_range(num_layers: int, pp: int, stage: int) -> range:
    base, rem = divmod(num_layers, pp)
    start = stage * base + min(stage, rem)
    return range(start, start + base + (1 if stage < rem else 0))


def balanced_layer_ranges(weights: List[float], pp: int, first_extra: float = 0.0, last_extra: float = 0.0) -> List[range]:
    """Cut the layers into `pp` contiguous, non-empty runs so that the heaviest run is as light as possible
    (`first_extra` / `last_extra`: what the first and the last stage carry besides their layers: embedding, final norm
    and output head).  Dynamic programme over prefix sums; a few hundred layers at most."""
    n = len(weights)
    if pp > n:
        raise ValueError(f"{pp} pipeline stages for {n} layers")
    pre = [0.0]
    for w in weights:
        pre.append(pre[-1] + float(w))

    def cost(a, b, k):                       # layers a..b-1 as stage k
        return pre[b] - pre[a] + (first_extra if k == 0 else 0.0) + (last_extra if k == pp - 1 else 0.0)
    inf = float("inf")
    best = [[inf] * (n + 1) for _ in range(pp + 1)]
    cut = [[0] * (n + 1) for _ in range(pp + 1)]
    best[0][0] = 0.0
    for k in range(1, pp + 1):
        for b in range(k, n - (pp - k) + 1):
            for a in range(k - 1, b):
                if best[k - 1][a] == inf:
                    continue
                c = max(best[k - 1][a], cost(a, b, k - 1))
                if c < best[k][b]:
                    best[k][b], cut[k][b] = c, a
    out, b = [], n
    for k in range(pp, 0, -1):
        a = cut[k][b]
        out.append(range(a, b))
        b = a
    return out[::-1]


def partition_layers(cfg, pp: int) -> List[range]:
    """Layer range of every stage under `pipe_partition_method` (the methods of DeepSpeed's PipelineModule, which the
    reference forwards this key to, savanna/model/backbone.py:281): `type:<class regex>` and `uniform` spread the blocks
    evenly (the reference's default `type:ParallelBlockPipe` balances exactly the blocks); `parameters` balances the
    parameter count, embedding and output head included, measured on a meta-device copy of the model."""
    method = str(cfg.pipe_partition_method or "type:ParallelBlockPipe").lower()
    if method.startswith("type:") or method == "uniform":
        return [stage_layer_range(cfg.num_layers, pp, s) for s in range(pp)]
    if method == "parameters":
        from ..models.backbone import Backbone
        meta = Backbone(cfg, device=torch.device("meta"))
        per_block = [sum(p.numel() for p in b.parameters()) for b in meta.blocks()]
        total = sum(p.numel() for p in meta.parameters())
        emb = sum(p.numel() for p in meta.embedding.parameters())
        tail = total - emb - sum(per_block)                       # final norm and, untied, the output head
        if not cfg.no_weight_tying:
            tail += emb                                           # the last stage holds a copy of the tied embedding
        return balanced_layer_ranges(per_block, pp, first_extra=emb, last_extra=tail)
    raise ValueError(f"pipe_partition_method {cfg.pipe_partition_method!r} unknown (type:<regex> | uniform | parameters)")


def build_pipeline_stage(cfg, device):
    from ..models.backbone import Backbone
    pp, stage = state.get_pipe_parallel_world_size(), state.get_pipe_parallel_rank()
    model = Backbone(cfg, device=device, layer_range=partition_layers(cfg, pp)[stage])
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


def _exchange(send: Optional[torch.Tensor], send_to: int, recv_like: Optional[Tuple], recv_from: int):
    """One batched point-to-point round: optionally send `send` to `send_to` and receive a tensor of shape / dtype
    `recv_like` from `recv_from`.  Both directions are posted together (`batch_isend_irecv`), which is what lets two
    neighbouring stages swap an activation and a gradient without ordering their blocking calls."""
    ops, buf = [], None
    if send is not None and send_to >= 0:
        ops.append(dist.P2POp(dist.isend, send.contiguous(), send_to))
    if recv_like is not None and recv_from >= 0:
        shape, dtype, dev = recv_like
        buf = torch.empty(shape, dtype=dtype, device=dev)
        ops.append(dist.P2POp(dist.irecv, buf, recv_from))
    if ops:
        for r in dist.batch_isend_irecv(ops):
            r.wait()
    return buf


def pipeline_train_step(trainer, data_iterator) -> torch.Tensor:
    """One optimizer step on the 1F1B schedule: stage s runs `pp - 1 - s` warm-up forwards, then alternates one
    forward with one backward, then drains its remaining backwards.  At most `pp - s` micro-batches' activations are
    alive on a stage, whatever the accumulation depth (the all-forward / all-backward order keeps all of them)."""
    cfg, model, dev = trainer.cfg, trainer.model, trainer.device
    prev, nxt = _neighbours()
    first, last = prev < 0, nxt < 0
    B, L, D = cfg.train_micro_batch_size_per_gpu, cfg.seq_length, cfg.hidden_size
    if state.get_context_parallel_world_size() > 1:
        L = L // state.get_context_parallel_world_size()
    if cfg.sequence_parallel and state.get_model_parallel_world_size() > 1:
        L = L // state.get_model_parallel_world_size()
    act = ((B, L, D), cfg.params_dtype, dev)
    model.train()
    trainer.optimizer.zero_grad()
    total = torch.zeros((), device=dev)
    gas = trainer.gas
    pp, stage = model.num_stages, model.stage
    warmup = min(pp - stage - 1, gas)
    steady = gas - warmup
    live: List[Tuple[Optional[torch.Tensor], torch.Tensor]] = []      # (stage input, stage output) awaiting backward
    trainer.pipeline_peak_live = 0

    def forward(x_in):
        nonlocal total
        b = batch_mod.get_batch(cfg, data_iterator, dev) if (first or last) else None
        if first:
            tokens = b["tokens"]
            if cfg.to_upper in ("upper", "weighted", "normalized_weighted"):
                tokens = batch_mod.to_upper_bytes(tokens)
            out = model(tokens, b["positions"], return_hidden=not last)
        else:
            x_in.requires_grad_()
            positions = b["positions"] if b is not None else torch.arange(L, device=dev)
            out = model(None, positions, hidden_in=x_in, return_hidden=not last)
        if last:
            loss = trainer.compute_loss(out, b)
            total += loss.detach()
            out = loss / gas
        live.append((x_in, out))
        trainer.pipeline_peak_live = max(trainer.pipeline_peak_live, len(live))
        return out

    def backward(g):
        x_in, out = live.pop(0)
        if last:
            out.backward()
        else:
            out.backward(g)
        return None if first else x_in.grad

    x_in = None
    for _ in range(warmup):
        x_in = _exchange(None, -1, act, prev)
        out = forward(x_in)
        _exchange(out.detach(), nxt, None, -1)
    if steady > 0:
        x_in = _exchange(None, -1, act, prev)
    for i in range(steady):
        out = forward(x_in)
        g = _exchange(None if last else out.detach(), nxt, None if last else act, nxt)
        dx = backward(g)
        if i == steady - 1:
            _exchange(dx, prev, None, -1)
        else:
            x_in = _exchange(dx, prev, act, prev)
    for _ in range(warmup):
        g = _exchange(None, -1, act, nxt)
        dx = backward(g)
        _exchange(dx, prev, None, -1)
    _sync_tied_embedding_grads(model)
    trainer._sync_replicated_grads()
    trainer.grad_norm = trainer.optimizer.step()
    trainer.lr_scheduler.step()
    trainer.iteration += 1
    trainer.tokens_seen += cfg.train_batch_size * cfg.seq_length
    if trainer.watchdog is not None:
        trainer.watchdog.beat(trainer.iteration)
    # everyone reports the last stage's loss
    loss = total / gas
    ranks = state.get_pipe_parallel_ranks()
    dist.broadcast(loss, ranks[-1], group=state.get_pipe_parallel_group())
    return trainer._reduce_loss(loss)
