"""Batch builders: turn a `[B, L+1]` token block into model inputs, labels and a loss mask.

Strategies (reference: savanna/training.py:637-927, masks in savanna/utils.py:144-440):
  AR      next-token prediction; tokens = text[:, :-1], labels = text[:, 1:]
  MLM     BERT-style masking: 15% of positions, 80/10/10 mask/random/keep
  SPAN / SPAN_R   contiguous span corruption (span at a random place / at the right end)
  OADM    order-agnostic diffusion: a random fraction of positions is masked
Under context parallelism every tensor is zigzag-split along the sequence after the broadcast.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..parallel import broadcast_data, state, zigzag_indices


def to_upper_bytes(tokens: torch.Tensor) -> torch.Tensor:
    """a..z -> A..Z on byte tokens (utils.py:77-87)."""
    lower = (tokens >= 97) & (tokens <= 122)
    return torch.where(lower, tokens - 32, tokens)


def mask_control_tags(tokens: torch.Tensor, loss_mask: torch.Tensor, eod: int) -> torch.Tensor:
    """Zero the loss on Evo 2 control / phylogenetic tags: spans delimited by '|' (124) and tokens that
    are neither DNA letters nor end-of-document (utils.py:387-440)."""
    bar = tokens == 124
    inside = (torch.cumsum(bar.int(), dim=-1) % 2 == 1) | bar
    dna = torch.zeros_like(bar)
    for c in (65, 67, 71, 84, 78, 97, 99, 103, 116, 110):
        dna |= tokens == c
    keep = (~inside) & (dna | (tokens == eod))
    return loss_mask * keep.to(loss_mask.dtype)


def ltor_masks_and_position_ids(tokens: torch.Tensor, eod: int, eod_mask_loss: bool, pad: Optional[int] = None,
                                pad_mask_loss: bool = False):
    B, L = tokens.shape
    loss_mask = torch.ones((B, L), dtype=torch.float32, device=tokens.device)
    if eod_mask_loss:
        loss_mask[tokens == eod] = 0.0
    if pad_mask_loss and pad is not None:
        loss_mask[tokens == pad] = 0.0
    positions = torch.arange(L, device=tokens.device)
    return loss_mask, positions


def _mlm_corrupt(tokens, vocab, mask_id, prob=0.15, gen=None):
    r = torch.rand(tokens.shape, device=tokens.device, generator=gen)
    sel = r < prob
    r2 = torch.rand(tokens.shape, device=tokens.device, generator=gen)
    out = tokens.clone()
    out[sel & (r2 < 0.8)] = mask_id
    rnd = torch.randint(0, vocab, tokens.shape, device=tokens.device, generator=gen)
    swap = sel & (r2 >= 0.8) & (r2 < 0.9)
    out[swap] = rnd[swap]
    return out, sel.float()


def _span_corrupt(tokens, mask_id, right: bool, frac=0.15, gen=None):
    B, L = tokens.shape
    n = max(1, int(L * frac))
    out, sel = tokens.clone(), torch.zeros_like(tokens, dtype=torch.float32)
    for b in range(B):
        s = L - n if right else int(torch.randint(0, L - n + 1, (1,), generator=gen))
        out[b, s:s + n] = mask_id
        sel[b, s:s + n] = 1.0
    return out, sel


def _oadm_corrupt(tokens, mask_id, gen=None):
    B, L = tokens.shape
    t = torch.rand(B, 1, device=tokens.device, generator=gen).clamp(min=1.0 / L)
    sel = torch.rand(tokens.shape, device=tokens.device, generator=gen) < t
    out = tokens.clone()
    out[sel] = mask_id
    return out, sel.float(), t


def build_batch(cfg, text: torch.Tensor, generator=None) -> Dict[str, torch.Tensor]:
    """text [B, L+1] int64 (already on the compute device)."""
    tok = cfg.tokenizer
    eod = tok.eod if tok is not None else 0
    pad = getattr(tok, "pad", None) if tok is not None else None
    strategy = cfg.pretraining_strategy
    if strategy == "AR":
        tokens, labels = text[:, :-1].contiguous(), text[:, 1:].contiguous()
        loss_mask, positions = ltor_masks_and_position_ids(tokens, eod, cfg.eod_mask_loss, pad, cfg.pad_mask_loss)
    else:
        clean = text[:, :-1].contiguous()
        labels = clean
        mask_id = (cfg.padded_vocab_size or 512) - 1
        if strategy == "MLM":
            tokens, loss_mask = _mlm_corrupt(clean, cfg.padded_vocab_size or 512, mask_id, gen=generator)
        elif strategy in ("SPAN", "SPAN_R"):
            tokens, loss_mask = _span_corrupt(clean, mask_id, right=strategy == "SPAN_R", gen=generator)
        elif strategy == "OADM":
            tokens, loss_mask, _ = _oadm_corrupt(clean, mask_id, gen=generator)
        else:
            raise ValueError(f"pretraining strategy {strategy!r} unknown")
        positions = torch.arange(clean.shape[1], device=clean.device)
    if cfg.mask_loss_control_tags:
        loss_mask = mask_control_tags(labels, loss_mask, eod)
    batch = {"tokens": tokens, "labels": labels, "loss_mask": loss_mask, "positions": positions}
    cp = state.get_context_parallel_world_size()
    if cp > 1:
        idx = zigzag_indices(tokens.shape[1], cp, state.get_context_parallel_rank(), tokens.device)
        batch = {k: (v.index_select(-1, idx) if k != "positions" else v[idx]) for k, v in batch.items()}
    return batch


def build_batch_dpo(cfg, rows: torch.Tensor) -> Dict[str, torch.Tensor]:
    """Preference pairs (reference: training.py:637-724).  `rows` [B, n] float32 in the format written by
    tools/preprocess_data_dpo.py: accept tokens, pad, reject tokens, pad, ref logprob accept, pad, ref logprob reject.
    Returns 2B sequences (all accepted first, then all rejected) padded with eod to `seq_length`, next-token labels, a
    loss mask without the eod padding, and the reference log-probabilities [2B]."""
    if state.get_context_parallel_world_size() > 1:
        raise ValueError("direct-preference batches do not support context parallelism")
    tok = cfg.tokenizer
    pad, eod = tok.pad, tok.eod
    acc, rej, lp_a, lp_r = [], [], [], []
    for row in rows:
        pads = (row == pad).nonzero(as_tuple=True)[0]
        if pads.numel() < 3:
            raise ValueError("malformed preference row: fewer than three pad separators")
        acc.append(row[: pads[0]].long())
        rej.append(row[pads[0] + 1: pads[1]].long())
        lp_a.append(row[pads[1] + 1])
        lp_r.append(row[pads[2] + 1])
    L = cfg.seq_length
    seqs = acc + rej
    if max(int(t.numel()) for t in seqs) > L + 1:
        raise ValueError(f"a preference text is longer than seq_length + 1 = {L + 1}")
    full = torch.full((len(seqs), L + 1), eod, dtype=torch.long, device=rows.device)
    for i, t in enumerate(seqs):
        full[i, : t.numel()] = t
    tokens, labels = full[:, :-1].contiguous(), full[:, 1:].contiguous()
    loss_mask, positions = ltor_masks_and_position_ids(tokens, eod, True, pad, cfg.pad_mask_loss)
    return {"tokens": tokens, "labels": labels, "loss_mask": loss_mask, "positions": positions,
            "ref_logps": torch.stack(lp_a + lp_r).float()}


def get_batch(cfg, data_iterator, device, max_len: Optional[int] = None) -> Dict[str, torch.Tensor]:
    """Fetch from the iterator on the data-reading rank, broadcast to tensor/context peers, build.  `max_len` (the
    sequence-length curriculum's current length) keeps the first `max_len` positions of every sample."""
    tp, cp = state.get_model_parallel_world_size(), state.get_context_parallel_world_size()
    data = next(data_iterator) if data_iterator is not None else None
    if cfg.alignment_method == "dpo":
        if tp == 1 and cp == 1:
            rows = data["text"].to(device, non_blocking=True).float()
        else:
            rows = broadcast_data(["text"], data, torch.float32)["text"].float()
        return build_batch_dpo(cfg, rows)
    if tp == 1 and cp == 1:
        text = data["text"].to(device, non_blocking=True).long()
    else:
        text = broadcast_data(["text"], data, torch.int64)["text"].long()
    if max_len is not None and max_len + 1 < text.shape[1]:
        unit = 2 * cp * (tp if cfg.sequence_parallel else 1)
        if max_len % unit:
            raise ValueError(f"curriculum length {max_len} must divide by {unit} (zigzag context shards x sequence-parallel ranks)")
        text = text[:, : max_len + 1]
    return build_batch(cfg, text)
