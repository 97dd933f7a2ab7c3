"""Batch builders: turn a `[B, L+1]` token block into model inputs, labels and a loss mask.

Strategies (reference: savanna/training.py:637-927, masks in savanna/utils.py:144-440):
  AR      next-token prediction; tokens = text[:, :-1], labels = text[:, 1:]
  MLM     15 % of the positions become the mask token '_' (95); of those ~10 % get a random token, ~10 % their own back
  SPAN    spans of geometric length are masked until 15 % of the tokens are drawn; SPAN_R adds the random / restore step
  OADM    order-agnostic diffusion: a uniformly drawn number of uniformly placed positions is masked
The labels are the uncorrupted tokens and the loss counts the masked positions only.
Under context parallelism every tensor is zigzag-split along the sequence after the broadcast.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..parallel import broadcast_data, state, zigzag_indices


def to_upper_bytes(tokens: torch.Tensor) -> torch.Tensor:
    """a..z -> A..Z on byte tokens (utils.py:77-87)."""
    lower = (tokens >= 97) & (tokens <= 122)
    return torch.where(lower, tokens - 32, tokens)


MASK_TOKEN_ID = 95          # '_' : the mask token of the byte-level vocabulary (reference: savanna/utils.py:207, 277, 349)
CONTROL_TAGS = (64, 35)     # '@' splice / window splits, '#' contig splits
TAG_DELIMITER = 124         # '|' opens and closes a phylogenetic tag
TAG_ONLY_CHARS = (95, 59, 32)   # '_', ';', ' ' occur inside tags only


def mask_control_tags(tokens: torch.Tensor, loss_mask: torch.Tensor, eod: int) -> torch.Tensor:
    """Zero the loss on Evo 2 control characters and phylogenetic tags (reference: savanna/utils.py:387-440).

    '@' and '#' never count.  For the tags, every row is cut at its '|' characters, its end-of-document tokens, its
    first and its last position; a piece [d_j, d_j+1) that holds one of the tag-only characters '_', ';', ' ' is a tag
    (whole, or the part of one that a sample boundary left over) and is masked together with both delimiters, except
    that an end-of-document token at either end keeps its loss.  Pieces without such a character are sequence and keep
    theirs.  Vectorised: no loop over rows, no host synchronisation.  (The reference's loop restarts one position early
    after a tag that ends at an end-of-document token; that only matters for a tag left open right before the token and
    is not reproduced.)"""
    B, L = tokens.shape
    pos = torch.arange(L, device=tokens.device)
    is_eod = tokens == eod
    delim = (tokens == TAG_DELIMITER) | is_eod | (pos == 0)[None] | (pos == L - 1)[None]
    piece = torch.cumsum(delim.int(), dim=-1) - 1                         # index j of the piece a position opens or lies in
    tagc = torch.zeros_like(delim)
    for c in TAG_ONLY_CHARS:
        tagc |= tokens == c
    tagc = tagc & (pos != L - 1)[None]                                     # the last position opens no piece of its own
    has_tag = torch.zeros(B, L + 1, dtype=torch.int32, device=tokens.device)
    has_tag.scatter_reduce_(1, piece.long(), tagc.int(), reduce="amax", include_self=True)
    own = has_tag.gather(1, piece.long()) > 0                              # T_j at every position of piece j
    prev = has_tag.gather(1, (piece - 1).clamp_min(0).long()) > 0
    prev = prev & (piece > 0)
    in_tag = torch.where(delim, (own | prev) & ~is_eod, own)
    control = torch.zeros_like(delim)
    for c in CONTROL_TAGS:
        control |= tokens == c
    keep = ~(in_tag | control)
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


def _dna_only(tokens: torch.Tensor) -> torch.Tensor:
    """Everything but A, C, G, T, end-of-document (0) and '0' becomes token 1 (reference: savanna/utils.py:66-75, applied to
    span-masking batches)."""
    ok = torch.zeros_like(tokens, dtype=torch.bool)
    for c in (65, 84, 67, 71, 0, 48):
        ok |= tokens == c
    return torch.where(ok, tokens, torch.ones_like(tokens))


def _randomize_and_unmask(out, clean, sel, vocab, random_percent=0.1, unmask_percent=0.1, gen=None):
    """Of the selected positions, ~10 % get a random token and ~10 % (drawn independently, applied last) get their
    original token back; the rest keep the mask token (savanna/utils.py:122-141)."""
    dev = out.device
    rnd_sel = (torch.rand(out.shape, device=dev, generator=gen) < random_percent) & sel
    keep_sel = (torch.rand(out.shape, device=dev, generator=gen) < unmask_percent) & sel
    rnd = torch.randint(0, vocab, out.shape, device=dev, generator=gen)
    out = torch.where(rnd_sel, rnd, out)
    return torch.where(keep_sel, clean, out)


def _mlm_corrupt(tokens, vocab, eod=None, pad=None, eod_mask_loss=False, pad_mask_loss=False, prob=0.15, gen=None):
    """Masked-language-model batch (savanna/utils.py:181-247): ceil(prob * L) distinct positions per row, minus
    end-of-document / pad positions when their loss is masked, become '_'; then 10 % random / 10 % restored.  The loss
    counts the selected positions only."""
    B, L = tokens.shape
    n = max(1, math.ceil(prob * L))
    idx = torch.rand((B, L), device=tokens.device, generator=gen).topk(n, dim=-1).indices
    sel = torch.zeros((B, L), dtype=torch.bool, device=tokens.device)
    sel.scatter_(1, idx, True)
    if eod_mask_loss and eod is not None:
        sel &= tokens != eod
    if pad_mask_loss and pad is not None:
        sel &= tokens != pad
    out = torch.where(sel, torch.full_like(tokens, MASK_TOKEN_ID), tokens)
    out = _randomize_and_unmask(out, tokens, sel, vocab, gen=gen)
    return out, sel.float()


def _span_corrupt(tokens, vocab, randomize: bool, eod=None, pad=None, eod_mask_loss=False, pad_mask_loss=False,
                  frac=0.15, p=0.2, max_span=10, gen=None):
    """Span masking (savanna/utils.py:250-331): spans of geometric length (success probability `p`, at most `max_span`)
    at uniform start positions are replaced by '_' until int(frac * L) tokens per row have been drawn (overlaps count
    twice, as in the reference); non-DNA bytes become token 1 first.  `randomize` (strategy SPAN_R) adds the 10 % / 10 %
    random / restored treatment of the masked positions."""
    tokens = _dna_only(tokens)
    B, L = tokens.shape
    target = int(frac * L)
    sel = torch.zeros((B, L), dtype=torch.bool, device=tokens.device)
    # span lengths and starts are drawn on the host (a few dozen per row) and applied with one scatter per row
    cpu_gen = torch.Generator().manual_seed(int(torch.randint(0, 2 ** 31 - 1, (1,), generator=gen).item())) if gen is not None else None
    for b in range(B):
        done = 0
        marks = torch.zeros(L + 1, dtype=torch.int32)
        while done < target:
            u = float(torch.rand((), generator=cpu_gen))
            length = min(int(math.floor(math.log(max(u, 1e-12)) / math.log(1.0 - p))), max_span)   # failures before a success
            length = min(length, target - done)
            start = int(torch.randint(0, L - length + 1, (1,), generator=cpu_gen))
            marks[start] += 1
            marks[start + length] -= 1
            done += length
        sel[b] = (torch.cumsum(marks[:L], 0) > 0).to(tokens.device)
    if pad_mask_loss and pad is not None:
        sel &= tokens != pad
    if eod_mask_loss and eod is not None:
        sel &= tokens != eod
    out = torch.where(sel, torch.full_like(tokens, MASK_TOKEN_ID), tokens)
    if randomize:
        out = _randomize_and_unmask(out, tokens, sel, vocab, gen=gen)
    return out, sel.float()


def _oadm_corrupt(tokens, eod=None, pad=None, eod_mask_loss=False, pad_mask_loss=False, gen=None):
    """Order-agnostic autoregressive diffusion (savanna/utils.py:334-384): per row a time t uniform in [0, L) and a
    uniformly random subset of L - t + 1 positions (at most L) that become '_' and carry the loss."""
    B, L = tokens.shape
    dev = tokens.device
    t = torch.randint(0, L, (B,), device=dev, generator=gen)
    count = (L - t + 1).clamp(max=L)
    order = torch.argsort(torch.rand((B, L), device=dev, generator=gen), dim=1)
    first = torch.arange(L, device=dev)[None] < count[:, None]
    sel = torch.zeros((B, L), dtype=torch.bool, device=dev)
    sel.scatter_(1, order, first)
    if eod_mask_loss and eod is not None:
        sel &= tokens != eod
    if pad_mask_loss and pad is not None:
        sel &= tokens != pad
    out = torch.where(sel, torch.full_like(tokens, MASK_TOKEN_ID), tokens)
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
        # the reference feeds seq_length + 1 tokens to the span and diffusion strategies; here every strategy works on
        # seq_length tokens, the length the kernels and the position tables are built for
        clean = text[:, :-1].contiguous()
        labels = clean
        vocab = cfg.padded_vocab_size or 512
        kw = dict(eod=eod, pad=pad, eod_mask_loss=cfg.eod_mask_loss, pad_mask_loss=cfg.pad_mask_loss, gen=generator)
        if strategy == "MLM":
            tokens, loss_mask = _mlm_corrupt(clean, vocab, **kw)
        elif strategy in ("SPAN", "SPAN_R"):
            tokens, loss_mask = _span_corrupt(clean, vocab, randomize=strategy == "SPAN_R", **kw)
        elif strategy == "OADM":
            tokens, loss_mask, _ = _oadm_corrupt(clean, **kw)
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
