"""Autoregressive text generation for evaluation and sampling.

`stream_tokens` re-runs the model on the growing context (the "recompute" mode of the reference,
savanna/text_generation_utils.py:173-365) with temperature / top-k / top-p sampling; `generate(..., use_cache=True)`
decodes with per-layer cached state instead (inference/cached.py: FIR tails, modal states, key/value cache), one
constant-time step per token.  Drivers for a single prompt, a prompt file, unconditional samples and an interactive
prompt loop mirror savanna/text_generation_utils.py:368-774 and savanna/inference/generation.py.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Dict, Iterator, List, Optional

import torch
import torch.nn.functional as F


@dataclass
class InferenceParams:
    max_seqlen: int
    max_batch_size: int
    seqlen_offset: int = 0
    batch_size_offset: int = 0
    key_value_memory_dict: Dict = field(default_factory=dict)
    lengths_per_sample: Optional[torch.Tensor] = None

    def reset(self, max_seqlen, max_batch_size):
        self.max_seqlen, self.max_batch_size, self.seqlen_offset = max_seqlen, max_batch_size, 0
        if self.lengths_per_sample is not None:
            self.lengths_per_sample.zero_()


def filter_logits(logits: torch.Tensor, top_k: int = 0, top_p: float = 0.0, filter_value: float = -float("inf")):
    """Top-k then nucleus filtering on [B, V] logits."""
    if top_k > 0:
        kth = torch.topk(logits, min(top_k, logits.shape[-1]))[0][..., -1, None]
        logits = logits.masked_fill(logits < kth, filter_value)
    if top_p > 0.0:
        sorted_logits, idx = torch.sort(logits, descending=True, dim=-1)
        cum = torch.cumsum(F.softmax(sorted_logits, dim=-1), dim=-1)
        remove = cum > top_p
        remove[..., 1:] = remove[..., :-1].clone()
        remove[..., 0] = False
        mask = torch.zeros_like(remove).scatter(-1, idx, remove)
        logits = logits.masked_fill(mask, filter_value)
    return logits


def sample_tokens(logits: torch.Tensor, temperature: float = 0.0, top_k: int = 0, top_p: float = 0.0, generator=None):
    if temperature == 0.0 and top_k == 0 and top_p == 0.0:
        return logits.argmax(dim=-1)
    logits = logits.float() / max(temperature, 1e-6)
    probs = F.softmax(filter_logits(logits, top_k, top_p), dim=-1)
    return torch.multinomial(probs, 1, generator=generator).squeeze(-1)


@torch.no_grad()
def stream_tokens(model, context_tokens: List[List[int]], eos_token_id: Optional[int] = None, maximum_tokens: int = 64,
                  temperature: float = 0.0, top_k: int = 0, top_p: float = 0.0, pad_id: int = 1,
                  max_seq_len: Optional[int] = None, generator=None) -> Iterator:
    """Yields (tokens [B, T], lengths [B], logits of the step, finished mask) after every generated token."""
    device = next(model.parameters()).device
    B = len(context_tokens)
    lens = torch.tensor([len(c) for c in context_tokens], device=device)
    limit = int(lens.max()) + maximum_tokens
    if max_seq_len is not None:
        limit = min(limit, max_seq_len)
    toks = torch.full((B, limit), pad_id, dtype=torch.long, device=device)
    for i, c in enumerate(context_tokens):
        toks[i, : len(c)] = torch.tensor(c, device=device)
    done = torch.zeros(B, dtype=torch.bool, device=device)
    cur = int(lens.min())
    was_training = model.training
    model.eval()
    try:
        while cur < limit and not bool(done.all()):
            logits = model(toks[:, :cur])[:, -1].float()
            nxt = sample_tokens(logits, temperature, top_k, top_p, generator)
            started = lens <= cur                      # rows whose prompt has been consumed take the sampled token
            new = torch.where(started & ~done, nxt, toks[:, cur])
            toks[:, cur] = new
            if eos_token_id is not None:
                just_done = started & (new == eos_token_id)
                done |= just_done
            cur += 1
            gen_len = torch.where(done, torch.minimum(lens.new_full((), cur), lens.new_full((B,), cur)), lens.new_full((B,), cur))
            yield toks[:, :cur], gen_len, logits, done
    finally:
        model.train(was_training)


def _generate_cached(model, tokenizer, prompts, ctx, maximum_tokens, temperature, top_k, top_p, eos_token_id, return_logits):
    """Cached decoding; prompts are grouped by length so that each group shares one prefill."""
    from .cached import stream_tokens_cached
    out: List[Optional[Dict]] = [None] * len(prompts)
    by_len: Dict[int, List[int]] = {}
    for i, c in enumerate(ctx):
        by_len.setdefault(len(c), []).append(i)
    for n, idxs in by_len.items():
        toks, steps, done_at = None, [], [None] * len(idxs)
        for toks, logits, done in stream_tokens_cached(model, [ctx[i] for i in idxs], eos_token_id, maximum_tokens,
                                                       temperature, top_k, top_p):
            steps.append(logits.cpu() if return_logits else None)
            for j in range(len(idxs)):
                if done_at[j] is None and bool(done[j]):
                    done_at[j] = toks.shape[1]
        for j, i in enumerate(idxs):
            end = done_at[j] if done_at[j] is not None else toks.shape[1]
            gen = toks[j, n:end].tolist()
            rec = {"context": prompts[i], "text": tokenizer.detokenize(gen), "length": len(gen)}
            if return_logits:
                rec["logits"] = torch.stack([l[j] for l in steps])
            out[i] = rec
    return out


def generate(model, tokenizer, prompts: List[str], maximum_tokens: int = 64, temperature: float = 0.0, top_k: int = 0,
             top_p: float = 0.0, eos_token_id: Optional[int] = None, return_logits: bool = False,
             use_cache: bool = False) -> List[Dict]:
    ctx = [tokenizer.tokenize(p) or [tokenizer.eod] for p in prompts]
    if use_cache:
        try:
            return _generate_cached(model, tokenizer, prompts, ctx, maximum_tokens, temperature, top_k, top_p, eos_token_id,
                                    return_logits)
        except NotImplementedError as exc:
            print(f"cached generation unavailable for this model ({exc}); recomputing the context every step")
    last = None
    all_logits = []
    for last in stream_tokens(model, ctx, eos_token_id, maximum_tokens, temperature, top_k, top_p,
                              pad_id=getattr(tokenizer, "pad", 1)):
        if return_logits:
            all_logits.append(last[2].cpu())
    out = []
    if last is None:
        return out
    toks, lengths, _, _ = last
    for i, p in enumerate(prompts):
        gen = toks[i, len(ctx[i]): int(lengths[i])].tolist()
        rec = {"context": p, "text": tokenizer.detokenize(gen), "length": len(gen)}
        if return_logits:
            rec["logits"] = torch.stack([l[i] for l in all_logits])
        out.append(rec)
    return out


def generate_samples_from_prompt(model, cfg, text, **kw) -> List[Dict]:
    prompts = [text] if isinstance(text, str) else list(text)
    return generate(model, cfg.tokenizer, prompts, maximum_tokens=kw.get("maximum_tokens", cfg.maximum_tokens),
                    temperature=kw.get("temperature", cfg.temperature), top_k=kw.get("top_k", cfg.top_k),
                    top_p=kw.get("top_p", cfg.top_p), eos_token_id=kw.get("eos_token_id"),
                    return_logits=cfg.return_logits, use_cache=kw.get("use_cache", not bool(cfg.recompute)))


def generate_samples_input_from_file(model, cfg, input_file: str, output_file: Optional[str] = None, **kw):
    # prompts are separated by `prompt_end` (a newline unless configured; other separators allow multi-line prompts)
    sep = kw.pop("prompt_end", None) or cfg.prompt_end or "\n"
    with open(input_file, encoding="utf-8") as fh:
        prompts = [p.strip() for p in fh.read().split(sep)]
    prompts = [p for p in prompts if p]
    results = generate_samples_from_prompt(model, cfg, prompts, **kw)
    if output_file:
        with open(output_file, "w") as fh:
            for r in results:
                r = {k: v for k, v in r.items() if k != "logits"}
                fh.write(json.dumps(r) + "\n")
    return results


def generate_samples_unconditional(model, cfg, number_of_samples: int = 1, output_file: Optional[str] = None, **kw):
    eod = cfg.tokenizer.eod
    prompts = [cfg.tokenizer.detokenize([eod])] * number_of_samples
    results = generate_samples_from_prompt(model, cfg, prompts, **kw)
    if output_file:
        with open(output_file, "w") as fh:
            for r in results:
                fh.write(json.dumps({k: v for k, v in r.items() if k != "logits"}) + "\n")
    return results


def generate_samples_interactive(model, cfg, input_fn=input, print_fn=print, **kw) -> None:
    """Prompt loop on the terminal (reference: text_generation_utils.py:672-774): read a context, stream the
    continuation as it is generated, repeat until an empty line, "stop" or end of input.  With several ranks only
    rank 0 talks to the terminal; the others would need the prompt broadcast, so this driver runs single-process."""
    tok = cfg.tokenizer
    use_cache = kw.get("use_cache", not bool(cfg.recompute))
    while True:
        try:
            text = input_fn("Context prompt >>> ")
        except EOFError:
            break
        if not text.strip() or text.strip().lower() == "stop":
            break
        ctx = [tok.tokenize(text) or [tok.eod]]
        shown = 0
        stream = None
        if use_cache:
            try:
                from .cached import CachedDecoder, stream_tokens_cached
                CachedDecoder(model)                      # raises when the model has no cached form
                stream = ((t, None, None, d) for t, _, d in stream_tokens_cached(
                    model, ctx, kw.get("eos_token_id"), kw.get("maximum_tokens", cfg.maximum_tokens),
                    kw.get("temperature", cfg.temperature), kw.get("top_k", cfg.top_k), kw.get("top_p", cfg.top_p)))
            except NotImplementedError:
                stream = None
        if stream is None:
            stream = stream_tokens(model, ctx, kw.get("eos_token_id"), kw.get("maximum_tokens", cfg.maximum_tokens),
                                   kw.get("temperature", cfg.temperature), kw.get("top_k", cfg.top_k), kw.get("top_p", cfg.top_p))
        for toks, _, _, _ in stream:
            gen = toks[0, len(ctx[0]):].tolist()
            piece = tok.detokenize(gen)
            print_fn(piece[shown:], end="", flush=True)
            shown = len(piece)
        print_fn("")
