"""Token embedding (+ optional learned / sinusoidal positions) with sequence-parallel scatter
(reference: savanna/model/operators/word_embeddings.py:9-227)."""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from ..parallel import mappings, state
from ..parallel.layers import VocabParallelEmbedding


class SinusoidalPositionalEmbedding(nn.Module):
    def __init__(self, dim: int, base: float = 10000.0):
        super().__init__()
        self.register_buffer("inv_freq", 1.0 / (base ** (torch.arange(0, dim, 2).float() / dim)))

    def forward(self, positions, dtype):
        ang = torch.outer(positions.float(), self.inv_freq)
        return torch.cat([ang.sin(), ang.cos()], dim=-1).to(dtype)[None]


class Embedding(nn.Module):
    """Word embedding + optional learned / sinusoidal positions + optional token-type embeddings (`num_tokentypes`
    segment ids, word_embeddings.py:88-136: built at construction or added later with `add_tokentype_embeddings`)."""

    def __init__(self, cfg, init_method, dtype=None, device=None, num_tokentypes: int = 0):
        super().__init__()
        self.cfg = cfg
        self._init_method, self._dtype = init_method, dtype
        self.num_tokentypes = 0
        self.tokentype_embeddings = None
        if num_tokentypes > 0:
            self._build_tokentypes(num_tokentypes, device)
        self.word_embeddings = VocabParallelEmbedding(cfg.padded_vocab_size, cfg.hidden_size, init_method, dtype, device)
        self.pos_kind = cfg.pos_emb
        if cfg.pos_emb == "learned":
            self.position_embeddings = nn.Embedding(cfg.max_position_embeddings, cfg.hidden_size, dtype=dtype, device=device)
            nn.init.normal_(self.position_embeddings.weight, std=cfg.init_method_std)
        elif cfg.pos_emb == "sinusoidal":
            self.position_embeddings = SinusoidalPositionalEmbedding(cfg.hidden_size)
        self.dropout = nn.Dropout(cfg.hidden_dropout)
        self.sequence_parallel = cfg.sequence_parallel and state.get_model_parallel_world_size() > 1
        self.mup_mult = cfg.mup_embedding_mult if cfg.use_mup else 1.0
        self.pos_mult = float(cfg.mup_rp_embedding_mult)      # multiplier of the position embeddings (word_embeddings.py:128)

    def _build_tokentypes(self, n: int, device) -> None:
        self.num_tokentypes = n
        self.tokentype_embeddings = nn.Embedding(n, self.cfg.hidden_size, dtype=self._dtype, device=device)
        self._init_method(self.tokentype_embeddings.weight)

    def add_tokentype_embeddings(self, num_tokentypes: int) -> None:
        """Add token-type embeddings to a model that was built (or pretrained) without them."""
        if self.tokentype_embeddings is not None:
            raise RuntimeError("tokentype embeddings are already initialised")
        self._build_tokentypes(num_tokentypes, self.word_embeddings.weight.device)

    def forward(self, ids: torch.Tensor, positions: torch.Tensor, tokentype_ids: torch.Tensor = None) -> torch.Tensor:
        x = self.word_embeddings(ids)
        if tokentype_ids is not None:
            if self.tokentype_embeddings is None:
                raise RuntimeError("tokentype ids given to a model without tokentype embeddings")
            x = x + self.tokentype_embeddings(tokentype_ids)
        if self.pos_kind == "learned":
            x = x + self.position_embeddings(positions + self.cfg.opt_pos_emb_offset)[None] * self.pos_mult
        elif self.pos_kind == "sinusoidal":
            x = x + self.position_embeddings(positions, x.dtype) * self.pos_mult
        if self.mup_mult != 1.0:
            x = x * self.mup_mult
        x = self.dropout(x)
        if self.sequence_parallel:
            x = mappings.scatter_to_sequence_parallel_region(x, 1)
        return x


class SoftEmbedding(nn.Module):
    """Prompt-tuning prefix (word_embeddings.py:172-227): `n_tokens` learned vectors prepended."""

    def __init__(self, cfg, wte, n_tokens: int = 10, init_range: float = 0.5, init_string: str = ""):
        super().__init__()
        self.n_tokens = n_tokens
        if init_string:
            ids = torch.tensor(cfg.tokenizer.tokenize(init_string))[:n_tokens]
            emb = wte(ids.to(wte.weight.device)).detach().float()
            if emb.shape[0] < n_tokens:
                emb = emb.repeat(math.ceil(n_tokens / emb.shape[0]), 1)[:n_tokens]
        else:
            emb = torch.empty(n_tokens, cfg.hidden_size).uniform_(-init_range, init_range)
        self.soft_embedding_weight = nn.Parameter(emb)

    def forward(self, x):
        pre = self.soft_embedding_weight.to(x.dtype)[None].expand(x.shape[0], -1, -1)
        return torch.cat([pre, x], dim=1)[:, : x.shape[1]]
