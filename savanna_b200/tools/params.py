"""Tensor-parallel partition dimension of every checkpoint key (reference table:
tools/7b/conversion/params.py:10-42).  None = replicated."""
from __future__ import annotations

import re
from typing import Optional

_RULES = [
    (r"word_embeddings\.weight$", 0),
    (r"(input|post_attention|pre_mlp|outer_mlp)_layernorm\.(weight|scale|bias)$", None),
    (r"mixer\.dense_projection\.weight$", 0),
    (r"mixer\.dense_projection\.bias$", 0),
    (r"hyena_proj_conv\.short_conv_weight$", 0),
    (r"mixer\.mixer\.conv_bias$", 0),
    (r"mixer\.mixer\.filter\.(h|decay|gamma|R|p)$", 0),           # 3-d R / p of the real modal filter: see partition_dim
    (r"mixer\.mixer\.filter\.dt$", 1),
    (r"mixer\.mixer\.filter\.inner_cls\.(log_dt|inv_A_real|A_imag|B)$", 0),
    (r"mixer\.mixer\.filter\.inner_cls\.C$", 1),
    (r"mixer\.mixer\.filter\.t$", None),
    (r"mixer\.mixer\.short_conv\.short_conv_weight$", 0),
    (r"rotary_emb\.inv_freq$", None),
    (r"mixer\.dense\.weight$", 1),
    (r"mixer\.dense\.bias$", None),
    (r"mlp\.w1\.weight$", 0),
    (r"mlp\.w2\.weight$", 0),
    (r"mlp\.w3\.weight$", 1),
    (r"mlp\.dense_projection\.weight$", 0),
    (r"mlp\.dense\.weight$", 1),
    (r"mlp\.dense\.bias$", None),
    (r"mlp\.dense_h_to_4h\.(weight|bias)$", 0),
    (r"mlp\.dense_4h_to_h\.weight$", 1),
    (r"mlp\.dense_4h_to_h\.bias$", None),
    (r"norm\.(weight|scale|bias)$", None),
    (r"final_linear\.weight$", 0),
    (r"_extra_state$", None),
]


def partition_dim(key: str, ndim: Optional[int] = None) -> Optional[int]:
    """`ndim` (the tensor's rank, when the caller has it) tells the factored real modal filter's `R` / `p`
    [order, channels, factors], split along dimension 1, from the modal filter's [channels, order]."""
    if ndim == 3 and re.search(r"mixer\.mixer\.filter\.(R|p)$", key):
        return 1
    for pat, dim in _RULES:
        if re.search(pat, key):
            return dim
    return None


def is_known(key: str) -> bool:
    return any(re.search(p, key) for p, _ in _RULES)
