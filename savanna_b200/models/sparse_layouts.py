"""Block-sparse attention layouts of the legacy operators `local`, `sparse_fixed`, `sparse_variable`, `bigbird` and
`bslongformer`.

The reference builds these layers from DeepSpeed's sparsity configurations with `attention="unidirectional"`
(savanna/model/utils.py:249-328): the [L, L] score matrix is cut into `block` x `block` tiles and a 0 / 1 layout
[heads, L / block, L / block] says which tiles exist; inside the existing tiles the usual causal mask applies.  This
module restates the five layout rules and hands the attention layer an additive mask (0 where a score is kept, -inf
elsewhere).  The layer then runs the materialised-score attention of the `global` operator: these operators are kept
for configuration compatibility with older byte-level transformer baselines, not as a fast path.

Rules, for block row r (queries) and block column c (keys), nb = L / block, always c <= r:
    local           c >= r - w // 2                               (w = num_sliding_window_blocks or num_local_blocks)
    sparse_fixed    c in the same window of `num_local_blocks` blocks as r; plus the last `num_global_blocks` block
                    columns of every window, seen by every later row
    sparse_variable windows of the sizes listed in `local_window_blocks` (the last size repeats); plus the block columns
                    `global_block_indices` (or ranges up to `global_block_end_indices`), seen by every later row; plus
                    `num_random_blocks` random earlier columns per row
    bigbird         sliding window w = num_sliding_window_blocks; the first `num_global_blocks` block columns for every
                    row; `num_random_blocks` random earlier columns per row
    bslongformer    sliding window; the block columns `global_block_indices` (or ranges) for every later row
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

SPARSE_OPERATORS = ("local", "sparse_fixed", "sparse_variable", "bigbird", "bslongformer")


def _windows(nb: int, sizes: List[int]):
    start, i = 0, 0
    while start < nb:
        size = max(1, int(sizes[min(i, len(sizes) - 1)]))
        yield start, min(start + size, nb)
        start += size
        i += 1


def _global_columns(indices: List[int], ends: Optional[List[int]], nb: int) -> List[int]:
    cols = []
    if ends is None:
        cols = [int(i) for i in indices if int(i) < nb]
    else:
        if len(ends) != len(indices):
            raise ValueError("global_block_end_indices needs one entry per global_block_indices entry")
        for a, b in zip(indices, ends):
            if int(b) <= int(a):
                raise ValueError("global block ranges need end > start")
            cols += [c for c in range(int(a), min(int(b), nb))]
    return cols


def _random_columns(layout: torch.Tensor, count: int, seed: int) -> None:
    if count <= 0:
        return
    g = torch.Generator().manual_seed(seed)
    nb = layout.shape[0]
    for r in range(nb):
        k = min(count, r + 1)
        cols = torch.randperm(r + 1, generator=g)[:k]
        layout[r, cols] = True


def block_layout(operator_type: str, num_heads: int, num_blocks: int, cfg: Dict) -> torch.Tensor:
    """Boolean [heads, nb, nb] layout of `operator_type` under the `sparsity_config` dictionary `cfg`."""
    nb = num_blocks
    per_head = bool(cfg.get("different_layout_per_head", False))
    out = torch.zeros(num_heads, nb, nb, dtype=torch.bool)
    rows = torch.arange(nb)[:, None]
    cols = torch.arange(nb)[None, :]
    for h in range(num_heads if per_head else 1):
        lay = torch.zeros(nb, nb, dtype=torch.bool)
        if operator_type == "local":
            w = int(cfg.get("num_local_blocks", cfg.get("num_sliding_window_blocks", 4)))
            lay |= cols >= rows - w // 2
        elif operator_type == "sparse_fixed":
            nl, ng = int(cfg.get("num_local_blocks", 4)), int(cfg.get("num_global_blocks", 1))
            patterns = int(cfg.get("num_different_global_patterns", 1))
            if nl % ng:
                raise ValueError("sparse_fixed: num_local_blocks must divide by num_global_blocks")
            if patterns > 1 and not per_head:
                raise ValueError("sparse_fixed: several global patterns need different_layout_per_head")
            if patterns > nl // ng:
                raise ValueError("sparse_fixed: more global patterns than a window has global positions")
            first = nl - (1 + h % patterns) * ng
            for s, e in _windows(nb, [nl]):
                lay[s:e, s:e] = True
                g0 = s + first
                if g0 >= nb:                          # partial last window: its last blocks play the global role
                    g0 = max(s, nb - ng)
                lay[g0:, g0:min(g0 + ng, nb)] = True
        elif operator_type == "sparse_variable":
            for s, e in _windows(nb, list(cfg.get("local_window_blocks", [4]))):
                lay[s:e, s:e] = True
            for c in _global_columns(list(cfg.get("global_block_indices", [0])), cfg.get("global_block_end_indices"), nb):
                lay[c:, c] = True
            _random_columns(lay, int(cfg.get("num_random_blocks", 0)), seed=1234 + h)
        elif operator_type in ("bigbird", "bslongformer"):
            w = int(cfg.get("num_sliding_window_blocks", 3))
            if nb < w:
                raise ValueError(f"{operator_type}: {w} sliding-window blocks for {nb} blocks in the sequence")
            lay |= cols >= rows - w // 2
            if operator_type == "bigbird":
                ng = int(cfg.get("num_global_blocks", 1))
                if nb < ng:
                    raise ValueError(f"bigbird: {ng} global blocks for {nb} blocks in the sequence")
                lay[:, :ng] = True
                _random_columns(lay, int(cfg.get("num_random_blocks", 1)), seed=1234 + h)
            else:
                for c in _global_columns(list(cfg.get("global_block_indices", [0])), cfg.get("global_block_end_indices"), nb):
                    lay[c:, c] = True
        else:
            raise ValueError(f"{operator_type!r} is not a block-sparse operator ({', '.join(SPARSE_OPERATORS)})")
        lay &= cols <= rows                            # unidirectional: no tile above the diagonal
        if per_head:
            out[h] = lay
        else:
            out[:] = lay
    return out


def additive_mask(operator_type: str, num_heads: int, seq_len: int, cfg: Dict, device=None) -> torch.Tensor:
    """[heads, L, L] float mask: 0 on kept scores, -inf on dropped tiles (the causal mask inside kept tiles is the
    attention function's own)."""
    block = int(cfg.get("block", 16))
    if seq_len % block:
        raise ValueError(f"sequence length {seq_len} must divide by the sparsity block size {block}")
    lay = block_layout(operator_type, num_heads, seq_len // block, cfg)
    keep = lay.repeat_interleave(block, dim=1).repeat_interleave(block, dim=2)
    mask = torch.zeros(keep.shape, dtype=torch.float32)
    mask.masked_fill_(~keep, float("-inf"))
    return mask.to(device) if device is not None else mask
