"""tcgen05 flash attention front-end (kernels: csrc/attn_sm100.cu)."""
from __future__ import annotations


def supported(q, k, v, causal) -> bool:
    return False


def attention(q, k, v, causal, return_lse=False):
    raise NotImplementedError
