"""Tensor-parallel layers: vocab-parallel embedding, column- and row-parallel linear.

Semantics follow savanna/mpu/layers.py:79-191 (embedding), :352-560 (column) and :563-786 (row).
Differences by design:
  * weights are initialised from a full-size master tensor drawn with the same generator on every
    rank and then sliced, so a model is bit-identical for every tensor-parallel size;
  * the row-parallel output is not reshaped to a configured sequence length, so variable sequence
    length works under context parallelism;
  * with sequence parallelism the all-gather -> GEMM and GEMM -> reduce-scatter pairs dispatch to the
    fused peer-memory kernels when they are available for the tensors' device (ops.linear_*).
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from . import mappings, state


def _master_init(full_shape, init_method, partition_dim, dtype, device, stride=1):
    tp, rank = state.get_model_parallel_world_size(), state.get_model_parallel_rank()
    master = torch.empty(full_shape, dtype=torch.float32, device=device)
    init_method(master)
    if tp > 1:
        master = master.chunk(tp, dim=partition_dim)[rank]
    return master.to(dtype).contiguous()


def mark_tp(param, is_parallel: bool, dim: int, stride: int = 1):
    param.model_parallel = is_parallel
    param.partition_dim = dim
    param.partition_stride = stride


class VocabParallelEmbedding(nn.Module):
    def __init__(self, num_embeddings: int, embedding_dim: int, init_method: Callable, dtype=None, device=None):
        super().__init__()
        tp, rank = state.get_model_parallel_world_size(), state.get_model_parallel_rank()
        if num_embeddings % tp:
            raise ValueError("padded vocabulary must be divisible by the tensor-parallel size")
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        per = num_embeddings // tp
        self.vocab_start, self.vocab_end = rank * per, (rank + 1) * per
        self.weight = nn.Parameter(_master_init((num_embeddings, embedding_dim), init_method, 0, dtype, device))
        mark_tp(self.weight, True, 0)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        tp = state.get_model_parallel_world_size()
        if tp == 1:
            return F.embedding(ids, self.weight)
        mask = (ids < self.vocab_start) | (ids >= self.vocab_end)
        local = (ids - self.vocab_start).masked_fill(mask, 0)
        out = F.embedding(local, self.weight)
        out = out.masked_fill(mask.unsqueeze(-1), 0.0)
        return mappings.reduce_from_model_parallel_region(out)


class ColumnParallelLinear(nn.Module):
    """Y = X A^T with A [out, in] split along `out`.  Returns (output, bias-or-None)."""

    def __init__(self, input_size: int, output_size: int, bias: bool = True, gather_output: bool = False,
                 init_method: Callable = nn.init.xavier_normal_, skip_bias_add: bool = False,
                 sequence_parallel: bool = False, seq_dim: int = 1, dtype=None, device=None, fp8: bool = False):
        super().__init__()
        tp = state.get_model_parallel_world_size()
        if output_size % tp:
            raise ValueError(f"output size {output_size} not divisible by tensor-parallel size {tp}")
        self.input_size, self.output_size = input_size, output_size
        self.gather_output, self.skip_bias_add = gather_output, skip_bias_add
        self.sequence_parallel, self.seq_dim, self.fp8 = sequence_parallel and tp > 1, seq_dim, fp8
        self.weight = nn.Parameter(_master_init((output_size, input_size), init_method, 0, dtype, device))
        mark_tp(self.weight, True, 0)
        if bias:
            self.bias = nn.Parameter(torch.zeros(output_size // tp, dtype=dtype, device=device))
            mark_tp(self.bias, True, 0)
        else:
            self.register_parameter("bias", None)

    def forward(self, x: torch.Tensor):
        bias = None if self.skip_bias_add else self.bias
        if self.sequence_parallel:
            y = ops.linear_allgather(x, self.weight, bias, self.seq_dim, fp8=self.fp8)
        else:
            x = mappings.copy_to_model_parallel_region(x) if state.get_model_parallel_world_size() > 1 else x
            y = ops.linear(x, self.weight, bias, fp8=self.fp8)
        if self.gather_output:
            y = mappings.gather_from_model_parallel_region(y)
        return y, (self.bias if self.skip_bias_add else None)

    def forward_normed(self, x: torch.Tensor, norm: nn.Module):
        """Projection of norm(x).  Returns (output, bias-or-None, x for the residual branch).  On one tensor-parallel
        rank an RMSNorm and the projection go through one fused op (ops.norm_linear): with fp8 projections the norm
        kernel writes the fp8 operand itself, and the residual branch's gradient is added in the norm's backward."""
        gain = getattr(norm, "gain", None)
        if gain is not None and state.get_model_parallel_world_size() == 1 and not self.gather_output:
            bias = None if self.skip_bias_add else self.bias
            y, res = ops.norm_linear(x, gain, norm.eps, norm.form, self.weight, bias, fp8=self.fp8)
            return y, (self.bias if self.skip_bias_add else None), res
        fn = getattr(norm, "forward_with_residual", None)
        u, res = fn(x) if fn is not None else (norm(x), x)
        y, b = self.forward(u)
        return y, b, res


class RowParallelLinear(nn.Module):
    """Y = X A^T with A [out, in] split along `in`; partial products are summed over the group."""

    def __init__(self, input_size: int, output_size: int, bias: bool = True, input_is_parallel: bool = True,
                 init_method: Callable = nn.init.xavier_normal_, skip_bias_add: bool = False,
                 parallel_output: bool = False, sequence_parallel: bool = False, seq_dim: int = 1,
                 dtype=None, device=None, fp8: bool = False):
        super().__init__()
        tp = state.get_model_parallel_world_size()
        if input_size % tp:
            raise ValueError(f"input size {input_size} not divisible by tensor-parallel size {tp}")
        self.input_is_parallel, self.skip_bias_add, self.parallel_output = input_is_parallel, skip_bias_add, parallel_output
        self.sequence_parallel, self.seq_dim, self.fp8 = sequence_parallel and tp > 1, seq_dim, fp8
        self.weight = nn.Parameter(_master_init((output_size, input_size), init_method, 1, dtype, device))
        mark_tp(self.weight, True, 1)
        if bias:
            self.bias = nn.Parameter(torch.zeros(output_size, dtype=dtype, device=device))
            mark_tp(self.bias, False, 0)
        else:
            self.register_parameter("bias", None)

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None):
        """With `residual` the layer returns (residual + x A^T + bias, None): on one tensor-parallel rank both
        additions happen in the GEMM epilogue."""
        tp = state.get_model_parallel_world_size()
        if residual is not None:
            if tp == 1 and self.input_is_parallel:
                return ops.linear(x, self.weight, self.bias, fp8=self.fp8, residual=residual), None
            y, b = self.forward(x, None)
            y = y + b if b is not None else y
            return residual + y, None
        if not self.input_is_parallel:
            x = mappings.scatter_to_model_parallel_region(x)
        if self.sequence_parallel and not self.parallel_output:
            y = ops.linear_reducescatter(x, self.weight, self.seq_dim, fp8=self.fp8)
        else:
            y = ops.linear(x, self.weight, None, fp8=self.fp8)
            if tp > 1 and not self.parallel_output:
                y = mappings.reduce_from_model_parallel_region(y)
        if self.skip_bias_add:
            return y, self.bias
        if self.bias is not None:
            y = y + self.bias
        return y, None

    def forward_glu(self, ab: torch.Tensor, act: str, residual: Optional[torch.Tensor] = None):
        """Projection of the gated activation act(a) * b for ab = [a | b]; on one tensor-parallel rank the gate and
        the projection are one fused op (with fp8 projections the gate kernel writes the fp8 operand)."""
        if state.get_model_parallel_world_size() == 1 and self.input_is_parallel and (residual is not None or not self.skip_bias_add):
            return ops.glu_linear(ab, act, self.weight, self.bias, residual, fp8=self.fp8), None
        return self.forward(ops.glu_act_packed(ab, act), residual)
