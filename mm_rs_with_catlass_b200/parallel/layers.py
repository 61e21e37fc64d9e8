"""Tensor-parallel linear layers built on the fused ops.

The reference ships the three communication patterns of a Megatron-style tensor / sequence
parallel block as stand-alone kernels and leaves the composition to the user; these modules
are that composition:

* :class:`ColumnParallelLinear`  — all-gather of the row-sharded activation fused into the
  GEMM with the column shard of the weight (``allgather_matmul``);
* :class:`RowParallelLinear`     — GEMM with the row shard of the weight fused with the
  reduce-scatter (sequence parallel) or the all-reduce (plain tensor parallel) of the partial
  sums (``matmul_reduce_scatter`` / ``matmul_allreduce``);
* :class:`QuantRowParallelLinear` — the int8 variant with per-token / per-channel scales.

Inference-only: weights are plain tensors, no autograd graph is recorded.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops import fused
from ..tiling.config import TilingConfig
from .shmem import ShmemContext


class ColumnParallelLinear:
    """``y[W*m, N/W] = act(all_gather(x_shard)[W*m, K] @ weight[K, N/W])`` on every rank; the optional
    activation runs in the GEMM's epilogue."""

    def __init__(self, weight: torch.Tensor, ctx: Optional[ShmemContext] = None, trans_b: bool = False,
                 tiling: Optional[TilingConfig] = None, activation: Optional[str] = None):
        self.weight, self.ctx, self.trans_b, self.tiling, self.activation = weight, ctx, trans_b, tiling, activation

    def __call__(self, x_shard: torch.Tensor, out: Optional[torch.Tensor] = None, return_gathered: bool = False):
        y, gathered = fused.allgather_matmul(x_shard, self.weight, trans_b=self.trans_b, out=out, tiling=self.tiling,
                                             activation=self.activation, ctx=self.ctx)
        return (y, gathered) if return_gathered else y


class RowParallelLinear:
    """``y = sum_r x_r[M, K/W] @ weight_r[K/W, N]``; ``scatter=True`` returns this rank's
    ``[M/W, N]`` rows (sequence parallel), otherwise the full ``[M, N]`` on every rank."""

    def __init__(self, weight: torch.Tensor, ctx: Optional[ShmemContext] = None, trans_b: bool = False,
                 scatter: bool = True, tiling: Optional[TilingConfig] = None):
        self.weight, self.ctx, self.trans_b, self.scatter, self.tiling = weight, ctx, trans_b, scatter, tiling

    def __call__(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        op = fused.matmul_reduce_scatter if self.scatter else fused.matmul_allreduce
        return op(x, self.weight, trans_b=self.trans_b, out=out, tiling=self.tiling, ctx=self.ctx)


class QuantRowParallelLinear:
    """int8 row-parallel linear with exact int32 reduce-scatter and fused dequantisation."""

    def __init__(self, weight_q: torch.Tensor, weight_scale: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 ctx: Optional[ShmemContext] = None, trans_b: bool = False, out_dtype: torch.dtype = torch.bfloat16,
                 tiling: Optional[TilingConfig] = None):
        self.weight_q, self.weight_scale, self.bias = weight_q, weight_scale, bias
        self.ctx, self.trans_b, self.out_dtype, self.tiling = ctx, trans_b, out_dtype, tiling

    def __call__(self, x_q: torch.Tensor, x_scale: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        return fused.quant_matmul_reduce_scatter(x_q, self.weight_q, x_scale, self.weight_scale, self.bias,
                                                 trans_b=self.trans_b, out_dtype=self.out_dtype, out=out,
                                                 tiling=self.tiling, ctx=self.ctx)
