"""The unfused pipeline the fused ops are measured against: a library GEMM (cuBLAS through
``torch.matmul`` / ``torch._int_mm``) followed by the NCCL collective. Never used by the fused
ops themselves.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist


def _world(group) -> Tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


class Baseline:
    """Pre-allocates the intermediates so that the timed region holds only GEMM + collective."""

    def __init__(self, group=None):
        self.group = group
        self.rank, self.world = _world(group)
        self._bufs = {}

    def _buf(self, key, shape, dtype, device) -> torch.Tensor:
        t = self._bufs.get(key)
        if t is None or t.shape != torch.Size(shape) or t.dtype != dtype or t.device != device:
            t = torch.empty(shape, dtype=dtype, device=device)
            self._bufs[key] = t
        return t

    def matmul_allreduce(self, a, b, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        out = out if out is not None else self._buf("ar", (a.shape[0], b.shape[1]), a.dtype, a.device)
        torch.matmul(a, b, out=out)
        if self.world > 1:
            dist.all_reduce(out, group=self.group)
        return out

    def matmul_reduce_scatter(self, a, b, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        m, n = a.shape[0], b.shape[1]
        full = self._buf("rs_full", (m, n), a.dtype, a.device)
        torch.matmul(a, b, out=full)
        if self.world == 1:
            return full
        out = out if out is not None else self._buf("rs", (m // self.world, n), a.dtype, a.device)
        dist.reduce_scatter_tensor(out, full, group=self.group)
        return out

    def allgather_matmul(self, a_shard, b, out: Optional[torch.Tensor] = None):
        m, k = a_shard.shape
        gathered = a_shard
        if self.world > 1:
            gathered = self._buf("ag_g", (m * self.world, k), a_shard.dtype, a_shard.device)
            dist.all_gather_into_tensor(gathered, a_shard, group=self.group)
        out = out if out is not None else self._buf("ag", (m * self.world, b.shape[1]), a_shard.dtype, a_shard.device)
        torch.matmul(gathered, b, out=out)
        return out, gathered

    def quant_matmul_reduce_scatter(self, x1, x2, scale_x1, scale_x2, bias=None, out_dtype=torch.bfloat16):
        """int8 GEMM (``torch._int_mm``, int32 accumulate) + bias, int32 reduce-scatter, dequant."""
        m, n = x1.shape[0], x2.shape[1]
        acc = torch._int_mm(x1, x2)
        if bias is not None:
            acc += bias[None, :]
        rows = m // self.world
        if self.world > 1:
            part = self._buf("q_rs", (rows, n), torch.int32, x1.device)
            dist.reduce_scatter_tensor(part, acc, group=self.group)
        else:
            part = acc
        sl = slice(self.rank * rows, (self.rank + 1) * rows)
        return (part.float() * scale_x2[None, :] * scale_x1[sl, None]).to(out_dtype)
