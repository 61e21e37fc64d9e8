"""Golden implementations of the four ops in plain PyTorch (fp32 / exact-integer accumulation).

They run on any device and any ``torch.distributed`` backend (``gloo`` on CPU), and are the
oracle for the CUDA kernels. The formulas generalise the reference's generators
(examples/utils/gen_data.py:33-45: ``W * (A @ B)`` and ``cat([A @ B] * W)``;
examples/utils/gen_quant_data.py:61-72: bias added once per rank, then both scales) to
per-rank different inputs.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist


def _world(group) -> Tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


def _logical(x: torch.Tensor, trans: bool) -> torch.Tensor:
    return x.t() if trans else x


def local_matmul_f32(a: torch.Tensor, b: torch.Tensor, trans_a: bool = False, trans_b: bool = False) -> torch.Tensor:
    return _logical(a, trans_a).float() @ _logical(b, trans_b).float()


def partial_magnitude(a, b, *, trans_a=False, trans_b=False, group=None) -> torch.Tensor:
    """``sum_r |A_r @ B_r|``: the scale of the rounding error when partial results are rounded
    before they are summed (see utils.verify.verify)."""
    mag = local_matmul_f32(a, b, trans_a, trans_b).abs()
    if _world(group)[1] > 1:
        dist.all_reduce(mag, group=group)
    return mag


def matmul_allreduce(a, b, *, trans_a=False, trans_b=False, out_dtype=None, group=None) -> torch.Tensor:
    """fp32 ``sum_r A_r @ B_r`` on every rank, rounded once to ``out_dtype``."""
    full = local_matmul_f32(a, b, trans_a, trans_b)
    if _world(group)[1] > 1:
        dist.all_reduce(full, group=group)
    return full.to(out_dtype or a.dtype)


def matmul_reduce_scatter(a, b, *, trans_a=False, trans_b=False, out_dtype=None, group=None) -> torch.Tensor:
    rank, world = _world(group)
    full = local_matmul_f32(a, b, trans_a, trans_b)
    if full.shape[0] % world:
        raise ValueError("M %% world != 0")
    if world > 1:
        dist.all_reduce(full, group=group)
    rows = full.shape[0] // world
    return full[rank * rows:(rank + 1) * rows].to(out_dtype or a.dtype)


def allgather_matmul(a_shard, b, *, trans_b=False, out_dtype=None, group=None) -> Tuple[torch.Tensor, torch.Tensor]:
    rank, world = _world(group)
    if world > 1:
        parts = [torch.empty_like(a_shard) for _ in range(world)]
        dist.all_gather(parts, a_shard.contiguous(), group=group)
        gathered = torch.cat(parts, dim=0)
    else:
        gathered = a_shard
    out = gathered.float() @ _logical(b, trans_b).float()
    return out.to(out_dtype or a_shard.dtype), gathered


def quant_matmul_reduce_scatter(x1, x2, scale_x1, scale_x2, bias: Optional[torch.Tensor] = None, *, trans_a=False,
                                trans_b=False, out_dtype=torch.bfloat16, group=None) -> torch.Tensor:
    """Exact integer accumulation (fp64 holds every int32 sum exactly), bias once per rank, sum
    over ranks, then ``* scale_x1[row] * scale_x2[col]`` in fp32 and one rounding."""
    rank, world = _world(group)
    acc = _logical(x1, trans_a).double() @ _logical(x2, trans_b).double()
    if bias is not None:
        acc = acc + bias.double()[None, :]
    if world > 1:
        dist.all_reduce(acc, group=group)
    m = acc.shape[0]
    if m % world:
        raise ValueError("M %% world != 0")
    rows = m // world
    sl = slice(rank * rows, (rank + 1) * rows)
    res = acc[sl].float() * scale_x2.float()[None, :] * scale_x1.float()[sl, None]
    return res.to(out_dtype)
