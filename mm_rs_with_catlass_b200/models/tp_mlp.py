"""Sequence-parallel transformer MLP block: the flagship composition of the fused ops.

    x_shard [M/W, H]  --all-gather + GEMM-->  h [M, F/W]  --act-->  --GEMM + reduce-scatter-->  y_shard [M/W, H]

with ``H`` = 8192 and ``F`` = 28672 in the benchmark configuration. Both halves are single
fused kernels. The activation runs in the epilogue of the first one (fp32, one rounding) where
that kernel's epilogue variant can feed the link: on one GPU, and from 4 GPUs on, where the shard
travels by multicast stores; on 2 GPUs it is a separate element-wise launch.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F_

from ..parallel.layers import ColumnParallelLinear, RowParallelLinear
from ..parallel.shmem import ShmemContext
from ..tiling.config import TilingConfig


@dataclass
class TPMLPConfig:
    hidden: int = 8192
    ffn: int = 28672
    dtype: torch.dtype = torch.bfloat16
    activation: str = "gelu"   # "gelu", "silu", "relu" or "none"
    init_std: float = 0.02


class TPMLP:
    """Random-initialised weights of one rank's shard; ``forward`` maps a row shard to a row shard."""

    def __init__(self, cfg: TPMLPConfig, ctx: Optional[ShmemContext], device: torch.device, seed: int = 0,
                 up_tiling: Optional[TilingConfig] = None, down_tiling: Optional[TilingConfig] = None):
        self.cfg, self.ctx = cfg, ctx
        world = ctx.world if ctx is not None else 1
        rank = ctx.rank if ctx is not None else 0
        if cfg.ffn % world:
            raise ValueError("ffn %d not divisible by world %d" % (cfg.ffn, world))
        g = torch.Generator(device=device)
        g.manual_seed(1234 + 17 * seed + rank)
        f = cfg.ffn // world
        self.w_up = (torch.randn((cfg.hidden, f), device=device, generator=g) * cfg.init_std).to(cfg.dtype)
        self.w_down = (torch.randn((f, cfg.hidden), device=device, generator=g) * cfg.init_std).to(cfg.dtype)
        # fuse the activation into the up projection where its epilogue variant (one communication
        # warp per CTA) does not starve the all-gather
        self.fuse_act = cfg.activation != "none" and (world == 1 or (world >= 4 and bool(ctx.mc_base)))
        if os.environ.get("CATCOC_FUSE_ACT") in ("0", "1"):
            self.fuse_act = cfg.activation != "none" and os.environ["CATCOC_FUSE_ACT"] == "1"
        self.up = ColumnParallelLinear(self.w_up, ctx, tiling=up_tiling,
                                       activation=cfg.activation if self.fuse_act else None)
        self.down = RowParallelLinear(self.w_down, ctx, scatter=True, tiling=down_tiling)

    def _act(self, h: torch.Tensor) -> torch.Tensor:
        a = self.cfg.activation
        if a == "gelu":
            return F_.gelu(h, approximate="tanh")
        if a == "silu":
            return F_.silu(h)
        if a == "relu":
            return F_.relu(h)
        return h

    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        h = self.up(x_shard)
        return self.down(h if self.fuse_act else self._act(h))

    __call__ = forward

    def reference_forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        """Same block with the golden ops (fp32 accumulate, any backend)."""
        from ..ops import reference as ref
        h, _ = ref.allgather_matmul(x_shard, self.w_up, out_dtype=self.cfg.dtype)
        return ref.matmul_reduce_scatter(self._act(h), self.w_down, out_dtype=self.cfg.dtype)
