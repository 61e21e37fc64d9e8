"""Tiling configuration of the fused ops.

``TilingConfig`` carries every field of the reference's ``CocTilingParams``
(examples/dynamic_tiling/include/info.h:29-42) so that tables and scripts written for the
reference keep their columns, plus the knobs that actually steer the Blackwell kernel.

How the reference's knobs map onto this kernel:

=================  ======================================  ==========================================
reference field    meaning there                           here
=================  ======================================  ==========================================
m0 / n0 / k0       GEMM block tile (fixed 128x256x256)     tile is 128 x ``bn`` (64/128/256), K stage
                                                           64 (16-bit) or 128 (8-bit) elements
commInterval       GEMM blocks per core per comm round     no rounds: every tile is published as it
                                                           retires; ``rounds`` lags the owner's work
commNpuSplit x     vector cores doing communication and    ``num_ctas`` persistent CTAs x ``comm_warps``
commDataSplit      peers addressed concurrently            communication / reducer warps per CTA
commBlockM /       rows per comm task / per DMA            fixed 32-row quarters x 128-byte windows
commTileM
swizzle <7,1>      L2-friendly block order                 ``swizzle`` tiles per column group
=================  ======================================  ==========================================
"""
from __future__ import annotations

from dataclasses import dataclass, asdict, replace
from typing import Dict


@dataclass(frozen=True)
class TilingConfig:
    # --- knobs of this kernel ---
    bn: int = 0            # tile columns: 64, 128, 256 (0 = 256)
    swizzle: int = 0       # tiles per column group of the raster (0 = 8)
    num_ctas: int = 0      # persistent CTAs (0 = one per SM)
    seg_dim: int = -1      # all-reduce ownership split: 0 rows, 1 cols, -1 auto
    use_multicast: bool = False  # all-reduce broadcast through the NVLS alias
    rounds: int = 0        # reduce-scatter / all-reduce: owner tiles are spread over this many lagged rounds (0 = 1)
    fp32_partials: bool = False  # partial tiles cross NVLink in fp32 instead of the operand dtype (2x bytes, no rounding)
    cta_pair: int = 0      # 2: 256-row tiles on 2-CTA clusters (tcgen05 cta_group::2); 1: single CTA; 0 = 1
    pull: int = -1         # reduce-scatter / all-reduce data path: 1 = partial tiles stay in the local heap and the
                           # owner sums them through NVSwitch (multimem.ld_reduce); 0 = partial tiles are pushed
                           # to the owner, who sums them in rank order (deterministic); -1 = pull when possible
    comm_warps: int = 0    # communication / reducer warps per CTA, 1..5 (0 = 5): all-gather and pull flavours
    push_tma: int = -1     # push flavour: partial tiles travel by TMA stores (1) or 16-byte stores (0); -1: the
                           # CATCOC_PUSH_TMA environment variable decides (default: 16-byte stores)
    # --- reference-compatible fields (carried, reported, not steering the kernel) ---
    m0: int = 128
    n0: int = 256
    k0: int = 64
    comm_interval: int = 1
    comm_tile_m: int = 32
    comm_block_m: int = 32
    comm_npu_split: int = 1
    comm_data_split: int = 4

    def validate(self) -> "TilingConfig":
        if self.bn not in (0, 64, 128, 256):
            raise ValueError("bn must be 0, 64, 128 or 256 (got %d)" % self.bn)
        if self.swizzle < 0 or self.swizzle > 64:
            raise ValueError("swizzle must be in [0, 64]")
        if self.num_ctas < 0:
            raise ValueError("num_ctas must be >= 0")
        if self.cta_pair not in (0, 1, 2):
            raise ValueError("cta_pair must be 0, 1 or 2")
        if self.cta_pair == 2 and self.bn not in (0, 128, 256):
            raise ValueError("cta_pair=2 needs bn of 128 or 256")
        if self.rounds < 0 or self.rounds > 64:
            raise ValueError("rounds must be in [0, 64]")
        if self.seg_dim not in (-1, 0, 1):
            raise ValueError("seg_dim must be -1, 0 or 1")
        if self.pull not in (-1, 0, 1):
            raise ValueError("pull must be -1, 0 or 1")
        if self.push_tma not in (-1, 0, 1):
            raise ValueError("push_tma must be -1, 0 or 1")
        if self.comm_warps < 0 or self.comm_warps > 5:
            raise ValueError("comm_warps must be in [0, 5]")
        return self

    def to_dict(self) -> Dict[str, object]:
        return asdict(self)

    def with_(self, **kw) -> "TilingConfig":
        return replace(self, **kw).validate()

    @property
    def effective_bn(self) -> int:
        return self.bn or 256
