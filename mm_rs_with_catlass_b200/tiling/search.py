"""Candidate generator and feasibility rules of the tiling sweep.

Counterpart of the reference's search-space header (examples/dynamic_tiling/include/tiling.h:19-105:
a recursive product over commInterval x commTileM x (npuSplit, dataSplit) filtered by per-op
constraints on divisibility and workspace size). The Blackwell kernel has different knobs, so
the space is the product of tile width, CTA pairing, raster group width, grid size and, for the
all-reduce, ownership split and NVLS broadcast; the constraints are the ones this kernel has.
"""
from __future__ import annotations

import itertools
import math
from dataclasses import dataclass
from typing import Iterable, List, Optional, Sequence

from .config import TilingConfig

OPS = ("matmul_allreduce", "allgather_matmul", "matmul_reduce_scatter", "quant_matmul_reduce_scatter", "matmul")

# reference enum values kept for table compatibility (examples/dynamic_tiling/include/launch_map.h:6-16)
COMM_TYPE = {"matmul_allreduce": 0, "allgather_matmul": 1, "matmul_reduce_scatter": 2,
             "quant_matmul_reduce_scatter": 3}
DATA_TYPE = {"fp16": 1, "bf16": 27, "int8": 2}

BN_SPACE = (256, 128, 64)
PAIR_SPACE = (1, 2)
SWIZZLE_SPACE = (4, 8, 16)
NUM_CTAS_SPACE = (0,)          # 0 = one CTA per SM
ROUNDS_SPACE = (0,)            # 0 = the launcher's default
PULL_SPACE = (0, 1)            # reduce-scatter / all-reduce: push to the owner, or pull through the switch
COMM_WARPS_SPACE = (0,)        # 0 = all five communication / reducer warps
NUM_SMS = 148


@dataclass(frozen=True)
class Problem:
    op: str
    m: int           # output rows of the whole op (all-gather: W * shard rows)
    n: int
    k: int           # per-rank reduction length
    world: int
    dtype: str = "bf16"
    trans_a: bool = False
    trans_b: bool = False
    multicast_available: bool = False
    heap_bytes: int = 6 << 30

    @property
    def elt(self) -> int:
        return 1 if self.dtype == "int8" else 2


def _seg_len(p: Problem, seg_dim: int) -> int:
    return math.ceil((p.m if seg_dim == 0 else p.n) / max(1, p.world))


def workspace_bytes(p: Problem, t: TilingConfig) -> int:
    """Symmetric-heap bytes one call needs with this tiling (staging, outputs, stamps)."""
    if p.world <= 1 or p.op == "matmul":
        return 0
    bm = 256 if t.cta_pair == 2 else 128
    bn = t.effective_bn
    seg_dim = t.seg_dim if (p.op == "matmul_allreduce" and t.seg_dim in (0, 1)) else 0
    seg = _seg_len(p, seg_dim)
    if seg_dim == 0:
        tiles_per_seg = math.ceil(seg / bm) * math.ceil(p.n / bn)
    else:
        tiles_per_seg = math.ceil(p.m / bm) * math.ceil(seg / bn)
    total = 0
    if p.op in ("matmul_allreduce", "matmul_reduce_scatter", "quant_matmul_reduce_scatter"):
        pelt = 4 if (p.op == "quant_matmul_reduce_scatter" or t.fp32_partials) else p.elt
        if t.pull == 1:
            total += 2 * p.m * p.n * pelt                                 # local partial matrix, two parities
        else:
            total += 2 * p.world * tiles_per_seg * bm * bn * pelt        # staging slabs, two parities
        total += 4 * tiles_per_seg * p.world * (bm // 32)                 # arrival stamps
    if p.op == "matmul_allreduce":
        total += 2 * p.m * p.n * p.elt + 4 * tiles_per_seg * p.world * (bm // 32)
    if p.op == "allgather_matmul":
        per16 = 16 // p.elt
        ld = math.ceil(p.k / per16) * per16
        total += 2 * p.m * ld * p.elt + 4 * p.world * math.ceil((p.m // p.world) / 128) * math.ceil(ld * p.elt / 512)
    return total


def infeasible_reason(p: Problem, t: TilingConfig) -> Optional[str]:
    """None when the tiling can run this problem, otherwise the violated rule."""
    try:
        t.validate()
    except ValueError as e:
        return str(e)
    bn = t.effective_bn
    per16, per128 = 16 // p.elt, 128 // p.elt
    if t.cta_pair == 2 and bn < 128:
        return "a CTA pair splits the tile's columns in two halves of at least 64"
    cols_per_cta = bn // 2 if t.cta_pair == 2 else bn
    if not p.trans_b and cols_per_cta < per128:
        return "a B stored [K, N] needs a full 128-byte run of N per CTA"
    if p.op in ("matmul_reduce_scatter", "quant_matmul_reduce_scatter") and p.world > 1 and p.m % p.world:
        return "rows must divide by the world size"
    if p.op == "allgather_matmul" and p.trans_a:
        return "allgather_matmul has no trans_a variant"
    if p.op == "matmul_allreduce" and p.world > 1 and t.seg_dim == 1 and not p.trans_b \
            and _seg_len(p, 1) % per16:
        return "column-split ownership needs 16-byte aligned segment origins"
    if t.use_multicast and (p.op not in ("matmul_allreduce", "allgather_matmul") or not p.multicast_available):
        return "multicast stores apply to matmul_allreduce and allgather_matmul on a heap with a multicast alias"
    if t.pull == 1:
        if p.op not in ("matmul_allreduce", "matmul_reduce_scatter") or p.world <= 1:
            return "the pull flavour exists for the 16-bit reduce-scatter and all-reduce"
        if not p.multicast_available:
            return "the pull flavour sums through the multicast alias"
        if t.fp32_partials:
            return "the pull flavour moves partial tiles in the operand dtype"
        if p.n % 8 or (t.seg_dim == 1 and _seg_len(p, 1) % 8):
            return "the pull flavour needs N (and the columns per rank) to be multiples of 8"
    if t.comm_warps and p.op not in ("allgather_matmul", "matmul_allreduce", "matmul_reduce_scatter"):
        return "only the all-gather and the pull flavours have communication warps"
    if t.seg_dim != -1 and p.op != "matmul_allreduce":
        return "ownership split is an all-reduce knob"
    if t.num_ctas and (t.num_ctas > NUM_SMS or (t.cta_pair == 2 and t.num_ctas % 2)):
        return "grid must fit the SMs (and be even for CTA pairs)"
    if workspace_bytes(p, t) > p.heap_bytes:
        return "workspace exceeds the symmetric heap"
    return None


def candidates(p: Problem, bn_space: Sequence[int] = BN_SPACE, pair_space: Sequence[int] = PAIR_SPACE,
               swizzle_space: Sequence[int] = SWIZZLE_SPACE, num_ctas_space: Sequence[int] = NUM_CTAS_SPACE,
               rounds_space: Sequence[int] = ROUNDS_SPACE, pull_space: Sequence[int] = PULL_SPACE,
               comm_warps_space: Sequence[int] = COMM_WARPS_SPACE) -> List[TilingConfig]:
    """Every feasible tiling of the search space for this problem, widest tiles first."""
    seg_space: Iterable[int] = (-1,)
    mc_space: Iterable[bool] = (False,)
    fused = p.world > 1 and p.op != "matmul"
    if p.op == "matmul_allreduce" and fused:
        seg_space = (0, 1)
    if p.op in ("matmul_allreduce", "allgather_matmul") and fused and p.multicast_available:
        mc_space = (False, True)
    if not (fused and p.op in ("matmul_allreduce", "matmul_reduce_scatter") and p.multicast_available):
        pull_space = (0,)
    if not (fused and p.op in ("allgather_matmul", "matmul_allreduce", "matmul_reduce_scatter")):
        comm_warps_space = (0,)
    out: List[TilingConfig] = []
    if not fused or p.op == "allgather_matmul":
        rounds_space = (0,)
    seen = set()
    for bn, pair, swz, nctas, seg, mc, rounds, pull, cw in itertools.product(
            bn_space, pair_space, swizzle_space, num_ctas_space, seg_space, mc_space, rounds_space, pull_space,
            comm_warps_space):
        if pull == 1:
            rounds = 0                                   # the pull flavour has no lagged rounds ...
            mc = p.op == "matmul_allreduce"              # ... and always broadcasts through the alias
        elif cw and p.op != "allgather_matmul":
            continue                                     # communication warps idle in the push flavours
        t = TilingConfig(bn=bn, cta_pair=pair, swizzle=swz, num_ctas=nctas, seg_dim=seg, use_multicast=mc,
                         rounds=rounds, pull=pull, comm_warps=cw)
        if t in seen:
            continue
        seen.add(t)
        if infeasible_reason(p, t) is None:
            out.append(t)
    return out
