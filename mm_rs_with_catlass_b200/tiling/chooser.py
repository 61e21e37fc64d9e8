"""Runtime tiling chooser: (op, M, N, K, world, dtype) -> :class:`TilingConfig`.

Order of precedence: an exact hit in the measured table, the nearest measured shape of the
same op / world / dtype in log-space (within a factor of two per dimension), then a heuristic
from a measured cost model: waves of tiles x the time of one wave, where a narrow tile costs far
more than its share of the output (it re-reads A once per column tile), so the widest tile wins
unless it leaves most SMs idle.

The reference only has the offline half of this (a sweep whose best rows are picked by hand,
examples/dynamic_tiling/utils/get_best_res.py:43-83; the default it falls back to is a
constant, examples/dynamic_tiling/dynamic_tiling.cpp:219-227).
"""
from __future__ import annotations

import math
import os
from typing import Optional

import torch

from .config import TilingConfig
from . import table as _table

_NUM_SMS = 148


# Measured on B200 (bf16, CUDA-graph replay): time of one wave of tiles relative to the 128 x 256
# single-CTA tile, per unit of output. Narrow tiles re-read A from L2 once per column tile and are
# bound by the fill rate of shared memory, so halving the width costs far more than half.
_TILE_EFF = {256: 1.0, 128: 0.56, 64: 0.43}
_PAIR_GAIN = {256: 1.10, 128: 1.35}     # 2-CTA tiles: each CTA fills half of B


def tile_cost(seg_rows: int, nseg: int, n: int, bn: int, pair: int, seg_cols: bool = False) -> float:
    """Relative time of a GEMM whose rows come in ``nseg`` segments of ``seg_rows`` rows (tiles never
    straddle segments): waves of tiles x time of one wave. With ``seg_cols`` the output is cut into
    ``nseg`` column segments instead and ``seg_rows`` is the full row count."""
    bm = 128 * pair
    if seg_cols:
        tiles = math.ceil(seg_rows / bm) * nseg * math.ceil(math.ceil(n / nseg) / bn)
    else:
        tiles = nseg * math.ceil(seg_rows / bm) * math.ceil(n / bn)
    units = _NUM_SMS // pair
    waves = math.ceil(tiles / units)
    eff = _TILE_EFF[bn] * (_PAIR_GAIN[bn] if pair == 2 else 1.0)
    return waves * bn / eff


def heuristic(op: str, m: int, n: int, k: int, world: int, dtype: torch.dtype) -> TilingConfig:
    rows = m
    fused = world > 1 and op in ("matmul_reduce_scatter", "quant_matmul_reduce_scatter", "matmul_allreduce",
                                 "allgather_matmul")
    nseg = world if fused else 1
    seg_rows = max(1, rows // nseg)
    allreduce = op == "matmul_allreduce" and world > 1
    ar_cols = allreduce and n % (world * 8) == 0     # the all-reduce then splits ownership by columns
    if ar_cols:
        seg_rows = rows
    forced = os.environ.get("CATCOC_CTA_PAIR")
    best = None
    for pair in (2, 1):
        if forced in ("1", "2") and pair != int(forced):
            continue
        if pair == 2 and (seg_rows < 256 or seg_rows % 256 != 0):
            continue   # ragged 256-row tiles are mostly padding
        for bn in (256, 128, 64):
            if pair == 2 and bn < 128:
                continue
            if dtype == torch.int8 and (bn < 128 or (pair == 2 and bn < 256)):
                continue   # 8-bit [K, N] operands need a full 128-byte run of N per TMA box and CTA
            cost = tile_cost(seg_rows, nseg, n, bn, pair, seg_cols=ar_cols)
            if best is None or cost < best[0] - 1e-9:
                best = (cost, bn, pair)
    if best is None:
        best = (0.0, 256, 1)
    _, bn, pair = best
    tiles_m = max(1, math.ceil(rows / 128))
    # column-group width: keep the concurrently running tiles roughly square in (rows, cols)
    # (measured on 8192 x 28672 x 8192 and 8192 x 8192 x 28672: groups of 3-4 column tiles run 3-5 % faster
    # than groups of 8 or 16)
    swizzle = 4 if tiles_m >= 8 else max(1, min(16, _NUM_SMS // max(1, tiles_m)))
    # measured at W = 8: the int32 partials of the quantised op are link bound, lagged owner
    # rounds overlap its owner-side reduce; the all-reduce gains from the NVLS broadcast (the op
    # layer drops the flag when the heap has no multicast alias) and from column ownership
    rounds = 4 if (op == "quant_matmul_reduce_scatter" and world > 1 and rows >= 2048) else 0
    if allreduce:
        return TilingConfig(bn=bn, swizzle=swizzle, cta_pair=pair, use_multicast=True, seg_dim=1 if ar_cols else -1)
    # the all-gather broadcasts its shard by multicast stores when the heap has the alias (measured at
    # M = 8192: 6 % faster than peer-by-peer stores on 4 GPUs, 7 % slower on 2, where one store per
    # 16 bytes reaches one peer either way)
    return TilingConfig(bn=bn, swizzle=swizzle, cta_pair=pair, rounds=rounds,
                        use_multicast=(op == "allgather_matmul" and world >= 4))


def choose(op: str, m: int, n: int, k: int, world: int, dtype: torch.dtype,
           table: Optional["_table.TilingTable"] = None) -> TilingConfig:
    tbl = table if table is not None else _table.default_table()
    hit = tbl.lookup(op, m, n, k, world, dtype)
    if hit is not None:
        return hit
    return heuristic(op, m, n, k, world, dtype)
