"""Runtime tiling chooser: (op, M, N, K, world, dtype) -> :class:`TilingConfig`.

Order of precedence: an exact hit in the measured table, the nearest measured shape of the
same op / world / dtype in log-space (within a factor of two per dimension), then a heuristic
derived from the roofline: small outputs cannot fill 148 SMs with 128 x 256 tiles, so the tile
narrows until there is at least one tile per SM; everything else runs the widest tile, which
has the best tensor-core to shared-memory ratio.

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


def heuristic(op: str, m: int, n: int, k: int, world: int, dtype: torch.dtype) -> TilingConfig:
    rows = m
    tiles_m = max(1, math.ceil(rows / 128))
    bn = 256
    for cand in (256, 128, 64):
        bn = cand
        if tiles_m * math.ceil(n / cand) >= _NUM_SMS:
            break
    if dtype == torch.int8 and bn < 128:
        bn = 128  # 8-bit [K, N] operands need a full 128-byte run of N per TMA box
    # column-group width: keep the concurrently running tiles roughly square in (rows, cols)
    swizzle = 8 if tiles_m >= 8 else max(1, min(16, _NUM_SMS // max(1, tiles_m)))
    # 2-CTA pairs halve the shared-memory traffic per FLOP; they pay off once every rank's
    # row range splits into whole 256-row tiles and there is enough work to fill the pairs.
    seg_rows = rows if (world <= 1 or op == "allgather_matmul" and False) else rows
    if op in ("matmul_reduce_scatter", "quant_matmul_reduce_scatter", "matmul_allreduce", "allgather_matmul"):
        seg_rows = rows // max(1, world) if world > 1 else rows
    pair = 1
    forced = os.environ.get("CATCOC_CTA_PAIR")
    if forced in ("1", "2"):
        pair = int(forced)
    elif (bn >= 128 and seg_rows >= 256 and seg_rows % 256 == 0
          and (rows // 256) * math.ceil(n / bn) >= _NUM_SMS // 2):
        pair = 2   # measured: 2-CTA tiles with two K-blocks per stage run within a few % of cuBLAS
    if pair == 2 and dtype == torch.int8:
        bn = 256  # each CTA of a pair loads bn / 2 columns, and 8-bit [K, N] needs 128 of them
    if pair == 2 and bn < 128:
        pair = 1
    # measured at W = 8: the int32 partials of the quantised op are link bound, lagged owner
    # rounds overlap its owner-side reduce; the all-reduce gains from the NVLS broadcast (the op
    # layer drops the flag when the heap has no multicast alias) and from column ownership
    rounds = 4 if (op == "quant_matmul_reduce_scatter" and world > 1 and rows >= 2048) else 0
    if op == "matmul_allreduce" and world > 1:
        return TilingConfig(bn=bn, swizzle=swizzle, cta_pair=1, use_multicast=True, seg_dim=1 if n % (world * 8) == 0 else -1)
    return TilingConfig(bn=bn, swizzle=swizzle, cta_pair=pair, rounds=rounds)


def choose(op: str, m: int, n: int, k: int, world: int, dtype: torch.dtype,
           table: Optional["_table.TilingTable"] = None) -> TilingConfig:
    tbl = table if table is not None else _table.default_table()
    hit = tbl.lookup(op, m, n, k, world, dtype)
    if hit is not None:
        return hit
    return heuristic(op, m, n, k, world, dtype)
