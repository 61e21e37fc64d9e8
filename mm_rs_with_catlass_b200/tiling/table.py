"""Measured tiling table: CSV rows of (op, dtype, world, M, K, N, tiling..., time) and lookups.

Column layout keeps the reference's tuning CSV
(``Op,M,K,N,Transpose A,Transpose B,commInterval,commTileM,commBlockM,commNpuSplit,commDataSplit,Time(us)``,
examples/dynamic_tiling/include/tiling.h:107-143) and appends the columns that steer this
kernel. Appending is incremental and resumable: a row that is already present (same key and
tiling) is skipped, so an interrupted sweep continues where it stopped
(the reference resumes by CSV line ranges, examples/dynamic_tiling/scripts/run.sh:33-40).
"""
from __future__ import annotations

import csv
import math
import os
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from .config import TilingConfig

COLUMNS = ["Op", "M", "K", "N", "Transpose A", "Transpose B", "commInterval", "commTileM", "commBlockM",
           "commNpuSplit", "commDataSplit", "Time(us)",
           "dtype", "world", "bn", "swizzle", "num_ctas", "seg_dim", "use_multicast", "cta_pair", "fp32_partials", "rounds", "baseline_us",
           "pull", "comm_warps", "push_tma"]

_DTYPE_NAMES = {torch.float16: "fp16", torch.bfloat16: "bf16", torch.int8: "int8"}
DEFAULT_TABLE_PATH = Path(__file__).resolve().parent / "best_tilings.csv"


def dtype_name(dt) -> str:
    return _DTYPE_NAMES.get(dt, str(dt).replace("torch.", ""))


@dataclass(frozen=True)
class Row:
    op: str
    m: int
    k: int
    n: int
    trans_a: int
    trans_b: int
    dtype: str
    world: int
    tiling: TilingConfig
    time_us: float
    baseline_us: float = float("nan")

    def key(self) -> Tuple:
        return (self.op, self.dtype, self.world, self.m, self.k, self.n, self.trans_a, self.trans_b)

    def to_csv(self) -> List[object]:
        t = self.tiling
        return [self.op, self.m, self.k, self.n, self.trans_a, self.trans_b, t.comm_interval, t.comm_tile_m,
                t.comm_block_m, t.comm_npu_split, t.comm_data_split,
                "" if math.isnan(self.time_us) else "%.3f" % self.time_us,
                self.dtype, self.world, t.bn, t.swizzle, t.num_ctas, t.seg_dim, int(t.use_multicast), t.cta_pair, int(t.fp32_partials), t.rounds,
                "" if math.isnan(self.baseline_us) else "%.3f" % self.baseline_us, t.pull, t.comm_warps, t.push_tma]

    @staticmethod
    def from_csv(r: Dict[str, str]) -> "Row":
        def f(x, default=float("nan")):
            return float(x) if x not in (None, "") else default
        t = TilingConfig(bn=int(r.get("bn") or 0), swizzle=int(r.get("swizzle") or 0), num_ctas=int(r.get("num_ctas") or 0),
                         seg_dim=int(r.get("seg_dim") or -1), use_multicast=bool(int(r.get("use_multicast") or 0)), cta_pair=int(r.get("cta_pair") or 0), fp32_partials=bool(int(r.get("fp32_partials") or 0)), rounds=int(r.get("rounds") or 0),
                         pull=int(r.get("pull") if r.get("pull") not in (None, "") else -1),
                         comm_warps=int(r.get("comm_warps") or 0),
                         push_tma=int(r.get("push_tma") if r.get("push_tma") not in (None, "") else -1),
                         comm_interval=int(r.get("commInterval") or 1), comm_tile_m=int(r.get("commTileM") or 32),
                         comm_block_m=int(r.get("commBlockM") or 32), comm_npu_split=int(r.get("commNpuSplit") or 1),
                         comm_data_split=int(r.get("commDataSplit") or 4))
        return Row(r["Op"], int(r["M"]), int(r["K"]), int(r["N"]), int(r.get("Transpose A") or 0),
                   int(r.get("Transpose B") or 0), r.get("dtype") or "bf16", int(r.get("world") or 1), t,
                   f(r.get("Time(us)")), f(r.get("baseline_us")))


class TilingTable:
    def __init__(self, rows: Iterable[Row] = ()):
        self.rows: List[Row] = list(rows)

    # ---- IO ----
    @staticmethod
    def load(path) -> "TilingTable":
        path = Path(path)
        if not path.exists():
            return TilingTable()
        with path.open(newline="") as fh:
            return TilingTable(Row.from_csv(r) for r in csv.DictReader(fh))

    def save(self, path) -> None:
        path = Path(path)
        tmp = path.with_suffix(path.suffix + ".tmp%d" % os.getpid())
        with tmp.open("w", newline="") as fh:
            w = csv.writer(fh)
            w.writerow(COLUMNS)
            for r in self.rows:
                w.writerow(r.to_csv())
        os.replace(tmp, path)

    @staticmethod
    def append_row(path, row: Row) -> bool:
        """Appends one measured row unless an identical (key, tiling) row exists. Returns
        whether a row was written."""
        path = Path(path)
        existing = TilingTable.load(path)
        if existing.has(row):
            return False
        new = not path.exists()
        with path.open("a", newline="") as fh:
            w = csv.writer(fh)
            if new:
                w.writerow(COLUMNS)
            w.writerow(row.to_csv())
        return True

    def has(self, row: Row) -> bool:
        return any(r.key() == row.key() and r.tiling == row.tiling for r in self.rows)

    # ---- queries ----
    def best(self) -> "TilingTable":
        """Arg-min of the time per (op, dtype, world, shape): the reference's best_result.csv."""
        best: Dict[Tuple, Row] = {}
        for r in self.rows:
            if math.isnan(r.time_us):
                continue
            cur = best.get(r.key())
            if cur is None or r.time_us < cur.time_us:
                best[r.key()] = r
        return TilingTable(best.values())

    def lookup(self, op: str, m: int, n: int, k: int, world: int, dtype) -> Optional[TilingConfig]:
        name = dtype if isinstance(dtype, str) else dtype_name(dtype)
        cands = [r for r in self.rows if r.op == op and r.world == world and r.dtype == name
                 and not math.isnan(r.time_us)]
        if not cands:
            return None
        exact = [r for r in cands if (r.m, r.n, r.k) == (m, n, k)]
        if exact:
            return min(exact, key=lambda r: r.time_us).tiling
        def dist(r: Row) -> float:
            return max(abs(math.log2(r.m / m)), abs(math.log2(r.n / n)), abs(math.log2(r.k / k)))
        near = min(cands, key=dist)
        if dist(near) <= 1.0:
            best_at = [r for r in cands if (r.m, r.n, r.k) == (near.m, near.n, near.k)]
            return min(best_at, key=lambda r: r.time_us).tiling
        return None


_default: Optional[TilingTable] = None


def default_table() -> TilingTable:
    global _default
    if _default is None:
        path = os.environ.get("CATCOC_TILING_TABLE", str(DEFAULT_TABLE_PATH))
        _default = TilingTable.load(path).best()
    return _default


def reload_default() -> TilingTable:
    global _default
    _default = None
    return default_table()
