"""Per-tile timeline of the fused kernels as a Chrome / Perfetto trace.

The diagnostic build of the library (``CATCOC_CHECKED=1``) can write one record per role and
tile boundary into a ring in device memory: the global nanosecond timer, the CTA, the role
(TMA producer, MMA issuer, epilogue, communication warp, reducer warp), begin or end, and the
tile (or reducer task) index. This module owns the ring and turns it into the JSON that
``chrome://tracing`` and Perfetto read: one process per rank, one thread row per (CTA, role).

    with EventTrace(capacity=1 << 16) as tr:          # every launch from here on records
        catcoc.matmul_reduce_scatter(a, b)
    tr.dump_chrome("rs_rank%d.json" % rank, pid=rank)

The reference has no in-kernel timers; its pipeline views come from the external profiler's
simulator traces (3rdparty/catlass/docs/tools/performance_tools.md:83-122).
"""
from __future__ import annotations

import json
from typing import Dict, List, Optional

import torch

from ..ops import _common as cm

ROLES = {0: "tma_producer", 1: "mma", 2: "epilogue", 3: "comm", 4: "reducer"}
PHASES = {0: "B", 1: "E", 2: "i"}


class EventTrace:
    def __init__(self, capacity: int = 1 << 16, device: Optional[torch.device] = None):
        self.capacity = int(capacity)
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        # word 0: write cursor; records of four words from word 4 on
        self.ring = torch.zeros(4 + 4 * self.capacity, dtype=torch.int32, device=self.device)

    def __enter__(self) -> "EventTrace":
        from .. import _native as N
        if N.lib().catcoc_is_checked_build() != 1:
            raise RuntimeError("the event ring is compiled into the diagnostic build only: set CATCOC_CHECKED=1 "
                               "before the library is loaded")
        self.ring.zero_()
        cm.set_event_ring(self.ring.data_ptr(), self.capacity)
        return self

    def __exit__(self, *exc) -> None:
        cm.set_event_ring(None, 0)
        torch.cuda.synchronize(self.device)

    def records(self) -> List[Dict[str, int]]:
        """The recorded events in time order (ring overflow drops the youngest)."""
        words = self.ring.cpu().numpy().astype("uint32")
        n = min(int(words[0]), self.capacity)
        out = []
        for i in range(n):
            lo, hi, tag, tile = (int(x) for x in words[4 + 4 * i: 8 + 4 * i])
            out.append({"t_ns": (hi << 32) | lo, "cta": tag >> 16, "role": (tag >> 8) & 0xff, "phase": tag & 0xff,
                        "tile": tile})
        out.sort(key=lambda r: r["t_ns"])
        return out

    @property
    def dropped(self) -> int:
        return max(0, int(self.ring[0].item()) - self.capacity)

    def dump_chrome(self, path: str, pid: int = 0) -> int:
        """Writes the Chrome trace and returns the number of events."""
        recs = self.records()
        t0 = recs[0]["t_ns"] if recs else 0
        events = []
        for r in recs:
            role = ROLES.get(r["role"], "role%d" % r["role"])
            events.append({"name": "%s %d" % ("task" if r["role"] == 4 else "tile", r["tile"]), "cat": role,
                           "ph": PHASES.get(r["phase"], "i"), "ts": (r["t_ns"] - t0) / 1e3, "pid": pid,
                           "tid": r["cta"] * 8 + r["role"]})
        meta = [{"name": "process_name", "ph": "M", "pid": pid, "args": {"name": "rank %d" % pid}}]
        for tid in sorted({e["tid"] for e in events}):
            meta.append({"name": "thread_name", "ph": "M", "pid": pid, "tid": tid,
                         "args": {"name": "cta %d %s" % (tid // 8, ROLES.get(tid % 8, "?"))}})
        with open(path, "w") as fh:
            json.dump({"traceEvents": meta + events, "displayTimeUnit": "ns"}, fh)
        return len(events)
