"""Offset allocator of the symmetric heap: first fit over a free list, then bump.

Every rank runs its own copy and makes the same sequence of calls, so every rank computes
the same offsets without talking to anyone (the job of ``shmem_malloc`` / ``shmem_free`` in the
reference, examples/00_matmul_allreduce/matmul_allreduce.cpp:274, :290).

A freed block is not handed out again at once. The ranks of a fused launch sequence may be one
launch apart, so a peer can still be writing into (or reading from) a block that this rank has
just released on its host thread; the block becomes reusable only once ``reuse_after`` further
launches have been issued (two: by then every rank has finished the launch that last used it).
Blocks are 256-byte granular; adjacent free blocks merge once both are reusable.
"""
from __future__ import annotations

from typing import List, Tuple

GRANULE = 256


class HeapExhausted(RuntimeError):
    pass


def _round_up(n: int, a: int) -> int:
    return (n + a - 1) // a * a


class SymmAllocator:
    def __init__(self, capacity: int, reuse_after: int = 2):
        self.capacity = int(capacity)
        self.reuse_after = int(reuse_after)
        self._cursor = 0
        self._free: List[Tuple[int, int, int]] = []   # (offset, nbytes, ready_tick), sorted by offset
        self._live = {}                               # offset -> nbytes

    # ------------------------------------------------------------------------------
    def malloc(self, nbytes: int, tick: int = 0) -> int:
        """Offset of a block of ``nbytes`` (rounded up to the granule). ``tick`` is the caller's
        launch counter: only blocks freed at least ``reuse_after`` ticks ago are considered."""
        if nbytes <= 0:
            raise ValueError("malloc of %d bytes" % nbytes)
        size = _round_up(int(nbytes), GRANULE)
        self._merge_ready(tick)
        for i, (off, n, ready) in enumerate(self._free):
            if ready <= tick and n >= size:
                if n == size:
                    self._free.pop(i)
                else:
                    self._free[i] = (off + size, n - size, ready)
                self._live[off] = size
                return off
        if self._cursor + size > self.capacity:
            # the top of the heap may be a free, ready block: take it back into the bump area
            self._reclaim_top(tick)
            if self._cursor + size > self.capacity:
                raise HeapExhausted(
                    "symmetric heap exhausted: need %d bytes, %d of %d in the bump area are used and the largest "
                    "reusable free block has %d bytes" % (size, self._cursor, self.capacity, self.largest_free(tick)))
        off = self._cursor
        self._cursor += size
        self._live[off] = size
        return off

    def free(self, offset: int, tick: int = 0) -> None:
        size = self._live.pop(offset, None)
        if size is None:
            raise ValueError("free of offset %d, which is not a live block" % offset)
        self._free.append((offset, size, tick + self.reuse_after))
        self._free.sort()

    def _merge_ready(self, tick: int) -> None:
        """Joins neighbouring free blocks that are both reusable at ``tick``. A block still in
        quarantine stays on its own, so that it cannot hold its neighbours back."""
        merged: List[Tuple[int, int, int]] = []
        for off, n, ready in self._free:
            if merged and ready <= tick and merged[-1][2] <= tick and merged[-1][0] + merged[-1][1] == off:
                po, pn, _ = merged[-1]
                merged[-1] = (po, pn + n, 0)
            else:
                merged.append((off, n, ready))
        self._free = merged

    # ------------------------------------------------------------------------------
    def _reclaim_top(self, tick: int) -> None:
        while self._free:
            off, n, ready = self._free[-1]
            if off + n == self._cursor and ready <= tick:
                self._free.pop()
                self._cursor = off
            else:
                break

    def largest_free(self, tick: int) -> int:
        self._merge_ready(tick)
        return max([n for _, n, ready in self._free if ready <= tick], default=0)

    @property
    def bytes_in_use(self) -> int:
        return sum(self._live.values())

    @property
    def high_water(self) -> int:
        return self._cursor

    def size_of(self, offset: int) -> int:
        return self._live[offset]
