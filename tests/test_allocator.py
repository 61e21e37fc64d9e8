"""Offset allocator of the symmetric heap (pure host code): first fit, merging, and the rule that
a freed block stays out of circulation until two more launches were issued."""
import random

import pytest

from mm_rs_with_catlass_b200.parallel.allocator import GRANULE, HeapExhausted, SymmAllocator


def test_blocks_are_granular_and_disjoint():
    a = SymmAllocator(1 << 20)
    offs = [(a.malloc(n), n) for n in (1, 255, 256, 257, 4096, 7)]
    for off, _ in offs:
        assert off % GRANULE == 0
    spans = sorted((off, off + (n + GRANULE - 1) // GRANULE * GRANULE) for off, n in offs)
    for (_, e0), (b1, _) in zip(spans, spans[1:]):
        assert e0 <= b1
    assert a.bytes_in_use == sum(e - b for b, e in spans)


def test_freed_block_is_quarantined_for_two_launches():
    a = SymmAllocator(1 << 20)
    x = a.malloc(4096, tick=10)
    a.malloc(256, tick=10)            # keeps x from being the top of the bump area
    a.free(x, tick=10)
    assert a.malloc(4096, tick=10) != x
    assert a.malloc(4096, tick=11) != x
    assert a.malloc(4096, tick=12) == x


def test_adjacent_free_blocks_merge_once_both_are_reusable():
    a = SymmAllocator(1 << 20)
    x, y, z = a.malloc(1024), a.malloc(1024), a.malloc(1024)
    a.malloc(256)
    a.free(x, tick=0)
    a.free(z, tick=5)
    a.free(y, tick=1)
    assert a.largest_free(tick=2) == 1024     # x alone; y and z are still in quarantine
    assert a.largest_free(tick=6) == 2048     # x + y; z (released at 5) must not be touched before 7
    assert a.largest_free(tick=7) == 3072
    assert a.malloc(3072, tick=7) == x


def test_growing_sequence_does_not_exhaust_the_heap():
    """A session that walks through growing shapes: each growth frees the old region. With the
    free list the heap's high-water mark stays bounded; a bump-only allocator would run out."""
    a = SymmAllocator(64 << 20)
    cur, tick = None, 0
    for step in range(200):
        size = (1 << 20) * (1 + step % 7) + 4096 * step
        if cur is not None:
            a.free(cur, tick)
        cur = a.malloc(size, tick)
        tick += 3
    assert a.high_water <= 64 << 20
    assert a.bytes_in_use == a.size_of(cur)


def test_top_of_heap_is_reclaimed_before_giving_up():
    a = SymmAllocator(1 << 20)
    x = a.malloc(768 << 10)
    a.free(x, tick=0)
    with pytest.raises(HeapExhausted):
        a.malloc(900 << 10, tick=1)           # still quarantined
    assert a.malloc(900 << 10, tick=2) == x   # reclaimed into the bump area and extended


def test_double_free_and_bad_sizes_are_errors():
    a = SymmAllocator(1 << 20)
    x = a.malloc(100)
    a.free(x)
    with pytest.raises(ValueError):
        a.free(x)
    with pytest.raises(ValueError):
        a.malloc(0)
    with pytest.raises(HeapExhausted):
        a.malloc(2 << 20)


def test_identical_call_sequences_give_identical_offsets():
    """Every rank runs its own allocator; symmetric addressing needs them to agree."""
    rng = random.Random(7)
    script = []
    live = 0
    for _ in range(500):
        if live and rng.random() < 0.45:
            script.append(("free", rng.randrange(live)))
            live -= 1
        else:
            script.append(("malloc", rng.randrange(1, 1 << 16)))
            live += 1

    def play():
        a = SymmAllocator(256 << 20)
        blocks, trace, tick = [], [], 0
        for op, arg in script:
            if op == "malloc":
                off = a.malloc(arg, tick)
                blocks.append(off)
                trace.append(off)
            else:
                a.free(blocks.pop(arg), tick)
            tick += 1
        return trace

    assert play() == play()
