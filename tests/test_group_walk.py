"""Host replay of the group walk (the tile list of grouped / batched / split-K launches): every
row of every group is covered exactly once per column tile, tiles never straddle groups, and the
walk tolerates empty groups, lists that stop short of M and malformed lists."""
import ctypes as C
import random

import pytest

from mm_rs_with_catlass_b200 import _native as N


def _replay(M, Nn, bm, bn, ends=None, group_rows=0, num_groups=None):
    lib = N.lib()
    g = num_groups if num_groups is not None else len(ends)
    arr = (C.c_int32 * g)(*ends) if ends is not None else None
    total = lib.catcoc_group_walk_replay(M, Nn, bm, bn, g, arr, group_rows, 0, None)
    assert total >= 0
    tiles = (N.Tile * max(1, total))()
    assert lib.catcoc_group_walk_replay(M, Nn, bm, bn, g, arr, group_rows, total, tiles) == total
    return [tiles[i] for i in range(total)]


def _check_cover(tiles, M, Nn, bm, bn, bounds):
    """bounds: list of (begin, end) per group."""
    nt = (Nn + bn - 1) // bn
    cover = {}
    for t in tiles:
        b, e = bounds[t.seg]
        assert b <= t.m0 < e and 0 < t.rows <= bm and t.m0 + t.rows <= e
        assert t.m0 == b + t.mi * bm and t.n0 == t.ni * bn and 0 <= t.ni < nt
        assert t.cols == min(bn, Nn - t.n0)
        for r in range(t.m0, t.m0 + t.rows):
            key = (r, t.ni)
            assert key not in cover
            cover[key] = 1
    want = sum(e - b for b, e in bounds if e > b) * nt
    assert len(cover) == want


@pytest.mark.parametrize("bm,bn", [(128, 256), (256, 128), (128, 64)])
@pytest.mark.parametrize("sizes", [[128, 256, 64], [5, 0, 300, 129, 1], [0, 0, 700], [33] * 9, [1], [0, 0]])
def test_ragged_groups_cover_exactly(bm, bn, sizes):
    ends, acc = [], 0
    for s in sizes:
        acc += s
        ends.append(acc)
    M = max(1, acc + 17)            # rows past the last group belong to nobody
    tiles = _replay(M, 520, bm, bn, ends)
    bounds = [(e - s, e) for s, e in zip(sizes, ends)]
    _check_cover(tiles, M, 520, bm, bn, bounds)
    # launch order: groups ascending, rows fastest inside a group
    keys = [(t.seg, t.ni, t.mi) for t in tiles]
    assert keys == sorted(keys)


@pytest.mark.parametrize("groups,rows", [(1, 77), (4, 128), (7, 200), (3, 513)])
def test_uniform_groups(groups, rows):
    M = groups * rows
    tiles = _replay(M, 300, 128, 128, None, rows, groups)
    _check_cover(tiles, M, 300, 128, 128, [(g * rows, (g + 1) * rows) for g in range(groups)])


def test_random_lists():
    rng = random.Random(7)
    for _ in range(50):
        g = rng.randint(1, 40)
        sizes = [rng.choice([0, 1, 31, 128, 129, 255, 256, 400]) for _ in range(g)]
        ends, acc = [], 0
        for s in sizes:
            acc += s
            ends.append(acc)
        M = max(1, acc)
        bm = rng.choice([128, 256])
        bn = rng.choice([64, 128, 256])
        nn = rng.choice([8, 100, 256, 777])
        tiles = _replay(M, nn, bm, bn, ends)
        _check_cover(tiles, M, nn, bm, bn, [(e - s, e) for s, e in zip(sizes, ends)])


def test_malformed_lists_stay_inside_the_output():
    """Decreasing, negative or oversized entries skip rows but never leave [0, M)."""
    M = 500
    for ends in ([300, 100, 450], [-5, 200, 9999], [600, 700], [0, -1, -2]):
        for t in _replay(M, 256, 128, 128, ends):
            assert 0 <= t.m0 and t.m0 + t.rows <= M and t.rows > 0
