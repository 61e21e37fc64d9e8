"""Host-side replay of the device tile scheduler (the same C++ header, compiled for the host):
coverage, uniqueness, visiting order and clipping for aligned and ragged shapes."""
import ctypes as C
import itertools

import numpy as np
import pytest

from mm_rs_with_catlass_b200 import _native as N


def tiles(M, Nn, bm, bn, W, seg_dim, first, swz):
    lib = N.lib()
    total = lib.catcoc_sched_total_tiles(M, Nn, bm, bn, W, seg_dim)
    out = []
    for t in range(total):
        ti = N.Tile()
        assert lib.catcoc_sched_get_tile(M, Nn, bm, bn, W, seg_dim, first, swz, t, C.byref(ti)) == 0
        out.append(ti)
    return out


SHAPES = [(256, 512), (1024, 1024), (23, 45), (4, 129), (200, 328), (1030, 260), (129, 8), (8192, 256)]


@pytest.mark.parametrize("M,Nn", SHAPES)
@pytest.mark.parametrize("W", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("seg_dim", [0, 1])
@pytest.mark.parametrize("bm,bn,swz", [(128, 256, 8), (128, 64, 3), (256, 128, 1), (128, 128, 16)])
def test_every_element_is_covered_exactly_once(M, Nn, W, seg_dim, bm, bn, swz):
    cover = np.zeros((M, Nn), dtype=np.int32)
    seen_ids = set()
    for ti in tiles(M, Nn, bm, bn, W, seg_dim, first=1 % W, swz=swz):
        assert 0 <= ti.rows <= bm and 0 <= ti.cols <= bn
        assert (ti.seg, ti.tile_in_seg) not in seen_ids
        seen_ids.add((ti.seg, ti.tile_in_seg))
        if ti.rows and ti.cols:
            assert ti.m0 + ti.rows <= M and ti.n0 + ti.cols <= Nn
            cover[ti.m0:ti.m0 + ti.rows, ti.n0:ti.n0 + ti.cols] += 1
    assert (cover == 1).all()


@pytest.mark.parametrize("W", [2, 4, 8])
@pytest.mark.parametrize("seg_dim", [0, 1])
def test_tiles_stay_inside_their_segment(W, seg_dim):
    M, Nn = 1024 + 8 * W, 768 + 8 * W
    seg_len = -(-(M if seg_dim == 0 else Nn) // W)
    for ti in tiles(M, Nn, 128, 256, W, seg_dim, 0, 8):
        if not (ti.rows and ti.cols):
            continue
        lo, n = (ti.m0, ti.rows) if seg_dim == 0 else (ti.n0, ti.cols)
        assert ti.seg * seg_len <= lo and lo + n <= (ti.seg + 1) * seg_len


@pytest.mark.parametrize("W", [2, 3, 8])
def test_segments_are_visited_in_rotated_order_own_last(W):
    for rank in range(W):
        first = (rank + 1) % W           # reduce-scatter / all-reduce order
        segs = [ti.seg for ti in tiles(1024, 512, 128, 256, W, 0, first, 8)]
        order = list(dict.fromkeys(segs))
        assert order == [(first + p) % W for p in range(W)]
        assert order[-1] == rank
        # segments are contiguous runs: a rank finishes one destination before the next
        assert segs == sorted(segs, key=order.index)


def test_tile_ids_do_not_depend_on_the_swizzle():
    base = {(t.seg, t.mi, t.ni): t.tile_in_seg for t in tiles(2048, 2048, 128, 256, 4, 0, 0, 1)}
    for swz in (2, 5, 8, 64):
        for t in tiles(2048, 2048, 128, 256, 4, 0, 2, swz):
            assert base[(t.seg, t.mi, t.ni)] == t.tile_in_seg


def test_serpentine_groups_keep_neighbours_close():
    ts = tiles(2048, 4096, 128, 256, 1, 0, 0, 4)
    for a, b in zip(ts, ts[1:]):
        assert abs(a.mi - b.mi) + abs(a.ni - b.ni) <= 4   # no jumps across the matrix


def test_workspace_geometry_matches_the_schedule():
    lib = N.lib()
    for (M, Nn, W, bn, pair) in itertools.product((1024, 8192), (512, 8192), (2, 8), (64, 256), (1, 2)):
        if pair == 2 and bn < 128:
            continue
        bm = 256 if pair == 2 else 128
        per_seg = lib.catcoc_sched_total_tiles(M, Nn, bm, bn, W, 0) // W
        assert lib.catcoc_stage_bytes(M, Nn, W, 0, bn, pair, N.FMT_BF16) == 2 * W * per_seg * bm * bn * 2
        assert lib.catcoc_stage_bytes(M, Nn, W, 0, bn, pair, N.FMT_S32) == 2 * W * per_seg * bm * bn * 4
        assert lib.catcoc_arrive_words(M, Nn, W, 0, bn, pair) == per_seg * W * (bm // 32)
        assert lib.catcoc_done_words(M, Nn, W, 0, bn, pair) == per_seg * W * (bm // 32)


def test_bad_tile_index_is_rejected():
    ti = N.Tile()
    assert N.lib().catcoc_sched_get_tile(256, 256, 128, 256, 1, 0, 0, 1, 99, C.byref(ti)) == N.E_BAD_ARG


def tiles_rounds(M, Nn, bm, bn, W, seg_dim, first, swz, rounds):
    lib = N.lib()
    total = lib.catcoc_sched_total_tiles(M, Nn, bm, bn, W, seg_dim)
    out = []
    for t in range(total):
        ti = N.Tile()
        assert lib.catcoc_sched_get_tile_rounds(M, Nn, bm, bn, W, seg_dim, first, swz, rounds, t, C.byref(ti)) == 0
        out.append(ti)
    return out


@pytest.mark.parametrize("M,Nn", [(8192, 2048), (1024 + 136, 520), (200, 4096), (23, 45)])
@pytest.mark.parametrize("W", [2, 3, 8])
@pytest.mark.parametrize("seg_dim", [0, 1])
@pytest.mark.parametrize("rounds", [1, 2, 4, 5, 64])
def test_rounds_keep_coverage_and_ids(M, Nn, W, seg_dim, rounds):
    base = {(t.seg, t.tile_in_seg): (t.m0, t.n0, t.rows, t.cols) for t in tiles(M, Nn, 128, 256, W, seg_dim, 1 % W, 8)}
    got = tiles_rounds(M, Nn, 128, 256, W, seg_dim, 1 % W, 8, rounds)
    assert len(got) == len(base)
    seen = {}
    for t in got:
        seen[(t.seg, t.tile_in_seg)] = (t.m0, t.n0, t.rows, t.cols)
    assert seen == base          # same tiles with the same ids and geometry, only the order differs


def test_owner_tiles_lag_one_round_behind_the_remote_tiles():
    W, rank, R = 8, 3, 4
    ts = tiles_rounds(8192, 8192, 128, 256, W, 0, (rank + 1) % W, 8, R)
    round_len = (8192 // W // 128) // R
    pos = {}
    for i, t in enumerate(ts):
        key = ("own" if t.seg == rank else "remote", t.mi // round_len)
        lo, hi = pos.get(key, (i, i))
        pos[key] = (min(lo, i), max(hi, i))
    for r in range(R - 1):
        assert pos[("remote", r + 1)][1] < pos[("own", r)][0]       # own(r) only after remote(r+1) is done
        if r + 2 < R:
            assert pos[("own", r)][1] < pos[("remote", r + 2)][0]   # ... and before remote(r+2) starts
    assert pos[("own", R - 1)][1] == len(ts) - 1                     # the last round's owner tiles close the kernel
    assert pos[("own", 0)][0] < len(ts) // 2                         # owner work starts early, not piled up at the end
    # within a round the remote segments still rotate starting at rank + 1
    first_round = [t.seg for t in ts[:pos[("remote", 0)][1] + 1]]
    assert list(dict.fromkeys(first_round)) == [(rank + 1 + p) % W for p in range(W - 1)]


def tiles_order(M, Nn, bm, bn, W, seg_dim, first, swz, order):
    lib = N.lib()
    total = lib.catcoc_sched_total_tiles(M, Nn, bm, bn, W, seg_dim)
    out = []
    for t in range(total):
        ti = N.Tile()
        assert lib.catcoc_sched_get_tile_order(M, Nn, bm, bn, W, seg_dim, first, swz, order, t, C.byref(ti)) == 0
        out.append(ti)
    return out


@pytest.mark.parametrize("M,Nn", [(1024, 1024), (200, 328), (1030, 260), (23, 45)])
@pytest.mark.parametrize("W", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("seg_dim", [0, 1])
@pytest.mark.parametrize("order", [1, 2])
def test_other_visiting_orders_cover_the_same_tiles(M, Nn, W, seg_dim, order):
    """Interleaved (pull flavours) and local-first (multicast all-gather) orders visit exactly the
    tiles of the rotated order, with the same ids and extents."""
    key = lambda t: (t.seg, t.tile_in_seg, t.mi, t.ni, t.m0, t.n0, t.rows, t.cols)
    base = sorted(key(t) for t in tiles(M, Nn, 128, 128, W, seg_dim, 1 % W, 4))
    got = sorted(key(t) for t in tiles_order(M, Nn, 128, 128, W, seg_dim, 1 % W, 4, order))
    assert got == base


@pytest.mark.parametrize("W", [2, 4, 8])
def test_interleaved_order_cycles_through_the_owners(W):
    ts = tiles_order(2048 * W, 1024, 128, 256, W, 0, 3 % W, 8, 1)
    for t0 in range(0, len(ts), W):
        grp = ts[t0:t0 + W]
        assert [t.seg for t in grp] == list(range(W))            # every owner once, the same on all ranks
        assert len({(t.mi, t.ni) for t in grp}) == 1             # the same tile position in every segment


@pytest.mark.parametrize("W", [2, 4, 8])
def test_local_first_order_finishes_the_own_shard_then_interleaves_the_peers(W):
    rank = W - 1
    ts = tiles_order(512 * W, 1024, 128, 256, W, 0, rank, 8, 2)
    per_seg = len(ts) // W
    assert all(t.seg == rank for t in ts[:per_seg])
    rest = ts[per_seg:]
    for t0 in range(0, len(rest), W - 1):
        grp = rest[t0:t0 + W - 1]
        assert [t.seg for t in grp] == [(rank + 1 + s) % W for s in range(W - 1)]
        assert len({(t.mi, t.ni) for t in grp}) == 1
