// Tile scheduling and offset arithmetic shared by host and device code.
//
// One persistent scheduler serves every fused op. The output grid [M, N] is cut into W
// "segments" along rows or columns (one per rank that owns / supplied that part), each segment
// is tiled independently with BM x BN tiles (ragged last tiles are clipped), and segments are
// visited in a rotated order so that every rank starts on a different peer:
//   matmul_reduce_scatter / matmul_allreduce : destination-major, first = rank+1, own last
//   allgather_matmul                        : source-major, first = rank (local rows need no wait)
// Inside a segment tiles run in column groups of `swizzle` tiles with a serpentine walk over
// rows, which keeps the set of concurrently running tiles compact for L2 reuse.
//
// Counterparts in the reference (same job, different construction):
//   3rdparty/catlass/include/catlass/gemm/block/block_swizzle.hpp:24-125   (tile swizzle)
//   include/catcoc/dgemm/block/block_swizzle_allgather.hpp:29-116          (source-major order)
//   include/catcoc/dgemm/kernel/matmul_reduce_scatter.hpp:157-166          (destination-major)
//   include/catcoc/comm_epilogue/block/comm_block_swizzle.hpp:148-186      (peer rotation)
#pragma once
#include <cstdint>

#if defined(__CUDACC__)
#define CATCOC_HD __host__ __device__ inline
#else
#define CATCOC_HD inline
#endif

namespace catcoc {

CATCOC_HD int ceil_div(int a, int b) { return (a + b - 1) / b; }
CATCOC_HD int round_up(int a, int b) { return ceil_div(a, b) * b; }
CATCOC_HD int imin(int a, int b) { return a < b ? a : b; }

enum SegDim : int { SEG_ROWS = 0, SEG_COLS = 1 };

// Order in which a rank visits the segments' tiles.
//   ORDER_ROTATED      segment after segment, starting at `first_seg` (push flavours: every rank
//                      starts on another peer; own segment last for RS / AR, first for AG)
//   ORDER_INTERLEAVED  tile i of segment 0, of segment 1, ..., of segment W-1, then tile i+1: all
//                      ranks compute the same tile at about the same time and the tiles in flight
//                      belong to all owners alike. For the pull flavours, where an owner reduces
//                      a tile through the switch as soon as every rank has stored its partial.
//   ORDER_LOCAL_FIRST  all tiles of segment `first_seg` (the local shard), then tile i of every
//                      other segment, tile i+1, ...: for the all-gather whose shards travel by
//                      multicast, where chunk i of every peer arrives at about the same time.
enum TileOrder : int { ORDER_ROTATED = 0, ORDER_INTERLEAVED = 1, ORDER_LOCAL_FIRST = 2 };

struct TileSched {
  int M, N;          // extent of the grid being tiled (output rows / cols)
  int BM, BN;        // tile shape
  int W;             // number of segments (= world size; 1 for a local GEMM)
  int seg_dim;       // SEG_ROWS or SEG_COLS
  int seg_len;       // rows (or cols) per segment
  int first_seg;     // segment visited first
  int swizzle;       // tiles per column group (>= 1)
  int seg_mt, seg_nt;    // tiles per segment along rows / cols
  int tiles_per_seg;     // seg_mt * seg_nt
  int total_tiles;       // W * tiles_per_seg
  // Rounds: every segment's tiles are cut into `rounds` groups (along rows for a row split,
  // along columns for a column split). Per round the W-1 remote segments are visited first;
  // the own segment follows one round late (see get_tile), so only the last round's owner
  // work is exposed. This is the reference's "comm interval" idea
  // (include/catcoc/dgemm/kernel/matmul_allreduce.hpp:116-133) without its global barriers.
  // Rounds apply to schedules whose own segment comes last (first_seg = rank + 1).
  int rounds;
  int round_len;         // tiles along the cut dimension per round (last round may be shorter)
  int order;             // TileOrder (rounds apply to ORDER_ROTATED only)
};

struct TileInfo {
  int seg;          // which segment (owner rank for RS/AR, source rank for AG)
  int tile_in_seg;  // 0 .. tiles_per_seg-1, identical on every rank for the same (seg, mi, ni)
  int mi, ni;       // tile coordinates inside the segment
  int m0, n0;       // first row / col in the full grid
  int rows, cols;   // valid rows / cols (clipped)
};

CATCOC_HD TileSched make_sched(int M, int N, int BM, int BN, int W, int seg_dim, int first_seg,
                               int swizzle, int rounds = 1, int order = ORDER_ROTATED) {
  TileSched s;
  s.order = (order == ORDER_INTERLEAVED || order == ORDER_LOCAL_FIRST) ? order : ORDER_ROTATED;
  if (s.order != ORDER_ROTATED) rounds = 1;
  s.M = M; s.N = N; s.BM = BM; s.BN = BN; s.W = W < 1 ? 1 : W;
  s.seg_dim = seg_dim;
  s.swizzle = swizzle < 1 ? 1 : swizzle;
  if (seg_dim == SEG_ROWS) {
    s.seg_len = ceil_div(M, s.W);
    s.seg_mt = ceil_div(s.seg_len, BM);
    s.seg_nt = ceil_div(N, BN);
  } else {
    s.seg_len = ceil_div(N, s.W);
    s.seg_mt = ceil_div(M, BM);
    s.seg_nt = ceil_div(s.seg_len, BN);
  }
  s.first_seg = ((first_seg % s.W) + s.W) % s.W;
  s.tiles_per_seg = s.seg_mt * s.seg_nt;
  s.total_tiles = s.tiles_per_seg * s.W;
  const int cut = (seg_dim == SEG_ROWS) ? s.seg_mt : s.seg_nt;
  s.rounds = rounds < 1 ? 1 : (rounds > cut ? cut : rounds);
  s.round_len = ceil_div(cut, s.rounds);
  s.rounds = ceil_div(cut, s.round_len);
  return s;
}

// Position of a tile inside an mt x nt grid from its linear index (swizzled order).
CATCOC_HD void grid_tile_coord(int mt, int nt, int swizzle, int i, int* mi, int* ni) {
  const int group_tiles = swizzle * mt;
  const int g = i / group_tiles;
  const int within = i - g * group_tiles;
  const int gw = imin(swizzle, nt - g * swizzle);
  int m = within / gw;
  const int n = g * swizzle + (within - m * gw);
  if (g & 1) m = mt - 1 - m;  // serpentine: odd groups walk rows bottom-up
  *mi = m;
  *ni = n;
}
CATCOC_HD void seg_tile_coord(const TileSched& s, int i, int* mi, int* ni) {
  grid_tile_coord(s.seg_mt, s.seg_nt, s.swizzle, i, mi, ni);
}

// Inverse of seg_tile_coord: the canonical id used to address staging slots and flags.
// The id is position-based (mi * seg_nt + ni), not order-based, so ranks that use different
// swizzles still agree on which slot a tile lives in.
CATCOC_HD int seg_tile_id(const TileSched& s, int mi, int ni) { return mi * s.seg_nt + ni; }

// Fills id, origin and clipped extent of a tile from (seg, mi, ni).
CATCOC_HD void fill_tile_extent(const TileSched& s, TileInfo* t) {
  TileInfo& ti = *t;
  ti.tile_in_seg = seg_tile_id(s, ti.mi, ti.ni);
  if (s.seg_dim == SEG_ROWS) {
    const int seg_begin = ti.seg * s.seg_len;
    const int seg_end = imin(seg_begin + s.seg_len, s.M);
    ti.m0 = seg_begin + ti.mi * s.BM;
    ti.n0 = ti.ni * s.BN;
    ti.rows = imin(s.BM, seg_end - ti.m0);
    ti.cols = imin(s.BN, s.N - ti.n0);
  } else {
    const int seg_begin = ti.seg * s.seg_len;
    const int seg_end = imin(seg_begin + s.seg_len, s.N);
    ti.m0 = ti.mi * s.BM;
    ti.n0 = seg_begin + ti.ni * s.BN;
    ti.rows = imin(s.BM, s.M - ti.m0);
    ti.cols = imin(s.BN, seg_end - ti.n0);
  }
  if (ti.rows < 0) ti.rows = 0;
  if (ti.cols < 0) ti.cols = 0;
}

CATCOC_HD TileInfo get_tile(const TileSched& s, int t) {
  TileInfo ti;
  // t -> (round, phase, index inside the round's slice of the segment)
  int round = 0, phase, i;
  if (s.order == ORDER_INTERLEAVED) {
    i = t / s.W;
    ti.seg = t - i * s.W;
    seg_tile_coord(s, i, &ti.mi, &ti.ni);
  } else if (s.order == ORDER_LOCAL_FIRST) {
    if (t < s.tiles_per_seg || s.W == 1) {
      i = t;
      ti.seg = s.first_seg;
    } else {
      const int r = t - s.tiles_per_seg;
      i = r / (s.W - 1);
      ti.seg = (s.first_seg + 1 + (r - i * (s.W - 1))) % s.W;
    }
    seg_tile_coord(s, i, &ti.mi, &ti.ni);
  } else if (s.rounds <= 1) {
    phase = t / s.tiles_per_seg;
    i = t - phase * s.tiles_per_seg;
    ti.seg = (s.first_seg + phase) % s.W;
    seg_tile_coord(s, i, &ti.mi, &ti.ni);
  } else {
    // Lagged rounds. Block order (W-1 "remote" segments per round, own segment one round late):
    //   remote(0) | remote(1) own(0) | remote(2) own(1) | ... | remote(R-1) own(R-2) | own(R-1)
    // The own segment is the LAST of the rotation (first_seg + W - 1): its partial tiles were
    // pushed by the peers a whole round earlier, so the owner never waits for them, and its
    // heavy epilogue (reduce, broadcast) overlaps the next round's tensor-core work.
    const int other = (s.seg_dim == SEG_ROWS) ? s.seg_nt : s.seg_mt;   // tiles along the uncut dim
    const int cut = (s.seg_dim == SEG_ROWS) ? s.seg_mt : s.seg_nt;
    const int full = s.round_len * other;                               // tiles of one segment in a full round
    const int last_len = cut - (s.rounds - 1) * s.round_len;
    int rem = t;
    bool own_block = false;
    for (int blk = 0;; ++blk) {
      // blk even: remote(blk/2) ; blk odd: own((blk-1)/2 ... lagging) ; final block own(R-1)
      const bool is_remote = (blk < 2 * s.rounds - 1) ? ((blk == 0) || (blk & 1)) : false;
      int rnd;
      if (blk == 0) rnd = 0;
      else if (blk < 2 * s.rounds - 1) rnd = (blk & 1) ? (blk + 1) / 2 : blk / 2 - 1;
      else rnd = s.rounds - 1;
      const int len = (rnd == s.rounds - 1) ? last_len : s.round_len;
      const int n = (is_remote ? (s.W - 1) : 1) * len * other;
      if (rem < n || blk >= 2 * s.rounds - 1) {
        round = rnd;
        own_block = !is_remote;
        break;
      }
      rem -= n;
      (void)full;
    }
    const int this_len = (round == s.rounds - 1) ? last_len : s.round_len;
    const int per_phase = this_len * other;
    if (own_block) {
      phase = s.W - 1;
      i = rem;
    } else {
      phase = rem / per_phase;
      i = rem - phase * per_phase;
    }
    ti.seg = (s.first_seg + phase) % s.W;
    if (s.seg_dim == SEG_ROWS) {
      grid_tile_coord(this_len, s.seg_nt, s.swizzle, i, &ti.mi, &ti.ni);
      ti.mi += round * s.round_len;
    } else {
      grid_tile_coord(s.seg_mt, this_len, s.swizzle, i, &ti.mi, &ti.ni);
      ti.ni += round * s.round_len;
    }
  }
  fill_tile_extent(s, &ti);
  return ti;
}

// The i-th tile (in the segment's swizzled order) of segment `seg`, whoever visits it when.
CATCOC_HD TileInfo seg_tile(const TileSched& s, int seg, int i) {
  TileInfo ti;
  ti.seg = seg;
  seg_tile_coord(s, i, &ti.mi, &ti.ni);
  fill_tile_extent(s, &ti);
  return ti;
}

// ---------------------------------------------------------------------------------------
// Group walk: the tile list of one launch over several products that share N and K (grouped,
// batched, split-K). It is the concatenation of the groups' tile grids, rows fastest inside a
// group so that tiles running side by side share the group's B columns. Group g owns the
// output rows [end(g-1), end(g)); `ends` (cumulative counts, possibly device memory) or, when it
// is null, uniform groups of `group_rows` rows. Extents are clamped to [0, M] and to be
// non-decreasing, so a malformed list can skip rows but never address outside the output.
// ---------------------------------------------------------------------------------------
struct GroupWalk {
  int g;           // current group
  int tile_base;   // tiles of the groups before g
  int row_begin;   // first output row of g
  int row_end;     // one past its last row
};

CATCOC_HD int group_end_row(const int32_t* ends, int group_rows, int M, int g) {
  const int e = (ends != nullptr) ? ends[g] : (g + 1) * group_rows;
  return e < 0 ? 0 : (e > M ? M : e);
}

CATCOC_HD GroupWalk group_walk_begin(int num_groups, const int32_t* ends, int group_rows, int M) {
  GroupWalk w;
  w.g = 0; w.tile_base = 0; w.row_begin = 0;
  w.row_end = (num_groups > 0) ? group_end_row(ends, group_rows, M, 0) : 0;
  return w;
}

CATCOC_HD int group_rows_of(const GroupWalk& w) { return w.row_end > w.row_begin ? w.row_end - w.row_begin : 0; }

// `t` must be below the walk's total and must not decrease between calls on one cursor.
CATCOC_HD TileInfo group_walk_tile(const TileSched& s, int num_groups, const int32_t* ends, int group_rows, int t,
                                   GroupWalk& w) {
  const int nt = (s.N + s.BN - 1) / s.BN;
  int mt = (group_rows_of(w) + s.BM - 1) / s.BM;
  while (t >= w.tile_base + mt * nt && w.g + 1 < num_groups) {
    w.tile_base += mt * nt;
    ++w.g;
    if (w.row_end > w.row_begin) w.row_begin = w.row_end;
    w.row_end = group_end_row(ends, group_rows, s.M, w.g);
    mt = (group_rows_of(w) + s.BM - 1) / s.BM;
  }
  TileInfo ti;
  const int local = t - w.tile_base;
  if (mt < 1) mt = 1;
  ti.seg = w.g;
  ti.tile_in_seg = local;
  ti.mi = local % mt;
  ti.ni = local / mt;
  ti.m0 = w.row_begin + ti.mi * s.BM;
  ti.n0 = ti.ni * s.BN;
  ti.rows = w.row_end - ti.m0;
  if (ti.rows > s.BM) ti.rows = s.BM;
  if (ti.rows < 0) ti.rows = 0;
  ti.cols = s.N - ti.n0;
  if (ti.cols > s.BN) ti.cols = s.BN;
  if (ti.cols < 0) ti.cols = 0;
  return ti;
}

// Serial count of the walk's tiles (the kernel computes the same sum with one warp).
CATCOC_HD int group_walk_total(const TileSched& s, int num_groups, const int32_t* ends, int group_rows) {
  const int nt = (s.N + s.BN - 1) / s.BN;
  int total = 0, begin = 0;
  for (int g = 0; g < num_groups; ++g) {
    const int e = group_end_row(ends, group_rows, s.M, g);
    if (e > begin) { total += ((e - begin + s.BM - 1) / s.BM) * nt; begin = e; }
  }
  return total;
}

// Order in which a pusher visits its peers: the peer that consumes this rank's data earliest
// comes first. For source-major consumers (allgather_matmul) rank r reads source q in phase
// (q - r) mod W, so q serves q-1, q-2, ... For destination-major producers the order is
// rank+1, rank+2, ...
CATCOC_HD int peer_for_push_ag(int rank, int step, int W) { return ((rank - step) % W + W) % W; }
CATCOC_HD int peer_for_push_rs(int rank, int step, int W) { return (rank + step) % W; }

// ---------------------------------------------------------------------------------------
// Workspace geometry (bytes) for the fused ops; all ranks compute identical numbers.
// ---------------------------------------------------------------------------------------
// Staging for pushed partial tiles: two parity halves, each [source W][tiles_per_seg] slabs of
// BM x BN elements. The distance between the halves (`parity_bytes`) is a property of the buffer,
// fixed when it is allocated, NOT of the launch: two launches with different tile geometries then
// still agree on which bytes belong to which parity, so a rank that runs one launch ahead never
// writes into the half its peers are still reading.
CATCOC_HD int64_t stage_tile_bytes(const TileSched& s, int elt_bytes) {
  return static_cast<int64_t>(s.BM) * s.BN * elt_bytes;
}
CATCOC_HD int64_t stage_half_bytes(const TileSched& s, int elt_bytes) {
  return static_cast<int64_t>(s.W) * s.tiles_per_seg * stage_tile_bytes(s, elt_bytes);
}
CATCOC_HD int64_t stage_slot_offset(const TileSched& s, int elt_bytes, int64_t parity_bytes, int parity,
                                    int src, int tile_in_seg) {
  return static_cast<int64_t>(parity) * parity_bytes +
         (static_cast<int64_t>(src) * s.tiles_per_seg + tile_in_seg) * stage_tile_bytes(s, elt_bytes);
}
// Smallest region that holds both halves (the halves are then `stage_half_bytes` apart).
CATCOC_HD int64_t stage_total_bytes(const TileSched& s, int elt_bytes) {
  return 2 * stage_half_bytes(s, elt_bytes);
}
// Arrival stamps: one 32-bit word per (tile_in_seg, source).
CATCOC_HD int64_t arrive_flag_index(const TileSched& s, int tile_in_seg, int src) {
  return static_cast<int64_t>(tile_in_seg) * s.W + src;
}

// All-gather chunk geometry: the local shard [m, K] is pushed in units of
// `chunk_rows` x `slice_cols` elements; a consumer needs every slice of a row chunk.
struct GatherPlan {
  int m, K;          // shard rows, row length (elements)
  int chunk_rows;    // rows per chunk (= BM of the consumer)
  int slice_cols;    // elements per slice
  int n_chunks, n_slices;
};
CATCOC_HD GatherPlan make_gather_plan(int m, int K, int chunk_rows, int slice_cols) {
  GatherPlan g;
  g.m = m; g.K = K; g.chunk_rows = chunk_rows; g.slice_cols = slice_cols;
  g.n_chunks = ceil_div(m, chunk_rows);
  g.n_slices = ceil_div(K, slice_cols);
  return g;
}
CATCOC_HD int64_t gather_flag_index(const GatherPlan& g, int src, int chunk, int slice) {
  return (static_cast<int64_t>(src) * g.n_chunks + chunk) * g.n_slices + slice;
}

}  // namespace catcoc
