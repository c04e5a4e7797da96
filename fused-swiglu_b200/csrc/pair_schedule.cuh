// Work list of the two-SM GEMM kernel and the host-side plan of its split last wave.  Plain
// integer arithmetic shared by the kernel (device) and the launcher (host), kept free of CUDA types
// so that it can be exercised on the CPU.
#pragma once

#ifdef __CUDACC__
#define FSW_HD __host__ __device__ __forceinline__
#else
#define FSW_HD inline
#endif

namespace fsw {

constexpr int kTailMaxSegmentsPerTile = 8;  // ranges that may share one tile

// One unit of a cluster's work list: k-blocks [kb0, kb1) of `tile`.
struct PairUnit {
  int tile;
  int kb0;
  int kb1;
  int tail_tile;  // index of the tile among the tail tiles, -1 for a whole-tile unit
  int half;       // -1: all columns of the tile; 0 / 1: its left / right half (width-split last wave)
};

// Enumerates the units of one cluster, in the order every role of the CTA pair walks them: whole
// tiles cluster, cluster + clusters, ... below tail_first, then the cluster's range
// [cluster * tail_len, (cluster + 1) * tail_len) of the tail's k-block sequence, cut at tile borders.
// With tail_halves != 0 (and tail_len == 0) the tiles from tail_first on are instead processed as two
// half-width units each, unit j (0 .. 2 * tail tiles - 1) by cluster j: same k order as a whole tile, so
// the results are bit-identical, and no partial sums exist.
struct PairSchedule {
  int num_clusters, num_kb, tail_first, num_tiles, half_unit;
  long long g, g_end;  // position and end of this cluster's range in the tail's k-block sequence
  int tile;            // next whole tile

  FSW_HD PairSchedule(int num_tiles_, int tail_first_, int tail_len, int tail_halves, int cluster, int clusters, int kb)
      : num_clusters(clusters), num_kb(kb), tail_first(tail_first_), num_tiles(num_tiles_),
        half_unit(tail_halves != 0 ? cluster : -1), tile(cluster) {
    const long long total = static_cast<long long>(num_tiles_ - tail_first_) * kb;
    g = static_cast<long long>(cluster) * tail_len;
    g_end = g + tail_len;
    if (g_end > total) g_end = total;
  }
  FSW_HD bool next(PairUnit* u) {
    u->half = -1;
    if (tile < tail_first) {
      u->tile = tile;
      u->kb0 = 0;
      u->kb1 = num_kb;
      u->tail_tile = -1;
      tile += num_clusters;
      return true;
    }
    if (half_unit >= 0) {
      const int j = half_unit;
      half_unit = -1;  // one half-width unit per cluster
      if (j < 2 * (num_tiles - tail_first)) {
        u->tile = tail_first + (j >> 1);
        u->kb0 = 0;
        u->kb1 = num_kb;
        u->tail_tile = -1;
        u->half = j & 1;
        return true;
      }
      return false;
    }
    if (g < g_end) {
      const int tt = static_cast<int>(g / num_kb);
      const int kb0 = static_cast<int>(g - static_cast<long long>(tt) * num_kb);
      long long kb1 = kb0 + (g_end - g);
      if (kb1 > num_kb) kb1 = num_kb;
      u->tile = tail_first + tt;
      u->kb0 = kb0;
      u->kb1 = static_cast<int>(kb1);
      u->tail_tile = tt;
      g += kb1 - kb0;
      return true;
    }
    return false;
  }
};

// How many ranges share tail tile `tt`, and which of them is cluster `cluster`'s (ranges of one
// tile belong to consecutive clusters).
FSW_HD void tail_tile_segments(int tt, int num_kb, int tail_len, int cluster, int* nseg, int* seg) {
  const long long t_begin = static_cast<long long>(tt) * num_kb;
  const int first_c = static_cast<int>(t_begin / tail_len);
  const int last_c = static_cast<int>((t_begin + num_kb - 1) / tail_len);
  *nseg = last_c - first_c + 1;
  *seg = cluster - first_c;
}

// Partial block of (cluster, tail tile), before the factor 2 and the CTA rank: unique per pair, and
// consecutive for the consecutive clusters that share one tile.
FSW_HD int tail_block_index(int cluster, int tt) { return cluster + tt; }

// Host-side plan.  tiles = whole problem, clusters = CTA pairs launched.  mode: 0 off, 1 when it
// pays, 2 whenever the last wave is partial.  On return tail_first == tiles and tail_len == 0 mean
// "no split".  Splitting pays when the wave would leave enough clusters idle: every shared tile costs
// a round trip of its 256 KiB accumulator through L2 (a few microseconds), a k-block about a third
// of a microsecond.
//
// Measured at the 7B prefill shape in bursts: a shared tile costs about 28 us (its 256 KiB accumulator is
// written once per range and read back by the last arriver with eight loads in flight per thread), a k-block
// a third of a microsecond - so the split only pays when it saves well over 85 k-blocks per cluster
// (the gate-up launch there saved 25 and lost 4 %; the down launch saved 93 and gained 0.5 %).
inline void plan_pair_tail_split(int tiles, int clusters, int num_kb, int mode, int* tail_first, int* tail_len) {
  *tail_first = tiles;
  *tail_len = 0;
  if (mode == 0 || clusters < 2) return;
  const int rem = tiles % clusters;
  if (rem == 0) return;
  const long long saved_kb = static_cast<long long>(clusters - rem) * num_kb / clusters;  // per cluster
  if (mode == 1 && saved_kb < 128) return;
  long long len = (static_cast<long long>(rem) * num_kb + clusters - 1) / clusters;
  const long long min_len = (num_kb + kTailMaxSegmentsPerTile - 2) / (kTailMaxSegmentsPerTile - 1);
  if (len < min_len) len = min_len;
  if (mode == 1 && len < 4) len = 4;
  if (len >= num_kb) return;  // nothing to share
  *tail_first = tiles - rem;
  *tail_len = static_cast<int>(len);
}

// Width-split of the last wave: worth it when its tiles fill at most half of the clusters (two units per
// tile still fit in one wave).  A half-width unit moves 1.5x the operand bytes per flop, so the wave takes
// more than half of a whole tile's time, but nothing has to be combined afterwards.
inline bool plan_pair_tail_halves(int tiles, int clusters, int tile_n, int* tail_first) {
  const int rem = tiles % clusters;
  if (clusters < 2 || rem == 0 || 2 * rem > clusters || tile_n % 32 != 0) return false;
  *tail_first = tiles - rem;
  return true;
}

}  // namespace fsw
