// CPU check of the two-SM GEMM kernel's work list (fused-swiglu_b200/csrc/pair_schedule.cuh): for many
// problem shapes, every (tile, k-block) is covered exactly once, the per-tile segment arithmetic the
// epilogue uses agrees with what the clusters actually enumerate, and the scratch indices stay inside
// the buffer the launcher provides.  Prints "ok <cases>" and exits 0, or describes the first failure.
#include <cstdio>
#include <cstdlib>
#include <map>
#include <set>
#include <utility>
#include <vector>

#include "pair_schedule.cuh"

using namespace fsw;

static int fail(const char* what, int tiles, int clusters, int num_kb, int mode) {
  std::printf("FAILED: %s (tiles=%d clusters=%d num_kb=%d mode=%d)\n", what, tiles, clusters, num_kb, mode);
  return 1;
}

int main() {
  long long cases = 0;
  const int kb_values[] = {1, 2, 3, 5, 8, 16, 27, 56, 64, 80, 128, 172, 448};
  const int cluster_values[] = {1, 2, 3, 5, 7, 10, 33, 66, 74};
  for (int mode = 0; mode <= 2; ++mode) {
    for (int clusters : cluster_values) {
      for (int num_kb : kb_values) {
        for (int tiles = 1; tiles <= 4 * clusters + 3; ++tiles) {
          int tail_first = 0, tail_len = 0;
          plan_pair_tail_split(tiles, clusters, num_kb, mode, &tail_first, &tail_len);
          if (tail_len == 0 && tail_first != tiles) return fail("disabled plan must keep all tiles whole", tiles, clusters, num_kb, mode);
          if (tail_len > 0 && (tail_first % clusters != 0 || tail_first >= tiles || tiles - tail_first >= clusters))
            return fail("tail must be the partial last wave", tiles, clusters, num_kb, mode);
          std::vector<std::vector<int>> covered(tiles, std::vector<int>(num_kb, 0));
          std::map<int, std::vector<std::pair<int, int>>> segs;  // tail tile -> (cluster, kb0) in cluster order
          std::set<int> blocks;
          for (int c = 0; c < clusters; ++c) {
            PairSchedule s(tiles, tail_first, tail_len, 0, c, clusters, num_kb);
            PairUnit u;
            int guard = 0;
            while (s.next(&u)) {
              if (++guard > tiles + 4) return fail("schedule does not terminate", tiles, clusters, num_kb, mode);
              if (u.tile < 0 || u.tile >= tiles || u.kb0 < 0 || u.kb1 > num_kb || u.kb0 >= u.kb1)
                return fail("unit out of range", tiles, clusters, num_kb, mode);
              for (int kb = u.kb0; kb < u.kb1; ++kb) covered[u.tile][kb]++;
              if (u.tail_tile >= 0) {
                if (u.tile != tail_first + u.tail_tile) return fail("tail tile index", tiles, clusters, num_kb, mode);
                segs[u.tail_tile].push_back({c, u.kb0});
                int nseg = 0, seg = 0;
                tail_tile_segments(u.tail_tile, num_kb, tail_len, c, &nseg, &seg);
                if (nseg < 1 || nseg > kTailMaxSegmentsPerTile || seg < 0 || seg >= nseg)
                  return fail("segment count out of bounds", tiles, clusters, num_kb, mode);
                const int block = tail_block_index(c, u.tail_tile);
                if (nseg > 1) {
                  if (block < 0 || block >= 2 * clusters) return fail("scratch block outside 4 * clusters blocks", tiles, clusters, num_kb, mode);
                  if (!blocks.insert(block).second) return fail("scratch block used twice", tiles, clusters, num_kb, mode);
                  if (block - seg != tail_block_index(c - seg, u.tail_tile)) return fail("blocks of a tile not consecutive", tiles, clusters, num_kb, mode);
                }
              } else if (u.kb0 != 0 || u.kb1 != num_kb) {
                return fail("whole-tile unit with a partial range", tiles, clusters, num_kb, mode);
              }
            }
          }
          for (int t = 0; t < tiles; ++t)
            for (int kb = 0; kb < num_kb; ++kb)
              if (covered[t][kb] != 1) return fail("k-block not covered exactly once", tiles, clusters, num_kb, mode);
          for (auto& kv : segs) {
            int nseg = 0, seg = 0;
            tail_tile_segments(kv.first, num_kb, tail_len, kv.second.front().first, &nseg, &seg);
            if (nseg != static_cast<int>(kv.second.size()) || seg != 0) return fail("segment arithmetic disagrees with the enumeration", tiles, clusters, num_kb, mode);
            for (size_t i = 0; i < kv.second.size(); ++i) {
              tail_tile_segments(kv.first, num_kb, tail_len, kv.second[i].first, &nseg, &seg);
              if (seg != static_cast<int>(i)) return fail("segment order is not cluster order", tiles, clusters, num_kb, mode);
            }
          }
          ++cases;
        }
      }
    }
  }
  // width-split of the last wave: every column half of every tail tile exactly once, whole tiles untouched
  for (int clusters : cluster_values) {
    for (int tiles = 1; tiles <= 4 * clusters + 3; ++tiles) {
      int tail_first = tiles;
      const bool on = plan_pair_tail_halves(tiles, clusters, 128, &tail_first);
      if (!on) continue;
      if (tail_first % clusters != 0 || 2 * (tiles - tail_first) > clusters) return fail("halves plan", tiles, clusters, 0, 3);
      std::vector<int> whole(tiles, 0), left(tiles, 0), right(tiles, 0);
      for (int c = 0; c < clusters; ++c) {
        PairSchedule s(tiles, tail_first, 0, 1, c, clusters, 5);
        PairUnit u;
        int guard = 0;
        while (s.next(&u)) {
          if (++guard > tiles + 4) return fail("halves schedule does not terminate", tiles, clusters, 5, 3);
          if (u.kb0 != 0 || u.kb1 != 5 || u.tail_tile != -1) return fail("half unit with a k range", tiles, clusters, 5, 3);
          if (u.half < 0) whole[u.tile]++; else if (u.half == 0) left[u.tile]++; else right[u.tile]++;
          if (u.half >= 0 && u.tile < tail_first) return fail("half unit outside the tail", tiles, clusters, 5, 3);
        }
      }
      for (int t = 0; t < tiles; ++t) {
        const bool tail = t >= tail_first;
        if (whole[t] != (tail ? 0 : 1) || left[t] != (tail ? 1 : 0) || right[t] != (tail ? 1 : 0))
          return fail("halves coverage", tiles, clusters, 5, 3);
      }
      ++cases;
    }
  }
  // the shapes the benchmark configurations produce on 74 clusters
  struct { int tiles, kb; bool split; } known[] = {{256, 172, false}, {1376, 64, false}, {1024, 448, false}, {4, 2048, true}};
  for (auto& k : known) {
    int tf = 0, tl = 0;
    plan_pair_tail_split(k.tiles, 74, k.kb, 1, &tf, &tl);
    if ((tl > 0) != k.split) return fail("unexpected plan for a benchmark shape", k.tiles, 74, k.kb, 1);
  }
  std::printf("ok %lld\n", cases);
  return 0;
}
