// Host-only check of the row-slab plan of the host-buffer pipeline (csrc/host_slabs.h): for every batch size
// the slabs are contiguous, non-empty, cover all rows, and never outnumber the events the pipeline owns.
#include <cstdio>

#include "host_slabs.h"

int main() {
  int64_t first[fsw::kMaxHostSlabs + 2], rows[fsw::kMaxHostSlabs + 2];
  long long checked = 0;
  int most = 0;
  for (int64_t M = 1; M <= 3000000; M += (M < 70000 ? 1 : 1009)) {
    const int n = fsw::host_slab_plan(M, first, rows);
    if (n < 1 || n > fsw::kMaxHostSlabs) {
      std::printf("M=%lld: %d slabs\n", static_cast<long long>(M), n);
      return 1;
    }
    int64_t next = 0;
    for (int i = 0; i < n; ++i) {
      if (first[i] != next || rows[i] <= 0) {
        std::printf("M=%lld: slab %d starts at %lld with %lld rows, expected start %lld\n", static_cast<long long>(M), i,
                    static_cast<long long>(first[i]), static_cast<long long>(rows[i]), static_cast<long long>(next));
        return 1;
      }
      next += rows[i];
    }
    if (next != M) {
      std::printf("M=%lld: slabs cover %lld rows\n", static_cast<long long>(M), static_cast<long long>(next));
      return 1;
    }
    // a short first and last slab only where there are tall slabs between them
    if (n >= 3 && rows[0] == 512 && rows[n - 1] == 512 && rows[1] < 512) {
      std::printf("M=%lld: edge slabs taller than the slab between them\n", static_cast<long long>(M));
      return 1;
    }
    if (n > most) most = n;
    ++checked;
  }
  // the plan at the 70B batch size: 512-row edges, 2048-row slabs between
  const int n = fsw::host_slab_plan(8192, first, rows);
  if (n != 6 || rows[0] != 512 || rows[1] != 2048 || rows[4] != 1024 || rows[5] != 512) {
    std::printf("unexpected plan for 8192 rows (%d slabs)\n", n);
    return 1;
  }
  std::printf("ok %lld batch sizes, at most %d slabs\n", checked, most);
  return 0;
}
