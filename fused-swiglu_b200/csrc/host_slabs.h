// Row slabs of the host-buffer pipeline (fswiglu_mlp_bf16_host): plain integer code, kept apart from the
// CUDA sources so that a host-only checker can include it.
#pragma once

#include <cstdint>
#include <cstdlib>

namespace fsw {

constexpr int kMaxHostSlabs = 64;  // events per direction the pipeline owns: no plan may have more slabs

// Rows per slab of the host-buffer pipeline: large enough that each slab still fills the
// machine (>= 1024 rows), small enough that the first copy in and the last copy out are short.
// Measured at the 70B shape in one process (20 steps each, power-capped): equal 1024-row slabs 9.89-9.96 ms per
// step, 1024-row slabs with 512-row first and last slab 9.89-9.91, equal 2048-row slabs 9.72-10.1, 2048-row slabs
// with 512-row first and last slab 9.58-9.66 (the device-resident step: 8.7-8.9 ms): taller slabs fill the GEMM
// waves better, short edge slabs expose less of the first copy in and the last copy out.
inline int64_t host_slab_rows(int64_t M) {
  int64_t rows = M >= 8192 ? 2048 : 1024;
  if (const char* env = std::getenv("FSWIGLU_HOST_SLAB")) {  // experiments only: rows per slab
    const int v = std::atoi(env);
    if (v >= 128 && v % 128 == 0) rows = v;
  }
  const int64_t min_rows = (M + kMaxHostSlabs - 1) / kMaxHostSlabs;
  if (rows < min_rows) rows = (min_rows + 127) / 128 * 128;
  if (rows > M) rows = M;
  return rows;
}

// Row slabs of the host-buffer pipeline.  The first slab's copy in and the last slab's copy out cannot overlap
// any compute, so with enough rows those two slabs are only 512 rows tall (at the 70B shape: 0.15 ms exposed at
// either end instead of 0.3-0.6 ms).  Returns the slab count; first[i] / rows[i] describe slab i.
inline int host_slab_plan(int64_t M, int64_t* first, int64_t* rows) {
  const int64_t slab = host_slab_rows(M);
  int n = 0;
  int64_t r = 0;
  auto push = [&](int64_t take) {
    first[n] = r;
    rows[n] = take;
    r += take;
    ++n;
  };
  bool short_edges = slab >= 1024 && slab % 1024 == 0 && M >= 4 * slab && M <= (kMaxHostSlabs - 4) * slab;
  if (const char* env = std::getenv("FSWIGLU_HOST_EDGES")) {  // experiments only: 0 = equal slabs
    if (env[0] == '0') short_edges = false;
  }
  if (!short_edges) {
    while (r < M) push(M - r < slab ? M - r : slab);
    return n;
  }
  const int64_t edge = 512, middle = M - 2 * edge;
  int64_t n_mid = (middle + slab - 1) / slab;
  int64_t rem = middle - (n_mid - 1) * slab;  // 1 .. slab rows in the last middle slab
  if (rem < 256 && n_mid > 1) {               // too few rows for a slab of their own: the one before takes them
    --n_mid;
    rem += slab;
  }
  push(edge);
  for (int64_t i = 0; i + 1 < n_mid; ++i) push(slab);
  push(rem);
  push(edge);
  return n;
}

}  // namespace fsw
