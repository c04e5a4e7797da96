// Pieces shared by the one-SM and the two-SM tcgen05 GEMM kernels: modes, tile constants, the
// parameter block, tile rasterisation and the epilogue (accumulator -> gate -> bf16/fp32 -> global).
//
// The epilogue is written once, against an "accumulator source": either this CTA's TMEM
// accumulator, or the fp32 partial tiles of a reduction that was split over several CTAs
// (summed in a fixed order).  Everything after the raw accumulator values is identical:
//   gated modes   h = silu(s*g) * (s*u)       s = optional per-row scale (fused RMSNorm statistic)
//   plain mode    out = acc (+ residual)      residual = optional bf16 matrix added in fp32
// then ONE rounding, a swizzled shared-memory transpose and 128-byte line stores.
#pragma once

#include "ptx_sm100.cuh"

namespace fsw {

enum GemmMode : int { kPlain = 0, kGatedSplit = 1, kGatedInterleaved = 2 };

constexpr int kBlockM = 128;
constexpr int kUmmaN = 256;
constexpr int kBlockK = 64;   // 64 bf16 = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kATileBytes = kBlockM * kBlockK * 2;      // 16 KiB
constexpr int kTmemCols = 512;
constexpr int kGemmThreads = 192;
constexpr int kNumEpilogueThreads = 128;
constexpr int kStoreStageBytes = 4 * 32 * 128;  // per epilogue warp: 32 rows x 128 bytes

// Split reduction of the last, partly filled wave (two-SM kernel only).  A 128-row half of a pair
// tile publishes its raw fp32 accumulator (all 256 columns) as one partial block.
constexpr int kTailBlockFloats = 128 * kUmmaN;            // 128 KiB per CTA and segment

struct GemmParams {
  void* out;          // bf16 (or fp32 when kOutF32) [M, n_out], row stride ld_out elements
  long long ld_out;
  int M;
  int n_out;          // number of output columns
  int tile_n;         // output columns per tile (multiple of 16; <= 256 plain, <= 128 gated)
  int K;
  int num_m_tiles;
  int num_n_tiles;
  int group_m;        // rasterisation: this many M-tiles share a sweep over N
  int hint_a, hint_b; // L2 residency class (L2Hint) of the A and B operand loads
  int k_alternate;    // two-SM kernel: every other whole tile of a cluster walks its k-blocks backwards, so
                      // that a wave starts on the operand columns the previous wave read last (L2 re-use)
  int vec_ok;         // 1 when every row start of `out` is 16-byte aligned
  // One-SM kernel, tail split by width: tiles with index >= split_from (the partly filled last wave
  // of the persistent schedule) are processed as two half-width units each.  split_from == number
  // of tiles disables it.  With half_boxes != 0 the B tensor maps are encoded with boxes of half a
  // tile's rows and a full-width tile takes two boxes per matrix.
  int split_from;
  int half_boxes;
  // Two-SM kernel, tail split along K: tiles [0, tail_first) are whole units dealt round-robin to
  // the clusters (tail_first is a multiple of the cluster count); the k-blocks of the remaining
  // tiles form one sequence that is cut into ranges of tail_len k-blocks, one range per cluster.
  // A tile whose k-blocks fall into several ranges is combined through fp32 partial blocks in
  // tail_partials; the CTA that arrives last at the tile's counter sums them in range order.
  // tail_len == 0 disables it (then tail_first == number of tiles).
  int tail_first;
  int tail_len;
  int tail_halves;    // two-SM kernel: tiles from tail_first on are two half-width units each (B boxes of 64 rows)
  float* tail_partials;          // [(cluster + tail tile) * 2 + cta rank][kTailBlockFloats]
  unsigned int* tail_counters;   // [tail tile * 2 + cta rank], zero on entry, zero again on exit
  uint32_t* status;   // device watchdog word (0 = healthy)
  unsigned long long wait_limit_ns;  // limit of every device-side wait in this launch
  // Test aid for the time-out path: when non-zero, the first CTA (the leader of the first pair) leaves
  // out one operand copy of its first k-block, so the wait for that k-block's bytes runs out, the CTA
  // unwinds and the launch reports a time-out instead of a result.  Never set outside tests.
  int withhold_one_copy;
  // Optional fusions.
  const float* row_scale;        // gated modes: per-row factor applied to gate and up before SiLU
  const void* residual;          // plain mode: bf16 [M, n_out] added to the accumulator in fp32
  long long ld_res;
  // Tensor-parallel reduce-scatter by direct stores (plain mode, bf16 out): when scatter_world > 0
  // output row r belongs to rank r / rows_per_owner and is written straight into that rank's
  // receive buffer peer_out[owner] (peer memory over NVLink, or local memory for the own rank),
  // at row  scatter_rank * rows_per_owner + (r mod rows_per_owner)  of a [world * rows_per_owner,
  // n_out] matrix with row pitch ld_out.  `out` is unused then.
  int scatter_world;
  int scatter_rank;
  int rows_per_owner;
  void* peer_out[8];
};

// Where output row `row` lives: (base pointer, row index inside that base).
__device__ __forceinline__ void* out_row_base(const GemmParams& p, int row, long long* local_row) {
  if (p.scatter_world > 0) {
    const int owner = row / p.rows_per_owner;
    *local_row = static_cast<long long>(p.scatter_rank) * p.rows_per_owner + (row - owner * p.rows_per_owner);
    return p.peer_out[owner];
  }
  *local_row = row;
  return p.out;
}

struct TileCoord {
  int m_tile;
  int n_tile;
};

// Grouped rasterisation: consecutive tile ids walk down `group_m` M-tiles
// before moving to the next N-tile, so the CTAs running at the same time share
// a few B tiles and a bounded slab of A that stays in L2.
__device__ __forceinline__ TileCoord tile_coord(int tile, const GemmParams& p) {
  const int per_group = p.group_m * p.num_n_tiles;
  const int g = tile / per_group;
  const int r = tile - g * per_group;
  const int first_m = g * p.group_m;
  const int gm = min(p.group_m, p.num_m_tiles - first_m);
  TileCoord c;
  c.n_tile = r / gm;
  c.m_tile = first_m + (r - c.n_tile * gm);
  return c;
}

// ---------------------------------------------------------------------------------------------
// Output staging.  A thread owns one output ROW in TMEM, but a warp store instruction should cover
// whole 128-byte lines of a few rows, not 16 bytes of 32 different rows (which matters most when
// the destination is another GPU: NVLink moves 128-byte payloads far better than 16-byte ones).
// Staging tile of one epilogue warp: 32 rows x 128 bytes, 16-byte segments XOR-swizzled by
// (row & 7) so that both the row-wise writes and the line-wise reads are bank-conflict free.
// ---------------------------------------------------------------------------------------------

// This thread's `ncols` (16 or 32) consecutive outputs -> segments of its row, from segment `seg0`.
template <bool kOutF32>
__device__ __forceinline__ void stage_piece(uint32_t warp_stage, uint32_t lane, int seg0, int ncols,
                                            const float (&v)[32]) {
  const uint32_t row_addr = warp_stage + lane * 128u;
  if constexpr (kOutF32) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (4 * i < ncols) {
        const uint32_t addr = row_addr + (static_cast<uint32_t>((seg0 + i) ^ (lane & 7u)) << 4);
        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v[4 * i]), "f"(v[4 * i + 1]),
                     "f"(v[4 * i + 2]), "f"(v[4 * i + 3])
                     : "memory");
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (8 * i < ncols) {
        const uint32_t addr = row_addr + (static_cast<uint32_t>((seg0 + i) ^ (lane & 7u)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pack_bf16x2(v[8 * i], v[8 * i + 1])),
                     "r"(pack_bf16x2(v[8 * i + 2], v[8 * i + 3])), "r"(pack_bf16x2(v[8 * i + 4], v[8 * i + 5])),
                     "r"(pack_bf16x2(v[8 * i + 6], v[8 * i + 7]))
                     : "memory");
      }
    }
  }
}

// Write the staged rows out.  `nsegs` 16-byte segments per row are valid, the chunk starts at
// output column `col0`, the warp's first row is `row0`.  Lane l handles segment l % 8 of rows
// l / 8, l / 8 + 4, ...: 8 lanes cover one 128-byte line.
template <bool kOutF32>
__device__ __forceinline__ void drain_chunk(const GemmParams& p, uint32_t warp_stage, uint32_t lane, int row0,
                                            int col0, int nsegs) {
  constexpr int kElemsPerSeg = kOutF32 ? 4 : 8;
  const int seg = static_cast<int>(lane & 7u);
  const int col = col0 + seg * kElemsPerSeg;
  __syncwarp();
  if (seg < nsegs && col < p.n_out) {
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int r = it * 4 + static_cast<int>(lane >> 3);
      const int row = row0 + r;
      if (row < p.M) {
        const uint32_t addr = warp_stage + static_cast<uint32_t>(r) * 128u +
                              (static_cast<uint32_t>(seg ^ (r & 7)) << 4);
        uint4 q;
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w) : "r"(addr));
        long long lrow;
        void* base = out_row_base(p, row, &lrow);
        if constexpr (kOutF32) {
          float* dst = reinterpret_cast<float*>(base) + lrow * p.ld_out + col;
          if (p.vec_ok && col + 4 <= p.n_out) {
            *reinterpret_cast<uint4*>(dst) = q;
          } else {
            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              if (col + e < p.n_out) dst[e] = __uint_as_float(w[e]);
            }
          }
        } else {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(base) + lrow * p.ld_out + col;
          if (p.vec_ok && col + 8 <= p.n_out) {
            *reinterpret_cast<uint4*>(dst) = q;
          } else {
            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
            unsigned short* d16 = reinterpret_cast<unsigned short*>(dst);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              if (col + e < p.n_out) d16[e] = static_cast<unsigned short>((w[e >> 1] >> ((e & 1) * 16)) & 0xffffu);
            }
          }
        }
      }
    }
  }
  __syncwarp();
}

// ---------------------------------------------------------------------------------------------
// Accumulator sources
// ---------------------------------------------------------------------------------------------

// This CTA's TMEM accumulator: `taddr` already carries the warp's lane field and the stage offset.
struct TmemSource {
  static constexpr bool kAsync = true;   // load() returns before the registers are written; wait() completes it
  uint32_t taddr;
  // n = 16 or 32 raw accumulator columns starting at column a0 -> r[0, n); asynchronous until wait()
  __device__ __forceinline__ void load(int a0, int n, uint32_t (&r)[32]) const {
    if (n == 32) {
      tmem_ld_32x32b_x32(taddr + static_cast<uint32_t>(a0), r);
    } else {
      uint32_t lo[16];
      tmem_ld_32x32b_x16(taddr + static_cast<uint32_t>(a0), lo);
#pragma unroll
      for (int i = 0; i < 16; ++i) r[i] = lo[i];
    }
  }
  __device__ __forceinline__ void wait() const { tmem_ld_wait(); }
};

// Partial block layout: accumulator columns in groups of four, rows fastest within a group
//   float index = ((a / 4) * 128 + row) * 4 + a % 4
// so the 32 threads (= rows) of a warp read and write 512 contiguous bytes per group.
__device__ __forceinline__ float4* partial_group(float* block, int a0, int row) {
  return reinterpret_cast<float4*>(block) + (a0 >> 2) * 128 + row;
}

// Sum of `nseg` partial blocks in index order (fixed order: results do not depend on arrival order).
struct PartialSource {
  static constexpr bool kAsync = false;  // load() sums the blocks before it returns
  float* first_block;      // block of segment 0 of this tile, for this CTA's rank
  long long seg_stride;    // floats between consecutive segments' blocks
  int nseg;
  int row;                 // this thread's row within the 128-row half
  __device__ __forceinline__ void load(int a0, int n, uint32_t (&r)[32]) const {
    float acc[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) acc[i] = 0.0f;
    for (int s = 0; s < nseg; ++s) {
      const float4* src = partial_group(first_block + s * seg_stride, a0, row);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (4 * i < n) {
          const float4 v = __ldcg(src + i * 128);
          acc[4 * i] += v.x;
          acc[4 * i + 1] += v.y;
          acc[4 * i + 2] += v.z;
          acc[4 * i + 3] += v.w;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(acc[i]);
  }
  __device__ __forceinline__ void wait() const {}
};

// Publish this thread's row of the raw accumulator (columns [0, ncols), ncols a multiple of 32).
__device__ __forceinline__ void store_partial_row(uint32_t taddr, float* block, int row, int ncols) {
#pragma unroll 1
  for (int a0 = 0; a0 < ncols; a0 += 32) {
    uint32_t r[32];
    tmem_ld_32x32b_x32(taddr + static_cast<uint32_t>(a0), r);
    tmem_ld_wait();
    float4* dst = partial_group(block, a0, row);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      __stcg(dst + i * 128, make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]),
                                        __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3])));
    }
  }
}

// Tell the compiler that r was (re)written here.  An asynchronous accumulator load names its destination
// registers long before they hold data; placed right after the wait that completes the load, this keeps every
// use of r behind that wait.
__device__ __forceinline__ void written_by_now(uint32_t (&r)[32]) {
  asm volatile(""
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
                 "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
                 "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
               :
               : "memory");
}

// ---------------------------------------------------------------------------------------------
// The epilogue of one unit of work, for one epilogue warp (32 rows starting at row0; thread = row).
// `width` output columns starting at col_base; accumulator columns as laid out by the mode.
// ---------------------------------------------------------------------------------------------
template <int kMode, bool kOutF32, typename Source>
__device__ __forceinline__ void epilogue_rows(const GemmParams& p, const Source& src, uint32_t warp_stage,
                                              uint32_t lane, int row0, int col_base, int width) {
  const int row = row0 + static_cast<int>(lane);
  float rs = 1.0f;
  if constexpr (kMode != kPlain) {
    if (p.row_scale != nullptr && row < p.M) rs = __ldg(p.row_scale + row);
  }
  // pieces of 32 output columns are staged; a chunk (128 bytes per row: 64 bf16 / 32 fp32
  // columns) is drained as soon as it is complete
  constexpr int kPiecesPerChunk = kOutF32 ? 1 : 2;
  constexpr int kSegsPerPiece = kOutF32 ? 8 : 4;  // 32 columns
  int piece = 0, chunk_col0 = col_base, chunk_segs = 0;

  // Raw accumulator values of the piece of output columns [c0, c0 + 32):
  //   plain        a = accumulator columns c0 ...
  //   split        a = gate columns c0 ..., b = up columns width + c0 ...
  //   interleaved  a, b = accumulator columns 2 c0 ... and 2 c0 + 32 ... (column 2j = up, 2j + 1 = gate)
  // Always 32 columns per request: a piece of 16 (odd width) reads 16 columns it does not use, which lie
  // inside the same accumulator (widths are multiples of 16 and below the full width whenever that happens).
  auto fetch = [&](int c0, int ncols, uint32_t (&a)[32], uint32_t (&b)[32]) {
    const int n = Source::kAsync ? 32 : ncols;
    if constexpr (kMode == kPlain) {
      src.load(c0, n, a);
    } else if constexpr (kMode == kGatedSplit) {
      src.load(c0, n, a);
      src.load(width + c0, n, b);
    } else {
      src.load(2 * c0, 32, a);
      if (Source::kAsync || ncols == 32) {
        src.load(2 * c0 + 32, 32, b);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) b[i] = 0u;
      }
    }
  };
  auto complete = [&](uint32_t (&a)[32], uint32_t (&b)[32]) {
    src.wait();
    if constexpr (Source::kAsync) {
      written_by_now(a);
      if constexpr (kMode != kPlain) written_by_now(b);
    }
  };

  // With an asynchronous source the request for the next piece is in flight while this piece is converted,
  // staged and stored; the registers it will land in are not touched until the wait at the end of the
  // iteration (no value crosses the loop's back edge before it is complete).
  uint32_t ra[32], rb[32];
  if constexpr (Source::kAsync) {
    fetch(0, min(32, width), ra, rb);
    complete(ra, rb);
  }
#pragma unroll 1
  for (int c0 = 0; c0 < width; c0 += 32) {
    if (col_base + c0 >= p.n_out) break;  // warp-uniform: the rest of the tile is past the edge
    const int ncols = min(32, width - c0);  // 32, or 16 for the last piece of an odd width
    float v[32];
    // plain mode: residual row segment first, so that its latency overlaps the accumulator read (ordinary
    // loads: the residual may be the output buffer itself; a warp reads a chunk's elements before it writes them)
    uint4 res[4];
    bool with_res = false;
    if constexpr (kMode == kPlain) {
      with_res = p.residual != nullptr && row < p.M;
      if (with_res) {
        const __nv_bfloat16* rrow =
            reinterpret_cast<const __nv_bfloat16*>(p.residual) + static_cast<long long>(row) * p.ld_res + col_base + c0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          res[i] = make_uint4(0u, 0u, 0u, 0u);
          if (8 * i < ncols && col_base + c0 + 8 * i < p.n_out) res[i] = *(reinterpret_cast<const uint4*>(rrow) + i);
        }
      }
    }
    if constexpr (!Source::kAsync) {
      fetch(c0, ncols, ra, rb);
      complete(ra, rb);
    }
    if constexpr (kMode == kPlain) {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(ra[i]);
      if (with_res) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint32_t w[4] = {res[i].x, res[i].y, res[i].z, res[i].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            v[8 * i + 2 * e] += __uint_as_float(w[e] << 16);
            v[8 * i + 2 * e + 1] += __uint_as_float(w[e] & 0xffff0000u);
          }
        }
      }
    } else if constexpr (kMode == kGatedSplit) {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = silu_mul(rs * __uint_as_float(ra[i]), rs * __uint_as_float(rb[i]));
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        v[i] = silu_mul(rs * __uint_as_float(ra[2 * i + 1]), rs * __uint_as_float(ra[2 * i]));
        v[16 + i] = silu_mul(rs * __uint_as_float(rb[2 * i + 1]), rs * __uint_as_float(rb[2 * i]));
      }
    }
    uint32_t na[32], nb[32];
    if constexpr (Source::kAsync) {
      // the next piece (or, at the end, this one again: the request is unconditional so that nothing but the
      // staging code sits between it and its wait)
      const bool more = c0 + 32 < width && col_base + c0 + 32 < p.n_out;
      fetch(more ? c0 + 32 : c0, 32, na, nb);
    }
    if (piece == 0) {
      chunk_col0 = col_base + c0;
      chunk_segs = 0;
    }
    stage_piece<kOutF32>(warp_stage, lane, piece * kSegsPerPiece, ncols, v);
    chunk_segs += ncols / (kOutF32 ? 4 : 8);
    if (++piece == kPiecesPerChunk) {
      drain_chunk<kOutF32>(p, warp_stage, lane, row0, chunk_col0, chunk_segs);
      piece = 0;
    }
    if constexpr (Source::kAsync) {
      complete(na, nb);
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        ra[i] = na[i];
        if constexpr (kMode != kPlain) rb[i] = nb[i];
      }
    }
  }
  if (piece != 0) drain_chunk<kOutF32>(p, warp_stage, lane, row0, chunk_col0, chunk_segs);
}

}  // namespace fsw
