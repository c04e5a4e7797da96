// Persistent, warp-specialised tcgen05 GEMM for the two prefill stages of the
// SwiGLU MLP forward:
//
//   gate-up stage  h[M,F]   = silu(x Wg^T) * (x Wu^T)      (gated epilogue)
//   down stage     out[M,d] = h Wd^T                        (plain epilogue)
//
// All operands are K-major ("TN"): A is [rows, K] row-major, B is [cols, K]
// row-major, exactly the layout of x / W_gate / W_up / h / W_down, so one TMA
// box of 64 bf16 x 128 rows with the 128-byte swizzle is a ready-made UMMA
// operand.  One CTA per SM:
//
//   warp 0       TMA producer (one lane): fills a 4-deep ring of
//                {A 128x64, B up to 256x64} stages, 48 KiB each
//   warp 1       TMEM owner + MMA issuer (one lane): 4 x tcgen05.mma
//                (M=128, N<=256, K=16) per stage into one of two 256-column
//                TMEM accumulators
//   warps 2..5   epilogue: tcgen05.ld the finished accumulator (one thread
//                per output row), apply SiLU(g)*u, round once to bf16, store
//
// The accumulator is double-buffered (2 x 256 of the 512 TMEM columns), so the
// epilogue of tile t overlaps the main loop of tile t+1.
//
// The width of a tile is a run-time choice (`tile_n` output columns, a multiple
// of 16): the host picks the width that wastes the least of the last wave of
// the persistent schedule.  The MMA N extent and what the B tile holds depend
// on the mode:
//   kPlain             tile_n consecutive rows of W              N = tile_n   (<= 256)
//   kGatedSplit        tile_n rows of W_gate, then of W_up       N = 2 tile_n (<= 256)
//   kGatedInterleaved  2 tile_n consecutive rows of the reference's packed W1W3
//                      (even row = up, odd row = gate; reference
//                      csrc/SwiGLU/swiglu.cu:376-383)            N = 2 tile_n (<= 256)
//
// Ragged edges cost nothing extra: TMA zero-fills out-of-range rows and
// K-columns on load, and stores are predicated per row / column.
#pragma once

#include "ptx_sm100.cuh"

namespace fsw {

enum GemmMode : int { kPlain = 0, kGatedSplit = 1, kGatedInterleaved = 2 };

constexpr int kBlockM = 128;
constexpr int kUmmaN = 256;
constexpr int kBlockK = 64;   // 64 bf16 = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kStages = 4;
constexpr int kATileBytes = kBlockM * kBlockK * 2;      // 16 KiB
constexpr int kBTileBytes = kUmmaN * kBlockK * 2;        // 32 KiB (room for the widest tile)
constexpr int kStageBytes = kATileBytes + kBTileBytes;  // 48 KiB
constexpr int kTmemCols = 512;
constexpr int kGemmThreads = 192;
constexpr int kNumEpilogueThreads = 128;
constexpr int kStoreStageBytes = 4 * 32 * 128;  // per epilogue warp: 32 rows x 128 bytes
// ring + 1 KiB alignment slack + barriers / bookkeeping + store staging
constexpr int kGemmSmemBytes = kStages * kStageBytes + 1024 + 256 + kStoreStageBytes;

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
  int vec_ok;         // 1 when every row start of `out` is 16-byte aligned
  // Tail split: tiles with index >= split_from (the partly filled last wave of the persistent
  // schedule) are processed as two half-width units each, so that twice as many SMs share that
  // wave.  split_from == number of tiles disables it.  With half_boxes != 0 the B tensor maps are
  // encoded with boxes of half a tile's rows and a full-width tile takes two boxes per matrix.
  int split_from;
  int half_boxes;
  uint32_t* status;   // device watchdog word (0 = healthy)
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

// Output goes through a small shared-memory transpose so that global (or peer) stores are
// coalesced: a thread owns one output ROW in TMEM, but a warp store instruction should cover whole
// 128-byte lines of a few rows, not 16 bytes of 32 different rows (which matters most when the
// destination is another GPU: NVLink moves 128-byte payloads far better than 16-byte ones).
//
// Staging tile of one epilogue warp: 32 rows x 128 bytes, 16-byte segments XOR-swizzled by (row & 7)
// so that both the row-wise writes and the line-wise reads are bank-conflict free.
//
// stage_piece: this thread's `ncols` (16 or 32) consecutive outputs -> segments of its row, starting
// at 16-byte segment `seg0`.
// One unit of work: a whole tile, or the left / right half of a tail tile.
struct Unit {
  int m_tile;
  int col0;   // first output column
  int width;  // output columns (tile_n or tile_n / 2)
};
__device__ __forceinline__ Unit unit_coord(int u, const GemmParams& p) {
  int tile = u, half = -1;
  if (u >= p.split_from) {
    const int s = u - p.split_from;
    tile = p.split_from + (s >> 1);
    half = s & 1;
  }
  const TileCoord tc = tile_coord(tile, p);
  Unit r;
  r.m_tile = tc.m_tile;
  r.width = half < 0 ? p.tile_n : p.tile_n / 2;
  r.col0 = tc.n_tile * p.tile_n + (half > 0 ? p.tile_n / 2 : 0);
  return r;
}

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

// drain_chunk: write the staged rows out.  `nsegs` 16-byte segments per row are valid, the chunk
// starts at output column `col0`, the warp's first row is `row0`.  Lane l handles segment l % 8 of
// rows l / 8, l / 8 + 4, ...: 8 lanes cover one 128-byte line.
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

// 16 or 32 accumulator columns of this thread's row into r[0, ncols).
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, int ncols, uint32_t (&r)[32]) {
  if (ncols == 32) {
    tmem_ld_32x32b_x32(taddr, r);
  } else {
    uint32_t lo[16];
    tmem_ld_32x32b_x16(taddr, lo);
#pragma unroll
    for (int i = 0; i < 16; ++i) r[i] = lo[i];
  }
}

template <int kMode, bool kOutF32>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a,
                    const __grid_constant__ CUtensorMap map_b0,
                    const __grid_constant__ CUtensorMap map_b1, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  // The 128-byte swizzle pattern repeats every 1024 bytes: tiles must start on that boundary.
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + kStages * kStageBytes;
  // barrier block: full[4], empty[4], tmem_full[2], tmem_empty[2], drain, tmem ptr, abort flag
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
  const uint32_t drain_bar = bar_base + 8u * (2 * kStages + 4);
  uint8_t* generic_base = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t* tmem_ptr_slot =
      reinterpret_cast<volatile uint32_t*>(generic_base + kStages * kStageBytes + 8 * (2 * kStages + 5));
  volatile uint32_t* abort_flag = tmem_ptr_slot + 1;

  const int warp = threadIdx.x >> 5;
  const uint32_t lane = lane_id();
  const Watchdog wd{abort_flag, p.status};

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), kNumEpilogueThreads);
    }
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b0);
    prefetch_tensormap(&map_b1);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_ptr_slot)), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_slot;

  const int num_tiles = p.num_m_tiles * p.num_n_tiles;
  const int num_units = p.split_from + 2 * (num_tiles - p.split_from);
  const int num_kb = (p.K + kBlockK - 1) / kBlockK;
  // MMA N extent (= accumulator columns in use, = B rows in shared memory) of a unit of `width` columns
  auto mma_n_of = [&](int width) { return (kMode == kPlain) ? width : 2 * width; };

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t issued_mask = 0, last_parity_mask = 0;
      bool alive = true;
      for (int unit = blockIdx.x; unit < num_units && alive; unit += gridDim.x) {
        const Unit un = unit_coord(unit, p);
        const int m0 = un.m_tile * kBlockM;
        // first B row of this unit: rows of W (plain), of W_gate and W_up (split), or of the
        // packed W1W3 (interleaved: two rows per output column)
        const int b_row = (kMode == kGatedInterleaved) ? 2 * un.col0 : un.col0;
        const uint32_t stage_tx_bytes = kATileBytes + static_cast<uint32_t>(mma_n_of(un.width)) * (kBlockK * 2);
        // a full-width tile needs two boxes per matrix when the maps hold half-width boxes
        const bool two_boxes = p.half_boxes != 0 && un.width == p.tile_n;
        const int half_rows = (kMode == kGatedInterleaved) ? p.tile_n : p.tile_n / 2;  // rows of a half box
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!wd.wait(empty_bar(stage), phase ^ 1u, kSiteProducerEmpty)) {
            alive = false;
            break;
          }
          const uint32_t a_dst = smem_base + stage * kStageBytes;
          const uint32_t b_dst = a_dst + kATileBytes;
          mbar_arrive_expect_tx(full_bar(stage), stage_tx_bytes);
          tma_load_2d(a_dst, &map_a, full_bar(stage), kb * kBlockK, m0);
          tma_load_2d(b_dst, &map_b0, full_bar(stage), kb * kBlockK, b_row);
          if (two_boxes) {
            tma_load_2d(b_dst + half_rows * (kBlockK * 2), &map_b0, full_bar(stage), kb * kBlockK, b_row + half_rows);
          }
          if (kMode == kGatedSplit) {
            // W_up rows go right behind the W_gate rows (width * 128 bytes, a multiple of 1024)
            const uint32_t up_dst = b_dst + un.width * (kBlockK * 2);
            tma_load_2d(up_dst, &map_b1, full_bar(stage), kb * kBlockK, b_row);
            if (two_boxes) {
              tma_load_2d(up_dst + half_rows * (kBlockK * 2), &map_b1, full_bar(stage), kb * kBlockK, b_row + half_rows);
            }
          }
          issued_mask |= 1u << stage;
          last_parity_mask = (last_parity_mask & ~(1u << stage)) | (phase << stage);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (wd.aborted()) {
        // Unwinding: let every copy this thread started land before the CTA exits.
        for (int s = 0; s < kStages; ++s) {
          if (issued_mask & (1u << s)) {
            const uint32_t par = (last_parity_mask >> s) & 1u;
            const unsigned long long t0 = global_timer_ns();
            while (!mbar_try_wait(full_bar(s), par)) {
              if (global_timer_ns() - t0 > 50000000ull) {  // 50 ms
                wd.give_up(kSiteDrainTma);
                break;
              }
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0) {
      const uint32_t idesc_full = umma_idesc_bf16_f32(kBlockM, mma_n_of(p.tile_n));
      const uint32_t idesc_half = umma_idesc_bf16_f32(kBlockM, mma_n_of(p.tile_n / 2));
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool alive = true;
      for (int unit = blockIdx.x; unit < num_units && alive; unit += gridDim.x) {
        const uint32_t idesc = unit < p.split_from ? idesc_full : idesc_half;
        if (!wd.wait(tempty_bar(acc), acc_phase ^ 1u, kSiteMmaTmemEmpty)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kUmmaN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!wd.wait(full_bar(stage), phase, kSiteMmaFull)) {
            alive = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_base + stage * kStageBytes;
          const uint64_t a_desc = umma_desc_k_sw128(a_addr);
          const uint64_t b_desc = umma_desc_k_sw128(a_addr + kATileBytes);
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            // advance 16 elements = 32 bytes along K inside the swizzled row: +2 in >>4 units
            umma_bf16_ss(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc,
                         (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));  // stage reusable once these MMAs retire
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!alive) break;
        umma_commit(tfull_bar(acc));  // accumulator complete
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
      if (wd.aborted()) {
        // Unwinding: wait for whatever MMAs are still in flight before TMEM is freed.
        umma_commit(drain_bar);
        const unsigned long long t0 = global_timer_ns();
        while (!mbar_try_wait(drain_bar, 0)) {
          if (global_timer_ns() - t0 > 50000000ull) {
            wd.give_up(kSiteDrainMma);
            break;
          }
        }
      }
    }
  } else {
    // -------------------------------- epilogue --------------------------------
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) belong to this warp
    const uint32_t lane_field = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t warp_stage = bar_base + 256u + static_cast<uint32_t>(quarter) * (32u * 128u);
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int unit = blockIdx.x; unit < num_units; unit += gridDim.x) {
      const Unit un = unit_coord(unit, p);
      uint32_t ok = 1;
      if (lane == 0) ok = wd.wait(tfull_bar(acc), acc_phase, kSiteEpilogueFull) ? 1u : 0u;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      __syncwarp();
      tc_fence_after_sync();
      const uint32_t t_acc = tmem_base + lane_field + static_cast<uint32_t>(acc * kUmmaN);
      const int row0 = un.m_tile * kBlockM + quarter * 32;  // first output row of this warp
      const int col_base = un.col0;
      const int width = un.width;
      // pieces of 32 output columns are staged; a chunk (128 bytes per row: 64 bf16 / 32 fp32
      // columns) is drained as soon as it is complete
      constexpr int kPiecesPerChunk = kOutF32 ? 1 : 2;
      int piece = 0, chunk_col0 = col_base, chunk_segs = 0;
#pragma unroll 1
      for (int c0 = 0; c0 < width; c0 += 32) {
        if (col_base + c0 >= p.n_out) break;  // warp-uniform: the rest of the tile is past the edge
        const int ncols = min(32, width - c0);  // 32, or 16 for the last piece of an odd width
        float v[32];
        if constexpr (kMode == kPlain) {
          uint32_t r[32];
          tmem_ld_cols(t_acc + c0, ncols, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
        } else if constexpr (kMode == kGatedSplit) {
          uint32_t g[32], u[32];
          tmem_ld_cols(t_acc + c0, ncols, g);             // gate columns [0, width)
          tmem_ld_cols(t_acc + width + c0, ncols, u);     // up columns [width, 2 width)
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = silu_mul(__uint_as_float(g[i]), __uint_as_float(u[i]));
        } else {
          // accumulator column 2j = up (linear), 2j+1 = gate (SiLU)
          uint32_t lo[32], hi[32];
          tmem_ld_32x32b_x32(t_acc + 2 * c0, lo);
          if (ncols == 32) {
            tmem_ld_32x32b_x32(t_acc + 2 * c0 + 32, hi);
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) hi[i] = 0u;
          }
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            v[i] = silu_mul(__uint_as_float(lo[2 * i + 1]), __uint_as_float(lo[2 * i]));
            v[16 + i] = silu_mul(__uint_as_float(hi[2 * i + 1]), __uint_as_float(hi[2 * i]));
          }
        }
        constexpr int kSegsPerPiece = kOutF32 ? 8 : 4;  // 32 columns
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
      }
      if (piece != 0) drain_chunk<kOutF32>(p, warp_stage, lane, row0, chunk_col0, chunk_segs);
      tc_fence_before_sync();
      mbar_arrive(tempty_bar(acc));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  // -------------------------------- teardown ----------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace fsw
