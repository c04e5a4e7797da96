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

#include "gemm_common.cuh"

namespace fsw {

constexpr int kStages = 4;
constexpr int kBTileBytes = kUmmaN * kBlockK * 2;        // 32 KiB (room for the widest tile)
constexpr int kStageBytes = kATileBytes + kBTileBytes;  // 48 KiB
// ring + 1 KiB alignment slack + barriers / bookkeeping + store staging
constexpr int kGemmSmemBytes = kStages * kStageBytes + 1024 + 256 + kStoreStageBytes;

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
  const Watchdog wd{abort_flag, p.status, p.wait_limit_ns};

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
          if (!(p.withhold_one_copy != 0 && blockIdx.x == 0 && unit == 0 && kb == 0)) {
            tma_load_2d(b_dst, &map_b0, full_bar(stage), kb * kBlockK, b_row);
          }
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
              if (global_timer_ns() - t0 > kDrainLimitNs) {  // 50 ms
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
          if (global_timer_ns() - t0 > kDrainLimitNs) {
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
      epilogue_rows<kMode, kOutF32>(p, TmemSource{t_acc}, warp_stage, lane, row0, un.col0, un.width);
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
