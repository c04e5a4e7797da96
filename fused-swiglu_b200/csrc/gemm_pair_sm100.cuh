// Two-SM variant of the tiled tcgen05 GEMM: a cluster of two CTAs works on one 256-row tile with
// `tcgen05.mma.cta_group::2`.  Each CTA loads its own 128 rows of A and only HALF of the B tile
// (the MMA reads the other half from the partner's shared memory), so a k-block costs each SM
// 32 KiB of L2 -> SM traffic instead of 48 KiB, and the ring holds 6 stages instead of 4.  No
// multicast loads are involved: every TMA load is an ordinary per-CTA load.
//
//   rank 0 ("leader")  warp 0 producer, warp 1 MMA issuer for BOTH CTAs, warps 2-5 epilogue
//   rank 1 ("partner") warp 0 producer (its loads count their bytes on the LEADER's stage barrier),
//                      warps 2-5 epilogue (its own 128 rows, from its own TMEM)
//
// What the B half of a CTA holds (N = MMA columns, half of them per CTA, leader first):
//   kPlain             rows [n0 + rank * tile_n/2, +tile_n/2) of W
//   kGatedSplit        leader: tile_n rows of W_gate; partner: tile_n rows of W_up
//   kGatedInterleaved  rows [2 n0 + rank * tile_n, +tile_n) of the packed W1W3
// so the accumulator columns mean the same as in the one-SM kernel and the epilogue is shared.
// Results are bit-identical to the one-SM kernel; the host selects this kernel when the problem
// fills at least one wave of pair tiles.
#pragma once

#include "gemm_sm100.cuh"

namespace fsw {

constexpr int kPairStages = 6;
constexpr int kPairBHalfBytes = 128 * kBlockK * 2;                       // 16 KiB
constexpr int kPairStageBytes = kATileBytes + kPairBHalfBytes;           // 32 KiB
constexpr int kPairSmemBytes = kPairStages * kPairStageBytes + 1024 + 512 + kStoreStageBytes;

__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  // arrive on the barrier at this offset in BOTH CTAs of the pair once the MMAs issued so far retire
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"(static_cast<uint16_t>(3))
      : "memory");
}

template <int kMode, bool kOutF32>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b0,
                 const __grid_constant__ CUtensorMap map_b1, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + kPairStages * kPairStageBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (2 * kPairStages + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (3 * kPairStages + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (3 * kPairStages + 2 + a); };
  const uint32_t drain_bar = bar_base + 8u * (3 * kPairStages + 4);
  uint8_t* generic_base = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t* tmem_ptr_slot = reinterpret_cast<volatile uint32_t*>(
      generic_base + kPairStages * kPairStageBytes + 8 * (3 * kPairStages + 5));
  volatile uint32_t* abort_flag = tmem_ptr_slot + 1;

  const int warp = threadIdx.x >> 5;
  const uint32_t lane = lane_id();
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const Watchdog wd{abort_flag, p.status};

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 8);  // 4 epilogue warps in each of the two CTAs
    }
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b0);
    prefetch_tensormap(&map_b1);
  }
  if (warp == 1) {
    tmem_alloc_2cta(smem_u32(const_cast<uint32_t*>(tmem_ptr_slot)), kTmemCols);
    tmem_relinquish_2cta();
  }
  tc_fence_before_sync();
  __syncthreads();
  // barriers of both CTAs are initialised before anybody signals across the pair
  cluster_arrive();
  cluster_wait();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_slot;

  // p.num_m_tiles counts 256-row pair tiles here
  const int num_tiles = p.num_m_tiles * p.num_n_tiles;
  const int num_kb = (p.K + kBlockK - 1) / kBlockK;
  const int num_clusters = gridDim.x / 2;
  const int cluster_id = blockIdx.x / 2;
  const int mma_n = (kMode == kPlain) ? p.tile_n : 2 * p.tile_n;  // columns of the pair's accumulator
  const int b_half_rows = mma_n / 2;
  const uint32_t stage_tx_bytes = kATileBytes + static_cast<uint32_t>(b_half_rows) * (kBlockK * 2);

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t issued_mask = 0, last_parity_mask = 0;
      bool alive = true;
      for (int tile = cluster_id; tile < num_tiles && alive; tile += num_clusters) {
        const TileCoord tc = tile_coord(tile, p);
        const int m0 = tc.m_tile * 256 + static_cast<int>(rank) * 128;
        const int n0 = tc.n_tile * p.tile_n;
        const CUtensorMap* bmap = &map_b0;
        int b_row;
        if (kMode == kPlain) {
          b_row = n0 + static_cast<int>(rank) * b_half_rows;
        } else if (kMode == kGatedSplit) {
          b_row = n0;  // leader: W_gate rows, partner: W_up rows
          if (rank == 1) bmap = &map_b1;
        } else {
          b_row = 2 * n0 + static_cast<int>(rank) * b_half_rows;
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!wd.wait(empty_bar(stage), phase ^ 1u, kSiteProducerEmpty)) {
            alive = false;
            break;
          }
          const uint32_t a_dst = smem_base + stage * kPairStageBytes;
          // one barrier per stage, in the leader: it expects the bytes of both CTAs' halves
          if (rank == 0) mbar_arrive_expect_tx(full_bar(stage), 2u * stage_tx_bytes);
          const uint32_t leader_full = map_to_cta(full_bar(stage), 0);
          tma_load_2d_pair(a_dst, &map_a, leader_full, kb * kBlockK, m0);
          tma_load_2d_pair(a_dst + kATileBytes, bmap, leader_full, kb * kBlockK, b_row);
          issued_mask |= 1u << stage;
          last_parity_mask = (last_parity_mask & ~(1u << stage)) | (phase << stage);
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (wd.aborted()) {
        if (rank == 0) {
          for (int s = 0; s < kPairStages; ++s) {
            if (issued_mask & (1u << s)) {
              const uint32_t par = (last_parity_mask >> s) & 1u;
              const unsigned long long t0 = global_timer_ns();
              while (!mbar_try_wait(full_bar(s), par)) {
                if (global_timer_ns() - t0 > 50000000ull) {
                  wd.give_up(kSiteDrainTma);
                  break;
                }
              }
            }
          }
        } else {
          // the partner's copies are counted in the leader: give them time to land before unwinding
          const unsigned long long t0 = global_timer_ns();
          while (global_timer_ns() - t0 < 100000ull) {
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      // ------------------------------- leader: MMA issuer for the pair -------------------------------
      const uint32_t idesc = umma_idesc_bf16_f32(256, mma_n);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool alive = true;
      for (int tile = cluster_id; tile < num_tiles && alive; tile += num_clusters) {
        if (!wd.wait<true>(tempty_bar(acc), acc_phase ^ 1u, kSiteMmaTmemEmpty)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kUmmaN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!wd.wait<true>(full_bar(stage), phase, kSiteMmaFull)) {
            alive = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_base + stage * kPairStageBytes;
          const uint64_t a_desc = umma_desc_k_sw128(a_addr);
          const uint64_t b_desc = umma_desc_k_sw128(a_addr + kATileBytes);
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            umma_bf16_ss_2cta(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit_pair(empty_bar(stage));  // both CTAs may refill this stage once the MMAs retire
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!alive) break;
        umma_commit_pair(tfull_bar(acc));  // accumulator complete, in both CTAs
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
      if (wd.aborted()) {
        umma_commit_2cta(drain_bar);
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
    // -------------------------------- epilogue (both CTAs, own 128 rows) --------------------------------
    const int quarter = warp & 3;
    const uint32_t lane_field = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t warp_stage = bar_base + 512u + static_cast<uint32_t>(quarter) * (32u * 128u);
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = cluster_id; tile < num_tiles; tile += num_clusters) {
      const TileCoord tc = tile_coord(tile, p);
      uint32_t ok = 1;
      if (lane == 0) ok = wd.wait(tfull_bar(acc), acc_phase, kSiteEpilogueFull) ? 1u : 0u;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      __syncwarp();
      tc_fence_after_sync();
      const uint32_t t_acc = tmem_base + lane_field + static_cast<uint32_t>(acc * kUmmaN);
      const int row0 = tc.m_tile * 256 + static_cast<int>(rank) * 128 + quarter * 32;
      const int col_base = tc.n_tile * p.tile_n;
      const int width = p.tile_n;
      constexpr int kPiecesPerChunk = kOutF32 ? 1 : 2;
      int piece = 0, chunk_col0 = col_base, chunk_segs = 0;
#pragma unroll 1
      for (int c0 = 0; c0 < width; c0 += 32) {
        if (col_base + c0 >= p.n_out) break;
        const int ncols = min(32, width - c0);
        float v[32];
        if constexpr (kMode == kPlain) {
          uint32_t r[32];
          tmem_ld_cols(t_acc + c0, ncols, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
        } else if constexpr (kMode == kGatedSplit) {
          uint32_t g[32], u[32];
          tmem_ld_cols(t_acc + c0, ncols, g);
          tmem_ld_cols(t_acc + width + c0, ncols, u);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = silu_mul(__uint_as_float(g[i]), __uint_as_float(u[i]));
        } else {
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
        constexpr int kSegsPerPiece = kOutF32 ? 8 : 4;
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
      // this warp is done with the accumulator: tell the leader's MMA issuer (one arrival per warp)
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (rank == 0) {
          mbar_arrive(tempty_bar(acc));
        } else {
          mbar_arrive_cluster(map_to_cta(tempty_bar(acc), 0));
        }
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  // -------------------------------- teardown ----------------------------------
  tc_fence_before_sync();
  __syncthreads();
  // nobody leaves (or frees TMEM) while the partner may still signal into this CTA
  cluster_arrive();
  cluster_wait();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc_2cta(tmem_base, kTmemCols);
  }
}

}  // namespace fsw
