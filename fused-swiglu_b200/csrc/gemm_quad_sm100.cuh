// Two-SM kernel with 512-row tiles: the variant for problems of many waves, where the power the chip spends
// on moving operands decides the clock it can hold.  A cluster of two CTAs owns a tile of 512 rows; each CTA
// holds 256 rows of A per k-block (two 128-row sub-tiles) and half of the B tile, and every k-step issues two
// `tcgen05.mma.cta_group::2` instructions (M = 256 across the pair, one per sub-tile) that share the B operand.
// Against the 256-row kernel (gemm_pair_sm100.cuh) a k-block moves 48 KiB instead of 2 x 32 KiB from L2 into
// an SM per 2 x the flops (0.75 x the bytes per flop), a wave of tiles touches fewer distinct operand rows per
// flop, and both accumulators together fill the 512 TMEM columns, so there is no second accumulator stage: the
// epilogue of a tile overlaps only the first k-blocks of the next one (below).  Measured at the 70B shape under
// the 1 kW cap this trade wins; on few-wave problems the coarser tiles lose more to the partly filled last wave
// than they gain, and the host keeps the 256-row kernel there.
//
//   rank 0 ("leader")  warp 0 producer, warp 1 MMA issuer for BOTH CTAs, warps 2-5 epilogue of sub-tile 0,
//                      warps 6-9 epilogue of sub-tile 1
//   rank 1 ("partner") warp 0 producer (bytes counted on the LEADER's stage barrier), warps 2-9 epilogue
//
// Rows of a tile: CTA `rank`, sub-tile h -> rows  m_tile * 512 + rank * 256 + h * 128 + [0, 128).
// Accumulator of sub-tile h: TMEM columns [h * 256, h * 256 + 256) of each CTA, laid out by the mode exactly as
// in the other kernels, so the epilogue is the shared one and results are bit-identical (same k order, same
// MMA shape).  B halves per CTA as in the 256-row kernel.
//
// Hand-over between tiles.  With no spare accumulator the tensor pipe idles while a tile's accumulators are
// drained, so the epilogue is made short rather than hidden: two groups of four warps drain the two sub-tiles
// at the same time and release them separately.  The MMA issuer starts the next tile with the sub-tile-0 MMAs
// of the first k-blocks (as many as the ring has stages) as soon as accumulator 0 is free, then waits for
// accumulator 1, issues the sub-tile-1 MMAs of those k-blocks and releases their stages; from there on both
// sub-tiles go k-block by k-block - except for the last three k-blocks of the tile, where sub-tile 0 is finished
// first (its accumulator is handed to its epilogue group while sub-tile 1's last MMAs still run).  Each
// accumulator has its own "full" barrier.
#pragma once

#include "gemm_common.cuh"
#include "gemm_pair_sm100.cuh"

namespace fsw {

constexpr int kQuadStages = 4;
constexpr int kQuadABytes = 2 * kATileBytes;                             // 32 KiB: two 128-row sub-tiles
constexpr int kQuadStageBytes = kQuadABytes + kPairBHalfBytes;           // 48 KiB
constexpr int kQuadThreads = 320;                                        // producer, MMA, 2 x 4 epilogue warps
constexpr int kQuadSmemBytes = kQuadStages * kQuadStageBytes + 1024 + 512 + 2 * kStoreStageBytes;
constexpr int kQuadTileRows = 512;

template <int kMode, bool kOutF32>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kQuadThreads, 1)
gemm_quad_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b0,
                 const __grid_constant__ CUtensorMap map_b1, const GemmParams p) {
  // map_a: 128-row boxes of A; map_b0 / map_b1: 128-row boxes of the B operand(s)
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + kQuadStages * kQuadStageBytes;
  // barrier block: full[4], empty[4], tmem_full[2], tmem_empty[2], drain, then bookkeeping words
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kQuadStages + s); };
  auto tfull_bar = [&](int h) { return bar_base + 8u * (2 * kQuadStages + h); };
  auto tempty_bar = [&](int h) { return bar_base + 8u * (2 * kQuadStages + 2 + h); };
  const uint32_t drain_bar = bar_base + 8u * (2 * kQuadStages + 4);
  uint8_t* generic_base = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t* tmem_ptr_slot = reinterpret_cast<volatile uint32_t*>(
      generic_base + kQuadStages * kQuadStageBytes + 8 * (2 * kQuadStages + 5));
  volatile uint32_t* abort_flag = tmem_ptr_slot + 1;
  volatile uint32_t* epi_ok = tmem_ptr_slot + 2;  // two entries per epilogue group, alternating per tile

  const int warp = threadIdx.x >> 5;
  const uint32_t lane = lane_id();
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const Watchdog wd{abort_flag, p.status, p.wait_limit_ns};

  if (threadIdx.x == 0) {
    for (int s = 0; s < kQuadStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(tfull_bar(0), 1);
    mbar_init(tfull_bar(1), 1);
    mbar_init(tempty_bar(0), 8);  // 4 epilogue warps in each of the two CTAs
    mbar_init(tempty_bar(1), 8);
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

  // p.num_m_tiles counts 512-row tiles here
  const int num_kb = (p.K + kBlockK - 1) / kBlockK;
  const int num_tiles = p.num_m_tiles * p.num_n_tiles;
  const int num_clusters = gridDim.x / 2;
  const int cluster_id = blockIdx.x / 2;
  const int mma_n = (kMode == kPlain) ? p.tile_n : 2 * p.tile_n;  // columns of one accumulator
  const int b_half_rows = mma_n / 2;                              // B rows a CTA holds per k-block

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t issued_mask = 0, last_parity_mask = 0;
      bool alive = true;
      bool withhold = p.withhold_one_copy != 0 && blockIdx.x == 0;  // one-shot, leader of the first pair
      const uint32_t stage_tx_bytes = kQuadABytes + static_cast<uint32_t>(b_half_rows) * (kBlockK * 2);
      const uint64_t pol_a = l2_policy_of(p.hint_a), pol_b = l2_policy_of(p.hint_b);
      for (int tile = cluster_id; tile < num_tiles && alive; tile += num_clusters) {
        const TileCoord tc = tile_coord(tile, p);
        const int m0 = tc.m_tile * kQuadTileRows + static_cast<int>(rank) * 256;
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
          const uint32_t a_dst = smem_base + stage * kQuadStageBytes;
          // one barrier per stage, in the leader: it expects the bytes of both CTAs
          if (rank == 0) mbar_arrive_expect_tx(full_bar(stage), 2u * stage_tx_bytes);
          const uint32_t leader_full = map_to_cta(full_bar(stage), 0);
          // no residency class: the plain load (the hardware's default policy), else the load with a hint
          if (p.hint_a == kL2Default) {
            tma_load_2d_pair(a_dst, &map_a, leader_full, kb * kBlockK, m0);
            tma_load_2d_pair(a_dst + kATileBytes, &map_a, leader_full, kb * kBlockK, m0 + 128);
          } else {
            tma_load_2d_pair_hint(a_dst, &map_a, leader_full, kb * kBlockK, m0, pol_a);
            tma_load_2d_pair_hint(a_dst + kATileBytes, &map_a, leader_full, kb * kBlockK, m0 + 128, pol_a);
          }
          if (!withhold) {
            if (p.hint_b == kL2Default) {
              tma_load_2d_pair(a_dst + kQuadABytes, bmap, leader_full, kb * kBlockK, b_row);
            } else {
              tma_load_2d_pair_hint(a_dst + kQuadABytes, bmap, leader_full, kb * kBlockK, b_row, pol_b);
            }
          }
          withhold = false;
          issued_mask |= 1u << stage;
          last_parity_mask = (last_parity_mask & ~(1u << stage)) | (phase << stage);
          if (++stage == kQuadStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (wd.aborted()) {
        if (rank == 0) {
          for (int s = 0; s < kQuadStages; ++s) {
            if (issued_mask & (1u << s)) {
              const uint32_t par = (last_parity_mask >> s) & 1u;
              const unsigned long long t0 = global_timer_ns();
              while (!mbar_try_wait(full_bar(s), par)) {
                if (global_timer_ns() - t0 > kDrainLimitNs) {
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
      const uint32_t d0 = tmem_base, d1 = tmem_base + static_cast<uint32_t>(kUmmaN);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase = 0;
      bool alive = true;
      // the MMAs of one sub-tile for the k-block held in stage s
      auto issue = [&](int s, int h, uint32_t d_tmem, bool first_kb) {
        const uint32_t a_addr = smem_base + s * kQuadStageBytes;
        const uint64_t a_desc = umma_desc_k_sw128(a_addr + h * kATileBytes);
        const uint64_t b_desc = umma_desc_k_sw128(a_addr + kQuadABytes);
#pragma unroll
        for (int k = 0; k < kBlockK / kUmmaK; ++k) {
          umma_bf16_ss_2cta(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc, (!first_kb || k > 0) ? 1u : 0u);
        }
      };
      for (int tile = cluster_id; tile < num_tiles && alive; tile += num_clusters) {
        const int lead = min(kQuadStages, num_kb);  // k-blocks whose sub-tile-0 MMAs run ahead
        if (!wd.wait<true>(tempty_bar(0), acc_phase ^ 1u, kSiteMmaTmemEmpty)) break;
        tc_fence_after_sync();
        {
          int s = stage;
          uint32_t ph = phase;
          for (int j = 0; j < lead; ++j) {
            if (!wd.wait<true>(full_bar(s), ph, kSiteMmaFull)) {
              alive = false;
              break;
            }
            tc_fence_after_sync();
            issue(s, 0, d0, j == 0);
            if (++s == kQuadStages) {
              s = 0;
              ph ^= 1u;
            }
          }
        }
        if (!alive) break;
        if (!wd.wait<true>(tempty_bar(1), acc_phase ^ 1u, kSiteMmaTmemEmpty)) break;
        tc_fence_after_sync();
        for (int j = 0; j < lead; ++j) {
          issue(stage, 1, d1, j == 0);
          umma_commit_pair(empty_bar(stage));  // both CTAs may refill this stage once the MMAs retire
          if (++stage == kQuadStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        // the last k-blocks of the tile (as many as fit in the ring beside one stage for the producer): sub-tile 0
        // first, so that its accumulator reaches its epilogue group while sub-tile 1's last MMAs still run
        const int trail = max(0, min(kQuadStages - 1, num_kb - lead));
        for (int kb = lead; kb < num_kb - trail; ++kb) {
          if (!wd.wait<true>(full_bar(stage), phase, kSiteMmaFull)) {
            alive = false;
            break;
          }
          tc_fence_after_sync();
          issue(stage, 0, d0, false);
          issue(stage, 1, d1, false);
          umma_commit_pair(empty_bar(stage));
          if (++stage == kQuadStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!alive) break;
        {
          int s = stage;
          uint32_t ph = phase;
          for (int j = 0; j < trail; ++j) {
            if (!wd.wait<true>(full_bar(s), ph, kSiteMmaFull)) {
              alive = false;
              break;
            }
            tc_fence_after_sync();
            issue(s, 0, d0, false);
            if (++s == kQuadStages) {
              s = 0;
              ph ^= 1u;
            }
          }
        }
        if (!alive) break;
        umma_commit_pair(tfull_bar(0));  // accumulator 0 complete, in both CTAs
        for (int j = 0; j < trail; ++j) {
          issue(stage, 1, d1, false);
          umma_commit_pair(empty_bar(stage));
          if (++stage == kQuadStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        umma_commit_pair(tfull_bar(1));  // accumulator 1 complete
        acc_phase ^= 1u;
      }
      if (wd.aborted()) {
        umma_commit_2cta(drain_bar);
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
    // ------------- epilogue (both CTAs, own 256 rows): warp group g drains sub-tile g -------------
    const int group = (warp - 2) >> 2;
    const int quarter = warp & 3;  // the TMEM lanes a warp may read: 32 * (warp id mod 4)
    const uint32_t lane_field = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t warp_stage = bar_base + 512u + static_cast<uint32_t>(warp - 2) * (32u * 128u);
    const int group_tid = static_cast<int>(threadIdx.x) - 64 - group * 128;
    volatile uint32_t* ok_slot = epi_ok + 2 * group;
    uint32_t acc_phase = 0;
    uint32_t iter = 0;
    const uint32_t t_acc = tmem_base + lane_field + static_cast<uint32_t>(group * kUmmaN);
    for (int tile = cluster_id; tile < num_tiles; tile += num_clusters) {
      const TileCoord tc = tile_coord(tile, p);
      // One thread of the group waits for the accumulators and tells the other 127: the four warps share a
      // named barrier, so they must all take the same exit if a wait gives up.
      if (group_tid == 0) ok_slot[iter & 1u] = wd.wait(tfull_bar(group), acc_phase, kSiteEpilogueFull) ? 1u : 0u;
      if (group == 0) {
        asm volatile("bar.sync 1, 128;" ::: "memory");
      } else {
        asm volatile("bar.sync 2, 128;" ::: "memory");
      }
      const uint32_t ok = ok_slot[iter & 1u];
      ++iter;
      if (!ok) break;
      tc_fence_after_sync();
      const int col_base = tc.n_tile * p.tile_n;
      const int row0 = tc.m_tile * kQuadTileRows + static_cast<int>(rank) * 256 + group * 128 + quarter * 32;
      epilogue_rows<kMode, kOutF32>(p, TmemSource{t_acc}, warp_stage, lane, row0, col_base, p.tile_n);
      // this warp is done with its accumulator: tell the leader's MMA issuer (one arrival per warp)
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (rank == 0) {
          mbar_arrive(tempty_bar(group));
        } else {
          mbar_arrive_cluster(map_to_cta(tempty_bar(group), 0));
        }
      }
      acc_phase ^= 1u;
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
