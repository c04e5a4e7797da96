// Two-SM variant of the tiled tcgen05 GEMM: a cluster of two CTAs works on one 256-row tile with
// `tcgen05.mma.cta_group::2`.  Each CTA loads its own 128 rows of A and only HALF of the B tile
// (the MMA reads the other half from the partner's shared memory), so a k-block costs each SM
// 32 KiB of L2 -> SM traffic instead of 48 KiB, and the ring holds 6 stages instead of 4.  Every
// TMA load is an ordinary per-CTA load.
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
//
// Schedule.  Whole tiles are dealt round-robin to the clusters.  When the tile count is not a
// multiple of the cluster count the last wave would leave clusters idle; with a scratch buffer
// from the host the k-blocks of that last wave's tiles are instead cut into equal contiguous ranges,
// one per cluster (a range covers the end of one tile and the beginning of the next).  A tile shared
// by several ranges is finished by whichever of them arrives last at the tile's counter: every
// range publishes its raw fp32 accumulator, the last one sums the blocks in range order (so the
// result does not depend on timing) and runs the normal epilogue.  Nobody waits for anybody.
#pragma once

#include "gemm_common.cuh"
#include "pair_schedule.cuh"

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
                 const __grid_constant__ CUtensorMap map_b1, const __grid_constant__ CUtensorMap map_h0,
                 const __grid_constant__ CUtensorMap map_h1, const GemmParams p) {
  // map_b0 / map_b1: B operand(s) with 128-row boxes (whole tiles); map_h0 / map_h1: the same matrices with
  // 64-row boxes, used by the half-width units of a width-split last wave only
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + kPairStages * kPairStageBytes;
  // barrier block: full[6], empty[6], tmem_full[2], tmem_empty[2], drain, then bookkeeping words
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kPairStages + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * kPairStages + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * kPairStages + 2 + a); };
  const uint32_t drain_bar = bar_base + 8u * (2 * kPairStages + 4);
  uint8_t* generic_base = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t* tmem_ptr_slot = reinterpret_cast<volatile uint32_t*>(
      generic_base + kPairStages * kPairStageBytes + 8 * (2 * kPairStages + 5));
  volatile uint32_t* abort_flag = tmem_ptr_slot + 1;
  volatile uint32_t* epi_ok = tmem_ptr_slot + 2;     // two entries, alternating per unit
  volatile uint32_t* last_flag = tmem_ptr_slot + 4;  // "this CTA arrived last at the tile's counter"

  const int warp = threadIdx.x >> 5;
  const uint32_t lane = lane_id();
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const Watchdog wd{abort_flag, p.status, p.wait_limit_ns};

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
    *last_flag = 0;
    fence_mbar_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b0);
    prefetch_tensormap(&map_b1);
    if (p.tail_halves != 0) {
      prefetch_tensormap(&map_h0);
      prefetch_tensormap(&map_h1);
    }
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
  const int num_kb = (p.K + kBlockK - 1) / kBlockK;
  const int num_clusters = gridDim.x / 2;
  const int cluster_id = blockIdx.x / 2;
  const int mma_n = (kMode == kPlain) ? p.tile_n : 2 * p.tile_n;  // columns of the pair's accumulator
  const int b_half_rows = mma_n / 2;  // B rows a CTA holds for a whole tile (128); a half-width unit takes half

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t issued_mask = 0, last_parity_mask = 0;
      bool alive = true;
      PairSchedule sched(p.num_m_tiles * p.num_n_tiles, p.tail_first, p.tail_len, p.tail_halves, cluster_id, num_clusters, num_kb);
      PairUnit un;
      bool withhold = p.withhold_one_copy != 0 && blockIdx.x == 0;  // one-shot, leader of the first pair
      const uint64_t pol_a = l2_policy_of(p.hint_a), pol_b = l2_policy_of(p.hint_b);
      int whole_tiles = 0;
      while (alive && sched.next(&un)) {
        const TileCoord tc = tile_coord(un.tile, p);
        const bool backwards = p.k_alternate != 0 && un.tail_tile < 0 && (whole_tiles++ & 1) != 0;
        const int m0 = tc.m_tile * 256 + static_cast<int>(rank) * 128;
        const int n0 = tc.n_tile * p.tile_n;
        const CUtensorMap* bmap = &map_b0;
        // B rows of this CTA: `rows` of them from b_row on (a half-width unit takes half as many, from
        // the half's first row, through the maps with 64-row boxes)
        const int rows = un.half < 0 ? b_half_rows : b_half_rows / 2;
        if (un.half >= 0) bmap = &map_h0;
        const int hsel = un.half < 0 ? 0 : un.half;
        int b_row;
        if (kMode == kPlain) {
          b_row = n0 + hsel * b_half_rows + static_cast<int>(rank) * rows;
        } else if (kMode == kGatedSplit) {
          b_row = n0 + hsel * rows;  // leader: W_gate rows, partner: W_up rows
          if (rank == 1) bmap = un.half < 0 ? &map_b1 : &map_h1;
        } else {
          b_row = 2 * n0 + hsel * b_half_rows + static_cast<int>(rank) * rows;
        }
        const uint32_t stage_tx_bytes = kATileBytes + static_cast<uint32_t>(rows) * (kBlockK * 2);
        for (int step = un.kb0; step < un.kb1; ++step) {
          const int kb = backwards ? un.kb1 - 1 - (step - un.kb0) : step;  // the sum does not care about the order
          if (!wd.wait(empty_bar(stage), phase ^ 1u, kSiteProducerEmpty)) {
            alive = false;
            break;
          }
          const uint32_t a_dst = smem_base + stage * kPairStageBytes;
          // one barrier per stage, in the leader: it expects the bytes of both CTAs' halves
          if (rank == 0) mbar_arrive_expect_tx(full_bar(stage), 2u * stage_tx_bytes);
          const uint32_t leader_full = map_to_cta(full_bar(stage), 0);
          // no residency class: the plain load (the hardware's default policy), else the load with a hint
          if (p.hint_a == kL2Default) {
            tma_load_2d_pair(a_dst, &map_a, leader_full, kb * kBlockK, m0);
          } else {
            tma_load_2d_pair_hint(a_dst, &map_a, leader_full, kb * kBlockK, m0, pol_a);
          }
          if (!withhold) {
            if (p.hint_b == kL2Default) {
              tma_load_2d_pair(a_dst + kATileBytes, bmap, leader_full, kb * kBlockK, b_row);
            } else {
              tma_load_2d_pair_hint(a_dst + kATileBytes, bmap, leader_full, kb * kBlockK, b_row, pol_b);
            }
          }
          withhold = false;
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
      const uint32_t idesc_full = umma_idesc_bf16_f32(256, mma_n);
      const uint32_t idesc_half = umma_idesc_bf16_f32(256, mma_n / 2);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool alive = true;
      PairSchedule sched(p.num_m_tiles * p.num_n_tiles, p.tail_first, p.tail_len, p.tail_halves, cluster_id, num_clusters, num_kb);
      PairUnit un;
      while (alive && sched.next(&un)) {
        if (!wd.wait<true>(tempty_bar(acc), acc_phase ^ 1u, kSiteMmaTmemEmpty)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kUmmaN);
        const uint32_t idesc = un.half < 0 ? idesc_full : idesc_half;
        for (int kb = un.kb0; kb < un.kb1; ++kb) {
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
            umma_bf16_ss_2cta(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc, (kb > un.kb0 || k > 0) ? 1u : 0u);
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
          if (global_timer_ns() - t0 > kDrainLimitNs) {
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
    const int epi_tid = static_cast<int>(threadIdx.x) - 64;
    const int row_in_half = quarter * 32 + static_cast<int>(lane);
    int acc = 0;
    uint32_t acc_phase = 0;
    uint32_t iter = 0;
    PairSchedule sched(p.num_m_tiles * p.num_n_tiles, p.tail_first, p.tail_len, p.tail_halves, cluster_id, num_clusters, num_kb);
    PairUnit un;
    while (sched.next(&un)) {
      const TileCoord tc = tile_coord(un.tile, p);
      // One thread waits for the accumulator and tells the other 127: the four warps share named
      // barriers below, so they must all take the same exit if a wait gives up.
      if (epi_tid == 0) epi_ok[iter & 1u] = wd.wait(tfull_bar(acc), acc_phase, kSiteEpilogueFull) ? 1u : 0u;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const uint32_t ok = epi_ok[iter & 1u];
      ++iter;
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t t_acc = tmem_base + lane_field + static_cast<uint32_t>(acc * kUmmaN);
      const int row0 = tc.m_tile * 256 + static_cast<int>(rank) * 128 + quarter * 32;
      const int width = un.half < 0 ? p.tile_n : p.tile_n / 2;
      const int col_base = tc.n_tile * p.tile_n + (un.half > 0 ? width : 0);
      auto release_accumulator = [&]() {
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
      };

      // how many ranges share this tile, and which of them is this cluster's
      int nseg = 1, seg = 0;
      if (un.tail_tile >= 0) tail_tile_segments(un.tail_tile, num_kb, p.tail_len, cluster_id, &nseg, &seg);
      if (nseg == 1) {
        epilogue_rows<kMode, kOutF32>(p, TmemSource{t_acc}, warp_stage, lane, row0, col_base, width);
        release_accumulator();
        continue;
      }
      // ---- shared tile: publish the raw accumulator, the last range to arrive finishes the tile ----
      // block of (cluster c, tail tile t) = (c + t) * 2 + rank: consecutive ranges of one tile are
      // consecutive clusters, so a tile's blocks are 2 * kTailBlockFloats apart
      float* my_block = p.tail_partials +
                        (static_cast<long long>(tail_block_index(cluster_id, un.tail_tile)) * 2 + rank) * kTailBlockFloats;
      store_partial_row(t_acc, my_block, row_in_half, mma_n);
      release_accumulator();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (epi_tid == 0) {
        __threadfence();  // the 128 threads' blocks (ordered before this by the barrier) become visible
        unsigned int* counter = p.tail_counters + un.tail_tile * 2 + rank;
        const unsigned int old = atomicAdd(counter, 1u);
        const bool last = old == static_cast<unsigned int>(nseg - 1);
        if (last) *counter = 0u;  // every range has arrived: leave the counter clean for the next launch
        *last_flag = last ? 1u : 0u;
        __threadfence();
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const bool reduce_here = (*last_flag != 0);
      asm volatile("bar.sync 1, 128;" ::: "memory");  // everyone has read the flag before it is reused
      if (reduce_here) {
        PartialSource src;
        src.first_block = my_block - static_cast<long long>(seg) * 2 * kTailBlockFloats;
        src.seg_stride = 2ll * kTailBlockFloats;
        src.nseg = nseg;
        src.row = row_in_half;
        epilogue_rows<kMode, kOutF32>(p, src, warp_stage, lane, row0, col_base, p.tile_n);
      }
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
