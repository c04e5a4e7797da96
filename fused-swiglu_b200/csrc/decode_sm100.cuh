// Small-batch (M <= 64 tokens) path of the SwiGLU MLP forward.  With so few
// tokens the work is streaming 3*d*F bf16 weights through the chip once, so
// the kernel is organised around HBM bandwidth, not around the tensor cores.
// ONE persistent launch does both projections:
//
//   phase 1   h[M,F]   = silu(x Wg^T) * (x Wu^T)
//   (grid-wide hand-over: every CTA has finished writing its part of h)
//   phase 2   out[M,d] = h Wd^T
//
//   * swap-AB: the WEIGHT tile (up to 128 rows x 64 k) is the MMA's M operand and
//     the tokens (padded to N = 16/32/64) are its N operand, so a TMEM
//     accumulator holds weight rows x tokens and no tensor-core work is spent on
//     padding M up to 128;
//   * phase 1 is a ROW split without split-K: each SM owns ceil(F / SMs)
//     consecutive rows of W_gate and W_up (97 of 14336 ...) for the whole
//     reduction length d.  A TMA box may have any number of rows, so the split
//     is even to within one row; the MMA still runs at M = 128 and accumulator
//     lanes past the tile are never read.  No partial sums: when the last byte
//     has arrived the tail is one TMEM read, SiLU(g)*u and the h stores, so the
//     hand-over to phase 2 follows the weight stream by a few microseconds;
//   * phase 2 is STREAM-K: W_down has few rows and a long reduction, so its
//     (128-row block, k-block) units are cut into equal contiguous ranges, one
//     per SM (full 128-row MMAs, and each SM reads only its own k-range of h).
//     Row-blocks whose K range spans several CTAs are combined through fp32
//     partial tiles in a workspace: every range but the first publishes its tile
//     and raises a flag; the CTA that owns the FIRST k-range of a row-block (the
//     last thing it does, so the others are normally done by then) adds the tiles
//     to its own accumulator in FIXED segment order, so results do not depend on
//     timing.  By then the CTA's shared-memory rings are idle, so the tiles are pulled
//     into shared memory by bulk copies (one round trip for all of them instead of one
//     per 16 token columns);
//   * two TMA rings per SM: 11 x 16 KiB weight slots (evict-first L2 hint) and a
//     32 KiB ring of token tiles (x in phase 1, h in phase 2).  The weight
//     producer never waits for the hand-over: while h is being completed it
//     already fills its ring with W_down tiles;
//   * cross-CTA signalling uses flags that carry a per-launch tag instead of counters:
//     nothing has to be zeroed before a launch (no memset in front of the kernel), and a
//     stale or uninitialised word never looks like a signal.  The waits on them (the
//     token-tile producer's on the phase-1 flags of all CTAs, the reducer's on its
//     row-block's segment flags) are bounded like every other wait, and the kernel is
//     launched cooperatively so that all CTAs are resident together.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "ptx_sm100.cuh"

namespace fsw {

constexpr int kDecodeMaxTokens = 64;
constexpr int kDecThreads = 224;              // 7 warps: W producer, MMA, 4 epilogue, token-tile producer
constexpr int kDecWSlotBytes = 16384;
constexpr int kDecWSlots = 11;
constexpr int kDecXRingBytes = 32768;
constexpr int kDecMaxXSlots = 16;
constexpr int kDecSmemBytes = kDecWSlots * kDecWSlotBytes + kDecXRingBytes + 1024 + 1024;

constexpr int kDecMaxSegments = 8;  // partial tiles kept per row-block of phase 2
constexpr int kDecMaxGrid = 255;    // CTAs the flag block has room for (plus one spare flag)

struct DecodeParams {
  // phase 1 (row split): h[M, F] = silu(x Wg^T) * (x Wu^T)
  void* h;            // bf16 [M, F], row pitch F
  int F;              // rows of W_gate / W_up
  int k_blocks1;      // ceil(d / 64)
  int tile_rows;      // weight rows per tile (1..128) = rows of one TMA box
  int tiles_per_cta;  // consecutive tiles each CTA owns
  // phase 2 (stream-K): out[M, d] = h Wd^T
  void* out;          // bf16 / fp32 [M, d]
  long long ld_out;
  int d;              // rows of W_down
  int row_blocks2;    // ceil(d / 128)
  int k_blocks2;      // ceil(F / 64)
  int out_f32;
  float* partials;        // [row_blocks2][kDecMaxSegments][128][n_pad] fp32
  unsigned int* seg_flags;   // [row_blocks2][kDecMaxSegments]: == tag once that segment's partial tile is published
  unsigned int* phase1_flags;// [grid + 1]: == tag once that CTA has written its part of h
  unsigned int tag;          // non-zero, different for every launch
  int M;                  // tokens (<= 64)
  int n_pad;              // tokens padded to 16 / 32 / 64 (the MMA N extent)
  int prefetch_units;     // how many W_down tiles ahead of the shared-memory ring are pulled into L2
  const float* row_scale; // optional per-token factor on gate and up before SiLU (fused RMSNorm statistic)
  const void* residual;   // optional bf16 [M, d] added to the output in fp32
  long long ld_res;
  uint32_t* status;
  unsigned long long wait_limit_ns;  // limit of every device-side wait in this launch
  unsigned int handover_target;      // CTAs that must have finished phase 1 (= the grid size; tests of the
                                     // time-out path pass one more, which nothing ever reaches)
  int w_slots;                       // weight-tile slots in use (<= kDecWSlots); the token-tile ring takes the rest
  int k_rotate;                      // phase 1: CTA c starts its reduction at k-block (c * k_rotate) mod k_blocks1
                                     // and wraps around, so that the CTAs do not all read the same columns of
                                     // the weight matrices at the same moment (0 = everybody starts at 0)
  int rows_per_cta;                  // phase-1 hidden units per CTA (tile_rows * tiles_per_cta)
  int reduce_via_smem;               // phase 2: the row-block owner copies the other ranges' partial tiles into
                                     // its (by then idle) shared-memory rings with bulk copies and sums from there
  unsigned long long* trace;         // optional: kDecTraceStamps %globaltimer stamps per CTA (profiling aid)
};

// Time stamps a CTA leaves in DecodeParams::trace (one 64-bit slot each, 0 = not reached).
enum DecodeStamp : int {
  kStampSetupDone = 0, kStampP1FirstTile, kStampP1MmasIssued, kStampP1HandoverSignalled, kStampP2FirstTile,
  kStampP2MmasIssued, kStampP2EpilogueDone, kStampHandoverObserved, kDecTraceStamps
};

// First unit of CTA c when `units` units are cut into `ctas` contiguous ranges.
__host__ __device__ inline long long dec_range_start(long long c, long long units, long long ctas) {
  return c * units / ctas;
}
// The CTA whose range contains unit u.
__host__ __device__ inline int dec_owner(long long u, long long units, long long ctas) {
  long long c = u * ctas / units;
  while (c + 1 < ctas && dec_range_start(c + 1, units, ctas) <= u) ++c;
  while (c > 0 && dec_range_start(c, units, ctas) > u) --c;
  return static_cast<int>(c);
}

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(unsigned int* p, unsigned int v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ unsigned int ld_relaxed_gpu(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Global -> shared bulk copy (no tensor map; both addresses 16-byte aligned, size a multiple of 16),
// completion counted in bytes on an mbarrier of this CTA.
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// Position (in 16-byte units) of the q-th group of four token columns inside a weight row's run of a partial
// tile.  Thread = row; rows are n_pad * 4 bytes apart, so without a permutation the eight lanes of a
// shared-memory access phase would all hit the same banks.  XOR with the row number (taken per 128 bytes)
// spreads them; writer and reader use the same function.
__device__ __forceinline__ int partial_pos(int q, int row, int groups_per_row) {
  const int s = groups_per_row >= 8 ? row : (row >> 1);
  return q ^ (s & (groups_per_row - 1));
}

__global__ void __launch_bounds__(kDecThreads, 1)
decode_fused_kernel(const __grid_constant__ CUtensorMap map_gate, const __grid_constant__ CUtensorMap map_up,
                    const __grid_constant__ CUtensorMap map_down, const __grid_constant__ CUtensorMap map_x,
                    const __grid_constant__ CUtensorMap map_h, const DecodeParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  // ring area: w_slots weight slots of 16 KiB, then the token-tile ring in what is left of the
  // (kDecWSlots * 16 KiB + 32 KiB) area; the barrier block follows at a fixed offset
  const int w_slots = p.w_slots;
  const uint32_t w_ring = smem_base;
  const uint32_t x_ring = smem_base + static_cast<uint32_t>(w_slots) * kDecWSlotBytes;
  const uint32_t bar_base = smem_base + kDecWSlots * kDecWSlotBytes + kDecXRingBytes;
  auto stamp = [&](int which) {
    if (p.trace != nullptr) p.trace[static_cast<size_t>(blockIdx.x) * kDecTraceStamps + which] = global_timer_ns();
  };
  auto w_full = [&](int s) { return bar_base + 8u * s; };
  auto w_empty = [&](int s) { return bar_base + 8u * (kDecWSlots + s); };
  auto x_full = [&](int s) { return bar_base + 8u * (2 * kDecWSlots + s); };
  auto x_empty = [&](int s) { return bar_base + 8u * (2 * kDecWSlots + kDecMaxXSlots + s); };
  constexpr int kBarsBeforeTmem = 2 * kDecWSlots + 2 * kDecMaxXSlots;
  auto tfull_bar = [&](int a) { return bar_base + 8u * (kBarsBeforeTmem + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (kBarsBeforeTmem + 2 + a); };
  const uint32_t drain_bar = bar_base + 8u * (kBarsBeforeTmem + 4);
  const uint32_t reduce_bar = bar_base + 8u * (kBarsBeforeTmem + 7);  // after the four words behind the TMEM pointer
  uint8_t* generic_base = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t* tmem_ptr_slot = reinterpret_cast<volatile uint32_t*>(
      generic_base + kDecWSlots * kDecWSlotBytes + kDecXRingBytes + 8 * (kBarsBeforeTmem + 5));
  volatile uint32_t* abort_flag = tmem_ptr_slot + 1;
  volatile uint32_t* epi_ok = tmem_ptr_slot + 2;  // two entries, alternating per tile / segment

  const int warp = threadIdx.x >> 5;
  const uint32_t lane = lane_id();
  const Watchdog wd{abort_flag, p.status, p.wait_limit_ns};

  constexpr int kAccStride = 128;  // TMEM columns per accumulator stage (2 stages)
  const uint32_t x_slot_bytes = static_cast<uint32_t>(p.n_pad) * 128u;
  const int x_slots = min(kDecMaxXSlots, (kDecXRingBytes + (kDecWSlots - w_slots) * kDecWSlotBytes) /
                                              static_cast<int>(x_slot_bytes));

  if (threadIdx.x == 0) {
    for (int s = 0; s < kDecWSlots; ++s) {
      mbar_init(w_full(s), 1);
      mbar_init(w_empty(s), 1);
    }
    for (int s = 0; s < kDecMaxXSlots; ++s) {
      mbar_init(x_full(s), 1);
      mbar_init(x_empty(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 128);
    }
    mbar_init(drain_bar, 1);
    mbar_init(reduce_bar, 1);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tensormap(&map_gate);
    prefetch_tensormap(&map_up);
    prefetch_tensormap(&map_down);
    prefetch_tensormap(&map_x);
    prefetch_tensormap(&map_h);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_ptr_slot)), 256);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_slot;
  if (threadIdx.x == 0) stamp(kStampSetupDone);

  // phase 1: first weight row of this CTA's i-th tile (>= F: the tile does not exist)
  auto tile_row0 = [&](int i) {
    return (static_cast<long long>(blockIdx.x) * p.tiles_per_cta + i) * p.tile_rows;
  };
  const int kb_first = p.k_rotate > 0 ? static_cast<int>((static_cast<long long>(blockIdx.x) * p.k_rotate) % p.k_blocks1) : 0;
  auto kb_of = [&](int step) {  // k-block handled at step `step` of a phase-1 tile
    const int kb = kb_first + step;
    return kb >= p.k_blocks1 ? kb - p.k_blocks1 : kb;
  };
  // phase 2: this CTA's contiguous range of (row-block, k-block) units
  const long long units2 = static_cast<long long>(p.row_blocks2) * p.k_blocks2;
  const long long u_begin = dec_range_start(blockIdx.x, units2, gridDim.x);
  const long long u_end = dec_range_start(blockIdx.x + 1, units2, gridDim.x);

  if (warp == 0) {
    // ------------------- weight-tile producer: never waits for the hand-over -------------------
    if (lane == 0) {
      const uint64_t stream_once = l2_policy_evict_first();
      int slot = 0;
      uint32_t phase = 0;
      uint32_t issued_mask = 0, last_parity_mask = 0;
      bool alive = true;
      auto fill = [&](const CUtensorMap* map, int x, int y, uint32_t bytes) -> bool {
        if (!wd.wait(w_empty(slot), phase ^ 1u, kSiteProducerEmpty)) return false;
        mbar_arrive_expect_tx(w_full(slot), bytes);
        tma_load_2d_hint(w_ring + slot * kDecWSlotBytes, map, w_full(slot), x, y, stream_once);
        issued_mask |= 1u << slot;
        last_parity_mask = (last_parity_mask & ~(1u << slot)) | (phase << slot);
        if (++slot == w_slots) {
          slot = 0;
          phase ^= 1u;
        }
        return true;
      };
      const uint32_t tile_bytes = static_cast<uint32_t>(p.tile_rows) * 128u;
      for (int i = 0; i < p.tiles_per_cta && alive; ++i) {
        const long long row0 = tile_row0(i);
        if (row0 >= p.F) break;
        for (int step = 0; step < p.k_blocks1 && alive; ++step) {
          const int kb = kb_of(step);
          alive = fill(&map_gate, kb * 64, static_cast<int>(row0), tile_bytes) &&
                  fill(&map_up, kb * 64, static_cast<int>(row0), tile_bytes);
        }
      }
      // Phase 2.  The ring cannot take W_down tiles faster than phase 1 frees its slots, and it
      // stalls completely while the hand-over is in flight; HBM would idle meanwhile.  So W_down tiles
      // are pulled into L2 a bounded distance ahead of the ring (fire and forget), and the ring's own
      // loads then hit L2.  The window is bounded because everything prefetched has to stay in L2
      // until it is used.
      long long pf = u_begin + w_slots;
      for (long long u = u_begin; u < u_end && alive; ++u) {
        for (; pf < u_end && pf < u + w_slots + p.prefetch_units; ++pf) {
          const int prb = static_cast<int>(pf / p.k_blocks2);
          const int pkb = static_cast<int>(pf - static_cast<long long>(prb) * p.k_blocks2);
          tma_prefetch_l2_2d(&map_down, pkb * 64, prb * 128);
        }
        const int rb = static_cast<int>(u / p.k_blocks2);
        const int kb = static_cast<int>(u - static_cast<long long>(rb) * p.k_blocks2);
        alive = fill(&map_down, kb * 64, rb * 128, 128u * 128u);
      }
      if (wd.aborted()) {
        for (int s = 0; s < w_slots; ++s) {
          if (issued_mask & (1u << s)) {
            const uint32_t par = (last_parity_mask >> s) & 1u;
            const unsigned long long t0 = global_timer_ns();
            while (!mbar_try_wait(w_full(s), par)) {
              if (global_timer_ns() - t0 > kDrainLimitNs) {
                wd.give_up(kSiteDrainTma);
                break;
              }
            }
          }
        }
      }
    }
  } else if (warp == 6) {
    // ------------------- token-tile producer: x in phase 1, h (after the hand-over) in phase 2 ----
    // Lane 0 issues the copies; the hand-over wait in the middle is done by the whole warp (every lane
    // polls a few of the per-CTA flags).
    const uint64_t keep = l2_policy_evict_last();
    int slot = 0;
    uint32_t phase = 0;
    uint32_t issued_mask = 0, last_parity_mask = 0;
    bool alive = true;
    auto push = [&](const CUtensorMap* map, int kb) -> bool {
      if (!wd.wait(x_empty(slot), phase ^ 1u, kSiteProducerEmpty)) return false;
      mbar_arrive_expect_tx(x_full(slot), x_slot_bytes);
      tma_load_2d_hint(x_ring + slot * x_slot_bytes, map, x_full(slot), kb * 64, 0, keep);
      issued_mask |= 1u << slot;
      last_parity_mask = (last_parity_mask & ~(1u << slot)) | (phase << slot);
      if (++slot == x_slots) {
        slot = 0;
        phase ^= 1u;
      }
      return true;
    };
    if (lane == 0) {
      for (int i = 0; i < p.tiles_per_cta && alive; ++i) {
        if (tile_row0(i) >= p.F) break;
        for (int step = 0; step < p.k_blocks1 && alive; ++step) alive = push(&map_x, kb_of(step));
      }
    }
    alive = __shfl_sync(0xffffffffu, alive ? 1 : 0, 0) != 0;
    // Phase 2 reads h.  Hidden unit j was written by CTA j / rows_per_cta, which raises its phase-1 flag for
    // this launch when its part of h is complete; a k-block of 64 hidden units therefore depends on one or
    // two CTAs only.  The warp keeps a bit map of the flags it has seen raised (one poll pass reads every
    // CTA's flag, a few loads per lane, all in flight together) and lane 0 loads h tiles as far as the map
    // allows; a new pass is made only when the next k-block's producers are not in the map yet.  So a CTA
    // starts phase 2 as soon as ITS producers are done, not when the whole grid is.
    constexpr int kFlagWords = (kDecMaxGrid + 32) / 32;
    uint32_t ready[kFlagWords];
#pragma unroll
    for (int i = 0; i < kFlagWords; ++i) ready[i] = 0u;
    auto is_ready = [&](unsigned int c) {
      uint32_t word = 0u;
#pragma unroll
      for (int i = 0; i < kFlagWords; ++i) word = (static_cast<int>(c >> 5) == i) ? ready[i] : word;
      return ((word >> (c & 31u)) & 1u) != 0u;
    };
    const unsigned int n_flags = p.handover_target;  // the grid size; one more in the time-out test
    const bool wait_spare = n_flags > gridDim.x;      // time-out test: a flag that nothing raises
    unsigned long long t0 = 0;
    bool stamped = false;
    // Running state, advanced without divisions (this loop has to keep pace with the weight stream):
    // kb = k-block of unit u; c_hi = last CTA whose rows reach into that k-block; boundary = first hidden
    // unit of CTA c_hi + 1; next_unseen = first CTA at or after the k-block's first producer that is not
    // known to be done (producers of consecutive k-blocks only move upwards within a row-block).
    int kb = static_cast<int>(u_begin % p.k_blocks2);
    unsigned int c_hi = static_cast<unsigned int>(min(p.F - 1, kb * 64 + 63) / p.rows_per_cta);
    long long boundary = static_cast<long long>(c_hi + 1) * p.rows_per_cta;
    unsigned int next_unseen = static_cast<unsigned int>((kb * 64) / p.rows_per_cta);
    long long u = u_begin;
    while (u < u_end && alive) {
      while (next_unseen <= c_hi && is_ready(next_unseen)) ++next_unseen;
      if (next_unseen <= c_hi || (wait_spare && !is_ready(n_flags - 1))) {
        // one poll pass over all flags (warp-uniform control flow: `ready` is the same in every lane)
        if (t0 == 0) t0 = global_timer_ns();
#pragma unroll
        for (int i = 0; i < kFlagWords; ++i) {
          const unsigned int c = static_cast<unsigned int>(i) * 32u + lane;
          bool up = ((ready[i] >> lane) & 1u) != 0u;
          if (!up && c < n_flags) up = ld_acquire_gpu(p.phase1_flags + c) == p.tag;
          ready[i] = __ballot_sync(0xffffffffu, up);
        }
        // h was written with ordinary stores by other SMs; order them before this SM's TMA reads
        asm volatile("fence.proxy.async;" ::: "memory");
        const bool late = global_timer_ns() - t0 > p.wait_limit_ns;
        if (__any_sync(0xffffffffu, late || wd.aborted())) {
          if (lane == 0 && late) wd.give_up(kSiteDecode);
          alive = false;
        }
        continue;
      }
      if (lane == 0) {
        if (!stamped) stamp(kStampHandoverObserved);
        alive = push(&map_h, kb);
      }
      stamped = true;
      alive = __shfl_sync(0xffffffffu, alive ? 1 : 0, 0) != 0;
      ++u;
      if (++kb == p.k_blocks2) {  // the range continues at the start of the next row-block
        kb = 0;
        c_hi = static_cast<unsigned int>(min(p.F - 1, 63) / p.rows_per_cta);
        boundary = static_cast<long long>(c_hi + 1) * p.rows_per_cta;
        next_unseen = 0;
      } else {
        const long long last_hidden = min(static_cast<long long>(p.F) - 1, static_cast<long long>(kb) * 64 + 63);
        while (last_hidden >= boundary) {
          ++c_hi;
          boundary += p.rows_per_cta;
        }
      }
    }
    if (lane == 0) {
      if (wd.aborted()) {
        for (int sl = 0; sl < x_slots; ++sl) {
          if (issued_mask & (1u << sl)) {
            const uint32_t par = (last_parity_mask >> sl) & 1u;
            const unsigned long long t0 = global_timer_ns();
            while (!mbar_try_wait(x_full(sl), par)) {
              if (global_timer_ns() - t0 > kDrainLimitNs) {
                wd.give_up(kSiteDrainTma);
                break;
              }
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------ MMA issuer ------------------------------------------
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16_f32(128, p.n_pad);
      int ws = 0, xs = 0;
      uint32_t wphase = 0, xphase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool alive = true;
      auto next_w = [&]() {
        if (++ws == w_slots) {
          ws = 0;
          wphase ^= 1u;
        }
      };
      auto next_x = [&]() {
        if (++xs == x_slots) {
          xs = 0;
          xphase ^= 1u;
        }
      };
      // ---- phase 1: one accumulator pair (gate | up) per tile, whole K ----
      for (int i = 0; i < p.tiles_per_cta && alive; ++i) {
        if (tile_row0(i) >= p.F) break;
        if (!wd.wait(tempty_bar(acc), acc_phase ^ 1u, kSiteMmaTmemEmpty)) {
          alive = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kAccStride);
        for (int kb = 0; kb < p.k_blocks1; ++kb) {
          const int w0 = ws;
          if (!wd.wait(w_full(w0), wphase, kSiteMmaFull)) {
            alive = false;
            break;
          }
          next_w();
          const int w1 = ws;
          if (!wd.wait(w_full(w1), wphase, kSiteMmaFull) || !wd.wait(x_full(xs), xphase, kSiteMmaFull)) {
            alive = false;
            break;
          }
          next_w();
          tc_fence_after_sync();
          if (i == 0 && kb == 0) stamp(kStampP1FirstTile);
          const uint64_t g_desc = umma_desc_k_sw128(w_ring + w0 * kDecWSlotBytes);
          const uint64_t u_desc = umma_desc_k_sw128(w_ring + w1 * kDecWSlotBytes);
          const uint64_t x_desc = umma_desc_k_sw128(x_ring + xs * x_slot_bytes);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint32_t accum = (kb > 0 || k > 0) ? 1u : 0u;
            umma_bf16_ss(d_tmem, g_desc + 2u * k, x_desc + 2u * k, idesc, accum);
            umma_bf16_ss(d_tmem + p.n_pad, u_desc + 2u * k, x_desc + 2u * k, idesc, accum);
          }
          umma_commit(w_empty(w0));
          umma_commit(w_empty(w1));
          umma_commit(x_empty(xs));
          next_x();
        }
        if (!alive) break;
        umma_commit(tfull_bar(acc));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
      if (alive) stamp(kStampP1MmasIssued);
      // ---- phase 2: one accumulator per (row-block, k-range) segment ----
      long long u = u_begin;
      while (u < u_end && alive) {
        const int rb = static_cast<int>(u / p.k_blocks2);
        const long long seg_end = min(u_end, static_cast<long long>(rb + 1) * p.k_blocks2);
        if (!wd.wait(tempty_bar(acc), acc_phase ^ 1u, kSiteMmaTmemEmpty)) {
          alive = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kAccStride);
        bool first = true;
        for (; u < seg_end; ++u) {
          if (!wd.wait(w_full(ws), wphase, kSiteMmaFull) || !wd.wait(x_full(xs), xphase, kSiteMmaFull)) {
            alive = false;
            break;
          }
          tc_fence_after_sync();
          if (u == u_begin) stamp(kStampP2FirstTile);
          const uint64_t w_desc = umma_desc_k_sw128(w_ring + ws * kDecWSlotBytes);
          const uint64_t x_desc = umma_desc_k_sw128(x_ring + xs * x_slot_bytes);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            umma_bf16_ss(d_tmem, w_desc + 2u * k, x_desc + 2u * k, idesc, (first && k == 0) ? 0u : 1u);
          }
          first = false;
          umma_commit(w_empty(ws));
          umma_commit(x_empty(xs));
          next_w();
          next_x();
        }
        if (!alive) break;
        umma_commit(tfull_bar(acc));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
      if (alive) stamp(kStampP2MmasIssued);
      if (wd.aborted()) {
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
    // -------------------------------------- epilogue -------------------------------------------
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + static_cast<int>(lane);  // weight row within the tile / row-block
    const uint32_t lane_field = static_cast<uint32_t>(quarter * 32) << 16;
    const int epi_tid = static_cast<int>(threadIdx.x) - 64;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool alive = true;
    uint32_t iter = 0;
    uint32_t reduce_phase = 0;
    const int groups_per_row = p.n_pad >> 2;               // 16-byte groups of a weight row's run in a partial tile
    const int tile_bytes = 128 * p.n_pad * 4;              // one partial tile
    constexpr int ring_bytes = kDecWSlots * kDecWSlotBytes + kDecXRingBytes;
    // One thread waits for the accumulator and tells the other 127: the four epilogue warps share
    // named barriers below, so they must all take the same exit if a wait gives up.
    auto accumulator_ready = [&]() -> bool {
      if (epi_tid == 0) epi_ok[iter & 1u] = wd.wait(tfull_bar(acc), acc_phase, kSiteEpilogueFull) ? 1u : 0u;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const uint32_t ok = epi_ok[iter & 1u];
      ++iter;
      return ok != 0;
    };
    auto release_accumulator = [&]() {
      tc_fence_before_sync();
      mbar_arrive(tempty_bar(acc));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    };

    // ---- phase 1: h = silu(g) * u straight from the accumulators ----
    for (int i = 0; i < p.tiles_per_cta; ++i) {
      const long long row0 = tile_row0(i);
      if (row0 >= p.F) break;
      if (!accumulator_ready()) {
        alive = false;
        break;
      }
      tc_fence_after_sync();
      const uint32_t t_acc = tmem_base + lane_field + static_cast<uint32_t>(acc * kAccStride);
      const long long j = row0 + row_in_tile;  // hidden unit
      const bool row_ok = row_in_tile < p.tile_rows && j < p.F;
      __nv_bfloat16* h = reinterpret_cast<__nv_bfloat16*>(p.h);
#pragma unroll 1
      for (int c0 = 0; c0 < p.n_pad; c0 += 16) {
        uint32_t g[16], uu[16];
        tmem_ld_32x32b_x16(t_acc + c0, g);
        tmem_ld_32x32b_x16(t_acc + p.n_pad + c0, uu);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int t = 0; t < 16; ++t) {
            if (c0 + t < p.M) {
              const float rs = p.row_scale != nullptr ? __ldg(p.row_scale + c0 + t) : 1.0f;
              h[static_cast<long long>(c0 + t) * p.F + j] =
                  __float2bfloat16_rn(silu_mul(rs * __uint_as_float(g[t]), rs * __uint_as_float(uu[t])));
            }
          }
        }
      }
      release_accumulator();
    }
    // hand-over: everything this CTA contributes to h is written; count it in.  The barrier orders
    // the 128 threads' stores before thread 0, whose release makes them visible device-wide (one
    // fence on the critical path instead of one per thread followed by another).
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (epi_tid == 0 && alive) {
      st_release_gpu(p.phase1_flags + blockIdx.x, p.tag);
      stamp(kStampP1HandoverSignalled);
    }

    // ---- phase 2: segments of row-blocks, combined through fp32 partial tiles ----
    long long u = u_begin;
    while (u < u_end && alive) {
      const int rb = static_cast<int>(u / p.k_blocks2);
      const long long rb_first = static_cast<long long>(rb) * p.k_blocks2;
      const long long seg_end = min(u_end, rb_first + p.k_blocks2);
      // which contiguous ranges (CTAs) share this row-block, and which of them am I
      const int first_cta = dec_owner(rb_first, units2, gridDim.x);
      const int last_cta = dec_owner(rb_first + p.k_blocks2 - 1, units2, gridDim.x);
      const int nseg = last_cta - first_cta + 1;
      const int seg = static_cast<int>(blockIdx.x) - first_cta;
      u = seg_end;
      if (!accumulator_ready()) {
        alive = false;
        break;
      }
      tc_fence_after_sync();
      const uint32_t t_acc = tmem_base + lane_field + static_cast<uint32_t>(acc * kAccStride);
      const long long out_row = static_cast<long long>(rb) * 128 + row_in_tile;

      if (nseg > 1 && seg != 0) {
        // publish this segment's partial sums: [row][n_pad] fp32, one contiguous run per thread
        float* my_tile =
            p.partials + ((static_cast<size_t>(rb) * kDecMaxSegments + seg) * 128 + row_in_tile) * p.n_pad;
#pragma unroll 1
        for (int c0 = 0; c0 < p.n_pad; c0 += 16) {
          uint32_t r[16];
          tmem_ld_32x32b_x16(t_acc + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            __stcg(reinterpret_cast<float4*>(my_tile) + partial_pos((c0 >> 2) + i, row_in_tile, groups_per_row),
                   make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]),
                               __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3])));
          }
        }
        release_accumulator();  // accumulator drained: the MMA warp may reuse it
        asm volatile("bar.sync 1, 128;" ::: "memory");
        // the barrier orders the 128 threads' stores before thread 0, whose release makes them visible
        if (epi_tid == 0) st_release_gpu(p.seg_flags + rb * kDecMaxSegments + seg, p.tag);
        continue;
      }
      int n_smem = 0;  // how many of the other ranges' tiles are summed from shared memory
      if (nseg > 1) {
        // This CTA owns the first k-range of the row-block, and the row-block continues in other CTAs, so this
        // is the last thing the CTA does: its shared-memory rings are idle (every copy into them was consumed
        // by MMAs that have completed, or this accumulator would not be ready).
        if (p.reduce_via_smem) n_smem = min(nseg - 1, ring_bytes / tile_bytes);
        if (epi_tid == 0) {
          // wait (bounded) for the other ranges' flags: all polled together, one round trip per pass
          uint32_t ok = 1;
          uint32_t pending = (1u << nseg) - 2u;  // bits 1 .. nseg-1
          const unsigned int* flags = p.seg_flags + rb * kDecMaxSegments;
          const unsigned long long t0 = global_timer_ns();
          while (true) {
            unsigned int seen[kDecMaxSegments];
#pragma unroll
            for (int sg = 1; sg < kDecMaxSegments; ++sg) seen[sg] = ((pending >> sg) & 1u) ? ld_relaxed_gpu(flags + sg) : p.tag;
#pragma unroll
            for (int sg = 1; sg < kDecMaxSegments; ++sg) {
              if (seen[sg] == p.tag) pending &= ~(1u << sg);
            }
            if (pending == 0u) break;
            if (wd.aborted()) {
              ok = 0;
              break;
            }
            if (global_timer_ns() - t0 > p.wait_limit_ns) {
              wd.give_up(kSiteDecode);
              ok = 0;
              break;
            }
          }
          asm volatile("fence.acq_rel.gpu;" ::: "memory");  // the relaxed polls above become an acquire
          if (ok && n_smem > 0) {
            // the tiles were written with ordinary stores by other SMs; order them before the bulk copies' reads
            asm volatile("fence.proxy.async;" ::: "memory");
            mbar_arrive_expect_tx(reduce_bar, static_cast<uint32_t>(n_smem * tile_bytes));
            for (int sg = 1; sg <= n_smem; ++sg) {
              bulk_copy_g2s(smem_base + static_cast<uint32_t>((sg - 1) * tile_bytes),
                            p.partials + (static_cast<size_t>(rb) * kDecMaxSegments + sg) * 128 * p.n_pad,
                            static_cast<uint32_t>(tile_bytes), reduce_bar);
            }
            if (!wd.wait(reduce_bar, reduce_phase, kSiteDecode)) {
              ok = 0;
              // the copies are under way and will land: give them time before the CTA lets go of its memory
              const unsigned long long t1 = global_timer_ns();
              while (!mbar_try_wait(reduce_bar, reduce_phase)) {
                if (global_timer_ns() - t1 > kDrainLimitNs) {
                  wd.give_up(kSiteDrainTma);
                  break;
                }
              }
            }
          }
          epi_ok[iter & 1u] = ok;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const uint32_t ok = epi_ok[iter & 1u];
        ++iter;
        if (!ok) {
          alive = false;
          break;
        }
        if (n_smem > 0) {
          // thread 0 has seen the copies complete; every reader takes its own acquire on the barrier (the
          // phase is over, so this returns at once)
          (void)mbar_try_wait(reduce_bar, reduce_phase);
          reduce_phase ^= 1u;
        }
      }
#pragma unroll 1
      for (int c0 = 0; c0 < p.n_pad; c0 += 16) {
        float a[16];
        {
          uint32_t r[16];
          tmem_ld_32x32b_x16(t_acc + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) a[i] = __uint_as_float(r[i]);
        }
        if (nseg > 1) {
          // Summed in fixed segment order: the result does not depend on arrival order.  Tiles in shared
          // memory first (they are segments 1 .. n_smem); what did not fit is read from the workspace, all
          // requests for these 16 columns in flight before any value is added.
          int pos[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) pos[i] = partial_pos((c0 >> 2) + i, row_in_tile, groups_per_row);
#pragma unroll
          for (int sg = 1; sg < kDecMaxSegments; ++sg) {
            if (sg <= n_smem) {
              const float4* row = reinterpret_cast<const float4*>(
                  generic_base + static_cast<size_t>(sg - 1) * tile_bytes + static_cast<size_t>(row_in_tile) * p.n_pad * 4);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float4 w = row[pos[i]];
                a[4 * i] += w.x;
                a[4 * i + 1] += w.y;
                a[4 * i + 2] += w.z;
                a[4 * i + 3] += w.w;
              }
            }
          }
          if (n_smem < nseg - 1) {
            float4 v[kDecMaxSegments - 1][4];
#pragma unroll
            for (int sg = 1; sg < kDecMaxSegments; ++sg) {
              if (sg > n_smem && sg < nseg) {
                const float4* row = reinterpret_cast<const float4*>(
                    p.partials + ((static_cast<size_t>(rb) * kDecMaxSegments + sg) * 128 + row_in_tile) * p.n_pad);
#pragma unroll
                for (int i = 0; i < 4; ++i) v[sg - 1][i] = __ldcg(row + pos[i]);
              }
            }
#pragma unroll
            for (int sg = 1; sg < kDecMaxSegments; ++sg) {
              if (sg > n_smem && sg < nseg) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  a[4 * i] += v[sg - 1][i].x;
                  a[4 * i + 1] += v[sg - 1][i].y;
                  a[4 * i + 2] += v[sg - 1][i].z;
                  a[4 * i + 3] += v[sg - 1][i].w;
                }
              }
            }
          }
        }
        if (out_row < p.d) {
#pragma unroll
          for (int t = 0; t < 16; ++t) {
            if (c0 + t < p.M) {
              const long long off = static_cast<long long>(c0 + t) * p.ld_out + out_row;
              float val = a[t];
              if (p.residual != nullptr) {
                val += __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.residual)[
                    static_cast<long long>(c0 + t) * p.ld_res + out_row]);
              }
              if (p.out_f32) {
                reinterpret_cast<float*>(p.out)[off] = val;
              } else {
                reinterpret_cast<__nv_bfloat16*>(p.out)[off] = __float2bfloat16_rn(val);
              }
            }
          }
        }
      }
      release_accumulator();
    }
    if (epi_tid == 0 && alive) stamp(kStampP2EpilogueDone);
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 256);
  }
}

// ------------------------------------------------------------------------------------------
// host side (used by api.cu)
// ------------------------------------------------------------------------------------------
inline cudaError_t decode_opt_in_smem() {
  return cudaFuncSetAttribute(decode_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDecSmemBytes);
}

inline int decode_pad_tokens(int64_t M) { return M <= 16 ? 16 : (M <= 32 ? 32 : 64); }

inline size_t decode_round256(size_t v) { return (v + 255) / 256 * 256; }

// phase-1 flags (one per CTA, room for kDecMaxGrid + 1) + segment flags per row-block | phase-2 partial tiles
inline size_t decode_counter_bytes(int64_t d) {
  return decode_round256((kDecMaxGrid + 1 + static_cast<size_t>((d + 127) / 128) * kDecMaxSegments) * sizeof(unsigned int));
}
inline size_t decode_workspace_bytes(int64_t M, int64_t d, int64_t) {
  const size_t n = static_cast<size_t>(decode_pad_tokens(M));
  const size_t rb2 = static_cast<size_t>((d + 127) / 128);
  return decode_counter_bytes(d) + decode_round256(rb2 * kDecMaxSegments * 128 * n * sizeof(float));
}

// Phase 1: even row split over `num_sms` CTAs, rows per CTA cut into tiles of <= 128 rows.
inline void decode_plan_rows(int64_t n_rows, int num_sms, int* tile_rows, int* tiles_per_cta, int* ctas_used) {
  int64_t per = (n_rows + num_sms - 1) / num_sms;
  if (per < 8) per = n_rows < 8 ? n_rows : 8;
  const int64_t tiles = (per + 127) / 128;
  const int64_t rows = (per + tiles - 1) / tiles;
  *tile_rows = static_cast<int>(rows);
  *tiles_per_cta = static_cast<int>(tiles);
  *ctas_used = static_cast<int>((n_rows + rows * tiles - 1) / (rows * tiles));
}

// Phase 2: largest grid (<= SM count) that keeps every row-block within kDecMaxSegments ranges.
inline int decode_grid_limit(int64_t row_blocks, int64_t k_blocks, int num_sms) {
  const int64_t units = row_blocks * k_blocks;
  int64_t g = units < num_sms ? units : num_sms;
  while (g > 1) {
    const int64_t per = units / g;
    // a row-block of k_blocks units overlaps at most ceil(k_blocks / per) + 1 ranges
    if (per >= 1 && (k_blocks + per - 1) / per + 1 <= kDecMaxSegments) break;
    --g;
  }
  return static_cast<int>(g < 1 ? 1 : g);
}

inline bool decode_supported(int64_t M, int64_t d, int64_t F, int64_t ldx, int64_t ldw_gu, int64_t ldw_d) {
  return M >= 1 && M <= kDecodeMaxTokens && d % 8 == 0 && F % 8 == 0 && ldx % 8 == 0 && ldw_gu % 8 == 0 &&
         ldw_d % 8 == 0;
}

}  // namespace fsw
