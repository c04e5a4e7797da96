// Small-batch (M <= 64 tokens) path of the SwiGLU MLP forward.  With so few
// tokens the work is streaming 3*d*F bf16 weights through the chip once, so
// the kernel is organised around HBM bandwidth, not around the tensor cores.
// ONE persistent launch does both projections:
//
//   phase 1   h[M,F]   = silu(x Wg^T) * (x Wu^T)
//   (grid-wide hand-over: every CTA has finished writing its part of h)
//   phase 2   out[M,d] = h Wd^T
//
//   * swap-AB: the WEIGHT tile (128 rows x 64 k) is the MMA's M operand and the
//     tokens (padded to N = 16/32/64) are its N operand, so a 128-lane TMEM
//     accumulator holds 128 weight rows x N tokens and no tensor-core work is
//     spent on padding M up to 128;
//   * stream-K: the (row-block, k-block) units of each phase are cut into equal
//     contiguous ranges, one per SM, so every SM streams the same number of
//     bytes however F/128 divides by the SM count;
//   * two TMA rings per SM: 11 x 16 KiB weight tiles (evict-first L2 hint) and
//     4 x 8 KiB token tiles (x in phase 1, h in phase 2).  The weight producer
//     never waits for the hand-over: while the last row-blocks of phase 1 are
//     being reduced it already fills its ring with W_down tiles, so the
//     hand-over costs no HBM idle time;
//   * row-blocks whose K range spans several CTAs are combined through fp32
//     partial tiles in a workspace; the CTA that arrives last (an atomic
//     counter per row-block, no spinning) sums the partials in FIXED segment
//     order, so results do not depend on timing, then applies SiLU(g)*u (the
//     gate is non-linear: it must see complete sums) and writes h / out;
//   * the only spin in the kernel is the token-tile producer waiting for the
//     hand-over counter; it is bounded like every other wait, and the kernel is
//     launched cooperatively so that all CTAs are resident together.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "ptx_sm100.cuh"

namespace fsw {

constexpr int kDecodeMaxTokens = 64;
constexpr int kDecThreads = 224;              // 7 warps: W producer, MMA, 4 epilogue, token-tile producer
constexpr int kDecWTileBytes = 128 * 64 * 2;  // 16 KiB: 128 weight rows x 64 k
constexpr int kDecXTileBytes = 64 * 64 * 2;   // 8 KiB: up to 64 tokens x 64 k
constexpr int kDecWSlots = 11;
constexpr int kDecXSlots = 4;
constexpr int kDecMaxSegments = 8;            // partial tiles kept per row-block
constexpr int kDecSmemBytes = kDecWSlots * kDecWTileBytes + kDecXSlots * kDecXTileBytes + 1024 + 512;

struct DecodePhase {
  void* out;              // phase 1: h bf16 [M, n_rows]; phase 2: out bf16/fp32 [M, n_rows]
  long long ld_out;
  float* partials;        // [row_blocks][kDecMaxSegments][128][acc_cols] fp32
  unsigned int* counters; // [row_blocks], zero on entry
  int n_rows;             // weight rows = output features (F, then d)
  int row_blocks;         // ceil(n_rows / 128)
  int k_blocks;           // ceil(K / 64) with K = d, then F
  int out_f32;
};

struct DecodeParams {
  DecodePhase ph[2];
  unsigned int* handover; // one counter, zero on entry: CTAs that finished phase 1
  int M;                  // tokens (<= 64)
  int n_pad;              // tokens padded to 16 / 32 / 64 (the MMA N extent)
  uint32_t* status;
#ifdef FSW_DECODE_TRACE
  unsigned long long* trace;  // [grid][8] globaltimer stamps, debug builds only
#endif
};

#ifdef FSW_DECODE_TRACE
#define FSW_TRACE(slot) do { if (p.trace) p.trace[blockIdx.x * 8 + (slot)] = global_timer_ns(); } while (0)
#else
#define FSW_TRACE(slot) do { } while (0)
#endif

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

__global__ void __launch_bounds__(kDecThreads, 1)
decode_fused_kernel(const __grid_constant__ CUtensorMap map_gate, const __grid_constant__ CUtensorMap map_up,
                    const __grid_constant__ CUtensorMap map_down, const __grid_constant__ CUtensorMap map_x,
                    const __grid_constant__ CUtensorMap map_h, const DecodeParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t w_ring = smem_base;
  const uint32_t x_ring = smem_base + kDecWSlots * kDecWTileBytes;
  const uint32_t bar_base = x_ring + kDecXSlots * kDecXTileBytes;
  auto w_full = [&](int s) { return bar_base + 8u * s; };
  auto w_empty = [&](int s) { return bar_base + 8u * (kDecWSlots + s); };
  auto x_full = [&](int s) { return bar_base + 8u * (2 * kDecWSlots + s); };
  auto x_empty = [&](int s) { return bar_base + 8u * (2 * kDecWSlots + kDecXSlots + s); };
  constexpr int kBarsBeforeTmem = 2 * kDecWSlots + 2 * kDecXSlots;
  auto tfull_bar = [&](int a) { return bar_base + 8u * (kBarsBeforeTmem + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (kBarsBeforeTmem + 2 + a); };
  const uint32_t drain_bar = bar_base + 8u * (kBarsBeforeTmem + 4);
  uint8_t* generic_base = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t* tmem_ptr_slot = reinterpret_cast<volatile uint32_t*>(
      generic_base + kDecWSlots * kDecWTileBytes + kDecXSlots * kDecXTileBytes + 8 * (kBarsBeforeTmem + 5));
  volatile uint32_t* abort_flag = tmem_ptr_slot + 1;
  volatile uint32_t* last_flag = tmem_ptr_slot + 2;
  volatile uint32_t* epi_ok = tmem_ptr_slot + 3;  // two entries, alternating per segment

  const int warp = threadIdx.x >> 5;
  const uint32_t lane = lane_id();
  const Watchdog wd{abort_flag, p.status};

  constexpr int kAccStride = 128;  // TMEM columns per accumulator stage (2 stages)
  const uint32_t x_tile_tx = static_cast<uint32_t>(p.n_pad) * 128u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kDecWSlots; ++s) {
      mbar_init(w_full(s), 1);
      mbar_init(w_empty(s), 1);
    }
    for (int s = 0; s < kDecXSlots; ++s) {
      mbar_init(x_full(s), 1);
      mbar_init(x_empty(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 128);
    }
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    *last_flag = 0;
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
  if (threadIdx.x == 0) FSW_TRACE(0);

  // This CTA's unit range in each phase.
  long long u_begin[2], u_end[2], units[2];
  for (int q = 0; q < 2; ++q) {
    units[q] = static_cast<long long>(p.ph[q].row_blocks) * p.ph[q].k_blocks;
    u_begin[q] = dec_range_start(blockIdx.x, units[q], gridDim.x);
    u_end[q] = dec_range_start(blockIdx.x + 1, units[q], gridDim.x);
  }

  if (warp == 0) {
    // ------------------- weight-tile producer: never waits for the hand-over -------------------
    if (lane == 0) {
      const uint64_t stream_once = l2_policy_evict_first();
      int slot = 0;
      uint32_t phase = 0;
      uint32_t issued_mask = 0, last_parity_mask = 0;
      bool alive = true;
      auto push = [&](const CUtensorMap* map, int x, int y) -> bool {
        if (!wd.wait(w_empty(slot), phase ^ 1u, kSiteProducerEmpty)) return false;
        mbar_arrive_expect_tx(w_full(slot), kDecWTileBytes);
        tma_load_2d_hint(w_ring + slot * kDecWTileBytes, map, w_full(slot), x, y, stream_once);
        issued_mask |= 1u << slot;
        last_parity_mask = (last_parity_mask & ~(1u << slot)) | (phase << slot);
        if (++slot == kDecWSlots) {
          slot = 0;
          phase ^= 1u;
        }
        return true;
      };
      for (int q = 0; q < 2 && alive; ++q) {
        const int kbs = p.ph[q].k_blocks;
        for (long long u = u_begin[q]; u < u_end[q] && alive; ++u) {
          const int rb = static_cast<int>(u / kbs);
          const int kb = static_cast<int>(u - static_cast<long long>(rb) * kbs);
          if (q == 0) {
            alive = push(&map_gate, kb * 64, rb * 128) && push(&map_up, kb * 64, rb * 128);
          } else {
            alive = push(&map_down, kb * 64, rb * 128);
          }
        }
      }
      if (wd.aborted()) {
        for (int s = 0; s < kDecWSlots; ++s) {
          if (issued_mask & (1u << s)) {
            const uint32_t par = (last_parity_mask >> s) & 1u;
            const unsigned long long t0 = global_timer_ns();
            while (!mbar_try_wait(w_full(s), par)) {
              if (global_timer_ns() - t0 > 50000000ull) {
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
    if (lane == 0) {
      const uint64_t keep = l2_policy_evict_last();
      int slot = 0;
      uint32_t phase = 0;
      uint32_t issued_mask = 0, last_parity_mask = 0;
      bool alive = true;
      for (int q = 0; q < 2 && alive; ++q) {
        if (q == 1 && u_begin[1] < u_end[1]) {
          // h is complete once every CTA has counted itself in (release/acquire through the counter)
          const unsigned long long t0 = global_timer_ns();
          while (ld_acquire_gpu(p.handover) < gridDim.x) {
            __nanosleep(64);
            if (wd.aborted()) {
              alive = false;
              break;
            }
            if (global_timer_ns() - t0 > kWaitLimitNs) {
              wd.give_up(kSiteDecode);
              alive = false;
              break;
            }
          }
          if (!alive) break;
          // h was written with ordinary stores by other SMs; order them before this SM's TMA reads
          asm volatile("fence.proxy.async;" ::: "memory");
          FSW_TRACE(7);
        }
        const CUtensorMap* map = (q == 0) ? &map_x : &map_h;
        const int kbs = p.ph[q].k_blocks;
        for (long long u = u_begin[q]; u < u_end[q]; ++u) {
          const int kb = static_cast<int>(u % kbs);
          if (!wd.wait(x_empty(slot), phase ^ 1u, kSiteProducerEmpty)) {
            alive = false;
            break;
          }
          mbar_arrive_expect_tx(x_full(slot), x_tile_tx);
          tma_load_2d_hint(x_ring + slot * kDecXTileBytes, map, x_full(slot), kb * 64, 0, keep);
          issued_mask |= 1u << slot;
          last_parity_mask = (last_parity_mask & ~(1u << slot)) | (phase << slot);
          if (++slot == kDecXSlots) {
            slot = 0;
            phase ^= 1u;
          }
        }
      }
      if (wd.aborted()) {
        for (int s = 0; s < kDecXSlots; ++s) {
          if (issued_mask & (1u << s)) {
            const uint32_t par = (last_parity_mask >> s) & 1u;
            const unsigned long long t0 = global_timer_ns();
            while (!mbar_try_wait(x_full(s), par)) {
              if (global_timer_ns() - t0 > 50000000ull) {
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
      for (int q = 0; q < 2 && alive; ++q) {
        const int kbs = p.ph[q].k_blocks;
        long long u = u_begin[q];
        while (u < u_end[q] && alive) {
          const int rb = static_cast<int>(u / kbs);
          const long long seg_end = min(u_end[q], static_cast<long long>(rb + 1) * kbs);
          if (!wd.wait(tempty_bar(acc), acc_phase ^ 1u, kSiteMmaTmemEmpty)) {
            alive = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kAccStride);
          bool first = true;
          for (; u < seg_end; ++u) {
            // weight tile(s) of this unit, then its token tile
            const int w0 = ws;
            if (!wd.wait(w_full(w0), wphase, kSiteMmaFull)) {
              alive = false;
              break;
            }
            if (++ws == kDecWSlots) {
              ws = 0;
              wphase ^= 1u;
            }
            int w1 = w0;
            if (q == 0) {
              w1 = ws;
              if (!wd.wait(w_full(w1), wphase, kSiteMmaFull)) {
                alive = false;
                break;
              }
              if (++ws == kDecWSlots) {
                ws = 0;
                wphase ^= 1u;
              }
            }
            if (!wd.wait(x_full(xs), xphase, kSiteMmaFull)) {
              alive = false;
              break;
            }
            tc_fence_after_sync();
            if (first && u == u_begin[q]) FSW_TRACE(q == 0 ? 1 : 4);
            const uint64_t w0_desc = umma_desc_k_sw128(w_ring + w0 * kDecWTileBytes);
            const uint64_t w1_desc = umma_desc_k_sw128(w_ring + w1 * kDecWTileBytes);
            const uint64_t x_desc = umma_desc_k_sw128(x_ring + xs * kDecXTileBytes);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const uint32_t accum = (first && k == 0) ? 0u : 1u;
              umma_bf16_ss(d_tmem, w0_desc + 2u * k, x_desc + 2u * k, idesc, accum);
              if (q == 0) umma_bf16_ss(d_tmem + p.n_pad, w1_desc + 2u * k, x_desc + 2u * k, idesc, accum);
            }
            first = false;
            umma_commit(w_empty(w0));
            if (q == 0) umma_commit(w_empty(w1));
            umma_commit(x_empty(xs));
            if (++xs == kDecXSlots) {
              xs = 0;
              xphase ^= 1u;
            }
          }
          if (!alive) break;
          umma_commit(tfull_bar(acc));
          acc ^= 1;
          if (acc == 0) acc_phase ^= 1u;
        }
        FSW_TRACE(q == 0 ? 2 : 5);
      }
      if (wd.aborted()) {
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
    // -------------------------------------- epilogue -------------------------------------------
    const int quarter = warp & 3;
    const int row_in_block = quarter * 32 + static_cast<int>(lane);  // weight row within the row-block
    const uint32_t lane_field = static_cast<uint32_t>(quarter * 32) << 16;
    const int epi_tid = static_cast<int>(threadIdx.x) - 64;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool alive = true;
    uint32_t seg_iter = 0;
    for (int q = 0; q < 2 && alive; ++q) {
      const DecodePhase& ph = p.ph[q];
      const bool gated = (q == 0);
      const int acc_cols = gated ? 2 * p.n_pad : p.n_pad;
      long long u = u_begin[q];
      while (u < u_end[q]) {
        const int rb = static_cast<int>(u / ph.k_blocks);
        const long long rb_first = static_cast<long long>(rb) * ph.k_blocks;
        const long long seg_end = min(u_end[q], rb_first + ph.k_blocks);
        // which contiguous ranges (CTAs) share this row-block, and which of them am I
        const int first_cta = dec_owner(rb_first, units[q], gridDim.x);
        const int last_cta = dec_owner(rb_first + ph.k_blocks - 1, units[q], gridDim.x);
        const int nseg = last_cta - first_cta + 1;
        const int seg = static_cast<int>(blockIdx.x) - first_cta;
        u = seg_end;

        // One thread waits for the accumulator and tells the other 127: the four epilogue warps
        // share named barriers below, so they must all take the same exit if a wait gives up.
        if (epi_tid == 0) epi_ok[seg_iter & 1u] = wd.wait(tfull_bar(acc), acc_phase, kSiteEpilogueFull) ? 1u : 0u;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const uint32_t ok = epi_ok[seg_iter & 1u];
        ++seg_iter;
        if (!ok) {
          alive = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t t_acc = tmem_base + lane_field + static_cast<uint32_t>(acc * kAccStride);
        const int out_row = rb * 128 + row_in_block;  // output feature index

        bool reduce_here = true;
        if (nseg > 1) {
          // publish this segment's partial sums: [row][acc_cols] fp32, one contiguous run per thread
          float* my_tile =
              ph.partials + ((static_cast<size_t>(rb) * kDecMaxSegments + seg) * 128 + row_in_block) * acc_cols;
#pragma unroll 1
          for (int c0 = 0; c0 < acc_cols; c0 += 16) {
            uint32_t r[16];
            tmem_ld_32x32b_x16(t_acc + c0, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              __stcg(reinterpret_cast<float4*>(my_tile + c0) + i,
                     make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]),
                                 __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3])));
            }
          }
          tc_fence_before_sync();
          mbar_arrive(tempty_bar(acc));  // accumulator drained: the MMA warp may reuse it
          __threadfence();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (epi_tid == 0) {
            const unsigned int old = atomicAdd(ph.counters + rb, 1u);
            *last_flag = (old == static_cast<unsigned int>(nseg - 1)) ? 1u : 0u;
            __threadfence();
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          reduce_here = (*last_flag != 0);
          asm volatile("bar.sync 1, 128;" ::: "memory");  // everyone has read the flag before it is reused
        }

        if (reduce_here) {
          // complete sums for this thread's weight row, 16 token columns at a time
#pragma unroll 1
          for (int c0 = 0; c0 < p.n_pad; c0 += 16) {
            float a[16], b[16];
            if (nseg > 1) {
#pragma unroll
              for (int i = 0; i < 16; ++i) a[i] = b[i] = 0.0f;
              for (int s = 0; s < nseg; ++s) {  // fixed order: the result does not depend on arrival order
                const float* tile =
                    ph.partials + ((static_cast<size_t>(rb) * kDecMaxSegments + s) * 128 + row_in_block) * acc_cols;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float4 v = __ldcg(reinterpret_cast<const float4*>(tile + c0) + i);
                  a[4 * i] += v.x; a[4 * i + 1] += v.y; a[4 * i + 2] += v.z; a[4 * i + 3] += v.w;
                  if (gated) {
                    const float4 w = __ldcg(reinterpret_cast<const float4*>(tile + p.n_pad + c0) + i);
                    b[4 * i] += w.x; b[4 * i + 1] += w.y; b[4 * i + 2] += w.z; b[4 * i + 3] += w.w;
                  }
                }
              }
            } else {
              uint32_t r[16], s2[16];
              tmem_ld_32x32b_x16(t_acc + c0, r);
              if (gated) tmem_ld_32x32b_x16(t_acc + p.n_pad + c0, s2);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                a[i] = __uint_as_float(r[i]);
                b[i] = gated ? __uint_as_float(s2[i]) : 0.0f;
              }
            }
            if (out_row < ph.n_rows) {
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const int t = c0 + i;  // token
                if (t < p.M) {
                  const float v = gated ? silu_mul(a[i], b[i]) : a[i];
                  const long long off = static_cast<long long>(t) * ph.ld_out + out_row;
                  if (!gated && ph.out_f32) {
                    reinterpret_cast<float*>(ph.out)[off] = v;
                  } else {
                    reinterpret_cast<__nv_bfloat16*>(ph.out)[off] = __float2bfloat16_rn(v);
                  }
                }
              }
            }
          }
        }
        if (nseg == 1) {
          tc_fence_before_sync();
          mbar_arrive(tempty_bar(acc));
        }
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
      if (q == 0) {
        // hand-over: everything this CTA contributes to h is written; count it in
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (epi_tid == 0 && alive) {
          asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.handover) : "memory");
          FSW_TRACE(3);
        }
      } else if (epi_tid == 0) {
        FSW_TRACE(6);
      }
    }
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

// hand-over counter + arrival counters (both phases) | phase-1 partial tiles | phase-2 partial tiles
inline size_t decode_counter_bytes(int64_t d, int64_t F) {
  const size_t rb1 = static_cast<size_t>((F + 127) / 128), rb2 = static_cast<size_t>((d + 127) / 128);
  return decode_round256((1 + rb1 + rb2) * sizeof(unsigned int));
}
inline size_t decode_workspace_bytes(int64_t M, int64_t d, int64_t F) {
  const size_t n = static_cast<size_t>(decode_pad_tokens(M));
  const size_t rb1 = static_cast<size_t>((F + 127) / 128), rb2 = static_cast<size_t>((d + 127) / 128);
  size_t bytes = decode_counter_bytes(d, F);
  bytes += decode_round256(rb1 * kDecMaxSegments * 128 * (2 * n) * sizeof(float));
  bytes += decode_round256(rb2 * kDecMaxSegments * 128 * n * sizeof(float));
  return bytes;
}

// Largest grid (<= SM count) that keeps every row-block of a phase within kDecMaxSegments ranges.
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
