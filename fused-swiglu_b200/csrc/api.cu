// C ABI of libfswiglu.so (declared in include/fswiglu.h): argument checks,
// TMA tensor-map encoding, tile rasterisation choices and kernel launches.
// No torch types and no allocation on the hot path; the only device memory
// this file owns is one 256-byte status block per device.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "../../include/fswiglu.h"
#include "decode_sm100.cuh"
#include "elementwise_sm100.cuh"
#include "gemm_pair_sm100.cuh"
#include "gemm_quad_sm100.cuh"
#include "gemm_sm100.cuh"
#include "host_slabs.h"

namespace fsw {

// fp32 -> bf16 (RNE), 8 elements per thread per step, grid-stride.
__global__ void __launch_bounds__(256) cast_f32_to_bf16_kernel(const float4* __restrict__ src,
                                                                uint4* __restrict__ dst, long long n8,
                                                                const float* __restrict__ src_tail,
                                                                __nv_bfloat16* __restrict__ dst_tail, int tail) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += stride) {
    const float4 a = src[2 * i];
    const float4 b = src[2 * i + 1];
    uint4 q;
    q.x = pack_bf16x2(a.x, a.y);
    q.y = pack_bf16x2(a.z, a.w);
    q.z = pack_bf16x2(b.x, b.y);
    q.w = pack_bf16x2(b.z, b.w);
    dst[i] = q;
  }
  if (blockIdx.x == 0 && static_cast<int>(threadIdx.x) < tail) {
    dst_tail[threadIdx.x] = __float2bfloat16_rn(src_tail[threadIdx.x]);
  }
}

// Second half of the tensor-parallel reduction: this rank owns `rows` rows; recv holds one bf16
// partial copy of them per source rank ([world][rows][cols], local memory, written by the ranks'
// down-GEMM epilogues).  Sum the copies in fp32 in rank order (every element is reduced by exactly one
// rank, so all ranks end up with identical bits), round once, and store the result into every
// rank's output buffer (peer stores over NVLink).  16 bytes per thread per step.  128 threads and no
// shared memory per CTA, so that these CTAs fit on an SM next to a persistent GEMM CTA (registers:
// 192 x 240 + 128 x 80 < 64 K) and the reduction of one row slab can run under the next slab's GEMMs
// without SMs being set aside for it.
struct ReduceBcastParams {
  const uint4* recv;
  void* out[8];          // per destination rank: base of its [*, cols] output, already offset to these rows
  long long n16;         // rows * cols / 8
  int world;
};
__global__ void __launch_bounds__(128) reduce_bcast_bf16_kernel(const ReduceBcastParams p) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < p.n16; i += stride) {
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.0f;
    uint4 v[8];
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      if (s < p.world) v[s] = __ldcs(p.recv + s * p.n16 + i);
    }
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      if (s < p.world) {
        const uint32_t w[4] = {v[s].x, v[s].y, v[s].z, v[s].w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          acc[2 * k] += __uint_as_float(w[k] << 16);
          acc[2 * k + 1] += __uint_as_float(w[k] & 0xffff0000u);
        }
      }
    }
    uint4 q;
    q.x = pack_bf16x2(acc[0], acc[1]);
    q.y = pack_bf16x2(acc[2], acc[3]);
    q.z = pack_bf16x2(acc[4], acc[5]);
    q.w = pack_bf16x2(acc[6], acc[7]);
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      if (s < p.world) reinterpret_cast<uint4*>(p.out[s])[i] = q;
    }
  }
}

// Per-row RMSNorm statistic  scale[r] = rsqrt(mean(x[r, :]^2) + eps)  in fp32: one warp per row,
// 16-byte loads, fixed reduction order.  The gate-up epilogue multiplies its fp32 accumulators by
// this factor, which equals normalising x before the GEMM (the norm's weight vector is folded into
// the columns of W_gate / W_up once, at load time).
__global__ void __launch_bounds__(256) rms_scale_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int M,
                                                         int d, float eps, float* __restrict__ scale) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < M; row += gridDim.x * warps_per_block) {
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<long long>(row) * ldx);
    float ss = 0.0f;
    for (int i = lane; i < d / 8; i += 32) {
      const uint4 q = __ldg(src + i);
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float a = __uint_as_float(w[k] << 16), b = __uint_as_float(w[k] & 0xffff0000u);
        ss = fmaf(a, a, ss);
        ss = fmaf(b, b, ss);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) scale[row] = rsqrtf(ss / static_cast<float>(d) + eps);
  }
}

}  // namespace fsw

namespace {

using namespace fsw;

constexpr int kMaxDevices = 64;


struct DeviceState {
  bool ready = false;
  int num_sms = 0;
  uint32_t* status = nullptr;  // device memory, 64 words
  int max_ctas = 0;            // upper bound on the CTAs of the tiled kernels on this device, 0 = every SM
  // Lazily created by the host-buffer entry point only.
  bool host_ready = false;
  cudaStream_t h2d_stream = nullptr;
  cudaStream_t d2h_stream = nullptr;
  cudaEvent_t ev_start = nullptr;
  cudaEvent_t ev_h2d[kMaxHostSlabs] = {};
  cudaEvent_t ev_done[kMaxHostSlabs] = {};
  std::mutex host_mutex;  // serialises the host-buffer entry point per device
};

std::mutex g_mutex;
DeviceState g_dev[kMaxDevices];
std::atomic<uint64_t> g_launches{0};
std::atomic<unsigned long long> g_wait_limit_ns{kWaitLimitNs};
std::atomic<unsigned long long*> g_decode_trace{nullptr};  // profiling aid, see fswiglu_set_decode_trace
std::atomic<int> g_withhold_one_copy{0};  // test aid, consumed by the next launch (see fswiglu_test_expire_next_wait)

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

template <typename Kernel>
cudaError_t opt_in_smem(Kernel k, int bytes) {
  return cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

// Capability check, driver entry point for tensor-map encoding and the kernels' shared-memory
// opt-in for device `dev` (the current device).  Allocates nothing.  Caller holds g_mutex.
int prepare_device(int dev, int* num_sms) {
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return FSWIGLU_ERR_NO_DEVICE;
  if (prop.major != 10) return FSWIGLU_ERR_NO_DEVICE;
  *num_sms = prop.multiProcessorCount;
  if (g_encode == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
        fn == nullptr) {
      return FSWIGLU_ERR_CUDA;
    }
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  cudaError_t e = cudaSuccess;
  e = e ? e : opt_in_smem(gemm_tcgen05_kernel<kPlain, false>, kGemmSmemBytes);
  e = e ? e : opt_in_smem(gemm_tcgen05_kernel<kPlain, true>, kGemmSmemBytes);
  e = e ? e : opt_in_smem(gemm_tcgen05_kernel<kGatedSplit, false>, kGemmSmemBytes);
  e = e ? e : opt_in_smem(gemm_tcgen05_kernel<kGatedInterleaved, false>, kGemmSmemBytes);
  e = e ? e : decode_opt_in_smem();
  e = e ? e : opt_in_smem(gemm_pair_kernel<kPlain, false>, kPairSmemBytes);
  e = e ? e : opt_in_smem(gemm_pair_kernel<kPlain, true>, kPairSmemBytes);
  e = e ? e : opt_in_smem(gemm_pair_kernel<kGatedSplit, false>, kPairSmemBytes);
  e = e ? e : opt_in_smem(gemm_pair_kernel<kGatedInterleaved, false>, kPairSmemBytes);
  e = e ? e : opt_in_smem(gemm_quad_kernel<kPlain, false>, kQuadSmemBytes);
  e = e ? e : opt_in_smem(gemm_quad_kernel<kPlain, true>, kQuadSmemBytes);
  e = e ? e : opt_in_smem(gemm_quad_kernel<kGatedSplit, false>, kQuadSmemBytes);
  e = e ? e : opt_in_smem(gemm_quad_kernel<kGatedInterleaved, false>, kQuadSmemBytes);
  return e == cudaSuccess ? FSWIGLU_OK : FSWIGLU_ERR_CUDA;
}

// One-time per-device set-up of the ordinary entry points: the above plus the 256-byte status block.
int device_state(DeviceState** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return FSWIGLU_ERR_NO_DEVICE;
  if (dev < 0 || dev >= kMaxDevices) return FSWIGLU_ERR_NO_DEVICE;
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceState& st = g_dev[dev];
  if (!st.ready) {
    if (int rc = prepare_device(dev, &st.num_sms)) return rc;
    if (cudaMalloc(&st.status, 256) != cudaSuccess) return FSWIGLU_ERR_CUDA;
    if (cudaMemset(st.status, 0, 256) != cudaSuccess) return FSWIGLU_ERR_CUDA;
    st.ready = true;
  }
  *out = &st;
  return FSWIGLU_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Tensor map over a row-major bf16 matrix [rows, cols] with pitch `ld` elements; one box is
// 64 columns (128 bytes, the swizzle width) x box_rows rows.
int encode_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld,
               uint32_t box_rows) {
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2u};
  const cuuint32_t box[2] = {64u, box_rows};
  const cuuint32_t elem_strides[2] = {1u, 1u};
  const CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                              strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FSWIGLU_OK : FSWIGLU_ERR_CUDA;
}

int check_matrix(const void* p, int64_t rows, int64_t cols, int64_t ld, bool tma_read) {
  if (p == nullptr) return FSWIGLU_ERR_BAD_ARG;
  if (rows < 0 || cols <= 0) return FSWIGLU_ERR_BAD_ARG;
  if (rows > 0x7fffffffll || cols > 0x7fffffffll) return FSWIGLU_ERR_SHAPE;
  if (ld < cols) return FSWIGLU_ERR_SHAPE;
  if (tma_read) {
    if (cols % 8 != 0) return FSWIGLU_ERR_SHAPE;
    if (!aligned16(p) || ld % 8 != 0) return FSWIGLU_ERR_ALIGNMENT;
  }
  return FSWIGLU_OK;
}

// How many 128-row M-tiles share one sweep over N.  B is re-read from DRAM once per group of
// M-tiles while the group's slab of A (group_m * 128 rows * K bf16) is read once and then
// served from the 126 MB L2, so DRAM traffic = |A| + |B| * groups: use as few groups as an
// 80 MB slab budget allows, of equal size.
int pick_group_m(int num_m_tiles, int64_t K) {
  int64_t slab_budget = 80ll << 20;
  if (const char* env = std::getenv("FSWIGLU_SLAB_MB")) {  // experiments only
    const int v = std::atoi(env);
    if (v >= 1 && v <= 4096) slab_budget = static_cast<int64_t>(v) << 20;
  }
  int64_t g = slab_budget / (128 * K * 2);
  if (g < 1) g = 1;
  if (g > num_m_tiles) g = num_m_tiles;
  const int64_t groups = (num_m_tiles + g - 1) / g;
  g = (num_m_tiles + groups - 1) / groups;
  return static_cast<int>(g);
}

// Raster of the two-SM kernel: how many 256-row M-tiles share a sweep over N.  The clusters that run at
// the same time work on group_m M-tiles x (clusters / group_m) N-tiles, and what they read from HBM is
// decided by what the L2 keeps between their reads.  Measured on B200 (DRAM counters and sustained rates at
// the 7B, 70B, 70B-shard and ragged-13B-shard shapes): operands shared by all SMs are kept in both halves of
// the L2, so only about 50 MB of such data stay resident, and a full-K operand row of one tile is large
// (256 rows x K x 2 bytes: 4 MB at K = 8192).
//   * B small enough to stay resident: a wave should span all N-tiles, so that every A row is read once;
//   * A small enough to stay resident: one group, every wave re-uses the same A rows;
//   * neither: the most compact wave, group_m ~ sqrt(clusters), which minimises the distinct operand rows
//     per wave (nothing survives from one wave to the next anyway).
int pick_pair_group_m(int num_m_tiles, int num_n_tiles, int64_t K, int clusters) {
  const int64_t row_bytes = 256 * K * 2;  // one M-tile of A, or one N-tile of B (256 operand rows in every mode)
  const int64_t resident = 48ll << 20;
  int g;
  if (num_n_tiles * row_bytes <= resident) {
    g = (clusters + num_n_tiles - 1) / num_n_tiles;
  } else if (num_m_tiles * row_bytes <= resident) {
    g = num_m_tiles;
  } else {
    g = 1;
    while ((g + 1) * (g + 1) <= clusters) ++g;  // floor(sqrt(clusters)): 8 for 74 clusters
  }
  return std::max(1, std::min(g, num_m_tiles));
}

// Width of a tile in output columns.  Measured on B200, a tile's main loop is bound by the
// bytes its CTA pulls from L2 per k-block (A: 128 rows, B: one row per MMA column; about
// 64 B/clk per SM), not by the MMA itself, so a tile costs time proportional to
// (128 + MMA columns) and narrower tiles move more bytes per flop.  The persistent schedule
// gives every CTA ceil(tiles / SMs) tiles, hence cost(width) = waves * (128 + MMA columns).
// Wide tiles win whenever the grid is full; narrower ones only pay off when the problem
// would otherwise leave SMs idle.  A narrower width must beat a wider one by 3 % to be
// chosen.  `mma_per_col` is 1 for the plain GEMM, 2 for the gated one (a gate and an up
// column per output column).  FSWIGLU_TILE_N overrides the choice, for experiments.
int pick_tile_n(int num_m_tiles, int64_t n_out, int max_tile, int mma_per_col, int num_sms) {
  if (const char* env = std::getenv("FSWIGLU_TILE_N")) {
    const int v = std::atoi(env);
    if (v >= 16 && v <= max_tile && v % 16 == 0) return v;
  }
  int best = max_tile;
  double best_cost = 1e300;
  for (int t = max_tile; t >= 32 / mma_per_col; t -= 16) {
    const int64_t n_tiles = (n_out + t - 1) / t;
    const int64_t tiles = n_tiles * num_m_tiles;
    const int64_t waves = (tiles + num_sms - 1) / num_sms;
    const double cost = static_cast<double>(waves) * (128 + t * mma_per_col);
    if (cost < best_cost * 0.97) {
      best_cost = cost;
      best = t;
    }
  }
  // never wider than the problem (rounded up to the 16-column granule)
  const int needed = static_cast<int>((n_out + 15) / 16 * 16);
  return best < needed ? best : (needed < 16 ? 16 : needed);
}

// Tail split (see GemmParams::split_from): on when FSWIGLU_TAIL_SPLIT=1, off when =0.
constexpr bool kTailSplitDefault = false;
bool tail_split_enabled() {
  const char* env = std::getenv("FSWIGLU_TAIL_SPLIT");
  if (env == nullptr || env[0] == '\0') return kTailSplitDefault;
  return env[0] != '0';
}

// Decide whether the tiles of the last, partly filled wave are processed as half-width units:
// worth it when that wave fills at most half of the CTAs (two units per tile still fit in one wave).
void plan_tail_split(GemmParams* p, int ctas) {
  const int tiles = p->num_m_tiles * p->num_n_tiles;
  p->split_from = tiles;
  p->half_boxes = 0;
  if (!tail_split_enabled() || p->tile_n % 32 != 0 || tiles <= ctas) return;
  const int rem = tiles % ctas;
  if (rem > 0 && 2 * rem <= ctas) {
    p->split_from = tiles - rem;
    p->half_boxes = 1;
  }
}

int effective_ctas(const DeviceState& st) {
  const int cap = st.max_ctas;
  return (cap > 0 && cap < st.num_sms) ? cap : st.num_sms;
}

template <int kMode, bool kOutF32>
int launch_gemm(const DeviceState& st, const CUtensorMap& ma, const CUtensorMap& mb0,
                const CUtensorMap& mb1, const GemmParams& p, cudaStream_t stream) {
  const int tiles = p.num_m_tiles * p.num_n_tiles;
  const int units = p.split_from + 2 * (tiles - p.split_from);
  const int ctas = effective_ctas(st);
  const int grid = units < ctas ? units : ctas;
  GemmParams q = p;
  q.wait_limit_ns = g_wait_limit_ns.load(std::memory_order_relaxed);
  q.withhold_one_copy = g_withhold_one_copy.exchange(0, std::memory_order_relaxed);
  gemm_tcgen05_kernel<kMode, kOutF32><<<grid, kGemmThreads, kGemmSmemBytes, stream>>>(ma, mb0, mb1, q);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? FSWIGLU_OK : FSWIGLU_ERR_CUDA;
}

// Two-SM kernel (gemm_pair_sm100.cuh): used whenever the problem fills at least one wave of 256-row
// pair tiles (otherwise the one-SM kernel with its adaptive tile width spreads the work better).
// Measured against the one-SM kernel at the 7B / 70B-shard shapes: bit-identical results, +10 ... +20 %
// in short bursts (1647 vs 1502 TF/s gate-up), +1 % once the 1 kW power cap sets the clock.
// FSWIGLU_PAIR=0 selects the one-SM kernel everywhere, FSWIGLU_PAIR=force the two-SM kernel
// everywhere (tests use it to run small ragged problems through the kernel the large shapes take).
int pair_mode() {  // 0 never, 1 automatic, 2 always
  const char* env = std::getenv("FSWIGLU_PAIR");
  if (env == nullptr || env[0] == '\0') return 1;
  if (env[0] == '0') return 0;
  return (env[0] == 'f' || env[0] == 'F') ? 2 : 1;
}
bool use_pair_kernel(const DeviceState& st, int64_t M, int64_t n_out, int tile_n) {
  const int mode = pair_mode();
  if (mode == 0 || effective_ctas(st) < 2) return false;
  if (mode == 2) return true;
  if (M <= 128) return false;
  const int64_t pairs = ((M + 255) / 256) * ((n_out + tile_n - 1) / tile_n);
  return pairs >= effective_ctas(st) / 2;
}

// Scratch of the split last wave (GemmParams::tail_*): a counter block, then the fp32 partial blocks.
// A launch uses blocks (cluster + tail tile) * 2 + rank with cluster < clusters and tail tile <
// clusters, so 4 * clusters blocks of 128 KiB always suffice; sized for the 74 clusters of a B200.
constexpr size_t kTailCounterBytes = 4096;
constexpr int kTailMaxClusters = 74;
constexpr size_t kTailScratchBytes =
    kTailCounterBytes + static_cast<size_t>(4) * kTailMaxClusters * kTailBlockFloats * sizeof(float);

struct Scratch {
  void* ptr = nullptr;
  size_t bytes = 0;
  bool counters_clean = false;  // the caller has already zeroed the counter block on this stream
};

// FSWIGLU_TAIL_SPLITK=0 turns the split off, =force applies it whenever the last wave is partial
// (tests use it to reach the shared-tile path with small problems).
int tail_split_k_mode() {  // 0 off, 1 when it pays, 2 always
  const char* env = std::getenv("FSWIGLU_TAIL_SPLITK");
  if (env == nullptr || env[0] == '\0') return 1;
  if (env[0] == '0') return 0;
  return (env[0] == 'f' || env[0] == 'F') ? 2 : 1;
}

// Decide how the last, partly filled wave of pair tiles is processed (pair_schedule.cuh).
void plan_pair_tail(GemmParams* p, int clusters, int num_kb, const Scratch& scratch) {
  const int tiles = p->num_m_tiles * p->num_n_tiles;
  p->tail_first = tiles;
  p->tail_len = 0;
  p->tail_partials = nullptr;
  p->tail_counters = nullptr;
  if (scratch.ptr == nullptr || scratch.bytes < kTailScratchBytes || clusters > kTailMaxClusters) return;
  plan_pair_tail_split(tiles, clusters, num_kb, tail_split_k_mode(), &p->tail_first, &p->tail_len);
  if (p->tail_len == 0) return;
  p->tail_counters = static_cast<unsigned int*>(scratch.ptr);
  p->tail_partials = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch.ptr) + kTailCounterBytes);
}

// FSWIGLU_TAIL_HALVES=0 turns the width-split of the last wave off (experiments, A/B timing).
bool tail_halves_enabled() {
  const char* env = std::getenv("FSWIGLU_TAIL_HALVES");
  return env == nullptr || env[0] != '0';
}

// `p` arrives filled for the one-SM kernel; re-plan it for 256-row pair tiles of full width.
template <int kMode, bool kOutF32>
int launch_gemm_pair(const DeviceState& st, const void* a, int64_t lda, const void* b0, const void* b1, int64_t ldb,
                     int64_t b_rows, GemmParams p, const Scratch& scratch, cudaStream_t stream) {
  p.tile_n = (kMode == kPlain) ? 256 : 128;
  p.num_m_tiles = (p.M + 255) / 256;
  p.num_n_tiles = (p.n_out + p.tile_n - 1) / p.tile_n;
  const int pairs = p.num_m_tiles * p.num_n_tiles;
  const int clusters = std::max(1, std::min(pairs, effective_ctas(st) / 2));
  p.group_m = pick_pair_group_m(p.num_m_tiles, p.num_n_tiles, p.K, clusters);
  if (const char* env = std::getenv("FSWIGLU_GROUP_M")) {  // experiments only
    const int v = std::atoi(env);
    if (v >= 1) p.group_m = std::min(v, p.num_m_tiles);
  }
  if (const char* env = std::getenv("FSWIGLU_K_ALTERNATE")) p.k_alternate = std::atoi(env) != 0 ? 1 : 0;
  if (const char* env = std::getenv("FSWIGLU_HINT_A")) p.hint_a = std::atoi(env);
  if (const char* env = std::getenv("FSWIGLU_HINT_B")) p.hint_b = std::atoi(env);
  p.split_from = p.num_m_tiles * p.num_n_tiles;
  p.half_boxes = 0;
  // last, partly filled wave: split along K when that clearly pays (needs scratch), else by width when its
  // tiles fill at most half of the clusters
  plan_pair_tail(&p, clusters, (p.K + kBlockK - 1) / kBlockK, scratch);
  p.tail_halves = 0;
  if (p.tail_len == 0 && tail_halves_enabled() && plan_pair_tail_halves(pairs, clusters, p.tile_n, &p.tail_first)) {
    p.tail_halves = 1;
  }
  int rc;
  CUtensorMap ma, mb0, mb1, mh0, mh1;
  if ((rc = encode_map(&ma, a, p.M, p.K, lda, 128))) return rc;
  if ((rc = encode_map(&mb0, b0, b_rows, p.K, ldb, 128))) return rc;
  mb1 = mb0;
  if (b1 != nullptr && (rc = encode_map(&mb1, b1, b_rows, p.K, ldb, 128))) return rc;
  mh0 = mb0;
  mh1 = mb1;
  if (p.tail_halves) {  // the half-width units' B boxes: 64 rows
    if ((rc = encode_map(&mh0, b0, b_rows, p.K, ldb, 64))) return rc;
    mh1 = mh0;
    if (b1 != nullptr && (rc = encode_map(&mh1, b1, b_rows, p.K, ldb, 64))) return rc;
  }
  if (p.tail_len > 0 && !scratch.counters_clean) {
    if (cudaMemsetAsync(p.tail_counters, 0, kTailCounterBytes, stream) != cudaSuccess) return FSWIGLU_ERR_CUDA;
  }
  p.wait_limit_ns = g_wait_limit_ns.load(std::memory_order_relaxed);
  p.withhold_one_copy = g_withhold_one_copy.exchange(0, std::memory_order_relaxed);
  gemm_pair_kernel<kMode, kOutF32><<<2 * clusters, kGemmThreads, kPairSmemBytes, stream>>>(ma, mb0, mb1, mh0, mh1, p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? FSWIGLU_OK : FSWIGLU_ERR_CUDA;
}

// 512-row tiles (gemm_quad_sm100.cuh).  They move 0.75 x the operand bytes per flop through the SMs and half
// the bytes through HBM, which under the power cap buys clock; but there is no second accumulator stage (the
// tensor pipe idles while a tile's accumulators are drained), and a wave is 74 tiles of 512 x 256 outputs, so
// a partly filled last wave costs more.  Measured on B200 in 0.3-0.6 s loops (same process, results
// bit-identical), 512-row against 256-row kernel:
//   70B shape   gate-up 5.73 against 5.79-5.83 ms (1344 / 1325 TF/s)   down 2.75 against 2.97 ms (1397 / 1294)
//   7B shape    gate-up 0.571 against 0.511-0.527 ms                   down 0.291 against 0.308-0.311 ms
// Both kernels' times fit  waves x tile cost  with, in units of a 256-row tile's main loop, a 512-row tile
// costing 2 x 0.905 + 18.5 / k-blocks (the drained-accumulator gap is worth about 18 k-blocks) and the
// 256-row kernel's partly filled last wave 0.85 (half-width units) or 1.  The 512-row kernel is taken when
// that arithmetic favours it by more than 1 %.  (At the 7B down shape the model says no although the loops
// above say yes: in short bursts, where power does not set the clock, the coarser wave loses.)
// FSWIGLU_QUAD=0 never, =force always (tests).
int quad_mode() {  // 0 never, 1 automatic, 2 always
  const char* env = std::getenv("FSWIGLU_QUAD");
  if (env == nullptr || env[0] == '\0') return 1;
  if (env[0] == '0') return 0;
  return (env[0] == 'f' || env[0] == 'F') ? 2 : 1;
}
bool use_quad_kernel(const DeviceState& st, const GemmParams& p, int tile_n) {
  const int mode = quad_mode();
  if (mode == 0 || effective_ctas(st) < 2 || pair_mode() == 0) return false;
  if (mode == 2) return true;
  if (pair_mode() == 2) return false;     // the 256-row kernel was asked for by name
  if (p.scatter_world > 0) return false;  // row slabs of a tensor-parallel step: few waves each
  const int64_t clusters = effective_ctas(st) / 2;
  const int64_t n_tiles = (p.n_out + tile_n - 1) / tile_n;
  const int64_t quad = ((p.M + 511) / 512) * n_tiles, pair = ((p.M + 255) / 256) * n_tiles;
  if (pair < clusters) return false;  // below one wave the one-SM kernel takes over
  const double num_kb = static_cast<double>((p.K + kBlockK - 1) / kBlockK);
  const double quad_cost = static_cast<double>((quad + clusters - 1) / clusters) * (2.0 * 0.905 + 18.5 / num_kb);
  const int64_t rem = pair % clusters;
  const double pair_cost = static_cast<double>(pair / clusters) + (rem == 0 ? 0.0 : (2 * rem <= clusters ? 0.85 : 1.0));
  return quad_cost < 0.99 * pair_cost;
}

// Raster for 512-row tiles: the same reasoning as pick_pair_group_m with twice the rows per M-tile.
int pick_quad_group_m(int num_m_tiles, int num_n_tiles, int64_t K, int clusters) {
  const int64_t a_bytes = 512 * K * 2, b_bytes = 256 * K * 2;
  const int64_t resident = 48ll << 20;
  int g;
  if (num_n_tiles * b_bytes <= resident) {
    g = (clusters + num_n_tiles - 1) / num_n_tiles;
  } else if (num_m_tiles * a_bytes <= resident) {
    g = num_m_tiles;
  } else {
    // measured at the 70B shape (gate-up / down TF/s in 0.6 s loops): g = 2 1248 / 1275, 4 1294 / 1358,
    // 8 1318 / 1359, 16 1283 / 1319
    g = 1;
    while ((g + 1) * (g + 1) <= clusters) ++g;  // floor(sqrt(clusters)): 8 for 74 clusters
  }
  return std::max(1, std::min(g, num_m_tiles));
}

// `p` arrives filled for the one-SM kernel; re-plan it for 512-row tiles of full width.
template <int kMode, bool kOutF32>
int launch_gemm_quad(const DeviceState& st, const void* a, int64_t lda, const void* b0, const void* b1, int64_t ldb,
                     int64_t b_rows, GemmParams p, cudaStream_t stream) {
  p.tile_n = (kMode == kPlain) ? 256 : 128;
  p.num_m_tiles = (p.M + 511) / 512;
  p.num_n_tiles = (p.n_out + p.tile_n - 1) / p.tile_n;
  const int tiles = p.num_m_tiles * p.num_n_tiles;
  const int clusters = std::max(1, std::min(tiles, effective_ctas(st) / 2));
  p.group_m = pick_quad_group_m(p.num_m_tiles, p.num_n_tiles, p.K, clusters);
  if (const char* env = std::getenv("FSWIGLU_GROUP_M")) {  // experiments only
    const int v = std::atoi(env);
    if (v >= 1) p.group_m = std::min(v, p.num_m_tiles);
  }
  if (const char* env = std::getenv("FSWIGLU_HINT_A")) p.hint_a = std::atoi(env);  // experiments only
  if (const char* env = std::getenv("FSWIGLU_HINT_B")) p.hint_b = std::atoi(env);
  int rc;
  CUtensorMap ma, mb0, mb1;
  if ((rc = encode_map(&ma, a, p.M, p.K, lda, 128))) return rc;
  if ((rc = encode_map(&mb0, b0, b_rows, p.K, ldb, 128))) return rc;
  mb1 = mb0;
  if (b1 != nullptr && (rc = encode_map(&mb1, b1, b_rows, p.K, ldb, 128))) return rc;
  p.wait_limit_ns = g_wait_limit_ns.load(std::memory_order_relaxed);
  p.withhold_one_copy = g_withhold_one_copy.exchange(0, std::memory_order_relaxed);
  gemm_quad_kernel<kMode, kOutF32><<<2 * clusters, kQuadThreads, kQuadSmemBytes, stream>>>(ma, mb0, mb1, p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? FSWIGLU_OK : FSWIGLU_ERR_CUDA;
}

// Very tall problems are run as row slabs of about 8192 rows, one launch each (rows are independent, results
// are bit-identical).  Measured at K = 8192, F = 28672 in 0.5 s loops: 65536 rows in one launch 1153-1217 TF/s
// (gate-up) / 1114-1128 (down), in slabs of 16384 rows 1295 / 1330, of 8192 rows 1345 / 1375, of 4096 rows
// 1328 / 1321; 32414 rows: 1245-1281 / 1197-1217 in one launch, 1331 / 1364 in slabs of 8192.  The per-wave
// operand sets are the same in all of them; what grows with M is the memory the launch walks over.
// FSWIGLU_TALL_SLAB=<rows> changes the slab height, 0 turns the slabs off (experiments, tests).
int64_t tall_slab_rows(int64_t M) {
  int64_t target = 8192;
  if (const char* env = std::getenv("FSWIGLU_TALL_SLAB")) {
    const long v = std::atol(env);
    if (v == 0) return M;
    if (v >= 512) target = v;
  }
  if (M <= target + target / 2) return M;
  const int64_t n = (M + target - 1) / target;
  return ((M + n - 1) / n + 511) / 512 * 512;  // equal slabs, whole 512-row tiles
}

int gateup_impl(DeviceState& st, const void* x, int64_t ldx, const void* w0, int64_t ldw,
                const void* w_up, void* h, int64_t ldh, int64_t M, int64_t F, int64_t d,
                int interleaved, const float* row_scale, const Scratch& scratch, cudaStream_t stream) {
  int rc;
  if (M == 0) return FSWIGLU_OK;  // empty batch: nothing to read or write, pointers may be null
  if (const int64_t slab = tall_slab_rows(M); slab < M) {
    for (int64_t r0 = 0; r0 < M; r0 += slab) {
      const int64_t rows = std::min(slab, M - r0);
      rc = gateup_impl(st, static_cast<const uint8_t*>(x) + r0 * ldx * 2, ldx, w0, ldw, w_up,
                       static_cast<uint8_t*>(h) + r0 * ldh * 2, ldh, rows, F, d, interleaved,
                       row_scale != nullptr ? row_scale + r0 : nullptr, scratch, stream);
      if (rc != FSWIGLU_OK) return rc;
    }
    return FSWIGLU_OK;
  }
  if ((rc = check_matrix(x, M, d, ldx, true))) return rc;
  if (interleaved) {
    if (w_up != nullptr) return FSWIGLU_ERR_BAD_ARG;
    if ((rc = check_matrix(w0, 2 * F, d, ldw, true))) return rc;
  } else {
    if ((rc = check_matrix(w0, F, d, ldw, true))) return rc;
    if ((rc = check_matrix(w_up, F, d, ldw, true))) return rc;
  }
  if ((rc = check_matrix(h, M, F, ldh, false))) return rc;
  if (row_scale != nullptr && (reinterpret_cast<uintptr_t>(row_scale) & 3u) != 0) return FSWIGLU_ERR_ALIGNMENT;

  GemmParams p = {};
  p.out = h;
  p.ld_out = ldh;
  p.M = static_cast<int>(M);
  p.n_out = static_cast<int>(F);
  p.K = static_cast<int>(d);
  p.vec_ok = (aligned16(h) && ldh % 8 == 0) ? 1 : 0;
  p.status = st.status;
  p.row_scale = row_scale;
  if (use_quad_kernel(st, p, 128)) {
    return interleaved ? launch_gemm_quad<kGatedInterleaved, false>(st, x, ldx, w0, nullptr, ldw, 2 * F, p, stream)
                       : launch_gemm_quad<kGatedSplit, false>(st, x, ldx, w0, w_up, ldw, F, p, stream);
  }
  if (use_pair_kernel(st, M, F, 128)) {
    return interleaved
               ? launch_gemm_pair<kGatedInterleaved, false>(st, x, ldx, w0, nullptr, ldw, 2 * F, p, scratch, stream)
               : launch_gemm_pair<kGatedSplit, false>(st, x, ldx, w0, w_up, ldw, F, p, scratch, stream);
  }
  p.num_m_tiles = static_cast<int>((M + 127) / 128);
  p.tile_n = pick_tile_n(p.num_m_tiles, F, 128, 2, effective_ctas(st));
  p.num_n_tiles = static_cast<int>((F + p.tile_n - 1) / p.tile_n);
  plan_tail_split(&p, effective_ctas(st));
  const int box_cols = p.half_boxes ? p.tile_n / 2 : p.tile_n;  // output columns covered by one B box
  CUtensorMap ma, mb0, mb1;
  if ((rc = encode_map(&ma, x, M, d, ldx, 128))) return rc;
  if (interleaved) {
    if ((rc = encode_map(&mb0, w0, 2 * F, d, ldw, 2 * box_cols))) return rc;
    mb1 = mb0;
  } else {
    if ((rc = encode_map(&mb0, w0, F, d, ldw, box_cols))) return rc;
    if ((rc = encode_map(&mb1, w_up, F, d, ldw, box_cols))) return rc;
  }
  p.group_m = pick_group_m(p.num_m_tiles, d);
  return interleaved ? launch_gemm<kGatedInterleaved, false>(st, ma, mb0, mb1, p, stream)
                     : launch_gemm<kGatedSplit, false>(st, ma, mb0, mb1, p, stream);
}

// The optional residual [M, d] (bf16) is read with 16-byte loads: aligned base, pitch and width.
int check_residual(const void* residual, int64_t ldr, int64_t d) {
  if (residual == nullptr) return FSWIGLU_OK;
  if (ldr < d || d % 8 != 0) return FSWIGLU_ERR_SHAPE;
  if (!aligned16(residual) || ldr % 8 != 0) return FSWIGLU_ERR_ALIGNMENT;
  return FSWIGLU_OK;
}

int down_impl(DeviceState& st, const void* h, int64_t ldh, const void* w_down, int64_t ldw, void* out,
              int64_t ldo, int64_t M, int64_t d, int64_t F, int out_dtype, const void* residual, int64_t ldr,
              const Scratch& scratch, cudaStream_t stream) {
  int rc;
  if (out_dtype != FSWIGLU_OUT_BF16 && out_dtype != FSWIGLU_OUT_F32) return FSWIGLU_ERR_BAD_ARG;
  if (M == 0) return FSWIGLU_OK;
  if (const int64_t slab = tall_slab_rows(M); slab < M) {  // very tall: row slabs, one launch each
    const int64_t out_bytes = out_dtype == FSWIGLU_OUT_F32 ? 4 : 2;
    for (int64_t r0 = 0; r0 < M; r0 += slab) {
      const int64_t rows = std::min(slab, M - r0);
      rc = down_impl(st, static_cast<const uint8_t*>(h) + r0 * ldh * 2, ldh, w_down, ldw,
                     static_cast<uint8_t*>(out) + r0 * ldo * out_bytes, ldo, rows, d, F, out_dtype,
                     residual != nullptr ? static_cast<const uint8_t*>(residual) + r0 * ldr * 2 : nullptr, ldr,
                     scratch, stream);
      if (rc != FSWIGLU_OK) return rc;
    }
    return FSWIGLU_OK;
  }
  if ((rc = check_matrix(h, M, F, ldh, true))) return rc;
  if ((rc = check_matrix(w_down, d, F, ldw, true))) return rc;
  if ((rc = check_matrix(out, M, d, ldo, false))) return rc;
  if ((rc = check_residual(residual, ldr, d))) return rc;

  GemmParams p = {};
  p.out = out;
  p.ld_out = ldo;
  p.M = static_cast<int>(M);
  p.n_out = static_cast<int>(d);
  p.K = static_cast<int>(F);
  const bool f32 = out_dtype == FSWIGLU_OUT_F32;
  p.vec_ok = (aligned16(out) && ldo % (f32 ? 4 : 8) == 0) ? 1 : 0;
  p.status = st.status;
  p.residual = residual;
  p.ld_res = ldr;
  if (use_quad_kernel(st, p, 256)) {
    return f32 ? launch_gemm_quad<kPlain, true>(st, h, ldh, w_down, nullptr, ldw, d, p, stream)
               : launch_gemm_quad<kPlain, false>(st, h, ldh, w_down, nullptr, ldw, d, p, stream);
  }
  if (use_pair_kernel(st, M, d, 256)) {
    return f32 ? launch_gemm_pair<kPlain, true>(st, h, ldh, w_down, nullptr, ldw, d, p, scratch, stream)
               : launch_gemm_pair<kPlain, false>(st, h, ldh, w_down, nullptr, ldw, d, p, scratch, stream);
  }
  p.num_m_tiles = static_cast<int>((M + 127) / 128);
  p.tile_n = pick_tile_n(p.num_m_tiles, d, 256, 1, effective_ctas(st));
  p.num_n_tiles = static_cast<int>((d + p.tile_n - 1) / p.tile_n);
  plan_tail_split(&p, effective_ctas(st));
  CUtensorMap ma, mb;
  if ((rc = encode_map(&ma, h, M, F, ldh, 128))) return rc;
  if ((rc = encode_map(&mb, w_down, d, F, ldw, p.half_boxes ? p.tile_n / 2 : p.tile_n))) return rc;
  p.group_m = pick_group_m(p.num_m_tiles, F);
  return f32 ? launch_gemm<kPlain, true>(st, ma, mb, mb, p, stream)
             : launch_gemm<kPlain, false>(st, ma, mb, mb, p, stream);
}

size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Small-batch MLP: one cooperative weight-streaming launch (gate-up, hand-over, down), nothing else on
// the stream.  `h` receives the bf16 hidden activations, `scratch` holds the tagged flags and the fp32
// partial tiles (decode_workspace_bytes); nothing in it has to be initialised.
struct Fusions {
  const float* row_scale = nullptr;  // [M] fp32, applied to gate and up before SiLU
  const void* residual = nullptr;    // bf16 [M, d], added to the output in fp32
  int64_t ld_res = 0;
};

// Per-launch tag of the small-batch kernel's flags: non-zero, never repeated within a process (2^32 launches),
// starting from a value that differs between processes.
uint32_t next_decode_tag() {
  static std::atomic<uint32_t> tag{static_cast<uint32_t>(
      std::chrono::steady_clock::now().time_since_epoch().count() * 2654435761ull >> 7)};
  uint32_t t = tag.fetch_add(1, std::memory_order_relaxed) + 1;
  if (t == 0) t = tag.fetch_add(1, std::memory_order_relaxed) + 1;
  return t;
}

int decode_prefetch_units() {
  if (const char* env = std::getenv("FSWIGLU_DECODE_PREFETCH")) {
    const int v = std::atoi(env);
    if (v >= 0 && v <= 4096) return v;
  }
  // Off by default.  Measured with per-CTA stamps at M = 16: a window of 24 tiles shortens phase 2 by
  // 3.5 us (its loads hit the L2) but the prefetches compete with the slowest CTAs' last phase-1 loads and
  // delay the hand-over by 5 us; a net loss until phase 1 ends more evenly.
  return 0;
}

int decode_impl(DeviceState& st, const void* x, int64_t ldx, const void* w_gate, const void* w_up, int64_t ldw_gu,
                const void* w_down, int64_t ldw_d, void* out, int64_t ldo, int out_dtype, int64_t M, int64_t d,
                int64_t F, const Fusions& fu, void* h, void* scratch, cudaStream_t stream) {
  int rc;
  if (out_dtype != FSWIGLU_OUT_BF16 && out_dtype != FSWIGLU_OUT_F32) return FSWIGLU_ERR_BAD_ARG;
  if ((rc = check_matrix(x, M, d, ldx, true))) return rc;
  if ((rc = check_matrix(w_gate, F, d, ldw_gu, true))) return rc;
  if ((rc = check_matrix(w_up, F, d, ldw_gu, true))) return rc;
  if ((rc = check_matrix(w_down, d, F, ldw_d, true))) return rc;
  if ((rc = check_matrix(out, M, d, ldo, false))) return rc;
  if ((rc = check_residual(fu.residual, fu.ld_res, d))) return rc;

  const int n_pad = decode_pad_tokens(M);
  const int rb2 = static_cast<int>((d + 127) / 128), kb2 = static_cast<int>((F + 63) / 64);
  uint8_t* ws = static_cast<uint8_t*>(scratch);
  unsigned int* flags = reinterpret_cast<unsigned int*>(ws);  // per-CTA phase-1 flags, then the segment flags

  DecodeParams p;
  int used1 = 0;
  decode_plan_rows(F, st.num_sms, &p.tile_rows, &p.tiles_per_cta, &used1);
  p.h = h;
  p.F = static_cast<int>(F);
  p.k_blocks1 = static_cast<int>((d + 63) / 64);
  p.out = out;
  p.ld_out = ldo;
  p.d = static_cast<int>(d);
  p.row_blocks2 = rb2;
  p.k_blocks2 = kb2;
  p.out_f32 = out_dtype == FSWIGLU_OUT_F32 ? 1 : 0;
  p.partials = reinterpret_cast<float*>(ws + decode_counter_bytes(d));
  p.phase1_flags = flags;
  p.seg_flags = flags + kDecMaxGrid + 1;
  p.tag = next_decode_tag();
  p.M = static_cast<int>(M);
  p.n_pad = n_pad;
  p.prefetch_units = decode_prefetch_units();
  // All eleven weight slots: giving two of them to the token-tile ring at M = 64 (8 instead of 4 token
  // slots) was slower (phase 1 median 37.6 us against 36.6 us, phase 2 six microseconds longer).
  p.w_slots = kDecWSlots;
  // CTA c starts phase 1 at k-block 7c mod k_blocks1.  With every CTA on the same columns at the same moment
  // the slowest CTA finished phase 1 at 42.5 us (median 36.4); staggered by 7: 37.4 us (median 34.3) - the
  // reads then spread over the memory channels instead of marching through them in step.
  p.k_rotate = 7;
  if (const char* env = std::getenv("FSWIGLU_DECODE_KROT")) {  // experiments only
    const int v = std::atoi(env);
    if (v >= 0 && v < 4096) p.k_rotate = v;
  }
  // Row-block owners sum the other k-ranges' partial tiles from shared memory (bulk copies into the idle
  // rings).  Measured at the 8B shape: M = 64 94.9 -> 87.3 us, M <= 16 78.8 -> 78.1 us.
  p.reduce_via_smem = 1;
  if (const char* env = std::getenv("FSWIGLU_DECODE_SMEMRED")) {  // experiments and tests: 0 = sum from the workspace
    if (std::atoi(env) == 0) p.reduce_via_smem = 0;
  }
  if (const char* env = std::getenv("FSWIGLU_DECODE_WSLOTS")) {  // experiments only
    const int v = std::atoi(env);
    if (v >= 4 && v <= kDecWSlots) p.w_slots = v;
  }
  p.trace = g_decode_trace.load(std::memory_order_relaxed);
  p.row_scale = fu.row_scale;
  p.residual = fu.residual;
  p.ld_res = fu.ld_res;
  p.status = st.status;
  p.wait_limit_ns = g_wait_limit_ns.load(std::memory_order_relaxed);

  CUtensorMap m_gate, m_up, m_x, m_down, m_h;
  if ((rc = encode_map(&m_gate, w_gate, F, d, ldw_gu, p.tile_rows))) return rc;
  if ((rc = encode_map(&m_up, w_up, F, d, ldw_gu, p.tile_rows))) return rc;
  if ((rc = encode_map(&m_x, x, M, d, ldx, n_pad))) return rc;
  if ((rc = encode_map(&m_down, w_down, d, F, ldw_d, 128))) return rc;
  if ((rc = encode_map(&m_h, h, M, F, F, n_pad))) return rc;
  // every CTA takes part in both phases: the grid must not exceed what phase 2 can split into
  const int grid = std::max(1, std::min(std::min(st.num_sms, kDecMaxGrid), decode_grid_limit(rb2, kb2, st.num_sms)));
  if (grid < used1) decode_plan_rows(F, grid, &p.tile_rows, &p.tiles_per_cta, &used1);
  if (grid < st.num_sms) {
    if ((rc = encode_map(&m_gate, w_gate, F, d, ldw_gu, p.tile_rows))) return rc;
    if ((rc = encode_map(&m_up, w_up, F, d, ldw_gu, p.tile_rows))) return rc;
  }
  p.rows_per_cta = p.tile_rows * p.tiles_per_cta;
  p.handover_target = static_cast<unsigned int>(grid) +
                      static_cast<unsigned int>(g_withhold_one_copy.exchange(0, std::memory_order_relaxed) != 0 ? 1 : 0);
  // Cooperative launch: the phase hand-over needs every CTA resident at the same time.
  void* args[] = {&m_gate, &m_up, &m_down, &m_x, &m_h, &p};
  const cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(decode_fused_kernel), dim3(grid),
                                                    dim3(kDecThreads), args, kDecSmemBytes, stream);
  if (e == cudaErrorCooperativeLaunchTooLarge) {
    // Not every CTA can be resident right now (SMs held by someone else): the hand-over inside the
    // kernel would not be safe, so the launch was refused.  The tiled kernels need no co-residency.
    (void)cudaGetLastError();
    if ((rc = gateup_impl(st, x, ldx, w_gate, ldw_gu, w_up, h, F, M, F, d, 0, fu.row_scale, Scratch{}, stream)))
      return rc;
    return down_impl(st, h, F, w_down, ldw_d, out, ldo, M, d, F, out_dtype, fu.residual, fu.ld_res, Scratch{},
                     stream);
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return e == cudaSuccess ? FSWIGLU_OK : FSWIGLU_ERR_CUDA;
}

// Workspace of the whole-MLP call: [h: M x F bf16][small-batch counters + partial tiles, M <= 64]
// [scratch of the split last wave, M > 128], every part 256-byte aligned.
size_t mlp_h_bytes(int64_t M, int64_t F) { return round_up(static_cast<size_t>(M) * static_cast<size_t>(F) * 2u, 256); }

int mlp_impl(DeviceState& st, const void* x, int64_t ldx, const void* w_gate, const void* w_up, int64_t ldw_gu,
             const void* w_down, int64_t ldw_d, void* out, int64_t ldo, int out_dtype, int64_t M, int64_t d,
             int64_t F, const Fusions& fu, void* workspace, size_t workspace_bytes, cudaStream_t s) {
  if (workspace == nullptr || workspace_bytes < fswiglu_workspace_bytes(M, d, F) ||
      (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) {
    return FSWIGLU_ERR_WORKSPACE;
  }
  void* h = workspace;
  uint8_t* after_h = static_cast<uint8_t*>(workspace) + mlp_h_bytes(M, F);
  if (M <= kDecodeMaxTokens && decode_supported(M, d, F, ldx, ldw_gu, ldw_d) &&
      std::getenv("FSWIGLU_NO_DECODE_PATH") == nullptr) {
    return decode_impl(st, x, ldx, w_gate, w_up, ldw_gu, w_down, ldw_d, out, ldo, out_dtype, M, d, F, fu, h, after_h,
                       s);
  }
  Scratch scratch;
  if (M > 128) {
    scratch.ptr = after_h + (M <= kDecodeMaxTokens ? decode_workspace_bytes(M, d, F) : 0);
    scratch.bytes = kTailScratchBytes;
    // one memset serves both launches: each leaves the counters it used at zero
    if (cudaMemsetAsync(scratch.ptr, 0, kTailCounterBytes, s) != cudaSuccess) return FSWIGLU_ERR_CUDA;
    scratch.counters_clean = true;
  }
  if (int rc = gateup_impl(st, x, ldx, w_gate, ldw_gu, w_up, h, F, M, F, d, 0, fu.row_scale, scratch, s)) return rc;
  return down_impl(st, h, F, w_down, ldw_d, out, ldo, M, d, F, out_dtype, fu.residual, fu.ld_res, scratch, s);
}

}  // namespace

extern "C" {

int fswiglu_gateup_bf16(const void* x, int64_t ldx, const void* w_gate_or_w13, int64_t ldw,
                        const void* w_up, void* h, int64_t ldh, int64_t M, int64_t F, int64_t d,
                        int interleaved, void* stream) {
  return fswiglu_gateup_bf16_ex(x, ldx, w_gate_or_w13, ldw, w_up, h, ldh, M, F, d, interleaved, nullptr, nullptr, 0,
                                stream);
}

int fswiglu_gateup_bf16_ex(const void* x, int64_t ldx, const void* w_gate_or_w13, int64_t ldw, const void* w_up,
                           void* h, int64_t ldh, int64_t M, int64_t F, int64_t d, int interleaved,
                           const float* row_scale, void* scratch, size_t scratch_bytes, void* stream) {
  if (M < 0 || F <= 0 || d <= 0) return FSWIGLU_ERR_BAD_ARG;
  DeviceState* st = nullptr;
  if (int rc = device_state(&st)) return rc;
  Scratch sc;
  if (scratch != nullptr && (reinterpret_cast<uintptr_t>(scratch) & 255u) != 0) return FSWIGLU_ERR_WORKSPACE;
  sc.ptr = scratch;
  sc.bytes = scratch_bytes;
  return gateup_impl(*st, x, ldx, w_gate_or_w13, ldw, w_up, h, ldh, M, F, d, interleaved, row_scale, sc,
                     static_cast<cudaStream_t>(stream));
}

int fswiglu_down_bf16(const void* h, int64_t ldh, const void* w_down, int64_t ldw, void* out,
                      int64_t ldo, int64_t M, int64_t d, int64_t F, int out_dtype, void* stream) {
  return fswiglu_down_bf16_ex(h, ldh, w_down, ldw, out, ldo, M, d, F, out_dtype, nullptr, 0, nullptr, 0, stream);
}

int fswiglu_down_bf16_ex(const void* h, int64_t ldh, const void* w_down, int64_t ldw, void* out, int64_t ldo,
                         int64_t M, int64_t d, int64_t F, int out_dtype, const void* residual, int64_t ldr,
                         void* scratch, size_t scratch_bytes, void* stream) {
  if (M < 0 || F <= 0 || d <= 0) return FSWIGLU_ERR_BAD_ARG;
  DeviceState* st = nullptr;
  if (int rc = device_state(&st)) return rc;
  Scratch sc;
  if (scratch != nullptr && (reinterpret_cast<uintptr_t>(scratch) & 255u) != 0) return FSWIGLU_ERR_WORKSPACE;
  sc.ptr = scratch;
  sc.bytes = scratch_bytes;
  return down_impl(*st, h, ldh, w_down, ldw, out, ldo, M, d, F, out_dtype, residual, ldr, sc,
                   static_cast<cudaStream_t>(stream));
}

size_t fswiglu_gemm_scratch_bytes(void) { return kTailScratchBytes; }

size_t fswiglu_workspace_bytes(int64_t M, int64_t d, int64_t F) {
  if (M <= 0 || d <= 0 || F <= 0) return 0;
  size_t bytes = mlp_h_bytes(M, F);
  if (M <= kDecodeMaxTokens) bytes += decode_workspace_bytes(M, d, F);
  if (M > 128) bytes += kTailScratchBytes;
  return bytes;
}

int fswiglu_mlp_bf16(const void* x, int64_t ldx, const void* w_gate, const void* w_up, int64_t ldw_gu,
                     const void* w_down, int64_t ldw_d, void* out, int64_t ldo, int out_dtype,
                     int64_t M, int64_t d, int64_t F, void* workspace, size_t workspace_bytes,
                     void* stream) {
  return fswiglu_mlp_bf16_ex(x, ldx, nullptr, w_gate, w_up, ldw_gu, w_down, ldw_d, nullptr, 0, out, ldo, out_dtype, M,
                             d, F, workspace, workspace_bytes, stream);
}

int fswiglu_mlp_bf16_ex(const void* x, int64_t ldx, const float* row_scale, const void* w_gate, const void* w_up,
                        int64_t ldw_gu, const void* w_down, int64_t ldw_d, const void* residual, int64_t ldr,
                        void* out, int64_t ldo, int out_dtype, int64_t M, int64_t d, int64_t F, void* workspace,
                        size_t workspace_bytes, void* stream) {
  if (M < 0 || F <= 0 || d <= 0) return FSWIGLU_ERR_BAD_ARG;
  if (M == 0) return FSWIGLU_OK;
  DeviceState* st = nullptr;
  if (int rc = device_state(&st)) return rc;
  Fusions fu;
  fu.row_scale = row_scale;
  fu.residual = residual;
  fu.ld_res = ldr;
  return mlp_impl(*st, x, ldx, w_gate, w_up, ldw_gu, w_down, ldw_d, out, ldo, out_dtype, M, d, F, fu, workspace,
                  workspace_bytes, static_cast<cudaStream_t>(stream));
}

int fswiglu_rms_scale_f32(const void* x, int64_t ldx, int64_t M, int64_t d, float eps, float* scale, void* stream) {
  if (M < 0 || d <= 0 || !(eps >= 0.0f)) return FSWIGLU_ERR_BAD_ARG;
  if (M == 0) return FSWIGLU_OK;
  if (int rc = check_matrix(x, M, d, ldx, true)) return rc;
  if (scale == nullptr) return FSWIGLU_ERR_BAD_ARG;
  DeviceState* st = nullptr;
  if (int rc = device_state(&st)) return rc;
  const long long blocks = std::min<long long>((M + 7) / 8, static_cast<long long>(st->num_sms) * 8);
  rms_scale_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), ldx, static_cast<int>(M), static_cast<int>(d), eps, scale);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? FSWIGLU_OK : FSWIGLU_ERR_CUDA;
}

namespace {

// Workspace of one slab's MLP call: slabs of different heights may take different paths (a last slab of
// <= 64 rows takes the small-batch kernel with its own partial tiles), so the largest request counts.
size_t host_slab_workspace_bytes(int64_t M, int64_t d, int64_t F) {
  int64_t first[kMaxHostSlabs + 2], rows[kMaxHostSlabs + 2];
  const int n = host_slab_plan(M, first, rows);
  size_t bytes = 0;
  for (int i = 0; i < n; ++i) bytes = std::max(bytes, fswiglu_workspace_bytes(rows[i], d, F));
  return round_up(bytes, 256);
}

int host_state(DeviceState& st) {
  std::lock_guard<std::mutex> lock(g_mutex);
  if (st.host_ready) return FSWIGLU_OK;
  if (cudaStreamCreateWithFlags(&st.h2d_stream, cudaStreamNonBlocking) != cudaSuccess ||
      cudaStreamCreateWithFlags(&st.d2h_stream, cudaStreamNonBlocking) != cudaSuccess ||
      cudaEventCreateWithFlags(&st.ev_start, cudaEventDisableTiming) != cudaSuccess) {
    return FSWIGLU_ERR_CUDA;
  }
  for (int i = 0; i < kMaxHostSlabs; ++i) {
    if (cudaEventCreateWithFlags(&st.ev_h2d[i], cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&st.ev_done[i], cudaEventDisableTiming) != cudaSuccess) {
      return FSWIGLU_ERR_CUDA;
    }
  }
  st.host_ready = true;
  return FSWIGLU_OK;
}

}  // namespace

size_t fswiglu_host_workspace_bytes(int64_t M, int64_t d, int64_t F) {
  if (M <= 0 || d <= 0 || F <= 0) return 0;
  const size_t act = round_up(static_cast<size_t>(M) * static_cast<size_t>(d) * 2u, 256);
  return 2 * act + host_slab_workspace_bytes(M, d, F);
}

int fswiglu_mlp_bf16_host(const void* x_host, const void* w_gate, const void* w_up,
                          const void* w_down, void* out_host, int64_t M, int64_t d, int64_t F,
                          void* workspace, size_t workspace_bytes, void* stream) {
  if (M < 0 || F <= 0 || d <= 0) return FSWIGLU_ERR_BAD_ARG;
  if (M == 0) return FSWIGLU_OK;
  if (x_host == nullptr || out_host == nullptr) return FSWIGLU_ERR_BAD_ARG;
  DeviceState* st = nullptr;
  if (int rc = device_state(&st)) return rc;
  if (int rc = host_state(*st)) return rc;
  if (workspace == nullptr || workspace_bytes < fswiglu_host_workspace_bytes(M, d, F) ||
      (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) {
    return FSWIGLU_ERR_WORKSPACE;
  }
  // The internal copy streams and events belong to the device: one host-buffer call per device at a time.
  std::lock_guard<std::mutex> lock(st->host_mutex);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t act = round_up(static_cast<size_t>(M) * static_cast<size_t>(d) * 2u, 256);
  uint8_t* x_dev = static_cast<uint8_t*>(workspace);
  uint8_t* out_dev = x_dev + act;
  uint8_t* mlp_ws = out_dev + act;
  const size_t mlp_ws_bytes = host_slab_workspace_bytes(M, d, F);
  int64_t slab_first[kMaxHostSlabs + 2], slab_rows[kMaxHostSlabs + 2];
  const int num_slabs = host_slab_plan(M, slab_first, slab_rows);
  const size_t row_bytes = static_cast<size_t>(d) * 2u;

  bool ok = cudaEventRecord(st->ev_start, s) == cudaSuccess &&
            cudaStreamWaitEvent(st->h2d_stream, st->ev_start, 0) == cudaSuccess &&
            cudaStreamWaitEvent(st->d2h_stream, st->ev_start, 0) == cudaSuccess;
  for (int i = 0; i < num_slabs && ok; ++i) {
    const int64_t r0 = slab_first[i], rows = slab_rows[i];
    ok = cudaMemcpyAsync(x_dev + r0 * row_bytes, static_cast<const uint8_t*>(x_host) + r0 * row_bytes,
                         rows * row_bytes, cudaMemcpyHostToDevice, st->h2d_stream) == cudaSuccess &&
         cudaEventRecord(st->ev_h2d[i], st->h2d_stream) == cudaSuccess;
  }
  int rc = FSWIGLU_OK;
  for (int i = 0; i < num_slabs && ok && rc == FSWIGLU_OK; ++i) {
    const int64_t r0 = slab_first[i], rows = slab_rows[i];
    ok = cudaStreamWaitEvent(s, st->ev_h2d[i], 0) == cudaSuccess;
    if (!ok) break;
    rc = fswiglu_mlp_bf16(x_dev + r0 * row_bytes, d, w_gate, w_up, d, w_down, F, out_dev + r0 * row_bytes,
                          d, FSWIGLU_OUT_BF16, rows, d, F, mlp_ws, mlp_ws_bytes, s);
    if (rc != FSWIGLU_OK) break;
    ok = cudaEventRecord(st->ev_done[i], s) == cudaSuccess &&
         cudaStreamWaitEvent(st->d2h_stream, st->ev_done[i], 0) == cudaSuccess &&
         cudaMemcpyAsync(static_cast<uint8_t*>(out_host) + r0 * row_bytes, out_dev + r0 * row_bytes,
                         rows * row_bytes, cudaMemcpyDeviceToHost, st->d2h_stream) == cudaSuccess;
  }
  // Always drain what was queued, also on the error paths: the caller owns the host buffers.
  const bool drained = cudaStreamSynchronize(st->h2d_stream) == cudaSuccess &&
                       cudaStreamSynchronize(s) == cudaSuccess &&
                       cudaStreamSynchronize(st->d2h_stream) == cudaSuccess;
  if (rc != FSWIGLU_OK) return rc;
  return (ok && drained) ? FSWIGLU_OK : FSWIGLU_ERR_CUDA;
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of the whole-MLP call (see include/fswiglu.h for who needs it).
// The hidden activations go into this fixed array instead of a caller workspace.  In host code
// the name `g_static_scratch` is only a handle for the runtime, not a device address: the address
// the kernels need is looked up once per device with cudaGetSymbolAddress and cached.
// Layout: [0, 256) error word of the bounded device-side waits (zero at load time),
//         [256, 256 + FSWIGLU_STATIC_SCRATCH_BYTES) hidden activations h, row pitch F.
// ---------------------------------------------------------------------------------------------
namespace {

constexpr size_t kStaticHeaderBytes = 256;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticHeaderBytes + FSWIGLU_STATIC_SCRATCH_BYTES];

struct StaticState {
  bool ready = false;
  DeviceState dev;          // num_sms + status pointer (into the static array), no owned memory
  unsigned char* base = nullptr;
};
StaticState g_static[kMaxDevices];

// Once per device, with that device current: capability check, address of the array, shared-memory
// opt-in of the kernels.  Nothing here allocates device memory.
int static_state(StaticState** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return FSWIGLU_ERR_NO_DEVICE;
  if (dev < 0 || dev >= kMaxDevices) return FSWIGLU_ERR_NO_DEVICE;
  std::lock_guard<std::mutex> lock(g_mutex);
  StaticState& st = g_static[dev];
  if (!st.ready) {
    int num_sms = 0;
    if (int rc = prepare_device(dev, &num_sms)) return rc;
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || ptr == nullptr) return FSWIGLU_ERR_CUDA;
    st.base = static_cast<unsigned char*>(ptr);
    st.dev.num_sms = num_sms;
    st.dev.status = reinterpret_cast<uint32_t*>(st.base);
    st.dev.ready = true;
    st.ready = true;
  }
  *out = &st;
  return FSWIGLU_OK;
}

// Copy a watchdog word to the host and clear it if it was set.  No allocation.
int read_and_clear_status(uint32_t* device_word, uint32_t* out, cudaStream_t s) {
  uint32_t word = 0;
  if (cudaMemcpyAsync(&word, device_word, sizeof(word), cudaMemcpyDeviceToHost, s) != cudaSuccess)
    return FSWIGLU_ERR_CUDA;
  if (cudaStreamSynchronize(s) != cudaSuccess) return FSWIGLU_ERR_CUDA;
  if (word != 0) {
    if (cudaMemsetAsync(device_word, 0, sizeof(word), s) != cudaSuccess) return FSWIGLU_ERR_CUDA;
    if (cudaStreamSynchronize(s) != cudaSuccess) return FSWIGLU_ERR_CUDA;
  }
  *out = word;
  return FSWIGLU_OK;
}

}  // namespace

int fswiglu_mlp_bf16_static(const void* x, int64_t ldx, const void* w_gate, const void* w_up,
                            int64_t ldw_gu, const void* w_down, int64_t ldw_d, void* out, int64_t ldo,
                            int out_dtype, int64_t M, int64_t d, int64_t F, void* stream) {
  if (M < 0 || F <= 0 || d <= 0) return FSWIGLU_ERR_BAD_ARG;
  if (M == 0) return FSWIGLU_OK;
  // reject before touching the device: the hidden activations must fit the built-in array
  if (static_cast<uint64_t>(M) > FSWIGLU_STATIC_SCRATCH_BYTES / 2u / static_cast<uint64_t>(F)) {
    return FSWIGLU_ERR_TOO_LARGE;
  }
  StaticState* st = nullptr;
  if (int rc = static_state(&st)) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  void* h = st->base + kStaticHeaderBytes;
  if (int rc = gateup_impl(st->dev, x, ldx, w_gate, ldw_gu, w_up, h, F, M, F, d, 0, nullptr, Scratch{}, s)) return rc;
  return down_impl(st->dev, h, F, w_down, ldw_d, out, ldo, M, d, F, out_dtype, nullptr, 0, Scratch{}, s);
}

int fswiglu_static_status(uint32_t* status, void* stream) {
  StaticState* st = nullptr;
  if (int rc = static_state(&st)) return rc;
  uint32_t word = 0;
  if (int rc = read_and_clear_status(st->dev.status, &word, static_cast<cudaStream_t>(stream))) return rc;
  if (status != nullptr) *status = word;
  return word == 0 ? FSWIGLU_OK : FSWIGLU_ERR_WATCHDOG;
}

// ---------------------------------------------------------------------------------------------
// Backward pass: seven K-major tensor-core GEMMs (the plain mode of the forward kernels) plus two
// bandwidth-bound kernels that produce their operands (elementwise_sm100.cuh).
// ---------------------------------------------------------------------------------------------
int fswiglu_gemm_tn_bf16(const void* a, int64_t lda, const void* b, int64_t ldb, void* c, int64_t ldc, int64_t M,
                         int64_t N, int64_t K, int out_dtype, void* scratch, size_t scratch_bytes, void* stream) {
  // C [M, N] = A [M, K] B [N, K]^T: exactly the down projection with (h, W_down, out, d, F) = (A, B, C, N, K)
  return fswiglu_down_bf16_ex(a, lda, b, ldb, c, ldc, M, N, K, out_dtype, nullptr, 0, scratch, scratch_bytes, stream);
}

namespace {

int ew_grid(const DeviceState& st, int64_t tiles) {
  const int64_t cap = static_cast<int64_t>(st.num_sms) * 8;
  return static_cast<int>(std::max<int64_t>(1, std::min(tiles, cap)));
}

int transpose_impl(DeviceState& st, const void* src, int64_t ld_src, void* dst, int64_t ld_dst, int64_t rows,
                   int64_t cols, cudaStream_t s) {
  if (rows == 0 || cols == 0) return FSWIGLU_OK;
  const int64_t dst_cols = (rows + 7) / 8 * 8;
  if (src == nullptr || dst == nullptr) return FSWIGLU_ERR_BAD_ARG;
  if (rows > 0x7fffffffll || cols > 0x7fffffffll) return FSWIGLU_ERR_SHAPE;
  if (cols % 8 != 0 || ld_src < cols || ld_dst < dst_cols) return FSWIGLU_ERR_SHAPE;
  if (!aligned16(src) || !aligned16(dst) || ld_src % 8 != 0 || ld_dst % 8 != 0) return FSWIGLU_ERR_ALIGNMENT;
  const int64_t tiles = ((dst_cols + kEwTile - 1) / kEwTile) * ((cols + kEwTile - 1) / kEwTile);
  transpose_bf16_kernel<<<ew_grid(st, tiles), kEwThreads, 0, s>>>(
      static_cast<const __nv_bfloat16*>(src), ld_src, static_cast<__nv_bfloat16*>(dst), ld_dst, static_cast<int>(rows),
      static_cast<int>(cols), static_cast<int>(dst_cols));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? FSWIGLU_OK : FSWIGLU_ERR_CUDA;
}

struct BackwardLayout {
  size_t g, u, dh, dgdu, dgT, duT, hT, doutT, xT, wdT, wguT, scratch, total;
  int64_t Mp;
};

BackwardLayout backward_layout(int64_t M, int64_t d, int64_t F) {
  BackwardLayout L = {};
  L.Mp = (M + 7) / 8 * 8;
  size_t off = 0;
  auto take = [&](size_t elems) {
    const size_t at = off;
    off += round_up(elems * 2u, 256);
    return at;
  };
  const size_t MF = static_cast<size_t>(M) * F, FMp = static_cast<size_t>(F) * L.Mp, dMp = static_cast<size_t>(d) * L.Mp;
  L.g = take(MF);
  L.u = take(MF);
  L.dh = take(MF);
  L.dgdu = take(2 * MF);
  L.dgT = take(FMp);
  L.duT = take(FMp);
  L.hT = take(FMp);
  L.doutT = take(dMp);
  L.xT = take(dMp);
  L.wdT = take(static_cast<size_t>(F) * d);
  L.wguT = take(2 * static_cast<size_t>(d) * F);
  L.scratch = off;
  off += kTailScratchBytes;
  L.total = off;
  return L;
}

}  // namespace

int fswiglu_transpose_bf16(const void* src, int64_t ld_src, void* dst, int64_t ld_dst, int64_t rows, int64_t cols,
                           void* stream) {
  if (rows < 0 || cols < 0) return FSWIGLU_ERR_BAD_ARG;
  DeviceState* st = nullptr;
  if (int rc = device_state(&st)) return rc;
  return transpose_impl(*st, src, ld_src, dst, ld_dst, rows, cols, static_cast<cudaStream_t>(stream));
}

size_t fswiglu_backward_workspace_bytes(int64_t M, int64_t d, int64_t F) {
  if (M <= 0 || d <= 0 || F <= 0) return 0;
  return backward_layout(M, d, F).total;
}

int fswiglu_mlp_backward_bf16(const void* x, int64_t ldx, const void* w_gate, const void* w_up, int64_t ldw_gu,
                              const void* w_down, int64_t ldw_d, const void* dout, int64_t ld_dout, void* dx,
                              int64_t ld_dx, void* d_w_gate, void* d_w_up, int64_t ld_dw_gu, void* d_w_down,
                              int64_t ld_dw_d, int grad_dtype, int64_t M, int64_t d, int64_t F, void* workspace,
                              size_t workspace_bytes, void* stream) {
  if (M < 0 || F <= 0 || d <= 0) return FSWIGLU_ERR_BAD_ARG;
  if (grad_dtype != FSWIGLU_OUT_BF16 && grad_dtype != FSWIGLU_OUT_F32) return FSWIGLU_ERR_BAD_ARG;
  if (M == 0) return FSWIGLU_OK;  // no tokens: the caller's weight gradients are zero, nothing is written
  if (d % 8 != 0 || F % 8 != 0) return FSWIGLU_ERR_SHAPE;
  DeviceState* st = nullptr;
  if (int rc = device_state(&st)) return rc;
  const BackwardLayout L = backward_layout(M, d, F);
  if (workspace == nullptr || workspace_bytes < L.total || (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0)
    return FSWIGLU_ERR_WORKSPACE;
  int rc;
  if ((rc = check_matrix(x, M, d, ldx, true))) return rc;
  if ((rc = check_matrix(dout, M, d, ld_dout, true))) return rc;
  if ((rc = check_matrix(w_gate, F, d, ldw_gu, true))) return rc;
  if ((rc = check_matrix(w_up, F, d, ldw_gu, true))) return rc;
  if ((rc = check_matrix(w_down, d, F, ldw_d, true))) return rc;
  if (dx == nullptr || d_w_gate == nullptr || d_w_up == nullptr || d_w_down == nullptr) return FSWIGLU_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  auto at = [&](size_t off) { return static_cast<void*>(ws + off); };
  void* scratch = at(L.scratch);
  const size_t sb = kTailScratchBytes;
  const int bf = FSWIGLU_OUT_BF16;
  // 1. recompute the pre-activations (the forward keeps only x): g = x Wg^T, u = x Wu^T
  if ((rc = fswiglu_gemm_tn_bf16(x, ldx, w_gate, ldw_gu, at(L.g), F, M, F, d, bf, scratch, sb, stream))) return rc;
  if ((rc = fswiglu_gemm_tn_bf16(x, ldx, w_up, ldw_gu, at(L.u), F, M, F, d, bf, scratch, sb, stream))) return rc;
  // 2. dh = dout Wd  (B operand K-major: Wd^T [F, d])
  if ((rc = transpose_impl(*st, w_down, ldw_d, at(L.wdT), d, d, F, s))) return rc;
  if ((rc = fswiglu_gemm_tn_bf16(dout, ld_dout, at(L.wdT), d, at(L.dh), F, M, F, d, bf, scratch, sb, stream))) return rc;
  // 3. gate derivative, with the transposes the weight-gradient products need
  {
    const int64_t tiles = ((L.Mp + kEwTile - 1) / kEwTile) * ((F + kEwTile - 1) / kEwTile);
    swiglu_bwd_kernel<<<ew_grid(*st, tiles), kEwThreads, 0, s>>>(
        static_cast<const __nv_bfloat16*>(at(L.g)), static_cast<const __nv_bfloat16*>(at(L.u)),
        static_cast<const __nv_bfloat16*>(at(L.dh)), F, static_cast<__nv_bfloat16*>(at(L.dgdu)), 2 * F,
        static_cast<__nv_bfloat16*>(at(L.dgT)), static_cast<__nv_bfloat16*>(at(L.duT)),
        static_cast<__nv_bfloat16*>(at(L.hT)), L.Mp, static_cast<int>(M), static_cast<int>(F), static_cast<int>(L.Mp));
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (cudaGetLastError() != cudaSuccess) return FSWIGLU_ERR_CUDA;
  }
  // 4. weight gradients, contracting over the (padded) token dimension
  if ((rc = transpose_impl(*st, dout, ld_dout, at(L.doutT), L.Mp, M, d, s))) return rc;
  if ((rc = transpose_impl(*st, x, ldx, at(L.xT), L.Mp, M, d, s))) return rc;
  if ((rc = fswiglu_gemm_tn_bf16(at(L.doutT), L.Mp, at(L.hT), L.Mp, d_w_down, ld_dw_d, d, F, L.Mp, grad_dtype, scratch, sb,
                                 stream)))
    return rc;
  if ((rc = fswiglu_gemm_tn_bf16(at(L.dgT), L.Mp, at(L.xT), L.Mp, d_w_gate, ld_dw_gu, F, d, L.Mp, grad_dtype, scratch, sb,
                                 stream)))
    return rc;
  if ((rc = fswiglu_gemm_tn_bf16(at(L.duT), L.Mp, at(L.xT), L.Mp, d_w_up, ld_dw_gu, F, d, L.Mp, grad_dtype, scratch, sb,
                                 stream)))
    return rc;
  // 5. dx = [dg | du] [Wg; Wu]: one product over K = 2F with B = [Wg^T | Wu^T] [d, 2F]
  if ((rc = transpose_impl(*st, w_gate, ldw_gu, at(L.wguT), 2 * F, F, d, s))) return rc;
  if ((rc = transpose_impl(*st, w_up, ldw_gu, static_cast<__nv_bfloat16*>(at(L.wguT)) + F, 2 * F, F, d, s))) return rc;
  return fswiglu_gemm_tn_bf16(at(L.dgdu), 2 * F, at(L.wguT), 2 * F, dx, ld_dx, M, d, 2 * F, grad_dtype, scratch, sb, stream);
}

int fswiglu_cast_f32_to_bf16(const void* src, void* dst, int64_t n, void* stream) {
  if (n < 0 || (n > 0 && (src == nullptr || dst == nullptr))) return FSWIGLU_ERR_BAD_ARG;
  if (n == 0) return FSWIGLU_OK;
  if (!aligned16(src) || !aligned16(dst)) return FSWIGLU_ERR_ALIGNMENT;
  DeviceState* st = nullptr;
  if (int rc = device_state(&st)) return rc;
  const long long n8 = n / 8;
  const int tail = static_cast<int>(n - n8 * 8);
  long long blocks = (n8 + 255) / 256;
  const long long cap = static_cast<long long>(st->num_sms) * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  cast_f32_to_bf16_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float4*>(src), static_cast<uint4*>(dst), n8, static_cast<const float*>(src) + n8 * 8,
      static_cast<__nv_bfloat16*>(dst) + n8 * 8, tail);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? FSWIGLU_OK : FSWIGLU_ERR_CUDA;
}

int fswiglu_down_scatter_bf16(const void* h, int64_t ldh, const void* w_down, int64_t ldw,
                              void* const* recv_ptrs, int world, int rank, int64_t rows_per_owner, int64_t M,
                              int64_t d, int64_t F, void* scratch, size_t scratch_bytes, void* stream) {
  if (M < 0 || F <= 0 || d <= 0 || world < 1 || world > 8 || rank < 0 || rank >= world || rows_per_owner <= 0 ||
      recv_ptrs == nullptr)
    return FSWIGLU_ERR_BAD_ARG;
  if (M > rows_per_owner * world) return FSWIGLU_ERR_SHAPE;
  if (M == 0) return FSWIGLU_OK;
  if (d % 8 != 0) return FSWIGLU_ERR_SHAPE;
  DeviceState* st = nullptr;
  if (int rc = device_state(&st)) return rc;
  int rc;
  if ((rc = check_matrix(h, M, F, ldh, true))) return rc;
  if ((rc = check_matrix(w_down, d, F, ldw, true))) return rc;
  GemmParams p = {};
  for (int r = 0; r < world; ++r) {
    if (recv_ptrs[r] == nullptr || !aligned16(recv_ptrs[r])) return FSWIGLU_ERR_ALIGNMENT;
    p.peer_out[r] = recv_ptrs[r];
  }
  p.out = nullptr;
  p.ld_out = d;
  p.M = static_cast<int>(M);
  p.n_out = static_cast<int>(d);
  p.K = static_cast<int>(F);
  p.num_m_tiles = static_cast<int>((M + 127) / 128);
  p.tile_n = pick_tile_n(p.num_m_tiles, d, 256, 1, effective_ctas(*st));
  p.num_n_tiles = static_cast<int>((d + p.tile_n - 1) / p.tile_n);
  p.group_m = pick_group_m(p.num_m_tiles, F);
  p.vec_ok = 1;
  p.status = st->status;
  p.scatter_world = world;
  p.scatter_rank = rank;
  p.rows_per_owner = static_cast<int>(rows_per_owner);
  if (use_pair_kernel(*st, M, d, 256)) {
    Scratch sc;
    if (scratch != nullptr && (reinterpret_cast<uintptr_t>(scratch) & 255u) != 0) return FSWIGLU_ERR_WORKSPACE;
    sc.ptr = scratch;
    sc.bytes = scratch_bytes;
    return launch_gemm_pair<kPlain, false>(*st, h, ldh, w_down, nullptr, ldw, d, p, sc,
                                           static_cast<cudaStream_t>(stream));
  }
  plan_tail_split(&p, effective_ctas(*st));
  CUtensorMap ma, mb;
  if ((rc = encode_map(&ma, h, M, F, ldh, 128))) return rc;
  if ((rc = encode_map(&mb, w_down, d, F, ldw, p.half_boxes ? p.tile_n / 2 : p.tile_n))) return rc;
  return launch_gemm<kPlain, false>(*st, ma, mb, mb, p, static_cast<cudaStream_t>(stream));
}

int fswiglu_reduce_bcast_bf16(const void* recv_local, void* const* out_ptrs, int world, int64_t rows, int64_t cols,
                              int max_ctas, void* stream) {
  if (world < 1 || world > 8 || rows < 0 || cols <= 0 || out_ptrs == nullptr) return FSWIGLU_ERR_BAD_ARG;
  if (rows == 0) return FSWIGLU_OK;
  if (recv_local == nullptr) return FSWIGLU_ERR_BAD_ARG;
  if ((rows * cols) % 8 != 0) return FSWIGLU_ERR_SHAPE;
  if (!aligned16(recv_local)) return FSWIGLU_ERR_ALIGNMENT;
  DeviceState* st = nullptr;
  if (int rc = device_state(&st)) return rc;
  ReduceBcastParams p = {};
  p.recv = static_cast<const uint4*>(recv_local);
  for (int r = 0; r < world; ++r) {
    if (out_ptrs[r] == nullptr || !aligned16(out_ptrs[r])) return FSWIGLU_ERR_ALIGNMENT;
    p.out[r] = out_ptrs[r];
  }
  p.n16 = rows * cols / 8;
  p.world = world;
  int ctas = max_ctas > 0 ? max_ctas : 128;
  const long long need = (p.n16 + 127) / 128;
  if (ctas > need) ctas = static_cast<int>(need);
  reduce_bcast_bf16_kernel<<<ctas, 128, 0, static_cast<cudaStream_t>(stream)>>>(p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? FSWIGLU_OK : FSWIGLU_ERR_CUDA;
}

int fswiglu_set_max_ctas(int max_ctas) {
  DeviceState* st = nullptr;
  if (int rc = device_state(&st)) return rc;
  std::lock_guard<std::mutex> lock(g_mutex);
  const int prev = st->max_ctas;
  st->max_ctas = max_ctas < 0 ? 0 : max_ctas;
  return prev;
}

int64_t fswiglu_set_wait_limit_us(int64_t limit_us) {
  const unsigned long long ns = limit_us > 0 ? static_cast<unsigned long long>(limit_us) * 1000ull : kWaitLimitNs;
  return static_cast<int64_t>(g_wait_limit_ns.exchange(ns, std::memory_order_relaxed) / 1000ull);
}

void fswiglu_set_decode_trace(void* device_buffer) {
  g_decode_trace.store(static_cast<unsigned long long*>(device_buffer), std::memory_order_relaxed);
}

void fswiglu_test_expire_next_wait(int enable) { g_withhold_one_copy.store(enable != 0 ? 1 : 0, std::memory_order_relaxed); }

int fswiglu_device_status(uint32_t* status, void* stream) {
  DeviceState* st = nullptr;
  if (int rc = device_state(&st)) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint32_t word = 0;
  if (int rc = read_and_clear_status(st->status, &word, s)) return rc;
  // the allocation-free entry point keeps its own word next to its built-in scratch: report it too
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < kMaxDevices && g_static[dev].ready) {
    uint32_t static_word = 0;
    if (int rc = read_and_clear_status(g_static[dev].dev.status, &static_word, s)) return rc;
    if (word == 0) word = static_word;
  }
  if (status != nullptr) *status = word;
  return word == 0 ? FSWIGLU_OK : FSWIGLU_ERR_WATCHDOG;
}

const char* fswiglu_status_string(int status) {
  switch (status) {
    case FSWIGLU_OK: return "ok";
    case FSWIGLU_ERR_BAD_ARG: return "bad argument (null pointer, negative size or unknown enum)";
    case FSWIGLU_ERR_ALIGNMENT: return "pointer or leading dimension not 16-byte aligned";
    case FSWIGLU_ERR_SHAPE: return "unsupported shape (d and F must be multiples of 8, ld >= row length)";
    case FSWIGLU_ERR_CUDA: return "CUDA call or kernel launch failed";
    case FSWIGLU_ERR_WATCHDOG: return "device-side wait exceeded its limit";
    case FSWIGLU_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
    case FSWIGLU_ERR_NO_DEVICE: return "current device is not an sm_100 GPU";
    case FSWIGLU_ERR_TOO_LARGE:
      return "M * F * 2 bytes exceeds the 32 MiB scratch built into fswiglu_mlp_bf16_static";
    default: return "unknown status";
  }
}

int fswiglu_plan_kernel(int64_t M, int64_t n_out, int64_t K, int gated) {
  if (M < 0 || n_out <= 0 || K <= 0) return FSWIGLU_ERR_SHAPE;
  DeviceState* st = nullptr;
  if (int rc = device_state(&st)) return rc;
  M = std::min(M, tall_slab_rows(M));  // very tall problems run as row slabs: the plan is that of one slab
  GemmParams p = {};
  p.M = static_cast<int>(M);
  p.n_out = static_cast<int>(n_out);
  p.K = static_cast<int>(K);
  const int tile_n = gated ? 128 : 256;
  if (use_quad_kernel(*st, p, tile_n)) return 2;
  return use_pair_kernel(*st, M, n_out, tile_n) ? 1 : 0;
}

const char* fswiglu_version(void) { return "0.2.0"; }

uint64_t fswiglu_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
