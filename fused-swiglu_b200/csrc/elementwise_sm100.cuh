// Bandwidth-bound helper kernels of the backward pass: a bf16 matrix transpose and the
// element-wise derivative of the SwiGLU gate.  Both move 64 x 64 tiles through shared memory so
// that global reads and writes are 16-byte vectors along the contiguous dimension on both sides.
//
// The tensor-core GEMM kernels take both operands K-major ("TN").  The backward pass needs products
// whose natural operands are not K-major (dW = dY^T X contracts over the token dimension); instead
// of a second family of GEMM kernels the operands are transposed once by these kernels (a few
// bytes per element against the thousands of flops per element the GEMMs spend on them).
#pragma once

#include <cuda_bf16.h>
#include <cstdint>

namespace fsw {

constexpr int kEwTile = 64;
constexpr int kEwPitch = kEwTile + 2;  // shared-memory row pitch in elements: column reads hit distinct banks
constexpr int kEwThreads = 256;

// Write the transposed tile held in shared memory: dst[(c0 + c) * ld + r0 + r] = tile[r][c].
// Rows of dst are padded with zeros up to `dst_cols` (a multiple of 8 >= src_rows), so that the padded
// matrix can be used as a K-major GEMM operand whose K extent is dst_cols.
__device__ __forceinline__ void store_tile_transposed(const __nv_bfloat16 (*tile)[kEwPitch], __nv_bfloat16* dst,
                                                      long long ld, int r0, int c0, int src_rows, int src_cols,
                                                      int dst_cols) {
  const int c = threadIdx.x & 63;        // column of the source tile = row of the destination
  const int rg = threadIdx.x >> 6;       // 4 groups, two 8-row vectors each
  if (c0 + c >= src_cols) return;
#pragma unroll
  for (int it = 0; it < 2; ++it) {
    const int r = (rg * 2 + it) * 8;     // first source row of this 8-element vector
    if (r0 + r >= dst_cols) continue;
    __align__(16) __nv_bfloat16 v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = (r0 + r + i < src_rows) ? tile[r + i][c] : __float2bfloat16(0.0f);
    *reinterpret_cast<uint4*>(dst + static_cast<long long>(c0 + c) * ld + r0 + r) = *reinterpret_cast<const uint4*>(v);
  }
}

// Load a 64 x 64 tile of a row-major bf16 matrix into shared memory (zeros outside the matrix).
__device__ __forceinline__ void load_tile(__nv_bfloat16 (*tile)[kEwPitch], const __nv_bfloat16* src, long long ld,
                                          int r0, int c0, int rows, int cols) {
#pragma unroll
  for (int it = 0; it < 2; ++it) {
    const int idx = threadIdx.x + it * kEwThreads;  // 512 vectors of 8 elements
    const int r = idx >> 3, cv = (idx & 7) * 8;
    uint4 q = make_uint4(0u, 0u, 0u, 0u);
    if (r0 + r < rows && c0 + cv < cols) q = *reinterpret_cast<const uint4*>(src + static_cast<long long>(r0 + r) * ld + c0 + cv);
    const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&q);
#pragma unroll
    for (int i = 0; i < 8; ++i) tile[r][cv + i] = e[i];
  }
}

// dst [cols, dst_cols] = src [rows, cols]^T, dst_cols = rows rounded up to a multiple of 8 (zero padded).
// rows arbitrary, cols % 8 == 0, ld_src % 8 == 0, ld_dst % 8 == 0, 16-byte aligned bases.
__global__ void __launch_bounds__(kEwThreads) transpose_bf16_kernel(const __nv_bfloat16* __restrict__ src, long long ld_src,
                                                                     __nv_bfloat16* __restrict__ dst, long long ld_dst,
                                                                     int rows, int cols, int dst_cols) {
  __shared__ __nv_bfloat16 tile[kEwTile][kEwPitch];
  const int tiles_c = (cols + kEwTile - 1) / kEwTile;
  const int tiles_r = (dst_cols + kEwTile - 1) / kEwTile;
  for (int t = blockIdx.x; t < tiles_r * tiles_c; t += gridDim.x) {
    const int r0 = (t / tiles_c) * kEwTile, c0 = (t % tiles_c) * kEwTile;
    load_tile(tile, src, ld_src, r0, c0, rows, cols);
    __syncthreads();
    store_tile_transposed(tile, dst, ld_dst, r0, c0, rows, cols, dst_cols);
    __syncthreads();
  }
}

// Derivative of h = silu(g) * u with respect to g and u, given dh, all [M, F] bf16 (row pitch ld):
//   s = 1 / (1 + e^-g)        dg = dh * u * s * (1 + g * (1 - s))        du = dh * g * s        h = g * s * u
// in fp32, one rounding per output.  Outputs:
//   dgdu [M, 2F] row-major (dg in columns [0, F), du in [F, 2F)): the K-major A operand of dx = [dg | du] [Wg; Wu]
//   dgT, duT, hT [F, Mp]: the transposes, K-major A operands of dWg = dg^T x, dWu = du^T x and B of dWd = dy^T h;
//   Mp = M rounded up to 8, pad columns zero.
__global__ void __launch_bounds__(kEwThreads) swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ g,
                                                                 const __nv_bfloat16* __restrict__ u,
                                                                 const __nv_bfloat16* __restrict__ dh, long long ld,
                                                                 __nv_bfloat16* __restrict__ dgdu, long long ld_dgdu,
                                                                 __nv_bfloat16* __restrict__ dgT,
                                                                 __nv_bfloat16* __restrict__ duT,
                                                                 __nv_bfloat16* __restrict__ hT, long long ld_t, int M,
                                                                 int F, int Mp) {
  __shared__ __nv_bfloat16 t_dg[kEwTile][kEwPitch];
  __shared__ __nv_bfloat16 t_du[kEwTile][kEwPitch];
  __shared__ __nv_bfloat16 t_h[kEwTile][kEwPitch];
  const int tiles_c = (F + kEwTile - 1) / kEwTile;
  const int tiles_r = (Mp + kEwTile - 1) / kEwTile;
  for (int t = blockIdx.x; t < tiles_r * tiles_c; t += gridDim.x) {
    const int r0 = (t / tiles_c) * kEwTile, c0 = (t % tiles_c) * kEwTile;
#pragma unroll
    for (int it = 0; it < 2; ++it) {
      const int idx = threadIdx.x + it * kEwThreads;
      const int r = idx >> 3, cv = (idx & 7) * 8;
      const bool in = r0 + r < M && c0 + cv < F;
      uint4 qg = make_uint4(0u, 0u, 0u, 0u), qu = qg, qd = qg;
      if (in) {
        const long long off = static_cast<long long>(r0 + r) * ld + c0 + cv;
        qg = *reinterpret_cast<const uint4*>(g + off);
        qu = *reinterpret_cast<const uint4*>(u + off);
        qd = *reinterpret_cast<const uint4*>(dh + off);
      }
      const __nv_bfloat16* eg = reinterpret_cast<const __nv_bfloat16*>(&qg);
      const __nv_bfloat16* eu = reinterpret_cast<const __nv_bfloat16*>(&qu);
      const __nv_bfloat16* ed = reinterpret_cast<const __nv_bfloat16*>(&qd);
      __align__(16) __nv_bfloat16 odg[8], odu[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float gv = __bfloat162float(eg[i]), uv = __bfloat162float(eu[i]), dv = __bfloat162float(ed[i]);
        const float s = 1.0f / (1.0f + __expf(-gv));
        const float dgv = dv * uv * s * (1.0f + gv * (1.0f - s));
        const float duv = dv * gv * s;
        odg[i] = __float2bfloat16_rn(dgv);
        odu[i] = __float2bfloat16_rn(duv);
        t_dg[r][cv + i] = odg[i];
        t_du[r][cv + i] = odu[i];
        t_h[r][cv + i] = __float2bfloat16_rn(gv * s * uv);
      }
      if (in) {
        __nv_bfloat16* row = dgdu + static_cast<long long>(r0 + r) * ld_dgdu + c0 + cv;
        *reinterpret_cast<uint4*>(row) = *reinterpret_cast<const uint4*>(odg);
        *reinterpret_cast<uint4*>(row + F) = *reinterpret_cast<const uint4*>(odu);
      }
    }
    __syncthreads();
    store_tile_transposed(t_dg, dgT, ld_t, r0, c0, M, F, Mp);
    store_tile_transposed(t_du, duT, ld_t, r0, c0, M, F, Mp);
    store_tile_transposed(t_h, hT, ld_t, r0, c0, M, F, Mp);
    __syncthreads();
  }
}

}  // namespace fsw
