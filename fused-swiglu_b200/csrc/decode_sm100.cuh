// Small-batch (M <= 64 tokens) path of the SwiGLU MLP forward: weight
// streaming bound by HBM bandwidth.  Interface used by api.cu.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace fsw {

constexpr int kDecodeMaxTokens = 64;

inline cudaError_t decode_opt_in_smem() { return cudaSuccess; }

inline bool decode_supported(int64_t, int64_t, int64_t, int64_t, int64_t, int64_t) { return false; }

inline size_t decode_workspace_bytes(int64_t, int64_t, int64_t) { return 0; }

inline cudaError_t decode_mlp_launch(const void*, int64_t, const void*, const void*, int64_t, const void*,
                                     int64_t, void*, int64_t, int, int64_t, int64_t, int64_t, void*, void*,
                                     int, uint32_t*, cudaStream_t, int*) {
  return cudaErrorNotSupported;
}

}  // namespace fsw
