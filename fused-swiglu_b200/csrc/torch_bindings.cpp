// Operator boundary: the same Python module (`fused_mlp_module`) and dispatcher library
// (`ASMLLM`) as the reference's csrc/torch_bindings.cpp:27-50, with the same two ops
//
//   fused_swiglu_bf16(Tensor X, Tensor W1W3) -> Tensor
//   swiglu_fwd_bf16(int m, int n, int k, Tensor A, int ldA, Tensor B, int ldB, Tensor C, int ldC) -> ()
//
// plus the split-weight and whole-MLP ops the reference lacks.  This file is the only one
// that sees torch types: it validates tensors, takes the current device / stream and hands
// raw pointers to the C ABI in include/fswiglu.h.  A non-zero status becomes a c10::Error
// (RuntimeError in Python), like the reference's TORCH_CHECKs (csrc/SwiGLU/swiglu.cu:475-480).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <optional>

#include "fswiglu.h"

namespace {

void check_status(int rc, const char* where) {
  TORCH_CHECK(rc == FSWIGLU_OK, where, ": ", fswiglu_status_string(rc), " (status ", rc, ")");
}

void check_bf16_cuda(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.scalar_type() == at::kBFloat16, name, " must be a bfloat16 tensor");
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
}

int64_t row_pitch(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.dim() == 2, name, " must be 2-D");
  TORCH_CHECK(t.size(1) <= 1 || t.stride(1) == 1, name, " must have unit stride along its last dimension");
  return t.size(0) > 1 ? t.stride(0) : std::max<int64_t>(t.stride(0), t.size(1));
}

void* current_stream(const at::Tensor& t) {
  return static_cast<void*>(at::cuda::getCurrentCUDAStream(t.get_device()).stream());
}

}  // namespace

// Raw launcher, reference semantics (csrc/SwiGLU/swiglu.cu:397-525): leading dimensions in elements,
// B holds up rows at even and gate rows at odd indices, the [m, n/2] result is written into C with
// row stride ldC/2.
void swiglu_fwd_bf16(int64_t m, int64_t n, int64_t k, at::Tensor const& A, int64_t ldA, at::Tensor const& B,
                     int64_t ldB, at::Tensor const& C, int64_t ldC) {
  check_bf16_cuda(A, "A");
  check_bf16_cuda(B, "B");
  check_bf16_cuda(C, "C");
  TORCH_CHECK(n % 2 == 0 && ldC % 2 == 0, "n and ldC must be even (up/gate rows are interleaved)");
  const c10::cuda::OptionalCUDAGuard guard(device_of(A));
  check_status(fswiglu_gateup_bf16(A.data_ptr(), ldA, B.data_ptr(), ldB, nullptr, C.data_ptr(), ldC / 2, m, n / 2,
                                   k, 1, current_stream(A)),
               "swiglu_fwd_bf16");
}

// Convenience wrapper, reference semantics (csrc/SwiGLU/swiglu.cu:538-553): allocates [M, N/2].
at::Tensor fused_swiglu_bf16(at::Tensor const& X, at::Tensor const& W1W3) {
  check_bf16_cuda(X, "X");
  check_bf16_cuda(W1W3, "W1W3");
  const int64_t M = X.size(0), N = W1W3.size(0), K = X.size(1);
  at::Tensor out = at::empty({M, N / 2}, X.options());
  swiglu_fwd_bf16(M, N, K, X, row_pitch(X, "X"), W1W3, row_pitch(W1W3, "W1W3"), out, N);
  return out;
}

// In-place form of the raw launcher with the mutation of C declared in its schema (Tensor(a!)), so that
// graph capture (torch.compile, export) keeps the call and orders it.  The reference's schema
// (csrc/torch_bindings.cpp:42) declares no mutation, which is why the op of that name is registered
// here without a shape-only kernel: like the reference's, it cannot be traced, instead of being
// traced wrongly.
void swiglu_fwd_bf16_out(int64_t m, int64_t n, int64_t k, at::Tensor const& A, int64_t ldA, at::Tensor const& B,
                         int64_t ldB, at::Tensor& C, int64_t ldC) {
  swiglu_fwd_bf16(m, n, k, A, ldA, B, ldB, C, ldC);
}

const float* optional_row_scale(const std::optional<at::Tensor>& row_scale, const at::Tensor& x) {
  if (!row_scale.has_value() || !row_scale->defined()) return nullptr;
  TORCH_CHECK(row_scale->scalar_type() == at::kFloat && row_scale->is_cuda() && row_scale->is_contiguous() &&
                  row_scale->numel() == x.size(0),
              "row_scale must be a contiguous float32 CUDA tensor with one entry per row of x");
  return row_scale->data_ptr<float>();
}

const void* optional_residual(const std::optional<at::Tensor>& residual, int64_t M, int64_t d, int64_t* ldr) {
  *ldr = 0;
  if (!residual.has_value() || !residual->defined()) return nullptr;
  check_bf16_cuda(*residual, "residual");
  TORCH_CHECK(residual->dim() == 2 && residual->size(0) == M && residual->size(1) == d, "residual must be [M, d]");
  *ldr = row_pitch(*residual, "residual");
  return residual->data_ptr();
}

// scale[r] = rsqrt(mean(x[r]^2) + eps): the RMSNorm statistic, consumed as `row_scale` below.
at::Tensor rms_scale(at::Tensor const& x, double eps) {
  check_bf16_cuda(x, "x");
  at::Tensor scale = at::empty({x.size(0)}, x.options().dtype(at::kFloat));
  const c10::cuda::OptionalCUDAGuard guard(device_of(x));
  check_status(fswiglu_rms_scale_f32(x.data_ptr(), row_pitch(x, "x"), x.size(0), x.size(1), static_cast<float>(eps),
                                     scale.data_ptr<float>(), current_stream(x)),
               "rms_scale");
  return scale;
}

at::Tensor fused_swiglu_gateup_bf16(at::Tensor const& x, at::Tensor const& W_gate, at::Tensor const& W_up,
                                    std::optional<at::Tensor> const& row_scale) {
  check_bf16_cuda(x, "x");
  check_bf16_cuda(W_gate, "W_gate");
  check_bf16_cuda(W_up, "W_up");
  const int64_t M = x.size(0), d = x.size(1), F = W_gate.size(0);
  TORCH_CHECK(W_up.sizes() == W_gate.sizes() && W_gate.size(1) == d, "W_gate and W_up must both be [F, d]");
  const int64_t ldw = row_pitch(W_gate, "W_gate");
  TORCH_CHECK(row_pitch(W_up, "W_up") == ldw, "W_gate and W_up must share one leading dimension");
  at::Tensor h = at::empty({M, F}, x.options());
  const c10::cuda::OptionalCUDAGuard guard(device_of(x));
  check_status(fswiglu_gateup_bf16_ex(x.data_ptr(), row_pitch(x, "x"), W_gate.data_ptr(), ldw, W_up.data_ptr(),
                                      h.data_ptr(), F, M, F, d, 0, optional_row_scale(row_scale, x), nullptr, 0,
                                      current_stream(x)),
               "fused_swiglu_gateup_bf16");
  return h;
}

at::Tensor swiglu_down_bf16(at::Tensor const& h, at::Tensor const& W_down, bool fp32_out,
                            std::optional<at::Tensor> const& residual) {
  check_bf16_cuda(h, "h");
  check_bf16_cuda(W_down, "W_down");
  const int64_t M = h.size(0), F = h.size(1), d = W_down.size(0);
  TORCH_CHECK(W_down.size(1) == F, "W_down must be [d, F]");
  at::Tensor out = at::empty({M, d}, h.options().dtype(fp32_out ? at::kFloat : at::kBFloat16));
  const c10::cuda::OptionalCUDAGuard guard(device_of(h));
  int64_t ldr = 0;
  const void* res = optional_residual(residual, M, d, &ldr);
  check_status(fswiglu_down_bf16_ex(h.data_ptr(), row_pitch(h, "h"), W_down.data_ptr(), row_pitch(W_down, "W_down"),
                                    out.data_ptr(), d, M, d, F, fp32_out ? FSWIGLU_OUT_F32 : FSWIGLU_OUT_BF16, res,
                                    ldr, nullptr, 0, current_stream(h)),
               "swiglu_down_bf16");
  return out;
}

// residual / row_scale: the fusions either side of the MLP (see include/fswiglu.h); fp32_out is the
// switch the reference makes at compile time (csrc/constants.cuh:9-14).
at::Tensor fused_swiglu_mlp_bf16(at::Tensor const& x, at::Tensor const& W_gate, at::Tensor const& W_up,
                                 at::Tensor const& W_down, std::optional<at::Tensor> const& residual,
                                 std::optional<at::Tensor> const& row_scale, bool fp32_out) {
  check_bf16_cuda(x, "x");
  check_bf16_cuda(W_gate, "W_gate");
  check_bf16_cuda(W_up, "W_up");
  check_bf16_cuda(W_down, "W_down");
  const int64_t M = x.size(0), d = x.size(1), F = W_gate.size(0);
  TORCH_CHECK(W_up.sizes() == W_gate.sizes() && W_gate.size(1) == d && W_down.size(0) == d && W_down.size(1) == F,
              "expected W_gate/W_up [F, d] and W_down [d, F]");
  const int64_t ldw = row_pitch(W_gate, "W_gate");
  TORCH_CHECK(row_pitch(W_up, "W_up") == ldw, "W_gate and W_up must share one leading dimension");
  at::Tensor out = at::empty({M, d}, x.options().dtype(fp32_out ? at::kFloat : at::kBFloat16));
  if (M == 0) return out;
  int64_t ldr = 0;
  const void* res = optional_residual(residual, M, d, &ldr);
  const int64_t ws_bytes = static_cast<int64_t>(fswiglu_workspace_bytes(M, d, F));
  at::Tensor ws = at::empty({std::max<int64_t>(ws_bytes, 256)}, x.options().dtype(at::kByte));
  const c10::cuda::OptionalCUDAGuard guard(device_of(x));
  check_status(fswiglu_mlp_bf16_ex(x.data_ptr(), row_pitch(x, "x"), optional_row_scale(row_scale, x),
                                   W_gate.data_ptr(), W_up.data_ptr(), ldw, W_down.data_ptr(),
                                   row_pitch(W_down, "W_down"), res, ldr, out.data_ptr(), d,
                                   fp32_out ? FSWIGLU_OUT_F32 : FSWIGLU_OUT_BF16, M, d, F, ws.data_ptr(),
                                   static_cast<size_t>(ws.numel()), current_stream(x)),
               "fused_swiglu_mlp_bf16");
  return out;
}

// Shape-only ("Meta") implementations: what fake-tensor tracing (torch.compile, export) needs to see
// through the ops without running them.  The reference registers CUDA kernels only
// (csrc/torch_bindings.cpp:45-50 there), so its ops cannot be traced.
at::Tensor fused_swiglu_bf16_meta(at::Tensor const& X, at::Tensor const& W1W3) {
  return at::empty({X.size(0), W1W3.size(0) / 2}, X.options());
}
void swiglu_fwd_bf16_out_meta(int64_t, int64_t, int64_t, at::Tensor const&, int64_t, at::Tensor const&, int64_t,
                              at::Tensor&, int64_t) {}
at::Tensor rms_scale_meta(at::Tensor const& x, double) { return at::empty({x.size(0)}, x.options().dtype(at::kFloat)); }
at::Tensor fused_swiglu_gateup_bf16_meta(at::Tensor const& x, at::Tensor const& W_gate, at::Tensor const&,
                                         std::optional<at::Tensor> const&) {
  return at::empty({x.size(0), W_gate.size(0)}, x.options());
}
at::Tensor swiglu_down_bf16_meta(at::Tensor const& h, at::Tensor const& W_down, bool fp32_out,
                                 std::optional<at::Tensor> const&) {
  return at::empty({h.size(0), W_down.size(0)}, h.options().dtype(fp32_out ? at::kFloat : at::kBFloat16));
}
at::Tensor fused_swiglu_mlp_bf16_meta(at::Tensor const& x, at::Tensor const&, at::Tensor const&,
                                      at::Tensor const& W_down, std::optional<at::Tensor> const&,
                                      std::optional<at::Tensor> const&, bool fp32_out) {
  return at::empty({x.size(0), W_down.size(0)}, x.options().dtype(fp32_out ? at::kFloat : at::kBFloat16));
}

namespace Fused_MLP {

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  namespace py = pybind11;
  m.def("fused_swiglu_bf16", &fused_swiglu_bf16, "fused SwiGLU for bf16");
  m.def("swiglu_fwd_bf16", &swiglu_fwd_bf16, "SwiGLU fwd bf16");
  m.def("rms_scale", &rms_scale, "rsqrt(mean(x^2) + eps) per row", py::arg("x"), py::arg("eps") = 1e-6);
  m.def("fused_swiglu_gateup_bf16", &fused_swiglu_gateup_bf16, "silu(s x Wg^T) * (s x Wu^T), split weights",
        py::arg("x"), py::arg("W_gate"), py::arg("W_up"), py::arg("row_scale") = py::none());
  m.def("swiglu_down_bf16", &swiglu_down_bf16, "(residual +) h Wd^T", py::arg("h"), py::arg("W_down"),
        py::arg("fp32_out") = false, py::arg("residual") = py::none());
  m.def("fused_swiglu_mlp_bf16", &fused_swiglu_mlp_bf16, "(residual +) (silu(s x Wg^T) * (s x Wu^T)) Wd^T",
        py::arg("x"), py::arg("W_gate"), py::arg("W_up"), py::arg("W_down"), py::arg("residual") = py::none(),
        py::arg("row_scale") = py::none(), py::arg("fp32_out") = false);
}

TORCH_LIBRARY(ASMLLM, m) {
  m.def("fused_swiglu_bf16(Tensor X, Tensor W1W3) -> Tensor");
  m.def("swiglu_fwd_bf16(int m, int n, int k, Tensor A, int ldA, Tensor B, int ldB, Tensor C, int ldC) -> ()");
  m.def("swiglu_fwd_bf16_out(int m, int n, int k, Tensor A, int ldA, Tensor B, int ldB, Tensor(a!) C, int ldC) -> ()");
  m.def("rms_scale(Tensor x, float eps=1e-6) -> Tensor");
  m.def("fused_swiglu_gateup_bf16(Tensor x, Tensor W_gate, Tensor W_up, Tensor? row_scale=None) -> Tensor");
  m.def("swiglu_down_bf16(Tensor h, Tensor W_down, bool fp32_out=False, Tensor? residual=None) -> Tensor");
  m.def("fused_swiglu_mlp_bf16(Tensor x, Tensor W_gate, Tensor W_up, Tensor W_down, Tensor? residual=None, "
        "Tensor? row_scale=None, bool fp32_out=False) -> Tensor");
}

TORCH_LIBRARY_IMPL(ASMLLM, CUDA, m) {
  m.impl("fused_swiglu_bf16", &fused_swiglu_bf16);
  m.impl("swiglu_fwd_bf16", &swiglu_fwd_bf16);
  m.impl("swiglu_fwd_bf16_out", &swiglu_fwd_bf16_out);
  m.impl("rms_scale", &rms_scale);
  m.impl("fused_swiglu_gateup_bf16", &fused_swiglu_gateup_bf16);
  m.impl("swiglu_down_bf16", &swiglu_down_bf16);
  m.impl("fused_swiglu_mlp_bf16", &fused_swiglu_mlp_bf16);
}

TORCH_LIBRARY_IMPL(ASMLLM, Meta, m) {
  m.impl("fused_swiglu_bf16", &fused_swiglu_bf16_meta);
  m.impl("swiglu_fwd_bf16_out", &swiglu_fwd_bf16_out_meta);
  m.impl("rms_scale", &rms_scale_meta);
  m.impl("fused_swiglu_gateup_bf16", &fused_swiglu_gateup_bf16_meta);
  m.impl("swiglu_down_bf16", &swiglu_down_bf16_meta);
  m.impl("fused_swiglu_mlp_bf16", &fused_swiglu_mlp_bf16_meta);
}

}  // namespace Fused_MLP
