/*
 * fswiglu.h -- C ABI of the B200 (sm_100a) fused SwiGLU MLP forward library, libfswiglu.so.
 *
 * The reference project (bit-ml/Fused-SwiGLU) has no C ABI: torch tensors cross its
 * operator boundary directly (csrc/torch_bindings.cpp:27-50).  This header is the
 * torch-free boundary underneath that operator surface; the torch extension
 * `fused_mlp_module` (same module and op names as the reference) is a thin caller of
 * these entry points, and so is any other host (ctypes, cgo, JNI ...).
 *
 * Conventions
 *   - all matrices are row-major bf16 in device memory of the CURRENT device; leading
 *     dimensions (ld*) are in ELEMENTS;
 *   - x [M, d], W_gate / W_up [F, d], h [M, F], W_down [d, F], out [M, d];
 *   - every call is asynchronous on `stream` (a cudaStream_t passed as void*), never
 *     synchronises, never throws; it returns FSWIGLU_OK or a negative status;
 *   - requirements checked on entry: 16-byte aligned base pointers, d % 8 == 0 and
 *     F % 8 == 0 (TMA needs 16-byte row pitches), ld >= row length, ld % 8 == 0 for
 *     TMA-read operands; M, d, F may otherwise be ragged (not tile multiples);
 *   - M == 0 (empty batch) is a successful no-op;
 *   - there is no CPU fallback: without a usable sm_100 device the calls fail.
 */
#ifndef FSWIGLU_H_
#define FSWIGLU_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  FSWIGLU_OK = 0,
  FSWIGLU_ERR_BAD_ARG = -1,    /* null pointer, negative size, unknown enum value      */
  FSWIGLU_ERR_ALIGNMENT = -2,  /* base pointer or leading dimension not 16-byte aligned */
  FSWIGLU_ERR_SHAPE = -3,      /* d or F not a multiple of 8, ld too small, size > 2^31 */
  FSWIGLU_ERR_CUDA = -4,       /* CUDA runtime / driver call or kernel launch failed    */
  FSWIGLU_ERR_WATCHDOG = -5,   /* a bounded device-side wait gave up (see device_status)*/
  FSWIGLU_ERR_WORKSPACE = -6,  /* workspace missing or smaller than workspace_bytes()   */
  FSWIGLU_ERR_NO_DEVICE = -7,  /* current device is not compute capability 10.x         */
  FSWIGLU_ERR_TOO_LARGE = -8   /* problem exceeds the built-in scratch of the _static call */
};

/* Output element type of the down projection. */
enum { FSWIGLU_OUT_BF16 = 0, FSWIGLU_OUT_F32 = 1 };

/*
 * Gate-up projection fused with the SwiGLU gate:  h = silu(x Wg^T) * (x Wu^T).
 *
 * Replaces the reference's swiglu_fwd<bf16,bf16,bf16> host launcher and its kernel
 * (csrc/SwiGLU/swiglu.cu:397-525 and :103-394; bound as `swiglu_fwd_bf16` at
 * csrc/torch_bindings.cpp:35,42,49).
 *
 *   interleaved == 0 : w_gate_or_w13 = W_gate [F, d], w_up = W_up [F, d]
 *   interleaved != 0 : w_gate_or_w13 = the reference's packed W1W3 [2F, d] with row 2j = up_j and
 *                      row 2j+1 = gate_j (csrc/SwiGLU/swiglu.cu:376-383); w_up must be NULL.
 *                      With ldh = ldC / 2 this is bit-for-bit the reference call
 *                      swiglu_fwd_bf16(M, 2F, d, x, ldx, W1W3, ldw, C, ldC).
 */
int fswiglu_gateup_bf16(const void* x, int64_t ldx, const void* w_gate_or_w13, int64_t ldw,
                        const void* w_up, void* h, int64_t ldh, int64_t M, int64_t F, int64_t d,
                        int interleaved, void* stream);

/*
 * The same stage with its two options (the reference's launcher, csrc/SwiGLU/swiglu.cu:397-525, has
 * neither):
 *   row_scale  NULL, or M fp32 factors s_r: the stage computes silu(s_r * (x Wg^T)_r) * (s_r * (x Wu^T)_r),
 *              i.e. the gate-up projection of the row-normalised input without materialising it.  With
 *              s_r from fswiglu_rms_scale_f32 and the norm's weight vector folded into the columns of
 *              W_gate / W_up this is RMSNorm followed by the gate-up stage.
 *   scratch    NULL, or a 256-byte aligned device buffer of fswiglu_gemm_scratch_bytes() bytes.  With it
 *              the two-SM kernel splits the reduction of its last, partly filled wave of tiles over all
 *              SMs (fp32 partial sums combined in a fixed order: deterministic, but the summation order
 *              of those tiles differs from the unsplit kernel's).  The buffer may be shared by calls
 *              that are ordered on one stream, not by concurrent ones.
 */
int fswiglu_gateup_bf16_ex(const void* x, int64_t ldx, const void* w_gate_or_w13, int64_t ldw,
                           const void* w_up, void* h, int64_t ldh, int64_t M, int64_t F, int64_t d,
                           int interleaved, const float* row_scale, void* scratch, size_t scratch_bytes,
                           void* stream);
size_t fswiglu_gemm_scratch_bytes(void);

/*
 * Down projection  out = h Wd^T  (absent from the reference, whose kernel stops at h; required by
 * the full-MLP expression (silu(x Wg^T) * (x Wu^T)) Wd^T the build is checked against).
 * out_dtype: FSWIGLU_OUT_BF16 (one rounding of the fp32 accumulator) or FSWIGLU_OUT_F32 (tensor-
 * parallel partial sums that are reduced before rounding).
 */
int fswiglu_down_bf16(const void* h, int64_t ldh, const void* w_down, int64_t ldw, void* out,
                      int64_t ldo, int64_t M, int64_t d, int64_t F, int out_dtype, void* stream);

/*
 * The same stage with its two options (no counterpart in the reference):
 *   residual   NULL, or a bf16 matrix [M, d] with row pitch ldr (16-byte aligned, ldr % 8 == 0,
 *              d % 8 == 0): out = residual + h Wd^T, added to the fp32 accumulator before the single
 *              rounding.  May be `out` itself (same base and pitch): the warp that writes a group of
 *              elements has read them first.
 *   scratch    as for fswiglu_gateup_bf16_ex.
 */
int fswiglu_down_bf16_ex(const void* h, int64_t ldh, const void* w_down, int64_t ldw, void* out,
                         int64_t ldo, int64_t M, int64_t d, int64_t F, int out_dtype, const void* residual,
                         int64_t ldr, void* scratch, size_t scratch_bytes, void* stream);

/*
 * Whole MLP forward on device buffers:  out = (silu(x Wg^T) * (x Wu^T)) Wd^T.
 * `workspace` holds the bf16 hidden activations (and, for M <= 64, the split-K partial sums of the
 * decode path); it must be 256-byte aligned and at least fswiglu_workspace_bytes(M, d, F) long.
 * The eager expression it replaces: numeric_tests.py:41-43 (gate-up part) extended with the down
 * projection.
 */
int fswiglu_mlp_bf16(const void* x, int64_t ldx, const void* w_gate, const void* w_up, int64_t ldw_gu,
                     const void* w_down, int64_t ldw_d, void* out, int64_t ldo, int out_dtype,
                     int64_t M, int64_t d, int64_t F, void* workspace, size_t workspace_bytes,
                     void* stream);

/* Bytes of workspace fswiglu_mlp_bf16 needs for this problem size (0 when M == 0). */
size_t fswiglu_workspace_bytes(int64_t M, int64_t d, int64_t F);

/*
 * The transformer block around the MLP, fused (the reference stops at the gate; its benchmark only
 * gestures at the surrounding module, bench_swiglu.py:22-32):
 *     out = residual + ( silu(s * (x Wg^T)) * (s * (x Wu^T)) ) Wd^T
 * row_scale (s, may be NULL) and residual (may be NULL) as described for the two stages above; the
 * workspace is the one of fswiglu_mlp_bf16.  All batch sizes, including the small-batch path.
 */
int fswiglu_mlp_bf16_ex(const void* x, int64_t ldx, const float* row_scale, const void* w_gate,
                        const void* w_up, int64_t ldw_gu, const void* w_down, int64_t ldw_d,
                        const void* residual, int64_t ldr, void* out, int64_t ldo, int out_dtype, int64_t M,
                        int64_t d, int64_t F, void* workspace, size_t workspace_bytes, void* stream);

/*
 * scale[r] = 1 / sqrt(mean_k x[r, k]^2 + eps) in fp32 for the M rows of the bf16 matrix x [M, d]: the
 * statistic of RMSNorm, the normalisation in front of the MLP in Llama-family blocks.  One pass over
 * x (bandwidth bound); feed the result to `row_scale` above.  No counterpart in the reference.
 */
int fswiglu_rms_scale_f32(const void* x, int64_t ldx, int64_t M, int64_t d, float eps, float* scale,
                          void* stream);

/*
 * Same MLP forward with HOST buffers for the activations: x_host [M, d] and out_host [M, d] are
 * (ideally pinned) host memory, weights stay resident on the device.  Rows are independent, so the
 * call cuts M into slabs and overlaps host->device copy, compute and device->host copy of
 * successive slabs on three internal streams ordered after `stream`; it returns after the last
 * slab has landed in out_host (this call synchronises).  Device staging comes from `workspace`
 * (fswiglu_host_workspace_bytes).
 */
int fswiglu_mlp_bf16_host(const void* x_host, const void* w_gate, const void* w_up,
                          const void* w_down, void* out_host, int64_t M, int64_t d, int64_t F,
                          void* workspace, size_t workspace_bytes, void* stream);
size_t fswiglu_host_workspace_bytes(int64_t M, int64_t d, int64_t F);

/*
 * Whole MLP forward for hosts that must not allocate device memory.  This entry point has no
 * counterpart in the reference; it exists for callers of this library that cannot call cudaMalloc
 * at all, or not where they call us: a serving process that hands the whole GPU to its own memory
 * pool when it starts (so a later cudaMalloc fails or fragments the pool), or a latency-critical loop
 * that cannot tolerate the device-wide synchronisation an allocation may cause.  It computes exactly
 * what fswiglu_mlp_bf16 computes (always with the tiled tensor-core kernels), but the hidden
 * activations h [M, F] live in a fixed array built into the library image instead of a caller
 * workspace, and the call itself performs no cudaMalloc / cudaFree and calls no allocating library
 * routine.
 *
 *   - Limit: M * F * 2 bytes must not exceed FSWIGLU_STATIC_SCRATCH_BYTES (32 MiB: e.g. M = 1024 at
 *     F = 14336, or M = 512 at F = 28672); beyond it the call returns FSWIGLU_ERR_TOO_LARGE and
 *     launches nothing.  Every GPU that loads the library carries the array until the process exits.
 *   - The first call on each device looks the array's device address up (and opts the kernels in to
 *     their shared-memory size); make that first call before any stream capture begins.
 *   - All calls on a device share the one array and it keeps the previous call's contents.  Nothing in
 *     it needs to start at zero (h is fully rewritten before it is read; the error word next to it is
 *     zero when the library is loaded and, by design, stays set after a device-side time-out).  Two
 *     calls whose kernels overlap on the GPU (different streams, no ordering between them) race on
 *     the array and produce garbage: order them.
 *   - When the memory is taken: the array is part of the library's device code image, so the CUDA
 *     driver reserves its 32 MiB (+256 bytes) on a device when it loads that image there - with the
 *     default lazy module loading that is the FIRST call into this library on the device, of any entry
 *     point, not only this one.  A host that hands the GPU to its own pool should make one cheap call
 *     (for instance fswiglu_static_status) on every device before it sizes the pool.
 *   - Device-side time-outs of this entry point are recorded in a word next to the array, not in the
 *     cudaMalloc'd status block the other entry points use.  fswiglu_static_status() reads and clears
 *     that word without allocating anything; fswiglu_device_status() reports it as well.
 */
#define FSWIGLU_STATIC_SCRATCH_BYTES (32u << 20)
int fswiglu_mlp_bf16_static(const void* x, int64_t ldx, const void* w_gate, const void* w_up,
                            int64_t ldw_gu, const void* w_down, int64_t ldw_d, void* out, int64_t ldo,
                            int out_dtype, int64_t M, int64_t d, int64_t F, void* stream);
/*
 * Synchronises `stream`, copies the time-out word of fswiglu_mlp_bf16_static on the current device
 * into *status (0 = healthy), clears it, and returns FSWIGLU_ERR_WATCHDOG if it was set.  Allocates
 * nothing (also sets the device up like a first fswiglu_mlp_bf16_static call).  No counterpart in the
 * reference.
 */
int fswiglu_static_status(uint32_t* status, void* stream);

/*
 * Backward pass of the MLP (no counterpart in the reference, which is forward only: its ops are named
 * *_fwd and register no autograd, csrc/torch_bindings.cpp:38-50).  Given dout = dL/d out [M, d]:
 *     g = x Wg^T, u = x Wu^T (recomputed), s = sigmoid(g), h = g s u
 *     dh = dout Wd        dg = dh u s (1 + g (1 - s))        du = dh g s
 *     dWd = dout^T h      dWg = dg^T x      dWu = du^T x      dx = dg Wg + du Wu
 * Seven tensor-core GEMMs (the forward kernels' plain mode; operands that are not K-major are transposed
 * first by a bandwidth-bound kernel) and one element-wise kernel; 16 M d F flops.  Intermediates are bf16,
 * accumulation fp32.  dx [M, d], d_w_gate / d_w_up [F, d], d_w_down [d, F] are written (not accumulated)
 * as bf16 or fp32 (grad_dtype).  The weight gradients contract over the token dimension, padded with
 * zeros to a multiple of 8.  Gradients of the fused options (row_scale, residual) are not provided: the
 * residual's is dout itself, the norm's belongs to the caller's norm.
 */
size_t fswiglu_backward_workspace_bytes(int64_t M, int64_t d, int64_t F);
int fswiglu_mlp_backward_bf16(const void* x, int64_t ldx, const void* w_gate, const void* w_up, int64_t ldw_gu,
                              const void* w_down, int64_t ldw_d, const void* dout, int64_t ld_dout, void* dx,
                              int64_t ld_dx, void* d_w_gate, void* d_w_up, int64_t ld_dw_gu, void* d_w_down,
                              int64_t ld_dw_d, int grad_dtype, int64_t M, int64_t d, int64_t F, void* workspace,
                              size_t workspace_bytes, void* stream);

/*
 * The two building blocks of the backward pass, usable on their own (no counterpart in the reference):
 * C [M, N] = A [M, K] B [N, K]^T with both operands K-major bf16 (fp32 accumulation; out_dtype and scratch
 * as for fswiglu_down_bf16_ex, which this is), and dst [cols, rows rounded up to 8] = src [rows, cols]^T
 * with zero padding (cols % 8 == 0, 16-byte aligned bases and pitches).
 */
int fswiglu_gemm_tn_bf16(const void* a, int64_t lda, const void* b, int64_t ldb, void* c, int64_t ldc, int64_t M,
                         int64_t N, int64_t K, int out_dtype, void* scratch, size_t scratch_bytes, void* stream);
int fswiglu_transpose_bf16(const void* src, int64_t ld_src, void* dst, int64_t ld_dst, int64_t rows, int64_t cols,
                           void* stream);

/*
 * dst[i] = bf16(src[i]) for n contiguous elements (round to nearest even): the single rounding after
 * tensor-parallel fp32 partial sums have been reduced.  No counterpart in the reference (single GPU).
 * src and dst must be 16-byte aligned.
 */
int fswiglu_cast_f32_to_bf16(const void* src, void* dst, int64_t n, void* stream);

/*
 * Tensor-parallel reduction over peer memory, in two calls (no counterpart in the reference).
 *
 * fswiglu_down_scatter_bf16: the down projection of this rank's shard, out_partial = h Wd^T, whose
 * epilogue is also the reduce-scatter: output row r belongs to rank r / rows_per_owner and its bf16
 * partial sum is stored directly into that rank's receive buffer recv_ptrs[owner] (a peer-mapped
 * device pointer; plain stores over NVLink, no TMA on peer memory), at row
 * rank * rows_per_owner + r % rows_per_owner of a [world * rows_per_owner, d] matrix.  The transfer
 * overlaps the GEMM tile by tile.  recv_ptrs is a HOST array of `world` (<= 8) device pointers.
 * `scratch` is the optional buffer of fswiglu_gateup_bf16_ex (NULL: no split of the last wave).
 *
 * fswiglu_reduce_bcast_bf16: once every rank's stores have landed (the caller separates the two
 * calls by a cross-rank barrier), each rank sums the `world` copies of its own `rows` rows in fp32
 * in rank order, rounds once, and stores the result into every rank's output (out_ptrs[r] = base of
 * rank r's output already offset to these rows).  A second barrier makes the outputs complete.
 */
int fswiglu_down_scatter_bf16(const void* h, int64_t ldh, const void* w_down, int64_t ldw,
                              void* const* recv_ptrs, int world, int rank, int64_t rows_per_owner, int64_t M,
                              int64_t d, int64_t F, void* scratch, size_t scratch_bytes, void* stream);
int fswiglu_reduce_bcast_bf16(const void* recv_local, void* const* out_ptrs, int world, int64_t rows, int64_t cols,
                              int max_ctas, void* stream);

/*
 * Upper bound on the CTAs (= SMs, one persistent CTA each) the tiled GEMM kernels occupy; 0 restores
 * "all SMs".  Tensor-parallel callers reserve a few SMs for the communication kernels that run
 * beside the GEMMs: a persistent GEMM that holds every SM would keep a collective launched later
 * from starting until the GEMM ends, and a collective that got there first would delay some of the
 * GEMM's CTAs to the very end.  The setting belongs to the CURRENT device; the call returns the
 * previous value (or a negative status when the device cannot be used).  No counterpart in the
 * reference (single GPU).
 */
int fswiglu_set_max_ctas(int max_ctas);

/*
 * Device-side watchdog.  Kernels never spin forever: a wait that exceeds its limit records where it
 * gave up and the kernel unwinds.  This call synchronises `stream`, copies the status word of the
 * current device into *status (0 = healthy), clears it, and returns FSWIGLU_ERR_WATCHDOG if it
 * was non-zero.  The word of fswiglu_mlp_bf16_static is included once that entry point has been used.
 */
int fswiglu_device_status(uint32_t* status, void* stream);

/*
 * Limit, in microseconds, of every device-side wait in kernels launched from now on (process-wide;
 * default 2 000 000; limit_us <= 0 restores the default).  Returns the previous limit.  A wait that runs
 * out makes its kernel unwind (copies and tensor-core work in flight are drained, tensor memory is freed)
 * and shows up in fswiglu_device_status().  No counterpart in the reference, whose kernel has no waits
 * that can run out (csrc/SwiGLU/swiglu.cu:290-343 uses cp.async groups and __syncthreads).
 */
int64_t fswiglu_set_wait_limit_us(int64_t limit_us);

/*
 * Test aid for the time-out path, no counterpart in the reference.  After fswiglu_test_expire_next_wait(1)
 * the NEXT kernel launch of this library (one launch, then the switch is off again) is made so that one of
 * its bounded waits cannot be satisfied: the first CTA of a tiled GEMM leaves out one operand copy, the
 * small-batch kernel expects one more CTA at its hand-over than exists.  Nothing faults, traps or spins
 * without bound: the wait runs out after the limit above, the kernel unwinds and returns, the launch's
 * output is undefined and fswiglu_device_status() reports FSWIGLU_ERR_WATCHDOG with the site of the wait.
 * Use it with a limit of a few milliseconds.
 */
void fswiglu_test_expire_next_wait(int enable);

/*
 * Profiling aid for the small-batch kernel, no counterpart in the reference.  With a device buffer of
 * (number of SMs) x 8 x 8 bytes set, every CTA of the small-batch kernel leaves eight %globaltimer stamps
 * (nanoseconds) in it: set-up done, first phase-1 tile ready, phase-1 MMAs issued, hand-over signalled, first
 * phase-2 tile ready, phase-2 MMAs issued, phase-2 epilogue done, hand-over observed.  NULL switches it off
 * (the default); process-wide; the buffer must outlive the launches.
 */
void fswiglu_set_decode_trace(void* device_buffer);

/* Human-readable name of a status code returned by this library. */
const char* fswiglu_status_string(int status);

/*
 * Which tiled GEMM kernel a launch of the given problem takes on the current device, with the current SM
 * budget and environment: 0 = one-SM kernel (128-row tiles), 1 = two-SM kernel with 256-row tiles, 2 = two-SM
 * kernel with 512-row tiles; negative = status code.  gated != 0: gate-up problem (n_out = F output columns,
 * K = d); gated == 0: plain problem (down projection: n_out = d, K = F).  The small-batch path (M <= 64 through
 * fswiglu_mlp_bf16) is not covered.  For launch accounting, labels and tests; no reference counterpart.
 */
int fswiglu_plan_kernel(int64_t M, int64_t n_out, int64_t K, int gated);

/* Library version, "major.minor.patch". */
const char* fswiglu_version(void);

/* Number of kernels this library has launched in this process (for launch accounting). */
uint64_t fswiglu_launch_count(void);

#ifdef __cplusplus
}
#endif

#endif /* FSWIGLU_H_ */
