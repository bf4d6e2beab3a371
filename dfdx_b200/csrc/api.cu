// C ABI of the library (include/dfdx_b200.h) and the host-side lowering of dfdx's kernel traits to
// the canonical GemmProblem.  The lowering functions restate, call for call, the argument
// computation of `impl MatMat*Kernel for Cuda` (dfdx-core/src/tensor_ops/matmul/cuda_kernel.rs)
// — which strides are swapped for the transposed operands of the backward GEMMs, which batch
// strides are zero — so a Rust caller can hand over `Tensor::strides` untouched.
#include "common.cuh"
#include <atomic>
#include <mutex>
#include <cstdio>
#include <cstring>

namespace b200 {

size_t conv2d_workspace_bytes(int dtype, const b200_conv2d_op* o, int backward);
int conv2d_forward(int dtype, const b200_conv2d_op* o, const void* img, const size_t is[4], const void* filters,
                   void* out, void* ws, cudaStream_t stream);
size_t convtrans2d_workspace_bytes(int dtype, const b200_convtrans2d_op* o, int backward);
int convtrans2d_forward(int dtype, const b200_convtrans2d_op* o, const void* img, const void* filters, const size_t fs[4],
                        void* out, void* ws, cudaStream_t stream);
int convtrans2d_backward(int dtype, const b200_convtrans2d_op* o, const void* img, void* grad_img, const void* filters,
                         const size_t fs[4], void* grad_filters, const void* grad_out, void* ws, cudaStream_t stream);
size_t conv1d_workspace_bytes(int dtype, const b200_conv1d_op* o, int backward);
int conv1d_forward(int dtype, const b200_conv1d_op* o, const void* img, const size_t is[3], const void* filters, void* out,
                   void* ws, cudaStream_t stream);
int conv1d_backward(int dtype, const b200_conv1d_op* o, const void* img, void* grad_img, const void* filters,
                    const size_t fs[3], void* grad_filters, const void* grad_out, void* ws, cudaStream_t stream);
int conv2d_backward(int dtype, const b200_conv2d_op* o, const void* img, void* grad_img, const void* filters,
                    const size_t fs[4], void* grad_filters, const void* grad_out, void* ws, cudaStream_t stream);
int conv_noalloc_setup_device();
uint64_t conv_implicit_passes();
void tc_set_xform_mode(int mode);
void tc_set_tile_n(int bn);
void tc_set_mn_box5(int on);
void tc_set_pair_mode(int mode);
void tc_set_store_mode(int mode);
void conv_set_lowering(int grad_img_mode, size_t group_bytes);
void tc_set_split_mode(int mode);
void tc_set_capture_split(int on);
void tc_set_wait_limit(long long cycles);
void tc_set_max_ctas(int n);
void tc_set_tail_mode(int mode);
int tc_wait_selftest(long long limit, long long* cycles, cudaStream_t stream);

namespace {

constexpr int MAX_DEVICES = 64;
DeviceState g_dev[MAX_DEVICES];
std::mutex g_dev_mutex;
std::atomic<int> g_path{B200_PATH_AUTO};
std::atomic<uint64_t> g_launches{0}, g_tc_launches{0};
thread_local char t_cuda_err[256] = "";

bool valid_dtype(int d) { return d == B200_F32 || d == B200_F64 || d == B200_F16 || d == B200_AMP_F16; }

// matmul/mod.rs:316-325: legal 2-D stride pairs have at least one unit stride.
bool matrix_strides_ok(const size_t s[2]) { return s[0] == 1 || s[1] == 1; }

}  // namespace

DeviceState* device_state() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return nullptr;
  return g_dev[dev].ready ? &g_dev[dev] : nullptr;
}

int note_cuda_error(cudaError_t e, const char* where) {
  if (e == cudaSuccess) return B200_OK;
  snprintf(t_cuda_err, sizeof(t_cuda_err), "%s: %s (%s)", where, cudaGetErrorName(e), cudaGetErrorString(e));
  return B200_ERR_CUDA;
}

int current_path() { return g_path.load(); }

void count_launch(bool tensor) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (tensor) g_tc_launches.fetch_add(1, std::memory_order_relaxed);
}

// Batch folding: when rhs is shared by the whole batch and lhs / out are stacked with the row
// stride, (B, M, K) x (K, N) is one (B*M, K) x (K, N) GEMM (no partial M tiles per batch item).
static void fold_batch(GemmProblem& p) {
  if (p.red != 1) return;
  if (p.bias && p.bias_dim == 1) return;   // a per-row bias repeats per batch item
  if (p.b1 > 1 && p.b_b1 == 0 && p.a_b1 == p.m * p.a_r && p.c_b1 == p.m * p.c_r && p.a_r != 0 && p.c_r != 0 &&
      (p.b0 == 1)) {
    p.m *= p.b1; p.b1 = 1; p.a_b1 = p.c_b1 = 0;
  }
}

int run_gemm(const GemmProblem& p0, cudaStream_t stream) {
  if (p0.m == 0 || p0.n == 0 || p0.b0 == 0 || p0.b1 == 0) return B200_OK;
  if (!device_state()) return note_cuda_error(cudaErrorInitializationError, "b200_init not called on this device");
  GemmProblem p = p0;
  fold_batch(p);
  const int path = g_path.load();
  if (path == B200_PATH_SIMT || p.dtype == B200_F64 || p.k == 0) return launch_gemm_simt(p, stream);
  if (path == B200_PATH_TENSOR) return launch_gemm_tc(p, stream);
  // AUTO: tensor cores unless the problem is tiny (exact-FP32 SIMT keeps the reference's 1e-6
  // absolute tolerance on its small known-answer tests) or not TMA-addressable.
  const double work = (double)p.m * (double)p.n * (double)p.k * (double)p.red * (double)p.b0 * (double)p.b1;
  if (work >= 262144.0 && p.m >= 8 && p.n >= 8 && p.k >= 8 && tc_eligible(p)) {
    const int rc = launch_gemm_tc(p, stream);
    if (rc != B200_ERR_UNSUPPORTED) return rc;
  }
  return launch_gemm_simt(p, stream);
}

}  // namespace b200

using namespace b200;

// ------------------------------------------------------------------------------------------------
extern "C" {

int b200_init(int ordinal) {
  if (ordinal < 0 || ordinal >= MAX_DEVICES) return B200_ERR_SHAPE;
  int rc = note_cuda_error(cudaSetDevice(ordinal), "cudaSetDevice");
  if (rc) return rc;
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  DeviceState& d = g_dev[ordinal];
  if (d.ready) return B200_OK;
  cudaDeviceProp prop;
  if ((rc = note_cuda_error(cudaGetDeviceProperties(&prop, ordinal), "cudaGetDeviceProperties"))) return rc;
  if (prop.major != 10) {
    snprintf(t_cuda_err, sizeof(t_cuda_err), "device %d is sm_%d%d; this library contains sm_100a code only",
             ordinal, prop.major, prop.minor);
    return B200_ERR_UNSUPPORTED;
  }
  d.sm_count = prop.multiProcessorCount;
  if ((rc = note_cuda_error(cudaMalloc(&d.status, sizeof(int)), "cudaMalloc(status)"))) return rc;
  if ((rc = note_cuda_error(cudaMemset(d.status, 0, sizeof(int)), "cudaMemset(status)"))) return rc;
  if ((rc = note_cuda_error(cudaMalloc(&d.split_scratch, SPLIT_SCRATCH_BYTES), "cudaMalloc(split-K scratch)"))) return rc;
  d.split_scratch_bytes = SPLIT_SCRATCH_BYTES;
  if ((rc = note_cuda_error(cudaEventCreateWithFlags(&d.split_event, cudaEventDisableTiming), "cudaEventCreate"))) return rc;
  if ((rc = tc_setup_device())) return rc;
  if ((rc = attention_setup_device())) return rc;
  if ((rc = attention_bwd_setup_device())) return rc;
  if ((rc = rowwise_setup_device())) return rc;
  if ((rc = conv_noalloc_setup_device())) return rc;
  d.ready = true;
  return B200_OK;
}

const char* b200_strerror(int status) {
  switch (status) {
    case B200_OK: return "ok";
    case B200_ERR_SHAPE: return "shape mismatch";
    case B200_ERR_STRIDE: return "illegal strides (at least a single stride must be 1; output/batch stride must be non-zero)";
    case B200_ERR_DTYPE: return "unknown dtype";
    case B200_ERR_NULL: return "null pointer";
    case B200_ERR_WORKSPACE: return "workspace too small";
    case B200_ERR_CUDA: return "CUDA error (see b200_last_cuda_error)";
    case B200_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait expired";
    case B200_ERR_UNSUPPORTED: return "unsupported on the requested path";
    case B200_ERR_NOT_CONTIGUOUS: return "image & filter inputs to conv2d must be contiguous";
    case B200_ERR_LIMIT: return "request exceeds a fixed capacity";
    default: return "unknown status";
  }
}

const char* b200_last_cuda_error(void) { return t_cuda_err; }

int b200_device_status(void* stream) {
  DeviceState* d = device_state();
  if (!d) return B200_ERR_CUDA;
  int rc = note_cuda_error(cudaStreamSynchronize((cudaStream_t)stream), "cudaStreamSynchronize");
  if (rc) return rc;
  int v = 0;
  if ((rc = note_cuda_error(cudaMemcpy(&v, d->status, sizeof(int), cudaMemcpyDeviceToHost), "cudaMemcpy(status)"))) return rc;
  if (v) cudaMemset(d->status, 0, sizeof(int));
  return v;
}

int b200_set_path(int path) {
  if (path < B200_PATH_AUTO || path > B200_PATH_TENSOR) return B200_ERR_UNSUPPORTED;
  g_path.store(path);
  return B200_OK;
}

/* Testing hook: how the `small` half of the 3xTF32 operand split is stored: 1 (default) as computed (the tensor
 * core keeps its top 19 bits), 0 rounded to tf32 first.  Both give results inside the f32 tolerance. */
int b200_set_tf32_split_mode(int mode) {
  if (mode != 0 && mode != 1) return B200_ERR_UNSUPPORTED;
  tc_set_xform_mode(mode);
  return B200_OK;
}

/* Testing hook: force the N extent of the tensor-core tile (64, 128 or 256); 0 restores the heuristic. */
int b200_set_tile_n(int bn) {
  if (bn != 0 && bn != 64 && bn != 128 && bn != 256 && bn != 512) return B200_ERR_UNSUPPORTED;
  tc_set_tile_n(bn);
  return B200_OK;
}

/* Testing hook: 1 (default) loads MN-major operands with one 5-D TMA box per stage where the extent is a
 * whole number of column chunks; 0 always uses one 4-D box per chunk. */
int b200_set_mn_single_box(int on) {
  tc_set_mn_box5(on ? 1 : 0);
  return B200_OK;
}

/* Testing hook: 1 (default) single-CTA tensor-core kernels only, 0 planner's choice, 2 forces the CTA-pair
 * kernels wherever the output is wider than 128 columns. */
int b200_set_cta_pair_mode(int mode) {
  if (mode < 0 || mode > 2) return B200_ERR_UNSUPPORTED;
  tc_set_pair_mode(mode);
  return B200_OK;
}

/* Testing hook: lowering of the convolution data gradient (see the header). */
int b200_set_conv_lowering(int grad_img_mode, size_t group_bytes) {
  if (grad_img_mode < 0 || grad_img_mode > 2) return B200_ERR_UNSUPPORTED;
  conv_set_lowering(grad_img_mode, group_bytes);
  return B200_OK;
}
/* Testing hook: epilogue store orientation of the tensor-core kernels: 0 (default) planner's choice,
 * 1 row stores only, 2 column stores wherever the output allows. */
int b200_set_store_mode(int mode) {
  if (mode < 0 || mode > 2) return B200_ERR_UNSUPPORTED;
  tc_set_store_mode(mode);
  return B200_OK;
}

/* Testing hook: split-K of the f32 tensor-core kernel: 0 (default) planner's choice, 1 never, n in 2..64 forces
 * n K-slices on single-batch problems. */
int b200_set_split_k(int mode) {
  if (mode < -1 || mode > 64) return B200_ERR_UNSUPPORTED;
  tc_set_split_mode(mode);
  return B200_OK;
}

/* f16 split-K inside stream captures: 0 (default) a GEMM enqueued on a capturing stream runs unsplit, 1 it may
 * use the device's split-K scratch (the caller orders graph replays against all other use of the library). */
int b200_set_capture_split_k(int on) {
  tc_set_capture_split(on);
  return B200_OK;
}

/* Upper bound on the grids of the persistent tensor-core GEMM kernels (0 = one CTA per SM). */
int b200_set_max_ctas(int n) {
  if (n < 0) return B200_ERR_UNSUPPORTED;
  tc_set_max_ctas(n);
  return B200_OK;
}

/* Testing hook: 0 (default) the planner may cut the tiles of a last, partial wave along K; 1 never. */
int b200_set_tail_split(int mode) {
  if (mode != 0 && mode != 1) return B200_ERR_UNSUPPORTED;
  tc_set_tail_mode(mode);
  return B200_OK;
}

/* Testing hook: clock budget of the device-side waits of the tensor-core GEMM kernels (0 = by problem size). */
int b200_set_wait_limit(long long cycles) {
  if (cycles < 0) return B200_ERR_UNSUPPORTED;
  tc_set_wait_limit(cycles);
  return B200_OK;
}

/* Testing hook: a one-CTA kernel whose only wait can never be satisfied (see the header). */
int b200_selftest_bounded_wait(long long limit_cycles, long long* waited_cycles, void* stream) {
  if (limit_cycles < 0) return B200_ERR_UNSUPPORTED;
  return tc_wait_selftest(limit_cycles, waited_cycles, (cudaStream_t)stream);
}

uint64_t b200_launch_count(void) { return g_launches.load(); }
uint64_t b200_tensor_launch_count(void) { return g_tc_launches.load(); }
uint64_t b200_conv_implicit_count(void) { return conv_implicit_passes(); }

// ---- Cuda::gemm / Cuda::gemm_batch ---------------------------------------------------------------
int b200_gemm(int dtype, size_t m, size_t k, size_t n, const void* lhs, const size_t ls[2], const void* rhs,
              const size_t rs[2], double beta, void* out, const size_t os[2], void* stream) {
  if (!valid_dtype(dtype)) return B200_ERR_DTYPE;
  if (!ls || !rs || !os) return B200_ERR_NULL;
  if (m && n && (!out || (k && (!lhs || !rhs)))) return B200_ERR_NULL;
  if (!matrix_strides_ok(ls) || !matrix_strides_ok(rs) || !matrix_strides_ok(os)) return B200_ERR_STRIDE;
  if (beta != 0.0 && beta != 1.0) return B200_ERR_UNSUPPORTED;
  GemmProblem p;
  p.dtype = dtype; p.beta = beta != 0.0; p.m = m; p.k = k; p.n = n;
  p.a = lhs; p.a_r = ls[0]; p.a_c = ls[1];
  p.b = rhs; p.b_r = rs[0]; p.b_c = rs[1];
  p.c = out; p.c_r = os[0]; p.c_c = os[1];
  return run_gemm(p, (cudaStream_t)stream);
}

int b200_gemm_batch(int dtype, size_t batch, size_t m, size_t k, size_t n, const void* lhs, const size_t ls[3],
                    const void* rhs, const size_t rs[3], double beta, void* out, const size_t os[3], void* stream) {
  if (!valid_dtype(dtype)) return B200_ERR_DTYPE;
  if (!ls || !rs || !os) return B200_ERR_NULL;
  if (batch && m && n && (!out || (k && (!lhs || !rhs)))) return B200_ERR_NULL;
  if (os[0] == 0) return B200_ERR_STRIDE;  // assert_ne!(out_strides[0], 0), cuda_kernel.rs:208
  if (!matrix_strides_ok(ls + 1) || !matrix_strides_ok(rs + 1) || !matrix_strides_ok(os + 1)) return B200_ERR_STRIDE;
  if (beta != 0.0 && beta != 1.0) return B200_ERR_UNSUPPORTED;
  GemmProblem p;
  p.dtype = dtype; p.beta = beta != 0.0; p.b1 = batch; p.m = m; p.k = k; p.n = n;
  p.a = lhs; p.a_b1 = ls[0]; p.a_r = ls[1]; p.a_c = ls[2];
  p.b = rhs; p.b_b1 = rs[0]; p.b_r = rs[1]; p.b_c = rs[2];
  p.c = out; p.c_b1 = os[0]; p.c_r = os[1]; p.c_c = os[2];
  return run_gemm(p, (cudaStream_t)stream);
}

// The stream that takes the grad_lhs GEMM of a backward pass.  dfdx enqueues it on the device's `par_stream`
// and the grad_rhs GEMM on the default stream (cuda_kernel.rs:282-310, :354-386, :432-460, :535-566), joining the two
// streams itself before (`par_stream.wait_for_default()`) and after (`dev.wait_for(par_stream)`).  A NULL
// par_stream means the caller has no second stream: both GEMMs then go to `stream`.
static void* lhs_stream_of(void* stream, void* par_stream) { return par_stream ? par_stream : stream; }

// ---- MatMatKernel (cuda_kernel.rs:244-312) -------------------------------------------------------
int b200_matmat_forward(int dtype, size_t m, size_t k, size_t n, const void* lhs, const size_t ls[2],
                        const void* rhs, const size_t rs[2], void* out, void* stream) {
  const size_t os[2] = {n, 1};
  return b200_gemm(dtype, m, k, n, lhs, ls, rhs, rs, 0.0, out, os, stream);
}

int b200_matmat_backward(int dtype, size_t m, size_t k, size_t n, const void* lhs, const size_t ls[2],
                         void* grad_lhs, const void* rhs, const size_t rs[2], void* grad_rhs,
                         const void* grad_out, void* stream, void* par_stream) {
  if (!ls || !rs) return B200_ERR_NULL;
  const size_t os[2] = {n, 1};
  int rc = B200_OK;
  if (grad_lhs) {  // grad_lhs += grad_out * rhs^T
    const size_t rs_t[2] = {rs[1], rs[0]};
    if ((rc = b200_gemm(dtype, m, n, k, grad_out, os, rhs, rs_t, 1.0, grad_lhs, ls, lhs_stream_of(stream, par_stream)))) return rc;
  }
  if (grad_rhs) {  // grad_rhs += lhs^T * grad_out
    const size_t ls_t[2] = {ls[1], ls[0]};
    rc = b200_gemm(dtype, k, m, n, lhs, ls_t, grad_out, os, 1.0, grad_rhs, rs, stream);
  }
  return rc;
}

// ---- MatMatBrKernel (cuda_kernel.rs:319-388) -----------------------------------------------------
int b200_matmat_br_forward(int dtype, size_t batch, size_t m, size_t k, size_t n, const void* lhs,
                           const size_t ls[3], const void* rhs, const size_t rs[2], void* out, void* stream) {
  if (!ls || !rs) return B200_ERR_NULL;
  const size_t rs3[3] = {0, rs[0], rs[1]};
  const size_t os[3] = {m * n, n, 1};
  return b200_gemm_batch(dtype, batch, m, k, n, lhs, ls, rhs, rs3, 0.0, out, os, stream);
}

static int matmat_br_backward_beta(int dtype, size_t batch, size_t m, size_t k, size_t n, const void* lhs,
                                   const size_t ls[3], void* grad_lhs, const void* rhs, const size_t rs[2],
                                   void* grad_rhs, const void* grad_out, void* stream, void* lhs_stream, int beta) {
  if (!valid_dtype(dtype)) return B200_ERR_DTYPE;
  if (!ls || !rs) return B200_ERR_NULL;
  if (!matrix_strides_ok(ls + 1) || !matrix_strides_ok(rs)) return B200_ERR_STRIDE;
  int rc = B200_OK;
  if (grad_rhs && batch && k && n) {
    // grad_rhs (+)= sum_b lhs_b^T * grad_out_b : one launch, the batch is an outer reduction index.
    if (!lhs || !grad_out) return B200_ERR_NULL;
    GemmProblem p;
    p.dtype = dtype; p.beta = beta; p.red = batch; p.m = k; p.k = m; p.n = n;
    p.a = lhs; p.a_red = ls[0]; p.a_r = ls[2]; p.a_c = ls[1];
    p.b = grad_out; p.b_red = m * n; p.b_r = n; p.b_c = 1;
    p.c = grad_rhs; p.c_r = rs[0]; p.c_c = rs[1];
    if ((rc = run_gemm(p, (cudaStream_t)stream))) return rc;
  }
  if (grad_lhs) {  // grad_lhs (+)= grad_out * rhs^T, rhs broadcast over the batch
    const size_t os[3] = {m * n, n, 1};
    const size_t rs_t[3] = {0, rs[1], rs[0]};
    rc = b200_gemm_batch(dtype, batch, m, n, k, grad_out, os, rhs, rs_t, beta ? 1.0 : 0.0, grad_lhs, ls, lhs_stream);
  }
  return rc;
}

int b200_matmat_br_backward(int dtype, size_t batch, size_t m, size_t k, size_t n, const void* lhs,
                            const size_t ls[3], void* grad_lhs, const void* rhs, const size_t rs[2],
                            void* grad_rhs, const void* grad_out, void* stream, void* par_stream) {
  return matmat_br_backward_beta(dtype, batch, m, k, n, lhs, ls, grad_lhs, rhs, rs, grad_rhs, grad_out, stream,
                                 lhs_stream_of(stream, par_stream), 1);
}

int b200_matmat_br_grad_rhs_f32(int dtype, size_t batch, size_t m, size_t k, size_t n, const void* lhs, const size_t ls[3],
                                const void* grad_out, float* grad_rhs, const size_t gs[2], void* stream) {
  if (!valid_dtype(dtype)) return B200_ERR_DTYPE;
  if (dtype != B200_F16 && dtype != B200_AMP_F16) return B200_ERR_UNSUPPORTED;
  if (!ls || !gs) return B200_ERR_NULL;
  if (!matrix_strides_ok(ls + 1) || !matrix_strides_ok(gs)) return B200_ERR_STRIDE;
  if (batch == 0 || m == 0 || k == 0 || n == 0) return B200_OK;
  if (!lhs || !grad_out || !grad_rhs) return B200_ERR_NULL;
  if ((k > 1 && gs[0] == 0) || (n > 1 && gs[1] == 0)) return B200_ERR_STRIDE;   // every element owns its storage
  if (!device_state()) return note_cuda_error(cudaErrorInitializationError, "b200_init not called on this device");
  GemmProblem p;
  p.dtype = dtype; p.beta = 1; p.acc32 = true; p.red = batch; p.m = k; p.k = m; p.n = n;
  p.a = lhs; p.a_red = ls[0]; p.a_r = ls[2]; p.a_c = ls[1];
  p.b = grad_out; p.b_red = m * n; p.b_r = n; p.b_c = 1;
  p.c = grad_rhs; p.c_r = gs[0]; p.c_c = gs[1];
  return launch_gemm_tc_acc32(p, (cudaStream_t)stream);
}

int b200_matmat_br_backward_overwrite(int dtype, size_t batch, size_t m, size_t k, size_t n, const void* lhs,
                                      const size_t ls[3], void* grad_lhs, const void* rhs, const size_t rs[2],
                                      void* grad_rhs, const void* grad_out, void* stream) {
  // writing instead of accumulating is only the same thing when no two elements of a view share storage
  if (ls && grad_lhs && ((batch > 1 && ls[0] == 0) || (m > 1 && ls[1] == 0) || (k > 1 && ls[2] == 0))) return B200_ERR_STRIDE;
  if (rs && grad_rhs && ((k > 1 && rs[0] == 0) || (n > 1 && rs[1] == 0))) return B200_ERR_STRIDE;
  return matmat_br_backward_beta(dtype, batch, m, k, n, lhs, ls, grad_lhs, rhs, rs, grad_rhs, grad_out, stream, stream, 0);
}

// ---- MatMatBatch3Kernel (cuda_kernel.rs:395-462) -------------------------------------------------
int b200_matmat_batch3_forward(int dtype, size_t batch, size_t m, size_t k, size_t n, const void* lhs,
                               const size_t ls[3], const void* rhs, const size_t rs[3], void* out, void* stream) {
  if (!ls || !rs) return B200_ERR_NULL;
  if (ls[0] == 0 || rs[0] == 0) return B200_ERR_STRIDE;  // assert_ne!, cuda_kernel.rs:400-401
  const size_t os[3] = {m * n, n, 1};
  return b200_gemm_batch(dtype, batch, m, k, n, lhs, ls, rhs, rs, 0.0, out, os, stream);
}

int b200_matmat_batch3_backward(int dtype, size_t batch, size_t m, size_t k, size_t n, const void* lhs,
                                const size_t ls[3], void* grad_lhs, const void* rhs, const size_t rs[3],
                                void* grad_rhs, const void* grad_out, void* stream, void* par_stream) {
  if (!ls || !rs) return B200_ERR_NULL;
  const size_t os[3] = {m * n, n, 1};
  int rc = B200_OK;
  if (grad_lhs) {
    const size_t rs_t[3] = {rs[0], rs[2], rs[1]};
    if ((rc = b200_gemm_batch(dtype, batch, m, n, k, grad_out, os, rhs, rs_t, 1.0, grad_lhs, ls,
                              lhs_stream_of(stream, par_stream)))) return rc;
  }
  if (grad_rhs) {
    const size_t ls_t[3] = {ls[0], ls[2], ls[1]};
    rc = b200_gemm_batch(dtype, batch, k, m, n, lhs, ls_t, grad_out, os, 1.0, grad_rhs, rs, stream);
  }
  return rc;
}

// ---- MatMatBatch4Kernel (cuda_kernel.rs:469-568) -------------------------------------------------
static int gemm_batch2(int dtype, size_t b0, size_t b1, size_t m, size_t k, size_t n, const void* lhs,
                       const size_t ls[4], const void* rhs, const size_t rs[4], int beta, void* out,
                       const size_t os[4], void* stream, const b200_epilogue* ep = nullptr) {
  if (!valid_dtype(dtype)) return B200_ERR_DTYPE;
  if (ep && (ep->activation != B200_ACT_NONE && ep->activation != B200_ACT_RELU)) return B200_ERR_UNSUPPORTED;
  if (ep && beta) return B200_ERR_UNSUPPORTED;
  if (b0 && b1 && m && n && (!out || (k && (!lhs || !rhs)))) return B200_ERR_NULL;
  if (!matrix_strides_ok(ls + 2) || !matrix_strides_ok(rs + 2) || !matrix_strides_ok(os + 2)) return B200_ERR_STRIDE;
  if ((b0 > 1 && os[0] == 0) || (b1 > 1 && os[1] == 0)) return B200_ERR_STRIDE;
  GemmProblem p;
  p.dtype = dtype; p.beta = beta; p.b0 = b0; p.b1 = b1; p.m = m; p.k = k; p.n = n;
  p.a = lhs; p.a_b0 = ls[0]; p.a_b1 = ls[1]; p.a_r = ls[2]; p.a_c = ls[3];
  p.b = rhs; p.b_b0 = rs[0]; p.b_b1 = rs[1]; p.b_r = rs[2]; p.b_c = rs[3];
  p.c = out; p.c_b0 = os[0]; p.c_b1 = os[1]; p.c_r = os[2]; p.c_c = os[3];
  if (ep) { p.alpha = ep->alpha; p.bias = ep->bias; p.bias_dim = 0; p.act = ep->activation; }
  return run_gemm(p, (cudaStream_t)stream);
}

// ---- fused epilogues ------------------------------------------------------------------------------
int b200_gemm_batch_fused(int dtype, size_t batch0, size_t batch1, size_t m, size_t k, size_t n, const void* lhs,
                          const size_t ls[4], const void* rhs, const size_t rs[4], const b200_epilogue* ep,
                          void* out, const size_t os[4], void* stream) {
  if (!ls || !rs || !os) return B200_ERR_NULL;
  return gemm_batch2(dtype, batch0, batch1, m, k, n, lhs, ls, rhs, rs, 0, out, os, stream, ep);
}

int b200_linear_forward(int dtype, size_t batch, size_t m, size_t i, size_t o, const void* x, const size_t xs[3],
                        const void* weight, const size_t ws[2], const void* bias, int activation, void* out,
                        void* stream) {
  if (!xs || !ws) return B200_ERR_NULL;
  const size_t ls[4] = {0, xs[0], xs[1], xs[2]};
  const size_t rs[4] = {0, 0, ws[0], ws[1]};
  const size_t os[4] = {batch * m * o, m * o, o, 1};
  b200_epilogue ep;
  ep.alpha = 1.0; ep.bias = bias; ep.activation = activation;
  return gemm_batch2(dtype, 1, batch, m, i, o, x, ls, weight, rs, 0, out, os, stream, &ep);
}

int b200_matmat_batch4_forward_scaled(int dtype, size_t batch, size_t seq, size_t m, size_t k, size_t n,
                                      const void* lhs, const size_t ls[4], const void* rhs, const size_t rs[4],
                                      double alpha, void* out, void* stream) {
  if (!ls || !rs) return B200_ERR_NULL;
  if (ls[0] == 0 || rs[0] == 0 || ls[1] == 0 || rs[1] == 0) return B200_ERR_STRIDE;
  const size_t os[4] = {seq * m * n, m * n, n, 1};
  b200_epilogue ep;
  ep.alpha = alpha; ep.bias = nullptr; ep.activation = B200_ACT_NONE;
  return gemm_batch2(dtype, batch, seq, m, k, n, lhs, ls, rhs, rs, 0, out, os, stream, &ep);
}

int b200_attention_forward(int dtype, size_t batch, size_t heads, size_t s1, size_t s2, size_t d, const void* q,
                           const size_t qs[4], const void* k, const size_t ks[4], const void* v, const size_t vs[4],
                           double alpha, void* out, const size_t os[4], float* lse, void* stream) {
  if (!valid_dtype(dtype)) return B200_ERR_DTYPE;
  if (!qs || !ks || !vs || !os) return B200_ERR_NULL;
  if (batch && heads && s1 && (!q || !k || !v || !out)) return B200_ERR_NULL;
  int64_t q4[4], k4[4], v4[4], o4[4];
  for (int i = 0; i < 4; ++i) { q4[i] = (int64_t)qs[i]; k4[i] = (int64_t)ks[i]; v4[i] = (int64_t)vs[i]; o4[i] = (int64_t)os[i]; }
  return attention_forward(dtype, (int64_t)batch, (int64_t)heads, (int64_t)s1, (int64_t)s2, (int64_t)d, q, q4, k, k4, v,
                           v4, alpha, out, o4, lse, (cudaStream_t)stream);
}

int b200_layer_norm_forward(int dtype, size_t rows, size_t cols, const void* x, size_t x_ld, const void* gamma, const void* beta,
                            double epsilon, void* y, size_t y_ld, float* stats, void* stream) {
  if (!valid_dtype(dtype)) return B200_ERR_DTYPE;
  if (rows && cols && (!x || !y)) return B200_ERR_NULL;
  if (rows > 1 && (x_ld < cols || y_ld < cols)) return B200_ERR_STRIDE;
  return layer_norm_forward(dtype, (int64_t)rows, (int64_t)cols, x, (int64_t)x_ld, gamma, beta, epsilon, y, (int64_t)y_ld, stats,
                            (cudaStream_t)stream);
}

int b200_layer_norm_backward(int dtype, size_t rows, size_t cols, const void* x, size_t x_ld, const void* gamma,
                             const float* stats, const void* grad_out, size_t grad_out_ld, void* grad_x, size_t grad_x_ld,
                             int accumulate_x, float* grad_gamma, float* grad_beta, void* stream) {
  if (!valid_dtype(dtype)) return B200_ERR_DTYPE;
  if (rows && cols && (!x || !grad_out || !stats)) return B200_ERR_NULL;
  if (rows > 1 && (x_ld < cols || grad_out_ld < cols || (grad_x && grad_x_ld < cols))) return B200_ERR_STRIDE;
  return layer_norm_backward(dtype, (int64_t)rows, (int64_t)cols, x, (int64_t)x_ld, gamma, stats, grad_out, (int64_t)grad_out_ld,
                             grad_x, (int64_t)grad_x_ld, accumulate_x, grad_gamma, grad_beta, nullptr, (cudaStream_t)stream);
}

int b200_layer_norm_backward_sum(int dtype, size_t rows, size_t cols, const void* x, size_t x_ld, const void* gamma,
                                 const float* stats, const void* grad_out, size_t grad_out_ld, void* grad_x, size_t grad_x_ld,
                                 float* grad_gamma, float* grad_beta, float* grad_x_sum, void* stream) {
  if (!valid_dtype(dtype)) return B200_ERR_DTYPE;
  if (rows && cols && (!x || !grad_out || !stats || !grad_x || !grad_x_sum)) return B200_ERR_NULL;
  if (rows > 1 && (x_ld < cols || grad_out_ld < cols || grad_x_ld < cols)) return B200_ERR_STRIDE;
  return layer_norm_backward(dtype, (int64_t)rows, (int64_t)cols, x, (int64_t)x_ld, gamma, stats, grad_out, (int64_t)grad_out_ld,
                             grad_x, (int64_t)grad_x_ld, 0, grad_gamma, grad_beta, grad_x_sum, (cudaStream_t)stream);
}

int b200_add_layer_norm_forward(int dtype, size_t rows, size_t cols, const void* a, size_t a_ld, const void* b, size_t b_ld,
                                void* sum, size_t sum_ld, const void* gamma, const void* beta, double epsilon, void* y,
                                size_t y_ld, float* stats, void* stream) {
  if (!valid_dtype(dtype)) return B200_ERR_DTYPE;
  if (rows && cols && (!a || !b || !sum || !y)) return B200_ERR_NULL;
  if (rows > 1 && (a_ld < cols || b_ld < cols || sum_ld < cols || y_ld < cols)) return B200_ERR_STRIDE;
  return add_layer_norm_forward(dtype, (int64_t)rows, (int64_t)cols, a, (int64_t)a_ld, b, (int64_t)b_ld, sum, (int64_t)sum_ld,
                                gamma, beta, epsilon, y, (int64_t)y_ld, stats, (cudaStream_t)stream);
}

int b200_relu_backward_bias_grad(int dtype, size_t rows, size_t cols, const void* y, size_t y_ld, void* grad, size_t grad_ld,
                                 float* grad_bias, void* stream) {
  if (!valid_dtype(dtype)) return B200_ERR_DTYPE;
  if (rows && cols && (!y || !grad)) return B200_ERR_NULL;
  if (rows > 1 && (y_ld < cols || grad_ld < cols)) return B200_ERR_STRIDE;
  return relu_backward_column_sum(dtype, (int64_t)rows, (int64_t)cols, y, (int64_t)y_ld, grad, (int64_t)grad_ld, grad_bias,
                                  (cudaStream_t)stream);
}

int b200_bias_grad(int dtype, size_t rows, size_t cols, const void* grad_out, size_t grad_out_ld, float* grad_bias, void* stream) {
  if (!valid_dtype(dtype)) return B200_ERR_DTYPE;
  if (rows && cols && (!grad_out || !grad_bias)) return B200_ERR_NULL;
  if (rows > 1 && grad_out_ld < cols) return B200_ERR_STRIDE;
  return column_sum(dtype, (int64_t)rows, (int64_t)cols, grad_out, (int64_t)grad_out_ld, grad_bias, (cudaStream_t)stream);
}

int b200_softmax_forward(int dtype, size_t rows, size_t cols, const void* x, size_t x_ld, double alpha, void* y, size_t y_ld,
                         void* stream) {
  if (!valid_dtype(dtype)) return B200_ERR_DTYPE;
  if (rows && cols && (!x || !y)) return B200_ERR_NULL;
  if (rows > 1 && (x_ld < cols || y_ld < cols)) return B200_ERR_STRIDE;
  return softmax_forward(dtype, (int64_t)rows, (int64_t)cols, x, (int64_t)x_ld, alpha, y, (int64_t)y_ld, (cudaStream_t)stream);
}

int b200_softmax_backward(int dtype, size_t rows, size_t cols, const void* y, size_t y_ld, const void* grad_out,
                          size_t grad_out_ld, double alpha, void* grad_x, size_t grad_x_ld, int accumulate, void* stream) {
  if (!valid_dtype(dtype)) return B200_ERR_DTYPE;
  if (rows && cols && (!y || !grad_out || !grad_x)) return B200_ERR_NULL;
  if (rows > 1 && (y_ld < cols || grad_out_ld < cols || grad_x_ld < cols)) return B200_ERR_STRIDE;
  return softmax_backward(dtype, (int64_t)rows, (int64_t)cols, y, (int64_t)y_ld, grad_out, (int64_t)grad_out_ld, alpha, grad_x,
                          (int64_t)grad_x_ld, accumulate, (cudaStream_t)stream);
}

size_t b200_attention_backward_workspace_bytes(size_t batch, size_t heads, size_t s1) {
  return attention_backward_workspace_bytes((int64_t)batch, (int64_t)heads, (int64_t)s1);
}

int b200_attention_backward(int dtype, size_t batch, size_t heads, size_t s1, size_t s2, size_t d, const void* q,
                            const size_t qs[4], const void* k, const size_t ks[4], const void* v, const size_t vs[4],
                            double alpha, const void* out, const size_t os[4], const float* lse, const void* grad_out,
                            const size_t gs[4], void* grad_q, const size_t gqs[4], void* grad_k, const size_t gks[4],
                            void* grad_v, const size_t gvs[4], int accumulate, void* workspace, size_t workspace_bytes,
                            void* stream) {
  if (!valid_dtype(dtype)) return B200_ERR_DTYPE;
  if (!qs || !ks || !vs || !os || !gs || !gqs || !gks || !gvs) return B200_ERR_NULL;
  if (batch && heads && s1 && s2 && d && (!q || !k || !v || !out || !lse || !grad_out || !workspace)) return B200_ERR_NULL;
  int64_t a[8][4];
  const size_t* src[8] = {qs, ks, vs, os, gs, gqs, gks, gvs};
  for (int t = 0; t < 8; ++t)
    for (int i = 0; i < 4; ++i) a[t][i] = (int64_t)src[t][i];
  return attention_backward(dtype, (int64_t)batch, (int64_t)heads, (int64_t)s1, (int64_t)s2, (int64_t)d, q, a[0], k, a[1], v,
                            a[2], alpha, out, a[3], lse, grad_out, a[4], grad_q, a[5], grad_k, a[6], grad_v, a[7],
                            accumulate, workspace, workspace_bytes, (cudaStream_t)stream);
}

int b200_matmat_batch4_forward(int dtype, size_t batch, size_t seq, size_t m, size_t k, size_t n,
                               const void* lhs, const size_t ls[4], const void* rhs, const size_t rs[4],
                               void* out, void* stream) {
  if (!ls || !rs) return B200_ERR_NULL;
  if (ls[0] == 0 || rs[0] == 0 || ls[1] == 0 || rs[1] == 0) return B200_ERR_STRIDE;  // cuda_kernel.rs:474-477
  const size_t os[4] = {seq * m * n, m * n, n, 1};
  return gemm_batch2(dtype, batch, seq, m, k, n, lhs, ls, rhs, rs, 0, out, os, stream);
}

int b200_matmat_batch4_backward(int dtype, size_t batch, size_t seq, size_t m, size_t k, size_t n,
                                const void* lhs, const size_t ls[4], void* grad_lhs, const void* rhs,
                                const size_t rs[4], void* grad_rhs, const void* grad_out, void* stream,
                                void* par_stream) {
  if (!ls || !rs) return B200_ERR_NULL;
  const size_t os[4] = {seq * m * n, m * n, n, 1};
  int rc = B200_OK;
  if (grad_lhs) {
    const size_t rs_t[4] = {rs[0], rs[1], rs[3], rs[2]};
    if ((rc = gemm_batch2(dtype, batch, seq, m, n, k, grad_out, os, rhs, rs_t, 1, grad_lhs, ls,
                          lhs_stream_of(stream, par_stream)))) return rc;
  }
  if (grad_rhs) {
    const size_t ls_t[4] = {ls[0], ls[1], ls[3], ls[2]};
    rc = gemm_batch2(dtype, batch, seq, k, m, n, lhs, ls_t, grad_out, os, 1, grad_rhs, rs, stream);
  }
  return rc;
}

// ---- conv2d ---------------------------------------------------------------------------------------
static int check_conv_op(const b200_conv2d_op* op) {
  if (!op) return B200_ERR_NULL;
  if (!op->groups || !op->stride || !op->dilation || !op->kernel) return B200_ERR_SHAPE;
  if (op->chan_in % op->groups || op->chan_out % op->groups) return B200_ERR_SHAPE;  // conv2d/mod.rs:281-286
  return B200_OK;
}

size_t b200_conv2d_workspace_bytes(int dtype, const b200_conv2d_op* op, int backward) {
  if (check_conv_op(op) || !valid_dtype(dtype)) return 0;
  return conv2d_workspace_bytes(dtype, op, backward);
}

int b200_conv2d_forward(int dtype, const b200_conv2d_op* op, const void* img, const size_t img_strides[4],
                        const void* filters, void* out, void* workspace, size_t workspace_bytes, void* stream) {
  if (!valid_dtype(dtype)) return B200_ERR_DTYPE;
  int rc = check_conv_op(op);
  if (rc) return rc;
  if (!img_strides) return B200_ERR_NULL;
  const size_t need = conv2d_workspace_bytes(dtype, op, 0);
  if (need == ~(size_t)0) return B200_ERR_LIMIT;             // the geometry's element counts overflow
  if (need == 0) return B200_OK;
  if (!img || !filters || !out || !workspace) return B200_ERR_NULL;
  if (workspace_bytes < need) return B200_ERR_WORKSPACE;
  if (!device_state()) return note_cuda_error(cudaErrorInitializationError, "b200_init not called on this device");
  return conv2d_forward(dtype, op, img, img_strides, filters, out, workspace, (cudaStream_t)stream);
}

int b200_conv2d_backward(int dtype, const b200_conv2d_op* op, const void* img, void* grad_img,
                         const void* filters, const size_t filters_strides[4], void* grad_filters,
                         const void* grad_out, void* workspace, size_t workspace_bytes, void* stream,
                         void* par_stream) {
  (void)par_stream;
  if (!valid_dtype(dtype)) return B200_ERR_DTYPE;
  int rc = check_conv_op(op);
  if (rc) return rc;
  if (!filters_strides) return B200_ERR_NULL;
  const size_t need = conv2d_workspace_bytes(dtype, op, 1);
  if (need == ~(size_t)0) return B200_ERR_LIMIT;             // the geometry's element counts overflow
  if (need == 0) return B200_OK;
  if (!img || !filters || !grad_out || !workspace) return B200_ERR_NULL;
  if (workspace_bytes < need) return B200_ERR_WORKSPACE;
  if (!device_state()) return note_cuda_error(cudaErrorInitializationError, "b200_init not called on this device");
  return conv2d_backward(dtype, op, img, grad_img, filters, filters_strides, grad_filters, grad_out, workspace,
                         (cudaStream_t)stream);
}

// ---- convtrans2d -----------------------------------------------------------------------------------
size_t b200_convtrans2d_workspace_bytes(int dtype, const b200_convtrans2d_op* op, int backward) {
  if (check_conv_op(op) || !valid_dtype(dtype)) return 0;
  return convtrans2d_workspace_bytes(dtype, op, backward);
}

int b200_convtrans2d_forward(int dtype, const b200_convtrans2d_op* op, const void* img, const void* filters,
                             const size_t filters_strides[4], void* out, void* workspace, size_t workspace_bytes,
                             void* stream) {
  if (!valid_dtype(dtype)) return B200_ERR_DTYPE;
  int rc = check_conv_op(op);
  if (rc) return rc;
  if (!filters_strides) return B200_ERR_NULL;
  const size_t need = convtrans2d_workspace_bytes(dtype, op, 0);
  if (need == ~(size_t)0) return B200_ERR_LIMIT;             // the geometry's element counts overflow
  if (need == 0 || op->batch * op->chan_out * op->h_out * op->w_out == 0) return B200_OK;
  if (!img || !filters || !out || !workspace) return B200_ERR_NULL;
  if (workspace_bytes < need) return B200_ERR_WORKSPACE;
  if (!device_state()) return note_cuda_error(cudaErrorInitializationError, "b200_init not called on this device");
  return convtrans2d_forward(dtype, op, img, filters, filters_strides, out, workspace, (cudaStream_t)stream);
}

int b200_convtrans2d_backward(int dtype, const b200_convtrans2d_op* op, const void* img, void* grad_img,
                              const void* filters, const size_t filters_strides[4], void* grad_filters,
                              const void* grad_out, void* workspace, size_t workspace_bytes, void* stream,
                              void* par_stream) {
  (void)par_stream;
  if (!valid_dtype(dtype)) return B200_ERR_DTYPE;
  int rc = check_conv_op(op);
  if (rc) return rc;
  if (!filters_strides) return B200_ERR_NULL;
  const size_t need = convtrans2d_workspace_bytes(dtype, op, 1);
  if (need == ~(size_t)0) return B200_ERR_LIMIT;             // the geometry's element counts overflow
  if (need == 0) return B200_OK;
  if (!img || !filters || !grad_out || !workspace) return B200_ERR_NULL;
  if (workspace_bytes < need) return B200_ERR_WORKSPACE;
  if (grad_img) {                       // the convolution that produces grad_img reads the filters as one dense block
    const size_t kk = op->kernel * op->kernel, og = op->chan_out / op->groups;
    if (filters_strides[3] != 1 || filters_strides[2] != op->kernel || filters_strides[1] != kk ||
        filters_strides[0] != og * kk)
      return B200_ERR_NOT_CONTIGUOUS;
  }
  if (!device_state()) return note_cuda_error(cudaErrorInitializationError, "b200_init not called on this device");
  return convtrans2d_backward(dtype, op, img, grad_img, filters, filters_strides, grad_filters, grad_out, workspace,
                              (cudaStream_t)stream);
}

// ---- conv1d ---------------------------------------------------------------------------------------
static int check_conv1d_op(const b200_conv1d_op* op) {
  if (!op) return B200_ERR_NULL;
  if (!op->groups || !op->stride || !op->dilation || !op->kernel) return B200_ERR_SHAPE;
  if (op->chan_in % op->groups || op->chan_out % op->groups) return B200_ERR_SHAPE;  // conv1d/mod.rs:246-250
  return B200_OK;
}

size_t b200_conv1d_workspace_bytes(int dtype, const b200_conv1d_op* op, int backward) {
  if (check_conv1d_op(op) || !valid_dtype(dtype)) return 0;
  return conv1d_workspace_bytes(dtype, op, backward);
}

int b200_conv1d_forward(int dtype, const b200_conv1d_op* op, const void* img, const size_t img_strides[3],
                        const void* filters, void* out, void* workspace, size_t workspace_bytes, void* stream) {
  if (!valid_dtype(dtype)) return B200_ERR_DTYPE;
  int rc = check_conv1d_op(op);
  if (rc) return rc;
  if (!img_strides) return B200_ERR_NULL;
  const size_t need = conv1d_workspace_bytes(dtype, op, 0);
  if (need == ~(size_t)0) return B200_ERR_LIMIT;             // the geometry's element counts overflow
  if (need == 0) return B200_OK;
  if (!img || !filters || !out || !workspace) return B200_ERR_NULL;
  if (workspace_bytes < need) return B200_ERR_WORKSPACE;
  if (!device_state()) return note_cuda_error(cudaErrorInitializationError, "b200_init not called on this device");
  return conv1d_forward(dtype, op, img, img_strides, filters, out, workspace, (cudaStream_t)stream);
}

int b200_conv1d_backward(int dtype, const b200_conv1d_op* op, const void* img, void* grad_img, const void* filters,
                         const size_t filters_strides[3], void* grad_filters, const void* grad_out, void* workspace,
                         size_t workspace_bytes, void* stream, void* par_stream) {
  (void)par_stream;
  if (!valid_dtype(dtype)) return B200_ERR_DTYPE;
  int rc = check_conv1d_op(op);
  if (rc) return rc;
  if (!filters_strides) return B200_ERR_NULL;
  const size_t need = conv1d_workspace_bytes(dtype, op, 1);
  if (need == ~(size_t)0) return B200_ERR_LIMIT;             // the geometry's element counts overflow
  if (need == 0) return B200_OK;
  if (!img || !filters || !grad_out || !workspace) return B200_ERR_NULL;
  if (workspace_bytes < need) return B200_ERR_WORKSPACE;
  if (!device_state()) return note_cuda_error(cudaErrorInitializationError, "b200_init not called on this device");
  return conv1d_backward(dtype, op, img, grad_img, filters, filters_strides, grad_filters, grad_out, workspace,
                         (cudaStream_t)stream);
}

}  // extern "C"
