// Shared definitions of the dfdx_b200 library: the canonical GEMM problem every entry point is
// lowered to, status codes, and small helpers.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stddef.h>
#include "../../include/dfdx_b200.h"

namespace b200 {

// One (possibly batched, possibly batch-reduced) strided GEMM in row-major index terms:
//   for (b0,b1) in batch:  C[b0,b1][i,j] = beta*C + sum_{r<red} sum_{p<k} A[b0,b1,r][i,p] * B[b0,b1,r][p,j]
// Strides are in elements.  `red` > 1 is how the broadcast-rhs weight gradient
// (matmul/cuda_kernel.rs:358-371 in dfdx: B serial beta=1 GEMMs) becomes a single launch.
struct GemmProblem {
  int dtype = B200_F32;
  int beta = 0;
  int64_t b0 = 1, b1 = 1, red = 1;
  int64_t m = 0, k = 0, n = 0;
  const void* a = nullptr;
  int64_t a_b0 = 0, a_b1 = 0, a_red = 0, a_r = 0, a_c = 0;
  const void* b = nullptr;
  int64_t b_b0 = 0, b_b1 = 0, b_red = 0, b_r = 0, b_c = 0;
  void* c = nullptr;
  int64_t c_b0 = 0, c_b1 = 0, c_r = 0, c_c = 0;
  // Optional fused epilogue (beta == 0 only):  C = act(alpha * (A.B) + bias), applied to the f32 (f64)
  // accumulator before the single rounding to C's type.  `bias` has C's element type and is indexed by the
  // output column j (bias_dim 0, e.g. Linear's bias over output features) or by the row i (bias_dim 1).
  double alpha = 1.0;
  const void* bias = nullptr;
  int bias_dim = 0;
  int act = B200_ACT_NONE;
  bool fused() const { return alpha != 1.0 || bias != nullptr || act != B200_ACT_NONE; }
  // f16 problems only: `c` is an f32 matrix (strides in f32 elements) that the f32 accumulator is ADDED to, without a
  // rounding to f16 in between (a mixed-precision trainer's f32 gradient of an f16 weight).  Tensor-core path only.
  bool acc32 = false;
};

static inline size_t dtype_size(int dtype) {
  switch (dtype) {
    case B200_F32: return 4;
    case B200_F64: return 8;
    case B200_F16:
    case B200_AMP_F16: return 2;
    default: return 0;
  }
}

// Per-device state created by b200_init.
struct DeviceState {
  bool ready = false;
  int sm_count = 0;
  int* status = nullptr;  // device word: 0 or a B200_ERR_* written by a kernel that gave up on a wait
  // f32 scratch for split-K partial sums of f16 GEMMs (fixed size, allocated by b200_init).  Uses on
  // different streams are ordered through `split_event`.
  float* split_scratch = nullptr;
  size_t split_scratch_bytes = 0;
  cudaEvent_t split_event = nullptr;
  cudaStream_t split_last_stream = nullptr;
  bool split_used = false;
};
constexpr size_t SPLIT_SCRATCH_BYTES = 64u << 20;

DeviceState* device_state();                 // state of the current device (nullptr before init)
int note_cuda_error(cudaError_t e, const char* where);
void count_launch(bool tensor);

int launch_gemm_simt(const GemmProblem& p, cudaStream_t stream);
// Returns B200_ERR_UNSUPPORTED (without launching) when the operands are not TMA-addressable.
int launch_gemm_tc(const GemmProblem& p, cudaStream_t stream);
// GemmProblem::acc32 (f16 operands added in f32 to an f32 C); B200_ERR_UNSUPPORTED without a launch otherwise.
int launch_gemm_tc_acc32(const GemmProblem& p, cudaStream_t stream);
bool tc_eligible(const GemmProblem& p);
int tc_setup_device();                       // cudaFuncSetAttribute for every tensor-core kernel

// Fused attention forward (attention.cu); strides in elements, see b200_attention_forward.
int attention_setup_device();
int attention_forward(int dtype, int64_t B, int64_t H, int64_t s1, int64_t s2, int64_t d, const void* q,
                      const int64_t qs[4], const void* k, const int64_t ks[4], const void* v, const int64_t vs[4],
                      double alpha, void* out, const int64_t os[4], float* lse, cudaStream_t stream);

// Fused attention backward (attention_bwd.cu); see b200_attention_backward.
int attention_bwd_setup_device();
size_t attention_backward_workspace_bytes(int64_t B, int64_t H, int64_t s1);
int attention_backward(int dtype, int64_t B, int64_t H, int64_t s1, int64_t s2, int64_t d, const void* q,
                       const int64_t qs[4], const void* k, const int64_t ks[4], const void* v, const int64_t vs[4],
                       double alpha, const void* out, const int64_t os[4], const float* lse, const void* go,
                       const int64_t gs[4], void* gq, const int64_t gqs[4], void* gk, const int64_t gks[4], void* gv,
                       const int64_t gvs[4], int accumulate, void* workspace, size_t workspace_bytes, cudaStream_t stream);

// Row-wise kernels (rowwise.cu); leading dimensions in elements.
int layer_norm_forward(int dtype, int64_t rows, int64_t cols, const void* x, int64_t x_ld, const void* gamma, const void* beta,
                       double eps, void* y, int64_t y_ld, float* stats, cudaStream_t stream);
int layer_norm_backward(int dtype, int64_t rows, int64_t cols, const void* x, int64_t x_ld, const void* gamma, const float* stats,
                        const void* g, int64_t g_ld, void* gx, int64_t gx_ld, int accumulate_x, float* ggamma, float* gbeta,
                        float* gxsum, cudaStream_t stream);
int add_layer_norm_forward(int dtype, int64_t rows, int64_t cols, const void* a, int64_t a_ld, const void* b, int64_t b_ld,
                           void* sum, int64_t sum_ld, const void* gamma, const void* beta, double eps, void* y, int64_t y_ld,
                           float* stats, cudaStream_t stream);
int relu_backward_column_sum(int dtype, int64_t rows, int64_t cols, const void* y, int64_t y_ld, void* g, int64_t ld, float* out,
                             cudaStream_t stream);
int rowwise_setup_device();                  // opt-in shared memory of the row-wise kernels
int softmax_forward(int dtype, int64_t rows, int64_t cols, const void* x, int64_t x_ld, double alpha, void* y, int64_t y_ld,
                    cudaStream_t stream);
int softmax_backward(int dtype, int64_t rows, int64_t cols, const void* y, int64_t y_ld, const void* g, int64_t g_ld,
                     double alpha, void* gx, int64_t gx_ld, int accumulate, cudaStream_t stream);
int column_sum(int dtype, int64_t rows, int64_t cols, const void* g, int64_t ld, float* out, cudaStream_t stream);

// Lowers one problem to a kernel family according to b200_set_path and eligibility.
int run_gemm(const GemmProblem& p, cudaStream_t stream);
int current_path();                          // b200_path in force

// Implicit-GEMM convolution on the f32 (3xTF32) tensor-core kernel (gemm_tc.cu): the im2col gather is done by the
// TMA loads from a channels-last copy of the image, no patch buffer exists.  Unit stride only.
//
// ConvImplicit: out[b, g*m + i, y, x] (beta) += sum_{tap=(k1,k2)} sum_c filt[g][i][tap][c] *
//                                              img_cl[b, y + h0 + k1*dh, x + w0 + k2*dw, g*cpad + c]
// with zeros outside the image.  The forward pass uses (h0, dh, w0, dw) = (-pad, dil, -pad, dil) on the input image;
// the data gradient is the same sum over grad_out with (pad, -dil, pad, -dil) and the filters' roles exchanged.
struct ConvImplicit {
  const float* img_cl = nullptr;             // (batch, h_img, w_img, groups * cpad), channels padded with zeros
  int64_t batch = 0, h_img = 0, w_img = 0, groups = 1, cpad = 0;   // cpad % 16 == 0
  const float* filt = nullptr;               // (groups, m, kh*kw, cpad)
  int64_t m = 0;                             // output channels per group
  int kh = 1, kw = 1, h0 = 0, dh = 1, w0 = 0, dw = 1;
  float* out = nullptr;                      // (batch, groups * m, h_out, w_out) contiguous
  int64_t h_out = 0, w_out = 0;              // w_out <= 256
  int beta = 0;
};
bool conv_implicit_ok(const ConvImplicit& c);
int launch_conv_implicit(const ConvImplicit& c, cudaStream_t stream);

// Filter gradient of the same convolution for one group:
//   out[i][tap][c] += sum_b sum_{y,x} gout[b, i, y, x] * img_cl[b, y + h0 + k1*dh, x + w0 + k2*dw, c]
// `out` (m, kh*kw, cpad) must hold zeros (or a running sum): the K slices of the reduction add into it atomically.
struct ConvImplicitWgrad {
  const float* gout = nullptr;               // this group's (m, h_out, w_out) planes; image stride gout_bs elements
  int64_t gout_bs = 0, m = 0, h_out = 0, w_out = 0;   // w_out % 4 == 0
  const float* img_cl = nullptr;             // this group's first channel of (batch, h_img, w_img, c_total)
  int64_t batch = 0, h_img = 0, w_img = 0, c_total = 0, cpad = 0;   // cpad % 32 == 0
  int kh = 1, kw = 1, h0 = 0, dh = 1, w0 = 0, dw = 1;
  float* out = nullptr;
};
bool conv_implicit_wgrad_ok(const ConvImplicitWgrad& c);
int launch_conv_implicit_wgrad(const ConvImplicitWgrad& c, cudaStream_t stream);

}  // namespace b200
