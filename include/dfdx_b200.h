/*
 * dfdx_b200 — C ABI of the B200 (sm_100a) matmul / conv2d hot path for dfdx's `Cuda` device.
 *
 * Every entry point is what dfdx's Rust side would bind (through cudarc-style raw device pointers
 * and raw CUDA streams) in place of the cuBLAS calls and helper kernels it uses today.  All paths
 * below are relative to the dfdx repository (v0.13.0).
 *
 * Conventions shared by all entry points
 *   - Pointers are device pointers owned by the caller; nothing is retained after the call returns.
 *   - Strides are ELEMENT strides exactly as stored in dfdx's `Tensor::strides`
 *     (dfdx-core/src/tensor/tensor_impls.rs:32-39): any permutation / broadcast of a contiguous
 *     layout.  A stride of 0 marks a broadcast dimension.
 *   - `stream` / `par_stream` are `cudaStream_t` / `CUstream` handles passed as `void*`
 *     (NULL = the legacy default stream).  Calls only enqueue work; ordering is stream order.
 *   - Return value: 0 on success, a negative `b200_status` otherwise.  No entry point aborts,
 *     throws or calls exit().  Shape / stride violations that the reference turns into a panic
 *     before any launch are reported as B200_ERR_SHAPE / B200_ERR_STRIDE before any launch.
 *   - The caller's CUDA context (device) must be current, as cudarc guarantees per call.
 */
#ifndef DFDX_B200_H
#define DFDX_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Element types of the path: the `Dtype`s for which dfdx implements `Device<E>` on `Cuda`
 * (dfdx-core/src/tensor_ops/utilities/device.rs:128-135). */
typedef enum {
  B200_F32 = 0,     /* f32: tensor cores via 3xTF32 (kind::tf32), exact-FP32 SIMT for small/unaligned */
  B200_F64 = 1,     /* f64: SIMT only */
  B200_F16 = 2,     /* half::f16 storage, f32 accumulate */
  B200_AMP_F16 = 3  /* AMP<f16>: f16 storage, f32 compute (matmul/cuda_kernel.rs:62-135) */
} b200_dtype;

typedef enum {
  B200_OK = 0,
  B200_ERR_SHAPE = -1,        /* inner dimensions / batch dimensions disagree (matmul/mod.rs:192,229,267,306) */
  B200_ERR_STRIDE = -2,       /* "At least a single stride must be 1" (matmul/mod.rs:323); zero out/batch stride
                                 where the reference asserts non-zero (cuda_kernel.rs:208,400,474) */
  B200_ERR_DTYPE = -3,
  B200_ERR_NULL = -4,
  B200_ERR_WORKSPACE = -5,    /* workspace smaller than b200_conv2d_workspace_bytes() */
  B200_ERR_CUDA = -6,         /* a CUDA runtime/driver call failed; see b200_last_cuda_error() */
  B200_ERR_DEVICE_TIMEOUT = -7, /* a bounded device-side wait expired (reported by b200_device_status) */
  B200_ERR_UNSUPPORTED = -8,
  B200_ERR_NOT_CONTIGUOUS = -9, /* conv2d: "Image & filter inputs to conv2d must be contiguous" (conv2d/mod.rs:287-289) */
  B200_ERR_LIMIT = -10          /* request exceeds a documented fixed capacity */
} b200_status;

/* Mirrors `Conv2DOp` bit for bit: 12 x usize, #[repr(C)]
 * (dfdx-core/src/tensor_ops/conv2d/mod.rs:14-29; device copy conv2d/conv2d.cu:3-16). */
typedef struct {
  size_t kernel, stride, padding, dilation, groups, batch;
  size_t chan_in, chan_out, h_in, h_out, w_in, w_out;
} b200_conv2d_op;

/* Mirrors `ConvTrans2DOp`: the same 12 x usize as `Conv2DOp`
 * (dfdx-core/src/tensor_ops/convtrans2d/mod.rs:12-28). */
typedef b200_conv2d_op b200_convtrans2d_op;

/* Mirrors `Conv1DOp`: 10 x usize, #[repr(C)] (dfdx-core/src/tensor_ops/conv1d/mod.rs:12-23). */
typedef struct {
  size_t kernel, stride, padding, dilation, groups, batch;
  size_t chan_in, chan_out, l_in, l_out;
} b200_conv1d_op;

/* Activation applied by a fused epilogue. */
typedef enum {
  B200_ACT_NONE = 0,
  B200_ACT_RELU = 1     /* max(x, 0), dfdx's `ReLU` (dfdx-core/src/tensor_ops/relu/mod.rs) */
} b200_activation;

/* Work done on each output element between the accumulator and the single store:
 *     out = activation(alpha * sum + bias[j])            (j = output column)
 * `bias` is NULL or `n` elements of the output's dtype, 16-byte aligned for the tensor-core kernels
 * (otherwise the SIMT kernel serves the call). */
typedef struct {
  double alpha;         /* 1.0 = no scaling */
  const void* bias;
  int activation;       /* b200_activation */
} b200_epilogue;

/* Which kernel family serves the contraction.  AUTO is the product behaviour. */
typedef enum {
  B200_PATH_AUTO = 0,   /* tensor cores when operands are TMA-addressable and the problem is not tiny */
  B200_PATH_SIMT = 1,   /* force the any-stride exact-FP32/FP64 SIMT kernels */
  B200_PATH_TENSOR = 2  /* force tcgen05; returns B200_ERR_UNSUPPORTED if operands are not TMA-addressable */
} b200_path;

/* ---- library / device ------------------------------------------------------------------------- */

/* Replaces `Cuda::try_build(ordinal, seed)`'s cuBLAS-handle creation
 * (dfdx-core/src/tensor/cuda/device.rs:72-91): selects the device, resolves the driver entry
 * point used to encode TMA descriptors, raises the kernels' dynamic shared-memory limits and
 * allocates the per-device status word, a 64 MiB f32 scratch for the split-K partial sums of f16
 * GEMMs and the event that orders its uses across streams.  These are the library's only device
 * allocations.  Idempotent; thread-safe. */
int b200_init(int ordinal);

const char* b200_strerror(int status);
/* Text of the last CUDA error seen by this thread inside the library ("" if none). */
const char* b200_last_cuda_error(void);
/* Reads (and clears) the device-side status word of the current device after synchronising
 * `stream`: 0, or B200_ERR_DEVICE_TIMEOUT if any kernel gave up on a bounded wait. */
int b200_device_status(void* stream);
/* Process-wide override of kernel-family selection (testing / profiling). */
int b200_set_path(int path);
/* f32 tensor-core operand split (testing / profiling).  Every staged f32 x is used in place as the `big`
 * tf32 operand (the tensor core reads its top 19 bits) and small = x - trunc_tf32(x) is written beside it.
 * mode 1 (default) stores small as computed, 0 rounds it to tf32 first (cvt.rna).  Both stay inside the f32
 * tolerance; any other value returns B200_ERR_UNSUPPORTED. */
int b200_set_tf32_split_mode(int mode);
/* Tensor-core tile width override (testing / profiling): 64, 128 or 256 output columns per CTA tile (128 rows);
 * 512 stands for the f16 kernel with 256 x 256 tiles (f32 problems then take 256 columns); 0 (default) lets a wave
 * model choose. */
int b200_set_tile_n(int bn);
/* MN-major operand loading (testing / profiling): 1 (default) brings a tile's column chunks with one
 * 5-D TMA box where the extent is a whole number of chunks; 0 always issues one 4-D box per chunk. */
int b200_set_mn_single_box(int on);
/* CTA-pair kernels (testing / profiling): 1 (default) uses the single-CTA tensor-core kernels only, 0 lets the
 * planner choose between them and the CTA-pair (cta_group::2, 256x256 tiles) kernels by a wave model, 2 forces
 * the pair kernels wherever the output is wider than 128 columns. */
int b200_set_cta_pair_mode(int mode);
/* Epilogue store path of the tensor-core kernels (testing / profiling): 0 (default) planner's choice (f16 outputs
 * with beta = 0 leave through shared memory and TMA bulk stores; otherwise row stores, or column stores where
 * the model says so), 1 per-thread row stores only (each thread writes 16- / 32-byte pieces of its output row),
 * 2 column stores wherever possible (the kernel's M runs along the output's unit-stride dimension; warp stores
 * are contiguous). */
int b200_set_store_mode(int mode);
/* Lowering of the convolutions (testing / profiling).  mode 0 (default): the planner's choice.  For f32 with unit
 * stride and tensor-core sized problems that is the implicit GEMM: the kernel's TMA loads gather the patches from a
 * channels-last copy of the image, no patch buffer exists (forward, filter gradient, and the data gradient when the
 * image has at least 64 channels per group); everything else takes the materialising lowerings of mode 2.
 * mode 2: always materialise: unfold + GEMM forward, one batch-reduced GEMM over the unfolded image for the filter
 * gradient, and for the data gradient (contiguous filters) filters^T x grad_out followed by a fold (col2im) of the
 * per-tap gradients into the image.  mode 1: as mode 2, but the data gradient always takes the reference's lowering
 * (gather grad_out into patches, then GEMM with the transposed filters).  group_bytes: the GEMM + fold pass runs over
 * groups of images whose per-tap gradients take at most this many bytes (0 = the default, all images at once).
 * Returns 0, or B200_ERR_UNSUPPORTED. */
int b200_set_conv_lowering(int grad_img_mode, size_t group_bytes);
/* K decomposition of the tensor-core kernels (testing / profiling): 0 (default) the planner cuts K into slices when
 * the output tiles alone would leave most SMs idle (partial results are then added atomically, so the last bits of
 * such results can differ between runs); 1 never splits; n in 2..64 forces n slices; -1 forces, for f32, the
 * stream-K decomposition (the (tile, k-block) space cut into one equal contiguous range per SM; tiles cut by a
 * range boundary are summed atomically), which the planner never picks on its own. */
int b200_set_split_k(int mode);
/* Tail split of the f32 tensor-core kernel (testing / profiling).  The kernel is persistent: tiles are dealt round
 * robin to one CTA per SM, so a tile count just above a multiple of the SM count leaves most SMs idle during the last
 * round.  mode 0 (default): when that costs more than about 5 %, the tiles of the last, partial round are cut into K
 * slices spread over all SMs; their partial results are added atomically (as with split-K, the last bits of those
 * output tiles can then differ between runs; outputs with beta = 0 have those tiles zeroed first).  mode 1: never. */
int b200_set_tail_split(int mode);
/* The split-K of an f16 GEMM keeps its partial sums in the one f32 scratch the device owns; uses on different
 * streams are ordered by an event recorded when the GEMM is enqueued.  A stream capture cannot take part in that
 * ordering (a replay neither waits on nor records the event), so by default (0) a GEMM enqueued on a capturing
 * stream runs unsplit.  1: such GEMMs may split; the caller then guarantees that every replay of its graphs is
 * ordered against all other work this library does on the device (one stream for everything is enough). */
int b200_set_capture_split_k(int on);
/* The tensor-core GEMM kernels are persistent: their grid is one CTA per SM (or one per work unit when there are
 * fewer), and each CTA takes nearly all of an SM's shared memory, so a kernel enqueued on another stream while a
 * GEMM runs finds no SM to start on until the GEMM ends.  n > 0 caps the grids at n CTAs, leaving the other SMs
 * to such kernels (a NCCL all-reduce of one gradient while the GEMM of the next runs); 0 (default) restores one
 * CTA per SM.  Process-wide; takes effect from the next launch.  Negative values return B200_ERR_UNSUPPORTED. */
int b200_set_max_ctas(int n);
/* Clock budget of the bounded device-side waits of the tensor-core GEMM kernels (testing).  Every wait on a
 * shared-memory barrier inside those kernels gives up after a budget of SM clock cycles; the kernel then drains,
 * frees its tensor memory, writes B200_ERR_DEVICE_TIMEOUT to the device status word (b200_device_status) and
 * returns, leaving the context usable; its output is undefined.  0 (default) sizes the budget by the problem
 * (hundreds of milliseconds); a small positive value makes a healthy kernel give up, which is how the tests
 * exercise that path.  Negative values return B200_ERR_UNSUPPORTED. */
int b200_set_wait_limit(long long cycles);
/* Self-test of that mechanism (testing): launches one small CTA in which a thread waits, with the kernels' own
 * bounded wait and a budget of `limit_cycles`, on a barrier that nothing ever completes; the wait gives up, the CTA
 * runs the kernels' teardown and sets the status word, so b200_device_status then reports
 * B200_ERR_DEVICE_TIMEOUT once.  Synchronises `stream`.  `waited_cycles` (host pointer, may be NULL) receives the SM
 * clock cycles the wait lasted: a failed poll suspends the thread for a hardware-defined time, so this exceeds the
 * budget by up to 64 such polls. */
int b200_selftest_bounded_wait(long long limit_cycles, long long* waited_cycles, void* stream);
/* Number of kernel launches this library has enqueued since load (all threads). */
uint64_t b200_launch_count(void);
/* Of those, launches of tcgen05 tensor-core kernels. */
uint64_t b200_tensor_launch_count(void);
/* Convolution passes (a forward, a filter gradient or a data gradient) that the implicit-GEMM lowering has served
 * since load (testing / profiling: tells which lowering a call took). */
uint64_t b200_conv_implicit_count(void);

/* ---- the two GEMM seams ---------------------------------------------------------------------- */

/* Replaces the body of `Cuda::gemm` (dfdx-core/src/tensor_ops/matmul/cuda_kernel.rs:153-181,
 * i.e. `gemm_cfg` :18-60 + cublas{S,D,H}gemm / cublasGemmEx):
 *     out[i*os0 + j*os1] = beta*out[..] + sum_p lhs[i*ls0 + p*ls1] * rhs[p*rs0 + j*rs1]
 * for i<m, j<n, p<k.  beta is 0 or 1; with beta == 0 `out` is never read (it comes from
 * `alloc_empty`, cuda_kernel.rs:253).  With beta == 1 and f16 storage the tensor-core path adds the
 * f16-rounded product into `out` (C += f16(acc), an element-wise add performed by the memory system on staged
 * tiles): two roundings where cuBLAS rounds f32(acc + C) once; both stay within one f16 ulp of the exact sum, and
 * accumulation into the zeroed buffers of `Gradients::try_alloc_for` is exact.  Legal stride pairs are those `matrix_strides`
 * accepts (matmul/mod.rs:316-325). */
int b200_gemm(int dtype, size_t m, size_t k, size_t n,
              const void* lhs, const size_t lhs_strides[2],
              const void* rhs, const size_t rhs_strides[2],
              double beta, void* out, const size_t out_strides[2], void* stream);

/* Replaces the body of `Cuda::gemm_batch` (cuda_kernel.rs:184-237, cublas*gemmStridedBatched[Ex]).
 * strides[0] is the batch stride; lhs/rhs batch stride may be 0, out batch stride must not be. */
int b200_gemm_batch(int dtype, size_t batch, size_t m, size_t k, size_t n,
                    const void* lhs, const size_t lhs_strides[3],
                    const void* rhs, const size_t rhs_strides[3],
                    double beta, void* out, const size_t out_strides[3], void* stream);

/* ---- the kernel-trait seams (fused forward / backward) ---------------------------------------- */

/* `MatMatKernel::forward/backward for Cuda` (cuda_kernel.rs:244-312): (M,K)x(K,N).
 * forward writes a contiguous (M,N) `out`.  backward accumulates grad_lhs += grad_out * rhs^T
 * through lhs_strides and grad_rhs += lhs^T * grad_out through rhs_strides; grad_out is a
 * contiguous (M,N).  Either gradient pointer may be NULL to skip it.  As in the reference
 * (cuda_kernel.rs:282-310) the grad_lhs GEMM is enqueued on `par_stream` and the grad_rhs GEMM on `stream`, and the
 * caller joins the two streams before and after the call, as dfdx does with `par_stream.wait_for_default()` and
 * `dev.wait_for(par_stream)`.  A NULL `par_stream` means there is no second stream: both GEMMs go to `stream`.
 * The same holds for the other three `*_backward` matmul entry points below. */
int b200_matmat_forward(int dtype, size_t m, size_t k, size_t n,
                        const void* lhs, const size_t lhs_strides[2],
                        const void* rhs, const size_t rhs_strides[2],
                        void* out, void* stream);
int b200_matmat_backward(int dtype, size_t m, size_t k, size_t n,
                         const void* lhs, const size_t lhs_strides[2], void* grad_lhs,
                         const void* rhs, const size_t rhs_strides[2], void* grad_rhs,
                         const void* grad_out, void* stream, void* par_stream);

/* `MatMatBrKernel for Cuda` (cuda_kernel.rs:319-388): (B,M,K)x(K,N), rhs broadcast over B.
 * backward: grad_rhs += sum_b lhs_b^T * grad_out_b is ONE launch that reduces over the batch
 * inside the kernel (the reference issues B serial beta=1 GEMMs, :358-371). */
int b200_matmat_br_forward(int dtype, size_t batch, size_t m, size_t k, size_t n,
                           const void* lhs, const size_t lhs_strides[3],
                           const void* rhs, const size_t rhs_strides[2],
                           void* out, void* stream);
int b200_matmat_br_backward(int dtype, size_t batch, size_t m, size_t k, size_t n,
                            const void* lhs, const size_t lhs_strides[3], void* grad_lhs,
                            const void* rhs, const size_t rhs_strides[2], void* grad_rhs,
                            const void* grad_out, void* stream, void* par_stream);

/* `MatMatBatch3Kernel for Cuda` (cuda_kernel.rs:395-462): (B,M,K)x(B,K,N); batch strides non-zero. */
int b200_matmat_batch3_forward(int dtype, size_t batch, size_t m, size_t k, size_t n,
                               const void* lhs, const size_t lhs_strides[3],
                               const void* rhs, const size_t rhs_strides[3],
                               void* out, void* stream);
int b200_matmat_batch3_backward(int dtype, size_t batch, size_t m, size_t k, size_t n,
                                const void* lhs, const size_t lhs_strides[3], void* grad_lhs,
                                const void* rhs, const size_t rhs_strides[3], void* grad_rhs,
                                const void* grad_out, void* stream, void* par_stream);

/* `MatMatBatch4Kernel for Cuda` (cuda_kernel.rs:469-568): (B,S,M,K)x(B,S,K,N) in one launch per
 * GEMM group (the reference loops over B on the host, :492-517, :538-564). */
int b200_matmat_batch4_forward(int dtype, size_t batch, size_t seq, size_t m, size_t k, size_t n,
                               const void* lhs, const size_t lhs_strides[4],
                               const void* rhs, const size_t rhs_strides[4],
                               void* out, void* stream);
int b200_matmat_batch4_backward(int dtype, size_t batch, size_t seq, size_t m, size_t k, size_t n,
                                const void* lhs, const size_t lhs_strides[4], void* grad_lhs,
                                const void* rhs, const size_t rhs_strides[4], void* grad_rhs,
                                const void* grad_out, void* stream, void* par_stream);

/* ---- GEMMs with a fused epilogue (API additions: no single counterpart in the reference) -------- */

/* Mixed-precision form of the broadcast-rhs weight gradient (the grad_rhs half of MatMatBrKernel::backward,
 * dfdx-core/src/tensor_ops/matmul/cuda_kernel.rs:358-371): f16 lhs and grad_out, and a gradient buffer that holds f32:
 *     grad_rhs[k x n, strides grad_rhs_strides in f32 elements] += sum_b lhs_b^T * grad_out_b
 * added in f32 without an f16 rounding in between -- what a trainer that keeps f32 master weights and f32 gradients
 * (dfdx's AMP dtype) otherwise gets from an f16 gradient buffer plus a cast, and one launch (the K slices add into
 * grad_rhs itself through bulk reduce-adds: no scratch, no zero fill, no second kernel).  dtype B200_F16 or
 * B200_AMP_F16; tensor cores only: B200_ERR_UNSUPPORTED without a launch where the operands are not TMA-addressable
 * (16-byte aligned bases, a unit stride per operand, other strides multiples of 8 elements; grad_rhs: a unit stride
 * and the other a multiple of 8). */
int b200_matmat_br_grad_rhs_f32(int dtype, size_t batch, size_t m, size_t k, size_t n,
                                const void* lhs, const size_t lhs_strides[3], const void* grad_out,
                                float* grad_rhs, const size_t grad_rhs_strides[2], void* stream);

/* `b200_matmat_br_backward` for the FIRST accumulation into freshly allocated gradient buffers: grad_lhs and grad_rhs
 * are written, not added to, so they need not be zero-filled and are not read (dfdx zero-fills every gradient buffer
 * in `Gradients::try_alloc_for` and the first backward op then adds into the zeros: two extra passes over each
 * buffer).  A view in which several elements share storage (a stride of 0 over an extent > 1) is rejected with
 * B200_ERR_STRIDE: there the sum over the aliased elements is the accumulation. */
int b200_matmat_br_backward_overwrite(int dtype, size_t batch, size_t m, size_t k, size_t n,
                                      const void* lhs, const size_t lhs_strides[3], void* grad_lhs,
                                      const void* rhs, const size_t rhs_strides[2], void* grad_rhs,
                                      const void* grad_out, void* stream);

/* A doubly batched strided GEMM (strides = [batch0, batch1, row, col] in elements; an lhs / rhs batch
 * stride may be 0) whose epilogue applies `ep` before the store: one kernel and one pass over `out`
 * where dfdx runs a GEMM and then one elementwise kernel per op, each re-reading and re-writing the GEMM's
 * output.  beta is 0: `out` is only written.  `ep` NULL = plain GEMM. */
int b200_gemm_batch_fused(int dtype, size_t batch0, size_t batch1, size_t m, size_t k, size_t n,
                          const void* lhs, const size_t lhs_strides[4],
                          const void* rhs, const size_t rhs_strides[4],
                          const b200_epilogue* ep, void* out, const size_t out_strides[4], void* stream);

/* `Linear::try_forward` in one launch (dfdx/src/nn/layers/linear.rs:82-89: `x.matmul(weight.permute())`,
 * then `Bias1D::try_forward`, bias1d.rs:66-79: `bias.broadcast_like(&x) + x`), optionally followed by the
 * `ReLU` of FeedForward (dfdx/src/nn/layers/transformer.rs:4-8):
 *     out[b, s, o] = act(sum_i x[b, s, i] * weight[i, o] + bias[o])
 * x: (batch, m, i) with strides `x_strides`; `weight` is the (i, o) VIEW with strides `w_strides`
 * (for dfdx's stored (O, I) weight: [1, I]); bias: o elements or NULL; out: contiguous (batch, m, o). */
int b200_linear_forward(int dtype, size_t batch, size_t m, size_t i, size_t o,
                        const void* x, const size_t x_strides[3],
                        const void* weight, const size_t w_strides[2],
                        const void* bias, int activation, void* out, void* stream);

/* `q.matmul(k) * scalar` of MultiHeadAttention in one launch
 * (dfdx/src/nn/layers/multi_head_attention.rs:136-137): `b200_matmat_batch4_forward` with every output
 * element multiplied by `alpha` before it is rounded and stored. */
int b200_matmat_batch4_forward_scaled(int dtype, size_t batch, size_t seq, size_t m, size_t k, size_t n,
                                      const void* lhs, const size_t lhs_strides[4],
                                      const void* rhs, const size_t rhs_strides[4],
                                      double alpha, void* out, void* stream);

/* ---- fused attention (API addition) --------------------------------------------------------------- */

/* The op sequence of `MultiHeadAttention::try_forward` between its projections
 * (dfdx/src/nn/layers/multi_head_attention.rs:136-141):
 *     weights = softmax(q.matmul(k) * alpha, last axis);   tokens = weights.matmul(v)
 * in one kernel: the (batch, heads, S1, S2) score tensor lives in tensor memory / shared memory and never
 * reaches HBM (the unfused path writes and re-reads it five times).  f16 / AMP f16 only; f32 accumulation
 * and an f32 softmax inside.
 *   q   : (batch, heads, S1, D) view      k : (batch, heads, D, S2) view — exactly what dfdx passes to matmul
 *   v   : (batch, heads, S2, D) view      out: (batch, heads, S1, D) view (e.g. a permuted (batch, S1, heads, D)
 *         buffer, which saves the copy `tokens.permute().reshape()` makes)
 * all with unit stride along D and every other stride a multiple of 8 elements, 16-byte aligned bases, D a
 * multiple of 8 and <= 128; anything else returns B200_ERR_UNSUPPORTED before any launch and the caller keeps
 * the unfused sequence.  `lse` is NULL or batch*heads*S1 floats that receive log(sum_j exp(alpha * s_ij)),
 * which b200_attention_backward needs. */
int b200_attention_forward(int dtype, size_t batch, size_t heads, size_t s1, size_t s2, size_t d,
                           const void* q, const size_t q_strides[4],
                           const void* k, const size_t k_strides[4],
                           const void* v, const size_t v_strides[4],
                           double alpha, void* out, const size_t out_strides[4], float* lse, void* stream);

/* Backward of b200_attention_forward: the tape entries of the same four ops (matmul, scalar mul, softmax,
 * matmul) in three launches, again without a score-sized tensor in HBM (P is recomputed from `lse`).
 *   out, lse      : what the forward returned          grad_out : gradient of `out`, a (batch, heads, S1, D) view
 *   grad_q / grad_v: views shaped and strided like q / v;  grad_k: a (batch, heads, D, S2) view like k
 *   accumulate    : 0 = the gradients are written; 1 = added to what the buffers hold, as dfdx's backward ops do
 *                   into `Gradients` buffers.  grad_q may be NULL (only dK, dV) or grad_k and grad_v both NULL.
 *   workspace     : b200_attention_backward_workspace_bytes(batch, heads, S1) bytes of device scratch, 16-byte aligned
 * Same layout limits as the forward (B200_ERR_UNSUPPORTED before any launch otherwise). */
size_t b200_attention_backward_workspace_bytes(size_t batch, size_t heads, size_t s1);
int b200_attention_backward(int dtype, size_t batch, size_t heads, size_t s1, size_t s2, size_t d,
                            const void* q, const size_t q_strides[4],
                            const void* k, const size_t k_strides[4],
                            const void* v, const size_t v_strides[4],
                            double alpha, const void* out, const size_t out_strides[4], const float* lse,
                            const void* grad_out, const size_t grad_out_strides[4],
                            void* grad_q, const size_t grad_q_strides[4],
                            void* grad_k, const size_t grad_k_strides[4],
                            void* grad_v, const size_t grad_v_strides[4],
                            int accumulate, void* workspace, size_t workspace_bytes, void* stream);

/* ---- row-wise neighbours of the GEMMs (API additions) --------------------------------------------- */

/* `LayerNorm1D::try_forward` (dfdx/src/nn/layers/layer_norm1d.rs:87-91) in one kernel:
 *     y[r, :] = (x[r, :] - mean_r) / sqrt(mean((x[r, :] - mean_r)^2) + epsilon) * gamma + beta
 * i.e. `normalize::<last axis>(epsilon)` (dfdx-core/src/tensor_ops/normalize.rs:33-50: mean, subtract, square,
 * mean, add epsilon, sqrt, divide) followed by the broadcast multiply and add.  x, y: rows x cols with unit
 * column stride and row strides x_ld / y_ld (elements); gamma, beta: cols elements of the same dtype or NULL
 * (NULL, NULL = plain normalize).  `stats` is NULL or 2*rows floats that receive (mean, 1/std) per row for the
 * backward.  f32 and f16 (f32 statistics); f64 returns B200_ERR_UNSUPPORTED. */
int b200_layer_norm_forward(int dtype, size_t rows, size_t cols, const void* x, size_t x_ld,
                            const void* gamma, const void* beta, double epsilon,
                            void* y, size_t y_ld, float* stats, void* stream);

/* The tape entries of the same ops in one kernel: grad_x (NULL = not wanted; written, or added to when
 * accumulate_x != 0) and the f32 sums grad_gamma[j] += sum_r g[r,j] * xhat[r,j], grad_beta[j] += sum_r g[r,j]
 * (either may be NULL; they are ADDED to, so zero them or pass f32 gradient buffers).  cols <= 1024 (f32) /
 * 2048 (f16), else B200_ERR_LIMIT. */
int b200_layer_norm_backward(int dtype, size_t rows, size_t cols, const void* x, size_t x_ld, const void* gamma,
                             const float* stats, const void* grad_out, size_t grad_out_ld,
                             void* grad_x, size_t grad_x_ld, int accumulate_x,
                             float* grad_gamma, float* grad_beta, void* stream);

/* b200_layer_norm_backward (grad_x written) that also returns the column sums of grad_x as it stores it (rounded to
 * dtype): grad_x_sum[j] += sum_r grad_x[r, j] in f32.  For `LayerNorm(x + Linear(h))`, where the residual add passes
 * the gradient on unchanged, that is the Linear's bias gradient (bias1d.rs:66-79), which otherwise costs a pass of
 * its own over grad_x.  One kernel where the rows allow 16-byte access and cols <= 512 (f16) / 256 (f32), otherwise the
 * plain backward followed by the column sum. */
int b200_layer_norm_backward_sum(int dtype, size_t rows, size_t cols, const void* x, size_t x_ld, const void* gamma,
                                 const float* stats, const void* grad_out, size_t grad_out_ld,
                                 void* grad_x, size_t grad_x_ld, float* grad_gamma, float* grad_beta,
                                 float* grad_x_sum, void* stream);

/* The residual add in front of a LayerNorm and the LayerNorm in one kernel (dfdx's transformer block computes
 * `norm(x + sublayer(x))`: ResidualAdd, dfdx/src/nn/layers/residual_add.rs, then LayerNorm1D,
 * dfdx/src/nn/layers/transformer.rs:27-30):
 *     sum[r, :] = a[r, :] + b[r, :]   (rounded to dtype, as the separate add stores it)
 *     y[r, :]   = LayerNorm(sum[r, :])
 * `sum` is kept because the LayerNorm's backward reads it.  Same limits and `stats` as b200_layer_norm_forward; rows
 * the one-kernel path does not take (cols > 512 (f16) / 256 (f32), or no 16-byte access) run as an add kernel followed
 * by the plain LayerNorm. */
int b200_add_layer_norm_forward(int dtype, size_t rows, size_t cols, const void* a, size_t a_ld, const void* b, size_t b_ld,
                                void* sum, size_t sum_ld, const void* gamma, const void* beta, double epsilon,
                                void* y, size_t y_ld, float* stats, void* stream);

/* ReLU's backward (dfdx-core/src/tensor_ops/relu/cpu_kernel.rs:11, grad * (y > 0)) and the bias gradient of the Linear in front of it in
 * one pass: grad[r, j] = y[r, j] > 0 ? grad[r, j] : 0, in place, and grad_bias[j] += sum_r grad[r, j] in f32
 * (grad_bias may be NULL: mask only). */
int b200_relu_backward_bias_grad(int dtype, size_t rows, size_t cols, const void* y, size_t y_ld,
                                 void* grad, size_t grad_ld, float* grad_bias, void* stream);

/* Backward of `bias.broadcast_like(&x) + x` (dfdx/src/nn/layers/bias1d.rs:66-79; the `sum` over the
 * broadcast axes): grad_bias[j] += sum_r grad_out[r, j] in f32, one pass over grad_out. */
int b200_bias_grad(int dtype, size_t rows, size_t cols, const void* grad_out, size_t grad_out_ld,
                   float* grad_bias, void* stream);

/* `softmax` over the last axis of a (rows, cols) matrix (dfdx-core/src/tensor_ops/softmax.rs:36-84: max, subtract,
 * exp, sum, divide — five kernels and their tape entries in the reference, one pass here), with the scalar multiply
 * that precedes it in MultiHeadAttention (multi_head_attention.rs:136-137) folded in:
 *     y = softmax(alpha * x),     grad_x (+)= alpha * y * (grad_out - sum_j grad_out_j * y_j).
 * f32 and f16 (f32 arithmetic); leading dimensions in elements, >= cols.  `accumulate` != 0 adds into grad_x
 * (dfdx's `+=` into a gradient buffer), 0 writes it.  y may alias x; grad_x may alias grad_out. */
int b200_softmax_forward(int dtype, size_t rows, size_t cols, const void* x, size_t x_ld, double alpha,
                         void* y, size_t y_ld, void* stream);
int b200_softmax_backward(int dtype, size_t rows, size_t cols, const void* y, size_t y_ld,
                          const void* grad_out, size_t grad_out_ld, double alpha,
                          void* grad_x, size_t grad_x_ld, int accumulate, void* stream);

/* ---- conv2d (unfold + GEMM lowering) ---------------------------------------------------------- */

/* Bytes of caller-provided scratch the conv2d entry points need; `backward` != 0 selects the
 * backward pass.  Plays the role of the sizes handed to `Cuda::get_workspace`
 * (conv2d/cuda_kernel.rs:91-95,156-168; tensor/cuda/device.rs:108-122).  Returns SIZE_MAX when the element
 * counts of the geometry do not fit a size_t; the forward / backward entry points then return B200_ERR_LIMIT
 * (the same holds for the conv1d and convtrans2d variants). */
size_t b200_conv2d_workspace_bytes(int dtype, const b200_conv2d_op* op, int backward);

/* `Conv2DKernel::forward for Cuda` (conv2d/cuda_kernel.rs:80-144 + conv2d.cu:18-52):
 * out(B,O,OH,OW) = conv(img(B,C,H,W) with 4-D element strides, filters(O,C/G,K,K) contiguous).
 * `out` is uninitialised on entry. */
int b200_conv2d_forward(int dtype, const b200_conv2d_op* op,
                        const void* img, const size_t img_strides[4],
                        const void* filters, void* out,
                        void* workspace, size_t workspace_bytes, void* stream);

/* `Conv2DKernel::backward for Cuda` (conv2d/cuda_kernel.rs:146-281 + conv2d.cu:54-168):
 * grad_img += conv_transpose(grad_out, filters); grad_filters (addressed through
 * filters_strides) += sum_b img_b (x) grad_out_b.  img, grad_img contiguous (B,C,H,W).  Both gradients share the
 * one workspace, so all of the pass is enqueued on `stream`; `par_stream` (on which the reference runs its grad_img
 * half, :171-227) is accepted for signature compatibility and unused, here and in the conv1d / convtrans2d
 * backward entry points. */
int b200_conv2d_backward(int dtype, const b200_conv2d_op* op,
                         const void* img, void* grad_img,
                         const void* filters, const size_t filters_strides[4], void* grad_filters,
                         const void* grad_out,
                         void* workspace, size_t workspace_bytes, void* stream, void* par_stream);

/* ---- conv1d (the same lowering over an image of height 1) ---------------------------------------- */

/* `Conv1DKernel for Cuda` (dfdx-core/src/tensor_ops/conv1d/cuda_kernel.rs:80-277 + conv1d.cu): unfold into patches
 * (B, C*K, L_out), one batched GEMM, and for the backward pass the transposed gather of grad_out, the transposed
 * filters and the batch sum of the filter gradient.  Same contracts as the conv2d entry points with 3-D strides:
 * img (B, C, L) through `img_strides`, filters (O, C/G, K) contiguous in forward and through `filters_strides` in
 * backward, out / grad_out (B, O, L_out) contiguous, img / grad_img contiguous in backward. */
size_t b200_conv1d_workspace_bytes(int dtype, const b200_conv1d_op* op, int backward);
int b200_conv1d_forward(int dtype, const b200_conv1d_op* op,
                        const void* img, const size_t img_strides[3],
                        const void* filters, void* out,
                        void* workspace, size_t workspace_bytes, void* stream);
int b200_conv1d_backward(int dtype, const b200_conv1d_op* op,
                         const void* img, void* grad_img,
                         const void* filters, const size_t filters_strides[3], void* grad_filters,
                         const void* grad_out,
                         void* workspace, size_t workspace_bytes, void* stream, void* par_stream);

/* ---- convtrans2d (the data gradient of a conv2d, run forward) ------------------------------------- */

/* `ConvTrans2DKernel for Cuda` (dfdx-core/src/tensor_ops/convtrans2d/cuda_kernel.rs:77-265 + convtrans2d.cu):
 * out (B, O, H_out, W_out) = convtrans2d(img (B, C, H, W), filters (C, O/G, K, K)); `out` is uninitialised on entry.
 * img, out, grad_out, grad_img contiguous (the reference panics otherwise, convtrans2d/mod.rs:242-244); filters and
 * grad_filters are addressed through `filters_strides`, and the backward pass needs them contiguous for grad_img
 * (B200_ERR_NOT_CONTIGUOUS otherwise).  backward: grad_img += ..., grad_filters += ...; either may be NULL. */
size_t b200_convtrans2d_workspace_bytes(int dtype, const b200_convtrans2d_op* op, int backward);
int b200_convtrans2d_forward(int dtype, const b200_convtrans2d_op* op,
                             const void* img, const void* filters, const size_t filters_strides[4], void* out,
                             void* workspace, size_t workspace_bytes, void* stream);
int b200_convtrans2d_backward(int dtype, const b200_convtrans2d_op* op,
                              const void* img, void* grad_img,
                              const void* filters, const size_t filters_strides[4], void* grad_filters,
                              const void* grad_out,
                              void* workspace, size_t workspace_bytes, void* stream, void* par_stream);

/* ---- conv2d forward without any allocation ------------------------------------------------------ */

/* Capacity of the library-resident scratch array used by b200_conv2d_forward_noalloc. */
#define B200_CONV2D_NOALLOC_SCRATCH_BYTES (32u << 20)

/* This entry point has no counterpart in the reference (dfdx always takes its patch buffer from
 * `Cuda::get_workspace`).  It is `b200_conv2d_forward` for callers that cannot provide a workspace
 * because they cannot allocate device memory where they run: the GPU's memory is already owned by their
 * own arena, a cudaMalloc (which synchronises the device) is not acceptable in their loop, or they are
 * handed nothing but input and output buffers.  The im2col patch buffer is a fixed
 * B200_CONV2D_NOALLOC_SCRATCH_BYTES array inside the library image; it becomes resident on a GPU when b200_init
 * runs for that GPU (which looks up the array's device address and thereby loads the module that holds it) and
 * stays until the process exits.  The call itself allocates and frees nothing, explicitly or implicitly: free
 * device memory is the same before and after it.
 *   - Limit: b200_conv2d_workspace_bytes(dtype, op, 0) must not exceed the capacity above, otherwise
 *     B200_ERR_LIMIT is returned and nothing is launched (use b200_conv2d_forward with a workspace).
 *   - b200_init(ordinal) must have been called for the current device; it performs the one-time set-up (the
 *     address lookup above), so call it before starting any stream capture and before handing the remaining
 *     device memory to an arena.
 *   - All calls on a device share the one array.  Every call overwrites all of the part it uses, so earlier
 *     contents never leak into a result; but two calls whose GPU work can overlap (different streams, or
 *     different threads without ordering) race on it — serialise them on one stream or with events.
 * Arguments and results are otherwise exactly those of b200_conv2d_forward. */
int b200_conv2d_forward_noalloc(int dtype, const b200_conv2d_op* op,
                                const void* img, const size_t img_strides[4],
                                const void* filters, void* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DFDX_B200_H */
