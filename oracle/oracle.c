/*
 * TEST INFRASTRUCTURE — CPU oracle for the matmul / conv2d hot path.  Not part of the product:
 * only the test-suite, the smoke check and the bench's CPU-baseline leg may load this file.
 *
 * It restates, in plain C with f64 arithmetic, the algorithm of dfdx's `Cpu` device for the
 * path (dfdx v0.13.0; paths relative to that repository):
 *   - strided GEMM ............ dfdx-core/src/tensor_ops/matmul/cpu_kernel.rs:10-36 (`naive_gemm`)
 *                               with the semantics of the `gemm` crate call at :164-184
 *                               (dst = (accum ? dst : 0) + lhs*rhs)
 *   - the four batch drivers ... cpu_kernel.rs:231-288, :290-352, :354-418, :420-486
 *   - conv2d ................... dfdx-core/src/tensor_ops/conv2d/cpu_kernel.rs:9-40 (`unfold_idx`),
 *                               :44-97 (forward im2col + GEMM), :99-172 (backward),
 *                               :221-276 (filter transpose / un-transpose through strides)
 *
 * The arithmetic of the real `Cpu` device lives in the third-party `gemm` crate (0.16.14,
 * dfdx-core/Cargo.toml:38), which is not vendored in the reference tree; what is restated here
 * is its published contract (a strided GEMM).  Inputs of any element type are widened to f64 by
 * the caller, so one set of functions serves f16 / f32 / f64 parity.
 *
 * Parity is pinned by the literal known-answer tests of the reference (tests/golden/*.json,
 * transcribed from matmul/mod.rs:367-702, nn/layers/linear.rs:97-204, conv2d/tests.rs:11-402).
 */
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

typedef struct {
  size_t kernel, stride, padding, dilation, groups, batch;
  size_t chan_in, chan_out, h_in, h_out, w_in, w_out;
} oracle_conv2d_op; /* conv2d/mod.rs:14-29 */

/* matmul/mod.rs:316-325: a 2-D stride pair is legal iff one of the listed patterns matches. */
int oracle_matrix_strides_ok(size_t s0, size_t s1) { return s0 == 1 || s1 == 1; }

/* cpu_kernel.rs:10-36 (loop nest) with gemm-crate semantics (:164-184). */
void oracle_gemm(size_t m, size_t k, size_t n, int accum,
                 const double* a, const size_t as[2],
                 const double* b, const size_t bs[2],
                 double* c, const size_t cs[2]) {
  for (size_t i = 0; i < m; ++i) {
    for (size_t j = 0; j < n; ++j) {
      double acc = 0.0;
      const double* ap = a + as[0] * i;
      const double* bp = b + bs[1] * j;
      for (size_t p = 0; p < k; ++p) acc += ap[as[1] * p] * bp[bs[0] * p];
      double* cp = c + cs[0] * i + cs[1] * j;
      *cp = accum ? *cp + acc : acc;
    }
  }
}

static void row_major(size_t r, size_t c, size_t out[2]) { (void)r; out[0] = c; out[1] = 1; }

/* ---- MatMatKernel (cpu_kernel.rs:231-288) ---------------------------------------------------- */
void oracle_matmat_forward(size_t m, size_t k, size_t n,
                           const double* lhs, const size_t ls[2],
                           const double* rhs, const size_t rs[2], double* out) {
  size_t os[2]; row_major(m, n, os);
  oracle_gemm(m, k, n, 0, lhs, ls, rhs, rs, out, os);
}

void oracle_matmat_backward(size_t m, size_t k, size_t n,
                            const double* lhs, const size_t ls[2], double* grad_lhs,
                            const double* rhs, const size_t rs[2], double* grad_rhs,
                            const double* grad_out) {
  size_t os[2]; row_major(m, n, os);
  size_t rs_t[2] = {rs[1], rs[0]}, ls_t[2] = {ls[1], ls[0]};
  if (grad_lhs) oracle_gemm(m, n, k, 1, grad_out, os, rhs, rs_t, grad_lhs, ls);
  if (grad_rhs) oracle_gemm(k, m, n, 1, lhs, ls_t, grad_out, os, grad_rhs, rs);
}

/* ---- MatMatBrKernel (cpu_kernel.rs:290-352) --------------------------------------------------- */
void oracle_matmat_br_forward(size_t batch, size_t m, size_t k, size_t n,
                              const double* lhs, const size_t ls[3],
                              const double* rhs, const size_t rs[2], double* out) {
  for (size_t b = 0; b < batch; ++b)
    oracle_matmat_forward(m, k, n, lhs + b * ls[0], ls + 1, rhs, rs, out + b * m * n);
}

void oracle_matmat_br_backward(size_t batch, size_t m, size_t k, size_t n,
                               const double* lhs, const size_t ls[3], double* grad_lhs,
                               const double* rhs, const size_t rs[2], double* grad_rhs,
                               const double* grad_out) {
  for (size_t b = 0; b < batch; ++b)
    oracle_matmat_backward(m, k, n, lhs + b * ls[0], ls + 1,
                           grad_lhs ? grad_lhs + b * ls[0] : NULL, rhs, rs, grad_rhs,
                           grad_out + b * m * n);
}

/* ---- MatMatBatch3Kernel (cpu_kernel.rs:354-418) ----------------------------------------------- */
void oracle_matmat_batch3_forward(size_t batch, size_t m, size_t k, size_t n,
                                  const double* lhs, const size_t ls[3],
                                  const double* rhs, const size_t rs[3], double* out) {
  for (size_t b = 0; b < batch; ++b)
    oracle_matmat_forward(m, k, n, lhs + b * ls[0], ls + 1, rhs + b * rs[0], rs + 1,
                          out + b * m * n);
}

void oracle_matmat_batch3_backward(size_t batch, size_t m, size_t k, size_t n,
                                   const double* lhs, const size_t ls[3], double* grad_lhs,
                                   const double* rhs, const size_t rs[3], double* grad_rhs,
                                   const double* grad_out) {
  for (size_t b = 0; b < batch; ++b)
    oracle_matmat_backward(m, k, n, lhs + b * ls[0], ls + 1,
                           grad_lhs ? grad_lhs + b * ls[0] : NULL,
                           rhs + b * rs[0], rs + 1,
                           grad_rhs ? grad_rhs + b * rs[0] : NULL, grad_out + b * m * n);
}

/* ---- MatMatBatch4Kernel (cpu_kernel.rs:420-486) ----------------------------------------------- */
void oracle_matmat_batch4_forward(size_t batch, size_t seq, size_t m, size_t k, size_t n,
                                  const double* lhs, const size_t ls[4],
                                  const double* rhs, const size_t rs[4], double* out) {
  for (size_t b = 0; b < batch; ++b)
    oracle_matmat_batch3_forward(seq, m, k, n, lhs + b * ls[0], ls + 1, rhs + b * rs[0], rs + 1,
                                 out + b * seq * m * n);
}

void oracle_matmat_batch4_backward(size_t batch, size_t seq, size_t m, size_t k, size_t n,
                                   const double* lhs, const size_t ls[4], double* grad_lhs,
                                   const double* rhs, const size_t rs[4], double* grad_rhs,
                                   const double* grad_out) {
  for (size_t b = 0; b < batch; ++b)
    oracle_matmat_batch3_backward(seq, m, k, n, lhs + b * ls[0], ls + 1,
                                  grad_lhs ? grad_lhs + b * ls[0] : NULL,
                                  rhs + b * rs[0], rs + 1,
                                  grad_rhs ? grad_rhs + b * rs[0] : NULL,
                                  grad_out + b * seq * m * n);
}

/* ---- conv2d ----------------------------------------------------------------------------------- */

/* conv2d/mod.rs:143-161: (dim + 2*padding - dilation*(kernel-1) - 1) / stride + 1.
 * Returns (size_t)-1 where the reference's checked_sub would panic. */
size_t oracle_conv2d_out_dim(size_t dim, size_t kernel, size_t stride, size_t padding, size_t dilation) {
  size_t lhs = dim + 2 * padding;
  size_t span = dilation * (kernel - 1) + 1;
  if (lhs < span) return (size_t)-1;
  return (lhs - span) / stride + 1;
}

/* conv2d/cpu_kernel.rs:9-40: which output pixel (if any) input pixel (y,x) feeds through tap (k1,k2). */
static int unfold_idx(const oracle_conv2d_op* op, size_t k1, size_t k2, size_t y, size_t x,
                      size_t* oh_out, size_t* ow_out) {
  size_t oh = y + op->padding;
  if (oh < op->dilation * k1) return 0;
  oh -= op->dilation * k1;
  if (oh % op->stride) return 0;
  oh /= op->stride;
  if (oh >= op->h_out) return 0;
  size_t ow = x + op->padding;
  if (ow < op->dilation * k2) return 0;
  ow -= op->dilation * k2;
  if (ow % op->stride) return 0;
  ow /= op->stride;
  if (ow >= op->w_out) return 0;
  *oh_out = oh; *ow_out = ow;
  return 1;
}

/* Forward of one image (cpu_kernel.rs:44-97): im2col in (c,k1,k2,oh,ow) order, then per group
 * out(O/G, OH*OW) = filters(O/G, C/G*K*K) * patches(C/G*K*K, OH*OW). */
static void conv2d_fwd_one(const oracle_conv2d_op* op, const double* img, const size_t is[3],
                           const double* filters, double* out, double* buf) {
  const size_t K = op->kernel, npos = op->h_out * op->w_out;
  size_t i = 0;
  for (size_t c = 0; c < op->chan_in; ++c)
    for (size_t k1 = 0; k1 < K; ++k1)
      for (size_t k2 = 0; k2 < K; ++k2)
        for (size_t oh = 0; oh < op->h_out; ++oh) {
          size_t y = oh * op->stride + op->dilation * k1 - op->padding; /* wraps when padded */
          for (size_t ow = 0; ow < op->w_out; ++ow, ++i) {
            size_t x = ow * op->stride + op->dilation * k2 - op->padding;
            buf[i] = (y < op->h_in && x < op->w_in) ? img[c * is[0] + y * is[1] + x * is[2]] : 0.0;
          }
        }
  const size_t m = op->chan_out / op->groups, k = (op->chan_in / op->groups) * K * K, n = npos;
  size_t fs[2] = {k, 1}, bs[2] = {n, 1}, os[2] = {n, 1};
  for (size_t g = 0; g < op->groups; ++g)
    oracle_gemm(m, k, n, 0, filters + g * m * k, fs, buf + g * k * n, bs, out + g * m * n, os);
}

/* cpu_kernel.rs:182-219.  img_strides is the 4-D element stride of the image; filters are
 * contiguous (O, C/G, K, K); out is contiguous (B, O, OH, OW).  Returns 0, or -1 on allocation failure. */
int oracle_conv2d_forward(const oracle_conv2d_op* op, const double* img, const size_t img_strides[4],
                          const double* filters, double* out) {
  size_t nbuf = op->chan_in * op->kernel * op->kernel * op->h_out * op->w_out;
  double* buf = (double*)malloc((nbuf ? nbuf : 1) * sizeof(double));
  if (!buf) return -1;
  for (size_t b = 0; b < op->batch; ++b)
    conv2d_fwd_one(op, img + b * img_strides[0], img_strides + 1, filters,
                   out + b * op->chan_out * op->h_out * op->w_out, buf);
  free(buf);
  return 0;
}

/* cpu_kernel.rs:99-172 for one image: unfold grad_out into (o,k1,k2,y,x) patches, then
 *   grad_img(C/G, H*W)        += filters_tr(C/G, O/G*K*K) * patches(O/G*K*K, H*W)
 *   grad_filters_tr(C/G, O/G*K*K) += img(C/G, H*W) * patches^T(H*W, O/G*K*K). */
static void conv2d_bwd_one(const oracle_conv2d_op* op, const double* img, double* grad_img,
                           const double* ftr, double* grad_ftr, const double* grad_out, double* buf) {
  const size_t K = op->kernel, hw = op->h_in * op->w_in;
  size_t i = 0;
  for (size_t o = 0; o < op->chan_out; ++o)
    for (size_t k1 = 0; k1 < K; ++k1)
      for (size_t k2 = 0; k2 < K; ++k2)
        for (size_t y = 0; y < op->h_in; ++y)
          for (size_t x = 0; x < op->w_in; ++x, ++i) {
            size_t oh, ow;
            buf[i] = unfold_idx(op, k1, k2, y, x, &oh, &ow)
                         ? grad_out[o * (op->h_out * op->w_out) + oh * op->w_out + ow] : 0.0;
          }
  const size_t m = op->chan_in / op->groups, kk = (op->chan_out / op->groups) * K * K;
  {
    size_t as[2] = {kk, 1}, bs[2] = {hw, 1}, cs[2] = {hw, 1};
    for (size_t g = 0; g < op->groups; ++g)
      oracle_gemm(m, kk, hw, 1, ftr + g * m * kk, as, buf + g * kk * hw, bs, grad_img + g * m * hw, cs);
  }
  {
    size_t as[2] = {hw, 1}, bs[2] = {1, hw}, cs[2] = {kk, 1};
    for (size_t g = 0; g < op->groups; ++g)
      oracle_gemm(m, hw, kk, 1, img + g * m * hw, as, buf + g * hw * kk, bs, grad_ftr + g * m * kk, cs);
  }
}

/* cpu_kernel.rs:221-279.  img / grad_img contiguous (B,C,H,W); filters and grad_filters are
 * addressed through the 4-D filter strides; grad_out contiguous (B,O,OH,OW).  Gradients accumulate. */
int oracle_conv2d_backward(const oracle_conv2d_op* op, const double* img, double* grad_img,
                           const double* filters, const size_t fstr[4], double* grad_filters,
                           const double* grad_out) {
  const size_t K = op->kernel, G = op->groups, cg = op->chan_in / G, og = op->chan_out / G;
  const size_t nf = G * cg * og * K * K;
  const size_t nbuf = op->chan_out * K * K * op->h_in * op->w_in;
  double* buf = (double*)malloc((nbuf ? nbuf : 1) * sizeof(double));
  double* ftr = (double*)malloc((nf ? nf : 1) * sizeof(double));
  double* gftr = (double*)calloc(nf ? nf : 1, sizeof(double));
  if (!buf || !ftr || !gftr) { free(buf); free(ftr); free(gftr); return -1; }
  /* (G, C/G, O/G, K, K) <- (O, C/G, K, K) through strides */
  size_t i = 0;
  for (size_t g = 0; g < G; ++g)
    for (size_t c = 0; c < cg; ++c)
      for (size_t o = 0; o < og; ++o)
        for (size_t k1 = 0; k1 < K; ++k1)
          for (size_t k2 = 0; k2 < K; ++k2, ++i)
            ftr[i] = filters[(g * og + o) * fstr[0] + c * fstr[1] + k1 * fstr[2] + k2 * fstr[3]];
  const size_t img_item = op->chan_in * op->h_in * op->w_in;
  const size_t out_item = op->chan_out * op->h_out * op->w_out;
  for (size_t b = 0; b < op->batch; ++b)
    conv2d_bwd_one(op, img + b * img_item, grad_img + b * img_item, ftr, gftr,
                   grad_out + b * out_item, buf);
  i = 0;
  for (size_t g = 0; g < G; ++g)
    for (size_t c = 0; c < cg; ++c)
      for (size_t o = 0; o < og; ++o)
        for (size_t k1 = 0; k1 < K; ++k1)
          for (size_t k2 = 0; k2 < K; ++k2, ++i)
            grad_filters[(g * og + o) * fstr[0] + c * fstr[1] + k1 * fstr[2] + k2 * fstr[3]] += gftr[i];
  free(buf); free(ftr); free(gftr);
  return 0;
}
