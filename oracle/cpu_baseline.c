/*
 * TEST INFRASTRUCTURE — timed CPU baseline ("port") for the matmul hot path.  Not part of the product:
 * only the bench's CPU-baseline / reference arm and the test-suite may load this file.
 *
 * dfdx's `Cpu` device computes this path with the third-party `gemm` crate (0.16.14) on all Rayon
 * threads (dfdx-core/src/tensor_ops/matmul/cpu_kernel.rs:164-184).  That crate is not in the
 * reference tree and no Rust toolchain exists here, so this file is a stand-in with the same call
 * structure: the kernel-trait drivers loop over the batch and issue one strided f32 GEMM per item
 * (cpu_kernel.rs:231-288 MatMat, :290-352 MatMatBr), and the GEMM is a cache-blocked, packed,
 * AVX2+FMA kernel parallelised with pthreads over output blocks.
 */
#include <stddef.h>
#include <stdlib.h>
#include <string.h>
#include <pthread.h>
#include <unistd.h>

typedef float v8 __attribute__((vector_size(32), aligned(4)));

enum { MR = 6, NR = 16, KC = 256, MB = 96, NB = 512, MAX_THREADS = 256 };

int cpu_baseline_supported(void) {
  __builtin_cpu_init();
  return __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma");
}

static int g_threads = 0;
void cpu_baseline_set_threads(int n) { g_threads = n; }
int cpu_baseline_threads(void) {
  if (g_threads > 0) return g_threads;
  long n = sysconf(_SC_NPROCESSORS_ONLN);
  return n > 0 ? (int)n : 1;
}

/* acc[MR][NR] = sum_p pa[p*MR + i] * pb[p*NR + j] */
static inline void micro_kernel(size_t kc, const float* pa, const float* pb, float* acc) {
  v8 c[MR][2];
  for (int i = 0; i < MR; ++i) { c[i][0] = (v8){0}; c[i][1] = (v8){0}; }
  for (size_t p = 0; p < kc; ++p) {
    const v8 b0 = *(const v8*)(pb + p * NR), b1 = *(const v8*)(pb + p * NR + 8);
    for (int i = 0; i < MR; ++i) {
      const float a = pa[p * MR + i];
      const v8 av = {a, a, a, a, a, a, a, a};
      c[i][0] += av * b0;
      c[i][1] += av * b1;
    }
  }
  for (int i = 0; i < MR; ++i) { *(v8*)(acc + i * NR) = c[i][0]; *(v8*)(acc + i * NR + 8) = c[i][1]; }
}

typedef struct {
  size_t m, k, n; int accum;
  const float* a; const size_t* as; const float* b; const size_t* bs; float* c; const size_t* cs;
  size_t mblocks, nblocks;
  size_t next;            /* shared work counter (atomic) */
} gemm_job;

static void gemm_block(const gemm_job* g, size_t bi, size_t bj, float* pa, float* pb) {
  const size_t m = g->m, k = g->k, n = g->n;
  const size_t *as = g->as, *bs = g->bs, *cs = g->cs;
  float acc[MR * NR] __attribute__((aligned(64)));
  const size_t i0 = bi * MB, j0 = bj * NB;
  const size_t mb = m - i0 < MB ? m - i0 : MB, nb = n - j0 < NB ? n - j0 : NB;
  const size_t mp = (mb + MR - 1) / MR, np = (nb + NR - 1) / NR;
  for (size_t p0 = 0; p0 < k || p0 == 0; p0 += KC) {
    const size_t kc = k - p0 < KC ? k - p0 : KC;
    for (size_t ip = 0; ip < mp; ++ip)              /* pack A into MR-row panels */
      for (size_t p = 0; p < kc; ++p)
        for (size_t i = 0; i < MR; ++i) {
          const size_t gi = i0 + ip * MR + i;
          pa[(ip * kc + p) * MR + i] = gi < m ? g->a[gi * as[0] + (p0 + p) * as[1]] : 0.f;
        }
    for (size_t jp = 0; jp < np; ++jp)              /* pack B into NR-column panels */
      for (size_t p = 0; p < kc; ++p)
        for (size_t j = 0; j < NR; ++j) {
          const size_t gj = j0 + jp * NR + j;
          pb[(jp * kc + p) * NR + j] = gj < n ? g->b[(p0 + p) * bs[0] + gj * bs[1]] : 0.f;
        }
    const int add = g->accum || p0 > 0;
    for (size_t ip = 0; ip < mp; ++ip)
      for (size_t jp = 0; jp < np; ++jp) {
        micro_kernel(kc, pa + ip * kc * MR, pb + jp * kc * NR, acc);
        for (size_t i = 0; i < MR; ++i) {
          const size_t gi = i0 + ip * MR + i;
          if (gi >= m) break;
          for (size_t j = 0; j < NR; ++j) {
            const size_t gj = j0 + jp * NR + j;
            if (gj >= n) break;
            float* d = g->c + gi * cs[0] + gj * cs[1];
            *d = add ? *d + acc[i * NR + j] : acc[i * NR + j];
          }
        }
      }
    if (k == 0) break;
  }
}

static void* gemm_worker(void* arg) {
  gemm_job* g = (gemm_job*)arg;
  float* pa = (float*)aligned_alloc(64, sizeof(float) * (MB + MR) * KC);
  float* pb = (float*)aligned_alloc(64, sizeof(float) * (NB + NR) * KC);
  const size_t total = g->mblocks * g->nblocks;
  for (;;) {
    const size_t t = __atomic_fetch_add(&g->next, 1, __ATOMIC_RELAXED);
    if (t >= total) break;
    gemm_block(g, t / g->nblocks, t % g->nblocks, pa, pb);
  }
  free(pa);
  free(pb);
  return NULL;
}

/* dst = (accum ? dst : 0) + a*b with element strides, like `MatMulImpl::<f32>::matmul` (cpu_kernel.rs:148-186),
 * on all host threads (the reference passes Parallelism::Rayon(current_num_threads())). */
void cpu_sgemm(size_t m, size_t k, size_t n, int accum,
               const float* a, const size_t as[2], const float* b, const size_t bs[2],
               float* c, const size_t cs[2]) {
  if (m == 0 || n == 0) return;
  gemm_job g = {m, k, n, accum, a, as, b, bs, c, cs, (m + MB - 1) / MB, (n + NB - 1) / NB, 0};
  size_t nthreads = (size_t)cpu_baseline_threads();
  const size_t total = g.mblocks * g.nblocks;
  if (nthreads > total) nthreads = total;
  if (nthreads > MAX_THREADS) nthreads = MAX_THREADS;
  pthread_t tid[MAX_THREADS];
  size_t started = 0;
  for (size_t t = 1; t < nthreads; ++t)
    if (pthread_create(&tid[started], NULL, gemm_worker, &g) == 0) ++started;
  gemm_worker(&g);
  for (size_t t = 0; t < started; ++t) pthread_join(tid[t], NULL);
}

/* MatMatKernel for Cpu (cpu_kernel.rs:231-288). */
void cpu_matmat_forward(size_t m, size_t k, size_t n, const float* lhs, const size_t ls[2],
                        const float* rhs, const size_t rs[2], float* out) {
  const size_t os[2] = {n, 1};
  cpu_sgemm(m, k, n, 0, lhs, ls, rhs, rs, out, os);
}

void cpu_matmat_backward(size_t m, size_t k, size_t n, const float* lhs, const size_t ls[2], float* grad_lhs,
                         const float* rhs, const size_t rs[2], float* grad_rhs, const float* grad_out) {
  const size_t os[2] = {n, 1}, rs_t[2] = {rs[1], rs[0]}, ls_t[2] = {ls[1], ls[0]};
  cpu_sgemm(m, n, k, 1, grad_out, os, rhs, rs_t, grad_lhs, ls);
  cpu_sgemm(k, m, n, 1, lhs, ls_t, grad_out, os, grad_rhs, rs);
}

/* MatMatBrKernel for Cpu (cpu_kernel.rs:290-352): per-batch loop over the 2-D kernel. */
void cpu_matmat_br_forward(size_t batch, size_t m, size_t k, size_t n, const float* lhs, const size_t ls[3],
                           const float* rhs, const size_t rs[2], float* out) {
  for (size_t b = 0; b < batch; ++b)
    cpu_matmat_forward(m, k, n, lhs + b * ls[0], ls + 1, rhs, rs, out + b * m * n);
}

void cpu_matmat_br_backward(size_t batch, size_t m, size_t k, size_t n, const float* lhs, const size_t ls[3],
                            float* grad_lhs, const float* rhs, const size_t rs[2], float* grad_rhs,
                            const float* grad_out) {
  for (size_t b = 0; b < batch; ++b)
    cpu_matmat_backward(m, k, n, lhs + b * ls[0], ls + 1, grad_lhs + b * ls[0], rhs, rs, grad_rhs,
                        grad_out + b * m * n);
}
