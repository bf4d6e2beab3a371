// Row-wise kernels that sit next to the GEMMs in a Transformer training step: LayerNorm forward / backward and the
// bias gradient (a column sum).  All are HBM-bound: every tensor is read from DRAM once (re-reads of a row hit
// L1 / L2) and written once; statistics and reductions are f32.
//
//   layer_norm_fwd_kernel   y = (x - mean) / sqrt(var + eps) * gamma + beta over the last axis
//                           (dfdx-core/src/tensor_ops/normalize.rs:33-50 as used by dfdx/src/nn/layers/layer_norm1d.rs:87-91:
//                           mean, centred, mean of squares + epsilon, sqrt, divide; then * gamma + beta: nine kernels and
//                           as many passes over the tensor in the reference, one here)
//   layer_norm_bwd_kernel   dx = rstd * (g*gamma - mean(g*gamma) - xhat * mean(g*gamma*xhat)),
//                           dgamma += sum_rows g * xhat,  dbeta += sum_rows g   (the tape entries of the same ops)
//   column_sum_kernel       out[j] += sum_i g[i, j]   (backward of `bias.broadcast_like(&x) + x`, bias1d.rs:66-79)
//   softmax_fwd_kernel      y = softmax(alpha * x) over the last axis = exp(alpha*x - max) / sum exp(alpha*x - max)
//                           (dfdx-core/src/tensor_ops/softmax.rs:36-84: max, subtract, exp, sum, divide: five kernels there)
//   softmax_bwd_kernel      dx (+)= alpha * y * (g - sum_j g_j y_j)   (the tape entries of div, sum, exp and the scalar mul)
// One warp per row; lanes walk the row in 16-byte vectors when the layout allows, element-wise otherwise.
#include "common.cuh"

namespace b200 {

namespace {

template <typename T> struct Vec;
template <> struct Vec<float> { static constexpr int N = 4; };
template <> struct Vec<__half> { static constexpr int N = 8; };

__device__ __forceinline__ float to_f(float x) { return x; }
__device__ __forceinline__ float to_f(__half x) { return __half2float(x); }
template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_f<__half>(float x) { return __float2half_rn(x); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Loads the n (= Vec<T>::N) elements that start at column c of a row into f[]; vec: 16-byte access is legal.
template <typename T>
__device__ __forceinline__ void load_vec(const T* row, int c, int cols, bool vec, float* f) {
  constexpr int N = Vec<T>::N;
  if (vec) {
    const uint4 raw = *reinterpret_cast<const uint4*>(row + c);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int q = 0; q < N; ++q) f[q] = to_f(e[q]);
  } else {
#pragma unroll
    for (int q = 0; q < N; ++q) f[q] = (c + q < cols) ? to_f(row[c + q]) : 0.f;
  }
}
template <typename T>
__device__ __forceinline__ void store_vec(T* row, int c, int cols, bool vec, const float* f) {
  constexpr int N = Vec<T>::N;
  if (vec) {
    uint4 raw;
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int q = 0; q < N; ++q) e[q] = from_f<T>(f[q]);
    *reinterpret_cast<uint4*>(row + c) = raw;
  } else {
#pragma unroll
    for (int q = 0; q < N; ++q)
      if (c + q < cols) row[c + q] = from_f<T>(f[q]);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) layer_norm_fwd_kernel(const T* __restrict__ x, long long x_ld, const T* __restrict__ gamma,
                                                             const T* __restrict__ beta, float eps, T* __restrict__ y,
                                                             long long y_ld, float* __restrict__ stats, long long rows, int cols,
                                                             int vec) {
  constexpr int N = Vec<T>::N;
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * 8 + (threadIdx.x >> 5), nwarps = (long long)gridDim.x * 8;
  const float inv_n = 1.f / (float)cols;
  for (long long r = warp0; r < rows; r += nwarps) {
    const T* xr = x + r * x_ld;
    float s = 0.f;
    for (int c = lane * N; c < cols; c += 32 * N) {
      float f[N];
      load_vec(xr, c, cols, vec, f);
#pragma unroll
      for (int q = 0; q < N; ++q) s += f[q];
    }
    const float mean = warp_sum(s) * inv_n;
    float sq = 0.f;
    for (int c = lane * N; c < cols; c += 32 * N) {
      float f[N];
      load_vec(xr, c, cols, vec, f);
#pragma unroll
      for (int q = 0; q < N; ++q) {
        const float d = (c + q < cols) ? f[q] - mean : 0.f;
        sq = fmaf(d, d, sq);
      }
    }
    const float rstd = 1.f / sqrtf(warp_sum(sq) * inv_n + eps);
    T* yr = y + r * y_ld;
    for (int c = lane * N; c < cols; c += 32 * N) {
      float f[N], gm[N], bt[N];
      load_vec(xr, c, cols, vec, f);
      if (gamma) load_vec(gamma, c, cols, vec, gm);
      if (beta) load_vec(beta, c, cols, vec, bt);
#pragma unroll
      for (int q = 0; q < N; ++q) {
        float v = (f[q] - mean) * rstd;
        if (gamma) v *= gm[q];
        if (beta) v += bt[q];
        f[q] = v;
      }
      store_vec(yr, c, cols, vec, f);
    }
    if (stats && lane == 0) { stats[2 * r] = mean; stats[2 * r + 1] = rstd; }
  }
}

// The same forward with the row kept in registers (cols <= 32 * N * MAXV): one global read per element, all of a
// lane's loads issued before the first use.
template <typename T, int MAXV>
__global__ void __launch_bounds__(256) layer_norm_fwd_reg_kernel(const T* __restrict__ x, long long x_ld,
                                                                 const T* __restrict__ gamma, const T* __restrict__ beta,
                                                                 float eps, T* __restrict__ y, long long y_ld,
                                                                 float* __restrict__ stats, long long rows, int cols, int vec) {
  constexpr int N = Vec<T>::N;
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * 8 + (threadIdx.x >> 5), nwarps = (long long)gridDim.x * 8;
  const float inv_n = 1.f / (float)cols;
  for (long long r = warp0; r < rows; r += nwarps) {
    const T* xr = x + r * x_ld;
    float f[MAXV][N];
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      const int c = (v * 32 + lane) * N;
      if (c < cols) load_vec(xr, c, cols, vec, f[v]);
      else {
#pragma unroll
        for (int q = 0; q < N; ++q) f[v][q] = 0.f;
      }
    }
    float s = 0.f;
#pragma unroll
    for (int v = 0; v < MAXV; ++v)
#pragma unroll
      for (int q = 0; q < N; ++q) s += f[v][q];                // columns beyond `cols` hold zeros
    const float mean = warp_sum(s) * inv_n;
    float sq = 0.f;
#pragma unroll
    for (int v = 0; v < MAXV; ++v)
#pragma unroll
      for (int q = 0; q < N; ++q) {
        const float d = ((v * 32 + lane) * N + q < cols) ? f[v][q] - mean : 0.f;
        sq = fmaf(d, d, sq);
      }
    const float rstd = 1.f / sqrtf(warp_sum(sq) * inv_n + eps);
    T* yr = y + r * y_ld;
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      const int c = (v * 32 + lane) * N;
      if (c < cols) {
        float gm[N], bt[N];
        if (gamma) load_vec(gamma, c, cols, vec, gm);
        if (beta) load_vec(beta, c, cols, vec, bt);
#pragma unroll
        for (int q = 0; q < N; ++q) {
          float o = (f[v][q] - mean) * rstd;
          if (gamma) o *= gm[q];
          if (beta) o += bt[q];
          f[v][q] = o;
        }
        store_vec(yr, c, cols, vec, f[v]);
      }
    }
    if (stats && lane == 0) { stats[2 * r] = mean; stats[2 * r + 1] = rstd; }
  }
}

template <typename T>
__device__ __forceinline__ void unpack_vec(const uint4& raw, float* f) {
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int q = 0; q < Vec<T>::N; ++q) f[q] = to_f(e[q]);
}

// The register kernel for rows that allow 16-byte access, with fewer instructions per row (one warp per row is bound
// by instruction issue): gamma and beta wait in shared memory as f32 (lane-major float4s), the next row's loads are
// issued one row ahead, and a launch-resident grid walks the rows.
constexpr int LN_FWD_VEC_BLOCKS_PER_SM = 3;
// ADD: the normalised row is x + res, rounded to T as a separate add would round it and also written to `sum` (the
// residual connection in front of the LayerNorm, whose backward needs that sum).
template <typename T, int MAXV, bool ADD>
__global__ void __launch_bounds__(256, LN_FWD_VEC_BLOCKS_PER_SM)
    layer_norm_fwd_vec_kernel(const T* __restrict__ x, long long x_ld, const T* __restrict__ res, long long res_ld,
                              T* __restrict__ sum, long long sum_ld, const T* __restrict__ gamma, const T* __restrict__ beta,
                              float eps, T* __restrict__ y, long long y_ld, float* __restrict__ stats, long long rows, int cols) {
  constexpr int N = Vec<T>::N, J = N / 4;
  __shared__ float4 gamma_s[MAXV * J][32], beta_s[MAXV * J][32];
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * 8 + (threadIdx.x >> 5), nwarps = (long long)gridDim.x * 8;
  const float inv_n = 1.f / (float)cols;
  for (int i = threadIdx.x; i < MAXV * J * 32; i += 256) {
    const int vj = i >> 5, ln = i & 31, col = ((vj / J) * 32 + ln) * N + (vj % J) * 4;
    float4 gv = make_float4(1.f, 1.f, 1.f, 1.f), bv = make_float4(0.f, 0.f, 0.f, 0.f);
    if (col < cols) {
      if (gamma) gv = make_float4(to_f(gamma[col]), to_f(gamma[col + 1]), to_f(gamma[col + 2]), to_f(gamma[col + 3]));
      if (beta) bv = make_float4(to_f(beta[col]), to_f(beta[col + 1]), to_f(beta[col + 2]), to_f(beta[col + 3]));
    }
    gamma_s[vj][ln] = gv;
    beta_s[vj][ln] = bv;
  }
  __syncthreads();
  uint4 nx[MAXV], nr[ADD ? MAXV : 1];
  auto fetch = [&](long long r) {
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      if ((v * 32 + lane) * N < cols) {
        nx[v] = *reinterpret_cast<const uint4*>(x + r * x_ld + (v * 32 + lane) * N);
        if constexpr (ADD) nr[v] = *reinterpret_cast<const uint4*>(res + r * res_ld + (v * 32 + lane) * N);
      }
    }
  };
  if (warp0 < rows) fetch(warp0);
  for (long long r = warp0; r < rows; r += nwarps) {
    float f[MAXV][N];
    float s = 0.f;
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      if ((v * 32 + lane) * N < cols) {
        unpack_vec<T>(nx[v], f[v]);
        if constexpr (ADD) {
          float fr[N];
          unpack_vec<T>(nr[v], fr);
#pragma unroll
          for (int q = 0; q < N; ++q) f[v][q] = to_f(from_f<T>(f[v][q] + fr[q]));
          store_vec(sum + r * sum_ld, (v * 32 + lane) * N, cols, true, f[v]);
        }
#pragma unroll
        for (int q = 0; q < N; ++q) s += f[v][q];
      }
    }
    if (r + nwarps < rows) fetch(r + nwarps);
    const float mean = warp_sum(s) * inv_n;
    float sq = 0.f;
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      if ((v * 32 + lane) * N < cols) {
#pragma unroll
        for (int q = 0; q < N; ++q) {
          f[v][q] -= mean;
          sq = fmaf(f[v][q], f[v][q], sq);
        }
      }
    }
    const float rstd = 1.f / sqrtf(warp_sum(sq) * inv_n + eps);
    T* yr = y + r * y_ld;
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      const int c = (v * 32 + lane) * N;
      if (c < cols) {
#pragma unroll
        for (int j = 0; j < J; ++j) {
          const float4 gm = gamma_s[v * J + j][lane], bt = beta_s[v * J + j][lane];
          const float* gmp = reinterpret_cast<const float*>(&gm);
          const float* btp = reinterpret_cast<const float*>(&bt);
#pragma unroll
          for (int e = 0; e < 4; ++e) f[v][j * 4 + e] = fmaf(f[v][j * 4 + e] * rstd, gmp[e], btp[e]);
        }
        store_vec(yr, c, cols, true, f[v]);
      }
    }
    if (stats && lane == 0) { stats[2 * r] = mean; stats[2 * r + 1] = rstd; }
  }
}

// Sums acc[v][q] (this lane's columns (v * 32 + lane) * N + q) over the block's eight warps and adds the result
// into out[] with one vector atomic per four columns; out may be null.  All threads of the block call it.
template <int N, int MAXV>
__device__ __forceinline__ void block_column_sums(float (*red)[32 * N + 1], const float (*acc)[N], float* __restrict__ out,
                                                  int cols, int warp, int lane) {
#pragma unroll
  for (int v = 0; v < MAXV; ++v) {
    if (v * 32 * N >= cols) break;
    __syncthreads();
#pragma unroll
    for (int q = 0; q < N; ++q) red[warp][lane * N + q] = acc[v][q];
    __syncthreads();
    if (out) {
      for (int i = threadIdx.x * 4; i < 32 * N; i += 256 * 4) {
        const int col = v * 32 * N + i;
        if (col < cols) {
          float t[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int w = 0; w < 8; ++w) {
#pragma unroll
            for (int e = 0; e < 4; ++e) t[e] += red[w][i + e];
          }
          if (col + 3 < cols && ((uintptr_t)(out + col) & 15) == 0) {
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(out + col), "f"(t[0]), "f"(t[1]), "f"(t[2]),
                         "f"(t[3]) : "memory");
          } else {
#pragma unroll
            for (int e = 0; e < 4; ++e)
              if (col + e < cols) atomicAdd(out + col + e, t[e]);
          }
        }
      }
    }
  }
}

// MAXV vectors per lane: cols <= 32 * N * MAXV.  Per-lane partial sums of dgamma / dbeta live in registers over all
// rows of the warp, are combined across the block's warps in shared memory and added to global memory once per block.
template <typename T, int MAXV>
__global__ void __launch_bounds__(256) layer_norm_bwd_kernel(const T* __restrict__ x, long long x_ld, const T* __restrict__ gamma,
                                                             const float* __restrict__ stats, const T* __restrict__ g,
                                                             long long g_ld, T* __restrict__ gx, long long gx_ld, int accumulate_x,
                                                             float* __restrict__ ggamma, float* __restrict__ gbeta, long long rows,
                                                             int cols, int vec) {
  constexpr int N = Vec<T>::N;
  __shared__ float red[8][32 * N + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long warp0 = (long long)blockIdx.x * 8 + warp, nwarps = (long long)gridDim.x * 8;
  const float inv_n = 1.f / (float)cols;
  float dg[MAXV][N], db[MAXV][N];
#pragma unroll
  for (int v = 0; v < MAXV; ++v)
#pragma unroll
    for (int q = 0; q < N; ++q) dg[v][q] = db[v][q] = 0.f;

  for (long long r = warp0; r < rows; r += nwarps) {
    const T* xr = x + r * x_ld;
    const T* gr = g + r * g_ld;
    const float mean = stats[2 * r], rstd = stats[2 * r + 1];
    float s1 = 0.f, s2 = 0.f;
    float xh[MAXV][N], gg[MAXV][N];                            // x-hat and g * gamma of this lane's columns
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      const int c = (v * 32 + lane) * N;
      if (c < cols) {
        float fx[N], fg[N], gm[N];
        load_vec(xr, c, cols, vec, fx);
        load_vec(gr, c, cols, vec, fg);
        if (gamma) load_vec(gamma, c, cols, vec, gm);
#pragma unroll
        for (int q = 0; q < N; ++q) {
          xh[v][q] = (c + q < cols) ? (fx[q] - mean) * rstd : 0.f;
          gg[v][q] = gamma ? fg[q] * gm[q] : fg[q];
          s1 += gg[v][q];
          s2 = fmaf(gg[v][q], xh[v][q], s2);
          dg[v][q] = fmaf(fg[q], xh[v][q], dg[v][q]);
          db[v][q] += fg[q];
        }
      } else {
#pragma unroll
        for (int q = 0; q < N; ++q) xh[v][q] = gg[v][q] = 0.f;
      }
    }
    const float c1 = warp_sum(s1) * inv_n, c2 = warp_sum(s2) * inv_n;
    if (gx) {
      T* or_ = gx + r * gx_ld;
#pragma unroll
      for (int v = 0; v < MAXV; ++v) {
        const int c = (v * 32 + lane) * N;
        if (c < cols) {
          float d[N], old[N];
          if (accumulate_x) load_vec(or_, c, cols, vec, old);
#pragma unroll
          for (int q = 0; q < N; ++q) {
            d[q] = rstd * (gg[v][q] - c1 - xh[v][q] * c2);
            if (accumulate_x) d[q] += old[q];
          }
          store_vec(or_, c, cols, vec, d);
        }
      }
    }
  }
  block_column_sums<N, MAXV>(red, dg, ggamma, cols, warp, lane);
  block_column_sums<N, MAXV>(red, db, gbeta, cols, warp, lane);
}

// The same for rows that allow 16-byte access, arranged for few instructions per row (with one warp per row the
// kernel is bound by instruction issue, not by DRAM): x and g are converted once, the row's result is two fused
// multiply-adds per element, gamma as f32 and the running column sums for dgamma / dbeta live in shared memory
// (lane-major float4s; the sums are touched only by their owner until the end), which frees the registers for the
// next row's loads, issued one row ahead.  Two blocks per SM, one launch-resident wave.

constexpr int LN_BWD_VEC_BLOCKS_PER_SM = 2;
// GSUM: a third running sum, of this op's grad_x as stored (rounded to T): the bias gradient of a Linear whose output
// fed the LayerNorm (through a residual add, which passes the gradient on unchanged).
template <typename T, int MAXV, bool GSUM>
struct LnBwdVecSmem {
  static constexpr int J = Vec<T>::N / 4, KINDS = GSUM ? 3 : 2;
  float4 acc[8][KINDS][MAXV * J][32];                          // [warp][g * x-hat | g | grad_x][vector, quarter][lane]
  float4 gamma[MAXV * J][32];                                  // gamma (ones without it) in the same order
};
template <typename T, int MAXV, bool GSUM>
__global__ void __launch_bounds__(256, LN_BWD_VEC_BLOCKS_PER_SM)
    layer_norm_bwd_vec_kernel(const T* __restrict__ x, long long x_ld, const T* __restrict__ gamma, const float* __restrict__ stats,
                              const T* __restrict__ g, long long g_ld, T* __restrict__ gx, long long gx_ld, int accumulate_x,
                              float* __restrict__ ggamma, float* __restrict__ gbeta, float* __restrict__ gxsum, long long rows,
                              int cols) {
  constexpr int N = Vec<T>::N, J = N / 4, KINDS = GSUM ? 3 : 2;
  extern __shared__ __align__(16) unsigned char ln_bwd_smem[];
  LnBwdVecSmem<T, MAXV, GSUM>& sm = *reinterpret_cast<LnBwdVecSmem<T, MAXV, GSUM>*>(ln_bwd_smem);
  auto& acc = sm.acc;
  auto& gamma_s = sm.gamma;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long warp0 = (long long)blockIdx.x * 8 + warp, nwarps = (long long)gridDim.x * 8;
  const float inv_n = 1.f / (float)cols;
#pragma unroll
  for (int i = 0; i < MAXV * J; ++i)
#pragma unroll
    for (int kd = 0; kd < KINDS; ++kd) acc[warp][kd][i][lane] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int i = threadIdx.x; i < MAXV * J * 32; i += 256) {
    const int vj = i >> 5, ln = i & 31, col = ((vj / J) * 32 + ln) * N + (vj % J) * 4;
    float4 gv = make_float4(1.f, 1.f, 1.f, 1.f);
    if (gamma && col < cols) gv = make_float4(to_f(gamma[col]), to_f(gamma[col + 1]), to_f(gamma[col + 2]), to_f(gamma[col + 3]));
    gamma_s[vj][ln] = gv;
  }
  __syncthreads();
  uint4 nx[MAXV], ng[MAXV];
  float nmean = 0.f, nrstd = 0.f;
  auto fetch = [&](long long r) {
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      const int c = (v * 32 + lane) * N;
      if (c < cols) {
        nx[v] = *reinterpret_cast<const uint4*>(x + r * x_ld + c);
        ng[v] = *reinterpret_cast<const uint4*>(g + r * g_ld + c);
      }
    }
    nmean = stats[2 * r]; nrstd = stats[2 * r + 1];
  };
  if (warp0 < rows) fetch(warp0);
  for (long long r = warp0; r < rows; r += nwarps) {
    // x-hat = x * rstd - mean * rstd; d = rstd * (gg - c1 - x-hat * c2) as two fused multiply-adds
    const float rstd = nrstd, shift = -nmean * nrstd;
    float xh[MAXV][N], gg[MAXV][N];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      if ((v * 32 + lane) * N < cols) {
        float fg[N];
        unpack_vec<T>(nx[v], xh[v]);
        unpack_vec<T>(ng[v], fg);
#pragma unroll
        for (int j = 0; j < J; ++j) {
          float4 dg = acc[warp][0][v * J + j][lane], db = acc[warp][1][v * J + j][lane];
          const float4 gm = gamma_s[v * J + j][lane];
          float* dgp = reinterpret_cast<float*>(&dg);
          float* dbp = reinterpret_cast<float*>(&db);
          const float* gmp = reinterpret_cast<const float*>(&gm);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int q = j * 4 + e;
            xh[v][q] = fmaf(xh[v][q], rstd, shift);
            gg[v][q] = fg[q] * gmp[e];
            s1 += gg[v][q];
            s2 = fmaf(gg[v][q], xh[v][q], s2);
            dgp[e] = fmaf(fg[q], xh[v][q], dgp[e]);
            dbp[e] += fg[q];
          }
          acc[warp][0][v * J + j][lane] = dg;
          acc[warp][1][v * J + j][lane] = db;
        }
      }
    }
    if (r + nwarps < rows) fetch(r + nwarps);                  // this row's packed copy is consumed: reuse its registers
    const float c1 = warp_sum(s1) * inv_n, c2 = warp_sum(s2) * inv_n;
    if (gx) {
      T* or_ = gx + r * gx_ld;
      const float k0 = -rstd * c1, k2 = -rstd * c2;
#pragma unroll
      for (int v = 0; v < MAXV; ++v) {
        const int c = (v * 32 + lane) * N;
        if (c < cols) {
          float d[N];
          if (accumulate_x) {
            const uint4 ro = *reinterpret_cast<const uint4*>(or_ + c);
            unpack_vec<T>(ro, d);
          }
#pragma unroll
          for (int q = 0; q < N; ++q) {
            const float t = fmaf(rstd, gg[v][q], fmaf(k2, xh[v][q], k0));
            d[q] = accumulate_x ? d[q] + t : t;
            if constexpr (GSUM) xh[v][q] = to_f(from_f<T>(t));   // x-hat is no longer needed: keep what is stored
          }
          store_vec(or_, c, cols, true, d);
          if constexpr (GSUM) {
#pragma unroll
            for (int j = 0; j < J; ++j) {
              float4 a = acc[warp][2][v * J + j][lane];
              a.x += xh[v][j * 4]; a.y += xh[v][j * 4 + 1]; a.z += xh[v][j * 4 + 2]; a.w += xh[v][j * 4 + 3];
              acc[warp][2][v * J + j][lane] = a;
            }
          }
        }
      }
    }
  }
  __syncthreads();
  // threads 0..127 add the eight warps' sums of g * x-hat into dgamma, threads 128..255 those of g into dbeta; then
  // (GSUM) threads 0..127 those of grad_x
#pragma unroll 1
  for (int pass = 0; pass < (GSUM ? 2 : 1); ++pass) {
  const int kind = pass ? 2 : (threadIdx.x >> 7);
  float* out = pass ? gxsum : (kind ? gbeta : ggamma);
  if (pass && threadIdx.x >= 128) out = nullptr;
  if (out) {
    for (int i = threadIdx.x & 127; i < MAXV * J * 32; i += 128) {
      const int vj = i >> 5, ln = i & 31, col = ((vj / J) * 32 + ln) * N + (vj % J) * 4;
      if (col < cols) {                                        // cols is a multiple of N here: the four columns exist
        float4 t = acc[0][kind][vj][ln];
#pragma unroll
        for (int w = 1; w < 8; ++w) {
          const float4 u = acc[w][kind][vj][ln];
          t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w;
        }
        if (((uintptr_t)(out + col) & 15) == 0) {
          asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(out + col), "f"(t.x), "f"(t.y), "f"(t.z), "f"(t.w)
                       : "memory");
        } else {
          atomicAdd(out + col, t.x); atomicAdd(out + col + 1, t.y); atomicAdd(out + col + 2, t.z); atomicAdd(out + col + 3, t.w);
        }
      }
    }
  }
  }
}

// out[j] += sum_i g[i, j].  grid.x walks column slabs of 32*N, grid.y row slabs; one atomic per column and block.
template <typename T>
__global__ void __launch_bounds__(256) column_sum_kernel(const T* __restrict__ g, long long ld, float* __restrict__ out,
                                                         long long rows, int cols, int vec) {
  constexpr int N = Vec<T>::N;
  __shared__ float red[8][32 * N + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = (blockIdx.x * 32 + lane) * N;
  float acc[N];
#pragma unroll
  for (int q = 0; q < N; ++q) acc[q] = 0.f;
  if (c < cols) {
    const long long step = (long long)gridDim.y * 8;
    long long r = (long long)blockIdx.y * 8 + warp;
    for (; r + 3 * step < rows; r += 4 * step) {             // four independent loads in flight per lane
      float f[4][N];
#pragma unroll
      for (int u = 0; u < 4; ++u) load_vec(g + (r + u * step) * ld, c, cols, vec, f[u]);
#pragma unroll
      for (int q = 0; q < N; ++q) acc[q] += (f[0][q] + f[1][q]) + (f[2][q] + f[3][q]);
    }
    for (; r < rows; r += step) {
      float f[N];
      load_vec(g + r * ld, c, cols, vec, f);
#pragma unroll
      for (int q = 0; q < N; ++q) acc[q] += f[q];
    }
  }
#pragma unroll
  for (int q = 0; q < N; ++q) red[warp][lane * N + q] = acc[q];
  __syncthreads();
  for (int i = threadIdx.x * 4; i < 32 * N; i += 256 * 4) {
    const int col = blockIdx.x * 32 * N + i;
    if (col < cols) {
      float t[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int w = 0; w < 8; ++w) {
#pragma unroll
        for (int e = 0; e < 4; ++e) t[e] += red[w][i + e];
      }
      if (col + 3 < cols && ((uintptr_t)(out + col) & 15) == 0) {
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(out + col), "f"(t[0]), "f"(t[1]), "f"(t[2]),
                     "f"(t[3]) : "memory");
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (col + e < cols) atomicAdd(out + col + e, t[e]);
      }
    }
  }
}

// sum[r, :] = a[r, :] + b[r, :] (the fallback of the fused add + LayerNorm for rows the vector kernel does not take).
template <typename T>
__global__ void __launch_bounds__(256) add_rows_kernel(const T* __restrict__ a, long long a_ld, const T* __restrict__ b,
                                                       long long b_ld, T* __restrict__ sum, long long sum_ld, long long rows,
                                                       int cols) {
  const long long total = rows * (long long)cols;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
    const long long r = i / cols;
    const int c = (int)(i - r * cols);
    sum[r * sum_ld + c] = from_f<T>(to_f(a[r * a_ld + c]) + to_f(b[r * b_ld + c]));
  }
}

// ReLU's backward and the bias gradient behind it in one pass: g[i, j] = y[i, j] > 0 ? g[i, j] : 0 (in place) and
// out[j] += sum_i g[i, j].  Same decomposition as column_sum_kernel.
template <typename T>
__global__ void __launch_bounds__(256) relu_bwd_column_sum_kernel(const T* __restrict__ y, long long y_ld, T* __restrict__ g,
                                                                  long long ld, float* __restrict__ out, long long rows, int cols,
                                                                  int vec) {
  constexpr int N = Vec<T>::N;
  __shared__ float red[8][32 * N + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = (blockIdx.x * 32 + lane) * N;
  float acc[N];
#pragma unroll
  for (int q = 0; q < N; ++q) acc[q] = 0.f;
  if (c < cols) {
    const long long step = (long long)gridDim.y * 8;
    long long r = (long long)blockIdx.y * 8 + warp;
    for (; r + step < rows; r += 2 * step) {                  // two rows (four loads) in flight per lane
      float fg[2][N], fy[2][N];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        load_vec(g + (r + u * step) * ld, c, cols, vec, fg[u]);
        load_vec(y + (r + u * step) * y_ld, c, cols, vec, fy[u]);
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
#pragma unroll
        for (int q = 0; q < N; ++q) {
          fg[u][q] = fy[u][q] > 0.f ? fg[u][q] : 0.f;
          acc[q] += fg[u][q];
        }
        store_vec(g + (r + u * step) * ld, c, cols, vec, fg[u]);
      }
    }
    for (; r < rows; r += step) {
      float fg[N], fy[N];
      load_vec(g + r * ld, c, cols, vec, fg);
      load_vec(y + r * y_ld, c, cols, vec, fy);
#pragma unroll
      for (int q = 0; q < N; ++q) {
        fg[q] = fy[q] > 0.f ? fg[q] : 0.f;
        acc[q] += fg[q];
      }
      store_vec(g + r * ld, c, cols, vec, fg);
    }
  }
#pragma unroll
  for (int q = 0; q < N; ++q) red[warp][lane * N + q] = acc[q];
  __syncthreads();
  if (out == nullptr) return;
  for (int i = threadIdx.x * 4; i < 32 * N; i += 256 * 4) {
    const int col = blockIdx.x * 32 * N + i;
    if (col < cols) {
      float t[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int w = 0; w < 8; ++w) {
#pragma unroll
        for (int e = 0; e < 4; ++e) t[e] += red[w][i + e];
      }
      if (col + 3 < cols && ((uintptr_t)(out + col) & 15) == 0) {
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(out + col), "f"(t[0]), "f"(t[1]), "f"(t[2]),
                     "f"(t[3]) : "memory");
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (col + e < cols) atomicAdd(out + col + e, t[e]);
      }
    }
  }
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// One warp per row, the row kept in registers (cols <= 32 * N * MAXV) or re-read from L1 / L2 (MAXV == 0).
template <typename T, int MAXV>
__global__ void __launch_bounds__(256) softmax_fwd_kernel(const T* __restrict__ x, long long x_ld, float alpha,
                                                          T* __restrict__ y, long long y_ld, long long rows, int cols, int vec) {
  constexpr int N = Vec<T>::N;
  constexpr float LOG2E = 1.4426950408889634f;
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * 8 + (threadIdx.x >> 5), nwarps = (long long)gridDim.x * 8;
  // t = alpha * x is rounded to f32 as the reference's scalar multiply rounds it; the maximum is subtracted before
  // the change of base, so large inputs lose nothing: exp(t - m) = exp2((t - m) * log2e)
  for (long long r = warp0; r < rows; r += nwarps) {
    const T* xr = x + r * x_ld;
    T* yr = y + r * y_ld;
    if constexpr (MAXV > 0) {
      float f[MAXV][N];
      float mx = -INFINITY;
#pragma unroll
      for (int v = 0; v < MAXV; ++v) {
        const int c = (v * 32 + lane) * N;
        if (c < cols) load_vec(xr, c, cols, vec, f[v]);
#pragma unroll
        for (int q = 0; q < N; ++q) {
          f[v][q] = (c + q < cols) ? f[v][q] * alpha : -INFINITY;
          mx = fmaxf(mx, f[v][q]);
        }
      }
      mx = warp_max(mx);
      if (mx == -INFINITY) mx = 0.f;                         // a row of -inf: exp2(-inf - 0) = 0, 0/0 -> NaN as the reference
      float s = 0.f;
#pragma unroll
      for (int v = 0; v < MAXV; ++v)
#pragma unroll
        for (int q = 0; q < N; ++q) { f[v][q] = exp2f((f[v][q] - mx) * LOG2E); s += f[v][q]; }
      const float inv = 1.f / warp_sum(s);
#pragma unroll
      for (int v = 0; v < MAXV; ++v) {
        const int c = (v * 32 + lane) * N;
#pragma unroll
        for (int q = 0; q < N; ++q) f[v][q] *= inv;
        if (c < cols) store_vec(yr, c, cols, vec, f[v]);
      }
    } else {
      float mx = -INFINITY;
      for (int c = lane * N; c < cols; c += 32 * N) {
        float f[N];
        load_vec(xr, c, cols, vec, f);
#pragma unroll
        for (int q = 0; q < N; ++q)
          if (c + q < cols) mx = fmaxf(mx, f[q] * alpha);
      }
      mx = warp_max(mx);
      if (mx == -INFINITY) mx = 0.f;
      float s = 0.f;
      for (int c = lane * N; c < cols; c += 32 * N) {
        float f[N];
        load_vec(xr, c, cols, vec, f);
#pragma unroll
        for (int q = 0; q < N; ++q)
          if (c + q < cols) s += exp2f((f[q] * alpha - mx) * LOG2E);
      }
      const float inv = 1.f / warp_sum(s);
      for (int c = lane * N; c < cols; c += 32 * N) {
        float f[N];
        load_vec(xr, c, cols, vec, f);
#pragma unroll
        for (int q = 0; q < N; ++q) f[q] = exp2f((f[q] * alpha - mx) * LOG2E) * inv;
        store_vec(yr, c, cols, vec, f);
      }
    }
  }
}

template <typename T, int MAXV>
__global__ void __launch_bounds__(256) softmax_bwd_kernel(const T* __restrict__ y, long long y_ld, const T* __restrict__ g,
                                                          long long g_ld, float alpha, T* __restrict__ gx, long long gx_ld,
                                                          int accumulate, long long rows, int cols, int vec) {
  constexpr int N = Vec<T>::N;
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * 8 + (threadIdx.x >> 5), nwarps = (long long)gridDim.x * 8;
  for (long long r = warp0; r < rows; r += nwarps) {
    const T* yr = y + r * y_ld;
    const T* gr = g + r * g_ld;
    T* dr = gx + r * gx_ld;
    if constexpr (MAXV > 0) {
      float yv[MAXV][N], gv[MAXV][N];
      float dot = 0.f;
#pragma unroll
      for (int v = 0; v < MAXV; ++v) {
        const int c = (v * 32 + lane) * N;
        if (c < cols) { load_vec(yr, c, cols, vec, yv[v]); load_vec(gr, c, cols, vec, gv[v]); }
#pragma unroll
        for (int q = 0; q < N; ++q) {
          if (c + q >= cols) { yv[v][q] = 0.f; gv[v][q] = 0.f; }
          dot = fmaf(yv[v][q], gv[v][q], dot);
        }
      }
      dot = warp_sum(dot);
#pragma unroll
      for (int v = 0; v < MAXV; ++v) {
        const int c = (v * 32 + lane) * N;
        if (c >= cols) continue;
        float o[N];
        if (accumulate) load_vec(dr, c, cols, vec, o);
#pragma unroll
        for (int q = 0; q < N; ++q) {
          const float d = alpha * yv[v][q] * (gv[v][q] - dot);
          o[q] = accumulate ? o[q] + d : d;
        }
        store_vec(dr, c, cols, vec, o);
      }
    } else {
      float dot = 0.f;
      for (int c = lane * N; c < cols; c += 32 * N) {
        float a[N], b[N];
        load_vec(yr, c, cols, vec, a);
        load_vec(gr, c, cols, vec, b);
#pragma unroll
        for (int q = 0; q < N; ++q)
          if (c + q < cols) dot = fmaf(a[q], b[q], dot);
      }
      dot = warp_sum(dot);
      for (int c = lane * N; c < cols; c += 32 * N) {
        float a[N], b[N], o[N];
        load_vec(yr, c, cols, vec, a);
        load_vec(gr, c, cols, vec, b);
        if (accumulate) load_vec(dr, c, cols, vec, o);
#pragma unroll
        for (int q = 0; q < N; ++q) {
          const float d = alpha * a[q] * (b[q] - dot);
          o[q] = accumulate ? o[q] + d : d;
        }
        store_vec(dr, c, cols, vec, o);
      }
    }
  }
}

bool vec_ok(size_t es, int64_t cols, std::initializer_list<int64_t> lds, std::initializer_list<const void*> ptrs) {
  const int64_t n = 16 / (int64_t)es;
  if (cols % n) return false;
  for (int64_t ld : lds)
    if (ld % n) return false;
  for (const void* p : ptrs)
    if ((uintptr_t)p & 15) return false;
  return true;
}

template <typename T>
int ln_forward_t(int64_t rows, int64_t cols, const void* x, int64_t x_ld, const void* gamma, const void* beta, double eps,
                 void* y, int64_t y_ld, float* stats, cudaStream_t stream) {
  DeviceState* ds = device_state();
  const int vec = vec_ok(sizeof(T), cols, {x_ld, y_ld}, {x, y, gamma, beta}) ? 1 : 0;
  const int64_t vecs = (cols + 32 * Vec<T>::N - 1) / (32 * Vec<T>::N);
  const bool fast = vec && vecs <= 2;
  long long blocks = (rows + 7) / 8;
  const long long cap = (long long)ds->sm_count * (fast ? LN_FWD_VEC_BLOCKS_PER_SM : 16);
  if (blocks > cap) blocks = cap;
  auto launch = [&](auto kernel) {
    kernel<<<(unsigned)blocks, 256, 0, stream>>>((const T*)x, x_ld, (const T*)gamma, (const T*)beta, (float)eps, (T*)y, y_ld,
                                                 stats, rows, (int)cols, vec);
  };
  if (fast) {
    layer_norm_fwd_vec_kernel<T, 2, false><<<(unsigned)blocks, 256, 0, stream>>>(
        (const T*)x, x_ld, nullptr, 0, nullptr, 0, (const T*)gamma, (const T*)beta, (float)eps, (T*)y, y_ld, stats, rows, (int)cols);
  } else if (vecs <= 2) launch(layer_norm_fwd_reg_kernel<T, 2>);
  else if (vecs <= 4) launch(layer_norm_fwd_reg_kernel<T, 4>);
  else if (vecs <= 8) launch(layer_norm_fwd_reg_kernel<T, 8>);
  else launch(layer_norm_fwd_kernel<T>);                     // long rows: three passes, re-reads hit L1 / L2
  count_launch(false);
  return note_cuda_error(cudaGetLastError(), "layer_norm forward launch");
}

// y = LayerNorm(a + b), sum = a + b: one kernel for rows the vector kernel takes, otherwise an add followed by the
// plain LayerNorm.
template <typename T>
int add_ln_forward_t(int64_t rows, int64_t cols, const void* a, int64_t a_ld, const void* b, int64_t b_ld, void* sum,
                     int64_t sum_ld, const void* gamma, const void* beta, double eps, void* y, int64_t y_ld, float* stats,
                     cudaStream_t stream) {
  DeviceState* ds = device_state();
  const int64_t vecs = (cols + 32 * Vec<T>::N - 1) / (32 * Vec<T>::N);
  if (vecs <= 2 && vec_ok(sizeof(T), cols, {a_ld, b_ld, sum_ld, y_ld}, {a, b, sum, y, gamma, beta})) {
    long long blocks = (rows + 7) / 8;
    const long long cap = (long long)ds->sm_count * LN_FWD_VEC_BLOCKS_PER_SM;
    if (blocks > cap) blocks = cap;
    layer_norm_fwd_vec_kernel<T, 2, true><<<(unsigned)blocks, 256, 0, stream>>>(
        (const T*)a, a_ld, (const T*)b, b_ld, (T*)sum, sum_ld, (const T*)gamma, (const T*)beta, (float)eps, (T*)y, y_ld, stats,
        rows, (int)cols);
    count_launch(false);
    return note_cuda_error(cudaGetLastError(), "add + layer_norm forward launch");
  }
  const long long total = rows * cols;
  long long blocks = (total + 255) / 256;
  if (blocks > (long long)ds->sm_count * 16) blocks = (long long)ds->sm_count * 16;
  add_rows_kernel<T><<<(unsigned)blocks, 256, 0, stream>>>((const T*)a, a_ld, (const T*)b, b_ld, (T*)sum, sum_ld, rows, (int)cols);
  count_launch(false);
  const int rc = note_cuda_error(cudaGetLastError(), "row add launch");
  if (rc) return rc;
  return ln_forward_t<T>(rows, cols, sum, sum_ld, gamma, beta, eps, y, y_ld, stats, stream);
}

template <typename T>
int column_sum_t(int64_t rows, int64_t cols, const void* g, int64_t ld, float* out, cudaStream_t stream);

// gxsum (may be NULL): receives the column sums of grad_x; needs grad_x written (not accumulated).
template <typename T>
int ln_backward_t(int64_t rows, int64_t cols, const void* x, int64_t x_ld, const void* gamma, const float* stats, const void* g,
                  int64_t g_ld, void* gx, int64_t gx_ld, int accumulate_x, float* ggamma, float* gbeta, float* gxsum,
                  cudaStream_t stream) {
  DeviceState* ds = device_state();
  constexpr int N = Vec<T>::N;
  const int vec = vec_ok(sizeof(T), cols, {x_ld, g_ld, gx ? gx_ld : 0}, {x, g, gx, gamma}) ? 1 : 0;
  const int64_t vecs = (cols + 32 * N - 1) / (32 * N);
  const bool fast = vec && vecs <= 2;
  long long blocks = (rows + 7) / 8;
  // few blocks: each ends with `cols` atomics per output; the fast kernel runs as one resident wave
  const long long cap = (long long)ds->sm_count * (fast ? LN_BWD_VEC_BLOCKS_PER_SM : 4);
  if (blocks > cap) blocks = cap;
  auto launch = [&](auto kernel) {
    kernel<<<(unsigned)blocks, 256, 0, stream>>>((const T*)x, x_ld, (const T*)gamma, stats, (const T*)g, g_ld, (T*)gx, gx_ld,
                                                 accumulate_x, ggamma, gbeta, rows, (int)cols, vec);
  };
  if (fast && gxsum) {
    layer_norm_bwd_vec_kernel<T, 2, true><<<(unsigned)blocks, 256, sizeof(LnBwdVecSmem<T, 2, true>), stream>>>(
        (const T*)x, x_ld, (const T*)gamma, stats, (const T*)g, g_ld, (T*)gx, gx_ld, accumulate_x, ggamma, gbeta, gxsum, rows,
        (int)cols);
    count_launch(false);
    return note_cuda_error(cudaGetLastError(), "layer_norm backward launch");
  }
  if (fast) {
    layer_norm_bwd_vec_kernel<T, 2, false><<<(unsigned)blocks, 256, sizeof(LnBwdVecSmem<T, 2, false>), stream>>>(
        (const T*)x, x_ld, (const T*)gamma, stats, (const T*)g, g_ld, (T*)gx, gx_ld, accumulate_x, ggamma, gbeta, nullptr, rows,
        (int)cols);
  } else if (vecs <= 2) launch(layer_norm_bwd_kernel<T, 2>);
  else if (vecs <= 4) launch(layer_norm_bwd_kernel<T, 4>);
  else if (vecs <= 8) launch(layer_norm_bwd_kernel<T, 8>);
  else return B200_ERR_LIMIT;
  count_launch(false);
  const int rc = note_cuda_error(cudaGetLastError(), "layer_norm backward launch");
  if (rc || !gxsum) return rc;
  return column_sum_t<T>(rows, cols, gx, gx_ld, gxsum, stream);   // the unfused route: one more pass over grad_x
}

template <typename T>
int column_sum_t(int64_t rows, int64_t cols, const void* g, int64_t ld, float* out, cudaStream_t stream) {
  DeviceState* ds = device_state();
  constexpr int N = Vec<T>::N;
  const int vec = vec_ok(sizeof(T), cols, {ld}, {g}) ? 1 : 0;
  const long long gx = (cols + 32 * N - 1) / (32 * N);
  long long gy = (rows + 63) / 64;                           // at least 8 rows per warp
  const long long cap = ((long long)ds->sm_count * 8 + gx - 1) / gx;
  if (gy > cap) gy = cap;
  if (gy < 1) gy = 1;
  if (gx > 0x7fffffffLL || gy > 65535) return B200_ERR_LIMIT;
  column_sum_kernel<T><<<dim3((unsigned)gx, (unsigned)gy), 256, 0, stream>>>((const T*)g, ld, out, rows, (int)cols, vec);
  count_launch(false);
  return note_cuda_error(cudaGetLastError(), "column sum launch");
}

template <typename T>
int relu_bwd_column_sum_t(int64_t rows, int64_t cols, const void* y, int64_t y_ld, void* g, int64_t ld, float* out,
                          cudaStream_t stream) {
  DeviceState* ds = device_state();
  constexpr int N = Vec<T>::N;
  const int vec = vec_ok(sizeof(T), cols, {ld, y_ld}, {g, y}) ? 1 : 0;
  const long long gx = (cols + 32 * N - 1) / (32 * N);
  long long gy = (rows + 63) / 64;                           // at least 8 rows per warp
  const long long cap = ((long long)ds->sm_count * 8 + gx - 1) / gx;
  if (gy > cap) gy = cap;
  if (gy < 1) gy = 1;
  if (gx > 0x7fffffffLL || gy > 65535) return B200_ERR_LIMIT;
  relu_bwd_column_sum_kernel<T><<<dim3((unsigned)gx, (unsigned)gy), 256, 0, stream>>>((const T*)y, y_ld, (T*)g, ld, out, rows,
                                                                                      (int)cols, vec);
  count_launch(false);
  return note_cuda_error(cudaGetLastError(), "relu backward + column sum launch");
}

template <typename T>
int softmax_forward_t(int64_t rows, int64_t cols, const void* x, int64_t x_ld, double alpha, void* y, int64_t y_ld,
                      cudaStream_t stream) {
  DeviceState* ds = device_state();
  const int vec = vec_ok(sizeof(T), cols, {x_ld, y_ld}, {x, y}) ? 1 : 0;
  const int64_t vecs = (cols + 32 * Vec<T>::N - 1) / (32 * Vec<T>::N);
  const bool fast = vec && vecs <= 2;
  long long blocks = (rows + 7) / 8;
  const long long cap = (long long)ds->sm_count * (fast ? LN_FWD_VEC_BLOCKS_PER_SM : 16);
  if (blocks > cap) blocks = cap;
  auto launch = [&](auto kernel) {
    kernel<<<(unsigned)blocks, 256, 0, stream>>>((const T*)x, x_ld, (float)alpha, (T*)y, y_ld, rows, (int)cols, vec);
  };
  if (vecs <= 2) launch(softmax_fwd_kernel<T, 2>);
  else if (vecs <= 4) launch(softmax_fwd_kernel<T, 4>);
  else if (vecs <= 8) launch(softmax_fwd_kernel<T, 8>);
  else launch(softmax_fwd_kernel<T, 0>);
  count_launch(false);
  return note_cuda_error(cudaGetLastError(), "softmax forward launch");
}

template <typename T>
int softmax_backward_t(int64_t rows, int64_t cols, const void* y, int64_t y_ld, const void* g, int64_t g_ld, double alpha,
                       void* gx, int64_t gx_ld, int accumulate, cudaStream_t stream) {
  DeviceState* ds = device_state();
  const int vec = vec_ok(sizeof(T), cols, {y_ld, g_ld, gx_ld}, {y, g, gx}) ? 1 : 0;
  const int64_t vecs = (cols + 32 * Vec<T>::N - 1) / (32 * Vec<T>::N);
  const bool fast = vec && vecs <= 2;
  long long blocks = (rows + 7) / 8;
  const long long cap = (long long)ds->sm_count * (fast ? LN_FWD_VEC_BLOCKS_PER_SM : 16);
  if (blocks > cap) blocks = cap;
  auto launch = [&](auto kernel) {
    kernel<<<(unsigned)blocks, 256, 0, stream>>>((const T*)y, y_ld, (const T*)g, g_ld, (float)alpha, (T*)gx, gx_ld, accumulate,
                                                 rows, (int)cols, vec);
  };
  if (vecs <= 2) launch(softmax_bwd_kernel<T, 2>);
  else if (vecs <= 4) launch(softmax_bwd_kernel<T, 4>);
  else launch(softmax_bwd_kernel<T, 0>);
  count_launch(false);
  return note_cuda_error(cudaGetLastError(), "softmax backward launch");
}

}  // namespace

int layer_norm_forward(int dtype, int64_t rows, int64_t cols, const void* x, int64_t x_ld, const void* gamma, const void* beta,
                       double eps, void* y, int64_t y_ld, float* stats, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return B200_OK;
  if (!device_state()) return note_cuda_error(cudaErrorInitializationError, "b200_init not called on this device");
  if (cols > 0x7fffffffLL) return B200_ERR_LIMIT;
  switch (dtype) {
    case B200_F32: return ln_forward_t<float>(rows, cols, x, x_ld, gamma, beta, eps, y, y_ld, stats, stream);
    case B200_F16:
    case B200_AMP_F16: return ln_forward_t<__half>(rows, cols, x, x_ld, gamma, beta, eps, y, y_ld, stats, stream);
    default: return B200_ERR_UNSUPPORTED;
  }
}

int layer_norm_backward(int dtype, int64_t rows, int64_t cols, const void* x, int64_t x_ld, const void* gamma, const float* stats,
                        const void* g, int64_t g_ld, void* gx, int64_t gx_ld, int accumulate_x, float* ggamma, float* gbeta,
                        float* gxsum, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return B200_OK;
  if (!device_state()) return note_cuda_error(cudaErrorInitializationError, "b200_init not called on this device");
  switch (dtype) {
    case B200_F32:
      return ln_backward_t<float>(rows, cols, x, x_ld, gamma, stats, g, g_ld, gx, gx_ld, accumulate_x, ggamma, gbeta, gxsum, stream);
    case B200_F16:
    case B200_AMP_F16:
      return ln_backward_t<__half>(rows, cols, x, x_ld, gamma, stats, g, g_ld, gx, gx_ld, accumulate_x, ggamma, gbeta, gxsum, stream);
    default: return B200_ERR_UNSUPPORTED;
  }
}

int add_layer_norm_forward(int dtype, int64_t rows, int64_t cols, const void* a, int64_t a_ld, const void* b, int64_t b_ld,
                           void* sum, int64_t sum_ld, const void* gamma, const void* beta, double eps, void* y, int64_t y_ld,
                           float* stats, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return B200_OK;
  if (!device_state()) return note_cuda_error(cudaErrorInitializationError, "b200_init not called on this device");
  if (cols > 0x7fffffffLL) return B200_ERR_LIMIT;
  switch (dtype) {
    case B200_F32:
      return add_ln_forward_t<float>(rows, cols, a, a_ld, b, b_ld, sum, sum_ld, gamma, beta, eps, y, y_ld, stats, stream);
    case B200_F16:
    case B200_AMP_F16:
      return add_ln_forward_t<__half>(rows, cols, a, a_ld, b, b_ld, sum, sum_ld, gamma, beta, eps, y, y_ld, stats, stream);
    default: return B200_ERR_UNSUPPORTED;
  }
}

int relu_backward_column_sum(int dtype, int64_t rows, int64_t cols, const void* y, int64_t y_ld, void* g, int64_t ld, float* out,
                             cudaStream_t stream) {
  if (rows == 0 || cols == 0) return B200_OK;
  if (!device_state()) return note_cuda_error(cudaErrorInitializationError, "b200_init not called on this device");
  if (cols > 0x7fffffffLL) return B200_ERR_LIMIT;
  switch (dtype) {
    case B200_F32: return relu_bwd_column_sum_t<float>(rows, cols, y, y_ld, g, ld, out, stream);
    case B200_F16:
    case B200_AMP_F16: return relu_bwd_column_sum_t<__half>(rows, cols, y, y_ld, g, ld, out, stream);
    default: return B200_ERR_UNSUPPORTED;
  }
}

int rowwise_setup_device() {
  int rc;
  auto opt_in = [&](auto kernel, size_t bytes) {
    return note_cuda_error(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes),
                           "cudaFuncSetAttribute(layer_norm backward)");
  };
  if ((rc = opt_in(layer_norm_bwd_vec_kernel<float, 2, false>, sizeof(LnBwdVecSmem<float, 2, false>)))) return rc;
  if ((rc = opt_in(layer_norm_bwd_vec_kernel<float, 2, true>, sizeof(LnBwdVecSmem<float, 2, true>)))) return rc;
  if ((rc = opt_in(layer_norm_bwd_vec_kernel<__half, 2, false>, sizeof(LnBwdVecSmem<__half, 2, false>)))) return rc;
  return opt_in(layer_norm_bwd_vec_kernel<__half, 2, true>, sizeof(LnBwdVecSmem<__half, 2, true>));
}

int column_sum(int dtype, int64_t rows, int64_t cols, const void* g, int64_t ld, float* out, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return B200_OK;
  if (!device_state()) return note_cuda_error(cudaErrorInitializationError, "b200_init not called on this device");
  if (cols > 0x7fffffffLL) return B200_ERR_LIMIT;
  switch (dtype) {
    case B200_F32: return column_sum_t<float>(rows, cols, g, ld, out, stream);
    case B200_F16:
    case B200_AMP_F16: return column_sum_t<__half>(rows, cols, g, ld, out, stream);
    default: return B200_ERR_UNSUPPORTED;
  }
}

int softmax_forward(int dtype, int64_t rows, int64_t cols, const void* x, int64_t x_ld, double alpha, void* y, int64_t y_ld,
                    cudaStream_t stream) {
  if (rows == 0 || cols == 0) return B200_OK;
  if (!device_state()) return note_cuda_error(cudaErrorInitializationError, "b200_init not called on this device");
  if (cols > 0x7fffffffLL) return B200_ERR_LIMIT;
  switch (dtype) {
    case B200_F32: return softmax_forward_t<float>(rows, cols, x, x_ld, alpha, y, y_ld, stream);
    case B200_F16:
    case B200_AMP_F16: return softmax_forward_t<__half>(rows, cols, x, x_ld, alpha, y, y_ld, stream);
    default: return B200_ERR_UNSUPPORTED;
  }
}

int softmax_backward(int dtype, int64_t rows, int64_t cols, const void* y, int64_t y_ld, const void* g, int64_t g_ld,
                     double alpha, void* gx, int64_t gx_ld, int accumulate, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return B200_OK;
  if (!device_state()) return note_cuda_error(cudaErrorInitializationError, "b200_init not called on this device");
  if (cols > 0x7fffffffLL) return B200_ERR_LIMIT;
  switch (dtype) {
    case B200_F32: return softmax_backward_t<float>(rows, cols, y, y_ld, g, g_ld, alpha, gx, gx_ld, accumulate, stream);
    case B200_F16:
    case B200_AMP_F16: return softmax_backward_t<__half>(rows, cols, y, y_ld, g, g_ld, alpha, gx, gx_ld, accumulate, stream);
    default: return B200_ERR_UNSUPPORTED;
  }
}

}  // namespace b200
