// Any-stride SIMT GEMM: the exact-arithmetic member of the kernel family.  It serves what the
// tensor-core kernels cannot address with TMA (odd leading dimensions, unaligned sub-slices,
// degenerate stride pairs such as [1,1] / [0,1] / [1,0] accepted by dfdx's `matrix_strides`,
// matmul/mod.rs:316-325), f64, and problems too small to be worth a tensor-core launch.  Arithmetic
// is plain FMA in f32 (f32 / f16 inputs) or f64, summed in k order, so tiny known-answer tests
// of the reference (absolute tolerance 1e-6, dfdx-core/src/lib.rs:236-270) hold.
#include "common.cuh"

namespace b200 {
namespace {

constexpr int TS = 64;   // output tile edge
constexpr int TK = 16;   // k slice per iteration
constexpr int NT = 256;  // threads per block (16 x 16, 4x4 outputs each)

template <typename T> struct Acc { using type = float; };
template <> struct Acc<double> { using type = double; };

template <typename T> __device__ __forceinline__ typename Acc<T>::type to_acc(T v) { return v; }
template <> __device__ __forceinline__ float to_acc<__half>(__half v) { return __half2float(v); }
template <typename T, typename A> __device__ __forceinline__ T from_acc(A v) { return (T)v; }
template <> __device__ __forceinline__ __half from_acc<__half, float>(float v) { return __float2half_rn(v); }

struct SimtArgs {
  int64_t b1, red, m, k, n;
  const void* a; int64_t a_b0, a_b1, a_red, a_r, a_c;
  const void* b; int64_t b_b0, b_b1, b_red, b_r, b_c;
  void* c; int64_t c_b0, c_b1, c_r, c_c;
  int beta;
  int fused; double alpha; const void* bias; int bias_dim, act;   // optional epilogue: act(alpha*acc + bias)
  int64_t tiles_m, tiles_n;
};

template <typename T>
__global__ void __launch_bounds__(NT) gemm_simt_kernel(const SimtArgs g) {
  using A = typename Acc<T>::type;
  __shared__ A sa[TK][TS + 1];
  __shared__ A sb[TK][TS + 1];

  int64_t tile = blockIdx.x;
  const int64_t tm = tile % g.tiles_m; tile /= g.tiles_m;
  const int64_t tn = tile % g.tiles_n; tile /= g.tiles_n;
  const int64_t ib1 = tile % g.b1, ib0 = tile / g.b1;

  const T* __restrict__ pa = (const T*)g.a + ib0 * g.a_b0 + ib1 * g.a_b1;
  const T* __restrict__ pb = (const T*)g.b + ib0 * g.b_b0 + ib1 * g.b_b1;
  T* pc = (T*)g.c + ib0 * g.c_b0 + ib1 * g.c_b1;

  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const int64_t row0 = tm * TS, col0 = tn * TS;
  A acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = (A)0;

  for (int64_t r = 0; r < g.red; ++r) {
    const T* ra = pa + r * g.a_red;
    const T* rb = pb + r * g.b_red;
    for (int64_t k0 = 0; k0 < g.k; k0 += TK) {
      // A slice: TS rows x TK k.  Pick the thread->element map that walks the unit stride.
      for (int e = threadIdx.x; e < TS * TK; e += NT) {
        int i, p;
        if (g.a_c == 1) { p = e % TK; i = e / TK; } else { i = e % TS; p = e / TS; }
        const int64_t gi = row0 + i, gp = k0 + p;
        sa[p][i] = (gi < g.m && gp < g.k) ? to_acc<T>(ra[gi * g.a_r + gp * g.a_c]) : (A)0;
      }
      for (int e = threadIdx.x; e < TS * TK; e += NT) {
        int j, p;
        if (g.b_c == 1) { j = e % TS; p = e / TS; } else { p = e % TK; j = e / TK; }
        const int64_t gj = col0 + j, gp = k0 + p;
        sb[p][j] = (gj < g.n && gp < g.k) ? to_acc<T>(rb[gp * g.b_r + gj * g.b_c]) : (A)0;
      }
      __syncthreads();
#pragma unroll
      for (int p = 0; p < TK; ++p) {
        A av[4], bv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) av[i] = sa[p][ty + 16 * i];
#pragma unroll
        for (int j = 0; j < 4; ++j) bv[j] = sb[p][tx + 16 * j];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fma(av[i], bv[j], acc[i][j]);
      }
      __syncthreads();
    }
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t gi = row0 + ty + 16 * i;
    if (gi >= g.m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t gj = col0 + tx + 16 * j;
      if (gj >= g.n) continue;
      T* dst = pc + gi * g.c_r + gj * g.c_c;
      A v = acc[i][j];
      if (g.beta) v += to_acc<T>(*dst);   // beta == 0 never reads the (uninitialised) output
      if (g.fused) {
        v *= (A)g.alpha;
        if (g.bias) v += to_acc<T>(reinterpret_cast<const T*>(g.bias)[g.bias_dim ? gi : gj]);
        if (g.act == B200_ACT_RELU) v = v > (A)0 ? v : (A)0;
      }
      *dst = from_acc<T, A>(v);
    }
  }
}

template <typename T>
int launch_t(const GemmProblem& p, cudaStream_t stream) {
  SimtArgs g;
  g.b1 = p.b1; g.red = p.red; g.m = p.m; g.k = p.k; g.n = p.n;
  g.a = p.a; g.a_b0 = p.a_b0; g.a_b1 = p.a_b1; g.a_red = p.a_red; g.a_r = p.a_r; g.a_c = p.a_c;
  g.b = p.b; g.b_b0 = p.b_b0; g.b_b1 = p.b_b1; g.b_red = p.b_red; g.b_r = p.b_r; g.b_c = p.b_c;
  g.c = p.c; g.c_b0 = p.c_b0; g.c_b1 = p.c_b1; g.c_r = p.c_r; g.c_c = p.c_c;
  g.beta = p.beta;
  g.fused = p.fused() ? 1 : 0; g.alpha = p.alpha; g.bias = p.bias; g.bias_dim = p.bias_dim; g.act = p.act;
  g.tiles_m = (p.m + TS - 1) / TS;
  g.tiles_n = (p.n + TS - 1) / TS;
  const int64_t blocks = g.tiles_m * g.tiles_n * p.b0 * p.b1;
  if (blocks <= 0) return B200_OK;
  if (blocks > 0x7fffffffLL) return B200_ERR_LIMIT;
  gemm_simt_kernel<T><<<(unsigned)blocks, NT, 0, stream>>>(g);
  count_launch(false);
  return note_cuda_error(cudaGetLastError(), "gemm_simt launch");
}

}  // namespace

int launch_gemm_simt(const GemmProblem& p, cudaStream_t stream) {
  switch (p.dtype) {
    case B200_F32: return launch_t<float>(p, stream);
    case B200_F64: return launch_t<double>(p, stream);
    case B200_F16:
    case B200_AMP_F16: return launch_t<__half>(p, stream);
    default: return B200_ERR_DTYPE;
  }
}

}  // namespace b200
