// conv2d lowered to unfold + GEMM: `Conv2DKernel for Cuda` of dfdx
// (dfdx-core/src/tensor_ops/conv2d/cuda_kernel.rs:80-281) on top of this library's GEMM kernels.
//
// Workspace layout (caller-provided, see b200_conv2d_workspace_bytes):
//   forward : patches (B, C, K, K, OH, OW)
//   backward: patches (B, O, K, K, H, W) | filters_tr (G, C/G, O/G, K, K) | grad_filters_tr (B, G, C/G, O/G, K, K)
// each region starts on a 256-byte boundary so the GEMM operands stay TMA-addressable.
#include "common.cuh"
#include <atomic>
#include <mutex>
#include <initializer_list>
#include <type_traits>

namespace b200 {
namespace {

constexpr int NT = 256;

// Geometry of one convolution.  Kernel extent and padding are per axis so that the same kernels serve conv2d
// (kh = kw, ph = pw) and conv1d (an image of height 1: kh = 1, ph = 0); stride and dilation are shared.
struct Op {
  int64_t kh, kw, stride, ph, pw, dilation, groups, batch, chan_in, chan_out, h_in, h_out, w_in, w_out;
};

Op to_op(const b200_conv2d_op* o) {
  Op r;
  r.kh = r.kw = (int64_t)o->kernel; r.stride = (int64_t)o->stride; r.ph = r.pw = (int64_t)o->padding;
  r.dilation = (int64_t)o->dilation; r.groups = (int64_t)o->groups; r.batch = (int64_t)o->batch;
  r.chan_in = (int64_t)o->chan_in; r.chan_out = (int64_t)o->chan_out; r.h_in = (int64_t)o->h_in;
  r.h_out = (int64_t)o->h_out; r.w_in = (int64_t)o->w_in; r.w_out = (int64_t)o->w_out;
  return r;
}

struct Strides4 { int64_t s[4]; };

// im2col.  One thread per element of patches (b, c, k1, k2, oh, ow); consecutive threads walk ow, so
// both the gather from the image row and the store are coalesced.  Zero where the tap falls in
// the padding (conv2d.cu:18-52 of dfdx computes the same values, one thread per (b,c,oh,ow)).
template <typename T>
__global__ void __launch_bounds__(NT) unfold_input_kernel(const Op op, const T* __restrict__ img,
                                                          const Strides4 st, T* __restrict__ patches,
                                                          const int64_t total) {
  for (int64_t i = (int64_t)blockIdx.x * NT + threadIdx.x; i < total; i += (int64_t)gridDim.x * NT) {
    int64_t idx = i;
    const int64_t ow = idx % op.w_out; idx /= op.w_out;
    const int64_t oh = idx % op.h_out; idx /= op.h_out;
    const int64_t k2 = idx % op.kw; idx /= op.kw;
    const int64_t k1 = idx % op.kh; idx /= op.kh;
    const int64_t c = idx % op.chan_in;
    const int64_t b = idx / op.chan_in;
    const int64_t y = oh * op.stride + op.dilation * k1 - op.ph;
    const int64_t x = ow * op.stride + op.dilation * k2 - op.pw;
    T v = T(0.0f);
    if (y >= 0 && y < op.h_in && x >= 0 && x < op.w_in)
      v = img[b * st.s[0] + c * st.s[1] + y * st.s[2] + x * st.s[3]];
    patches[i] = v;
  }
}

// Transposed-convolution gather: patches (b, o, k1, k2, y, x) = grad_out[b, o, oh, ow] where
// (oh, ow) is the output pixel that input pixel (y, x) feeds through tap (k1, k2), if any
// (conv2d.cu:54-94; conv2d/cpu_kernel.rs:9-40 `unfold_idx`).
template <typename T>
__global__ void __launch_bounds__(NT) unfold_output_kernel(const Op op, const T* __restrict__ gout,
                                                           T* __restrict__ patches, const int64_t total) {
  for (int64_t i = (int64_t)blockIdx.x * NT + threadIdx.x; i < total; i += (int64_t)gridDim.x * NT) {
    int64_t idx = i;
    const int64_t x = idx % op.w_in; idx /= op.w_in;
    const int64_t y = idx % op.h_in; idx /= op.h_in;
    const int64_t k2 = idx % op.kw; idx /= op.kw;
    const int64_t k1 = idx % op.kh; idx /= op.kh;
    const int64_t o = idx % op.chan_out;
    const int64_t b = idx / op.chan_out;
    T v = T(0.0f);
    const int64_t ohs = y + op.ph - op.dilation * k1;
    const int64_t ows = x + op.pw - op.dilation * k2;
    if (ohs >= 0 && ows >= 0 && ohs % op.stride == 0 && ows % op.stride == 0) {
      const int64_t oh = ohs / op.stride, ow = ows / op.stride;
      if (oh < op.h_out && ow < op.w_out)
        v = gout[((b * op.chan_out + o) * op.h_out + oh) * op.w_out + ow];
    }
    patches[i] = v;
  }
}

// filters (O, C/G, K, K) through strides  ->  filters_tr (G, C/G, O/G, K, K) contiguous (conv2d.cu:96-127).
template <typename T>
__global__ void __launch_bounds__(NT) transpose_filters_kernel(const Op op, const T* __restrict__ f,
                                                               const Strides4 st, T* __restrict__ ftr,
                                                               const int64_t total) {
  const int64_t cg = op.chan_in / op.groups, og = op.chan_out / op.groups;
  for (int64_t i = (int64_t)blockIdx.x * NT + threadIdx.x; i < total; i += (int64_t)gridDim.x * NT) {
    int64_t idx = i;
    const int64_t k2 = idx % op.kw; idx /= op.kw;
    const int64_t k1 = idx % op.kh; idx /= op.kh;
    const int64_t o = idx % og; idx /= og;
    const int64_t c = idx % cg;
    const int64_t g = idx / cg;
    ftr[i] = f[(g * og + o) * st.s[0] + c * st.s[1] + k1 * st.s[2] + k2 * st.s[3]];
  }
}

// grad_filters[o, c, k1, k2] (through strides) += sum_b grad_filters_tr[b, g, c, o, k1, k2]
// (conv2d.cu:129-168).  The sum runs in f32 (f64 for double) in batch order.
template <typename T, typename A>
__global__ void __launch_bounds__(NT) sum_transposed_filters_kernel(const Op op, const T* __restrict__ gftr,
                                                                    T* __restrict__ gf, const Strides4 st,
                                                                    const int64_t total) {
  const int64_t cg = op.chan_in / op.groups, og = op.chan_out / op.groups;
  for (int64_t i = (int64_t)blockIdx.x * NT + threadIdx.x; i < total; i += (int64_t)gridDim.x * NT) {
    int64_t idx = i;
    const int64_t k2 = idx % op.kw; idx /= op.kw;
    const int64_t k1 = idx % op.kh; idx /= op.kh;
    const int64_t o = idx % og; idx /= og;
    const int64_t c = idx % cg;
    const int64_t g = idx / cg;
    A acc = A(0);
    for (int64_t b = 0; b < op.batch; ++b) acc += (A)gftr[b * total + i];
    T* dst = gf + (g * og + o) * st.s[0] + c * st.s[1] + k1 * st.s[2] + k2 * st.s[3];
    *dst = (T)((A)*dst + acc);
  }
}

// ---- plane-staged unfold kernels (fast path) -----------------------------------------------------
// One block per (batch, channel) plane: the plane is read from global memory once into shared
// memory, then all K*K shifted copies of it are written with 16-byte stores.  Used when a plane fits
// 48 KB of shared memory and the patch row length is a whole number of vectors; otherwise the
// element-per-thread kernels above serve.
template <typename T> struct VecOf;
template <> struct VecOf<float> { static constexpr int N = 4; using type = float4; };
template <> struct VecOf<double> { static constexpr int N = 2; using type = double2; };
template <> struct VecOf<__half> { static constexpr int N = 8; using type = uint4; };

struct Op32 {
  int kh, kw, stride, ph, pw, dilation, chan_in, chan_out, h_in, h_out, w_in, w_out;
};

template <typename T>
__global__ void __launch_bounds__(NT) unfold_input_plane_kernel(const Op32 op, const T* __restrict__ img,
                                                                const Strides4 st, T* __restrict__ patches) {
  // The plane is staged with its zero padding, so the copy loop below has no bounds checks: the kernel is
  // bound by instruction issue, not by the 16-byte stores.
  constexpr int V = VecOf<T>::N;
  using VT = typename VecOf<T>::type;
  extern __shared__ __align__(16) unsigned char plane_raw[];
  T* plane = reinterpret_cast<T*>(plane_raw);
  const int id = blockIdx.x, b = id / op.chan_in, c = id - b * op.chan_in;
  const T* src = img + (int64_t)b * st.s[0] + (int64_t)c * st.s[1];
  const int pw_in = op.w_in + 2 * op.pw, ph_in = op.h_in + 2 * op.ph;
  for (int i = threadIdx.x; i < ph_in * pw_in; i += NT) {
    const int yy = i / pw_in, y = yy - op.ph, x = i - yy * pw_in - op.pw;
    plane[i] = (y >= 0 && y < op.h_in && x >= 0 && x < op.w_in) ? src[(int64_t)y * st.s[2] + (int64_t)x * st.s[3]]
                                                                : T(0.0f);
  }
  __syncthreads();
  const int npos = op.h_out * op.w_out, vrow = op.w_out / V, nvec = op.h_out * vrow;
  T* dst = patches + (int64_t)id * op.kh * op.kw * npos;
  for (int v = threadIdx.x; v < nvec; v += NT) {
    const int oh = v / vrow, ow0 = (v - oh * vrow) * V;
    const T* corner = plane + oh * op.stride * pw_in + ow0 * op.stride;
    T* out = dst + oh * op.w_out + ow0;
    for (int k1 = 0; k1 < op.kh; ++k1) {
      const T* row = corner + op.dilation * k1 * pw_in;
      for (int k2 = 0; k2 < op.kw; ++k2, row += op.dilation, out += npos) {
        __align__(16) T vals[V];
#pragma unroll
        for (int e = 0; e < V; ++e) vals[e] = row[e * op.stride];
        *reinterpret_cast<VT*>(out) = *reinterpret_cast<const VT*>(vals);
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(NT) unfold_output_plane_kernel(const Op32 op, const T* __restrict__ gout,
                                                                 T* __restrict__ patches) {
  constexpr int V = VecOf<T>::N;
  using VT = typename VecOf<T>::type;
  extern __shared__ __align__(16) unsigned char plane_raw[];
  T* plane = reinterpret_cast<T*>(plane_raw);
  const int id = blockIdx.x;                                   // b * chan_out + o
  const int npos = op.h_out * op.w_out;
  const T* src = gout + (int64_t)id * npos;
  for (int i = threadIdx.x; i < npos; i += NT) plane[i] = src[i];
  __syncthreads();
  const int hw = op.h_in * op.w_in, vrow = op.w_in / V, nvec = op.h_in * vrow;
  T* dst = patches + (int64_t)id * op.kh * op.kw * hw;
  for (int v = threadIdx.x; v < nvec; v += NT) {
    const int y = v / vrow, x0 = (v - y * vrow) * V;
    for (int k1 = 0; k1 < op.kh; ++k1) {
      const int ohs = y + op.ph - op.dilation * k1;
      const int oh = ohs / op.stride;
      const bool yok = ohs >= 0 && ohs - oh * op.stride == 0 && oh < op.h_out;
      for (int k2 = 0; k2 < op.kw; ++k2) {
        __align__(16) T vals[V];
#pragma unroll
        for (int e = 0; e < V; ++e) {
          const int ows = x0 + e + op.pw - op.dilation * k2;
          const int ow = ows / op.stride;
          vals[e] = (yok && ows >= 0 && ows - ow * op.stride == 0 && ow < op.w_out) ? plane[oh * op.w_out + ow]
                                                                                    : T(0.0f);
        }
        *reinterpret_cast<VT*>(dst + (int64_t)(k1 * op.kw + k2) * hw + y * op.w_in + x0) =
            *reinterpret_cast<const VT*>(vals);
      }
    }
  }
}

Op32 to_op32(const Op& o);

// Division of a non-negative 31-bit integer by a launch constant as a multiply and a shift:
// n / d = umulhi(n, ceil(2^p / d)) >> (p - 32) with p = 31 + ceil(log2 d), exact for 0 <= n < 2^31.
struct FastDiv {
  uint32_t mul, shr, d;
  __device__ __forceinline__ int div(int n) const { return d == 1 ? n : (int)(__umulhi((uint32_t)n, mul) >> shr); }
};
FastDiv fast_div(int64_t d) {
  FastDiv f{0u, 0u, (uint32_t)d};
  if (d > 1) {
    uint32_t l = 0;
    while (((int64_t)1 << l) < d) ++l;
    f.mul = (uint32_t)((((uint64_t)1 << (31 + l)) + (uint64_t)d - 1) / (uint64_t)d);
    f.shr = l - 1;
  }
  return f;
}

// col2im: grad_img[b, c, y, x] += sum over the taps (k1, k2) that reach an output pixel of
// cols[b, c, k1, k2, oh, ow], the per-tap data gradients produced by filters^T x grad_out.
//
// The kernel is issue-bound long before it is bandwidth-bound (a tap costs a few dozen instructions of index
// work against one 4-byte load), so the index work is shared: a thread owns FOLD_P runs of V consecutive
// pixels of a row (V = 4 when the row length allows, else 1), works out the row and the validity of a filter
// row once per run, and with unit stride (UNIT) reaches the V pixels of a tap from one base address; launch
// constants divide by multiply-and-shift.  Loads of two taps for all runs are issued before the adds.  A block
// covers FOLD_P * NT consecutive runs of one (b, c) plane.  The sum runs in tap order in A (f32 for half); the
// image element is read and written once.
constexpr int FOLD_P = 2;
template <typename T, typename A, int V, bool UNIT>
__global__ void __launch_bounds__(NT) fold_cols_kernel(const Op32 op, const FastDiv by_vrow, const FastDiv by_stride,
                                                       const unsigned blocks_per_plane, const T* __restrict__ cols,
                                                       T* __restrict__ grad_img) {
  constexpr int P = FOLD_P;
  const unsigned plane = blockIdx.x / blocks_per_plane, chunk = blockIdx.x - plane * blocks_per_plane;
  const int vrow = op.w_in / V, nvec = op.h_in * vrow, npos = op.h_out * op.w_out;
  const T* src = cols + (int64_t)plane * op.kh * op.kw * npos;
  T* dst = grad_img + (int64_t)plane * op.h_in * op.w_in;
  int vi[P], ys[P], xs[P];
  A acc[P][V];
#pragma unroll
  for (int p = 0; p < P; ++p) {
    vi[p] = (int)(chunk * (NT * P) + p * NT + threadIdx.x);
    const int vv = vi[p] < nvec ? vi[p] : 0;
    const int y = by_vrow.div(vv);
    ys[p] = y + op.ph; xs[p] = (vv - y * vrow) * V + op.pw;
#pragma unroll
    for (int e = 0; e < V; ++e) acc[p][e] = A(0);
  }
  for (int k1 = 0; k1 < op.kh; ++k1) {
    int rowoff[P];                                           // offset of row oh inside a tap plane, -1 if the tap misses
#pragma unroll
    for (int p = 0; p < P; ++p) {
      const int ohs = ys[p] - op.dilation * k1;
      const int oh = UNIT ? ohs : by_stride.div(ohs < 0 ? 0 : ohs);
      rowoff[p] = (vi[p] < nvec && ohs >= 0 && oh * op.stride == ohs && oh < op.h_out) ? oh * op.w_out : -1;
    }
    const T* tap = src + (int64_t)k1 * op.kw * npos;
    for (int k2 = 0; k2 < op.kw; k2 += 2) {
      T v[2][P][V];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int p = 0; p < P; ++p) {
          const bool ok = k2 + j < op.kw && rowoff[p] >= 0;
          const int ows0 = xs[p] - op.dilation * (k2 + j);
          const T* q = tap + (int64_t)(k2 + j) * npos + (ok ? rowoff[p] : 0);
#pragma unroll
          for (int e = 0; e < V; ++e) {
            const int ows = ows0 + e;
            const int ow = UNIT ? ows : by_stride.div(ows < 0 ? 0 : ows);
            const bool hit = ok && ows >= 0 && ow < op.w_out && (UNIT || ow * op.stride == ows);
            v[j][p][e] = T(0.0f);
            if (hit) v[j][p][e] = q[ow];
          }
        }
      }
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int p = 0; p < P; ++p)
#pragma unroll
          for (int e = 0; e < V; ++e) acc[p][e] += (A)v[j][p][e];
    }
  }
#pragma unroll
  for (int p = 0; p < P; ++p) {
    if (vi[p] >= nvec) continue;
    T* d = dst + (int64_t)vi[p] * V;
#pragma unroll
    for (int e = 0; e < V; ++e) d[e] = (T)((A)d[e] + acc[p][e]);
  }
}

template <typename T, typename A>
void launch_fold(const Op& op, int64_t planes, const T* cols, T* grad_img, cudaStream_t stream) {
  const int v = op.w_in % 4 == 0 ? 4 : 1;
  const int64_t nvec = op.h_in * (op.w_in / v);
  const unsigned bpp = (unsigned)((nvec + NT * FOLD_P - 1) / (NT * FOLD_P));
  const unsigned grid = (unsigned)(planes * bpp);
  const Op32 o = to_op32(op);
  const FastDiv by_vrow = fast_div(op.w_in / v), by_stride = fast_div(op.stride);
  const bool unit = op.stride == 1;
  if (v == 4 && unit) fold_cols_kernel<T, A, 4, true><<<grid, NT, 0, stream>>>(o, by_vrow, by_stride, bpp, cols, grad_img);
  else if (v == 4) fold_cols_kernel<T, A, 4, false><<<grid, NT, 0, stream>>>(o, by_vrow, by_stride, bpp, cols, grad_img);
  else if (unit) fold_cols_kernel<T, A, 1, true><<<grid, NT, 0, stream>>>(o, by_vrow, by_stride, bpp, cols, grad_img);
  else fold_cols_kernel<T, A, 1, false><<<grid, NT, 0, stream>>>(o, by_vrow, by_stride, bpp, cols, grad_img);
}

Op32 to_op32(const Op& o) {
  return Op32{(int)o.kh, (int)o.kw, (int)o.stride, (int)o.ph, (int)o.pw, (int)o.dilation, (int)o.chan_in, (int)o.chan_out,
              (int)o.h_in, (int)o.h_out, (int)o.w_in, (int)o.w_out};
}

bool fits_int(const Op& o) {
  const int64_t lim = 1 << 30;
  return o.batch * o.chan_in < lim && o.batch * o.chan_out < lim && o.h_in * o.w_in < lim &&
         o.h_out * o.w_out < lim && o.kh < 4096 && o.kw < 4096 && o.stride < lim && o.ph < lim && o.pw < lim && o.dilation < lim;
}

size_t padded_plane_bytes(const Op& o, size_t es) { return (size_t)((o.h_in + 2 * o.ph) * (o.w_in + 2 * o.pw)) * es; }
template <typename T>
bool plane_path_input(const Op& o) {
  // every tap of every output pixel must fall inside the padded plane (true for consistent geometries)
  return fits_int(o) && o.w_out % VecOf<T>::N == 0 && o.h_out * o.w_out > 0 &&
         (o.h_in + 2 * o.ph) * (o.w_in + 2 * o.pw) < ((int64_t)1 << 24) && padded_plane_bytes(o, sizeof(T)) <= 48 * 1024 &&
         (o.h_out - 1) * o.stride + o.dilation * (o.kh - 1) < o.h_in + 2 * o.ph &&
         (o.w_out - 1) * o.stride + o.dilation * (o.kw - 1) < o.w_in + 2 * o.pw;
}
template <typename T>
bool plane_path_output(const Op& o) {
  return fits_int(o) && o.w_in % VecOf<T>::N == 0 && (size_t)(o.h_out * o.w_out) * sizeof(T) <= 48 * 1024 &&
         o.h_in * o.w_in > 0;
}

unsigned grid_for(int64_t total, int sms) {
  int64_t blocks = (total + NT - 1) / NT;
  const int64_t cap = (int64_t)sms * 16;
  if (blocks > cap) blocks = cap;
  return (unsigned)(blocks < 1 ? 1 : blocks);
}

size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

// Tuning knobs (b200_set_conv_lowering): 0 = choose, 1 = data gradient by gather + GEMM only; bytes of cols per group of images.
// Atomics: a thread may change a knob while another thread launches.
constexpr size_t CONV_GROUP_BYTES_DEFAULT = ~(size_t)0;
std::atomic<int> g_conv_grad_img_mode{0};
std::atomic<size_t> g_conv_group_bytes{CONV_GROUP_BYTES_DEFAULT};

// ---- implicit-GEMM path (f32, unit stride): no patch buffer ------------------------------------------
// The tensor-core kernel gathers the patches itself, by TMA, from a channels-last copy of the image (a TMA box
// must start on a 16-byte boundary, which a one-pixel shift along the rows of an NCHW image is not; with the
// channels innermost every shift is a whole number of pixels = whole vectors).  What is left of the lowering is
// this layout change (one read and one write of the image instead of K*K writes and reads of it) and a re-layout
// of the filters.

// (B, C, H, W) through strides -> (B, H, W, G*cpad); channel c = g*cg + ci goes to g*cpad + ci, the rest is zero.
// A block moves a tile of 32 output channels x 128 pixels through shared memory: coalesced 128-byte reads along the
// pixels of each channel plane, 16-byte writes along the channels of each pixel.  The kernel is bound by instruction
// issue before it is bound by DRAM, so the per-element work is a handful of instructions: the channel -> plane
// offsets of the tile are worked out once per block, pixel offsets once per thread.
// The small job that every pass needs beside the layout change rides in the same launch (a dependent launch costs
// 3-4 us of an otherwise idle GPU): blocks with blockIdx.z == images write the re-laid-out filters,
//   rows[g][i][tap][cp], zero padded:  transpose 0: i = output channel in the group, cp = input channel
//                                      (forward: M = O/G, K = taps x C/G);
//                                      transpose 1: i = input channel, cp = output channel in the group
//                                      (data gradient: M = C/G, K = taps x O/G);
// or, with f == nullptr, fill `rows` with zeros (the filter gradient accumulates into it).
struct FilterJob {
  const float* f;
  Strides4 st;
  float* rows;
  int og, cg, kk, kw, cpad, transpose;
  int64_t total;
};
__device__ __forceinline__ void filter_job(const FilterJob& j, int64_t first, int64_t step) {
  const int m = j.transpose ? j.cg : j.og, inner = j.transpose ? j.og : j.cg;
  for (int64_t i = first; i < j.total; i += step) {
    float v = 0.f;
    if (j.f) {
      int64_t idx = i;
      const int cp = (int)(idx % j.cpad); idx /= j.cpad;
      const int tap = (int)(idx % j.kk); idx /= j.kk;
      const int mi = (int)(idx % m);
      const int64_t g = idx / m;
      const int k1 = tap / j.kw, k2 = tap - k1 * j.kw;
      if (cp < inner) {
        const int64_t o = g * j.og + (j.transpose ? cp : mi), ci = j.transpose ? mi : cp;
        v = j.f[o * j.st.s[0] + ci * j.st.s[1] + (int64_t)k1 * j.st.s[2] + (int64_t)k2 * j.st.s[3]];
      }
    }
    j.rows[i] = v;
  }
}

constexpr int CL_PIX = 128, CL_CH = 32;
__global__ void __launch_bounds__(256) to_channels_last_kernel(const float* __restrict__ in, const Strides4 st,
                                                               float* __restrict__ out, const int cg, const int cpad,
                                                               const int ctot, const int hw, const int w,
                                                               const int images, const FilterJob job) {
  __shared__ float tile[CL_CH][CL_PIX + 1];
  __shared__ long long chan_off[CL_CH];                      // offset of the tile's channel planes; -1: padding
  const int tid = threadIdx.x;
  if ((int)blockIdx.z >= images) {
    const int64_t nb = (int64_t)gridDim.x * gridDim.y, bid = (int64_t)blockIdx.y * gridDim.x + blockIdx.x;
    filter_job(job, bid * 256 + tid, nb * 256);
    return;
  }
  const long long b = blockIdx.z;
  const int p0 = blockIdx.x * CL_PIX, c0 = blockIdx.y * CL_CH;
  if (tid < CL_CH) {
    const int cp = c0 + tid, g = cp / cpad, ci = cp - g * cpad;
    chan_off[tid] = (cp < ctot && ci < cg) ? (long long)(g * cg + ci) * st.s[1] : -1;
  }
  // this thread's pixel (the same for all its loads) and its offset inside a plane
  const int px = tid & (CL_PIX - 1), p = p0 + px;
  long long poff = -1;
  if (p < hw) {
    const int y = p / w, x = p - y * w;
    poff = b * st.s[0] + (long long)y * st.s[2] + (long long)x * st.s[3];
  }
  __syncthreads();
  // all of the thread's loads are issued before the first is used (memory-level parallelism, not instruction count,
  // is what this kernel runs on)
  float v[CL_CH / 2];
#pragma unroll
  for (int k = 0; k < CL_CH / 2; ++k) {
    const long long co = chan_off[2 * k + (tid >> 7)];
    v[k] = (co >= 0 && poff >= 0) ? __ldg(in + co + poff) : 0.f;
  }
#pragma unroll
  for (int k = 0; k < CL_CH / 2; ++k) tile[2 * k + (tid >> 7)][px] = v[k];
  __syncthreads();
  // 8 lanes cover the 32 channels of one pixel with 16-byte stores; a warp writes 4 pixels per instruction
  const int c4 = (tid & 7) * 4, pl = (tid >> 3) & 3, wq = tid >> 5;
  if (c0 + c4 < ctot) {
#pragma unroll
    for (int it = 0; it < CL_PIX / 32; ++it) {
      const int q = wq * (CL_PIX / 8) + it * 4 + pl;
      if (p0 + q < hw) {
        const float4 v = make_float4(tile[c4][q], tile[c4 + 1][q], tile[c4 + 2][q], tile[c4 + 3][q]);
        *reinterpret_cast<float4*>(out + ((b * hw + p0 + q) * ctot + c0 + c4)) = v;
      }
    }
  }
}

// grad_filters[g*og + o, c, k1, k2] (through strides) += rows[g][o][tap][c]
__global__ void __launch_bounds__(NT) add_filter_rows_kernel(const float* __restrict__ rows, float* __restrict__ gf,
                                                             const Strides4 st, const int og, const int cg, const int kk,
                                                             const int kw, const int cpad, const int64_t total) {
  for (int64_t i = (int64_t)blockIdx.x * NT + threadIdx.x; i < total; i += (int64_t)gridDim.x * NT) {
    int64_t idx = i;
    const int c = (int)(idx % cg); idx /= cg;
    const int tap = (int)(idx % kk); idx /= kk;
    const int64_t o = idx;                                     // g*og + o
    const int k1 = tap / kw, k2 = tap - k1 * kw;
    gf[o * st.s[0] + (int64_t)c * st.s[1] + (int64_t)k1 * st.s[2] + (int64_t)k2 * st.s[3]] +=
        rows[(o * kk + tap) * cpad + c];
  }
}

int64_t round_up(int64_t x, int64_t to) { return (x + to - 1) / to * to; }

int launch_to_channels_last(const float* in, const Strides4& st, float* out, int64_t batch, int64_t groups, int64_t cg,
                            int64_t cpad, int64_t h, int64_t w, const FilterJob& job, cudaStream_t stream) {
  const int64_t ctot = groups * cpad, hw = h * w;
  dim3 grid((unsigned)((hw + CL_PIX - 1) / CL_PIX), (unsigned)((ctot + CL_CH - 1) / CL_CH), (unsigned)batch + 1);
  to_channels_last_kernel<<<grid, 256, 0, stream>>>(in, st, out, (int)cg, (int)cpad, (int)ctot, (int)hw, (int)w,
                                                    (int)batch, job);
  count_launch(false);
  return note_cuda_error(cudaGetLastError(), "to_channels_last launch");
}

std::atomic<uint64_t> g_implicit_passes{0};

// Which passes of a geometry the implicit path serves (f32, unit stride, a tensor-core sized problem whose padded
// channel counts at most double the work).
struct ImplicitPlan {
  bool fwd = false, wgrad = false, dgrad = false;
  int64_t cpad16 = 0, cpad32 = 0, opad16 = 0;
};
ImplicitPlan implicit_plan(int dtype, const Op& o) {
  ImplicitPlan pl;
  if (dtype != B200_F32 || o.stride != 1 || current_path() == B200_PATH_SIMT || !fits_int(o)) return pl;
  if (o.groups < 1 || o.batch < 1 || o.batch > 65534) return pl;   // images + 1 is a grid dimension
  const int64_t cg = o.chan_in / o.groups, og = o.chan_out / o.groups, kk = o.kh * o.kw;
  const int64_t npos = o.h_out * o.w_out, hw = o.h_in * o.w_in;
  if (cg < 8 || og < 8 || npos < 8 || hw < 8) return pl;
  const double work = (double)o.batch * (double)o.chan_out * (double)cg * (double)kk * (double)npos;
  if (work < 4194304.0) return pl;
  pl.cpad16 = round_up(cg, 16); pl.cpad32 = round_up(cg, 32); pl.opad16 = round_up(og, 16);
  if (o.groups * pl.cpad32 > (1 << 30) || o.groups * pl.opad16 > (1 << 30)) return pl;
  pl.fwd = pl.cpad16 <= 2 * cg && o.w_out <= 256 && npos % 4 == 0;
  pl.wgrad = pl.cpad32 <= 2 * cg && o.w_out % 4 == 0 && (o.groups * pl.cpad32) % 4 == 0;
  // the data gradient's GEMM has C/G rows: below half an MMA tile the materialising lowering (full tiles) wins
  pl.dgrad = pl.opad16 <= 2 * og && o.w_in <= 256 && hw % 4 == 0 && cg >= 64;
  return pl;
}

// out (beta) += conv(img, filters) without a patch buffer.  Workspace: channels-last image | filter rows.
int forward_implicit(const Op& op, const ImplicitPlan& pl, const float* img, const Strides4& ist, const float* filters,
                     const Strides4& fst, float* out, void* ws, cudaStream_t stream, int beta) {
  DeviceState* ds = device_state();
  const int sms = ds ? ds->sm_count : 148;
  const int64_t G = op.groups, cg = op.chan_in / G, og = op.chan_out / G, kk = op.kh * op.kw, cpad = pl.cpad16;
  float* img_cl = (float*)ws;
  float* rows = (float*)((uint8_t*)ws + align256((size_t)(op.batch * op.h_in * op.w_in * G * cpad) * 4));
  ConvImplicit c;
  c.img_cl = img_cl; c.batch = op.batch; c.h_img = op.h_in; c.w_img = op.w_in; c.groups = G; c.cpad = cpad;
  c.filt = rows; c.m = og; c.kh = (int)op.kh; c.kw = (int)op.kw;
  c.h0 = -(int)op.ph; c.dh = (int)op.dilation; c.w0 = -(int)op.pw; c.dw = (int)op.dilation;
  c.out = out; c.h_out = op.h_out; c.w_out = op.w_out; c.beta = beta;
  if (!conv_implicit_ok(c)) return B200_ERR_UNSUPPORTED;
  const FilterJob job{filters, fst, rows, (int)og, (int)cg, (int)kk, (int)op.kw, (int)cpad, 0, G * og * kk * cpad};
  int rc = launch_to_channels_last(img, ist, img_cl, op.batch, G, cg, cpad, op.h_in, op.w_in, job, stream);
  if (rc) return rc;
  g_implicit_passes.fetch_add(1, std::memory_order_relaxed);
  return launch_conv_implicit(c, stream);
}

// grad_filters (through strides) += the filter gradient, without a patch buffer.
// Workspace: channels-last image | gradient rows (G, O/G, taps, cpad).
int wgrad_implicit(const Op& op, const ImplicitPlan& pl, const float* img, const Strides4& fst, float* grad_filters,
                   const float* grad_out, void* ws, cudaStream_t stream) {
  DeviceState* ds = device_state();
  const int sms = ds ? ds->sm_count : 148;
  const int64_t G = op.groups, cg = op.chan_in / G, og = op.chan_out / G, kk = op.kh * op.kw, cpad = pl.cpad32;
  const int64_t npos = op.h_out * op.w_out, hw = op.h_in * op.w_in;
  float* img_cl = (float*)ws;
  float* rows = (float*)((uint8_t*)ws + align256((size_t)(op.batch * hw * G * cpad) * 4));
  ConvImplicitWgrad c;
  c.gout = grad_out; c.gout_bs = op.chan_out * npos; c.m = og; c.h_out = op.h_out; c.w_out = op.w_out;
  c.img_cl = img_cl; c.batch = op.batch; c.h_img = op.h_in; c.w_img = op.w_in; c.c_total = G * cpad; c.cpad = cpad;
  c.kh = (int)op.kh; c.kw = (int)op.kw;
  c.h0 = -(int)op.ph; c.dh = (int)op.dilation; c.w0 = -(int)op.pw; c.dw = (int)op.dilation;
  c.out = rows;
  if (!conv_implicit_wgrad_ok(c)) return B200_ERR_UNSUPPORTED;
  const Strides4 ist{{op.chan_in * hw, hw, op.w_in, 1}};
  const FilterJob job{nullptr, fst, rows, (int)og, (int)cg, (int)kk, (int)op.kw, (int)cpad, 0, G * og * kk * cpad};   // zero fill
  int rc = launch_to_channels_last(img, ist, img_cl, op.batch, G, cg, cpad, op.h_in, op.w_in, job, stream);
  if (rc) return rc;
  g_implicit_passes.fetch_add(1, std::memory_order_relaxed);
  for (int64_t g = 0; g < G; ++g) {
    c.gout = grad_out + g * og * npos;
    c.img_cl = img_cl + g * cpad;
    c.out = rows + g * og * kk * cpad;
    if ((rc = launch_conv_implicit_wgrad(c, stream))) return rc;
  }
  const int64_t total = op.chan_out * kk * cg;
  add_filter_rows_kernel<<<grid_for(total, sms), NT, 0, stream>>>(rows, grad_filters, fst, (int)og, (int)cg, (int)kk,
                                                                  (int)op.kw, (int)cpad, total);
  count_launch(false);
  return note_cuda_error(cudaGetLastError(), "add_filter_rows launch");
}

// grad_img += the data gradient, as a convolution of grad_out with the filters' roles exchanged, without a patch
// buffer.  Workspace: channels-last grad_out | filter rows (G, C/G, taps, opad).
int dgrad_implicit(const Op& op, const ImplicitPlan& pl, float* grad_img, const float* filters, const Strides4& fst,
                   const float* grad_out, void* ws, cudaStream_t stream) {
  DeviceState* ds = device_state();
  const int sms = ds ? ds->sm_count : 148;
  const int64_t G = op.groups, cg = op.chan_in / G, og = op.chan_out / G, kk = op.kh * op.kw, opad = pl.opad16;
  const int64_t npos = op.h_out * op.w_out;
  float* gout_cl = (float*)ws;
  float* rows = (float*)((uint8_t*)ws + align256((size_t)(op.batch * npos * G * opad) * 4));
  ConvImplicit c;
  c.img_cl = gout_cl; c.batch = op.batch; c.h_img = op.h_out; c.w_img = op.w_out; c.groups = G; c.cpad = opad;
  c.filt = rows; c.m = cg; c.kh = (int)op.kh; c.kw = (int)op.kw;
  c.h0 = (int)op.ph; c.dh = -(int)op.dilation; c.w0 = (int)op.pw; c.dw = -(int)op.dilation;
  c.out = grad_img; c.h_out = op.h_in; c.w_out = op.w_in; c.beta = 1;
  if (!conv_implicit_ok(c)) return B200_ERR_UNSUPPORTED;
  const Strides4 gst{{op.chan_out * npos, npos, op.w_out, 1}};
  const FilterJob job{filters, fst, rows, (int)og, (int)cg, (int)kk, (int)op.kw, (int)opad, 1, G * cg * kk * opad};
  int rc = launch_to_channels_last(grad_out, gst, gout_cl, op.batch, G, og, opad, op.h_out, op.w_out, job, stream);
  if (rc) return rc;
  g_implicit_passes.fetch_add(1, std::memory_order_relaxed);
  return launch_conv_implicit(c, stream);
}

template <typename T, typename A>
int forward_t(int dtype, const Op& op, const T* img, const size_t is[4], const T* filters, T* out,
              void* ws, cudaStream_t stream, int beta = 0) {
  DeviceState* ds = device_state();
  const int sms = ds ? ds->sm_count : 148;
  T* patches = (T*)ws;
  const int64_t total = op.batch * op.chan_in * op.kh * op.kw * op.h_out * op.w_out;
  if (total == 0) return B200_OK;
  Strides4 st{{(int64_t)is[0], (int64_t)is[1], (int64_t)is[2], (int64_t)is[3]}};
  if constexpr (std::is_same<T, float>::value) {
    const ImplicitPlan ip = implicit_plan(dtype, op);
    if (ip.fwd && g_conv_grad_img_mode.load() == 0) {
      const int64_t cgk = (op.chan_in / op.groups) * op.kh * op.kw;
      const Strides4 fst{{cgk, op.kh * op.kw, op.kw, 1}};     // the forward pass takes contiguous filters
      const int rc = forward_implicit(op, ip, img, st, filters, fst, out, ws, stream, beta);
      if (rc != B200_ERR_UNSUPPORTED) return rc;
    }
  }
  if (plane_path_input<T>(op))
    unfold_input_plane_kernel<T><<<(unsigned)(op.batch * op.chan_in), NT, padded_plane_bytes(op, sizeof(T)),
                                   stream>>>(to_op32(op), img, st, patches);
  else
    unfold_input_kernel<T><<<grid_for(total, sms), NT, 0, stream>>>(op, img, st, patches, total);
  count_launch(false);
  int rc = note_cuda_error(cudaGetLastError(), "unfold_input launch");
  if (rc) return rc;

  // filters (G, O/G, C/G*K*K) x patches (B, G, C/G*K*K, OH*OW) -> out (B, G, O/G, OH*OW)
  const int64_t m = op.chan_out / op.groups, k = (op.chan_in / op.groups) * op.kh * op.kw,
                n = op.h_out * op.w_out, G = op.groups;
  GemmProblem p;
  p.dtype = dtype; p.beta = beta; p.b0 = op.batch; p.b1 = G; p.m = m; p.k = k; p.n = n;
  p.a = filters; p.a_b0 = 0; p.a_b1 = m * k; p.a_r = k; p.a_c = 1;
  p.b = patches; p.b_b0 = G * k * n; p.b_b1 = k * n; p.b_r = n; p.b_c = 1;
  p.c = out; p.c_b0 = G * m * n; p.c_b1 = m * n; p.c_r = n; p.c_c = 1;
  return run_gemm(p, stream);
}

template <typename T, typename A>
int backward_t(int dtype, const Op& op, const T* img, T* grad_img, const T* filters, const size_t fs[4],
               T* grad_filters, const T* grad_out, void* ws, cudaStream_t stream) {
  DeviceState* ds = device_state();
  const int sms = ds ? ds->sm_count : 148;
  const int64_t G = op.groups, cg = op.chan_in / G, og = op.chan_out / G, KK = op.kh * op.kw;
  const int64_t hw = op.h_in * op.w_in;
  const int64_t n_patches = op.batch * op.chan_out * KK * hw;
  const int64_t n_filters = G * cg * og * KK;
  if (n_patches == 0 || n_filters == 0) return B200_OK;
  uint8_t* base = (uint8_t*)ws;
  T* patches = (T*)base;
  const int64_t n_fwd_patches = op.batch * op.chan_in * KK * op.h_out * op.w_out;
  T* ftr = (T*)(base + align256((size_t)(n_patches > n_fwd_patches ? n_patches : n_fwd_patches) * sizeof(T)));
  T* gftr = (T*)((uint8_t*)ftr + align256((size_t)n_filters * sizeof(T)));
  Strides4 st{{(int64_t)fs[0], (int64_t)fs[1], (int64_t)fs[2], (int64_t)fs[3]}};
  int rc;

  // The implicit-GEMM lowerings (no patch buffer) where they apply; each pass uses the workspace from its start,
  // one after the other on the stream.
  if constexpr (std::is_same<T, float>::value) {
    const ImplicitPlan ip = implicit_plan(dtype, op);
    if (g_conv_grad_img_mode.load() == 0) {
      if (grad_filters && img && ip.wgrad) {
        rc = wgrad_implicit(op, ip, img, st, grad_filters, grad_out, ws, stream);
        if (rc == B200_OK) grad_filters = nullptr;
        else if (rc != B200_ERR_UNSUPPORTED) return rc;
      }
      if (grad_img && ip.dgrad) {
        rc = dgrad_implicit(op, ip, grad_img, filters, st, grad_out, ws, stream);
        if (rc == B200_OK) grad_img = nullptr;
        else if (rc != B200_ERR_UNSUPPORTED) return rc;
      }
      if (!grad_filters && !grad_img) return B200_OK;
    }
  }

  // grad_filters first, while the workspace is free: with contiguous filters,
  //   grad_filters (G, O/G, C/G*K*K) += sum_b grad_out_b (G, O/G, OH*OW) x patches(img_b)^T (G, OH*OW, C/G*K*K)
  // is one batch-reduced GEMM per group (O/G rows: full tiles) that accumulates straight into the filter
  // layout, instead of per-image GEMMs into a B-fold temporary followed by a sum.
  const bool filters_contig = (int64_t)fs[3] == 1 && (int64_t)fs[2] == op.kw && (int64_t)fs[1] == KK &&
                              (int64_t)fs[0] == cg * KK;
  bool grad_filters_done = false;
  // (tensor-core dtypes only: their kernels cut the long reduction into K slices.)
  if (grad_filters && filters_contig && n_fwd_patches > 0 && dtype != B200_F64) {
    const int64_t npos = op.h_out * op.w_out;
    Strides4 ist{{op.chan_in * hw, hw, op.w_in, 1}};
    if (plane_path_input<T>(op))
      unfold_input_plane_kernel<T><<<(unsigned)(op.batch * op.chan_in), NT, padded_plane_bytes(op, sizeof(T)), stream>>>(
          to_op32(op), img, ist, patches);
    else
      unfold_input_kernel<T><<<grid_for(n_fwd_patches, sms), NT, 0, stream>>>(op, img, ist, patches, n_fwd_patches);
    count_launch(false);
    if ((rc = note_cuda_error(cudaGetLastError(), "unfold_input launch (backward)"))) return rc;
    for (int64_t gi = 0; gi < G; ++gi) {
      GemmProblem p;
      p.dtype = dtype; p.beta = 1; p.red = op.batch; p.m = og; p.k = npos; p.n = cg * KK;
      p.a = grad_out + gi * og * npos; p.a_red = op.chan_out * npos; p.a_r = npos; p.a_c = 1;
      p.b = patches + gi * cg * KK * npos; p.b_red = op.chan_in * KK * npos; p.b_r = 1; p.b_c = npos;
      p.c = grad_filters + gi * og * cg * KK; p.c_r = cg * KK; p.c_c = 1;
      if ((rc = run_gemm(p, stream))) return rc;
    }
    grad_filters_done = true;
    if (!grad_img) return B200_OK;
  }

  // grad_img with contiguous filters: the transposed filters times grad_out give the per-tap data gradients
  //   cols (B, G, C/G*K*K, OH*OW) = filters^T (G, C/G*K*K, O/G) x grad_out (B, G, O/G, OH*OW)
  // and a gather (col2im) folds them into the image.  Against the gather-then-GEMM lowering below this
  // moves B*C*K*K*OH*OW elements through the workspace instead of B*O*K*K*H*W, and the GEMM has C/G*K*K rows
  // (full MMA tiles) instead of C/G.  Images go through in groups whose cols stay resident in L2 between the
  // GEMM that writes them and the fold that reads them.
  bool grad_img_done = !grad_img;
  const int64_t blocks_per_plane = (hw + NT * FOLD_P - 1) / (NT * FOLD_P);   // upper bound of the fold's grid
  if (grad_img && filters_contig && n_fwd_patches > 0 && g_conv_grad_img_mode != 1 && fits_int(op) &&
      op.batch * op.chan_in * blocks_per_plane < ((int64_t)1 << 31) &&
      op.dilation * (op.kw + 4) + op.w_in + op.pw < ((int64_t)1 << 31) && op.dilation * op.kh + op.h_in + op.ph < ((int64_t)1 << 31)) {
    const int64_t npos = op.h_out * op.w_out, per_image = op.chan_in * KK * npos;
    int64_t group = op.batch;
    const size_t group_bytes = g_conv_group_bytes.load();
    if (group_bytes > 0) {
      group = (int64_t)(group_bytes / ((size_t)per_image * sizeof(T)));
      group = group < 1 ? 1 : (group > op.batch ? op.batch : group);
    }
    for (int64_t b0 = 0; b0 < op.batch; b0 += group) {
      const int64_t nb = op.batch - b0 < group ? op.batch - b0 : group;
      GemmProblem p;
      p.dtype = dtype; p.beta = 0; p.b0 = nb; p.b1 = G; p.m = cg * KK; p.k = og; p.n = npos;
      p.a = filters; p.a_b0 = 0; p.a_b1 = og * cg * KK; p.a_r = 1; p.a_c = cg * KK;
      p.b = grad_out + b0 * op.chan_out * npos; p.b_b0 = op.chan_out * npos; p.b_b1 = og * npos; p.b_r = npos; p.b_c = 1;
      p.c = patches; p.c_b0 = per_image; p.c_b1 = cg * KK * npos; p.c_r = npos; p.c_c = 1;
      if ((rc = run_gemm(p, stream))) return rc;
      T* dst = grad_img + b0 * op.chan_in * hw;
      launch_fold<T, A>(op, nb * op.chan_in, patches, dst, stream);
      count_launch(false);
      if ((rc = note_cuda_error(cudaGetLastError(), "fold_cols launch"))) return rc;
    }
    grad_img_done = true;
  }
  if (grad_img_done && (grad_filters_done || !grad_filters)) return B200_OK;

  if (plane_path_output<T>(op))
    unfold_output_plane_kernel<T><<<(unsigned)(op.batch * op.chan_out), NT,
                                    (size_t)(op.h_out * op.w_out) * sizeof(T), stream>>>(to_op32(op), grad_out, patches);
  else
    unfold_output_kernel<T><<<grid_for(n_patches, sms), NT, 0, stream>>>(op, grad_out, patches, n_patches);
  count_launch(false);
  if ((rc = note_cuda_error(cudaGetLastError(), "unfold_output launch"))) return rc;

  if (!grad_img_done) {
    transpose_filters_kernel<T><<<grid_for(n_filters, sms), NT, 0, stream>>>(op, filters, st, ftr, n_filters);
    count_launch(false);
    if ((rc = note_cuda_error(cudaGetLastError(), "transpose_filters launch"))) return rc;
    // grad_img (B, G, C/G, H*W) += filters_tr (G, C/G, O/G*K*K) x patches (B, G, O/G*K*K, H*W)
    const int64_t m = cg, k = og * KK, n = hw;
    GemmProblem p;
    p.dtype = dtype; p.beta = 1; p.b0 = op.batch; p.b1 = G; p.m = m; p.k = k; p.n = n;
    p.a = ftr; p.a_b0 = 0; p.a_b1 = m * k; p.a_r = k; p.a_c = 1;
    p.b = patches; p.b_b0 = G * k * n; p.b_b1 = k * n; p.b_r = n; p.b_c = 1;
    p.c = grad_img; p.c_b0 = G * m * n; p.c_b1 = m * n; p.c_r = n; p.c_c = 1;
    if ((rc = run_gemm(p, stream))) return rc;
  }
  if (grad_filters && !grad_filters_done) {
    // grad_filters_tr (B, G, C/G, O/G*K*K) = img (B, G, C/G, H*W) x patches^T (B, G, H*W, O/G*K*K)
    const int64_t m = cg, k = hw, n = og * KK;
    GemmProblem p;
    p.dtype = dtype; p.beta = 0; p.b0 = op.batch; p.b1 = G; p.m = m; p.k = k; p.n = n;
    p.a = img; p.a_b0 = G * m * k; p.a_b1 = m * k; p.a_r = k; p.a_c = 1;
    p.b = patches; p.b_b0 = G * k * n; p.b_b1 = k * n; p.b_r = 1; p.b_c = k;
    p.c = gftr; p.c_b0 = G * m * n; p.c_b1 = m * n; p.c_r = n; p.c_c = 1;
    if ((rc = run_gemm(p, stream))) return rc;
    sum_transposed_filters_kernel<T, A><<<grid_for(n_filters, sms), NT, 0, stream>>>(op, gftr, grad_filters, st,
                                                                                      n_filters);
    count_launch(false);
    if ((rc = note_cuda_error(cudaGetLastError(), "sum_transposed_filters launch"))) return rc;
  }
  return B200_OK;
}

}  // namespace

namespace {
// Overflow-checked products of caller-supplied extents: false when the product does not fit a size_t.
bool mul_ok(size_t* acc, int64_t f) {
  if (f < 0) return false;
  return !__builtin_mul_overflow(*acc, (size_t)f, acc);
}
bool product(size_t* out, std::initializer_list<int64_t> factors) {
  size_t acc = 1;
  for (int64_t f : factors)
    if (!mul_ok(&acc, f)) return false;
  *out = acc;
  return true;
}
constexpr size_t WS_OVERFLOW = ~(size_t)0;

// Bytes of workspace one pass needs; WS_OVERFLOW when the geometry's element counts do not fit a size_t (or the
// 31-bit index arithmetic of the kernels), 0 when there is nothing to compute.
size_t workspace_bytes_op(int dtype, const Op& o, int backward) {
  const size_t es = dtype_size(dtype);
  if (!es || !o.groups) return 0;
  size_t fwd_patches, bwd_patches, nf, bnf, img_elems, out_elems;
  if (!product(&fwd_patches, {o.batch, o.chan_in, o.kh, o.kw, o.h_out, o.w_out, (int64_t)es}) ||
      !product(&bwd_patches, {o.batch, o.chan_out, o.kh, o.kw, o.h_in, o.w_in, (int64_t)es}) ||
      !product(&nf, {o.groups, o.chan_in / o.groups, o.chan_out / o.groups, o.kh, o.kw, (int64_t)es}) ||
      !product(&bnf, {o.batch, (int64_t)nf}) ||
      !product(&img_elems, {o.batch, o.chan_in, o.h_in, o.w_in, (int64_t)es}) ||
      !product(&out_elems, {o.batch, o.chan_out, o.h_out, o.w_out, (int64_t)es}))
    return WS_OVERFLOW;
  const size_t big = (size_t)1 << 62;
  if (fwd_patches > big || bwd_patches > big || bnf > big) return WS_OVERFLOW;
  // the implicit-GEMM lowerings keep a channels-last copy of the image (or of grad_out) with padded channels and
  // the re-laid-out filters instead of patches; with a 1x1 filter that can be more than the patches take
  size_t impl_fwd = 0, impl_bwd = 0;
  if (dtype == B200_F32 && o.stride == 1) {
    const int64_t cg = o.chan_in / o.groups, og = o.chan_out / o.groups;
    const int64_t c16 = round_up(cg, 16), c32 = round_up(cg, 32), o16 = round_up(og, 16);
    size_t a, b, c, d, e, f;
    if (!product(&a, {o.batch, o.h_in, o.w_in, o.groups, c16, 4}) || !product(&b, {o.groups, og, o.kh, o.kw, c16, 4}) ||
        !product(&c, {o.batch, o.h_in, o.w_in, o.groups, c32, 4}) || !product(&d, {o.groups, og, o.kh, o.kw, c32, 4}) ||
        !product(&e, {o.batch, o.h_out, o.w_out, o.groups, o16, 4}) || !product(&f, {o.groups, cg, o.kh, o.kw, o16, 4}) ||
        a > big || c > big || e > big)
      return WS_OVERFLOW;
    impl_fwd = align256(a) + align256(b);
    const size_t w = align256(c) + align256(d), g = align256(e) + align256(f);
    impl_bwd = w > g ? w : g;
  }
  if (!backward) return align256(fwd_patches) > impl_fwd ? align256(fwd_patches) : impl_fwd;
  const size_t old_bwd = align256(bwd_patches > fwd_patches ? bwd_patches : fwd_patches) + align256(nf) + align256(bnf);
  return old_bwd > impl_bwd ? old_bwd : impl_bwd;
}

int forward_any(int dtype, const Op& op, const void* img, const size_t is[4], const void* filters, void* out, void* ws,
                cudaStream_t stream, int beta = 0) {
  switch (dtype) {
    case B200_F32: return forward_t<float, float>(dtype, op, (const float*)img, is, (const float*)filters, (float*)out, ws, stream, beta);
    case B200_F64: return forward_t<double, double>(dtype, op, (const double*)img, is, (const double*)filters, (double*)out, ws, stream, beta);
    case B200_F16:
    case B200_AMP_F16: return forward_t<__half, float>(dtype, op, (const __half*)img, is, (const __half*)filters, (__half*)out, ws, stream, beta);
    default: return B200_ERR_DTYPE;
  }
}

int backward_any(int dtype, const Op& op, const void* img, void* grad_img, const void* filters, const size_t fs[4],
                 void* grad_filters, const void* grad_out, void* ws, cudaStream_t stream) {
  switch (dtype) {
    case B200_F32: return backward_t<float, float>(dtype, op, (const float*)img, (float*)grad_img, (const float*)filters, fs, (float*)grad_filters, (const float*)grad_out, ws, stream);
    case B200_F64: return backward_t<double, double>(dtype, op, (const double*)img, (double*)grad_img, (const double*)filters, fs, (double*)grad_filters, (const double*)grad_out, ws, stream);
    case B200_F16:
    case B200_AMP_F16: return backward_t<__half, float>(dtype, op, (const __half*)img, (__half*)grad_img, (const __half*)filters, fs, (__half*)grad_filters, (const __half*)grad_out, ws, stream);
    default: return B200_ERR_DTYPE;
  }
}

// conv1d (dfdx-core/src/tensor_ops/conv1d/mod.rs:12-23) as a convolution over an image of height 1.
Op to_op(const b200_conv1d_op* o) {
  Op r;
  r.kh = 1; r.kw = (int64_t)o->kernel; r.stride = (int64_t)o->stride; r.ph = 0; r.pw = (int64_t)o->padding;
  r.dilation = (int64_t)o->dilation; r.groups = (int64_t)o->groups; r.batch = (int64_t)o->batch;
  r.chan_in = (int64_t)o->chan_in; r.chan_out = (int64_t)o->chan_out; r.h_in = 1; r.h_out = 1;
  r.w_in = (int64_t)o->l_in; r.w_out = (int64_t)o->l_out;
  return r;
}
// A transposed convolution is the data gradient of a convolution: convtrans2d(img, w) with img (B, C, H, W) and
// w (C, O/G, K, K) equals the grad_img of the conv2d that maps (B, O, H_out, W_out) to (B, C, H, W) with the same
// filters, fed with img as its grad_out.  `to_op_ct` is that conv2d (dfdx lowers it the same way:
// convtrans2d/cuda_kernel.rs:77-148 gathers patches over the output positions and multiplies by transposed filters).
Op to_op_ct(const b200_convtrans2d_op* o) {
  Op r;
  r.kh = r.kw = (int64_t)o->kernel; r.stride = (int64_t)o->stride; r.ph = r.pw = (int64_t)o->padding;
  r.dilation = (int64_t)o->dilation; r.groups = (int64_t)o->groups; r.batch = (int64_t)o->batch;
  r.chan_in = (int64_t)o->chan_out; r.chan_out = (int64_t)o->chan_in;
  r.h_in = (int64_t)o->h_out; r.w_in = (int64_t)o->w_out; r.h_out = (int64_t)o->h_in; r.w_out = (int64_t)o->w_in;
  return r;
}
}  // namespace

size_t convtrans2d_workspace_bytes(int dtype, const b200_convtrans2d_op* o, int backward) {
  (void)backward;                                            // both passes use the conv2d-backward layout
  return o ? workspace_bytes_op(dtype, to_op_ct(o), 1) : 0;
}

// out (B, O, H_out, W_out) = convtrans2d(img (B, C, H, W) contiguous, filters (C, O/G, K, K) through `fs`).
int convtrans2d_forward(int dtype, const b200_convtrans2d_op* o, const void* img, const void* filters, const size_t fs[4],
                        void* out, void* ws, cudaStream_t stream) {
  const Op op = to_op_ct(o);
  const size_t out_bytes = (size_t)(op.batch * op.chan_in * op.h_in * op.w_in) * dtype_size(dtype);
  if (out_bytes == 0) return B200_OK;
  const int rc = note_cuda_error(cudaMemsetAsync(out, 0, out_bytes, stream), "cudaMemsetAsync(convtrans2d out)");
  if (rc) return rc;                                         // the data-gradient path accumulates
  return backward_any(dtype, op, nullptr, out, filters, fs, nullptr, img, ws, stream);
}

// grad_img += conv2d(grad_out, filters);  grad_filters (through `fs`) += the filter gradient of that conv2d with
// grad_out as its image and img as its output gradient (convtrans2d/cuda_kernel.rs:150-265).
int convtrans2d_backward(int dtype, const b200_convtrans2d_op* o, const void* img, void* grad_img, const void* filters,
                         const size_t fs[4], void* grad_filters, const void* grad_out, void* ws, cudaStream_t stream) {
  const Op op = to_op_ct(o);
  int rc = B200_OK;
  if (grad_img) {
    const size_t gs[4] = {(size_t)(op.chan_in * op.h_in * op.w_in), (size_t)(op.h_in * op.w_in), (size_t)op.w_in, 1};
    if ((rc = forward_any(dtype, op, grad_out, gs, filters, grad_img, ws, stream, 1))) return rc;
  }
  if (grad_filters) rc = backward_any(dtype, op, grad_out, nullptr, filters, fs, grad_filters, img, ws, stream);
  return rc;
}

uint64_t conv_implicit_passes() { return g_implicit_passes.load(); }

void conv_set_lowering(int grad_img_mode, size_t group_bytes) {
  g_conv_grad_img_mode.store(grad_img_mode);
  g_conv_group_bytes.store(group_bytes ? group_bytes : CONV_GROUP_BYTES_DEFAULT);
}

size_t conv2d_workspace_bytes(int dtype, const b200_conv2d_op* o, int backward) {
  return o ? workspace_bytes_op(dtype, to_op(o), backward) : 0;
}
size_t conv1d_workspace_bytes(int dtype, const b200_conv1d_op* o, int backward) {
  return o ? workspace_bytes_op(dtype, to_op(o), backward) : 0;
}
// (B, C, L) and (O, C/G, K) strides are widened to the 4-D form the kernels index with (height stride unused).
int conv1d_forward(int dtype, const b200_conv1d_op* o, const void* img, const size_t is[3], const void* filters, void* out,
                   void* ws, cudaStream_t stream) {
  const size_t is4[4] = {is[0], is[1], 0, is[2]};
  return forward_any(dtype, to_op(o), img, is4, filters, out, ws, stream);
}
int conv1d_backward(int dtype, const b200_conv1d_op* o, const void* img, void* grad_img, const void* filters,
                    const size_t fs[3], void* grad_filters, const void* grad_out, void* ws, cudaStream_t stream) {
  const size_t fs4[4] = {fs[0], fs[1], fs[2] * (size_t)o->kernel, fs[2]};
  return backward_any(dtype, to_op(o), img, grad_img, filters, fs4, grad_filters, grad_out, ws, stream);
}

int conv2d_forward(int dtype, const b200_conv2d_op* o, const void* img, const size_t is[4], const void* filters,
                   void* out, void* ws, cudaStream_t stream) {
  return forward_any(dtype, to_op(o), img, is, filters, out, ws, stream);
}

int conv2d_backward(int dtype, const b200_conv2d_op* o, const void* img, void* grad_img, const void* filters,
                    const size_t fs[4], void* grad_filters, const void* grad_out, void* ws, cudaStream_t stream) {
  return backward_any(dtype, to_op(o), img, grad_img, filters, fs, grad_filters, grad_out, ws, stream);
}

}  // namespace b200

// ------------------------------------------------------------------------------------------------
// conv2d forward for callers that cannot allocate device memory.
//
// Some users of this library have no way to obtain scratch memory at the moment they need a
// convolution: a process that has handed every byte of the GPU to its own arena at start-up, a
// latency-critical loop in which cudaMalloc's implicit device synchronisation is unacceptable, or a
// component that is only ever given input and output buffers by its host application.  For them the
// im2col patch buffer lives in a fixed array inside the library image instead of in a caller-provided
// workspace.  The array costs B200_CONV2D_NOALLOC_SCRATCH_BYTES on every GPU for which b200_init has run,
// for the life of the process, whether or not this entry point is ever called.
// ------------------------------------------------------------------------------------------------
namespace b200 {
namespace {

constexpr size_t NOALLOC_SCRATCH_BYTES = (size_t)B200_CONV2D_NOALLOC_SCRATCH_BYTES;

// File-scope device array.  In host code this name is only a handle for the runtime's symbol
// table, never a device address: the address a kernel can use comes from cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];

constexpr int NOALLOC_MAX_DEVICES = 64;
void* g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {};
std::mutex g_noalloc_mutex;

// Resolves the array's address on the CURRENT device, once per device.  Under CUDA's lazy module loading this
// lookup is also what makes the array resident, so it runs inside b200_init: a caller that gives the rest of the
// GPU to its own arena afterwards can no longer be surprised by the array's 32 MiB.
int noalloc_scratch(void** out) {
  int dev = -1;
  int rc = note_cuda_error(cudaGetDevice(&dev), "cudaGetDevice");
  if (rc) return rc;
  if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return B200_ERR_LIMIT;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (!g_noalloc_ptr[dev]) {
    void* p = nullptr;
    rc = note_cuda_error(cudaGetSymbolAddress(&p, g_noalloc_scratch), "cudaGetSymbolAddress(conv2d scratch)");
    if (rc) return rc;
    if (!p) return B200_ERR_CUDA;
    g_noalloc_ptr[dev] = p;
  }
  if (out) *out = g_noalloc_ptr[dev];
  return B200_OK;
}

}  // namespace

// Called by b200_init with the device current.
int conv_noalloc_setup_device() { return noalloc_scratch(nullptr); }

}  // namespace b200

extern "C" int b200_conv2d_forward_noalloc(int dtype, const b200_conv2d_op* op, const void* img,
                                           const size_t img_strides[4], const void* filters, void* out,
                                           void* stream) {
  using namespace b200;
  if (dtype_size(dtype) == 0) return B200_ERR_DTYPE;
  if (!op || !img_strides) return B200_ERR_NULL;
  if (!op->groups || !op->stride || !op->dilation || !op->kernel) return B200_ERR_SHAPE;
  if (op->chan_in % op->groups || op->chan_out % op->groups) return B200_ERR_SHAPE;
  const size_t need = conv2d_workspace_bytes(dtype, op, 0);   // overflow-checked: SIZE_MAX when the extents wrap
  if (need == 0) return B200_OK;
  if (need > NOALLOC_SCRATCH_BYTES) return B200_ERR_LIMIT;   // use b200_conv2d_forward with a workspace instead
  if (!img || !filters || !out) return B200_ERR_NULL;
  if (!device_state()) return note_cuda_error(cudaErrorInitializationError, "b200_init not called on this device");
  void* scratch = nullptr;
  const int rc = noalloc_scratch(&scratch);
  if (rc) return rc;
  // The unfold kernel writes every element of the patch buffer (zeros where a tap falls in the
  // padding), so nothing left over from an earlier call is ever read: no clearing is needed.
  return conv2d_forward(dtype, op, img, img_strides, filters, out, scratch, (cudaStream_t)stream);
}
