// Fused scaled-dot-product attention for f16 tensors:  O = softmax(alpha * Q K^T) V  (forward), keeping the
// score matrix in tensor memory / shared memory instead of HBM.
//
// It stands for the op sequence of dfdx's MultiHeadAttention between the input and output projections
// (dfdx/src/nn/layers/multi_head_attention.rs:136-141: q.matmul(k) * scalar, softmax over the last axis,
// .matmul(v)), which on the unfused path costs two batched GEMMs plus three elementwise passes over the
// (batch, heads, S1, S2) score tensor.
//
// One CTA per (batch, head, 128-query tile); key/value tiles of 128 rows stream through TMA rings.
//   warp 4      TMA producer: Q once, then K_j and V_j
//   warp 5      MMA issuer:   S_j = Q K_j^T (kind::f16, M=128, N=128) into one of two TMEM buffers;
//                             PV_j = P_j V_j (M=128, N=DP) into one of two more.  QK of tile j+1 is issued
//                             before PV of tile j, so the tensor pipe works while the softmax warps are busy.
//   warps 0..3  softmax: thread r owns query row r.  Reads S_j from TMEM, keeps the running row maximum m and
//               sum l (base-2 exponent domain), writes P_j = exp2(x - m) as f16 into shared memory in the
//               128B-swizzled K-major layout the MMA reads, then adds the finished PV_{j-1} into its f32 output
//               registers and rescales them to the new maximum.  After the last tile: O = acc / l, and the
//               row's log-sum-exp for the backward pass.
// Every wait is bounded; on expiry the CTA raises its abort flag, all roles drain and the kernel reports
// B200_ERR_DEVICE_TIMEOUT through the device status word.
#include "tc_device.cuh"
#include <mutex>

namespace b200 {

namespace {

using namespace tcx;

struct AttnArgs {
  int s1, s2, d;
  int heads, q_tiles, kv_tiles;
  float scale_log2;               // alpha * log2(e)
  __half* out;
  long long o_b, o_h, o_s;        // element strides of the (batch, head, query) axes; d has unit stride
  float* lse;                     // (batch, heads, s1) natural-log sum of exp(alpha * s), or nullptr
  long long wait_limit;
  int* status;
};

template <int DP>
struct AttnCfg {
  static constexpr int KV_STAGES = DP == 64 ? 3 : 2;
  static constexpr int Q_BYTES = 128 * DP * 2;
  static constexpr int KV_BYTES = 128 * DP * 2;            // one K or V tile
  static constexpr int P_BYTES = 128 * 128 * 2;
  static constexpr int OFF_K = Q_BYTES;
  static constexpr int OFF_V = OFF_K + KV_STAGES * KV_BYTES;
  static constexpr int OFF_P = OFF_V + KV_STAGES * KV_BYTES;
  static constexpr int SMEM_BYTES = OFF_P + 2 * P_BYTES + 1024;
  static constexpr int THREADS = 192;
  static constexpr int TMEM_COLS = 512;                    // S: 2 x 128, PV: 2 x DP
  static constexpr uint32_t TM_S = 0, TM_O = 256;
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

template <int DP>
__global__ void __launch_bounds__(AttnCfg<DP>::THREADS, 1)
attention_fwd_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                     const __grid_constant__ CUtensorMap tma_v, const AttnArgs g) {
  using C = AttnCfg<DP>;
  constexpr int ST = C::KV_STAGES;
  constexpr int DCH = DP / 64;                             // 64-element chunks of the head dimension

  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t bar_q;
  __shared__ __align__(8) uint64_t bar_k_full[ST], bar_k_empty[ST], bar_v_full[ST], bar_v_empty[ST];
  __shared__ __align__(8) uint64_t bar_s_full[2], bar_s_empty[2], bar_p_full[2], bar_p_empty[2];
  __shared__ __align__(8) uint64_t bar_o_full[2], bar_o_empty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abortp = &abort_flag;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar_q), 1);
    for (int s = 0; s < ST; ++s) {
      mbar_init(smem_u32(&bar_k_full[s]), 1);
      mbar_init(smem_u32(&bar_k_empty[s]), 1);
      mbar_init(smem_u32(&bar_v_full[s]), 1);
      mbar_init(smem_u32(&bar_v_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bar_s_full[b]), 1);
      mbar_init(smem_u32(&bar_s_empty[b]), 128);
      mbar_init(smem_u32(&bar_p_full[b]), 128);
      mbar_init(smem_u32(&bar_p_empty[b]), 1);
      mbar_init(smem_u32(&bar_o_full[b]), 1);
      mbar_init(smem_u32(&bar_o_empty[b]), 128);
    }
    abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(&tmem_slot), C::TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tma_q);
    tma_prefetch_desc(&tma_k);
    tma_prefetch_desc(&tma_v);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;

  // tile -> (batch, head, query tile); query tiles of one head are neighbours so they share K / V in L2
  const int qt = blockIdx.x % g.q_tiles;
  const int bh = blockIdx.x / g.q_tiles;
  const int ih = bh % g.heads, ib = bh / g.heads;
  const int T = g.kv_tiles;
  const int ksteps_qk = (g.d + 15) / 16;                    // k-steps that hold data (the rest of DP is zero fill)

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const uint32_t bq = smem_u32(&bar_q);
      mbar_expect_tx(bq, C::Q_BYTES);
      for (int c = 0; c < DCH; ++c) tma_load_4d(smem_base + c * 16384, &tma_q, bq, c * 64, qt * 128, ih, ib);
      bool ok = true;
      for (int j = 0; ok && j < T; ++j) {
        const int s = j % ST;
        const uint32_t ph = (j / ST) & 1u;
        if (!mbar_wait(smem_u32(&bar_k_empty[s]), ph ^ 1u, abortp, g.wait_limit)) { ok = false; break; }
        const uint32_t fk = smem_u32(&bar_k_full[s]);
        mbar_expect_tx(fk, C::KV_BYTES);
        for (int c = 0; c < DCH; ++c)
          tma_load_4d(smem_base + C::OFF_K + s * C::KV_BYTES + c * 16384, &tma_k, fk, c * 64, j * 128, ih, ib);
        if (!mbar_wait(smem_u32(&bar_v_empty[s]), ph ^ 1u, abortp, g.wait_limit)) { ok = false; break; }
        const uint32_t fv = smem_u32(&bar_v_full[s]);
        mbar_expect_tx(fv, C::KV_BYTES);
        for (int c = 0; c < DCH; ++c)
          tma_load_4d(smem_base + C::OFF_V + s * C::KV_BYTES + c * 16384, &tma_v, fv, c * 64, j * 128, ih, ib);
      }
    }
    __syncwarp();
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // S = Q K^T: A and B K-major, N = 128.   PV = P V: A K-major, B MN-major (V rows are keys), N = DP.
      const uint32_t idesc_qk = (1u << 4) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      const uint32_t idesc_pv = (1u << 4) | (1u << 16) | ((uint32_t)(DP >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      bool ok = mbar_wait(smem_u32(&bar_q), 0, abortp, g.wait_limit);
      auto issue_qk = [&](int j) -> bool {
        const int s = j % ST, buf = j & 1;
        if (!mbar_wait(smem_u32(&bar_k_full[s]), (j / ST) & 1u, abortp, g.wait_limit)) return false;
        if (!mbar_wait(smem_u32(&bar_s_empty[buf]), ((j >> 1) & 1u) ^ 1u, abortp, g.wait_limit)) return false;
        tc_fence_after();
        const uint32_t qb = smem_base, kb = smem_base + C::OFF_K + s * C::KV_BYTES;
        for (int ks = 0; ks < ksteps_qk; ++ks) {
          const uint32_t off = (ks >> 2) * 16384 + (ks & 3) * 32;
          umma<2>(tmem_base + C::TM_S + buf * 128, make_smem_desc(qb + off, 16, 1024, 2),
                  make_smem_desc(kb + off, 16, 1024, 2), idesc_qk, ks > 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(&bar_k_empty[s]));
        umma_commit(smem_u32(&bar_s_full[buf]));
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; ok && j < T; ++j) {
        if (j + 1 < T && !issue_qk(j + 1)) { ok = false; break; }
        const int s = j % ST, buf = j & 1;
        const uint32_t ph2 = (j >> 1) & 1u;
        if (!mbar_wait(smem_u32(&bar_v_full[s]), (j / ST) & 1u, abortp, g.wait_limit)) { ok = false; break; }
        if (!mbar_wait(smem_u32(&bar_o_empty[buf]), ph2 ^ 1u, abortp, g.wait_limit)) { ok = false; break; }
        if (!mbar_wait(smem_u32(&bar_p_full[buf]), ph2, abortp, g.wait_limit)) { ok = false; break; }
        tc_fence_after();
        const uint32_t pb = smem_base + C::OFF_P + buf * C::P_BYTES, vb = smem_base + C::OFF_V + s * C::KV_BYTES;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {                    // 128 keys, 16 per MMA
          const uint64_t ad = make_smem_desc(pb + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024, 2);
          const uint64_t bd = make_smem_desc(vb + ks * 2048, 16384, 1024, 2);
          umma<2>(tmem_base + C::TM_O + buf * DP, ad, bd, idesc_pv, ks > 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(&bar_v_empty[s]));
        umma_commit(smem_u32(&bar_p_empty[buf]));
        umma_commit(smem_u32(&bar_o_full[buf]));
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ softmax / output (warps 0..3)
    const int r = warp * 32 + lane;                          // query row inside the tile = TMEM lane
    const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
    const uint32_t p_row = (uint32_t)(r >> 3) * 1024 + (uint32_t)(r & 7) * 128;
    const uint32_t sw = (uint32_t)(r & 7);
    float acc[DP];
#pragma unroll
    for (int q = 0; q < DP; ++q) acc[q] = 0.f;
    float m = -INFINITY, l = 0.f;
    bool ok = true;

    auto add_pv = [&](int j) -> bool {                       // acc += PV_j
      const int buf = j & 1;
      if (!mbar_wait(smem_u32(&bar_o_full[buf]), (j >> 1) & 1u, abortp, g.wait_limit)) return false;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < DP / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(lane_addr + C::TM_O + buf * DP + c * 32, v);
        tmem_wait_ld();
#pragma unroll
        for (int q = 0; q < 32; ++q) acc[c * 32 + q] += __uint_as_float(v[q]);
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&bar_o_empty[buf]));
      return true;
    };

    for (int j = 0; j < T; ++j) {
      const int buf = j & 1;
      const uint32_t ph2 = (j >> 1) & 1u;
      if (!mbar_wait(smem_u32(&bar_s_full[buf]), ph2, abortp, g.wait_limit)) { ok = false; break; }
      tc_fence_after();
      float x[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(lane_addr + C::TM_S + buf * 128 + c * 32, v);
        tmem_wait_ld();
#pragma unroll
        for (int q = 0; q < 32; ++q) x[c * 32 + q] = __uint_as_float(v[q]) * g.scale_log2;
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&bar_s_empty[buf]));
      const int valid = g.s2 - j * 128;                      // keys of this tile that exist
      if (valid < 128) {
#pragma unroll
        for (int q = 0; q < 128; ++q)
          if (q >= valid) x[q] = -INFINITY;
      }
      float mx = x[0];
#pragma unroll
      for (int q = 1; q < 128; ++q) mx = fmaxf(mx, x[q]);
      const float m_new = fmaxf(m, mx);
      // the P buffer is free once PV_{j-2} has been read by the tensor core
      if (!mbar_wait(smem_u32(&bar_p_empty[buf]), ph2 ^ 1u, abortp, g.wait_limit)) { ok = false; break; }
      const uint32_t pb = smem_base + C::OFF_P + buf * C::P_BYTES + p_row;
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < 16; ++c) {                         // 16-byte chunks of 8 probabilities
        float p[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          p[e] = ex2_approx(x[c * 8 + e] - m_new);
          sum += p[e];
        }
        st_shared_v4(pb + (uint32_t)(c >> 3) * 16384 + ((((uint32_t)c & 7u) ^ sw) << 4),
                     pack_half2(p[0], p[1]), pack_half2(p[2], p[3]), pack_half2(p[4], p[5]), pack_half2(p[6], p[7]));
      }
      fence_proxy_async_smem();                              // generic-proxy writes -> visible to the MMA
      mbar_arrive(smem_u32(&bar_p_full[buf]));
      // fold the previous tile's product in and move everything to the new maximum
      if (j > 0 && !add_pv(j - 1)) { ok = false; break; }
      const float corr = ex2_approx(m - m_new);              // first tile: exp2(-inf) = 0, acc and l are 0
      l = l * corr + sum;
      if (corr != 1.f) {
#pragma unroll
        for (int q = 0; q < DP; ++q) acc[q] *= corr;
      }
      m = m_new;
    }
    if (ok && T > 0) ok = add_pv(T - 1);
    const int row = qt * 128 + r;
    if (ok && row < g.s1) {
      const float inv = 1.f / l;
      __half* dst = g.out + ib * g.o_b + ih * g.o_h + (long long)row * g.o_s;
#pragma unroll
      for (int c = 0; c < DP / 8; ++c) {
        if (c * 8 < g.d) {                                   // d is a multiple of 8
          uint4 o;
          o.x = pack_half2(acc[c * 8 + 0] * inv, acc[c * 8 + 1] * inv);
          o.y = pack_half2(acc[c * 8 + 2] * inv, acc[c * 8 + 3] * inv);
          o.z = pack_half2(acc[c * 8 + 4] * inv, acc[c * 8 + 5] * inv);
          o.w = pack_half2(acc[c * 8 + 6] * inv, acc[c * 8 + 7] * inv);
          *reinterpret_cast<uint4*>(dst + c * 8) = o;
        }
      }
      if (g.lse) g.lse[((long long)ib * g.heads + ih) * g.s1 + row] = (m + log2f(l)) * 0.6931471805599453f;
    }
  }

  tc_fence_before();
  __syncthreads();
  teardown(abort_flag, g.status);
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn attn_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  });
  return fn;
}

// f16 tensor (d, s, h, b) with unit stride along d; box = [64, rows, 1, 1] under the 128B swizzle.
int encode_bhsd(CUtensorMap* map, const void* base, int64_t d, int64_t s, int64_t h, int64_t b, int64_t ss,
                int64_t hs, int64_t bs, uint32_t rows) {
  EncodeTiledFn fn = attn_encode_fn();
  if (!fn) return B200_ERR_CUDA;
  const cuuint64_t dims[4] = {(cuuint64_t)d, (cuuint64_t)s, (cuuint64_t)h, (cuuint64_t)b};
  const uint64_t row = (uint64_t)(s > 1 ? ss : d) * 2;
  const cuuint64_t strides[3] = {row, h > 1 ? (cuuint64_t)hs * 2 : row, b > 1 ? (cuuint64_t)bs * 2 : row};
  const cuuint32_t box[4] = {64, rows, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? B200_OK : B200_ERR_UNSUPPORTED;
}

bool stride_ok(int64_t extent, int64_t stride) { return extent <= 1 || (stride > 0 && stride % 8 == 0); }

template <int DP>
int launch_fwd(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const AttnArgs& g, int64_t ctas,
               cudaStream_t stream) {
  attention_fwd_kernel<DP><<<(unsigned)ctas, AttnCfg<DP>::THREADS, AttnCfg<DP>::SMEM_BYTES, stream>>>(mq, mk, mv, g);
  count_launch(true);
  return note_cuda_error(cudaGetLastError(), "attention forward launch");
}

}  // namespace

int attention_setup_device() {
  int rc = note_cuda_error(cudaFuncSetAttribute(attention_fwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                AttnCfg<64>::SMEM_BYTES), "cudaFuncSetAttribute(attention 64)");
  if (rc) return rc;
  return note_cuda_error(cudaFuncSetAttribute(attention_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              AttnCfg<128>::SMEM_BYTES), "cudaFuncSetAttribute(attention 128)");
}

// q: (B, H, S1, D) view, k: (B, H, D, S2) view (what MultiHeadAttention hands to matmul), v: (B, H, S2, D) view,
// out: (B, H, S1, D) view; all with unit stride along D.
int attention_forward(int dtype, int64_t B, int64_t H, int64_t s1, int64_t s2, int64_t d, const void* q,
                      const int64_t qs[4], const void* k, const int64_t ks[4], const void* v, const int64_t vs[4],
                      double alpha, void* out, const int64_t os[4], float* lse, cudaStream_t stream) {
  if (dtype != B200_F16 && dtype != B200_AMP_F16) return B200_ERR_UNSUPPORTED;
  if (B == 0 || H == 0 || s1 == 0) return B200_OK;
  if (s2 == 0 || d == 0) return B200_ERR_SHAPE;             // a softmax over no keys is undefined
  DeviceState* ds = device_state();
  if (!ds || !ds->ready) return note_cuda_error(cudaErrorInitializationError, "b200_init not called on this device");
  if (d % 8 || d > 128) return B200_ERR_UNSUPPORTED;
  if (qs[3] != 1 || ks[2] != 1 || vs[3] != 1 || os[3] != 1) return B200_ERR_UNSUPPORTED;
  if (!stride_ok(s1, qs[2]) || !stride_ok(H, qs[1]) || !stride_ok(B, qs[0]) || !stride_ok(s2, ks[3]) ||
      !stride_ok(H, ks[1]) || !stride_ok(B, ks[0]) || !stride_ok(s2, vs[2]) || !stride_ok(H, vs[1]) ||
      !stride_ok(B, vs[0]) || !stride_ok(s1, os[2]) || !stride_ok(H, os[1]) || !stride_ok(B, os[0]))
    return B200_ERR_UNSUPPORTED;
  if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) & 15) return B200_ERR_UNSUPPORTED;
  if (s1 > 0x7fffff00LL || s2 > 0x7fffff00LL || B * H > 0x7fffffffLL) return B200_ERR_LIMIT;
  const int64_t q_tiles = (s1 + 127) / 128, ctas = q_tiles * H * B;
  if (ctas > 0x7fffffffLL) return B200_ERR_LIMIT;

  alignas(64) CUtensorMap mq, mk, mv;
  int rc;
  if ((rc = encode_bhsd(&mq, q, d, s1, H, B, qs[2], qs[1], qs[0], 128))) return rc;
  if ((rc = encode_bhsd(&mk, k, d, s2, H, B, ks[3], ks[1], ks[0], 128))) return rc;
  if ((rc = encode_bhsd(&mv, v, d, s2, H, B, vs[2], vs[1], vs[0], 128))) return rc;
  AttnArgs g;
  g.s1 = (int)s1; g.s2 = (int)s2; g.d = (int)d;
  g.heads = (int)H; g.q_tiles = (int)q_tiles; g.kv_tiles = (int)((s2 + 127) / 128);
  g.scale_log2 = (float)(alpha * 1.4426950408889634);
  g.out = (__half*)out; g.o_b = os[0]; g.o_h = os[1]; g.o_s = os[2];
  g.lse = lse;
  g.wait_limit = 400000000LL + (long long)g.kv_tiles * 400000LL;
  g.status = ds->status;
  return d <= 64 ? launch_fwd<64>(mq, mk, mv, g, ctas, stream) : launch_fwd<128>(mq, mk, mv, g, ctas, stream);
}

}  // namespace b200
