// Fused scaled-dot-product attention for f16 tensors:  O = softmax(alpha * Q K^T) V  (forward), keeping the
// score matrix in tensor memory / shared memory instead of HBM.
//
// It stands for the op sequence of dfdx's MultiHeadAttention between the input and output projections
// (dfdx/src/nn/layers/multi_head_attention.rs:136-141: q.matmul(k) * scalar, softmax over the last axis,
// .matmul(v)), which on the unfused path costs two batched GEMMs plus three elementwise passes over the
// (batch, heads, S1, S2) score tensor.
//
// One work item per (batch, head, 256 queries), walked by a grid of at most one CTA per SM (item = blockIdx.x,
// + gridDim.x, ...: every barrier keeps counting across items, so the next item's loads and first S = Q K^T run
// under the current item's last exponentials and output): two query tiles of 128 rows, each owned by one softmax warpgroup,
// share the key/value tiles (128 rows each) that stream through TMA rings.
//   warpgroup 2  warp 8: TMA producer (both Q tiles once, then K_j and V_j); warps 9, 10, 11: MMA issuers (one
//                thread each: all S_t = Q_t K_j^T (kind::f16, M=128, N=128); PV_0 = P_0 V_j; PV_1 = P_1 V_j with
//                M=128, N=DP), results in TMEM.  QK of tile j+1 is issued as soon as the softmax warps have read S_t(j), so the
//                tensor pipe works while they are busy.
//   warpgroups 0, 1  softmax: thread r owns query row r of tile t.  Reads S_t(j) from TMEM, adds the finished
//                PV_t(j-1) into its f32 output registers, keeps the running row maximum m and sum l (base-2
//                exponent domain), rescales, writes P = exp2(s*scale - m) as f16 into shared memory in the
//                128B-swizzled K-major layout the MMA reads.  After the last tile: O = acc / l, and the row's
//                log-sum-exp for the backward pass.  Two warpgroups give every scheduler two independent
//                softmax warps (the exponentials run on the 16-per-clock SFU pipe and bound the kernel).
//   Registers are moved from warpgroup 2 to the softmax warpgroups with setmaxnreg.
// Every wait is bounded; on expiry the CTA raises its abort flag, all roles drain and the kernel reports
// B200_ERR_DEVICE_TIMEOUT through the device status word.
#include "attention_common.cuh"

namespace b200 {

namespace {

using namespace tcx;
using namespace attn;

struct AttnArgs {
  int s1, s2, d;
  int heads, q_pairs, kv_tiles;    // q_pairs: work items per (batch, head), each 256 queries
  long long items;                // batch * heads * q_pairs; CTA c takes items c, c + gridDim.x, ...
  float scale_log2;               // alpha * log2(e)
  __half* out;
  long long o_b, o_h, o_s;        // element strides of the (batch, head, query) axes; d has unit stride
  float* lse;                     // (batch, heads, s1) natural-log sum of exp(alpha * s), or nullptr
  long long wait_limit;
  int* status;
};

template <int DP>
struct AttnCfg {
  static constexpr int KV_STAGES = DP == 64 ? 2 : 1;       // DP = 128: shared memory holds one K and one V tile
  static constexpr int NB = DP == 64 ? 2 : 1;              // buffers per query tile for P (shared memory) and PV (TMEM)
  static constexpr int Q_BYTES = 128 * DP * 2;             // one query tile
  static constexpr int KV_BYTES = 128 * DP * 2;            // one K or V tile
  static constexpr int P_BYTES = 128 * 128 * 2;            // one probability tile
  static constexpr int OFF_K = 2 * Q_BYTES;
  static constexpr int OFF_V = OFF_K + KV_STAGES * KV_BYTES;
  static constexpr int OFF_P = OFF_V + KV_STAGES * KV_BYTES;
  static constexpr int SMEM_BYTES = OFF_P + 2 * NB * P_BYTES + 1024;
  static constexpr int THREADS = 384;
  static constexpr int TMEM_COLS = 512;                    // per query tile: S 128 columns, PV DP columns
  static constexpr uint32_t TM_S = 0, TM_O = 256;
};
// setmaxnreg budget: 384 threads x 168 registers at launch; 2 x 128 x 232 + 128 x 40 = 64512.
constexpr int ATT_REGS_LAUNCH = 168, ATT_REGS_SOFTMAX = 232, ATT_REGS_LOW = 40;
static_assert(2 * 128 * ATT_REGS_SOFTMAX + 128 * ATT_REGS_LOW <= 384 * ATT_REGS_LAUNCH,
              "setmaxnreg budget exceeds the CTA's launch allocation");

template <int DP>
__global__ void __launch_bounds__(AttnCfg<DP>::THREADS, 1)
attention_fwd_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                     const __grid_constant__ CUtensorMap tma_v, const AttnArgs g) {
  using C = AttnCfg<DP>;
  constexpr int ST = C::KV_STAGES;
  constexpr int DCH = DP / 64;                             // 64-element chunks of the head dimension
  constexpr int NB = C::NB;
  constexpr int P_STRIDE = NB * C::P_BYTES;                // per query tile
  // DP = 128: the output accumulator takes 128 registers, so the score row is not kept in registers between
  // the maximum and the exponentials but read from tensor memory twice.
  constexpr bool TWO_PASS = DP == 128;

  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t bar_q, bar_q_empty;
  __shared__ __align__(8) uint64_t bar_k_full[ST], bar_k_empty[ST], bar_v_full[ST], bar_v_empty[ST];
  // per query tile, one completion per key tile
  __shared__ __align__(8) uint64_t bar_s_full[2], bar_s_empty[2];
  __shared__ __align__(8) uint64_t bar_p_full[2][NB], bar_p_empty[2][NB], bar_o_full[2][NB], bar_o_empty[2][NB];
  __shared__ __align__(8) uint64_t bar_turn[2];           // ping-pong of the two softmax warpgroups' exponential phases
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wg = warp >> 2;
  volatile int* abortp = &abort_flag;

  // query tiles that hold rows: the same for every item of this CTA (a grid smaller than the item count is only
  // launched when all items have two)
  const int ntile0 = (((int)(blockIdx.x % g.q_pairs) * 2 + 1) * 128 < g.s1) ? 2 : 1;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar_q), 1);
    mbar_init(smem_u32(&bar_q_empty), 1);
    for (int s = 0; s < ST; ++s) {
      mbar_init(smem_u32(&bar_k_full[s]), 1);
      mbar_init(smem_u32(&bar_k_empty[s]), 1);
      mbar_init(smem_u32(&bar_v_full[s]), 1);
      mbar_init(smem_u32(&bar_v_empty[s]), ntile0);         // released by the PV issuer of every query tile
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(smem_u32(&bar_s_full[t]), 1);
      mbar_init(smem_u32(&bar_s_empty[t]), 4);              // one arrival per softmax warp
      for (int b = 0; b < NB; ++b) {
        mbar_init(smem_u32(&bar_p_full[t][b]), 4);
        mbar_init(smem_u32(&bar_p_empty[t][b]), 1);
        mbar_init(smem_u32(&bar_o_full[t][b]), 1);
        mbar_init(smem_u32(&bar_o_empty[t][b]), 4);
      }
      mbar_init(smem_u32(&bar_turn[t]), 4);
    }
    abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 9) {
    tmem_alloc(smem_u32(&tmem_slot), C::TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 8 && lane == 0) {
    tma_prefetch_desc(&tma_q);
    tma_prefetch_desc(&tma_k);
    tma_prefetch_desc(&tma_v);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;

  // CTA -> (batch, head, pair of query tiles); the pairs of one head are neighbours so they share K / V in L2
  const int T = g.kv_tiles;
  const int ntile = ntile0;                                 // query tiles of this CTA that hold rows
  const int ksteps_qk = (g.d + 15) / 16;                    // k-steps that hold data (the rest of DP is zero fill)

  if (wg == 2) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 8) {
      // ---------------------------------------------------------------- TMA producer
      if (lane == 0) {
        const uint32_t bq = smem_u32(&bar_q);
        bool ok = true;
        int it = 0;
        for (long long item = blockIdx.x; ok && item < g.items; item += gridDim.x, ++it) {
        const int qp = (int)(item % g.q_pairs);
        const long long bh = item / g.q_pairs;
        const int ih = (int)(bh % g.heads), ib = (int)(bh / g.heads);
        // the Q tiles are free once the previous item's last S = Q K^T has been computed
        if (it > 0 && !mbar_wait(smem_u32(&bar_q_empty), (uint32_t)(it - 1) & 1u, abortp, g.wait_limit)) break;
        mbar_expect_tx(bq, ntile * C::Q_BYTES);
        for (int t = 0; t < ntile; ++t)
          for (int c = 0; c < DCH; ++c)
            tma_load_4d(smem_base + t * C::Q_BYTES + c * 16384, &tma_q, bq, c * 64, (qp * 2 + t) * 128, ih, ib);
        for (int j = 0; ok && j < T; ++j) {
          const int jg = it * T + j;                           // tiles this CTA has streamed so far: ring position
          const int s = jg % ST;
          const uint32_t ph = (jg / ST) & 1u;
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
      }
      __syncwarp();
    } else {
      // ---------------------------------------------------------------- MMA issuers
      // Three single-thread issuers: warp 9 issues every S = Q K^T, warps 10 and 11 issue PV for query tile 0
      // and 1.  One thread doing all of it was the kernel's critical path: each wait, descriptor update and
      // commit is a short dependent instruction chain that competes with the softmax warps for issue slots.
      if (lane == 0) {
        // descriptor words: low = (address >> 4) | (leading offset >> 4) << 16, high = (stride offset >> 4) | version | swizzle
        const uint64_t dk = make_smem_desc(smem_base, 16, 1024, 2);             // K-major tiles (Q, K, P)
        const uint64_t dv = make_smem_desc(smem_base, 16384, 1024, 2);          // MN-major tile (V)
        const uint32_t hi_k = (uint32_t)(dk >> 32), hi_v = (uint32_t)(dv >> 32);
        if (warp == 9) {
          // S = Q K^T: A and B K-major, N = 128
          const uint32_t idesc_qk = (1u << 4) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
          const uint32_t q_lo = (uint32_t)dk, k_lo = (uint32_t)dk + (uint32_t)(C::OFF_K >> 4);
          bool ok = true;
          int it = 0;
          for (long long item = blockIdx.x; ok && item < g.items; item += gridDim.x, ++it) {
          ok = mbar_wait(smem_u32(&bar_q), (uint32_t)it & 1u, abortp, g.wait_limit);
          // S_t(j): needs K_j and the softmax warps of tile t to have read the S_t before it (the previous item's last
          // one for j = 0)
          for (int j = 0; ok && j < T; ++j) {
            const int jg = it * T + j;
            const int s = jg % ST;
            if (!mbar_wait(smem_u32(&bar_k_full[s]), (jg / ST) & 1u, abortp, g.wait_limit)) { ok = false; break; }
            const uint32_t klo = k_lo + (uint32_t)(s * (C::KV_BYTES >> 4));
            for (int t = 0; t < ntile; ++t) {
              if (jg > 0 && !mbar_wait(smem_u32(&bar_s_empty[t]), (uint32_t)(jg - 1) & 1u, abortp, g.wait_limit)) { ok = false; break; }
              tc_fence_after();
              const uint32_t alo = q_lo + (uint32_t)(t * C::Q_BYTES >> 4);
              if (ksteps_qk == DP / 16) {
#pragma unroll
                for (int ks = 0; ks < DP / 16; ++ks) {
                  const uint32_t off = (uint32_t)(((ks >> 2) * 16384 + (ks & 3) * 32) >> 4);
                  umma_lohi<2>(tmem_base + C::TM_S + t * 128, alo + off, hi_k, klo + off, hi_k, idesc_qk, ks > 0 ? 1u : 0u);
                }
              } else {
                for (int ks = 0; ks < ksteps_qk; ++ks) {
                  const uint32_t off = (uint32_t)(((ks >> 2) * 16384 + (ks & 3) * 32) >> 4);
                  umma_lohi<2>(tmem_base + C::TM_S + t * 128, alo + off, hi_k, klo + off, hi_k, idesc_qk, ks > 0 ? 1u : 0u);
                }
              }
              umma_commit(smem_u32(&bar_s_full[t]));
            }
            if (ok) umma_commit(smem_u32(&bar_k_empty[s]));
          }
          if (ok) umma_commit(smem_u32(&bar_q_empty));       // all of this item's S MMAs have read Q
          }
        } else if (warp - 10 < ntile) {
          // PV = P V: A K-major, B MN-major (V rows are keys), N = DP
          const int t = warp - 10;
          const uint32_t idesc_pv = (1u << 4) | (1u << 16) | ((uint32_t)(DP >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
          const uint32_t p_lo = (uint32_t)dk + (uint32_t)((C::OFF_P + t * P_STRIDE) >> 4);
          const uint32_t v_lo = (uint32_t)dv + (uint32_t)(C::OFF_V >> 4);
          bool ok = true;
          int it = 0;
          for (long long item = blockIdx.x; ok && item < g.items; item += gridDim.x, ++it)
          for (int j = 0; j < T; ++j) {
            const int jg = it * T + j;
            const int s = jg % ST;
            // PV_t(j): needs V_j, P_t(j) and the softmax warps to have taken the PV_t that last used the buffer out of
            // tensor memory
            if (!mbar_wait(smem_u32(&bar_v_full[s]), (jg / ST) & 1u, abortp, g.wait_limit)) { ok = false; break; }
            const int b = jg % NB;
            const uint32_t bph = (uint32_t)(jg / NB) & 1u;
            if (jg >= NB && !mbar_wait(smem_u32(&bar_o_empty[t][b]), bph ^ 1u, abortp, g.wait_limit)) { ok = false; break; }
            if (!mbar_wait(smem_u32(&bar_p_full[t][b]), bph, abortp, g.wait_limit)) { ok = false; break; }
            const uint32_t plo = p_lo + (uint32_t)(b * (C::P_BYTES >> 4));
            tc_fence_after();
            const uint32_t vlo = v_lo + (uint32_t)(s * (C::KV_BYTES >> 4));
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)                    // 128 keys, 16 per MMA
              umma_lohi<2>(tmem_base + C::TM_O + (t * NB + b) * DP, plo + (uint32_t)(((ks >> 2) * 16384 + (ks & 3) * 32) >> 4), hi_k,
                            vlo + (uint32_t)(ks * 2048 >> 4), hi_v, idesc_pv, ks > 0 ? 1u : 0u);
            umma_commit(smem_u32(&bar_p_empty[t][b]));
            umma_commit(smem_u32(&bar_o_full[t][b]));
            umma_commit(smem_u32(&bar_v_empty[s]));           // one arrival per query tile
          }
        }
      }
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------------ softmax / output (warpgroups 0, 1)
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    const int t = wg;                                        // query tile of this warpgroup
    if (t < ntile) {
      const int r = (warp & 3) * 32 + lane;                  // query row inside the tile = TMEM lane
      const uint32_t lane_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
      const uint32_t p_row = (uint32_t)(r >> 3) * 1024 + (uint32_t)(r & 7) * 128;
      const uint32_t sw = (uint32_t)(r & 7);
      const uint32_t pb0 = smem_base + C::OFF_P + t * P_STRIDE + p_row;
      const float scale = g.scale_log2;
      const bool pos = scale >= 0.f;
      bool ok = true;
      int it = 0;
      for (long long item = blockIdx.x; ok && item < g.items; item += gridDim.x, ++it) {
      const int qp = (int)(item % g.q_pairs);
      const long long bh = item / g.q_pairs;
      const int ih = (int)(bh % g.heads), ib = (int)(bh / g.heads);
      const int jg0 = it * T;                                // tiles this CTA has worked through before this item
      float acc[DP];
#pragma unroll
      for (int q = 0; q < DP; ++q) acc[q] = 0.f;
      float m = -INFINITY, l = 0.f;                          // m in the scaled base-2 domain

      float corr = 1.f;                                      // factor that moves acc to the current maximum
      auto add_pv = [&](int jg) -> bool {                    // acc = acc * corr + PV_t(jg)
        const int b = jg % NB;
        if (!mbar_wait_warp(smem_u32(&bar_o_full[t][b]), (uint32_t)(jg / NB) & 1u, abortp, g.wait_limit)) return false;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < DP / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(lane_addr + C::TM_O + (t * NB + b) * DP + c * 32, v);
          tmem_wait_ld();
#pragma unroll
          for (int q = 0; q < 32; ++q) acc[c * 32 + q] = fmaf(acc[c * 32 + q], corr, __uint_as_float(v[q]));
        }
        tc_fence_before();
        warp_arrive(smem_u32(&bar_o_empty[t][b]), lane);
        return true;
      };

      for (int j = 0; j < T; ++j) {
        const int jg = jg0 + j;
        if (!mbar_wait_warp(smem_u32(&bar_s_full[t]), (uint32_t)jg & 1u, abortp, g.wait_limit)) { ok = false; break; }
        tc_fence_after();
        const int valid = g.s2 - j * 128;                    // keys of this tile that exist
        const float gone = pos ? -INFINITY : INFINITY;       // a masked score: scaled it is -inf, probability 0
        constexpr int KEEP = TWO_PASS ? 32 : 128;
        uint32_t xr[KEEP];                                   // raw scores of this row (f32 bits)
        float ext;
        const uint32_t s_addr = lane_addr + C::TM_S + t * 128;
        if constexpr (!TWO_PASS) {
#pragma unroll
          for (int c = 0; c < 4; ++c) tmem_ld_32x32(s_addr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&xr[c * 32]));
          tmem_wait_ld();
          tc_fence_before();
          warp_arrive(smem_u32(&bar_s_empty[t]), lane);
          if (valid < 128) {
#pragma unroll
            for (int q = 0; q < 128; ++q)
              if (q >= valid) xr[q] = __float_as_uint(gone);
          }
          float e4[4] = {gone, gone, gone, gone};            // four independent chains
          if (pos) {
#pragma unroll
            for (int q = 0; q < 128; ++q) e4[q & 3] = fmaxf(e4[q & 3], __uint_as_float(xr[q]));
            ext = fmaxf(fmaxf(e4[0], e4[1]), fmaxf(e4[2], e4[3]));
          } else {
#pragma unroll
            for (int q = 0; q < 128; ++q) e4[q & 3] = fminf(e4[q & 3], __uint_as_float(xr[q]));
            ext = fminf(fminf(e4[0], e4[1]), fminf(e4[2], e4[3]));
          }
        } else {
          float e4[4] = {gone, gone, gone, gone};
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            tmem_ld_32x32(s_addr + c * 32, xr);
            tmem_wait_ld();
#pragma unroll
            for (int q = 0; q < 32; ++q) {
              float sv = __uint_as_float(xr[q]);
              if (c * 32 + q >= valid) sv = gone;
              e4[q & 3] = pos ? fmaxf(e4[q & 3], sv) : fminf(e4[q & 3], sv);
            }
          }
          ext = pos ? fmaxf(fmaxf(e4[0], e4[1]), fmaxf(e4[2], e4[3])) : fminf(fminf(e4[0], e4[1]), fminf(e4[2], e4[3]));
        }
        const float m_new = fmaxf(m, ext * scale);
        const float corr_new = ex2_approx(m - m_new);        // first tile: exp2(-inf) = 0, acc and l are 0
        // the P tile is free once PV(j-1) has been read by the tensor core
        const int pbuf = jg % NB;
        if (jg >= NB && !mbar_wait_warp(smem_u32(&bar_p_empty[t][pbuf]), ((uint32_t)(jg / NB) & 1u) ^ 1u, abortp, g.wait_limit)) { ok = false; break; }
        const uint32_t pb = pb0 + pbuf * C::P_BYTES;
        // (With single P / PV buffers, DP = 128, the turns would add to the tensor-core round trip instead.)
        // The two warpgroups take turns in the exponential phase: it saturates the SFU pipe, and in lockstep that
        // pipe would idle while both read scores / fold PV in.  Tile 0 goes first; tile 1 follows in the same j.
        if (NB == 2 && ntile == 2) {
          const bool go = t == 0 ? (jg == 0 || mbar_wait_warp(smem_u32(&bar_turn[1]), (uint32_t)(jg - 1) & 1u, abortp, g.wait_limit))
                                 : mbar_wait_warp(smem_u32(&bar_turn[0]), (uint32_t)jg & 1u, abortp, g.wait_limit);
          if (!go) { ok = false; break; }
        }
        float s4[4] = {0.f, 0.f, 0.f, 0.f};
        const float nm = -m_new;
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4) {                     // 32 scores at a time
          if constexpr (TWO_PASS) {
            tmem_ld_32x32(s_addr + c4 * 32, xr);
            tmem_wait_ld();
            if (valid < 128) {
#pragma unroll
              for (int q = 0; q < 32; ++q)
                if (c4 * 32 + q >= valid) xr[q] = __float_as_uint(gone);
            }
          }
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {                   // 16-byte chunks of 8 probabilities
            const int c = c4 * 4 + cc;
            float p[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              p[e] = ex2_approx(fmaf(__uint_as_float(xr[(TWO_PASS ? cc * 8 : c * 8) + e]), scale, nm));
              s4[e & 3] += p[e];
            }
            st_shared_v4(pb + (uint32_t)(c >> 3) * 16384 + ((((uint32_t)c & 7u) ^ sw) << 4),
                         pack_half2(p[0], p[1]), pack_half2(p[2], p[3]), pack_half2(p[4], p[5]), pack_half2(p[6], p[7]));
          }
        }
        if (TWO_PASS) {
          tc_fence_before();
          warp_arrive(smem_u32(&bar_s_empty[t]), lane);
        }
        fence_proxy_async_smem();                            // generic-proxy writes -> visible to the MMA
        warp_arrive(smem_u32(&bar_p_full[t][pbuf]), lane);
        if (NB == 2 && ntile == 2) warp_arrive(smem_u32(&bar_turn[t]), lane);
        l = l * corr_new + ((s4[0] + s4[1]) + (s4[2] + s4[3]));
        m = m_new;
        // PV(j-1) was issued a whole iteration ago: taking it out here (rather than before the exponentials)
        // keeps the tensor core's latency off this warpgroup's critical path
        if (j > 0 && !add_pv(jg - 1)) { ok = false; break; }
        corr = corr_new;
      }
      if (ok && T > 0) ok = add_pv(jg0 + T - 1);
      const int row = (qp * 2 + t) * 128 + r;
      if (ok && row < g.s1) {
        const float inv = 1.f / l;
        __half* dst = g.out + ib * g.o_b + ih * g.o_h + (long long)row * g.o_s;
#pragma unroll
        for (int c = 0; c < DP / 8; ++c) {
          if (c * 8 < g.d) {                                 // d is a multiple of 8
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
    }
  }

  tc_fence_before();
  __syncthreads();
  teardown(abort_flag, g.status);
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
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
  const int64_t q_pairs = (s1 + 255) / 256, items = q_pairs * H * B;
  if (items > 0x7fffffffLL) return B200_ERR_LIMIT;
  // One CTA per SM walks the items when every item has both of its query tiles (the barriers' arrival counts are set
  // once per CTA); otherwise one CTA per item.
  const bool uniform = s1 % 256 == 0 || s1 % 256 > 128;
  const int64_t ctas = (uniform && items > ds->sm_count) ? ds->sm_count : items;

  alignas(64) CUtensorMap mq, mk, mv;
  int rc;
  if ((rc = encode_bhsd(&mq, q, d, s1, H, B, qs[2], qs[1], qs[0], 128))) return rc;
  if ((rc = encode_bhsd(&mk, k, d, s2, H, B, ks[3], ks[1], ks[0], 128))) return rc;
  if ((rc = encode_bhsd(&mv, v, d, s2, H, B, vs[2], vs[1], vs[0], 128))) return rc;
  AttnArgs g;
  g.s1 = (int)s1; g.s2 = (int)s2; g.d = (int)d;
  g.heads = (int)H; g.q_pairs = (int)q_pairs; g.kv_tiles = (int)((s2 + 127) / 128);
  g.items = items;
  g.scale_log2 = (float)(alpha * 1.4426950408889634);
  if (g.scale_log2 == 0.f) g.scale_log2 = 1e-30f;           // keeps (masked score = -inf) * scale = -inf
  g.out = (__half*)out; g.o_b = os[0]; g.o_h = os[1]; g.o_s = os[2];
  g.lse = lse;
  g.wait_limit = 400000000LL + (long long)g.kv_tiles * 400000LL;
  g.status = ds->status;
  return d <= 64 ? launch_fwd<64>(mq, mk, mv, g, ctas, stream) : launch_fwd<128>(mq, mk, mv, g, ctas, stream);
}

}  // namespace b200
