// Backward of the fused attention  O = softmax(alpha * Q K^T) V  for f16 tensors.
//
// With P = softmax(alpha * S), S = Q K^T, and Dl_i = sum_d dO_id * O_id:
//     dV = P^T dO          dP = dO V^T          dS = P o (dP - Dl)          dQ = alpha dS K          dK = alpha dS^T Q
// which is what the tape of dfdx's MultiHeadAttention runs op by op (backward of matmul, softmax, scalar mul and
// matmul again: dfdx/src/nn/layers/multi_head_attention.rs:136-141) with five passes over score-sized tensors.
// Here P is recomputed from the forward's log-sum-exp and no score-sized tensor touches HBM.
//
// Three launches:
//   attention_bwd_prep_kernel     aux[b, h, i] = (lse_i * log2(e), Dl_i) as float2, padded per (b, h) to a multiple
//                                 of 64 rows with (+inf, 0): a padded row then has P = exp2(x - inf) = 0.
//   attention_bwd_kernel<DP, 0>   dQ: one CTA per (b, h, 128 queries), streams key / value tiles of 64 rows.
//   attention_bwd_kernel<DP, 1>   dK, dV: one CTA per (b, h, 128 keys), streams query / dO tiles of 64 rows.
// Each is launched as at most one CTA per SM that walks its work items (item = blockIdx.x, + gridDim.x, ...): every
// barrier keeps counting across items, so the next item's loads and first S' / dP' run under the current item's last
// steps, and (DP = 64) its accumulators are written into the other half of tensor memory while the row threads still
// turn the finished ones into gradients.
// Both use one template: "rows" (128, resident in shared memory: R1, R2) against "columns" (64 per step, TMA
// ring: C1, C2):
//   mode 0: R1 = Q, R2 = dO, C1 = K_j, C2 = V_j      S' = R1 C1^T = S,    dP' = R2 C2^T = dP
//   mode 1: R1 = K, R2 = V,  C1 = Q_i, C2 = dO_i     S' = R1 C1^T = S^T,  dP' = R2 C2^T = dP^T
// Warps 0..15 = four threads per row (each takes a quarter of a step's 64 columns; no reduction across a row is needed
// in the backward pass): read S' and dP' from TMEM, P' = exp2(s * scale - L), dS' = P' (dP' - Dl), write dS' (and P') as
// f16 MMA operands into shared memory.  Warp 16 = TMA producer, warps 17, 18, 19 = MMA issuers (S', the accumulators,
// dP'; S' and dP' into double-buffered TMEM; accumulators acc1 += dS' C1 and, mode 1, acc2 += P' C2 stay in TMEM over
// an item's loop).
// The same shared-memory image of a column tile serves as the K-major B operand of S' / dP' and as the MN-major
// B operand of the accumulator MMAs.  Every wait is bounded (abort flag, device status word).
#include "attention_common.cuh"

namespace b200 {

namespace {

using namespace tcx;
using namespace attn;

struct BwdArgs {
  int n_rows, n_cols, d;            // extent of the row / column axis (mode 0: s1, s2; mode 1: s2, s1)
  int heads, row_tiles, col_tiles;
  long long items;                  // batch * heads * row_tiles; CTA c takes items c, c + gridDim.x, ...
  int aux_pad;                      // rows of aux per (b, h)
  float scale_log2, alpha;
  const float2* aux;
  __half* out1; long long o1_b, o1_h, o1_r;   // mode 0: dQ.  mode 1: dK        (unit stride along d)
  __half* out2; long long o2_b, o2_h, o2_r;   // mode 1: dV
  int accumulate;                   // 1: add to what the gradient buffers hold (dfdx's backward ops accumulate)
  long long wait_limit;
  int* status;
};

template <int DP, int MODE>
struct BwdCfg {
  static constexpr int ST = DP == 64 ? 4 : 2;              // ring stages of (C1, C2)
  static constexpr int R_BYTES = 128 * DP * 2;             // one resident row operand
  static constexpr int C_BYTES = 64 * DP * 2;              // one streamed column operand
  static constexpr int A_BYTES = 128 * 64 * 2;             // one dS' (or P') tile
  static constexpr int OFF_C = 2 * R_BYTES;
  static constexpr int OFF_A = OFF_C + ST * 2 * C_BYTES;   // dS'[0], dS'[1], then (mode 1) P'[0], P'[1]
  static constexpr int SMEM_BYTES = OFF_A + (MODE == 1 ? 4 : 2) * A_BYTES + 1024;
  static constexpr int ROW_WARPS = 16;                     // four threads per row: the row threads' chains of waits, tensor-memory
                                                           // loads and exponentials are latency-bound, so warps per scheduler count
  static constexpr int W_TMA = ROW_WARPS, W_S = ROW_WARPS + 1, W_ACC = ROW_WARPS + 2, W_DP = ROW_WARPS + 3;
  static constexpr int THREADS = (ROW_WARPS + 4) * 32;     // row warps, TMA warp, three MMA issuers
  static constexpr int TMEM_COLS = 512;
  static constexpr int NACC = DP == 64 ? 2 : 1;            // accumulator sets (acc1, acc2) in tensor memory
  static constexpr uint32_t TM_S = 0, TM_DP = 128, TM_ACC1 = 256, TM_ACC2 = 256 + DP, TM_ACC_STRIDE = 2 * DP;
};

// aux[(b*H + h) * pad + i] = (lse * log2 e, sum_d dO * O) for i < s1, (+inf, 0) for the padding rows.
// Eight lanes share a row (16 bytes of O and of dO each per step), so a warp reads four rows as whole 128-byte lines.
__global__ void __launch_bounds__(256) attention_bwd_prep_kernel(const __half* __restrict__ o, long long o_b, long long o_h,
                                                                 long long o_s, const __half* __restrict__ go, long long g_b,
                                                                 long long g_h, long long g_s, const float* __restrict__ lse,
                                                                 float2* __restrict__ aux, int heads, int s1, int pad, int d,
                                                                 long long total) {
  const long long idx = ((long long)blockIdx.x * 256 + threadIdx.x) >> 3;   // row of aux
  const int sub = threadIdx.x & 7;
  const bool live = idx < total;                             // whole 8-lane groups are live or not
  const int i = live ? (int)(idx % pad) : 0;
  const long long bh = live ? idx / pad : 0;
  float acc = 0.f;
  if (live && i < s1) {
    const int h = (int)(bh % heads);
    const long long b = bh / heads;
    const __half* po = o + b * o_b + h * o_h + (long long)i * o_s;
    const __half* pg = go + b * g_b + h * g_h + (long long)i * g_s;
    for (int c = sub * 8; c < d; c += 64) {                  // d is a multiple of 8, rows are 16-byte aligned
      const uint4 a = *reinterpret_cast<const uint4*>(po + c);
      const uint4 g = *reinterpret_cast<const uint4*>(pg + c);
      const __half2* ha = reinterpret_cast<const __half2*>(&a);
      const __half2* hg = reinterpret_cast<const __half2*>(&g);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 fa = __half22float2(ha[e]), fg = __half22float2(hg[e]);
        acc = fmaf(fa.x, fg.x, acc);
        acc = fmaf(fa.y, fg.y, acc);
      }
    }
  }
  acc += __shfl_xor_sync(0xffffffffu, acc, 1);
  acc += __shfl_xor_sync(0xffffffffu, acc, 2);
  acc += __shfl_xor_sync(0xffffffffu, acc, 4);
  if (live && sub == 0)
    aux[idx] = i < s1 ? make_float2(lse[bh * s1 + i] * 1.4426950408889634f, acc) : make_float2(INFINITY, 0.f);
}

template <int DP, int MODE>
__global__ void __launch_bounds__(BwdCfg<DP, MODE>::THREADS, 1)
attention_bwd_kernel(const __grid_constant__ CUtensorMap tma_r1, const __grid_constant__ CUtensorMap tma_r2,
                     const __grid_constant__ CUtensorMap tma_c1, const __grid_constant__ CUtensorMap tma_c2,
                     const BwdArgs g) {
  using C = BwdCfg<DP, MODE>;
  constexpr int ST = C::ST;
  constexpr int DCH = DP / 64;

  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t bar_r, bar_r_empty, bar_acc_full[C::NACC], bar_acc_empty[C::NACC];
  __shared__ __align__(8) uint64_t bar_c_full[ST], bar_c_empty[ST];
  __shared__ __align__(8) uint64_t bar_sdp_full[2], bar_sdp_empty[2], bar_a_full[2], bar_a_empty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abortp = &abort_flag;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar_r), 1);
    mbar_init(smem_u32(&bar_r_empty), 2);                   // the S' and the dP' issuer
    for (int a = 0; a < C::NACC; ++a) {
      mbar_init(smem_u32(&bar_acc_full[a]), 1);
      mbar_init(smem_u32(&bar_acc_empty[a]), C::ROW_WARPS); // one arrival per row warp
    }
    for (int s = 0; s < ST; ++s) {
      mbar_init(smem_u32(&bar_c_full[s]), 1);
      mbar_init(smem_u32(&bar_c_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bar_sdp_full[b]), 2);             // S' and dP' are committed by different issuers
      mbar_init(smem_u32(&bar_sdp_empty[b]), C::ROW_WARPS); // one arrival per row warp
      mbar_init(smem_u32(&bar_a_full[b]), C::ROW_WARPS);
      mbar_init(smem_u32(&bar_a_empty[b]), 1);
    }
    abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == C::W_S) {
    tmem_alloc(smem_u32(&tmem_slot), C::TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == C::W_TMA && lane == 0) {
    tma_prefetch_desc(&tma_r1);
    tma_prefetch_desc(&tma_r2);
    tma_prefetch_desc(&tma_c1);
    tma_prefetch_desc(&tma_c2);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;

  constexpr int NACC = C::NACC;
  const int T = g.col_tiles;
  const int ksteps = (g.d + 15) / 16;                       // k-steps of S' / dP' that hold data

  if (warp == C::W_TMA) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const uint32_t br = smem_u32(&bar_r);
      bool ok = true;
      int it = 0;
      for (long long item = blockIdx.x; ok && item < g.items; item += gridDim.x, ++it) {
      const int rt = (int)(item % g.row_tiles);
      const long long bh = item / g.row_tiles;
      const int ih = (int)(bh % g.heads), ib = (int)(bh / g.heads);
      // the row operands are free once the previous item's last S' and dP' have been computed
      if (it > 0 && !mbar_wait(smem_u32(&bar_r_empty), (uint32_t)(it - 1) & 1u, abortp, g.wait_limit)) break;
      mbar_expect_tx(br, 2 * C::R_BYTES);
      for (int c = 0; c < DCH; ++c) {
        tma_load_4d(smem_base + c * 16384, &tma_r1, br, c * 64, rt * 128, ih, ib);
        tma_load_4d(smem_base + C::R_BYTES + c * 16384, &tma_r2, br, c * 64, rt * 128, ih, ib);
      }
      for (int j = 0; j < T; ++j) {
        const int jg = it * T + j;                             // column tiles this CTA has streamed so far
        const int s = jg % ST;
        if (!mbar_wait(smem_u32(&bar_c_empty[s]), (((uint32_t)(jg / ST)) & 1u) ^ 1u, abortp, g.wait_limit)) { ok = false; break; }
        const uint32_t f = smem_u32(&bar_c_full[s]);
        mbar_expect_tx(f, 2 * C::C_BYTES);
        const uint32_t dst = smem_base + C::OFF_C + s * 2 * C::C_BYTES;
        for (int c = 0; c < DCH; ++c) {
          tma_load_4d(dst + c * 8192, &tma_c1, f, c * 64, j * 64, ih, ib);
          tma_load_4d(dst + C::C_BYTES + c * 8192, &tma_c2, f, c * 64, j * 64, ih, ib);
        }
      }
      }
    }
    __syncwarp();
  } else if (warp > C::W_TMA) {
    // ------------------------------------------------------------------ MMA issuers
    // one warp issues S', one dP', one the accumulator MMAs: three short instruction streams instead of one
    // long one (each wait, MMA and commit of the issuing thread is a serial, long-latency step).
    if (lane == 0) {
      const uint32_t idesc_s = (1u << 4) | ((uint32_t)(64 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);             // N = 64
      const uint32_t idesc_acc = (1u << 4) | (1u << 16) | ((uint32_t)(DP >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);  // B MN-major
      const uint64_t dk = make_smem_desc(smem_base, 16, 1024, 2);              // K-major operands
      const uint64_t dm = make_smem_desc(smem_base, 8192, 1024, 2);            // MN-major column tile (d-chunk stride 8192)
      const uint32_t hi_k = (uint32_t)(dk >> 32), hi_m = (uint32_t)(dm >> 32);
      const uint32_t lo_k = (uint32_t)dk, lo_m = (uint32_t)dm;
      if (warp == C::W_S || warp == C::W_DP) {
        const bool second = warp == C::W_DP;                      // false: S' = R1 C1^T, true: dP' = R2 C2^T
        const uint32_t r_off = second ? (uint32_t)C::R_BYTES : 0u, c_off = second ? (uint32_t)C::C_BYTES : 0u;
        const uint32_t d_off = second ? C::TM_DP : C::TM_S;
        bool ok = true;
        int it = 0;
        for (long long item = blockIdx.x; ok && item < g.items; item += gridDim.x, ++it) {
        ok = mbar_wait(smem_u32(&bar_r), (uint32_t)it & 1u, abortp, g.wait_limit);
        // (j): needs column tile j and the row threads to have read what buffer j & 1 held two steps before
        for (int j = 0; ok && j < T; ++j) {
          const int jg = it * T + j;
          const int s = jg % ST, b = jg & 1;
          if (!mbar_wait(smem_u32(&bar_c_full[s]), ((uint32_t)(jg / ST)) & 1u, abortp, g.wait_limit)) { ok = false; break; }
          if (jg >= 2 && !mbar_wait(smem_u32(&bar_sdp_empty[b]), (((uint32_t)(jg >> 1)) & 1u) ^ 1u, abortp, g.wait_limit)) { ok = false; break; }
          tc_fence_after();
          const uint32_t c_lo = lo_k + (uint32_t)((C::OFF_C + s * 2 * C::C_BYTES) >> 4);
          for (int ks = 0; ks < ksteps; ++ks) {
            const uint32_t ro = (uint32_t)((r_off + (ks >> 2) * 16384 + (ks & 3) * 32) >> 4);
            const uint32_t co = (uint32_t)((c_off + (ks >> 2) * 8192 + (ks & 3) * 32) >> 4);
            umma_lohi<2>(tmem_base + d_off + b * 64, lo_k + ro, hi_k, c_lo + co, hi_k, idesc_s, ks > 0 ? 1u : 0u);
          }
          umma_commit(smem_u32(&bar_sdp_full[b]));
        }
        if (ok) umma_commit(smem_u32(&bar_r_empty));         // this issuer's MMAs of the item have read the row operands
        }
      } else {
        bool ok = true;
        int it = 0;
        for (long long item = blockIdx.x; ok && item < g.items; item += gridDim.x, ++it) {
        const int ab = it % NACC;                            // accumulator set of this item
        const uint32_t acc_off = (uint32_t)ab * C::TM_ACC_STRIDE;
        // the set is free once the row threads have turned the item that last used it into gradients
        if (it >= NACC && !mbar_wait(smem_u32(&bar_acc_empty[ab]), (((uint32_t)(it / NACC)) & 1u) ^ 1u, abortp, g.wait_limit)) { ok = false; break; }
        for (int j = 0; j < T; ++j) {
          const int jg = it * T + j;
          const int s = jg % ST, b = jg & 1;
          if (!mbar_wait(smem_u32(&bar_c_full[s]), ((uint32_t)(jg / ST)) & 1u, abortp, g.wait_limit)) { ok = false; break; }
          if (!mbar_wait(smem_u32(&bar_a_full[b]), ((uint32_t)(jg >> 1)) & 1u, abortp, g.wait_limit)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_lo = lo_k + (uint32_t)((C::OFF_A + b * C::A_BYTES) >> 4);
          const uint32_t c_lo = lo_m + (uint32_t)((C::OFF_C + s * 2 * C::C_BYTES) >> 4);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)                      // 64 columns of S', 16 per MMA
            umma_lohi<2>(tmem_base + C::TM_ACC1 + acc_off, a_lo + (uint32_t)(ks * 32 >> 4), hi_k, c_lo + (uint32_t)(ks * 2048 >> 4), hi_m,
                         idesc_acc, (j > 0 || ks > 0) ? 1u : 0u);
          if (MODE == 1) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
              umma_lohi<2>(tmem_base + C::TM_ACC2 + acc_off, a_lo + (uint32_t)((2 * C::A_BYTES + ks * 32) >> 4), hi_k,
                           c_lo + (uint32_t)((C::C_BYTES + ks * 2048) >> 4), hi_m, idesc_acc, (j > 0 || ks > 0) ? 1u : 0u);
          }
          umma_commit(smem_u32(&bar_a_empty[b]));
          umma_commit(smem_u32(&bar_c_empty[s]));
        }
        if (ok) umma_commit(smem_u32(&bar_acc_full[ab]));
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ row threads (warps 0..15)
    // warps w, w + 4, w + 8, w + 12 share the rows of TMEM lane quadrant w & 3 and split each step's 64 columns in
    // quarters
    constexpr int CW = 64 / (C::ROW_WARPS / 4);              // columns of a step per thread: 16
    const int quad = warp & 3, part = warp >> 2;
    const int r = quad * 32 + lane;                          // row inside the tile = TMEM lane
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    const uint32_t a_row = (uint32_t)(r >> 3) * 1024 + (uint32_t)(r & 7) * 128;
    const uint32_t sw = (uint32_t)(r & 7);
    const float scale = g.scale_log2;
    bool ok = true;
    int it = 0;
    for (long long item = blockIdx.x; ok && item < g.items; item += gridDim.x, ++it) {
    const int rt = (int)(item % g.row_tiles);
    const long long bh = item / g.row_tiles;
    const int ih = (int)(bh % g.heads), ib = (int)(bh / g.heads);
    const int row = rt * 128 + r;
    const float2* aux = g.aux + bh * g.aux_pad;
    float row_l = 0.f, row_d = 0.f;
    if (MODE == 0) {                                         // per-row constants; rows beyond the extent are never stored
      const float2 a = aux[row < g.aux_pad ? row : g.aux_pad - 1];
      row_l = a.x; row_d = a.y;
    }
    for (int j = 0; j < T; ++j) {
      const int jg = it * T + j;
      const int b = jg & 1;
      const uint32_t ph = ((uint32_t)(jg >> 1)) & 1u;
      // mode 1: per-column constants (padded to 64), requested before the wait so that they are there after it
      float4 cl[CW / 2];
      if (MODE == 1) {
        const float2* caux = aux + j * 64 + part * CW;
#pragma unroll
        for (int e = 0; e < CW / 2; ++e) cl[e] = __ldg(reinterpret_cast<const float4*>(caux + 2 * e));
      }
      if (!mbar_wait_warp(smem_u32(&bar_sdp_full[b]), ph, abortp, g.wait_limit)) { ok = false; break; }
      tc_fence_after();
      uint32_t sv[CW], dv[CW];
      tmem_ld_32x16(lane_addr + C::TM_S + b * 64 + part * CW, sv);
      tmem_ld_32x16(lane_addr + C::TM_DP + b * 64 + part * CW, dv);
      tmem_wait_ld();
      tc_fence_before();
      warp_arrive(smem_u32(&bar_sdp_empty[b]), lane);
      // the operand buffers of this parity are free once the accumulator MMAs of step j-2 have read them
      if (jg >= 2 && !mbar_wait_warp(smem_u32(&bar_a_empty[b]), ph ^ 1u, abortp, g.wait_limit)) { ok = false; break; }
      const uint32_t ds_dst = smem_base + C::OFF_A + b * C::A_BYTES + a_row;
      const int valid = g.n_cols - j * 64 - part * CW;       // columns of this thread's part that exist
#pragma unroll
      for (int c = 0; c < CW / 8; ++c) {                     // 16-byte chunks of 8 columns
        float pv[8], dsv[8];
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          float l0, d0, l1, d1;
          if (MODE == 1) {
            const float4 a = cl[(c * 8 + e) / 2];
            l0 = a.x; d0 = a.y; l1 = a.z; d1 = a.w;
          } else {
            l0 = l1 = row_l; d0 = d1 = row_d;
          }
          float p0 = ex2_approx(fmaf(__uint_as_float(sv[c * 8 + e]), scale, -l0));
          float p1 = ex2_approx(fmaf(__uint_as_float(sv[c * 8 + e + 1]), scale, -l1));
          if (MODE == 0) {                                   // mode 1 masks through the (+inf, 0) padding of aux
            if (c * 8 + e >= valid) p0 = 0.f;
            if (c * 8 + e + 1 >= valid) p1 = 0.f;
          }
          pv[e] = p0; pv[e + 1] = p1;
          dsv[e] = p0 * (__uint_as_float(dv[c * 8 + e]) - d0);
          dsv[e + 1] = p1 * (__uint_as_float(dv[c * 8 + e + 1]) - d1);
        }
        const uint32_t off = (((uint32_t)(part * (CW / 8) + c) ^ sw) << 4);
        st_shared_v4(ds_dst + off, pack_half2(dsv[0], dsv[1]), pack_half2(dsv[2], dsv[3]), pack_half2(dsv[4], dsv[5]),
                     pack_half2(dsv[6], dsv[7]));
        if (MODE == 1)
          st_shared_v4(ds_dst + 2 * C::A_BYTES + off, pack_half2(pv[0], pv[1]), pack_half2(pv[2], pv[3]),
                       pack_half2(pv[4], pv[5]), pack_half2(pv[6], pv[7]));
      }
      fence_proxy_async_smem();
      warp_arrive(smem_u32(&bar_a_full[b]), lane);
    }
    // ---- accumulators -> gradients: each of a row's four threads stores a quarter of the columns
    const int ab = it % NACC;
    if (ok) ok = mbar_wait_warp(smem_u32(&bar_acc_full[ab]), ((uint32_t)(it / NACC)) & 1u, abortp, g.wait_limit);
    if (ok) {
      tc_fence_after();
      const bool store = row < g.n_rows;                     // only the global accesses are per-lane
      constexpr int CP = DP / (C::ROW_WARPS / 4);            // columns per thread: 16 (DP = 64) or 32
#pragma unroll
      for (int which = 0; which < (MODE == 1 ? 2 : 1); ++which) {
        __half* dst = which == 0 ? g.out1 + ib * g.o1_b + ih * g.o1_h + (long long)row * g.o1_r
                                 : g.out2 + ib * g.o2_b + ih * g.o2_h + (long long)row * g.o2_r;
        const float mul = which == 0 ? g.alpha : 1.f;         // dQ and dK carry the score scale, dV does not
        const uint32_t tm = (which == 0 ? C::TM_ACC1 : C::TM_ACC2) + (uint32_t)ab * C::TM_ACC_STRIDE;
        const int c0 = part * CP;
        uint32_t v[CP];
        if constexpr (CP == 16) tmem_ld_32x16(lane_addr + tm + c0, v);
        else tmem_ld_32x32(lane_addr + tm + c0, v);
        // what the gradient buffer holds: all 16-byte pieces are requested before any is used, so the row-strided
        // (uncoalesced) reads overlap instead of costing one memory round trip each
        uint4 old[CP / 8];
        if (g.accumulate) {
#pragma unroll
          for (int q8 = 0; q8 < CP / 8; ++q8)
            old[q8] = (store && c0 + q8 * 8 < g.d) ? *reinterpret_cast<const uint4*>(dst + c0 + q8 * 8)
                                                   : make_uint4(0u, 0u, 0u, 0u);
        }
        tmem_wait_ld();
#pragma unroll
        for (int q8 = 0; q8 < CP / 8; ++q8) {
          const int col = c0 + q8 * 8;
          if (store && col < g.d) {                          // d is a multiple of 8
            float f[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(v[q8 * 8 + e]) * mul;
            if (g.accumulate) {
              const __half2* ho = reinterpret_cast<const __half2*>(&old[q8]);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 fo = __half22float2(ho[e]);
                f[2 * e] += fo.x; f[2 * e + 1] += fo.y;
              }
            }
            uint4 o;
            o.x = pack_half2(f[0], f[1]); o.y = pack_half2(f[2], f[3]);
            o.z = pack_half2(f[4], f[5]); o.w = pack_half2(f[6], f[7]);
            *reinterpret_cast<uint4*>(dst + col) = o;
          }
        }
      }
      tc_fence_before();
      warp_arrive(smem_u32(&bar_acc_empty[ab]), lane);       // this warp has read its part of the accumulator set
    }
    }
  }

  tc_fence_before();
  __syncthreads();
  teardown(abort_flag, g.status);
  if (warp == C::W_S) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

template <int DP, int MODE>
int launch_bwd(const CUtensorMap& r1, const CUtensorMap& r2, const CUtensorMap& c1, const CUtensorMap& c2,
               const BwdArgs& g, int64_t ctas, cudaStream_t stream) {
  using C = BwdCfg<DP, MODE>;
  attention_bwd_kernel<DP, MODE><<<(unsigned)ctas, C::THREADS, C::SMEM_BYTES, stream>>>(r1, r2, c1, c2, g);
  count_launch(true);
  return note_cuda_error(cudaGetLastError(), "attention backward launch");
}

template <int DP, int MODE>
int set_attr_bwd() {
  return note_cuda_error(cudaFuncSetAttribute(attention_bwd_kernel<DP, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              BwdCfg<DP, MODE>::SMEM_BYTES), "cudaFuncSetAttribute(attention backward)");
}

}  // namespace

int attention_bwd_setup_device() {
  int rc;
  if ((rc = set_attr_bwd<64, 0>())) return rc;
  if ((rc = set_attr_bwd<64, 1>())) return rc;
  if ((rc = set_attr_bwd<128, 0>())) return rc;
  return set_attr_bwd<128, 1>();
}

size_t attention_backward_workspace_bytes(int64_t B, int64_t H, int64_t s1) {
  return (size_t)B * (size_t)H * (size_t)((s1 + 63) / 64 * 64) * sizeof(float2);
}

// Layouts as in attention_forward; go / gq like out / q, gk like k ((B,H,D,S2) view), gv like v.
int attention_backward(int dtype, int64_t B, int64_t H, int64_t s1, int64_t s2, int64_t d, const void* q,
                       const int64_t qs[4], const void* k, const int64_t ks[4], const void* v, const int64_t vs[4],
                       double alpha, const void* out, const int64_t os[4], const float* lse, const void* go,
                       const int64_t gs[4], void* gq, const int64_t gqs[4], void* gk, const int64_t gks[4], void* gv,
                       const int64_t gvs[4], int accumulate, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  if (dtype != B200_F16 && dtype != B200_AMP_F16) return B200_ERR_UNSUPPORTED;
  if (B == 0 || H == 0 || (s1 == 0 && s2 == 0) || d == 0) return B200_OK;
  if (s1 == 0 || s2 == 0) return B200_ERR_SHAPE;
  DeviceState* ds = device_state();
  if (!ds || !ds->ready) return note_cuda_error(cudaErrorInitializationError, "b200_init not called on this device");
  if (d % 8 || d > 128) return B200_ERR_UNSUPPORTED;
  if (qs[3] != 1 || ks[2] != 1 || vs[3] != 1 || os[3] != 1 || gs[3] != 1 || gqs[3] != 1 || gks[2] != 1 || gvs[3] != 1)
    return B200_ERR_UNSUPPORTED;
  const int64_t* all[8] = {qs, ks, vs, os, gs, gqs, gks, gvs};
  for (int t = 0; t < 8; ++t) {
    const bool kt = (t == 1 || t == 6);                    // (B, H, D, S2) views: the sequence stride is index 3
    const int64_t seq = (t == 1 || t == 2 || t == 6 || t == 7) ? s2 : s1;
    if (!stride_ok(seq, all[t][kt ? 3 : 2]) || !stride_ok(H, all[t][1]) || !stride_ok(B, all[t][0])) return B200_ERR_UNSUPPORTED;
  }
  if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out | (uintptr_t)go | (uintptr_t)gq | (uintptr_t)gk |
       (uintptr_t)gv | (uintptr_t)workspace) & 15)
    return B200_ERR_UNSUPPORTED;
  if (s1 > 0x7fffff00LL || s2 > 0x7fffff00LL || B * H > 0x7fffffffLL) return B200_ERR_LIMIT;
  if (workspace_bytes < attention_backward_workspace_bytes(B, H, s1)) return B200_ERR_WORKSPACE;
  const int64_t pad = (s1 + 63) / 64 * 64;
  const int64_t q_tiles = (s1 + 127) / 128, k_tiles = (s2 + 127) / 128;
  if (q_tiles * B * H > 0x7fffffffLL || k_tiles * B * H > 0x7fffffffLL) return B200_ERR_LIMIT;

  // 1. aux = (lse * log2 e, rowsum(dO o O))
  {
    const long long total = (long long)B * H * pad;
    attention_bwd_prep_kernel<<<(unsigned)((total * 8 + 255) / 256), 256, 0, stream>>>(
        (const __half*)out, os[0], os[1], os[2], (const __half*)go, gs[0], gs[1], gs[2], lse, (float2*)workspace, (int)H,
        (int)s1, (int)pad, (int)d, total);
    count_launch(false);
    const int rc = note_cuda_error(cudaGetLastError(), "attention backward prep launch");
    if (rc) return rc;
  }
  alignas(64) CUtensorMap mq128, mg128, mk64, mv64, mk128, mv128, mq64, mg64;
  int rc;
  if ((rc = encode_bhsd(&mq128, q, d, s1, H, B, qs[2], qs[1], qs[0], 128))) return rc;
  if ((rc = encode_bhsd(&mg128, go, d, s1, H, B, gs[2], gs[1], gs[0], 128))) return rc;
  if ((rc = encode_bhsd(&mk64, k, d, s2, H, B, ks[3], ks[1], ks[0], 64))) return rc;
  if ((rc = encode_bhsd(&mv64, v, d, s2, H, B, vs[2], vs[1], vs[0], 64))) return rc;
  if ((rc = encode_bhsd(&mk128, k, d, s2, H, B, ks[3], ks[1], ks[0], 128))) return rc;
  if ((rc = encode_bhsd(&mv128, v, d, s2, H, B, vs[2], vs[1], vs[0], 128))) return rc;
  if ((rc = encode_bhsd(&mq64, q, d, s1, H, B, qs[2], qs[1], qs[0], 64))) return rc;
  if ((rc = encode_bhsd(&mg64, go, d, s1, H, B, gs[2], gs[1], gs[0], 64))) return rc;

  BwdArgs g;
  g.d = (int)d; g.heads = (int)H; g.aux_pad = (int)pad;
  g.scale_log2 = (float)(alpha * 1.4426950408889634);
  g.alpha = (float)alpha;
  g.aux = (const float2*)workspace;
  g.accumulate = accumulate ? 1 : 0;
  g.status = ds->status;
  // 2. dQ: rows = queries, columns = keys
  if (gq) {
    g.n_rows = (int)s1; g.n_cols = (int)s2; g.row_tiles = (int)q_tiles; g.col_tiles = (int)((s2 + 63) / 64);
    g.out1 = (__half*)gq; g.o1_b = gqs[0]; g.o1_h = gqs[1]; g.o1_r = gqs[2];
    g.out2 = nullptr; g.o2_b = g.o2_h = g.o2_r = 0;
    g.wait_limit = 400000000LL + (long long)g.col_tiles * 400000LL;
    g.items = q_tiles * H * B;
    rc = d <= 64 ? launch_bwd<64, 0>(mq128, mg128, mk64, mv64, g, g.items < ds->sm_count ? g.items : ds->sm_count, stream)
                 : launch_bwd<128, 0>(mq128, mg128, mk64, mv64, g, g.items < ds->sm_count ? g.items : ds->sm_count, stream);
    if (rc) return rc;
  }
  // 3. dK, dV: rows = keys, columns = queries
  if (gk || gv) {
    if (!gk || !gv) return B200_ERR_NULL;
    g.n_rows = (int)s2; g.n_cols = (int)s1; g.row_tiles = (int)k_tiles; g.col_tiles = (int)(pad / 64);
    g.out1 = (__half*)gk; g.o1_b = gks[0]; g.o1_h = gks[1]; g.o1_r = gks[3];
    g.out2 = (__half*)gv; g.o2_b = gvs[0]; g.o2_h = gvs[1]; g.o2_r = gvs[2];
    g.wait_limit = 400000000LL + (long long)g.col_tiles * 400000LL;
    g.items = k_tiles * H * B;
    rc = d <= 64 ? launch_bwd<64, 1>(mk128, mv128, mq64, mg64, g, g.items < ds->sm_count ? g.items : ds->sm_count, stream)
                 : launch_bwd<128, 1>(mk128, mv128, mq64, mg64, g, g.items < ds->sm_count ? g.items : ds->sm_count, stream);
    if (rc) return rc;
  }
  return B200_OK;
}

}  // namespace b200
