// tcgen05 tensor-core GEMMs for sm_100a: persistent, warp-specialised, TMA-fed.
//
//   C[b][128-row tile, BN-col tile] (beta) += sum_r sum_k A[b,r] * B[b,r]
//
// Two kernels share the scaffolding (TMA producer warp -> shared-memory ring -> single-thread MMA
// issuer -> TMEM accumulators -> epilogue warps; one CTA per SM, tiles assigned round-robin):
//
// gemm_f16_kernel   f16 operands, kind::f16, f32 accumulation in TMEM.  6 warps.  128B-swizzled stages
//                   (BK = 64).  The accumulator is double-buffered in TMEM so the epilogue of tile i
//                   overlaps the main loop of tile i+1.
//
// gemm_tf32x3_kernel  f32 operands as 3xTF32 (kind::tf32).  20 warps in five warpgroups: WG0/WG1 =
//                   epilogue, WG2 = TMA producer warp + MMA warp, WG3/WG4 = operand split.
//                   Each staged f32 x stays in place as the `big` operand (the tensor core reads its top
//                   19 bits) and small = x - trunc_tf32(x) is written beside it; every k-step issues
//                   small*big, big*small, big*big (K = 8).  The tensor core adds into its f32
//                   accumulator with truncation, so the error of one long accumulation grows linearly
//                   with K; therefore K is cut into chunks of 256: each chunk accumulates in one of two
//                   TMEM buffers and the epilogue warpgroups add finished chunks into f32 registers
//                   (round-to-nearest) while the next chunk runs.  setmaxnreg moves registers from the
//                   producer / MMA / split warpgroups to the epilogue warpgroups.  Problems with few
//                   output tiles are cut along K as well (split-K): a work unit is (tile, K slice) and
//                   the slices add their partial results into C with vector atomics.
//
// Operands are read in place from dfdx's strides: K-major rows, or MN-major (the transposed views that
// the backward GEMMs and `permute` produce).  MN-major tiles are brought in as column chunks:
// 64 x f16 under the 128B swizzle, 32 x f32 under the 128B swizzle with 32-byte atoms (the only
// MN-major layout kind::tf32 accepts); K-major f32 tiles use the 64B swizzle (BK = 16).
//
// Every wait on an mbarrier is bounded: on expiry the CTA raises an abort flag in shared memory, all
// roles drain, TMEM is freed, the kernel writes B200_ERR_DEVICE_TIMEOUT to the device status word and
// returns normally.
#include "tc_device.cuh"
#include <atomic>
#include <mutex>

namespace b200 {

int pair_tile_m();
int pair_tile_n();
int pair_block_k(int esize);
int pair_chunk(int esize);
int pair_setup_device();
int launch_pair(int esize, const CUtensorMap& ma, const CUtensorMap& mb, const tcx::TcArgs& g, int sm_count,
                cudaStream_t stream);

namespace {

using namespace tcx;

// ---------------------------------------------------------------------------------------------
// f16 kernel
// ---------------------------------------------------------------------------------------------
template <int BN>
__global__ void __launch_bounds__(CfgH<BN>::THREADS, 1)
gemm_f16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                const __grid_constant__ CUtensorMap tma_c, const TcArgs g) {
  using C = CfgH<BN>;
  constexpr int STAGES = C::STAGES;
  constexpr int PRODUCER_WARP = 8, MMA_WARP = 9;       // warps 0..7: epilogue

  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t bar_full[STAGES];
  __shared__ __align__(8) uint64_t bar_empty[STAGES];
  __shared__ __align__(8) uint64_t bar_tfull[2];
  __shared__ __align__(8) uint64_t bar_tempty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ __align__(16) float bias_s[2][128];     // per epilogue group: the column bias of its part of the tile

  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abortp = &abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bar_tfull[b]), 1);
      mbar_init(smem_u32(&bar_tempty[b]), 256);
    }
    abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == MMA_WARP) {
    tmem_alloc(smem_u32(&tmem_slot), C::TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == PRODUCER_WARP && lane == 0) {
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  const int total_kb = g.red * g.k_blocks;

  if (warp == PRODUCER_WARP) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (long long unit = blockIdx.x; ok && unit < g.total_units; unit += gridDim.x) {
        const Unit un = decode_unit(g, unit, total_kb);
        const TileCoord t = decode_tile(g, un.tile);
        for (int i = un.kb_lo; i < un.kb_hi; ++i, ++it) {
          const int r = i / g.k_blocks, kb = i - r * g.k_blocks;
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, abortp, g.wait_limit)) { ok = false; break; }
          const uint32_t full = smem_u32(&bar_full[s]);
          mbar_expect_tx(full, C::STAGE_BYTES);
          const uint32_t a_dst = smem_base + s * C::STAGE_BYTES;
          load_operand<BM, C::BK, C::CH, C::MN_LBO>(a_dst, &tma_a, full, g.a_ld, t.mt * BM, kb * C::BK,
                                                     g.a_x1 * t.ib1 + g.a_xr * r, g.a_y0 * t.ib0);
          load_operand<BN, C::BK, C::CH, C::MN_LBO>(a_dst + C::A_BYTES, &tma_b, full, g.b_ld, t.nt * BN, kb * C::BK,
                                                     g.b_x1 * t.ib1 + g.b_xr * r, g.b_y0 * t.ib0);
        }
      }
    }
    __syncwarp();
  } else if (warp == MMA_WARP) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // instruction descriptor: D = f32, A = B = f16, majors, N >> 3, M >> 4
      const uint32_t idesc = (1u << 4) | ((uint32_t)(g.a_mn ? 1 : 0) << 15) | ((uint32_t)(g.b_mn ? 1 : 0) << 16) |
                             ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      const uint32_t a_lbo = g.a_mn ? C::MN_LBO : 16u, b_lbo = g.b_mn ? C::MN_LBO : 16u;
      const uint32_t a_kadv = g.a_mn ? C::MN_KADV : C::K_KADV, b_kadv = g.b_mn ? C::MN_KADV : C::K_KADV;
      // descriptor words of stage 0 (see umma_lohi): per stage and per k-step only the low word moves
      const uint64_t da0 = make_smem_desc(smem_base, a_lbo, C::SBO, C::LAYOUT);
      const uint64_t db0 = make_smem_desc(smem_base + C::A_BYTES, b_lbo, C::SBO, C::LAYOUT);
      const uint32_t a_hi = (uint32_t)(da0 >> 32), b_hi = (uint32_t)(db0 >> 32);
      const uint32_t a_lo0 = (uint32_t)da0, b_lo0 = (uint32_t)db0;
      const uint32_t a_k16 = a_kadv >> 4, b_k16 = b_kadv >> 4;
      constexpr uint32_t STAGE16 = C::STAGE_BYTES >> 4;
      uint32_t ring_s = 0, ring_ph = 0, tcount = 0;        // stage ring position and its phase bit
      bool ok = true;
      for (long long unit = blockIdx.x; ok && unit < g.total_units; unit += gridDim.x, ++tcount) {
        const Unit un = decode_unit(g, unit, total_kb);
        const uint32_t buf = tcount & 1u, tph = (tcount >> 1) & 1u;
        if (!mbar_wait(smem_u32(&bar_tempty[buf]), tph ^ 1u, abortp, g.wait_limit)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int i = un.kb_lo; i < un.kb_hi; ++i) {
          const uint32_t s = ring_s, ph = ring_ph;
          if (++ring_s == (uint32_t)STAGES) { ring_s = 0; ring_ph ^= 1u; }
          if (!mbar_wait(smem_u32(&bar_full[s]), ph, abortp, g.wait_limit)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + (uint32_t)s * STAGE16, b_lo = b_lo0 + (uint32_t)s * STAGE16;
#pragma unroll
          for (int ks = 0; ks < C::KSTEPS; ++ks) {
            umma_lohi<2>(d_tmem, a_lo + ks * a_k16, a_hi, b_lo + ks * b_k16, b_hi, idesc, (i > un.kb_lo || ks > 0) ? 1u : 0u);
          }
          umma_commit(smem_u32(&bar_empty[s]));       // stage reusable once these MMAs retire
        }
        if (ok) umma_commit(smem_u32(&bar_tfull[buf]));
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue (warps 0..7)
    // Two groups of four warps (a warp reads the TMEM lanes 32 * (warp % 4) ...): group eg takes every other
    // 64-column (staged) or 32-column (per-thread) piece of the tile, with its own staging buffer and named barrier,
    // so that a short-K tile's epilogue does not outlast the next tile's main loop.
    const int eg = warp >> 2, ew = warp & 3;
    const int bar_id = 1 + eg;
    const bool leader = (threadIdx.x & 127) == 0;
    uint32_t tcount = 0;
    bool ok = true;
    for (long long unit = blockIdx.x; ok && unit < g.total_units; unit += gridDim.x, ++tcount) {
      const Unit un = decode_unit(g, unit, total_kb);
      const TileCoord t = decode_tile(g, un.tile);
      const uint32_t buf = tcount & 1u, tph = (tcount >> 1) & 1u;
      const int row = t.mt * BM + ew * 32 + lane;
      __half* cbase = (__half*)g.c + t.ib0 * g.c_b0 + t.ib1 * g.c_b1;
      // beta = 1 with row stores: the values the row already holds do not depend on the accumulator, so
      // they are fetched before waiting for it, four 32-column chunks ahead of their use.
      constexpr int NCH = BN / 32, MINE = NCH / 2, AHEAD = MINE < 4 ? MINE : 4;   // this group: chunks 2 i + eg
      const bool rmw = g.beta && !g.c_col && row < g.m && g.ksplit == 1 && !g.c_tma;
      const __half* orow = cbase + (long long)row * g.ldc + t.nt * BN;
      uint32_t oldv[AHEAD][16];
      if (rmw) {
#pragma unroll
        for (int pc = 0; pc < AHEAD; ++pc)
          if (t.nt * BN + (2 * pc + eg) * 32 + 32 <= g.n) load_old_f16(orow + (2 * pc + eg) * 32, oldv[pc], g.c_wide);
      }
      // column bias of this group's 64-column pieces (2 i + eg), as f32, fetched before the accumulator is waited for;
      // the group's barriers below order these writes before the reads and the reads before the next tile's writes
      const bool bias_cols = g.fused && g.c_tma && !g.bias_row;
      if (bias_cols) {
        const int j = threadIdx.x & 127, c2j = (j >> 6) * 2 + eg, colj = t.nt * BN + c2j * 64 + (j & 63);
        float bv = 0.f;
        if (g.bias != nullptr && c2j < BN / 64 && colj < g.n) bv = __half2float(__ldg(reinterpret_cast<const __half*>(g.bias) + colj));
        bias_s[eg][j] = bv;
      }
      bool got = mbar_wait(smem_u32(&bar_tfull[buf]), tph, abortp, g.wait_limit);
      // the staged epilogue below synchronises the four epilogue warps with named barriers, which have no
      // time-out: all of them take this tile or none does
      got = g.c_tma ? named_barrier_and(bar_id, 128, got) : __all_sync(0xffffffffu, got);
      if (!got) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(ew * 32) << 16) + buf * BN;
      if (g.c_tma) {
        // Output through shared memory and TMA: per-thread row stores hand the memory system 32 separate
        // 32-byte pieces per instruction (rows are ldc apart), which bounds GEMMs with a short K and a wide
        // output; a staged 128 x 64 group leaves as one bulk tensor store of whole 128-byte lines.
        const int r_in = ew * 32 + lane;
        const uint32_t sw = (uint32_t)(r_in & 7);
#pragma unroll
        for (int c2 = 0; c2 < BN / 64; ++c2) {
          const int col0 = t.nt * BN + c2 * 64;
          if ((c2 & 1) == eg && col0 < g.n) {        // group-uniform
            const uint32_t stage = smem_base + C::OFF_OUT + (uint32_t)eg * C::OUT_BYTES;
            if (leader) bulk_wait_group_read<0>();   // the store that last used this buffer has read it
            named_barrier_sync(bar_id, 128);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint32_t v[32];
              tmem_ld_32x32(taddr + c2 * 64 + h * 32, v);
              tmem_wait_ld();
              float f[32];
#pragma unroll
              for (int q = 0; q < 32; ++q) f[q] = __uint_as_float(v[q]);
              if (bias_cols) {
                fused_epilogue_cols(f, g, &bias_s[eg][(c2 >> 1) * 64 + h * 32]);
              } else if (g.fused && row < g.m) {
                const int valid = (g.n - col0 - h * 32) < 32 ? (g.n - col0 - h * 32) : 32;
                if (valid > 0) fused_epilogue<__half>(f, g, row, col0 + h * 32, valid);
              }
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4) {
                uint32_t w[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const __half2 hh = __floats2half2_rn(f[q4 * 8 + 2 * e], f[q4 * 8 + 2 * e + 1]);
                  w[e] = *reinterpret_cast<const uint32_t*>(&hh);
                }
                st_shared_v4_u32(stage + (uint32_t)r_in * 128u + ((((uint32_t)(h * 4 + q4)) ^ sw) << 4), w[0], w[1], w[2], w[3]);
              }
            }
            fence_proxy_async_smem();
            named_barrier_sync(bar_id, 128);
            if (leader) {
              if (g.c_tma == 2) tma_reduce_add_4d(&tma_c, stage, col0, t.mt * BM, t.ib1, t.ib0);
              else tma_store_4d(&tma_c, stage, col0, t.mt * BM, t.ib1, t.ib0);
              bulk_commit_group();
            }
          }
        }
        tc_fence_before();
        mbar_arrive(smem_u32(&bar_tempty[buf]));
        continue;
      }
#pragma unroll
      for (int ci = 0; ci < MINE; ++ci) {
        const int c = 2 * ci + eg;
        const int col0 = t.nt * BN + c * 32;
        if (col0 < g.n) {                            // warp-uniform
          uint32_t v[32];
          tmem_ld_32x32(taddr + c * 32, v);
          tmem_wait_ld();
          const int valid = (g.n - col0) < 32 ? (g.n - col0) : 32;
          if (row < g.m) {
            float f[32];
#pragma unroll
            for (int q = 0; q < 32; ++q) f[q] = __uint_as_float(v[q]);
            if (g.fused) fused_epilogue<__half>(f, g, row, col0, valid);
            if (g.ksplit > 1) {                      // K slice: partial sums go to the f32 scratch
              add_chunk_atomic(g.split_out + (long long)row * g.split_ld + col0, f, valid);
            } else if (g.c_col) {
              store_chunk_col(cbase + (long long)col0 * g.ldc + row, f, valid, g.ldc, g.beta);
            } else if (rmw && valid == 32) {
              add_old_f16(f, oldv[ci % AHEAD]);
              store_chunk(cbase + (long long)row * g.ldc + col0, f, 32, 0, g.c_wide);
            } else {
              store_chunk(cbase + (long long)row * g.ldc + col0, f, valid, g.beta, g.c_wide);
            }
          }
          if (rmw && ci + AHEAD < MINE && col0 + 2 * AHEAD * 32 + 32 <= g.n)
            load_old_f16(orow + (c + 2 * AHEAD) * 32, oldv[ci % AHEAD], g.c_wide);
        }
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&bar_tempty[buf]));
    }
    if (leader) bulk_wait_group_read<0>();               // shared memory must outlive the last bulk stores' reads
  }

  tc_fence_before();
  __syncthreads();
  teardown(abort_flag, g.status);
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------
// f16 kernel with a 256 x 256 tile per CTA (CfgHB): same roles as gemm_f16_kernel; each k-step issues two MMAs (rows
// 0..127 and 128..255 of the A tile against the same B tile) into two accumulators; epilogue warp group eg drains
// accumulator eg.  Row-major outputs through the staged TMA store / reduce-add; K slices (ksplit > 1) add their f32
// partial sums into the device's scratch matrix the same way.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(CfgHB::THREADS, 1)
gemm_f16_big_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                    const __grid_constant__ CUtensorMap tma_c, const TcArgs g) {
  using C = CfgHB;
  constexpr int STAGES = C::STAGES, BN = C::BN;
  constexpr int PRODUCER_WARP = 8, MMA_WARP = 9;

  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t bar_full[STAGES];
  __shared__ __align__(8) uint64_t bar_empty[STAGES];
  __shared__ __align__(8) uint64_t bar_tfull;
  __shared__ __align__(8) uint64_t bar_tempty;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ __align__(16) __half bias_s[2][256];    // per epilogue group: the tile's column bias (f16: 3 stages and the
                                                     // staging buffers leave 2 KB of static shared memory)

  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abortp = &abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    mbar_init(smem_u32(&bar_tfull), 1);
    mbar_init(smem_u32(&bar_tempty), 256);
    abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == MMA_WARP) {
    tmem_alloc(smem_u32(&tmem_slot), C::TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == PRODUCER_WARP && lane == 0) {
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  const int total_kb = g.red * g.k_blocks;

  if (warp == PRODUCER_WARP) {
    if (lane == 0) {
      uint32_t ring_s = 0, ring_ph = 0;
      bool ok = true;
      for (long long unit = blockIdx.x; ok && unit < g.total_units; unit += gridDim.x) {
        const Unit un = decode_unit(g, unit, total_kb);
        const TileCoord t = decode_tile(g, un.tile);
        int r = un.kb_lo / g.k_blocks, kx = (un.kb_lo - r * g.k_blocks) * C::BK;
        const int k_end = g.k_blocks * C::BK;
        const int ax = g.a_x1 * t.ib1, ay = g.a_y0 * t.ib0, bx = g.b_x1 * t.ib1, by = g.b_y0 * t.ib0;
        for (int i = un.kb_lo; i < un.kb_hi; ++i) {
          const uint32_t s = ring_s, ph = ring_ph;
          if (++ring_s == (uint32_t)STAGES) { ring_s = 0; ring_ph ^= 1u; }
          if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, abortp, g.wait_limit)) { ok = false; break; }
          const uint32_t full = smem_u32(&bar_full[s]);
          mbar_expect_tx(full, C::STAGE_BYTES);
          const uint32_t a_dst = smem_base + s * C::STAGE_BYTES;
          load_operand<C::BMB, C::BK, C::CH, C::MN_LBO>(a_dst, &tma_a, full, g.a_ld, t.mt * C::BMB, kx, ax + g.a_xr * r, ay);
          load_operand<BN, C::BK, C::CH, C::MN_LBO>(a_dst + C::A_BYTES, &tma_b, full, g.b_ld, t.nt * BN, kx,
                                                     bx + g.b_xr * r, by);
          kx += C::BK;
          if (kx == k_end) { kx = 0; ++r; }
        }
      }
    }
    __syncwarp();
  } else if (warp == MMA_WARP) {
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | ((uint32_t)(g.a_mn ? 1 : 0) << 15) | ((uint32_t)(g.b_mn ? 1 : 0) << 16) |
                             ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      const uint32_t a_lbo = g.a_mn ? C::MN_LBO : 16u, b_lbo = g.b_mn ? C::MN_LBO : 16u;
      const uint32_t a_kadv = g.a_mn ? C::MN_KADV : C::K_KADV, b_kadv = g.b_mn ? C::MN_KADV : C::K_KADV;
      const uint64_t da0 = make_smem_desc(smem_base, a_lbo, C::SBO, C::LAYOUT);
      const uint64_t db0 = make_smem_desc(smem_base + C::A_BYTES, b_lbo, C::SBO, C::LAYOUT);
      const uint32_t a_hi = (uint32_t)(da0 >> 32), b_hi = (uint32_t)(db0 >> 32);
      const uint32_t a_lo0 = (uint32_t)da0, b_lo0 = (uint32_t)db0;
      const uint32_t a_k16 = a_kadv >> 4, b_k16 = b_kadv >> 4;
      constexpr uint32_t STAGE16 = C::STAGE_BYTES >> 4, HALF16 = C::A_HALF >> 4;
      uint32_t ring_s = 0, ring_ph = 0, tcount = 0;
      bool ok = true;
      for (long long unit = blockIdx.x; ok && unit < g.total_units; unit += gridDim.x, ++tcount) {
        const Unit un = decode_unit(g, unit, total_kb);
        // both accumulators are free once the epilogue has read the previous tile out of them
        if (!mbar_wait(smem_u32(&bar_tempty), (tcount & 1u) ^ 1u, abortp, g.wait_limit)) { ok = false; break; }
        tc_fence_after();
        for (int i = un.kb_lo; i < un.kb_hi; ++i) {
          const uint32_t s = ring_s, ph = ring_ph;
          if (++ring_s == (uint32_t)STAGES) { ring_s = 0; ring_ph ^= 1u; }
          if (!mbar_wait(smem_u32(&bar_full[s]), ph, abortp, g.wait_limit)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + (uint32_t)s * STAGE16, b_lo = b_lo0 + (uint32_t)s * STAGE16;
#pragma unroll
          for (int ks = 0; ks < C::KSTEPS; ++ks) {
            const uint32_t acc = (i > un.kb_lo || ks > 0) ? 1u : 0u;
            umma_lohi<2>(tmem_base, a_lo + ks * a_k16, a_hi, b_lo + ks * b_k16, b_hi, idesc, acc);
            umma_lohi<2>(tmem_base + BN, a_lo + HALF16 + ks * a_k16, a_hi, b_lo + ks * b_k16, b_hi, idesc, acc);
          }
          umma_commit(smem_u32(&bar_empty[s]));
        }
        if (ok) umma_commit(smem_u32(&bar_tfull));
      }
    }
    __syncwarp();
  } else {
    // epilogue: warp group eg (warps 4 eg .. 4 eg + 3) owns accumulator eg = rows 128 eg .. 128 eg + 127 of the tile
    const int eg = warp >> 2, ew = warp & 3;
    const int bar_id = 1 + eg;
    const bool leader = (threadIdx.x & 127) == 0;
    uint32_t tcount = 0;
    bool ok = true;
    for (long long unit = blockIdx.x; ok && unit < g.total_units; unit += gridDim.x, ++tcount) {
      const TileCoord t = decode_tile(g, decode_unit(g, unit, total_kb).tile);
      const int row0 = t.mt * C::BMB + eg * BM;              // first output row of this group's accumulator
      const int row = row0 + ew * 32 + lane;
      // the tile's column bias, fetched before the accumulators are waited for; the group's barriers below order
      // these writes before the reads and the reads before the next tile's writes
      const bool bias_cols = g.fused && !g.bias_row && g.ksplit == 1 && !g.acc32;
      if (bias_cols) {
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {
          const int j = (threadIdx.x & 127) + jj * 128, colj = t.nt * BN + j;
          __half bv = __float2half_rn(0.f);
          if (g.bias != nullptr && colj < g.n) bv = __ldg(reinterpret_cast<const __half*>(g.bias) + colj);
          bias_s[eg][j] = bv;
        }
      }
      bool got = mbar_wait(smem_u32(&bar_tfull), tcount & 1u, abortp, g.wait_limit);
      got = named_barrier_and(bar_id, 128, got);             // the staged stores use named barriers: all or none
      if (!got) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(ew * 32) << 16) + (uint32_t)eg * BN;
      const int r_in = ew * 32 + lane;
      const uint32_t sw = (uint32_t)(r_in & 7);
      const uint32_t stage = smem_base + C::OFF_OUT + (uint32_t)eg * C::OUT_BYTES;
      if ((g.ksplit > 1 || g.acc32) && row0 < g.m) {
        // K slice, or an f32 destination: the f32 sums are added into the device's scratch matrix / into C (tma_c maps
        // it here), 32 columns
        // = one 128-byte line per row at a time through the same staging buffer
#pragma unroll 1
        for (int c4 = 0; c4 < BN / 32; ++c4) {
          const int col0 = t.nt * BN + c4 * 32;
          if (col0 < g.n) {
            if (leader) bulk_wait_group_read<0>();
            named_barrier_sync(bar_id, 128);
            uint32_t v[32];
            tmem_ld_32x32(taddr + c4 * 32, v);
            tmem_wait_ld();
#pragma unroll
            for (int q4 = 0; q4 < 8; ++q4)
              st_shared_v4_u32(stage + (uint32_t)r_in * 128u + ((((uint32_t)q4) ^ sw) << 4), v[q4 * 4], v[q4 * 4 + 1],
                               v[q4 * 4 + 2], v[q4 * 4 + 3]);
            fence_proxy_async_smem();
            named_barrier_sync(bar_id, 128);
            if (leader) {
              tma_reduce_add_4d(&tma_c, stage, col0, row0, 0, 0);
              bulk_commit_group();
            }
          }
        }
      } else if (row0 < g.m) {                               // group-uniform
#pragma unroll
        for (int c2 = 0; c2 < BN / 64; ++c2) {
          const int col0 = t.nt * BN + c2 * 64;
          if (col0 < g.n) {
            if (leader) bulk_wait_group_read<0>();           // the store that last used this buffer has read it
            named_barrier_sync(bar_id, 128);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint32_t v[32];
              tmem_ld_32x32(taddr + c2 * 64 + h * 32, v);
              tmem_wait_ld();
              float f[32];
#pragma unroll
              for (int q = 0; q < 32; ++q) f[q] = __uint_as_float(v[q]);
              if (bias_cols) {
                fused_epilogue_cols(f, g, &bias_s[eg][c2 * 64 + h * 32]);
              } else if (g.fused && row < g.m) {
                const int valid = (g.n - col0 - h * 32) < 32 ? (g.n - col0 - h * 32) : 32;
                if (valid > 0) fused_epilogue<__half>(f, g, row, col0 + h * 32, valid);
              }
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4) {
                uint32_t w[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const __half2 hh = __floats2half2_rn(f[q4 * 8 + 2 * e], f[q4 * 8 + 2 * e + 1]);
                  w[e] = *reinterpret_cast<const uint32_t*>(&hh);
                }
                st_shared_v4_u32(stage + (uint32_t)r_in * 128u + ((((uint32_t)(h * 4 + q4)) ^ sw) << 4), w[0], w[1], w[2], w[3]);
              }
            }
            fence_proxy_async_smem();
            named_barrier_sync(bar_id, 128);
            if (leader) {
              if (g.c_tma == 2) tma_reduce_add_4d(&tma_c, stage, col0, row0, t.ib1, t.ib0);
              else tma_store_4d(&tma_c, stage, col0, row0, t.ib1, t.ib0);
              bulk_commit_group();
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&bar_tempty));
    }
    if (leader) bulk_wait_group_read<0>();
  }

  tc_fence_before();
  __syncthreads();
  teardown(abort_flag, g.status);
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// 3xTF32 operand split of the stages, run by SPLIT_THREADS threads (tt = 0 .. SPLIT_THREADS-1).
// Each raw f32 x stays in place as the `big` operand (the tensor core reads its top 19 bits) and
// small = x - trunc_tf32(x) (exact; the tensor core again keeps its top 19 bits) is written RAW_BYTES
// further on.  A stage is a whole number of 16-byte vectors per thread; all of a thread's vectors are
// loaded before any is stored, to cover the shared-memory latency.
constexpr int SPLIT_WARPS = 8;
constexpr int SPLIT_THREADS = SPLIT_WARPS * 32;

// `skip_a_hi`: rows 64..127 of the A tile are not in use (an output with at most 64 rows): their vectors (the second
// SPLIT_THREADS * 16 bytes of a stage) are left alone.
template <typename C>
__device__ __forceinline__ void split_role(const TcArgs& g, uint32_t smem_base, uint64_t* bar_full,
                                           uint64_t* bar_xform, volatile int* abortp, int total_kb, int tt,
                                           bool skip_a_hi = false) {
  static_assert(SPLIT_THREADS * 16 == C::A_BYTES / 2, "the A tile's upper half must be one vector per split thread");
  constexpr int STAGES = C::STAGES;
  constexpr int NVEC = C::RAW_BYTES / 16;
  static_assert(NVEC % SPLIT_THREADS == 0, "a stage must be a whole number of vectors per split thread");
  constexpr int PER = NVEC / SPLIT_THREADS;             // 6 (BN = 256), 4 (128), 3 (64)
  uint32_t it = 0;
  bool ok = true;
  for (long long unit = blockIdx.x; ok && unit < g.total_units; unit += gridDim.x) {
    const Unit un = decode_unit(g, unit, total_kb);
    for (int i = un.kb_lo; i < un.kb_hi; ++i, ++it) {
      const int s = it % STAGES;
      const uint32_t ph = (it / STAGES) & 1u;
      if (!mbar_wait(smem_u32(&bar_full[s]), ph, abortp, g.wait_limit)) { ok = false; break; }
      const uint32_t raw = smem_base + s * C::STAGE_BYTES + tt * 16;
      {
        uint32_t x[PER][4];
#pragma unroll
        for (int u = 0; u < PER; ++u) {
          if (u == 1 && skip_a_hi) continue;
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(x[u][0]), "=r"(x[u][1]), "=r"(x[u][2]), "=r"(x[u][3])
                       : "r"(raw + u * (SPLIT_THREADS * 16)));
        }
#pragma unroll
        for (int u = 0; u < PER; ++u) {
          if (u == 1 && skip_a_hi) continue;
          uint32_t sm[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float d = __uint_as_float(x[u][e]) - __uint_as_float(x[u][e] & 0xffffe000u);
            d = (d != d) ? 0.f : d;                     // inf - inf: keep inf / nan in `big` only
            if ((g.xform_mode & 1) == 0) asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(sm[e]) : "f"(d));
            else sm[e] = __float_as_uint(d);
          }
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                       ::"r"(raw + C::RAW_BYTES + u * (SPLIT_THREADS * 16)), "r"(sm[0]), "r"(sm[1]), "r"(sm[2]), "r"(sm[3])
                       : "memory");
        }
      }
      fence_proxy_async_smem();                         // generic-proxy writes -> visible to tcgen05.mma
      mbar_arrive(smem_u32(&bar_xform[s]));
    }
  }
}

// ---------------------------------------------------------------------------------------------
// f32 kernel (3xTF32 with chunked promotion)
// ---------------------------------------------------------------------------------------------
// CV: 0 = GEMM over strided matrices; 1, 2 = implicit convolution (see TcArgs): only the producer's TMA
// coordinates, the MMA's N and the epilogue's column range differ.
template <int BN, int CV = 0>
__global__ void __launch_bounds__(CfgS<BN>::THREADS, 1)
gemm_tf32x3_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                   const __grid_constant__ CUtensorMap tma_c, const TcArgs g) {
  using C = CfgS<BN>;
  constexpr int STAGES = C::STAGES;
  constexpr int PRODUCER_WARP = 8, MMA_WARP = 9;      // warpgroup 2; warpgroups 3 and 4 split operands

  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t bar_full[STAGES];
  __shared__ __align__(8) uint64_t bar_empty[STAGES];
  __shared__ __align__(8) uint64_t bar_xform[STAGES];
  __shared__ __align__(8) uint64_t bar_tfull[2];
  __shared__ __align__(8) uint64_t bar_tempty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wg = warp >> 2;
  volatile int* abortp = &abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
      mbar_init(smem_u32(&bar_xform[s]), SPLIT_THREADS);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bar_tfull[b]), 1);
      mbar_init(smem_u32(&bar_tempty[b]), 256);
    }
    abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == MMA_WARP) {
    tmem_alloc(smem_u32(&tmem_slot), C::TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == PRODUCER_WARP && lane == 0) {
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  const int total_kb = g.red * g.k_blocks;

  if (wg == 2) {
    setmaxnreg_dec_low();
    if (warp == PRODUCER_WARP && (CV == 2 || lane == 0)) {
      // ---------------------------------------------------------------- TMA producer
      // One thread (CV 2: one warp).  Its instruction stream is a chain of dependent operations at some 15-20 clocks
      // each, so everything a k-block needs beyond the loads themselves is kept out of the loop: ring position, tap
      // and pixel counters advance by increments, divisions happen once per work unit.
      uint32_t ring_s = 0, ring_ph = 0;                    // stage ring position and its phase bit
      bool ok = true;
      for (long long unit = blockIdx.x; ok && unit < g.total_units; unit += gridDim.x) {
        const Unit un = decode_unit(g, unit, total_kb);
        const TileCoord t = decode_tile(g, un.tile);
        if constexpr (CV == 0) {
          int r = un.kb_lo / g.k_blocks, kx = (un.kb_lo - r * g.k_blocks) * C::BK;
          const int k_end = g.k_blocks * C::BK;
          const int ax = g.a_x1 * t.ib1, ay = g.a_y0 * t.ib0, bx = g.b_x1 * t.ib1, by = g.b_y0 * t.ib0;
          for (int i = un.kb_lo; i < un.kb_hi; ++i) {
            const uint32_t s = ring_s, ph = ring_ph;
            if (++ring_s == (uint32_t)STAGES) { ring_s = 0; ring_ph ^= 1u; }
            if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, abortp, g.wait_limit)) { ok = false; break; }
            const uint32_t full = smem_u32(&bar_full[s]);
            const uint32_t a_dst = smem_base + s * C::STAGE_BYTES;
            mbar_expect_tx(full, C::RAW_BYTES);
            load_operand<BM, C::BK, C::CH, C::MN_LBO>(a_dst, &tma_a, full, g.a_ld, t.mt * BM, kx, ax + g.a_xr * r, ay);
            load_operand<BN, C::BK, C::CH, C::MN_LBO>(a_dst + C::A_BYTES, &tma_b, full, g.b_ld, t.nt * BN, kx,
                                                       bx + g.b_xr * r, by);
            kx += C::BK;
            if (kx == k_end) { kx = 0; ++r; }
          }
        } else if constexpr (CV == 1) {
          // k-block = (tap, block of 16 channels): A = the re-laid-out filters (k = tap * channels + channel), B = one
          // box of the channels-last image shifted by the tap; pixels outside the image arrive as zeros
          int tap = un.kb_lo / g.cv_cblocks, cb = un.kb_lo - tap * g.cv_cblocks;
          int k1 = tap / g.cv_kw, k2 = tap - k1 * g.cv_kw;
          int kx = un.kb_lo * C::BK, bw = g.cv_w0 + k2 * g.cv_dw, bh = t.nt * g.cv_rows + g.cv_h0 + k1 * g.cv_dh;
          int bc = t.ib1 * g.cv_cpad + cb * C::BK;
          const int bc_end = (t.ib1 + 1) * g.cv_cpad, w_end = g.cv_w0 + g.cv_kw * g.cv_dw;
          const uint32_t tx = (uint32_t)((g.m64 ? C::A_BYTES / 2 : C::A_BYTES) + g.b_tx_bytes);   // m64: the A box has 64 rows
          for (int i = un.kb_lo; i < un.kb_hi; ++i) {
            const uint32_t s = ring_s, ph = ring_ph;
            if (++ring_s == (uint32_t)STAGES) { ring_s = 0; ring_ph ^= 1u; }
            if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, abortp, g.wait_limit)) { ok = false; break; }
            const uint32_t full = smem_u32(&bar_full[s]);
            const uint32_t a_dst = smem_base + s * C::STAGE_BYTES;
            mbar_expect_tx(full, tx);
            tma_load_4d(a_dst, &tma_a, full, kx, t.mt * BM, t.ib1, 0);
            tma_load_4d(a_dst + C::A_BYTES, &tma_b, full, bc, bw, bh, t.ib0);
            kx += C::BK; bc += C::BK;
            if (bc == bc_end) {                              // next tap
              bc -= g.cv_cpad; bw += g.cv_dw;
              if (bw == w_end) { bw = g.cv_w0; bh += g.cv_dh; }
            }
          }
        } else {
          // CV 2.  k-block = 16 pixels of output row `oh` of image r: A = that box of grad_out for 128 output channels
          // (lane 0), B = for each 32-column chunk of the tile the same pixels of the image shifted by the chunk's tap
          // (lane j + 1 loads chunk j, all chunks in one instruction).
          const int nch = g.tile_cols / 32;
          const int n = t.nt * g.tile_cols + (lane - 1) * 32, tap = n / g.cv_cpad, tk1 = tap / g.cv_kw;
          const bool loader = lane >= 1 && lane <= nch;
          const int my_c = n - tap * g.cv_cpad, my_w = g.cv_w0 + (tap - tk1 * g.cv_kw) * g.cv_dw;
          const int my_h = tap < g.cv_taps ? g.cv_h0 + tk1 * g.cv_dh : (1 << 20);   // past the last tap: zero fill
          const uint32_t my_dst = C::A_BYTES + (uint32_t)(lane - 1) * C::MN_LBO;
          // k-block = a box of cv_bw x cv_bh = 16 output pixels (the shape that wastes least on the image's edges)
          int r = un.kb_lo / g.k_blocks, rem = un.kb_lo - r * g.k_blocks;
          int oh = rem / g.cv_wblocks, w = (rem - oh * g.cv_wblocks) * g.cv_bw;
          oh *= g.cv_bh;
          const int w_end = g.cv_wblocks * g.cv_bw, h_end = g.cv_rows * g.cv_bh;
          const uint32_t tx = (uint32_t)(C::A_BYTES + g.b_tx_bytes);
          for (int i = un.kb_lo; i < un.kb_hi; ++i) {
            const uint32_t s = ring_s, ph = ring_ph;
            if (++ring_s == (uint32_t)STAGES) { ring_s = 0; ring_ph ^= 1u; }
            if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, abortp, g.wait_limit))) { ok = false; break; }
            const uint32_t full = smem_u32(&bar_full[s]);
            const uint32_t a_dst = smem_base + s * C::STAGE_BYTES;
            if (lane == 0) {
              mbar_expect_tx(full, tx);
              tma_load_4d(a_dst, &tma_a, full, w, oh, t.mt * BM, r);
            }
            if (loader) tma_load_4d(a_dst + my_dst, &tma_b, full, my_c, w + my_w, oh + my_h, r);
            w += g.cv_bw;
            if (w == w_end) { w = 0; oh += g.cv_bh; if (oh == h_end) { oh = 0; ++r; } }
          }
        }
      }
    } else if (warp == MMA_WARP && lane == 0) {
      // ---------------------------------------------------------------- MMA issuer
      // instruction descriptor: D = f32, A = B = tf32 (format 2), majors, N >> 3, M >> 4
      const uint32_t mma_n = CV ? (uint32_t)g.mma_n : (uint32_t)BN;
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(g.a_mn ? 1 : 0) << 15) |
                             ((uint32_t)(g.b_mn ? 1 : 0) << 16) | ((mma_n >> 3) << 17) |
                             ((uint32_t)(((CV == 1 && g.m64) ? 64 : BM) >> 4) << 24);
      const uint32_t a_lbo = g.a_mn ? C::MN_LBO : 16u, b_lbo = g.b_mn ? C::MN_LBO : 16u;
      const uint32_t a_sbo = g.a_mn ? C::MN_SBO : C::K_SBO, b_sbo = g.b_mn ? C::MN_SBO : C::K_SBO;
      const uint32_t a_lay = g.a_mn ? C::MN_LAYOUT : C::K_LAYOUT, b_lay = g.b_mn ? C::MN_LAYOUT : C::K_LAYOUT;
      const uint32_t a_kadv = g.a_mn ? C::MN_KADV : C::K_KADV, b_kadv = g.b_mn ? C::MN_KADV : C::K_KADV;
      // descriptor words of stage 0 (see umma_lohi): per stage, per operand copy and per k-step only the low word moves
      const uint64_t da0 = make_smem_desc(smem_base, a_lbo, a_sbo, a_lay);
      const uint64_t db0 = make_smem_desc(smem_base + C::A_BYTES, b_lbo, b_sbo, b_lay);
      const uint32_t a_hi = (uint32_t)(da0 >> 32), b_hi = (uint32_t)(db0 >> 32);
      const uint32_t a_lo0 = (uint32_t)da0, b_lo0 = (uint32_t)db0;
      const uint32_t a_k16 = a_kadv >> 4, b_k16 = b_kadv >> 4;
      constexpr uint32_t STAGE16 = C::STAGE_BYTES >> 4, SMALL16 = C::RAW_BYTES >> 4;
      uint32_t ring_s = 0, ring_ph = 0, ccount = 0;        // stage ring position and its phase bit
      bool ok = true;
      for (long long unit = blockIdx.x; ok && unit < g.total_units; unit += gridDim.x) {
        const Unit un = decode_unit(g, unit, total_kb);
        for (int kb0 = un.kb_lo; ok && kb0 < un.kb_hi; kb0 += C::CHUNK_KB, ++ccount) {
          const uint32_t buf = ccount & 1u, cph = (ccount >> 1) & 1u;
          if (!mbar_wait(smem_u32(&bar_tempty[buf]), cph ^ 1u, abortp, g.wait_limit)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + buf * BN;
          const int nkb = (un.kb_hi - kb0) < C::CHUNK_KB ? (un.kb_hi - kb0) : C::CHUNK_KB;
          for (int i = 0; i < nkb; ++i) {
            const uint32_t s = ring_s, ph = ring_ph;
            if (++ring_s == (uint32_t)STAGES) { ring_s = 0; ring_ph ^= 1u; }
            if (!mbar_wait(smem_u32(&bar_xform[s]), ph, abortp, g.wait_limit)) { ok = false; break; }
            tc_fence_after();
            const uint32_t a_lo = a_lo0 + (uint32_t)s * STAGE16, b_lo = b_lo0 + (uint32_t)s * STAGE16;
#pragma unroll
            for (int ks = 0; ks < C::KSTEPS; ++ks) {
              const uint32_t al = a_lo + ks * a_k16, bl = b_lo + ks * b_k16;
              umma_lohi<4>(d_tmem, al + SMALL16, a_hi, bl, b_hi, idesc, (i > 0 || ks > 0) ? 1u : 0u);   // small * big
              umma_lohi<4>(d_tmem, al, a_hi, bl + SMALL16, b_hi, idesc, 1u);                            // big * small
              umma_lohi<4>(d_tmem, al, a_hi, bl, b_hi, idesc, 1u);                                      // big * big
            }
            umma_commit(smem_u32(&bar_empty[s]));
          }
          if (ok) umma_commit(smem_u32(&bar_tfull[buf]));
        }
      }
    }
    __syncwarp();
  } else if (wg >= 3) {
    // ------------------------------------------------------------------ operand split (warps 12..19)
    setmaxnreg_dec_split();
    split_role<C>(g, smem_base, bar_full, bar_xform, abortp, total_kb, threadIdx.x - 384, CV == 1 && g.m64);
  } else {
    // ------------------------------------------------------------------ epilogue (warpgroups 0 and 1)
    setmaxnreg_inc_epi();
    const int quad = warp & 3;                        // TMEM lane quadrant this warp may read
    const int col_base = wg * C::HALF;                // this warpgroup's half of the tile's columns
    uint32_t ccount = 0;
    bool ok = true;
    for (long long unit = blockIdx.x; ok && unit < g.total_units; unit += gridDim.x) {
      const Unit un = decode_unit(g, unit, total_kb);
      const TileCoord t = decode_tile(g, un.tile);
      float acc[C::HALF];
#pragma unroll
      for (int q = 0; q < C::HALF; ++q) acc[q] = 0.f;
      for (int kb0 = un.kb_lo; kb0 < un.kb_hi; kb0 += C::CHUNK_KB, ++ccount) {
        const uint32_t buf = ccount & 1u, cph = (ccount >> 1) & 1u;
        if (!mbar_wait(smem_u32(&bar_tfull[buf]), cph, abortp, g.wait_limit)) { ok = false; break; }
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + buf * BN + col_base;
#pragma unroll
        for (int c = 0; c < C::HALF / 16; ++c) {
          uint32_t v[16];
          tmem_ld_32x16(taddr + c * 16, v);
          tmem_wait_ld();
#pragma unroll
          for (int q = 0; q < 16; ++q) acc[c * 16 + q] += __uint_as_float(v[q]);   // round-to-nearest add
        }
        tc_fence_before();
        mbar_arrive(smem_u32(&bar_tempty[buf]));
      }
      // the staged stores below synchronise a warpgroup with a named barrier, which has no time-out: all of its
      // threads take this unit's output or none does
      if (g.c_tma) ok = named_barrier_and(1 + wg, 128, ok);
      if (!ok) break;
      if (un.kb_lo >= un.kb_hi) continue;               // an empty unit of the stream-K decomposition
      // partial sums (a K slice, or a stream-K range that does not span the tile's whole K) are added atomically
      const bool partial = g.ksplit > 1 || ((g.streamk || g.tail_per > 0 || g.kt_cut > 0) && !(un.kb_lo == 0 && un.kb_hi == total_kb));
      // An MMA with M = 64 (m64: outputs of at most 64 rows) keeps row r in TMEM lane (r / 16) * 32 + r % 16: each
      // warp's lanes 0..15 hold 16 rows, its lanes 16..31 nothing.
      const bool m64 = CV == 1 && g.m64;
      const int r_in = m64 ? quad * 16 + (lane & 15) : quad * 32 + lane;
      const int row = (m64 && lane >= 16) ? g.m : t.mt * BM + r_in;     // row >= g.m: this thread stores nothing
      // columns of this tile: [tile_col0, n_end).  An implicit-convolution tile holds tile_valid columns (whole image
      // rows) and the next tile starts tile_cols further on.
      const int tile_col0 = CV ? t.nt * g.tile_cols : t.nt * BN;
      const int n_end = (CV && tile_col0 + g.tile_valid < g.n) ? tile_col0 + g.tile_valid : g.n;
      float* cbase = (float*)g.c + t.ib0 * g.c_b0 + t.ib1 * g.c_b1;
      if (g.c_tma) {
        // Output through shared memory and TMA, as in the f16 kernel: per-thread row stores hand the memory
        // system 32 separate 16- or 32-byte pieces per instruction, which bounds GEMMs with a short K and a
        // wide output; a staged group of 128 rows x 32 columns leaves as one bulk tensor store (beta = 0) or
        // reduce-add (beta = 1) of whole 128-byte lines.  Rows and columns past the output's extent are clipped
        // by the tensor map.
        const uint32_t stage = smem_base + C::OFF_OUT + (uint32_t)wg * C::OUT_BYTES;
        const uint32_t sw = (uint32_t)(r_in & 7);
        const bool leader = (threadIdx.x & 127) == 0;
#pragma unroll
        for (int c = 0; c < C::HALF / 32; ++c) {
          const int col0 = tile_col0 + col_base + c * 32;
          if (col0 < n_end) {                            // warpgroup-uniform
            const int valid = (n_end - col0) < 32 ? (n_end - col0) : 32;
            if (g.fused && row < g.m) fused_epilogue<float>(&acc[c * 32], g, row, col0, valid);
            if (CV && valid < 32 && n_end < g.n) {
              // the group's other columns belong to the next tile (the map clips only at the output's end)
              if (row < g.m) {
                if (partial) add_chunk_atomic(cbase + (long long)row * g.ldc + col0, &acc[c * 32], valid);
                else store_chunk(cbase + (long long)row * g.ldc + col0, &acc[c * 32], valid, g.beta, 0);
              }
              continue;
            }
            if (leader) bulk_wait_group_read<0>();       // the store that last used this buffer has read it
            named_barrier_sync(1 + wg, 128);
            if (!m64 || lane < 16) {
#pragma unroll
              for (int q = 0; q < 8; ++q)
                st_shared_v4_u32(stage + (uint32_t)r_in * 128u + ((((uint32_t)q) ^ sw) << 4),
                                 __float_as_uint(acc[c * 32 + q * 4]), __float_as_uint(acc[c * 32 + q * 4 + 1]),
                                 __float_as_uint(acc[c * 32 + q * 4 + 2]), __float_as_uint(acc[c * 32 + q * 4 + 3]));
            }
            fence_proxy_async_smem();
            named_barrier_sync(1 + wg, 128);
            if (leader) {
              // a partial sum (K slice, tail range) is ADDED, whatever beta is: the output holds zeros or beta * C;
              // the bulk reduce-add works on whole 128-byte lines, where per-thread red.global.add.v4 touches 32 lines
              // per instruction
              if (g.c_tma == 2 || partial) tma_reduce_add_4d(&tma_c, stage, col0, t.mt * BM, t.ib1, t.ib0);
              else tma_store_4d(&tma_c, stage, col0, t.mt * BM, t.ib1, t.ib0);
              bulk_commit_group();
            }
          }
        }
      } else if (row < g.m) {
#pragma unroll
        for (int c = 0; c < C::HALF / 32; ++c) {
          const int col0 = tile_col0 + col_base + c * 32;
          if (col0 < n_end) {
            const int valid = (n_end - col0) < 32 ? (n_end - col0) : 32;
            if (g.fused) fused_epilogue<float>(&acc[c * 32], g, row, col0, valid);
            if (partial) {
              if (g.c_col) add_chunk_atomic_col(cbase + (long long)col0 * g.ldc + row, &acc[c * 32], valid, g.ldc);
              else add_chunk_atomic(cbase + (long long)row * g.ldc + col0, &acc[c * 32], valid);
            } else if (g.c_col) {
              store_chunk_col(cbase + (long long)col0 * g.ldc + row, &acc[c * 32], valid, g.ldc, g.beta);
            } else {
              store_chunk(cbase + (long long)row * g.ldc + col0, &acc[c * 32], valid, g.beta, g.c_wide);
            }
          }
        }
      }
    }
    if ((threadIdx.x & 127) == 0) bulk_wait_group_read<0>();   // shared memory must outlive the last bulk stores' reads
  }

  tc_fence_before();
  __syncthreads();
  teardown(abort_flag, g.status);
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// Split-K of an f16 GEMM: C = f16(beta * C + S) for the m x n f32 partial-sum matrix S (row-major, ld = lds).
// C element (i, j) sits at i*c_r + j*c_c.
__global__ void __launch_bounds__(256) splitk_finalize_f16_kernel(const float* __restrict__ S, long long lds,
                                                                  __half* C, long long c_r, long long c_c, int m, int n,
                                                                  int beta) {
  const long long total = (long long)m * n;
  for (long long idx = (long long)blockIdx.x * 256 + threadIdx.x; idx < total; idx += (long long)gridDim.x * 256) {
    // walk C's unit-stride dimension fastest
    int i, j;
    if (c_c == 1) { i = (int)(idx / n); j = (int)(idx - (long long)i * n); }
    else { j = (int)(idx / m); i = (int)(idx - (long long)j * m); }
    float v = S[(long long)i * lds + j];
    __half* dst = C + (long long)i * c_r + (long long)j * c_c;
    if (beta) v += __half2float(*dst);
    *dst = __float2half_rn(v);
  }
}

// Self-test of the bounded wait: one thread waits on a barrier that nothing ever completes.  The wait must give up
// after its clock budget, raise the abort flag and let the CTA run the same teardown as the GEMM kernels (status
// word = B200_ERR_DEVICE_TIMEOUT).  The cycles the wait took are left in g_selftest_cycles; with a budget of 0 that
// is the time the polls themselves take (a failed try_wait suspends the thread for a hardware-defined while).
__device__ long long g_selftest_cycles;
__global__ void __launch_bounds__(128) wait_selftest_kernel(long long limit, int* status) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const long long t0 = clock64();
    mbar_wait(smem_u32(&bar), 0u, &abort_flag, limit);
    g_selftest_cycles = clock64() - t0;
  }
  __syncthreads();
  teardown(abort_flag, status);
}

// ---------------------------------------------------------------------------------------------
// Host side: operand classification, tensor maps, launch
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
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

// How a 2-D operand (rows x cols, element strides sr / sc) can be walked by TMA.
struct Layout2D {
  bool ok = false;
  bool cols_contig = false;   // true: cols is the unit-stride dim; false: rows is
  int64_t ld = 0;             // stride of the other dim (elements)
};

Layout2D classify(int64_t rows, int64_t cols, int64_t sr, int64_t sc, size_t esize) {
  Layout2D L;
  const int64_t align = 16 / (int64_t)esize;
  auto pad = [&](int64_t x) { return (x + align - 1) / align * align; };
  if (rows == 1 && cols == 1) { L.ok = true; L.cols_contig = true; L.ld = align; return L; }
  if (cols == 1) {
    if (sr == 1) { L.ok = true; L.cols_contig = false; L.ld = pad(rows); }
    else if (sr > 0 && sr % align == 0) { L.ok = true; L.cols_contig = true; L.ld = sr; }
    return L;
  }
  if (rows == 1) {
    if (sc == 1) { L.ok = true; L.cols_contig = true; L.ld = pad(cols); }
    else if (sc > 0 && sc % align == 0) { L.ok = true; L.cols_contig = false; L.ld = sc; }
    return L;
  }
  if (sc == 1 && sr > 0 && sr % align == 0) { L.ok = true; L.cols_contig = true; L.ld = sr; return L; }
  if (sr == 1 && sc > 0 && sc % align == 0) { L.ok = true; L.cols_contig = false; L.ld = sc; return L; }
  return L;
}

bool batch_stride_ok(int64_t count, int64_t stride, size_t esize) {
  if (count <= 1 || stride == 0) return true;
  return stride > 0 && (stride * (int64_t)esize) % 16 == 0;
}

// The transposed problem C^T = B^T A^T (same memory, m <-> n, operands exchanged).
GemmProblem transposed(const GemmProblem& p) {
  GemmProblem q = p;
  q.m = p.n; q.n = p.m;
  q.a = p.b; q.a_b0 = p.b_b0; q.a_b1 = p.b_b1; q.a_red = p.b_red; q.a_r = p.b_c; q.a_c = p.b_r;
  q.b = p.a; q.b_b0 = p.a_b0; q.b_b1 = p.a_b1; q.b_red = p.a_red; q.b_r = p.a_c; q.b_c = p.a_r;
  q.c_r = p.c_c; q.c_c = p.c_r;
  q.bias_dim = p.bias_dim ? 0 : 1;
  return q;
}

struct Plan {
  bool ok = false;
  GemmProblem p;
  Layout2D la, lb;
  int64_t ldc = 0;
  int c_col = 0;     // 1: C element (i, j) of the kernel's problem sits at j*ldc + i (column store)
};

// Two ways to run a GEMM whose C has a unit stride along one dimension:
//   row store    : the kernel's N runs along C's unit-stride dimension; each epilogue thread writes
//                  16-byte vectors of its own row (needs ldc to be a multiple of 16 bytes);
//   column store : the kernel's M runs along C's unit-stride dimension; for every output column the 32
//                  lanes of a warp write 32 consecutive elements (fully coalesced, any ldc).
// Whichever of the problem and its transpose has the required unit stride is used.
Plan make_plan(const GemmProblem& p0, bool col_store) {
  Plan pl;
  if (p0.dtype == B200_F64) return pl;
  const size_t es = dtype_size(p0.dtype);
  const bool unit_n = (p0.c_c == 1 || p0.n == 1), unit_m = (p0.c_r == 1 || p0.m == 1);
  if (!col_store) {
    if (unit_n) pl.p = p0; else if (unit_m) pl.p = transposed(p0); else return pl;
  } else {
    if (unit_m) pl.p = p0; else if (unit_n) pl.p = transposed(p0); else return pl;
  }
  pl.c_col = col_store ? 1 : 0;
  const GemmProblem& p = pl.p;
  if (p.m < 1 || p.n < 1 || p.k < 1 || p.b0 < 1 || p.b1 < 1 || p.red < 1) return pl;
  if (p.red > 1 && (p.b0 != 1 || p.b1 != 1)) return pl;
  if (p.m > 0x7fffff00LL || p.n > 0x7fffff00LL || p.k > 0x7fffff00LL) return pl;
  if (p.b0 > 0x7fffffffLL || p.b1 > 0x7fffffffLL || p.red > 0x7fffffffLL) return pl;
  pl.la = classify(p.m, p.k, p.a_r, p.a_c, es);
  pl.lb = classify(p.k, p.n, p.b_r, p.b_c, es);
  if (!pl.la.ok || !pl.lb.ok) return pl;
  const int64_t align = 16 / (int64_t)es;
  if (!col_store) {
    // row-major C with an aligned leading dimension (vector stores in the epilogue)
    pl.ldc = p.c_r;
    if (p.m == 1 && pl.ldc <= 0) pl.ldc = (p.n + align - 1) / align * align;
    if (pl.ldc <= 0 || pl.ldc % align) return pl;
    if ((uintptr_t)p.c & 15) return pl;
    if ((p.b0 > 1 && (p.c_b0 <= 0 || p.c_b0 % align)) || (p.b1 > 1 && (p.c_b1 <= 0 || p.c_b1 % align))) return pl;
  } else {
    // column-major C: scalar stores, only element alignment is needed
    pl.ldc = p.c_c;
    if (p.n == 1 && pl.ldc <= 0) pl.ldc = p.m;
    if (pl.ldc <= 0) return pl;
    if ((p.b0 > 1 && p.c_b0 <= 0) || (p.b1 > 1 && p.c_b1 <= 0)) return pl;
  }
  if (((uintptr_t)p.a | (uintptr_t)p.b | (uintptr_t)p.bias) & 15) return pl;
  if (!batch_stride_ok(p.b0, p.a_b0, es) || !batch_stride_ok(p.b1, p.a_b1, es) ||
      !batch_stride_ok(p.red, p.a_red, es) || !batch_stride_ok(p.b0, p.b_b0, es) ||
      !batch_stride_ok(p.b1, p.b_b1, es) || !batch_stride_ok(p.red, p.b_red, es))
    return pl;
  pl.ok = true;
  return pl;
}

// 5-D map of an MN-major operand seen as (CH, K, MN/CH, x, y): element (e, k, c) sits at
// (c*CH + e) + k*ld.  box = [CH, BK, chunks, 1, 1]: one TMA brings all column chunks of a tile.
int encode_map_mn5(CUtensorMap* map, const void* base, size_t esize, int64_t mn, int64_t k, int64_t ld,
                   int64_t xn, int64_t xs, int64_t yn, int64_t ys, uint32_t ch, uint32_t bk, uint32_t chunks,
                   CUtensorMapSwizzle sw) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return B200_ERR_CUDA;
  const cuuint64_t dims[5] = {ch, (cuuint64_t)k, (cuuint64_t)(mn / ch), (cuuint64_t)(xn > 0 ? xn : 1),
                              (cuuint64_t)(yn > 0 ? yn : 1)};
  const uint64_t ldb = (uint64_t)ld * esize;
  const uint64_t xsb = (dims[3] > 1) ? (uint64_t)xs * esize : ldb;
  const uint64_t ysb = (dims[4] > 1) ? (uint64_t)ys * esize : ldb;
  const cuuint64_t strides[4] = {ldb, (cuuint64_t)ch * esize, xsb, ysb};
  const cuuint32_t box[5] = {ch, bk, chunks, 1, 1};
  const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  const CUtensorMapDataType dt = (esize == 2) ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  const CUresult r = fn(map, dt, 5, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? B200_OK : B200_ERR_UNSUPPORTED;
}

// 4-D map [inner (unit stride), outer (ld), x, y]; box = [box_inner, box_outer, 1, 1].
int encode_map(CUtensorMap* map, const void* base, size_t esize, int64_t inner, int64_t outer, int64_t ld,
               int64_t xn, int64_t xs, int64_t yn, int64_t ys, uint32_t box_inner, uint32_t box_outer,
               CUtensorMapSwizzle sw) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return B200_ERR_CUDA;
  const cuuint64_t dims[4] = {(cuuint64_t)inner, (cuuint64_t)outer, (cuuint64_t)(xn > 0 ? xn : 1),
                              (cuuint64_t)(yn > 0 ? yn : 1)};
  const uint64_t ldb = (uint64_t)ld * esize;
  // Size-1 dimensions still need a legal (multiple-of-16, non-zero) stride.
  const uint64_t xsb = (dims[2] > 1) ? (uint64_t)xs * esize : ldb;
  const uint64_t ysb = (dims[3] > 1) ? (uint64_t)ys * esize : ldb;
  const cuuint64_t strides[3] = {ldb, xsb, ysb};
  const cuuint32_t box[4] = {box_inner, box_outer, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUtensorMapDataType dt = (esize == 2) ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  const CUresult r = fn(map, dt, 4, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? B200_OK : B200_ERR_UNSUPPORTED;
}

// Process-wide testing / profiling knobs.  Atomics: a thread may change one while another thread launches.
std::atomic<int> g_xform_mode{1};
std::atomic<int> g_force_bn{0};   // 0 = choose by problem shape
std::atomic<int> g_mn_box5{1};    // MN-major operands: one 5-D TMA box per stage where the extent allows
std::mutex g_split_mutex;
std::atomic<int> g_split_mode{0}; // split-K of the f32 kernel: 0 = choose, 1 = never, n >= 2 = force n slices (testing)
std::atomic<int> g_store_mode{0}; // 0 = choose, 1 = row stores only, 2 = column stores where possible
std::atomic<int> g_capture_split{0}; // 1 = f16 split-K also on capturing streams (the caller orders graph replays)
std::atomic<int> g_max_ctas{0};   // upper bound on the persistent grids; 0 = one CTA per SM (b200_set_max_ctas)
std::atomic<long long> g_wait_limit{0}; // clock budget of every device-side wait; 0 = by problem size (testing)
std::atomic<int> g_pair_mode{1};  // 0 = choose by problem shape, 1 = never use CTA pairs (default: not faster yet), 2 = always (n > 128)

// Tensor maps and kernel arguments for a tile grid of TM x TN outputs per scheduling unit, where one
// CTA stages BMC rows of A and BNC columns of B per k-block of BK (MN-major operands in chunks of CH).
struct Launch {
  alignas(64) CUtensorMap ma, mb, mc;
  TcArgs g;
};

// SMs the persistent grids may occupy: all of them, unless the caller keeps some free for kernels that have to
// run beside a GEMM (a collective on another stream).
int grid_sms(const DeviceState* ds) {
  const int all = ds ? ds->sm_count : 148, cap = g_max_ctas.load();
  return (cap > 0 && cap < all) ? cap : all;
}

int build_launch(Launch& L, const Plan& pl, int esize, int tm, int tn, int bmc, int bnc, int bk, int ch) {
  const GemmProblem& p = pl.p;
  DeviceState* ds = device_state();
  if (!ds || !ds->ready) return B200_ERR_CUDA;

  // A is (m x k): cols_contig => K-major.  B is (k x n): cols_contig (n unit stride) => MN-major.
  const bool a_mn = !pl.la.cols_contig;
  const bool b_mn = pl.lb.cols_contig;
  const bool reduce = p.red > 1;
  // x / y batch dimensions of each operand map and the coordinate multipliers the kernel applies.
  const int64_t a_xn = reduce ? (p.a_red ? p.red : 1) : (p.a_b1 ? p.b1 : 1), a_xs = reduce ? p.a_red : p.a_b1;
  const int64_t b_xn = reduce ? (p.b_red ? p.red : 1) : (p.b_b1 ? p.b1 : 1), b_xs = reduce ? p.b_red : p.b_b1;
  const int64_t a_yn = reduce ? 1 : (p.a_b0 ? p.b0 : 1), b_yn = reduce ? 1 : (p.b_b0 ? p.b0 : 1);

  // Swizzle of the shared-memory tile: f16 128B everywhere; f32 64B for K-major rows, 128B with 32-byte
  // atoms for MN-major chunks.
  const CUtensorMapSwizzle sw_k = (esize == 2) ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  const CUtensorMapSwizzle sw_mn = (esize == 2) ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B;

  // MN-major operands whose MN extent is a whole number of chunks come in with one 5-D box per stage
  // (a partial last chunk would make that box read past the end of a row).
  const int a_ld = !a_mn ? 0 : ((p.m % ch == 0 && g_mn_box5) ? 2 : 1);
  const int b_ld = !b_mn ? 0 : ((p.n % ch == 0 && g_mn_box5) ? 2 : 1);
  int st;
  if (a_ld == 0)      st = encode_map(&L.ma, p.a, esize, p.k, p.m, pl.la.ld, a_xn, a_xs, a_yn, p.a_b0, bk, bmc, sw_k);
  else if (a_ld == 1) st = encode_map(&L.ma, p.a, esize, p.m, p.k, pl.la.ld, a_xn, a_xs, a_yn, p.a_b0, ch, bk, sw_mn);
  else                st = encode_map_mn5(&L.ma, p.a, esize, p.m, p.k, pl.la.ld, a_xn, a_xs, a_yn, p.a_b0, ch, bk,
                                          bmc / ch, sw_mn);
  if (st) return st;
  if (b_ld == 0)      st = encode_map(&L.mb, p.b, esize, p.k, p.n, pl.lb.ld, b_xn, b_xs, b_yn, p.b_b0, bk, bnc, sw_k);
  else if (b_ld == 1) st = encode_map(&L.mb, p.b, esize, p.n, p.k, pl.lb.ld, b_xn, b_xs, b_yn, p.b_b0, ch, bk, sw_mn);
  else                st = encode_map_mn5(&L.mb, p.b, esize, p.n, p.k, pl.lb.ld, b_xn, b_xs, b_yn, p.b_b0, ch, bk,
                                          bnc / ch, sw_mn);
  if (st) return st;

  TcArgs& g = L.g;
  g.m = (int)p.m; g.n = (int)p.n;
  g.m_tiles = (int)((p.m + tm - 1) / tm);
  g.n_tiles = (int)((p.n + tn - 1) / tn);
  g.nb1 = (int)p.b1;
  // Walk the dimension with fewer tiles fastest: the CTAs of one wave then share as many operand panels as
  // possible (an A panel is consumed by all its N tiles at once), which keeps DRAM reads near one pass.
  g.n_fast = g.n_tiles < g.m_tiles ? 1 : 0;
  g.total_tiles = (long long)g.m_tiles * g.n_tiles * p.b0 * p.b1;
  g.ksplit = 1; g.kb_per_slice = 0; g.total_units = g.total_tiles;   // launch_cfg fills the slice length
  g.tail_from = 0; g.tail_per = 0; g.tail_parts = 0; g.kt_cut = 0; g.kt_per = 0;
  g.streamk = 0; g.sk_per_cta = 0;
  g.red = (int)p.red;
  g.k_blocks = (int)((p.k + bk - 1) / bk);
  g.a_mn = a_mn; g.b_mn = b_mn;
  g.a_ld = a_ld; g.b_ld = b_ld;
  g.a_x1 = (!reduce && a_xn > 1) ? 1 : 0; g.a_xr = (reduce && a_xn > 1) ? 1 : 0; g.a_y0 = (a_yn > 1) ? 1 : 0;
  g.b_x1 = (!reduce && b_xn > 1) ? 1 : 0; g.b_xr = (reduce && b_xn > 1) ? 1 : 0; g.b_y0 = (b_yn > 1) ? 1 : 0;
  g.c = p.c; g.c_b0 = p.c_b0; g.c_b1 = p.c_b1; g.ldc = pl.ldc; g.c_col = pl.c_col;
  {
    const uint64_t es = (uint64_t)esize;
    const bool wide = !pl.c_col && ((uintptr_t)p.c % 32 == 0) && ((uint64_t)pl.ldc * es % 32 == 0) &&
                      (p.b0 <= 1 || (uint64_t)p.c_b0 * es % 32 == 0) && (p.b1 <= 1 || (uint64_t)p.c_b1 * es % 32 == 0);
    g.c_wide = wide ? 1 : 0;
  }
  g.c_tma = 0;
  L.mc = L.ma;                                               // a valid descriptor even when it is not used
  if (!pl.c_col && g_store_mode != 1 && (tm == BM || tm == 2 * BM)) {
    // output map (n, m, b1, b0), box 128 bytes x 128 rows, 128B swizzle: the epilogue stages groups of 64 f16 or
    // 32 f32 columns
    if (encode_map(&L.mc, p.c, esize, p.n, p.m, pl.ldc, p.b1, p.c_b1, p.b0, p.c_b0, 128 / esize, 128,
                   CU_TENSOR_MAP_SWIZZLE_128B) == B200_OK)
      g.c_tma = p.beta ? 2 : 1;
  }
  g.beta = p.beta;
  g.fused = p.fused() ? 1 : 0; g.alpha = (float)p.alpha; g.bias = p.bias; g.bias_row = p.bias_dim ? 1 : 0; g.act = p.act;
  g.acc32 = 0;
  g.xform_mode = g_xform_mode;
  g.tile_cols = tn; g.tile_valid = tn; g.mma_n = tn; g.b_tx_bytes = 0;
  g.cv_cblocks = 1; g.cv_cpad = 16; g.cv_kw = 1; g.cv_taps = 1; g.cv_w0 = g.cv_dw = g.cv_h0 = g.cv_dh = 0;
  g.cv_rows = 1; g.cv_wout = 1; g.cv_wblocks = 1; g.cv_bw = 16; g.cv_bh = 1; g.m64 = 0;
  const long long forced_limit = g_wait_limit.load();
  g.wait_limit = forced_limit > 0 ? forced_limit : 400000000LL + (long long)g.red * g.k_blocks * 40000LL;
  g.status = ds->status;
  return B200_OK;
}

// Tail split (f32 kernel, see TcArgs): decides whether the tiles of the last, partial wave are cut along K, fills
// the arguments and, for outputs that are written rather than added to, zeroes those tiles (they are then summed
// atomically).  Only for row-major outputs without a fused epilogue; at most MAX_ZEROED tiles are zeroed.
constexpr int TAIL_MAX_ZEROED = 8;
struct TailTiles { float* p[TAIL_MAX_ZEROED]; int rows[TAIL_MAX_ZEROED], cols[TAIL_MAX_ZEROED]; };
// Zeroes up to TAIL_MAX_ZEROED output tiles (blockIdx.x: tile, rows x cols floats, row pitch ldc; blockIdx.y: a
// group of 8 of its rows) in one launch.
__global__ void __launch_bounds__(256) zero_tiles_kernel(const TailTiles t, long long ldc) {
  float* p = t.p[blockIdx.x];
  const int rows = t.rows[blockIdx.x], cols = t.cols[blockIdx.x];
  const int r = blockIdx.y * 8 + (threadIdx.x >> 5);
  if (r >= rows) return;
  float* row = p + (long long)r * ldc;
  for (int c = threadIdx.x & 31; c < cols; c += 32) row[c] = 0.f;
}
std::atomic<int> g_tail_mode{0};   // 0 = choose, 1 = never (testing)

int plan_tail_split(TcArgs& g, int sms, int total_kb, cudaStream_t stream) {
  if (g_tail_mode.load() == 1 || g.ksplit != 1 || g.streamk || g.fused || g.c_col) return B200_OK;
  const long long full = g.total_tiles / sms, rem = g.total_tiles % sms;
  if (rem == 0) return B200_OK;
  if (full < 1) {
    // Less than one round of tiles (and more than half of one: fewer take the K split), an output that is added to (a
    // gradient: no tile needs a zero fill first).  CTA c < tiles computes k-blocks [0, cut) of tile c; the CTAs that
    // would idle share out the tiles' last total - cut k-blocks, `per` tiles each, and add their sums to the same
    // output.  (Dealing out one contiguous range of the whole (tile, k-block) space per CTA, as for a tail, puts every
    // CTA at a different K position at any time: no two of them share an operand panel in L2 any more and the launch
    // becomes DRAM-bound -- measured: no gain at all.)
    if (!g.beta || 2 * rem < sms) return B200_OK;
    const long long extra = sms - rem, per = (rem + extra - 1) / extra;
    const double fixed = 8.0;                              // k-blocks a unit costs beside its main loop (4 .. 16 measure alike)
    const long long cut = (long long)((per * (double)total_kb + fixed * per) / (1.0 + per)) + 1;   // cut ~ per * (total - cut + fixed)
    if (cut >= total_kb || total_kb - cut < 4) return B200_OK;
    if ((double)cut + fixed > 0.95 * ((double)total_kb + fixed)) return B200_OK;
    g.kt_cut = (int)cut; g.kt_per = (int)per;
    g.total_units = (long long)sms * per;
    return B200_OK;
  }
  if (!g.beta && rem > TAIL_MAX_ZEROED) return B200_OK;
  // one contiguous range of the tail's (tile, k-block) space per CTA; at least four k-blocks per range
  long long per = (rem * total_kb + sms - 1) / sms;
  if (per < 4) per = 4;
  if (per >= total_kb) return B200_OK;
  const int parts = 2;                                     // a range shorter than a tile touches at most two tiles
  // cost in k-blocks per SM; a unit costs about 8 k-blocks beside its main loop (pipeline fill, epilogue)
  const double fixed = 8.0, before = (double)(full + 1) * (total_kb + fixed),
               after = full * (total_kb + fixed) + (double)per + 2 * fixed;
  if (after > 0.95 * before) return B200_OK;
  g.tail_from = full * sms; g.tail_per = (int)per; g.tail_parts = parts;
  g.total_units = g.tail_from + (long long)sms * parts;
  if (!g.beta) {
    const long long per_batch = (long long)g.m_tiles * g.n_tiles;
    TailTiles tt;
    int cnt = 0;
    for (long long tile = g.tail_from; tile < g.total_tiles; ++tile, ++cnt) {
      const long long bt = tile / per_batch;
      const int r = (int)(tile - bt * per_batch);
      const int nt = g.n_fast ? r % g.n_tiles : r / g.m_tiles, mt = g.n_fast ? r / g.n_tiles : r % g.m_tiles;
      const long long ib1 = bt % g.nb1, ib0 = bt / g.nb1;
      const long long col0 = (long long)nt * g.tile_cols;
      tt.cols[cnt] = (int)(g.n - col0 < g.tile_valid ? g.n - col0 : g.tile_valid);
      tt.rows[cnt] = (int)(g.m - (long long)mt * BM < BM ? g.m - (long long)mt * BM : BM);
      tt.p[cnt] = (float*)g.c + ib0 * g.c_b0 + ib1 * g.c_b1 + (long long)mt * BM * g.ldc + col0;
    }
    zero_tiles_kernel<<<dim3((unsigned)cnt, BM / 8), 256, 0, stream>>>(tt, g.ldc);
    const int rc = note_cuda_error(cudaGetLastError(), "zero_tiles launch");
    if (rc) return rc;
  }
  return B200_OK;
}

// f16 split-K: `launch_main(scratch, lds)` launches a kernel whose K slices add f32 partial sums into the device's
// zeroed scratch matrix (m rows of lds floats); a second kernel then folds the scratch into C.  *done stays false
// (and nothing is enqueued) when the scratch cannot be used: too small, or the stream is capturing -- the one scratch
// per device is ordered across streams by an event that is recorded eagerly, and a replayed graph would neither wait
// on it nor record it.  A caller that orders every replay of its graphs against all other work of the library on
// the device (one stream, say) may ask for split-K inside captures (b200_set_capture_split_k); the event is then left
// alone.
template <typename Fn>
int run_f16_split(const Plan& pl, cudaStream_t stream, bool* done, Fn launch_main) {
  const GemmProblem& p = pl.p;   // single batch item (checked by the caller)
  DeviceState* ds = device_state();
  *done = false;
  const long long lds = (p.n + 3) / 4 * 4;
  const size_t need = (size_t)p.m * (size_t)lds * sizeof(float);
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess) cap = cudaStreamCaptureStatusActive;
  const bool capturing = cap != cudaStreamCaptureStatusNone;
  if (need > ds->split_scratch_bytes || (capturing && !g_capture_split.load())) return B200_OK;
  std::lock_guard<std::mutex> lock(g_split_mutex);
  int rc;
  // Order this use after the previous one when that ran on another stream.
  if (!capturing && ds->split_used && ds->split_last_stream != stream &&
      (rc = note_cuda_error(cudaStreamWaitEvent(stream, ds->split_event, 0), "cudaStreamWaitEvent(split-K)")))
    return rc;
  if ((rc = note_cuda_error(cudaMemsetAsync(ds->split_scratch, 0, need, stream), "cudaMemsetAsync(split-K)"))) return rc;
  *done = true;
  if ((rc = launch_main(ds->split_scratch, lds))) return rc;
  const long long total = (long long)p.m * p.n;
  long long blocks = (total + 255) / 256;
  if (blocks > (long long)ds->sm_count * 8) blocks = (long long)ds->sm_count * 8;
  const long long c_r = pl.c_col ? 1 : pl.ldc, c_c = pl.c_col ? pl.ldc : 1;
  splitk_finalize_f16_kernel<<<(unsigned)blocks, 256, 0, stream>>>(ds->split_scratch, lds, (__half*)p.c, c_r, c_c,
                                                                   (int)p.m, (int)p.n, p.beta);
  count_launch(false);
  if ((rc = note_cuda_error(cudaGetLastError(), "split-K finalize launch"))) return rc;
  if (capturing) return B200_OK;
  ds->split_used = true;
  ds->split_last_stream = stream;
  return note_cuda_error(cudaEventRecord(ds->split_event, stream), "cudaEventRecord(split-K)");
}

// C: CfgH<BN> or CfgS<BN>; KERNEL: the matching kernel.  ksplit > 1 (f32 kernel only): K is cut into that many
// slices, each (tile, slice) is a work unit and the slices' partial results are added into C atomically; for
// beta = 0 the output is zeroed first.
template <typename C, int ESIZE, int BN, typename Kernel>
int launch_cfg(const Plan& pl, cudaStream_t stream, Kernel kernel, int ksplit) {
  Launch L;
  const int st = build_launch(L, pl, ESIZE, BM, BN, BM, BN, C::BK, C::CH);
  if (st) return st;
  DeviceState* ds = device_state();
  TcArgs& g = L.g;
  const int total_kb = g.red * g.k_blocks;
  g.kb_per_slice = total_kb;
  g.split_out = nullptr; g.split_ld = 0;
  if (ksplit == -1 && ESIZE == 4) {
    // stream-K: one contiguous range of the (tile, k-block) space per CTA, so that every SM gets the same amount
    // of work when the tile count is not a multiple of the SM count; tiles cut by a range boundary are summed
    // atomically (beta = 0 outputs are zeroed first)
    const GemmProblem& p = pl.p;
    const long long all = g.total_tiles * (long long)total_kb;
    const long long grid = grid_sms(ds);
    g.streamk = 1;
    g.sk_per_cta = (all + grid - 1) / grid;
    const long long per_cta_tiles = (g.sk_per_cta + total_kb - 1) / total_kb + 1;      // tiles a range can touch
    g.total_units = grid * per_cta_tiles;
    if (!g.beta) {
      const size_t width = (size_t)(pl.c_col ? p.m : p.n) * 4, height = (size_t)(pl.c_col ? p.n : p.m);
      const int rc = note_cuda_error(cudaMemset2DAsync(p.c, (size_t)pl.ldc * 4, 0, width, height, stream),
                                     "cudaMemset2DAsync(stream-K output)");
      if (rc) return rc;
    }
  } else if (ksplit > 1 && total_kb >= 2 * ksplit) {
    const GemmProblem& p = pl.p;   // single batch item (checked by the caller)
    const int kb_per = (total_kb + ksplit - 1) / ksplit, slices = (total_kb + kb_per - 1) / kb_per;
    if (ESIZE == 4 && slices > 1) {
      g.kb_per_slice = kb_per; g.ksplit = slices; g.total_units = g.total_tiles * slices;
      if (!g.beta) {
        const size_t width = (size_t)(pl.c_col ? p.m : p.n) * 4, height = (size_t)(pl.c_col ? p.n : p.m);
        const int rc = note_cuda_error(cudaMemset2DAsync(p.c, (size_t)pl.ldc * 4, 0, width, height, stream),
                                       "cudaMemset2DAsync(split-K output)");
        if (rc) return rc;
      }
    } else if (ESIZE == 2 && slices > 1) {
      bool done = false;
      const int rc = run_f16_split(pl, stream, &done, [&](float* scratch, long long lds) {
        g.kb_per_slice = kb_per; g.ksplit = slices; g.total_units = g.total_tiles * slices;
        g.split_out = scratch; g.split_ld = lds;
        const long long grid2 = g.total_units < grid_sms(ds) ? g.total_units : grid_sms(ds);
        L.g.c_tma = 0;                                       // partial sums go to the scratch, not to C
        kernel<<<(unsigned)grid2, C::THREADS, C::SMEM_BYTES, stream>>>(L.ma, L.mb, L.mc, L.g);
        count_launch(true);
        return note_cuda_error(cudaGetLastError(), "tensor-core gemm launch");
      });
      if (rc || done) return rc;
    }
  }
  if constexpr (ESIZE == 4) {
    const int rc = plan_tail_split(g, grid_sms(ds), total_kb, stream);
    if (rc) return rc;
  }
  const long long grid = g.total_units < grid_sms(ds) ? g.total_units : grid_sms(ds);
  if (grid <= 0) return B200_OK;
  kernel<<<(unsigned)grid, C::THREADS, C::SMEM_BYTES, stream>>>(L.ma, L.mb, L.mc, L.g);
  count_launch(true);
  return note_cuda_error(cudaGetLastError(), "tensor-core gemm launch");
}

// CTA-pair kernels (gemm_tc_pair.cu): 256 x 256 tiles, each CTA stages 128 rows of A and 128 columns of B.
int launch_pair_plan(const Plan& pl, int esize, cudaStream_t stream) {
  Launch L;
  const int tm = pair_tile_m(), tn = pair_tile_n();
  const int st = build_launch(L, pl, esize, tm, tn, tm / 2, tn / 2, pair_block_k(esize), pair_chunk(esize));
  if (st) return st;
  return launch_pair(esize, L.ma, L.mb, L.g, grid_sms(device_state()), stream);
}

// f16, 256 x 256 tiles (gemm_f16_big_kernel).  ksplit == 1: whole-K tiles; returns B200_ERR_UNSUPPORTED when the
// output cannot leave through the staged TMA store (the only direct epilogue that kernel has).  ksplit > 1 (one batch
// item, no fused epilogue): K slices through the f32 scratch (run_f16_split), any output layout; returns
// B200_ERR_UNSUPPORTED when the scratch cannot be used.
int encode_map_f32(CUtensorMap* map, const void* base, const uint64_t dims[4], const uint64_t strides_b[3],
                   const uint32_t box[4], CUtensorMapSwizzle sw);
int launch_big_f16(const Plan& pl, cudaStream_t stream, int ksplit) {
  Launch L;
  const int st = build_launch(L, pl, 2, CfgHB::BMB, CfgHB::BN, CfgHB::BMB, CfgHB::BN, CfgHB::BK, CfgHB::CH);
  if (st) return st;
  DeviceState* ds = device_state();
  TcArgs& g = L.g;
  const int total_kb = g.red * g.k_blocks;
  g.kb_per_slice = total_kb;
  if (ksplit > 1 && total_kb >= 2 * ksplit) {
    const int kb_per = (total_kb + ksplit - 1) / ksplit, slices = (total_kb + kb_per - 1) / kb_per;
    bool done = false;
    const int rc = run_f16_split(pl, stream, &done, [&](float* scratch, long long lds) {
      // the scratch as a (columns, rows) f32 tensor: boxes of 32 columns (one swizzled 128-byte line) x 128 rows
      const uint64_t dims[4] = {(uint64_t)lds, (uint64_t)pl.p.m, 1, 1};
      const uint64_t strides[3] = {(uint64_t)lds * 4, (uint64_t)lds * 4 * (uint64_t)pl.p.m, (uint64_t)lds * 4 * (uint64_t)pl.p.m};
      const uint32_t box[4] = {32, (uint32_t)BM, 1, 1};
      const int er = encode_map_f32(&L.mc, scratch, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
      if (er) return er;
      g.kb_per_slice = kb_per; g.ksplit = slices; g.total_units = g.total_tiles * slices;
      g.split_out = scratch; g.split_ld = lds;
      const long long grid2 = g.total_units < grid_sms(ds) ? g.total_units : grid_sms(ds);
      gemm_f16_big_kernel<<<(unsigned)grid2, CfgHB::THREADS, CfgHB::SMEM_BYTES, stream>>>(L.ma, L.mb, L.mc, L.g);
      count_launch(true);
      return note_cuda_error(cudaGetLastError(), "tensor-core gemm launch (256 x 256 tiles, K slices)");
    });
    if (rc) return rc;
    return done ? B200_OK : B200_ERR_UNSUPPORTED;
  }
  if (!g.c_tma) return B200_ERR_UNSUPPORTED;
  const long long grid = g.total_units < grid_sms(ds) ? g.total_units : grid_sms(ds);
  if (grid <= 0) return B200_OK;
  gemm_f16_big_kernel<<<(unsigned)grid, CfgHB::THREADS, CfgHB::SMEM_BYTES, stream>>>(L.ma, L.mb, L.mc, L.g);
  count_launch(true);
  return note_cuda_error(cudaGetLastError(), "tensor-core gemm launch (256 x 256 tiles)");
}

// f16 operands, f32 destination that is added to (GemmProblem::acc32): 256 x 256 tiles whose accumulators leave as
// bulk reduce-adds into C itself, whole-K tiles or K slices alike -- no scratch, no zero fill, no second kernel.
int launch_big_f16_acc32(const Plan& pl, cudaStream_t stream) {
  const GemmProblem& p = pl.p;
  if (pl.c_col || p.b0 != 1 || p.b1 != 1 || p.fused() || (pl.ldc % 4) || ((uintptr_t)p.c & 15)) return B200_ERR_UNSUPPORTED;
  Launch L;
  const int st = build_launch(L, pl, 2, CfgHB::BMB, CfgHB::BN, CfgHB::BMB, CfgHB::BN, CfgHB::BK, CfgHB::CH);
  if (st) return st;
  DeviceState* ds = device_state();
  const int sms = grid_sms(ds);
  TcArgs& g = L.g;
  const int total_kb = g.red * g.k_blocks;
  // K slices by the same model as the scratch route: per 64-wide k-block 0.6 us, per unit about 10 us beside it
  int slices = 1;
  {
    double t_best = (double)((g.total_tiles + sms - 1) / sms) * ((double)total_kb * 0.6 + 10.0);
    for (int s_ = 2; s_ <= 64; ++s_) {
      if (total_kb / s_ < 8) break;
      const double waves = (double)((g.total_tiles * s_ + sms - 1) / sms);
      const double t = waves * ((double)((total_kb + s_ - 1) / s_) * 0.6 + 10.0);
      if (t < 0.85 * t_best) { t_best = t; slices = s_; }
    }
  }
  const int kb_per = (total_kb + slices - 1) / slices;
  slices = (total_kb + kb_per - 1) / kb_per;
  const uint64_t dims[4] = {(uint64_t)p.n, (uint64_t)p.m, 1, 1};
  const uint64_t strides[3] = {(uint64_t)pl.ldc * 4, (uint64_t)pl.ldc * 4 * (uint64_t)p.m, (uint64_t)pl.ldc * 4 * (uint64_t)p.m};
  const uint32_t box[4] = {32, (uint32_t)BM, 1, 1};
  const int er = encode_map_f32(&L.mc, p.c, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
  if (er) return er;
  g.acc32 = 1; g.c_tma = 0; g.beta = 1;
  g.kb_per_slice = kb_per; g.ksplit = slices; g.total_units = g.total_tiles * slices;
  g.split_out = nullptr; g.split_ld = 0;
  const long long grid = g.total_units < sms ? g.total_units : sms;
  if (grid <= 0) return B200_OK;
  gemm_f16_big_kernel<<<(unsigned)grid, CfgHB::THREADS, CfgHB::SMEM_BYTES, stream>>>(L.ma, L.mb, L.mc, L.g);
  count_launch(true);
  return note_cuda_error(cudaGetLastError(), "tensor-core gemm launch (f32 destination)");
}

template <int ESIZE, int BN>
int launch_bn(const Plan& pl, cudaStream_t stream, int ksplit) {
  if constexpr (ESIZE == 2) return launch_cfg<CfgH<BN>, 2, BN>(pl, stream, gemm_f16_kernel<BN>, ksplit);
  else return launch_cfg<CfgS<BN>, 4, BN>(pl, stream, gemm_tf32x3_kernel<BN>, ksplit);
}

// Tile width by a wave model: time ~ ceil(tiles / SMs) * (cost of one tile of that width).  The relative
// per-tile costs are measured (a 128-wide tile takes about 3/4 of the time of a 256-wide one because its
// main loop is bound by shared-memory traffic, not by the tensor pipe).  Returns the modelled cost.
double choose_tile(const Plan& pl, int esize, int* bn_out) {
  const GemmProblem& p = pl.p;
  DeviceState* ds = device_state();
  const int sms = grid_sms(ds);
  auto tiles = [&](int bn) { return ((p.m + BM - 1) / BM) * ((p.n + bn - 1) / bn) * p.b0 * p.b1; };
  const double w256 = 1.0, w128 = (esize == 4) ? 0.75 : 0.87, w64 = (esize == 4) ? 0.55 : 0.70;
  auto waves = [&](int bn_) { return (double)((tiles(bn_) + sms - 1) / sms); };
  int bn = 64;
  double best = waves(64) * w64;
  if (p.n > 64 && waves(128) * w128 <= best) { best = waves(128) * w128; bn = 128; }
  if (p.n > 128 && waves(256) * w256 <= best) { best = waves(256) * w256; bn = 256; }
  *bn_out = bn;
  return best;
}

template <int ESIZE>
int launch_es(const Plan& pl, cudaStream_t stream) {
  const GemmProblem& p = pl.p;
  DeviceState* ds = device_state();
  const int sms = grid_sms(ds);
  int bn = 64;
  const double best = choose_tile(pl, ESIZE, &bn);
  const int g_force_bn = b200::g_force_bn.load(), g_pair_mode = b200::g_pair_mode.load(),
            g_split_mode = b200::g_split_mode.load();     // one read per launch
  if (g_force_bn && g_force_bn != 512) bn = g_force_bn;
  // f16: 256 x 256 tiles per CTA where a wave model says they win (their main loop keeps the tensor pipe busier, but
  // nothing overlaps their epilogue): measured per 64-wide k-block 0.55 us for a 128 x 256 tile against 0.83 us for a
  // 256 x 256 one, and per tile about 1 us against 3.7 us beside the main loop.
  if constexpr (ESIZE == 2) {
    if ((g_force_bn == 0 || g_force_bn == 512) && !pl.c_col && p.m > BM && p.n > 128 && b200::g_store_mode.load() != 1) {
      const int64_t kb = p.red * ((p.k + 63) / 64);
      const int64_t t_small = ((p.m + BM - 1) / BM) * ((p.n + 255) / 256) * p.b0 * p.b1;
      const int64_t t_big = ((p.m + 255) / 256) * ((p.n + 255) / 256) * p.b0 * p.b1;
      const double c_small = (double)((t_small + sms - 1) / sms) * ((double)kb * 0.55 + 1.0);
      const double c_big = (double)((t_big + sms - 1) / sms) * ((double)kb * 0.83 + 3.7);
      // below about two thirds of a wave of big tiles the K split of the small-tile kernel is the better tool
      const bool forced_slices = g_force_bn == 512 && g_split_mode >= 2;   // testing: K slices of big tiles, below
      if (!forced_slices && (g_force_bn == 512 || (bn == 256 && 3 * t_big >= 2 * sms && c_big < 0.9 * c_small))) {
        const int rc = launch_big_f16(pl, stream, 1);
        if (rc != B200_ERR_UNSUPPORTED) return rc;
      }
    }
  }
  if (g_force_bn == 512) bn = 256;
  // CTA pairs (256 x 256 tiles on two SMs) when the problem fills the machine with them.
  if (!g_force_bn && g_pair_mode != 1 && p.n > 128 && !p.fused()) {   // the pair kernels have no fused epilogue
    const int64_t tiles2 = ((p.m + 255) / 256) * ((p.n + 255) / 256) * p.b0 * p.b1;
    const int64_t pairs = sms / 2;
    const double cost2 = (double)((tiles2 + pairs - 1) / pairs) * 0.8;   // a pair wave of 256x256 tiles vs a wave of 128x256 tiles
    if (g_pair_mode == 2 || (p.m > 128 && cost2 <= best)) return launch_pair_plan(pl, ESIZE, stream);
  }
  // Split-K (f32, one batch item): when the tiles alone leave most SMs idle, K slices become extra work
  // units.  Model: time = waves * (k-blocks per unit * t_kb(tile width) + t_fixed), in microseconds.
  int ksplit = 1;
  if (g_split_mode != 1 && p.b0 == 1 && p.b1 == 1 && !p.fused()) {   // a fused epilogue needs the whole sum in one unit
    const int bk = (ESIZE == 4) ? 16 : 64;
    const int64_t total_kb = p.red * ((p.k + bk - 1) / bk);
    auto model = [&](int bn_, int s_) {
      const int64_t tiles = ((p.m + BM - 1) / BM) * ((p.n + bn_ - 1) / bn_);
      const double t_kb = (ESIZE == 4) ? (bn_ == 256 ? 0.65 : (bn_ == 128 ? 0.48 : 0.36))
                                       : (bn_ == 256 ? 0.52 : (bn_ == 128 ? 0.42 : 0.36));
      const double waves = (double)((tiles * s_ + sms - 1) / sms);
      return waves * ((double)((total_kb + s_ - 1) / s_) * t_kb + 4.0 + (s_ > 1 ? 2.0 : 0.0));
    };
    double best_t = model(bn, 1);
    const int widths[3] = {256, 128, 64};
    for (int wi = 0; wi < 3; ++wi) {
      const int bn_ = widths[wi];
      if ((bn_ == 256 && p.n <= 128) || (bn_ == 128 && p.n <= 64) || (g_force_bn && bn_ != g_force_bn)) continue;
      for (int s_ = 2; s_ <= 64; ++s_) {
        if (total_kb / s_ < (ESIZE == 4 ? 16 : 8)) break;    // keep slices long enough to amortise their fixed cost
        const double t = model(bn_, s_);
        if (t < 0.85 * best_t) { best_t = t; bn = bn_; ksplit = s_; }
      }
    }
    // f16: K slices of 256 x 256 tiles.  Per 64-wide k-block 0.6 us in a long main loop; per unit about 10 us beside it
    // (pipeline fill and the 256 KB of f32 partial sums that leave through bulk reduce-adds, which nothing overlaps).
    if constexpr (ESIZE == 2) {
      const bool forced_slices = g_force_bn == 512 && g_split_mode >= 2;
      if (forced_slices) {
        const int rc = launch_big_f16(pl, stream, g_split_mode);
        if (rc != B200_ERR_UNSUPPORTED) return rc;
      } else if (g_force_bn == 0 && g_split_mode <= 0 && p.m > BM && p.n > 128 && b200::g_store_mode.load() != 1) {
        const int64_t t_big = ((p.m + 255) / 256) * ((p.n + 255) / 256);
        int s_best = 0;
        double t_best = 0.85 * best_t;
        for (int s_ = 2; s_ <= 64; ++s_) {
          if (total_kb / s_ < 8) break;
          const double waves = (double)((t_big * s_ + sms - 1) / sms);
          const double t = waves * ((double)((total_kb + s_ - 1) / s_) * 0.6 + 10.0);
          if (t < t_best) { t_best = t; s_best = s_; }
        }
        if (s_best) {
          const int rc = launch_big_f16(pl, stream, s_best);
          if (rc != B200_ERR_UNSUPPORTED) return rc;
        }
      }
    }
    if (g_split_mode >= 2) ksplit = g_split_mode;           // testing: force this many slices
    // Stream-K (f32) is built and tested but only taken on request (b200_set_split_k(-1)): on the benchmark's
    // backward GEMMs it measured -6 % (512 tiles, 3.46 waves) and +4 % (128 tiles: every tile becomes a pair of
    // atomically summed halves), and it makes the gradient's last bits depend on scheduling.
    if (g_split_mode == -1) ksplit = ESIZE == 4 ? -1 : 1;
  }
  switch (bn) {
    case 256: return launch_bn<ESIZE, 256>(pl, stream, ksplit);
    case 128: return launch_bn<ESIZE, 128>(pl, stream, ksplit);
    default: return launch_bn<ESIZE, 64>(pl, stream, ksplit);
  }
}

template <typename C, typename Kernel>
int set_attr(Kernel kernel) {
  return note_cuda_error(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES),
                         "cudaFuncSetAttribute");
}

}  // namespace

// ---------------------------------------------------------------------------------------------
// Implicit-GEMM convolution: tensor maps and launch (kernels: gemm_tf32x3_kernel<256, 1> and <256, 2>)
// ---------------------------------------------------------------------------------------------
namespace {

// 4-D f32 map with explicit extents, byte strides of dimensions 1..3 and box.
int encode_map_f32(CUtensorMap* map, const void* base, const uint64_t dims[4], const uint64_t strides_b[3],
                   const uint32_t box[4], CUtensorMapSwizzle sw) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return B200_ERR_CUDA;
  cuuint64_t d[4], st[3];
  cuuint32_t bx[4], es[4] = {1, 1, 1, 1};
  for (int i = 0; i < 4; ++i) { d[i] = dims[i] ? dims[i] : 1; bx[i] = box[i]; }
  for (int i = 0; i < 3; ++i) st[i] = strides_b[i];
  // size-1 dimensions still need a legal (multiple-of-16, non-zero) stride
  for (int i = 0; i < 3; ++i)
    if (d[i + 1] == 1 && (st[i] == 0 || st[i] % 16)) st[i] = i ? st[i - 1] : 16;
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(base), d, st, bx, es,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? B200_OK : B200_ERR_UNSUPPORTED;
}

constexpr int CV_BN = 256;
using CvCfg = CfgS<CV_BN>;

// Image rows per N tile of the forward / data-gradient kernel: whole rows, at most 256 positions, a multiple of
// four positions (16-byte output accesses); among those the count that minimises waves x (per-tile cost).
int conv_rows_per_tile(const ConvImplicit& c, int sms) {
  const int64_t m_tiles = (c.m + BM - 1) / BM;
  int best = 0;
  double best_cost = 0;
  for (int r = 1; r * c.w_out <= CV_BN && r <= c.h_out; ++r) {
    if ((r * c.w_out) % 4) continue;
    const int64_t tiles = c.batch * c.groups * m_tiles * ((c.h_out + r - 1) / r);
    const double cost = (double)((tiles + sms - 1) / sms) * (64.0 + (double)(r * c.w_out));
    if (!best || cost < best_cost) { best = r; best_cost = cost; }
  }
  return best;
}

void cv_common_args(TcArgs& g, DeviceState* ds) {
  g.nb1 = 1; g.n_fast = 0;
  g.ksplit = 1; g.streamk = 0; g.sk_per_cta = 0; g.split_out = nullptr; g.split_ld = 0;
  g.tail_from = 0; g.tail_per = 0; g.tail_parts = 0; g.kt_cut = 0; g.kt_per = 0;
  g.red = 1;
  g.a_mn = 0; g.b_mn = 0; g.a_ld = 0; g.b_ld = 0;
  g.a_x1 = g.a_xr = g.a_y0 = g.b_x1 = g.b_xr = g.b_y0 = 0;
  g.c_b0 = g.c_b1 = 0; g.c_col = 0; g.c_wide = 0; g.c_tma = 0; g.beta = 0;
  g.xform_mode = g_xform_mode.load();
  g.status = ds->status;
  g.fused = 0; g.alpha = 1.f; g.bias = nullptr; g.bias_row = 0; g.act = B200_ACT_NONE; g.acc32 = 0;
  g.cv_cblocks = 1; g.cv_cpad = 16; g.cv_kw = 1; g.cv_taps = 1; g.cv_w0 = g.cv_dw = g.cv_h0 = g.cv_dh = 0;
  g.cv_rows = 1; g.cv_wout = 1; g.cv_wblocks = 1; g.cv_bw = 16; g.cv_bh = 1; g.m64 = 0;
}

}  // namespace

bool conv_implicit_ok(const ConvImplicit& c) {
  DeviceState* ds = device_state();
  if (!ds || !encode_fn()) return false;
  if (c.batch < 1 || c.groups < 1 || c.m < 1 || c.h_out < 1 || c.w_out < 1 || c.w_out > CV_BN) return false;
  if (c.cpad < 16 || c.cpad % 16 || c.kh < 1 || c.kw < 1) return false;
  const int64_t lim = 0x7fffff00LL;
  if (c.batch > lim || c.groups * c.cpad > lim || c.h_img > lim || c.w_img > lim || c.h_out * c.w_out > lim ||
      (int64_t)c.kh * c.kw * c.cpad > lim || c.m > lim || c.batch * c.groups > lim)
    return false;
  if (((uintptr_t)c.img_cl | (uintptr_t)c.filt | (uintptr_t)c.out) & 15) return false;
  if ((c.h_out * c.w_out) % 4) return false;                 // batch / channel strides of the output: 16 bytes
  return conv_rows_per_tile(c, grid_sms(ds)) > 0;
}

int launch_conv_implicit(const ConvImplicit& c, cudaStream_t stream) {
  DeviceState* ds = device_state();
  if (!ds || !ds->ready) return B200_ERR_CUDA;
  if (!conv_implicit_ok(c)) return B200_ERR_UNSUPPORTED;
  const int sms = grid_sms(ds);
  const int rows = conv_rows_per_tile(c, sms);
  const int64_t taps = (int64_t)c.kh * c.kw, kr = taps * c.cpad, npos = c.h_out * c.w_out, ct = c.groups * c.cpad;
  Launch L;
  // A: filters (groups, m, taps*cpad), K-major rows
  {
    const uint64_t dims[4] = {(uint64_t)kr, (uint64_t)c.m, (uint64_t)c.groups, 1};
    const uint64_t st[3] = {(uint64_t)kr * 4, (uint64_t)c.m * kr * 4, (uint64_t)c.groups * c.m * kr * 4};
    const uint32_t box[4] = {(uint32_t)CvCfg::BK, (uint32_t)(c.m <= 64 ? 64 : BM), 1, 1};
    const int rc = encode_map_f32(&L.ma, c.filt, dims, st, box, CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc) return rc;
  }
  // B: channels-last image (channel, x, y, image); one box = 16 channels x w_out pixels x `rows` image rows
  {
    const uint64_t dims[4] = {(uint64_t)ct, (uint64_t)c.w_img, (uint64_t)c.h_img, (uint64_t)c.batch};
    const uint64_t st[3] = {(uint64_t)ct * 4, (uint64_t)c.w_img * ct * 4, (uint64_t)c.h_img * c.w_img * ct * 4};
    const uint32_t box[4] = {(uint32_t)CvCfg::BK, (uint32_t)c.w_out, (uint32_t)rows, 1};
    const int rc = encode_map_f32(&L.mb, c.img_cl, dims, st, box, CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc) return rc;
  }
  TcArgs& g = L.g;
  cv_common_args(g, ds);
  g.m = (int)c.m; g.n = (int)npos;
  g.m_tiles = (int)((c.m + BM - 1) / BM);
  g.n_tiles = (int)((c.h_out + rows - 1) / rows);
  g.nb1 = (int)c.groups;
  g.total_tiles = (long long)g.m_tiles * g.n_tiles * c.batch * c.groups;
  g.total_units = g.total_tiles;
  g.k_blocks = (int)(taps * (c.cpad / CvCfg::BK));
  g.kb_per_slice = g.k_blocks;
  g.c = c.out; g.c_b0 = c.groups * c.m * npos; g.c_b1 = c.m * npos; g.ldc = npos;
  g.tile_cols = rows * (int)c.w_out; g.tile_valid = g.tile_cols;
  g.mma_n = (g.tile_cols + 15) / 16 * 16;
  g.b_tx_bytes = CvCfg::BK * 4 * g.tile_cols;
  g.c_wide = (g.tile_cols % 8 == 0 && npos % 8 == 0 && ((uintptr_t)c.out % 32 == 0)) ? 1 : 0;
  g.beta = c.beta ? 1 : 0;
  L.mc = L.ma;
  if (g_store_mode.load() != 1 &&
      encode_map(&L.mc, c.out, 4, npos, c.m, npos, c.groups, c.m * npos, c.batch, c.groups * c.m * npos, 32, 128,
                 CU_TENSOR_MAP_SWIZZLE_128B) == B200_OK)
    g.c_tma = g.beta ? 2 : 1;
  g.cv_cblocks = (int)(c.cpad / CvCfg::BK); g.cv_cpad = (int)c.cpad; g.cv_kw = c.kw; g.cv_taps = (int)taps;
  g.cv_w0 = c.w0; g.cv_dw = c.dw; g.cv_h0 = c.h0; g.cv_dh = c.dh;
  g.cv_rows = rows; g.cv_wout = (int)c.w_out;
  g.m64 = c.m <= 64 ? 1 : 0;
  const long long forced_limit = g_wait_limit.load();
  g.wait_limit = forced_limit > 0 ? forced_limit : 400000000LL + (long long)g.k_blocks * 40000LL;
  {
    const int rc = plan_tail_split(g, sms, g.k_blocks, stream);
    if (rc) return rc;
  }
  const long long grid = g.total_units < sms ? g.total_units : sms;
  if (grid <= 0) return B200_OK;
  gemm_tf32x3_kernel<CV_BN, 1><<<(unsigned)grid, CvCfg::THREADS, CvCfg::SMEM_BYTES, stream>>>(L.ma, L.mb, L.mc, L.g);
  count_launch(true);
  return note_cuda_error(cudaGetLastError(), "implicit convolution launch");
}

namespace {
// Width of the N tiles of the filter-gradient kernel: a multiple of 32 columns (one chunk = 32 channels of one tap),
// the one that covers taps*cpad columns with the least padding, then the widest.
int wgrad_tile_cols(int64_t kr) {
  int best = 32;
  int64_t best_pad = -1;
  for (int tc = CV_BN; tc >= 32; tc -= 32) {
    const int64_t padded = (kr + tc - 1) / tc * tc;
    if (best_pad < 0 || padded < best_pad) { best = tc; best_pad = padded; }
  }
  return best;
}
}  // namespace

bool conv_implicit_wgrad_ok(const ConvImplicitWgrad& c) {
  DeviceState* ds = device_state();
  if (!ds || !encode_fn()) return false;
  if (c.batch < 1 || c.m < 1 || c.h_out < 1 || c.w_out < 1 || c.w_out % 4) return false;
  if (c.cpad < 32 || c.cpad % 32 || c.c_total % 4 || c.kh < 1 || c.kw < 1 || c.gout_bs % 4) return false;
  const int64_t lim = 0x7fffff00LL;
  if (c.batch > lim || c.c_total > lim || c.h_img > lim || c.w_img > lim || c.h_out * c.w_out > lim ||
      (int64_t)c.kh * c.kw * c.cpad > lim || c.m > lim || c.h_out * c.w_out > lim / (c.batch > 0 ? c.batch : 1))
    return false;
  if (((uintptr_t)c.img_cl | (uintptr_t)c.gout | (uintptr_t)c.out) & 15) return false;
  return true;
}

int launch_conv_implicit_wgrad(const ConvImplicitWgrad& c, cudaStream_t stream) {
  DeviceState* ds = device_state();
  if (!ds || !ds->ready) return B200_ERR_CUDA;
  if (!conv_implicit_wgrad_ok(c)) return B200_ERR_UNSUPPORTED;
  const int sms = grid_sms(ds);
  const int64_t taps = (int64_t)c.kh * c.kw, kr = taps * c.cpad, npos = c.h_out * c.w_out;
  const int tile_cols = wgrad_tile_cols(kr);
  // A k-block is 16 pixels of one output row.  (Boxes of 8 x 2 or 4 x 4 pixels would waste less on ragged rows, but a
  // swizzled TMA box narrower than the swizzle span does not land in the dense layout the MMA descriptor expects.)
  const int bw = CvCfg::BK, bh = 1;
  Launch L;
  // A: grad_out of this group as (x, y, channel, image); one box = 16 pixels of one row x 128 channels
  {
    const uint64_t dims[4] = {(uint64_t)c.w_out, (uint64_t)c.h_out, (uint64_t)c.m, (uint64_t)c.batch};
    const uint64_t st[3] = {(uint64_t)c.w_out * 4, (uint64_t)npos * 4, (uint64_t)c.gout_bs * 4};
    const uint32_t box[4] = {(uint32_t)bw, (uint32_t)bh, (uint32_t)BM, 1};
    const int rc = encode_map_f32(&L.ma, c.gout, dims, st, box, CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc) return rc;
  }
  // B: this group's channels of the channels-last image; one box = 32 channels x 16 pixels of one row
  {
    const uint64_t dims[4] = {(uint64_t)c.cpad, (uint64_t)c.w_img, (uint64_t)c.h_img, (uint64_t)c.batch};
    const uint64_t st[3] = {(uint64_t)c.c_total * 4, (uint64_t)c.w_img * c.c_total * 4,
                            (uint64_t)c.h_img * c.w_img * c.c_total * 4};
    const uint32_t box[4] = {(uint32_t)CvCfg::CH, (uint32_t)bw, (uint32_t)bh, 1};
    const int rc = encode_map_f32(&L.mb, c.img_cl, dims, st, box, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
    if (rc) return rc;
  }
  L.mc = L.ma;
  const bool out_map = encode_map(&L.mc, c.out, 4, kr, c.m, kr, 1, 0, 1, 0, 32, 128, CU_TENSOR_MAP_SWIZZLE_128B) == B200_OK;
  TcArgs& g = L.g;
  cv_common_args(g, ds);
  g.m = (int)c.m; g.n = (int)kr;
  g.m_tiles = (int)((c.m + BM - 1) / BM);
  g.n_tiles = (int)((kr + tile_cols - 1) / tile_cols);
  g.total_tiles = (long long)g.m_tiles * g.n_tiles;
  g.red = (int)c.batch;
  g.cv_bw = bw; g.cv_bh = bh;
  g.cv_wblocks = (int)((c.w_out + bw - 1) / bw);
  g.cv_rows = (int)((c.h_out + bh - 1) / bh);
  g.k_blocks = g.cv_rows * g.cv_wblocks;
  const long long total_kb = (long long)g.red * g.k_blocks;
  // K slices: as many work units as SMs; the slices add into `out` atomically
  long long slices = sms / g.total_tiles;
  if (slices < 1) slices = 1;
  if (slices > total_kb) slices = total_kb;
  const long long kb_per = (total_kb + slices - 1) / slices;
  slices = (total_kb + kb_per - 1) / kb_per;
  g.kb_per_slice = (int)kb_per; g.ksplit = (int)slices;
  // a single slice still adds into `out` (which holds zeros or a running sum): ksplit > 1 selects the atomic path
  if (g.ksplit == 1) { g.beta = 1; }
  if (out_map && g_store_mode.load() != 1) g.c_tma = 2;    // the slices' sums leave as bulk reduce-adds
  g.total_units = g.total_tiles * slices;
  g.b_mn = 1;
  g.c = c.out; g.ldc = kr;
  g.tile_cols = tile_cols; g.tile_valid = tile_cols; g.mma_n = tile_cols;
  g.b_tx_bytes = tile_cols * CvCfg::BK * 4;
  g.cv_cpad = (int)c.cpad; g.cv_kw = c.kw; g.cv_taps = (int)taps;
  g.cv_w0 = c.w0; g.cv_dw = c.dw; g.cv_h0 = c.h0; g.cv_dh = c.dh;
  const long long forced_limit = g_wait_limit.load();
  g.wait_limit = forced_limit > 0 ? forced_limit : 400000000LL + kb_per * 40000LL;
  const long long grid = g.total_units < sms ? g.total_units : sms;
  if (grid <= 0) return B200_OK;
  gemm_tf32x3_kernel<CV_BN, 2><<<(unsigned)grid, CvCfg::THREADS, CvCfg::SMEM_BYTES, stream>>>(L.ma, L.mb, L.mc, L.g);
  count_launch(true);
  return note_cuda_error(cudaGetLastError(), "implicit filter-gradient launch");
}

bool tc_eligible(const GemmProblem& p) { return make_plan(p, false).ok || make_plan(p, true).ok; }

int tc_setup_device() {
  int st = 0;
  if ((st = set_attr<CfgH<64>>(gemm_f16_kernel<64>))) return st;
  if ((st = set_attr<CfgH<128>>(gemm_f16_kernel<128>))) return st;
  if ((st = set_attr<CfgH<256>>(gemm_f16_kernel<256>))) return st;
  if ((st = set_attr<CfgHB>(gemm_f16_big_kernel))) return st;
  if ((st = set_attr<CfgS<64>>(gemm_tf32x3_kernel<64>))) return st;
  if ((st = set_attr<CfgS<128>>(gemm_tf32x3_kernel<128>))) return st;
  if ((st = set_attr<CfgS<256>>(gemm_tf32x3_kernel<256>))) return st;
  if ((st = set_attr<CfgS<256>>(gemm_tf32x3_kernel<256, 1>))) return st;
  if ((st = set_attr<CfgS<256>>(gemm_tf32x3_kernel<256, 2>))) return st;
  if ((st = pair_setup_device())) return st;
  return encode_fn() ? B200_OK : B200_ERR_CUDA;
}

int launch_gemm_tc(const GemmProblem& p, cudaStream_t stream) {
  const int es = (p.dtype == B200_F32) ? 4 : 2;
  Plan row = make_plan(p, false), col = make_plan(p, true);
  const int g_store_mode = b200::g_store_mode.load();
  if (g_store_mode == 1) col.ok = false;
  if (g_store_mode == 2 && col.ok) row.ok = false;
  if (!row.ok && !col.ok) return B200_ERR_UNSUPPORTED;
  const Plan* pl = &row;
  if (!row.ok) {
    pl = &col;
  } else if (col.ok) {
    // Both orientations are possible.  Row stores (vector accesses) are much faster per tile (measured: even an
    // output with 64 rows, half of a 128-row tile, is faster with row stores), so the column-store orientation is
    // taken only where the model says it halves the work.
    int bn;
    const double cr = choose_tile(row, es, &bn), cc = choose_tile(col, es, &bn);
    if (g_store_mode == 2 || (es == 4 && cc < 0.5 * cr)) pl = &col;
  }
  if (p.dtype == B200_F32) return launch_es<4>(*pl, stream);
  return launch_es<2>(*pl, stream);
}

// GemmProblem::acc32: f16 operands, f32 destination.  Only the row-store orientation (the kernel's N along C's unit
// stride); B200_ERR_UNSUPPORTED without a launch where the operands are not TMA-addressable.
int launch_gemm_tc_acc32(const GemmProblem& p, cudaStream_t stream) {
  if (!p.acc32 || (p.dtype != B200_F16 && p.dtype != B200_AMP_F16)) return B200_ERR_UNSUPPORTED;
  const Plan row = make_plan(p, false);
  if (!row.ok) return B200_ERR_UNSUPPORTED;
  return launch_big_f16_acc32(row, stream);
}

int tc_wait_selftest(long long limit, long long* cycles, cudaStream_t stream) {
  DeviceState* ds = device_state();
  if (!ds) return note_cuda_error(cudaErrorInitializationError, "b200_init not called on this device");
  wait_selftest_kernel<<<1, 128, 0, stream>>>(limit, ds->status);
  count_launch(false);
  int rc = note_cuda_error(cudaGetLastError(), "wait self-test launch");
  if (rc) return rc;
  if ((rc = note_cuda_error(cudaStreamSynchronize(stream), "cudaStreamSynchronize(wait self-test)"))) return rc;
  long long v = 0;
  if ((rc = note_cuda_error(cudaMemcpyFromSymbol(&v, g_selftest_cycles, sizeof(v)), "cudaMemcpyFromSymbol"))) return rc;
  if (cycles) *cycles = v;
  return B200_OK;
}

void tc_set_xform_mode(int mode) { g_xform_mode = mode; }
void tc_set_tile_n(int bn) { g_force_bn = bn; }
void tc_set_mn_box5(int on) { g_mn_box5 = on; }
void tc_set_pair_mode(int mode) { g_pair_mode = mode; }
void tc_set_store_mode(int mode) { g_store_mode = mode; }
void tc_set_split_mode(int mode) { g_split_mode = mode; }
void tc_set_max_ctas(int n) { g_max_ctas = n; }
void tc_set_tail_mode(int mode) { g_tail_mode = mode; }
void tc_set_wait_limit(long long cycles) { g_wait_limit = cycles; }
void tc_set_capture_split(int on) { g_capture_split = on ? 1 : 0; }

}  // namespace b200
