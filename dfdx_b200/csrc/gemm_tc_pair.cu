// CTA-pair tensor-core GEMMs: tcgen05.mma cta_group::2.
//
// Two CTAs of a cluster (on the two SMs of one TPC) compute one 256 x 256 output tile.  Each CTA
// stages its own 128 rows of A and its own 128 of the tile's 256 columns of B; the leader CTA
// (cluster rank 0) issues the MMAs, which read both CTAs' shared memory and write 128 rows x 256
// columns of f32 into each CTA's tensor memory.  Per CTA the shared-memory pipe therefore carries
// half of B per MMA (8 KB instead of 12 KB per 128 x 256 x K-step), which is what bounds the
// single-CTA kernels.  Everything else follows gemm_tc.cu: persistent tiles, TMA-fed ring, bounded
// waits, f16 with a double-buffered accumulator, f32 as 3xTF32 with 256-wide K chunks promoted to
// registers by two epilogue warpgroups.
//
// Cross-CTA signalling.  Barriers the MMA issuer waits on live in the leader: the peer's split warps
// and epilogue warps arrive on them remotely (mapa + mbarrier.arrive.release.cluster).  Barriers the
// peer's own warps wait on (stage empty, accumulator full) live in each CTA: the leader's MMA thread
// commits to both CTAs' copies.  f16 stages have no per-CTA consumer, so both CTAs' TMA loads
// complete on the leader's `full` barrier (cp.async.bulk.tensor with .cta_group::2), armed by the
// leader with the byte count of both halves.  No load in this file uses multicast.
#include "tc_device.cuh"
#include <mutex>

namespace b200 {

using namespace tcx;

namespace {

// ---------------------------------------------------------------------------------------------
// cluster / pair PTX
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of `local_smem_addr` as seen in CTA `rank` of the cluster (shared::cluster window).
__device__ __forceinline__ uint32_t mapa(uint32_t local_smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc2(uint32_t slot_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// Arrives (once the issuing thread's earlier MMAs retire) on a barrier given by its cluster address.
__device__ __forceinline__ void umma_commit2(uint32_t cluster_bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}
template <int ESIZE>
__device__ __forceinline__ void umma2(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                      uint32_t accumulate) {
  if constexpr (ESIZE == 2) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
  }
}
// TMA loads whose completion is counted on a barrier that may live in the pair's other CTA.
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const CUtensorMap* map, uint32_t cluster_bar,
                                                 int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tma_load_5d_pair(uint32_t dst, const CUtensorMap* map, uint32_t cluster_bar,
                                                 int c0, int c1, int c2, int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4) : "memory");
}
template <int ROWS, int BK, int CH, uint32_t MN_LBO>
__device__ __forceinline__ void load_operand_pair(uint32_t dst, const CUtensorMap* map, uint32_t cluster_bar,
                                                  int mode, int row0, int k0, int x, int y) {
  if (mode == 0) {
    tma_load_4d_pair(dst, map, cluster_bar, k0, row0, x, y);
  } else if (mode == 2) {
    tma_load_5d_pair(dst, map, cluster_bar, 0, k0, row0 / CH, x, y);
  } else {
#pragma unroll 1
    for (int c = 0; c < ROWS / CH; ++c) tma_load_4d_pair(dst + c * MN_LBO, map, cluster_bar, row0 + c * CH, k0, x, y);
  }
}

constexpr int PBM = 128;      // rows of A (and of the accumulator) per CTA
constexpr int PBN = 256;      // tile columns
constexpr int PBNL = 128;     // columns of B staged per CTA

// ---------------------------------------------------------------------------------------------
// f16 pair kernel
// ---------------------------------------------------------------------------------------------
struct PCfgH {
  static constexpr int BK = 64, CH = 64, KSTEPS = 4;
  static constexpr int A_BYTES = PBM * 128, B_BYTES = PBNL * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;                 // 32 KB per CTA
  static constexpr int STAGES = 6;
  static constexpr int THREADS = 192;
  static constexpr int TMEM_COLS = 2 * PBN;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;
  static constexpr uint32_t LAYOUT = 2u, SBO = 1024, MN_LBO = BK * 128, MN_KADV = 2 * 1024, K_KADV = 32;
};

__global__ void __launch_bounds__(PCfgH::THREADS, 1)
gemm_f16_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                     const TcArgs g) {
  using C = PCfgH;
  constexpr int STAGES = C::STAGES;
  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t bar_full[STAGES];     // leader's copy is used: both CTAs' loads land on it
  __shared__ __align__(8) uint64_t bar_empty[STAGES];    // per CTA, committed by the leader's MMA thread
  __shared__ __align__(8) uint64_t bar_tfull[2];         // per CTA, committed by the leader's MMA thread
  __shared__ __align__(8) uint64_t bar_tempty[2];        // leader's copy: 8 epilogue warps arrive
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  volatile int* abortp = &abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bar_tfull[b]), 1);
      mbar_init(smem_u32(&bar_tempty[b]), 8);
    }
    abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 5) {
    tmem_alloc2(smem_u32(&tmem_slot), C::TMEM_COLS);
    tmem_relinquish2();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                    // the peer's barriers exist before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  const int total_kb = g.red * g.k_blocks;
  const long long cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (long long tile = cluster_id; ok && tile < g.total_tiles; tile += n_clusters) {
        const TileCoord t = decode_tile(g, tile);
        for (int i = 0; i < total_kb; ++i, ++it) {
          const int r = i / g.k_blocks, kb = i - r * g.k_blocks;
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, abortp, g.wait_limit)) { ok = false; break; }
          if (rank == 0) mbar_expect_tx(smem_u32(&bar_full[s]), 2 * C::STAGE_BYTES);   // both CTAs' bytes
          const uint32_t full = mapa(smem_u32(&bar_full[s]), 0);
          const uint32_t a_dst = smem_base + s * C::STAGE_BYTES;
          load_operand_pair<PBM, C::BK, C::CH, C::MN_LBO>(a_dst, &tma_a, full, g.a_ld,
                                                          t.mt * 2 * PBM + rank * PBM, kb * C::BK,
                                                          g.a_x1 * t.ib1 + g.a_xr * r, g.a_y0 * t.ib0);
          load_operand_pair<PBNL, C::BK, C::CH, C::MN_LBO>(a_dst + C::A_BYTES, &tma_b, full, g.b_ld,
                                                           t.nt * PBN + rank * PBNL, kb * C::BK,
                                                           g.b_x1 * t.ib1 + g.b_xr * r, g.b_y0 * t.ib0);
        }
      }
    }
    __syncwarp();
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer (leader only)
    if (lane == 0 && rank == 0) {
      // instruction descriptor: D = f32, A = B = f16, majors, N >> 3, M = 256 >> 4
      const uint32_t idesc = (1u << 4) | ((uint32_t)(g.a_mn ? 1 : 0) << 15) | ((uint32_t)(g.b_mn ? 1 : 0) << 16) |
                             ((uint32_t)(PBN >> 3) << 17) | ((uint32_t)((2 * PBM) >> 4) << 24);
      const uint32_t a_lbo = g.a_mn ? C::MN_LBO : 16u, b_lbo = g.b_mn ? C::MN_LBO : 16u;
      const uint32_t a_kadv = g.a_mn ? C::MN_KADV : C::K_KADV, b_kadv = g.b_mn ? C::MN_KADV : C::K_KADV;
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (long long tile = cluster_id; ok && tile < g.total_tiles; tile += n_clusters, ++tcount) {
        const uint32_t buf = tcount & 1u, tph = (tcount >> 1) & 1u;
        if (!mbar_wait(smem_u32(&bar_tempty[buf]), tph ^ 1u, abortp, g.wait_limit)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * PBN;
        for (int i = 0; i < total_kb; ++i, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(smem_u32(&bar_full[s]), ph, abortp, g.wait_limit)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_base = smem_base + s * C::STAGE_BYTES;
          const uint32_t b_base = a_base + C::A_BYTES;
#pragma unroll
          for (int ks = 0; ks < C::KSTEPS; ++ks) {
            const uint64_t ad = make_smem_desc(a_base + ks * a_kadv, a_lbo, C::SBO, C::LAYOUT);
            const uint64_t bd = make_smem_desc(b_base + ks * b_kadv, b_lbo, C::SBO, C::LAYOUT);
            umma2<2>(d_tmem, ad, bd, idesc, (i > 0 || ks > 0) ? 1u : 0u);
          }
          umma_commit2(mapa(smem_u32(&bar_empty[s]), 0));   // stage reusable in both CTAs
          umma_commit2(mapa(smem_u32(&bar_empty[s]), 1));
        }
        if (ok) {
          umma_commit2(mapa(smem_u32(&bar_tfull[buf]), 0));
          umma_commit2(mapa(smem_u32(&bar_tfull[buf]), 1));
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue (warps 0..3, both CTAs)
    uint32_t tcount = 0;
    bool ok = true;
    for (long long tile = cluster_id; ok && tile < g.total_tiles; tile += n_clusters, ++tcount) {
      const TileCoord t = decode_tile(g, tile);
      const uint32_t buf = tcount & 1u, tph = (tcount >> 1) & 1u;
      if (!mbar_wait(smem_u32(&bar_tfull[buf]), tph, abortp, g.wait_limit)) { ok = false; break; }
      tc_fence_after();
      const int row = t.mt * 2 * PBM + rank * PBM + warp * 32 + lane;
      __half* cbase = (__half*)g.c + t.ib0 * g.c_b0 + t.ib1 * g.c_b1;
      const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + buf * PBN;
#pragma unroll 1
      for (int c = 0; c < PBN / 32; ++c) {
        const int col0 = t.nt * PBN + c * 32;
        if (col0 >= g.n) break;                      // warp-uniform
        uint32_t v[32];
        tmem_ld_32x32(taddr + c * 32, v);
        tmem_wait_ld();
        if (row < g.m) {
          float f[32];
#pragma unroll
          for (int q = 0; q < 32; ++q) f[q] = __uint_as_float(v[q]);
          const int valid = (g.n - col0) < 32 ? (g.n - col0) : 32;
          if (g.c_col) store_chunk_col(cbase + (long long)col0 * g.ldc + row, f, valid, g.ldc, g.beta);
          else store_chunk(cbase + (long long)row * g.ldc + col0, f, valid, g.beta, g.c_wide);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa(smem_u32(&bar_tempty[buf]), 0));
    }
  }

  tc_fence_before();
  __syncthreads();
  teardown(abort_flag, g.status);
  cluster_sync_all();                                    // nobody leaves while the peer may still signal it
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, C::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------
// f32 (3xTF32) pair kernel
// ---------------------------------------------------------------------------------------------
struct PCfgS {
  static constexpr int BK = 16, CH = 32, KSTEPS = 2;
  static constexpr int A_BYTES = PBM * 64, B_BYTES = PBNL * 64;
  static constexpr int RAW_BYTES = A_BYTES + B_BYTES;                   // 16 KB
  static constexpr int STAGE_BYTES = 2 * RAW_BYTES;                     // raw (big) + small copy
  static constexpr int STAGES = 6;
  static constexpr int THREADS = 512;
  static constexpr int TMEM_COLS = 2 * PBN;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;
  static constexpr int CHUNK_KB = 16;                                   // promotion chunk: K = 256
  static constexpr int HALF = PBN / 2;
  static constexpr int SPLIT_WARPS = 6;
  static constexpr uint32_t K_LAYOUT = 4u, K_SBO = 512, K_KADV = 32;
  static constexpr uint32_t MN_LAYOUT = 1u, MN_SBO = 512, MN_LBO = BK * 128, MN_KADV = 8 * 128;
};

// Operand split of this CTA's stages (see gemm_tc.cu); one elected lane per warp then arrives on the
// leader's `xform` barrier.
__device__ __forceinline__ void split_role_pair(const TcArgs& g, uint32_t smem_base, uint64_t* bar_full,
                                                uint64_t* bar_xform, volatile int* abortp, int total_kb, int tt,
                                                long long cluster_id, long long n_clusters) {
  using C = PCfgS;
  constexpr int STAGES = C::STAGES;
  constexpr int NVEC = C::RAW_BYTES / 16;
  constexpr int NT = C::SPLIT_WARPS * 32;
  uint32_t it = 0;
  bool ok = true;
  for (long long tile = cluster_id; ok && tile < g.total_tiles; tile += n_clusters) {
    for (int i = 0; i < total_kb; ++i, ++it) {
      const int s = it % STAGES;
      const uint32_t ph = (it / STAGES) & 1u;
      if (!mbar_wait(smem_u32(&bar_full[s]), ph, abortp, g.wait_limit)) { ok = false; break; }
      const uint32_t raw = smem_base + s * C::STAGE_BYTES;
      constexpr int nvec = NVEC;
#pragma unroll 1
      for (int v0 = tt; v0 < nvec; v0 += 4 * NT) {
        uint32_t x[4][4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int v = v0 + u * NT;
          if (v < NVEC)
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(x[u][0]), "=r"(x[u][1]), "=r"(x[u][2]), "=r"(x[u][3]) : "r"(raw + v * 16));
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int v = v0 + u * NT;
          if (v < NVEC) {
            uint32_t sm[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float d = __uint_as_float(x[u][e]) - __uint_as_float(x[u][e] & 0xffffe000u);
              d = (d != d) ? 0.f : d;                   // inf - inf: keep inf / nan in `big` only
              asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(sm[e]) : "f"(d));
            }
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                         ::"r"(raw + C::RAW_BYTES + v * 16), "r"(sm[0]), "r"(sm[1]), "r"(sm[2]), "r"(sm[3]) : "memory");
          }
        }
      }
      fence_proxy_async_all();                          // generic-proxy writes -> visible to tcgen05.mma
      __syncwarp();
      if ((threadIdx.x & 31) == 0) mbar_arrive_cluster(mapa(smem_u32(&bar_xform[s]), 0));
    }
  }
}

__global__ void __launch_bounds__(PCfgS::THREADS, 1)
gemm_tf32x3_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                        const TcArgs g) {
  using C = PCfgS;
  constexpr int STAGES = C::STAGES;
  constexpr int PRODUCER_WARP = 12, MMA_WARP = 13;

  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t bar_full[STAGES];     // per CTA: this CTA's TMA bytes
  __shared__ __align__(8) uint64_t bar_empty[STAGES];    // per CTA, committed by the leader's MMA thread
  __shared__ __align__(8) uint64_t bar_xform[STAGES];    // leader's copy: 12 split warps arrive
  __shared__ __align__(8) uint64_t bar_tfull[2];         // per CTA, committed by the leader's MMA thread
  __shared__ __align__(8) uint64_t bar_tempty[2];        // leader's copy: 16 epilogue warps arrive
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wg = warp >> 2;
  const uint32_t rank = cluster_ctarank();
  volatile int* abortp = &abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
      mbar_init(smem_u32(&bar_xform[s]), 2 * C::SPLIT_WARPS);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bar_tfull[b]), 1);
      mbar_init(smem_u32(&bar_tempty[b]), 16);
    }
    abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == MMA_WARP) {
    tmem_alloc2(smem_u32(&tmem_slot), C::TMEM_COLS);
    tmem_relinquish2();
  }
  if (warp == PRODUCER_WARP && lane == 0) {
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  const int total_kb = g.red * g.k_blocks;
  const long long cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;

  if (wg == 3) {
    setmaxnreg_dec_56();
    if (warp == PRODUCER_WARP && lane == 0) {
      // ---------------------------------------------------------------- TMA producer (both CTAs)
      uint32_t it = 0;
      bool ok = true;
      for (long long tile = cluster_id; ok && tile < g.total_tiles; tile += n_clusters) {
        const TileCoord t = decode_tile(g, tile);
        for (int i = 0; i < total_kb; ++i, ++it) {
          const int r = i / g.k_blocks, kb = i - r * g.k_blocks;
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, abortp, g.wait_limit)) { ok = false; break; }
          const uint32_t full = smem_u32(&bar_full[s]);
          mbar_expect_tx(full, C::RAW_BYTES);
          const uint32_t a_dst = smem_base + s * C::STAGE_BYTES;
          load_operand<PBM, C::BK, C::CH, C::MN_LBO>(a_dst, &tma_a, full, g.a_ld, t.mt * 2 * PBM + rank * PBM,
                                                      kb * C::BK, g.a_x1 * t.ib1 + g.a_xr * r, g.a_y0 * t.ib0);
          load_operand<PBNL, C::BK, C::CH, C::MN_LBO>(a_dst + C::A_BYTES, &tma_b, full, g.b_ld,
                                                       t.nt * PBN + rank * PBNL, kb * C::BK,
                                                       g.b_x1 * t.ib1 + g.b_xr * r, g.b_y0 * t.ib0);
        }
      }
    } else if (warp == MMA_WARP && lane == 0 && rank == 0) {
      // ---------------------------------------------------------------- MMA issuer (leader only)
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(g.a_mn ? 1 : 0) << 15) |
                             ((uint32_t)(g.b_mn ? 1 : 0) << 16) | ((uint32_t)(PBN >> 3) << 17) |
                             ((uint32_t)((2 * PBM) >> 4) << 24);
      const uint32_t a_lbo = g.a_mn ? C::MN_LBO : 16u, b_lbo = g.b_mn ? C::MN_LBO : 16u;
      const uint32_t a_sbo = g.a_mn ? C::MN_SBO : C::K_SBO, b_sbo = g.b_mn ? C::MN_SBO : C::K_SBO;
      const uint32_t a_lay = g.a_mn ? C::MN_LAYOUT : C::K_LAYOUT, b_lay = g.b_mn ? C::MN_LAYOUT : C::K_LAYOUT;
      const uint32_t a_kadv = g.a_mn ? C::MN_KADV : C::K_KADV, b_kadv = g.b_mn ? C::MN_KADV : C::K_KADV;
      uint32_t it = 0, ccount = 0;
      bool ok = true;
      for (long long tile = cluster_id; ok && tile < g.total_tiles; tile += n_clusters) {
        for (int kb0 = 0; ok && kb0 < total_kb; kb0 += C::CHUNK_KB, ++ccount) {
          const uint32_t buf = ccount & 1u, cph = (ccount >> 1) & 1u;
          if (!mbar_wait(smem_u32(&bar_tempty[buf]), cph ^ 1u, abortp, g.wait_limit)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + buf * PBN;
          const int nkb = (total_kb - kb0) < C::CHUNK_KB ? (total_kb - kb0) : C::CHUNK_KB;
          for (int i = 0; i < nkb; ++i, ++it) {
            const int s = it % STAGES;
            const uint32_t ph = (it / STAGES) & 1u;
            if (!mbar_wait(smem_u32(&bar_xform[s]), ph, abortp, g.wait_limit)) { ok = false; break; }
            tc_fence_after();
            const uint32_t a_base = smem_base + s * C::STAGE_BYTES;
            const uint32_t b_base = a_base + C::A_BYTES;
#pragma unroll
            for (int ks = 0; ks < C::KSTEPS; ++ks) {
              const uint64_t ad = make_smem_desc(a_base + ks * a_kadv, a_lbo, a_sbo, a_lay);
              const uint64_t bd = make_smem_desc(b_base + ks * b_kadv, b_lbo, b_sbo, b_lay);
              const uint64_t ads = make_smem_desc(a_base + C::RAW_BYTES + ks * a_kadv, a_lbo, a_sbo, a_lay);
              const uint64_t bds = make_smem_desc(b_base + C::RAW_BYTES + ks * b_kadv, b_lbo, b_sbo, b_lay);
              umma2<4>(d_tmem, ads, bd, idesc, (i > 0 || ks > 0) ? 1u : 0u);   // small * big
              umma2<4>(d_tmem, ad, bds, idesc, 1u);                            // big * small
              umma2<4>(d_tmem, ad, bd, idesc, 1u);                             // big * big
            }
            umma_commit2(mapa(smem_u32(&bar_empty[s]), 0));
            umma_commit2(mapa(smem_u32(&bar_empty[s]), 1));
          }
          if (ok) {
            umma_commit2(mapa(smem_u32(&bar_tfull[buf]), 0));
            umma_commit2(mapa(smem_u32(&bar_tfull[buf]), 1));
          }
        }
      }
    } else if (warp >= 14) {
      split_role_pair(g, smem_base, bar_full, bar_xform, abortp, total_kb, threadIdx.x - 448 + 128, cluster_id,
                      n_clusters);
    }
    __syncwarp();
  } else if (wg == 2) {
    setmaxnreg_dec_56();
    split_role_pair(g, smem_base, bar_full, bar_xform, abortp, total_kb, threadIdx.x - 256, cluster_id, n_clusters);
  } else {
    // ------------------------------------------------------------------ epilogue (warpgroups 0 and 1, both CTAs)
    setmaxnreg_inc_200();
    const int quad = warp & 3;
    const int col_base = wg * C::HALF;
    uint32_t ccount = 0;
    bool ok = true;
    for (long long tile = cluster_id; ok && tile < g.total_tiles; tile += n_clusters) {
      const TileCoord t = decode_tile(g, tile);
      float acc[C::HALF];
#pragma unroll
      for (int q = 0; q < C::HALF; ++q) acc[q] = 0.f;
      for (int kb0 = 0; kb0 < total_kb; kb0 += C::CHUNK_KB, ++ccount) {
        const uint32_t buf = ccount & 1u, cph = (ccount >> 1) & 1u;
        if (!mbar_wait(smem_u32(&bar_tfull[buf]), cph, abortp, g.wait_limit)) { ok = false; break; }
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + buf * PBN + col_base;
#pragma unroll
        for (int c = 0; c < C::HALF / 16; ++c) {
          uint32_t v[16];
          tmem_ld_32x16(taddr + c * 16, v);
          tmem_wait_ld();
#pragma unroll
          for (int q = 0; q < 16; ++q) acc[c * 16 + q] += __uint_as_float(v[q]);   // round-to-nearest add
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(mapa(smem_u32(&bar_tempty[buf]), 0));
      }
      if (!ok) break;
      const int row = t.mt * 2 * PBM + rank * PBM + quad * 32 + lane;
      if (row < g.m) {
        float* cbase = (float*)g.c + t.ib0 * g.c_b0 + t.ib1 * g.c_b1;
#pragma unroll
        for (int c = 0; c < C::HALF / 32; ++c) {
          const int col0 = t.nt * PBN + col_base + c * 32;
          if (col0 < g.n) {
            const int valid = (g.n - col0) < 32 ? (g.n - col0) : 32;
            if (g.c_col) store_chunk_col(cbase + (long long)col0 * g.ldc + row, &acc[c * 32], valid, g.ldc, g.beta);
            else store_chunk(cbase + (long long)row * g.ldc + col0, &acc[c * 32], valid, g.beta, g.c_wide);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  teardown(abort_flag, g.status);
  cluster_sync_all();
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, C::TMEM_COLS);
  }
}

template <typename Kernel>
int launch_pair_kernel(Kernel kernel, int threads, int smem, int sm_count, const CUtensorMap& ma, const CUtensorMap& mb,
                       TcArgs g, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  cfg.blockDim = dim3(threads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  long long clusters = sm_count / 2;
  if (g.total_tiles < clusters) clusters = g.total_tiles;
  if (clusters <= 0) return B200_OK;
  cfg.gridDim = dim3((unsigned)(2 * clusters), 1, 1);
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, ma, mb, g);
  count_launch(true);
  return note_cuda_error(e, "tensor-core pair gemm launch");
}

}  // namespace

// Tile extents of the pair kernels, for the host-side planner.
int pair_tile_m() { return 2 * PBM; }
int pair_tile_n() { return PBN; }
int pair_block_k(int esize) { return esize == 2 ? PCfgH::BK : PCfgS::BK; }
int pair_chunk(int esize) { return esize == 2 ? PCfgH::CH : PCfgS::CH; }

int pair_setup_device() {
  int st = note_cuda_error(cudaFuncSetAttribute(gemm_f16_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                PCfgH::SMEM_BYTES), "cudaFuncSetAttribute(pair f16)");
  if (st) return st;
  return note_cuda_error(cudaFuncSetAttribute(gemm_tf32x3_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              PCfgS::SMEM_BYTES), "cudaFuncSetAttribute(pair tf32x3)");
}

// `g` arrives filled for a 256 x 256 tile grid (m_tiles = ceil(m / 256), n_tiles = ceil(n / 256)).
int launch_pair(int esize, const CUtensorMap& ma, const CUtensorMap& mb, const TcArgs& g, int sm_count,
                cudaStream_t stream) {
  if (esize == 2)
    return launch_pair_kernel(gemm_f16_pair_kernel, PCfgH::THREADS, PCfgH::SMEM_BYTES, sm_count, ma, mb, g, stream);
  return launch_pair_kernel(gemm_tf32x3_pair_kernel, PCfgS::THREADS, PCfgS::SMEM_BYTES, sm_count, ma, mb, g, stream);
}

}  // namespace b200
