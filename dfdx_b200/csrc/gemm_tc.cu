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
// gemm_tf32x3_kernel  f32 operands as 3xTF32 (kind::tf32).  16 warps in four warpgroups:
//                   WG3 = TMA producer warp + MMA warp, WG2 = operand split, WG0/WG1 = epilogue.
//                   Each staged f32 x stays in place as the `big` operand (the tensor core reads its top
//                   19 bits) and small = tf32_rn(x - trunc_tf32(x)) is written beside it; every k-step
//                   issues small*big, big*small, big*big (K = 8).  The tensor core adds into its f32
//                   accumulator with truncation, so the error of one long accumulation grows linearly
//                   with K; therefore K is cut into chunks of 256: each chunk accumulates in one of two
//                   TMEM buffers and the epilogue warpgroups add finished chunks into f32 registers
//                   (round-to-nearest) while the next chunk runs.  setmaxnreg moves registers from the
//                   producer / MMA / split warpgroups to the epilogue warpgroups.
//
// Operands are read in place from dfdx's strides: K-major rows, or MN-major (the transposed views that
// the backward GEMMs and `permute` produce).  MN-major tiles are brought in as column chunks:
// 64 x f16 under the 128B swizzle, 32 x f32 under the 128B swizzle with 32-byte atoms (the only
// MN-major layout kind::tf32 accepts); K-major f32 tiles use the 64B swizzle (BK = 16).
//
// Every wait on an mbarrier is bounded: on expiry the CTA raises an abort flag in shared memory, all
// roles drain, TMEM is freed, the kernel writes B200_ERR_DEVICE_TIMEOUT to the device status word and
// returns normally.
#include "common.cuh"
#include <cuda.h>
#include <mutex>

namespace b200 {
namespace {

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok;
}
// Bounded wait.  Returns false (and raises *abort_flag) if `limit` clock cycles pass, or as soon as
// another role has raised the flag.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          long long limit) {
#pragma unroll 1
  for (int i = 0; i < 64; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
#pragma unroll 1
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > limit) { *abort_flag = 1; return false; }
  }
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(m) : "memory");
}
// Tiled 4-D TMA load, completion counted in bytes on `bar`.  Coordinates innermost first.
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2, int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4) : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
template <int ESIZE>
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                     uint32_t accumulate) {
  if constexpr (ESIZE == 2) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
  }
}
// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives lane (base+i), columns c..c+31.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor (sm_100 format): start address, leading / stride byte offsets in
// 16-byte units, descriptor version 1 at bit 46, swizzle mode at bits 61..63 (2 = 128B, 4 = 64B).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                   uint32_t layout_type) {
  uint64_t d = (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;
  d |= (uint64_t)layout_type << 61;
  return d;
}

__device__ __forceinline__ void setmaxnreg_dec_56() { asm volatile("setmaxnreg.dec.sync.aligned.u32 56;"); }
__device__ __forceinline__ void setmaxnreg_inc_200() { asm volatile("setmaxnreg.inc.sync.aligned.u32 200;"); }

// ---------------------------------------------------------------------------------------------
// Kernel configuration
// ---------------------------------------------------------------------------------------------
constexpr int BM = 128;

// f16: every operand tile is made of 128-byte rows under the 128B swizzle.
template <int BN>
struct CfgH {
  static constexpr int BK = 64;                             // k extent of a stage (elements)
  static constexpr int CH = 64;                             // MN elements per MN-major chunk
  static constexpr int KSTEPS = 4;                          // MMAs per stage (K = 16 each)
  static constexpr int A_BYTES = BM * 128;
  static constexpr int B_BYTES = BN * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES_FIT = (192 * 1024) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_FIT > 8 ? 8 : STAGES_FIT;
  static constexpr int THREADS = 192;
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;
  static constexpr uint32_t LAYOUT = 2u;                    // SWIZZLE_128B
  static constexpr uint32_t SBO = 1024;                     // 8 rows of 128 bytes
  static constexpr uint32_t MN_LBO = BK * 128;              // distance between MN-major chunks
  static constexpr uint32_t MN_KADV = 2 * 1024;             // 16 k rows per MMA
  static constexpr uint32_t K_KADV = 32;                    // 16 elements of K per MMA
};

// f32 (3xTF32): K-major tiles are 64-byte rows under the 64B swizzle; MN-major tiles are chunks of
// 32 columns x BK k-rows of 128 bytes under the 128B swizzle with 32-byte atoms.
template <int BN>
struct CfgS {
  static constexpr int BK = 16;
  static constexpr int CH = 32;
  static constexpr int KSTEPS = 2;                          // k-steps per stage (K = 8 each), 3 MMAs per step
  static constexpr int A_BYTES = BM * 64;
  static constexpr int B_BYTES = BN * 64;
  static constexpr int RAW_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGE_BYTES = 2 * RAW_BYTES;         // raw (big) + small copy
  static constexpr int STAGES_FIT = (192 * 1024) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_FIT > 8 ? 8 : STAGES_FIT;
  static constexpr int THREADS = 512;
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;
  static constexpr int CHUNK_KB = 16;                       // k-blocks per promotion chunk (K = 256)
  static constexpr int HALF = BN / 2;                       // columns owned by one epilogue warpgroup
  static constexpr uint32_t K_LAYOUT = 4u;                  // SWIZZLE_64B
  static constexpr uint32_t K_SBO = 512;                    // 8 rows of 64 bytes
  static constexpr uint32_t K_KADV = 32;                    // 8 elements of K per MMA
  static constexpr uint32_t MN_LAYOUT = 1u;                 // SWIZZLE_128B_BASE32B
  static constexpr uint32_t MN_SBO = 512;                   // 4 k-rows of 128 bytes
  static constexpr uint32_t MN_LBO = BK * 128;              // distance between MN-major chunks
  static constexpr uint32_t MN_KADV = 8 * 128;              // 8 k-rows per MMA
};

struct TcArgs {
  int m, n;                       // output extent of one batch item
  int m_tiles, n_tiles;
  int nb1;                        // inner batch count (tile id -> (b0, b1))
  long long total_tiles;
  int red, k_blocks;              // k iterations per tile = red * k_blocks
  int a_mn, b_mn;                 // operand is MN-major (else K-major)
  int a_ld, b_ld;                 // load_operand mode: 0 K-major, 1 MN-major per chunk, 2 MN-major one box
  int a_x1, a_xr, a_y0;           // TMA x = a_x1*ib1 + a_xr*r ; y = a_y0*ib0
  int b_x1, b_xr, b_y0;
  void* c;
  long long c_b0, c_b1, ldc;      // element strides
  int beta;
  int xform_mode;                 // f32: 1 = big stays raw, write small only; 0 = also rewrite big = tf32_rn(x)
  long long wait_limit;           // clock cycles
  int* status;
};

// 32 consecutive f32 accumulator columns of one output row -> global memory.
__device__ __forceinline__ void store_chunk(float* dst, const float* v, int valid, int beta) {
  if (valid == 32) {
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      float4 o = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
      if (beta) {
        const float4 old = *reinterpret_cast<const float4*>(dst + 4 * q);
        o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
      }
      *reinterpret_cast<float4*>(dst + 4 * q) = o;
    }
  } else {
#pragma unroll
    for (int q = 0; q < 32; ++q)
      if (q < valid) {
        float o = v[q];
        if (beta) o += dst[q];
        dst[q] = o;
      }
  }
}

__device__ __forceinline__ void store_chunk(__half* dst, const float* v, int valid, int beta) {
  if (valid == 32) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float f[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = v[8 * q + e];
      if (beta) {
        const uint4 old = *reinterpret_cast<const uint4*>(dst + 8 * q);
        const __half2* oh = reinterpret_cast<const __half2*>(&old);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 t = __half22float2(oh[e]);
          f[2 * e] += t.x; f[2 * e + 1] += t.y;
        }
      }
      uint4 pk;
      __half2* ph = reinterpret_cast<__half2*>(&pk);
#pragma unroll
      for (int e = 0; e < 4; ++e) ph[e] = __floats2half2_rn(f[2 * e], f[2 * e + 1]);
      *reinterpret_cast<uint4*>(dst + 8 * q) = pk;
    }
  } else {
#pragma unroll
    for (int q = 0; q < 32; ++q)
      if (q < valid) {
        float o = v[q];
        if (beta) o += __half2float(dst[q]);
        dst[q] = __float2half_rn(o);
      }
  }
}

struct TileCoord { int mt, nt, ib0, ib1; };
__device__ __forceinline__ TileCoord decode_tile(const TcArgs& g, long long tile) {
  const long long per_batch = (long long)g.m_tiles * g.n_tiles;
  const long long bt = tile / per_batch;
  const int rem = (int)(tile - bt * per_batch);
  TileCoord t;
  t.mt = rem % g.m_tiles; t.nt = rem / g.m_tiles;
  t.ib1 = (int)(bt % g.nb1); t.ib0 = (int)(bt / g.nb1);
  return t;
}

// Issues the TMA loads of one stage.  mode 0, K-major operand: one 4-D box [BK, rows].  MN-major
// operand: mode 2 = one 5-D box [CH, BK, rows/CH] over the view (CH, K, MN/CH, x, y) of the matrix
// (needs MN % CH == 0); mode 1 = one 4-D box [CH, BK] per chunk of CH columns.  Either way chunk c of
// the tile lands at dst + c * MN_LBO.
template <int ROWS, int BK, int CH, uint32_t MN_LBO>
__device__ __forceinline__ void load_operand(uint32_t dst, const CUtensorMap* map, uint32_t bar, int mode,
                                             int row0, int k0, int x, int y) {
  if (mode == 0) {
    tma_load_4d(dst, map, bar, k0, row0, x, y);
  } else if (mode == 2) {
    tma_load_5d(dst, map, bar, 0, k0, row0 / CH, x, y);
  } else {
#pragma unroll 1
    for (int c = 0; c < ROWS / CH; ++c) tma_load_4d(dst + c * MN_LBO, map, bar, row0 + c * CH, k0, x, y);
  }
}

__device__ __forceinline__ void teardown(int abort_flag, int* status) {
  if (abort_flag) {
    // Give copies that may still be in flight time to land before shared memory is released.
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) __nanosleep(1000);
    if (threadIdx.x == 0) atomicExch(status, (int)B200_ERR_DEVICE_TIMEOUT);
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------------------------
// f16 kernel
// ---------------------------------------------------------------------------------------------
template <int BN>
__global__ void __launch_bounds__(CfgH<BN>::THREADS, 1)
gemm_f16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                const TcArgs g) {
  using C = CfgH<BN>;
  constexpr int STAGES = C::STAGES;

  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t bar_full[STAGES];
  __shared__ __align__(8) uint64_t bar_empty[STAGES];
  __shared__ __align__(8) uint64_t bar_tfull[2];
  __shared__ __align__(8) uint64_t bar_tempty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

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
      mbar_init(smem_u32(&bar_tempty[b]), 128);
    }
    abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(&tmem_slot), C::TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  const int total_kb = g.red * g.k_blocks;

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (long long tile = blockIdx.x; ok && tile < g.total_tiles; tile += gridDim.x) {
        const TileCoord t = decode_tile(g, tile);
        for (int i = 0; i < total_kb; ++i, ++it) {
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
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // instruction descriptor: D = f32, A = B = f16, majors, N >> 3, M >> 4
      const uint32_t idesc = (1u << 4) | ((uint32_t)(g.a_mn ? 1 : 0) << 15) | ((uint32_t)(g.b_mn ? 1 : 0) << 16) |
                             ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      const uint32_t a_lbo = g.a_mn ? C::MN_LBO : 16u, b_lbo = g.b_mn ? C::MN_LBO : 16u;
      const uint32_t a_kadv = g.a_mn ? C::MN_KADV : C::K_KADV, b_kadv = g.b_mn ? C::MN_KADV : C::K_KADV;
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (long long tile = blockIdx.x; ok && tile < g.total_tiles; tile += gridDim.x, ++tcount) {
        const uint32_t buf = tcount & 1u, tph = (tcount >> 1) & 1u;
        if (!mbar_wait(smem_u32(&bar_tempty[buf]), tph ^ 1u, abortp, g.wait_limit)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
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
            umma<2>(d_tmem, ad, bd, idesc, (i > 0 || ks > 0) ? 1u : 0u);
          }
          umma_commit(smem_u32(&bar_empty[s]));       // stage reusable once these MMAs retire
        }
        if (ok) umma_commit(smem_u32(&bar_tfull[buf]));
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue (warps 0..3)
    uint32_t tcount = 0;
    bool ok = true;
    for (long long tile = blockIdx.x; ok && tile < g.total_tiles; tile += gridDim.x, ++tcount) {
      const TileCoord t = decode_tile(g, tile);
      const uint32_t buf = tcount & 1u, tph = (tcount >> 1) & 1u;
      if (!mbar_wait(smem_u32(&bar_tfull[buf]), tph, abortp, g.wait_limit)) { ok = false; break; }
      tc_fence_after();
      const int row = t.mt * BM + warp * 32 + lane;
      __half* crow = (__half*)g.c + t.ib0 * g.c_b0 + t.ib1 * g.c_b1 + (long long)row * g.ldc;
      const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = t.nt * BN + c * 32;
        if (col0 >= g.n) break;                      // warp-uniform
        uint32_t v[32];
        tmem_ld_32x32(taddr + c * 32, v);
        tmem_wait_ld();
        if (row < g.m) {
          float f[32];
#pragma unroll
          for (int q = 0; q < 32; ++q) f[q] = __uint_as_float(v[q]);
          store_chunk(crow + col0, f, (g.n - col0) < 32 ? (g.n - col0) : 32, g.beta);
        }
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&bar_tempty[buf]));
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

// 3xTF32 operand split of the stages, run by SPLIT_THREADS threads (tt = 0 .. SPLIT_THREADS-1).
// Each raw f32 x stays in place as the `big` operand (the tensor core reads its top 19 bits) and
// small = tf32_rn(x - trunc_tf32(x)) is written RAW_BYTES further on.  Four 16-byte vectors are in
// flight per thread to cover the shared-memory latency.
constexpr int SPLIT_THREADS = 192;

template <typename C>
__device__ __forceinline__ void split_role(const TcArgs& g, uint32_t smem_base, uint64_t* bar_full,
                                           uint64_t* bar_xform, volatile int* abortp, int total_kb, int tt) {
  constexpr int STAGES = C::STAGES;
  constexpr int NVEC = C::RAW_BYTES / 16;
  uint32_t it = 0;
  bool ok = true;
  for (long long tile = blockIdx.x; ok && tile < g.total_tiles; tile += gridDim.x) {
    for (int i = 0; i < total_kb; ++i, ++it) {
      const int s = it % STAGES;
      const uint32_t ph = (it / STAGES) & 1u;
      if (!mbar_wait(smem_u32(&bar_full[s]), ph, abortp, g.wait_limit)) { ok = false; break; }
      const uint32_t raw = smem_base + s * C::STAGE_BYTES;
      const int nvec = (g.xform_mode & 2) ? 0 : NVEC;   // bit 1: timing experiment, no split
#pragma unroll 1
      for (int v0 = tt; v0 < nvec; v0 += 4 * SPLIT_THREADS) {
        uint32_t x[4][4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int v = v0 + u * SPLIT_THREADS;
          if (v < NVEC)
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(x[u][0]), "=r"(x[u][1]), "=r"(x[u][2]), "=r"(x[u][3]) : "r"(raw + v * 16));
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int v = v0 + u * SPLIT_THREADS;
          if (v < NVEC) {
            uint32_t sm[4];
            if ((g.xform_mode & 1) == 0) {              // optional: rewrite big = tf32_rn(x) as well
              uint32_t big[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(big[e]) : "f"(__uint_as_float(x[u][e])));
                float d = __uint_as_float(x[u][e]) - __uint_as_float(big[e]);
                d = (d != d) ? 0.f : d;
                asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(sm[e]) : "f"(d));
              }
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                           ::"r"(raw + v * 16), "r"(big[0]), "r"(big[1]), "r"(big[2]), "r"(big[3]) : "memory");
            } else {
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                float d = __uint_as_float(x[u][e]) - __uint_as_float(x[u][e] & 0xffffe000u);
                d = (d != d) ? 0.f : d;                 // inf - inf: keep inf / nan in `big` only
                asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(sm[e]) : "f"(d));
              }
            }
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                         ::"r"(raw + C::RAW_BYTES + v * 16), "r"(sm[0]), "r"(sm[1]), "r"(sm[2]), "r"(sm[3]) : "memory");
          }
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
template <int BN>
__global__ void __launch_bounds__(CfgS<BN>::THREADS, 1)
gemm_tf32x3_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                   const TcArgs g) {
  using C = CfgS<BN>;
  constexpr int STAGES = C::STAGES;
  constexpr int PRODUCER_WARP = 12, MMA_WARP = 13;

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

  if (wg == 3) {
    setmaxnreg_dec_56();
    if (warp == PRODUCER_WARP && lane == 0) {
      // ---------------------------------------------------------------- TMA producer
      uint32_t it = 0;
      bool ok = true;
      for (long long tile = blockIdx.x; ok && tile < g.total_tiles; tile += gridDim.x) {
        const TileCoord t = decode_tile(g, tile);
        for (int i = 0; i < total_kb; ++i, ++it) {
          const int r = i / g.k_blocks, kb = i - r * g.k_blocks;
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, abortp, g.wait_limit)) { ok = false; break; }
          const uint32_t full = smem_u32(&bar_full[s]);
          mbar_expect_tx(full, C::RAW_BYTES);
          const uint32_t a_dst = smem_base + s * C::STAGE_BYTES;
          load_operand<BM, C::BK, C::CH, C::MN_LBO>(a_dst, &tma_a, full, g.a_ld, t.mt * BM, kb * C::BK,
                                                     g.a_x1 * t.ib1 + g.a_xr * r, g.a_y0 * t.ib0);
          load_operand<BN, C::BK, C::CH, C::MN_LBO>(a_dst + C::A_BYTES, &tma_b, full, g.b_ld, t.nt * BN, kb * C::BK,
                                                     g.b_x1 * t.ib1 + g.b_xr * r, g.b_y0 * t.ib0);
        }
      }
    } else if (warp == MMA_WARP && lane == 0) {
      // ---------------------------------------------------------------- MMA issuer
      // instruction descriptor: D = f32, A = B = tf32 (format 2), majors, N >> 3, M >> 4
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(g.a_mn ? 1 : 0) << 15) |
                             ((uint32_t)(g.b_mn ? 1 : 0) << 16) | ((uint32_t)(BN >> 3) << 17) |
                             ((uint32_t)(BM >> 4) << 24);
      const uint32_t a_lbo = g.a_mn ? C::MN_LBO : 16u, b_lbo = g.b_mn ? C::MN_LBO : 16u;
      const uint32_t a_sbo = g.a_mn ? C::MN_SBO : C::K_SBO, b_sbo = g.b_mn ? C::MN_SBO : C::K_SBO;
      const uint32_t a_lay = g.a_mn ? C::MN_LAYOUT : C::K_LAYOUT, b_lay = g.b_mn ? C::MN_LAYOUT : C::K_LAYOUT;
      const uint32_t a_kadv = g.a_mn ? C::MN_KADV : C::K_KADV, b_kadv = g.b_mn ? C::MN_KADV : C::K_KADV;
      uint32_t it = 0, ccount = 0;
      bool ok = true;
      for (long long tile = blockIdx.x; ok && tile < g.total_tiles; tile += gridDim.x) {
        for (int kb0 = 0; ok && kb0 < total_kb; kb0 += C::CHUNK_KB, ++ccount) {
          const uint32_t buf = ccount & 1u, cph = (ccount >> 1) & 1u;
          if (!mbar_wait(smem_u32(&bar_tempty[buf]), cph ^ 1u, abortp, g.wait_limit)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + buf * BN;
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
              if (g.xform_mode & 4) {                                         // bit 2: timing experiment
                umma<4>(d_tmem, ad, bd, idesc, (i > 0 || ks > 0) ? 1u : 0u);
                continue;
              }
              umma<4>(d_tmem, ads, bd, idesc, (i > 0 || ks > 0) ? 1u : 0u);   // small * big
              umma<4>(d_tmem, ad, bds, idesc, 1u);                            // big * small
              umma<4>(d_tmem, ad, bd, idesc, 1u);                             // big * big
            }
            umma_commit(smem_u32(&bar_empty[s]));
          }
          if (ok) umma_commit(smem_u32(&bar_tfull[buf]));
        }
      }
    }
    else if (warp >= 14) {
      // ---------------------------------------------------------------- operand split (warps 14, 15)
      split_role<C>(g, smem_base, bar_full, bar_xform, abortp, total_kb, threadIdx.x - 448 + 128);
    }
    __syncwarp();
  } else if (wg == 2) {
    // ------------------------------------------------------------------ operand split (warps 8..11)
    setmaxnreg_dec_56();
    split_role<C>(g, smem_base, bar_full, bar_xform, abortp, total_kb, threadIdx.x - 256);
  } else {
    // ------------------------------------------------------------------ epilogue (warpgroups 0 and 1)
    setmaxnreg_inc_200();
    const int quad = warp & 3;                        // TMEM lane quadrant this warp may read
    const int col_base = wg * C::HALF;                // this warpgroup's half of the tile's columns
    uint32_t ccount = 0;
    bool ok = true;
    for (long long tile = blockIdx.x; ok && tile < g.total_tiles; tile += gridDim.x) {
      const TileCoord t = decode_tile(g, tile);
      float acc[C::HALF];
#pragma unroll
      for (int q = 0; q < C::HALF; ++q) acc[q] = 0.f;
      for (int kb0 = 0; kb0 < total_kb; kb0 += C::CHUNK_KB, ++ccount) {
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
      if (!ok) break;
      const int row = t.mt * BM + quad * 32 + lane;
      if (row < g.m) {
        float* crow = (float*)g.c + t.ib0 * g.c_b0 + t.ib1 * g.c_b1 + (long long)row * g.ldc;
#pragma unroll
        for (int c = 0; c < C::HALF / 32; ++c) {
          const int col0 = t.nt * BN + col_base + c * 32;
          if (col0 < g.n) store_chunk(crow + col0, &acc[c * 32], (g.n - col0) < 32 ? (g.n - col0) : 32, g.beta);
        }
      }
    }
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

// Output canonicalisation: a transposed C (unit row stride) is computed as C^T = B^T A^T.
GemmProblem canonical(const GemmProblem& p) {
  if (p.c_c == 1 || p.n == 1) return p;
  if (p.c_r != 1 && p.m != 1) return p;  // not addressable either way; classification will reject it
  GemmProblem q = p;
  q.m = p.n; q.n = p.m;
  q.a = p.b; q.a_b0 = p.b_b0; q.a_b1 = p.b_b1; q.a_red = p.b_red; q.a_r = p.b_c; q.a_c = p.b_r;
  q.b = p.a; q.b_b0 = p.a_b0; q.b_b1 = p.a_b1; q.b_red = p.a_red; q.b_r = p.a_c; q.b_c = p.a_r;
  q.c_r = p.c_c; q.c_c = p.c_r;
  return q;
}

struct Plan {
  bool ok = false;
  GemmProblem p;
  Layout2D la, lb;
  int64_t ldc = 0;
};

Plan make_plan(const GemmProblem& p0) {
  Plan pl;
  if (p0.dtype == B200_F64) return pl;
  const size_t es = dtype_size(p0.dtype);
  pl.p = canonical(p0);
  const GemmProblem& p = pl.p;
  if (p.m < 1 || p.n < 1 || p.k < 1 || p.b0 < 1 || p.b1 < 1 || p.red < 1) return pl;
  if (p.red > 1 && (p.b0 != 1 || p.b1 != 1)) return pl;
  if (p.m > 0x7fffff00LL || p.n > 0x7fffff00LL || p.k > 0x7fffff00LL) return pl;
  if (p.b0 > 0x7fffffffLL || p.b1 > 0x7fffffffLL || p.red > 0x7fffffffLL) return pl;
  pl.la = classify(p.m, p.k, p.a_r, p.a_c, es);
  pl.lb = classify(p.k, p.n, p.b_r, p.b_c, es);
  if (!pl.la.ok || !pl.lb.ok) return pl;
  const int64_t align = 16 / (int64_t)es;
  // C: row-major with an aligned leading dimension (vector stores in the epilogue).
  if (p.n == 1) pl.ldc = p.c_r; else if (p.c_c == 1) pl.ldc = p.c_r; else return pl;
  if (p.m == 1 && pl.ldc <= 0) pl.ldc = (p.n + align - 1) / align * align;
  if (pl.ldc <= 0 || pl.ldc % align) return pl;
  if (((uintptr_t)p.a | (uintptr_t)p.b | (uintptr_t)p.c) & 15) return pl;
  if (!batch_stride_ok(p.b0, p.a_b0, es) || !batch_stride_ok(p.b1, p.a_b1, es) ||
      !batch_stride_ok(p.red, p.a_red, es) || !batch_stride_ok(p.b0, p.b_b0, es) ||
      !batch_stride_ok(p.b1, p.b_b1, es) || !batch_stride_ok(p.red, p.b_red, es))
    return pl;
  if ((p.b0 > 1 && (p.c_b0 <= 0 || p.c_b0 % align)) || (p.b1 > 1 && (p.c_b1 <= 0 || p.c_b1 % align))) return pl;
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

int g_xform_mode = 1;
int g_force_bn = 0;   // 0 = choose by problem shape
int g_mn_box5 = 1;    // MN-major operands: one 5-D TMA box per stage where the extent allows

// C: CfgH<BN> or CfgS<BN>; KERNEL: the matching kernel.
template <typename C, int ESIZE, int BN, typename Kernel>
int launch_cfg(const Plan& pl, cudaStream_t stream, Kernel kernel) {
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
  const CUtensorMapSwizzle sw_k = (ESIZE == 2) ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  const CUtensorMapSwizzle sw_mn = (ESIZE == 2) ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B;

  // MN-major operands whose MN extent is a whole number of chunks come in with one 5-D box per stage
  // (a partial last chunk would make that box read past the end of a row).
  const int a_ld = !a_mn ? 0 : ((p.m % C::CH == 0 && g_mn_box5) ? 2 : 1);
  const int b_ld = !b_mn ? 0 : ((p.n % C::CH == 0 && g_mn_box5) ? 2 : 1);
  alignas(64) CUtensorMap ma, mb;
  int st;
  if (a_ld == 0)      st = encode_map(&ma, p.a, ESIZE, p.k, p.m, pl.la.ld, a_xn, a_xs, a_yn, p.a_b0, C::BK, BM, sw_k);
  else if (a_ld == 1) st = encode_map(&ma, p.a, ESIZE, p.m, p.k, pl.la.ld, a_xn, a_xs, a_yn, p.a_b0, C::CH, C::BK, sw_mn);
  else                st = encode_map_mn5(&ma, p.a, ESIZE, p.m, p.k, pl.la.ld, a_xn, a_xs, a_yn, p.a_b0, C::CH, C::BK,
                                          BM / C::CH, sw_mn);
  if (st) return st;
  if (b_ld == 0)      st = encode_map(&mb, p.b, ESIZE, p.k, p.n, pl.lb.ld, b_xn, b_xs, b_yn, p.b_b0, C::BK, BN, sw_k);
  else if (b_ld == 1) st = encode_map(&mb, p.b, ESIZE, p.n, p.k, pl.lb.ld, b_xn, b_xs, b_yn, p.b_b0, C::CH, C::BK, sw_mn);
  else                st = encode_map_mn5(&mb, p.b, ESIZE, p.n, p.k, pl.lb.ld, b_xn, b_xs, b_yn, p.b_b0, C::CH, C::BK,
                                          BN / C::CH, sw_mn);
  if (st) return st;

  TcArgs g;
  g.m = (int)p.m; g.n = (int)p.n;
  g.m_tiles = (int)((p.m + BM - 1) / BM);
  g.n_tiles = (int)((p.n + BN - 1) / BN);
  g.nb1 = (int)p.b1;
  g.total_tiles = (long long)g.m_tiles * g.n_tiles * p.b0 * p.b1;
  g.red = (int)p.red;
  g.k_blocks = (int)((p.k + C::BK - 1) / C::BK);
  g.a_mn = a_mn; g.b_mn = b_mn;
  g.a_ld = a_ld; g.b_ld = b_ld;
  g.a_x1 = (!reduce && a_xn > 1) ? 1 : 0; g.a_xr = (reduce && a_xn > 1) ? 1 : 0; g.a_y0 = (a_yn > 1) ? 1 : 0;
  g.b_x1 = (!reduce && b_xn > 1) ? 1 : 0; g.b_xr = (reduce && b_xn > 1) ? 1 : 0; g.b_y0 = (b_yn > 1) ? 1 : 0;
  g.c = p.c; g.c_b0 = p.c_b0; g.c_b1 = p.c_b1; g.ldc = pl.ldc;
  g.beta = p.beta;
  g.xform_mode = g_xform_mode;
  g.wait_limit = 400000000LL + (long long)g.red * g.k_blocks * 40000LL;
  g.status = ds->status;

  const long long grid = g.total_tiles < ds->sm_count ? g.total_tiles : ds->sm_count;
  if (grid <= 0) return B200_OK;
  kernel<<<(unsigned)grid, C::THREADS, C::SMEM_BYTES, stream>>>(ma, mb, g);
  count_launch(true);
  return note_cuda_error(cudaGetLastError(), "tensor-core gemm launch");
}

template <int ESIZE, int BN>
int launch_bn(const Plan& pl, cudaStream_t stream) {
  if constexpr (ESIZE == 2) return launch_cfg<CfgH<BN>, 2, BN>(pl, stream, gemm_f16_kernel<BN>);
  else return launch_cfg<CfgS<BN>, 4, BN>(pl, stream, gemm_tf32x3_kernel<BN>);
}

template <int ESIZE>
int launch_es(const Plan& pl, cudaStream_t stream) {
  const GemmProblem& p = pl.p;
  DeviceState* ds = device_state();
  const int sms = ds ? ds->sm_count : 148;
  auto tiles = [&](int bn) {
    return ((p.m + BM - 1) / BM) * ((p.n + bn - 1) / bn) * p.b0 * p.b1;
  };
  // Tile width by a wave model: time ~ ceil(tiles / SMs) * (cost of one tile of that width).  The
  // relative per-tile costs are measured (a 128-wide tile takes about 3/4 of the time of a 256-wide
  // one because its main loop is bound by shared-memory bandwidth, not by the tensor pipe).
  const double w256 = 1.0, w128 = (ESIZE == 4) ? 0.75 : 0.87, w64 = (ESIZE == 4) ? 0.55 : 0.70;
  auto waves = [&](int bn_) { return (double)((tiles(bn_) + sms - 1) / sms); };
  int bn = 64;
  double best = waves(64) * w64;
  if (p.n > 64 && waves(128) * w128 <= best) { best = waves(128) * w128; bn = 128; }
  if (p.n > 128 && waves(256) * w256 <= best) { best = waves(256) * w256; bn = 256; }
  if (g_force_bn) bn = g_force_bn;
  switch (bn) {
    case 256: return launch_bn<ESIZE, 256>(pl, stream);
    case 128: return launch_bn<ESIZE, 128>(pl, stream);
    default: return launch_bn<ESIZE, 64>(pl, stream);
  }
}

template <typename C, typename Kernel>
int set_attr(Kernel kernel) {
  return note_cuda_error(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES),
                         "cudaFuncSetAttribute");
}

}  // namespace

bool tc_eligible(const GemmProblem& p) { return make_plan(p).ok; }

int tc_setup_device() {
  int st = 0;
  if ((st = set_attr<CfgH<64>>(gemm_f16_kernel<64>))) return st;
  if ((st = set_attr<CfgH<128>>(gemm_f16_kernel<128>))) return st;
  if ((st = set_attr<CfgH<256>>(gemm_f16_kernel<256>))) return st;
  if ((st = set_attr<CfgS<64>>(gemm_tf32x3_kernel<64>))) return st;
  if ((st = set_attr<CfgS<128>>(gemm_tf32x3_kernel<128>))) return st;
  if ((st = set_attr<CfgS<256>>(gemm_tf32x3_kernel<256>))) return st;
  return encode_fn() ? B200_OK : B200_ERR_CUDA;
}

int launch_gemm_tc(const GemmProblem& p, cudaStream_t stream) {
  const Plan pl = make_plan(p);
  if (!pl.ok) return B200_ERR_UNSUPPORTED;
  if (p.dtype == B200_F32) return launch_es<4>(pl, stream);
  return launch_es<2>(pl, stream);
}

void tc_set_xform_mode(int mode) { g_xform_mode = mode; }
void tc_set_tile_n(int bn) { g_force_bn = bn; }
void tc_set_mn_box5(int on) { g_mn_box5 = on; }

}  // namespace b200
