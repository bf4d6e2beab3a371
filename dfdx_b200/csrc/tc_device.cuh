// Device-side building blocks shared by the tensor-core GEMM kernels (gemm_tc.cu: one CTA per MMA;
// gemm_tc_pair.cu: CTA pairs): PTX wrappers for mbarriers, TMA, tcgen05 and TMEM, the shared-memory
// descriptor, tile configurations, kernel arguments and the epilogue store.
#pragma once
#include "common.cuh"
#include <cuda.h>

namespace b200 {
namespace tcx {

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
// Tiled 4-D TMA store shared -> global (bulk async-group completion).  Rows / columns of the box that fall outside
// the tensor are not written.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
      ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
// The same box added element-wise into global memory (f16 add performed by the memory system).
__device__ __forceinline__ void tma_reduce_add_4d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
      ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until at most N of this thread's bulk groups still have to READ their shared-memory source.
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// Named barrier over `count` threads (id 0 is __syncthreads).
__device__ __forceinline__ void named_barrier_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
// The same barrier carrying a vote: returns true iff `pred` holds in every participating thread.
__device__ __forceinline__ bool named_barrier_and(int id, int count, bool pred) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 q, %3, 0;\n\t"
      "barrier.cta.red.and.pred p, %1, %2, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(out) : "r"(id), "r"(count), "r"((uint32_t)pred) : "memory");
  return out != 0;
}
__device__ __forceinline__ void st_shared_v4_u32(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
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
// The same MMA with each shared-memory descriptor given as (low, high) 32-bit words.  Inside a kernel the high
// word (stride offset, version, swizzle mode) is constant and the low word ((address >> 4) | (leading offset
// >> 4) << 16) moves by a constant per stage and k-step, so the issuing thread spends one integer add per
// descriptor instead of rebuilding 64-bit fields: that thread's dependent instruction chain, competing for
// issue slots with the busy warps of its scheduler, otherwise bounds how fast MMAs are issued.
template <int ESIZE>
__device__ __forceinline__ void umma_lohi(uint32_t d_tmem, uint32_t alo, uint32_t ahi, uint32_t blo, uint32_t bhi,
                                          uint32_t idesc, uint32_t accumulate) {
  if constexpr (ESIZE == 2) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %6, 0;\n\t"
        "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
        ::"r"(d_tmem), "r"(alo), "r"(ahi), "r"(blo), "r"(bhi), "r"(idesc), "r"(accumulate) : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %6, 0;\n\t"
        "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], da, db, %5, p;\n\t}"
        ::"r"(d_tmem), "r"(alo), "r"(ahi), "r"(blo), "r"(bhi), "r"(idesc), "r"(accumulate) : "memory");
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

// Register split of the single-CTA f32 kernel.  setmaxnreg only redistributes what the CTA was given at
// launch (640 threads x 96 registers = 61440): a request beyond that blocks forever, so the budget is
// checked at compile time.
constexpr int F32_REGS_LAUNCH = 96, F32_REGS_EPI = 192, F32_REGS_LOW = 32, F32_REGS_SPLIT = 32;
static_assert(2 * 128 * F32_REGS_EPI + 128 * F32_REGS_LOW + 2 * 128 * F32_REGS_SPLIT <= 640 * F32_REGS_LAUNCH,
              "setmaxnreg budget exceeds the CTA's launch allocation");
__device__ __forceinline__ void setmaxnreg_dec_low() { asm volatile("setmaxnreg.dec.sync.aligned.u32 32;"); }
__device__ __forceinline__ void setmaxnreg_dec_split() { asm volatile("setmaxnreg.dec.sync.aligned.u32 32;"); }
__device__ __forceinline__ void setmaxnreg_inc_epi() { asm volatile("setmaxnreg.inc.sync.aligned.u32 192;"); }
// Pair f32 kernel (512 threads x 128 registers = 65536): 2 x 128 x 200 + 2 x 128 x 56 = 65536.
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
  static constexpr int THREADS = 320;                       // 8 epilogue warps, TMA producer warp, MMA warp
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int OUT_BYTES = 128 * 128;               // one staged output group: 128 rows x 64 f16 (TMA-store epilogue)
  static constexpr int OFF_OUT = STAGES * STAGE_BYTES;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 2 * OUT_BYTES + 1024;
  static constexpr uint32_t LAYOUT = 2u;                    // SWIZZLE_128B
  static constexpr uint32_t SBO = 1024;                     // 8 rows of 128 bytes
  static constexpr uint32_t MN_LBO = BK * 128;              // distance between MN-major chunks
  static constexpr uint32_t MN_KADV = 2 * 1024;             // 16 k rows per MMA
  static constexpr uint32_t K_KADV = 32;                    // 16 elements of K per MMA
};

// f16, 256 x 256 output tile per CTA (two 128-row accumulators that fill the 512 TMEM columns): per 64-wide k-block
// 64 KB are staged and the MMAs read 96 KB for 1024 tensor clocks, 160 B/clock against the 192 B/clock of the
// 128 x 256 tile, which is what lets the main loop run at the tensor pipe's pace.  No spare TMEM, so a tile's
// epilogue does not overlap the next tile's main loop: for long K and outputs of many tiles.
struct CfgHB {
  static constexpr int BMB = 256, BN = 256;
  static constexpr int BK = 64, CH = 64, KSTEPS = 4;
  static constexpr int A_BYTES = BMB * 128;
  static constexpr int B_BYTES = BN * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = 3;
  static constexpr int THREADS = 320;                       // 8 epilogue warps, TMA producer warp, MMA warp
  static constexpr int TMEM_COLS = 512;
  static constexpr int OUT_BYTES = 128 * 128;               // one staged output group per epilogue warp group
  static constexpr int OFF_OUT = STAGES * STAGE_BYTES;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 2 * OUT_BYTES + 1024;
  static constexpr uint32_t LAYOUT = 2u;                    // SWIZZLE_128B
  static constexpr uint32_t SBO = 1024;
  static constexpr uint32_t MN_LBO = BK * 128;
  static constexpr uint32_t MN_KADV = 2 * 1024;
  static constexpr uint32_t K_KADV = 32;
  static constexpr uint32_t A_HALF = 128 * 128;             // bytes from the first to the second 128-row block of A
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
  static constexpr int THREADS = 640;                       // 5 warpgroups: 2 epilogue, 1 producer + MMA, 2 operand split
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int OUT_BYTES = 128 * 128;               // one staged output group per epilogue warpgroup: 128 rows x 32 f32
  static constexpr int OFF_OUT = STAGES * STAGE_BYTES;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 2 * OUT_BYTES + 1024;
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
  int n_fast;                     // tile order inside a batch item: 1 = N tiles fastest, 0 = M tiles fastest
  long long total_tiles;
  int ksplit, kb_per_slice;       // f32 kernel: K is cut into ksplit slices of kb_per_slice k-blocks; a work unit is
  long long total_units;          // (tile, slice); slices of one tile add their partial results atomically
  // f32 kernel, ksplit == 1: when the tiles do not fill a whole number of waves, the (tile, k-block) space of the
  // last, partial wave (tiles >= tail_from) is dealt out as one contiguous range of tail_per k-blocks per CTA, so
  // that every SM gets an equal share; a range touches at most tail_parts tiles, parts of tiles add their partial
  // results atomically like split-K slices.  tail_per == 0: off.
  long long tail_from;
  int tail_per, tail_parts;
  // fewer tiles than CTAs (beta = 1): k-blocks [0, kt_cut) of tile c on CTA c, the rest on the other CTAs, kt_per
  // tiles each (decode_unit).  kt_cut == 0: off.
  int kt_cut, kt_per;
  int streamk;                    // f32 kernel: the (tile, k-block) space is cut into one contiguous range per CTA
  long long sk_per_cta;           // k-blocks per CTA; a unit is the part of one tile inside the CTA's range (may be empty)
  float* split_out;               // f16 kernel with ksplit > 1: f32 scratch (m x split_ld, zeroed) that takes the
  long long split_ld;             // partial sums; a finalize kernel then writes C = f16(beta*C + scratch)
  int red, k_blocks;              // k iterations per tile = red * k_blocks
  int a_mn, b_mn;                 // operand is MN-major (else K-major)
  int a_ld, b_ld;                 // load_operand mode: 0 K-major, 1 MN-major per chunk, 2 MN-major one box
  int a_x1, a_xr, a_y0;           // TMA x = a_x1*ib1 + a_xr*r ; y = a_y0*ib0
  int b_x1, b_xr, b_y0;
  void* c;
  long long c_b0, c_b1, ldc;      // element strides
  int c_col;                      // 0: C(i,j) at i*ldc + j (row store); 1: at j*ldc + i (column store)
  int c_wide;                     // row store: every row start is 32-byte aligned (256-bit accesses)
  int c_tma;                      // f16 kernel, row store: groups of 64 columns are staged in shared memory and leave by
                                  // TMA (tensor map `tma_c`) instead of per-thread row accesses: 1 = store (beta = 0),
                                  // 2 = element-wise add into C (beta = 1: C += f16(acc), two roundings instead of one)
  int beta;
  int xform_mode;                 // f32: 1 = big stays raw, write small only; 0 = also rewrite big = tf32_rn(x)
  long long wait_limit;           // clock cycles
  int* status;
  // optional epilogue (beta == 0, no split-K):  C = act(alpha * acc + bias)
  int fused;                      // any of the three below is active
  float alpha;
  const void* bias;               // C's element type, 16-byte aligned; indexed by the kernel's column, or
  int bias_row;                   // (bias_row) by the kernel's row
  int acc32;                      // f16 kernels: the f32 accumulator is added to an f32 C through bulk reduce-adds
  int act;                        // B200_ACT_*
  // Implicit convolution (f32 kernel, template parameter CV != 0): the im2col happens in the TMA loads.
  //   CV 1 (forward / data gradient): the B tile of k-block (tap, channel block) is ONE box of a channels-last
  //        image, `cv_rows` image rows x `cv_wout` pixels x 16 channels, shifted by the tap; an N tile is those
  //        cv_rows x cv_wout output positions of one image (ib0), group ib1.
  //   CV 2 (filter gradient): the reduction runs over output positions, 16 pixels of one image row per k-block
  //        (red = images); A is a box of grad_out, B tile chunk j is a box of the channels-last image for the tap
  //        and channel range that columns 32 j .. 32 j + 31 of the tile stand for.
  int tile_cols;                  // output columns from one N tile to the next (BN for a plain GEMM)
  int tile_valid;                 // columns of a tile that exist (<= tile_cols)
  int mma_n;                      // N of the MMA instruction (multiple of 16, >= tile_valid)
  int b_tx_bytes;                 // bytes the B loads of one stage deliver
  int cv_cblocks;                 // CV 1: k-blocks per tap (padded channels per group / 16)
  int cv_cpad;                    // padded channels per group in the channels-last image
  int cv_kw, cv_taps;             // filter taps per row, taps in all
  int cv_w0, cv_dw, cv_h0, cv_dh; // tap (k1, k2) reads the image at (row + cv_h0 + k1 * cv_dh, col + cv_w0 + k2 * cv_dw)
  int cv_rows, cv_wout;           // CV 1: image rows and pixels per row of one N tile; CV 2: cv_rows = output rows per image
  int cv_wblocks;                 // CV 2: k-blocks per row of boxes (ceil(w_out / cv_bw)); cv_rows = rows of boxes per image
  int cv_bw, cv_bh;               // CV 2: a k-block's 16 output pixels are a box of cv_bw x cv_bh pixels
  int m64;                        // CV 1: the output has at most 64 rows: A boxes of 64 rows, MMAs with M = 64
};

// Fused epilogue on 32 consecutive accumulator columns [col0, col0+32) of output row `row` (row < m):
// f = act(alpha * f + bias).  T is C's element type (the bias has the same type).
__device__ __forceinline__ float bias_to_float(float x) { return x; }
__device__ __forceinline__ float bias_to_float(__half x) { return __half2float(x); }

template <typename T>
__device__ __forceinline__ void fused_epilogue(float* f, const TcArgs& g, int row, int col0, int valid) {
  const T* bias = reinterpret_cast<const T*>(g.bias);
  const float alpha = g.alpha;
  if (bias == nullptr) {
#pragma unroll
    for (int q = 0; q < 32; ++q) f[q] *= alpha;
  } else if (g.bias_row) {
    const float br = bias_to_float(__ldg(bias + row));
#pragma unroll
    for (int q = 0; q < 32; ++q) f[q] = fmaf(f[q], alpha, br);
  } else if (valid == 32) {
    // all lanes read the same 32 bias values: broadcast 16-byte loads
    constexpr int PER = 16 / (int)sizeof(T);          // elements per 16-byte vector
#pragma unroll
    for (int v = 0; v < 32 / PER; ++v) {
      const uint4 raw = __ldg(reinterpret_cast<const uint4*>(bias + col0) + v);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int q = 0; q < PER; ++q) f[v * PER + q] = fmaf(f[v * PER + q], alpha, bias_to_float(e[q]));
    }
  } else {
#pragma unroll
    for (int q = 0; q < 32; ++q)
      if (q < valid) f[q] = fmaf(f[q], alpha, bias_to_float(__ldg(bias + col0 + q)));
  }
  if (g.act == B200_ACT_RELU) {
#pragma unroll
    for (int q = 0; q < 32; ++q) f[q] = fmaxf(f[q], 0.f);
  }
}

// The same with a column bias that waits in shared memory as f32 (`bs`: this chunk's 32 values, zeros where there is
// no bias or no column): broadcast 16-byte reads instead of global loads in the accumulator's way.
__device__ __forceinline__ void fused_epilogue_cols(float* f, const TcArgs& g, const float* bs) {
  const float alpha = g.alpha;
  const float4* b4 = reinterpret_cast<const float4*>(bs);
#pragma unroll
  for (int v = 0; v < 8; ++v) {
    const float4 b = b4[v];
    f[4 * v] = fmaf(f[4 * v], alpha, b.x);
    f[4 * v + 1] = fmaf(f[4 * v + 1], alpha, b.y);
    f[4 * v + 2] = fmaf(f[4 * v + 2], alpha, b.z);
    f[4 * v + 3] = fmaf(f[4 * v + 3], alpha, b.w);
  }
  if (g.act == B200_ACT_RELU) {
#pragma unroll
    for (int q = 0; q < 32; ++q) f[q] = fmaxf(f[q], 0.f);
  }
}

// The same with the bias kept as f16 in shared memory (where the f32 copy does not fit).
__device__ __forceinline__ void fused_epilogue_cols(float* f, const TcArgs& g, const __half* bs) {
  const float alpha = g.alpha;
  const uint4* b4 = reinterpret_cast<const uint4*>(bs);
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    const uint4 raw = b4[v];
    const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 b = __half22float2(h2[e]);
      f[8 * v + 2 * e] = fmaf(f[8 * v + 2 * e], alpha, b.x);
      f[8 * v + 2 * e + 1] = fmaf(f[8 * v + 2 * e + 1], alpha, b.y);
    }
  }
  if (g.act == B200_ACT_RELU) {
#pragma unroll
    for (int q = 0; q < 32; ++q) f[q] = fmaxf(f[q], 0.f);
  }
}

// 256-bit global accesses (sm_100): one 32-byte sector per thread and instruction.
__device__ __forceinline__ void ld_global_v8(const void* p, uint32_t (&r)[8]) {
  asm volatile("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "l"(p));
}
__device__ __forceinline__ void st_global_v8(void* p, const uint32_t (&r)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"l"(p), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}

// 32 consecutive f32 accumulator columns of one output row -> global memory.  `wide`: the row start is
// 32-byte aligned, so whole sectors are written per thread; otherwise 16-byte pieces.
__device__ __forceinline__ void store_chunk(float* dst, const float* v, int valid, int beta, int wide) {
  if (valid == 32 && wide) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint32_t o[8];
      if (beta) {
        uint32_t old[8];
        ld_global_v8(dst + 8 * q, old);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = __float_as_uint(v[8 * q + e] + __uint_as_float(old[e]));
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = __float_as_uint(v[8 * q + e]);
      }
      st_global_v8(dst + 8 * q, o);
    }
  } else if (valid == 32) {
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

// The 32 f16 values (64 bytes) a row already holds at dst, as 16 packed registers.
__device__ __forceinline__ void load_old_f16(const __half* src, uint32_t (&old)[16], int wide) {
  if (wide) {
    uint32_t a[8], b[8];
    ld_global_v8(src, a);
    ld_global_v8(src + 16, b);
#pragma unroll
    for (int e = 0; e < 8; ++e) { old[e] = a[e]; old[8 + e] = b[e]; }
  } else {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint4 t = *reinterpret_cast<const uint4*>(src + 8 * q);
      old[4 * q] = t.x; old[4 * q + 1] = t.y; old[4 * q + 2] = t.z; old[4 * q + 3] = t.w;
    }
  }
}
__device__ __forceinline__ void add_old_f16(float* v, const uint32_t (&old)[16]) {
#pragma unroll
  for (int e = 0; e < 16; ++e) {
    const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&old[e]));
    v[2 * e] += t.x; v[2 * e + 1] += t.y;
  }
}

__device__ __forceinline__ void store_chunk(__half* dst, const float* v, int valid, int beta, int wide) {
  if (valid == 32) {
    uint32_t pk[16];
    if (beta) {
      uint32_t old[16];
      load_old_f16(dst, old, wide);
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&old[e]));
        const __half2 h = __floats2half2_rn(v[2 * e] + t.x, v[2 * e + 1] + t.y);
        pk[e] = *reinterpret_cast<const uint32_t*>(&h);
      }
    } else {
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        const __half2 h = __floats2half2_rn(v[2 * e], v[2 * e + 1]);
        pk[e] = *reinterpret_cast<const uint32_t*>(&h);
      }
    }
    if (wide) {
      uint32_t a[8], b[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) { a[e] = pk[e]; b[e] = pk[8 + e]; }
      st_global_v8(dst, a);
      st_global_v8(dst + 16, b);
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q)
        *reinterpret_cast<uint4*>(dst + 8 * q) = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
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

// Column store: the 32 lanes of a warp hold 32 consecutive rows, so for every column they write 32
// consecutive elements.  dst points at (row, col0); v holds the row's 32 columns from col0 on.
template <typename OutT>
__device__ __forceinline__ void store_chunk_col(OutT* dst, const float* v, int valid, long long ldc, int beta) {
#pragma unroll
  for (int q = 0; q < 32; ++q)
    if (q < valid) {
      float o = v[q];
      if constexpr (sizeof(OutT) == 2) {
        if (beta) o += __half2float(dst[q * ldc]);
        dst[q * ldc] = __float2half_rn(o);
      } else {
        if (beta) o += dst[q * ldc];
        dst[q * ldc] = o;
      }
    }
}

// Split-K: partial results of a K slice are added into C (which holds beta*C_old, or zeros) with vector
// reductions; the order of the additions is not fixed, so the last bits can differ between runs.
__device__ __forceinline__ void add_chunk_atomic(float* dst, const float* v, int valid) {
  if (valid == 32) {
#pragma unroll
    for (int q = 0; q < 8; ++q)
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                   ::"l"(dst + 4 * q), "f"(v[4 * q]), "f"(v[4 * q + 1]), "f"(v[4 * q + 2]), "f"(v[4 * q + 3]) : "memory");
  } else {
#pragma unroll
    for (int q = 0; q < 32; ++q)
      if (q < valid) atomicAdd(dst + q, v[q]);
  }
}
__device__ __forceinline__ void add_chunk_atomic_col(float* dst, const float* v, int valid, long long ldc) {
#pragma unroll
  for (int q = 0; q < 32; ++q)
    if (q < valid) atomicAdd(dst + q * ldc, v[q]);
}

struct TileCoord { int mt, nt, ib0, ib1; };
struct Unit { long long tile; int kb_lo, kb_hi; };
// Work unit -> (tile, k-block range) for a launch of `grid` CTAs; CTA c takes units c, c + grid, ...  A pure function of
// its arguments (the host-side test of the schedules calls it as it is).
__host__ __device__ __forceinline__ Unit decode_unit_on(const TcArgs& g, long long unit, int total_kb, long long grid) {
  Unit u;
  if (g.streamk) {
    // unit = blockIdx.x + i * grid is the i-th tile that CTA blockIdx.x's k-block range touches
    const long long cta = unit % grid, i = unit / grid;
    const long long start = cta * g.sk_per_cta;
    long long end = start + g.sk_per_cta;
    const long long all = g.total_tiles * (long long)total_kb;
    if (end > all) end = all;
    u.tile = start / total_kb + i;
    const long long t0 = u.tile * (long long)total_kb;
    const long long lo = start > t0 ? start : t0, hi = end < t0 + total_kb ? end : t0 + total_kb;
    if (hi <= lo || u.tile >= g.total_tiles) { u.tile = 0; u.kb_lo = u.kb_hi = 0; }   // nothing of that tile in the range
    else { u.kb_lo = (int)(lo - t0); u.kb_hi = (int)(hi - t0); }
    return u;
  }
  if (g.kt_cut > 0) {
    // Fewer tiles than CTAs, an output that is added to: CTA c < tiles takes k-blocks [0, kt_cut) of tile c -- all of
    // them at the same K position at the same time, so that the CTAs of a row / column of tiles share their operand
    // panels in L2 as in the unsplit launch -- and the remaining CTAs take the tiles' last k-blocks [kt_cut, total),
    // kt_per tiles each.
    const long long part = unit / grid, cta = unit - part * grid;
    u.tile = 0; u.kb_lo = u.kb_hi = 0;
    if (cta < g.total_tiles) {
      if (part == 0) { u.tile = cta; u.kb_hi = g.kt_cut; }
    } else {
      const long long seg = (cta - g.total_tiles) * g.kt_per + part;
      if (part < g.kt_per && seg < g.total_tiles) { u.tile = seg; u.kb_lo = g.kt_cut; u.kb_hi = total_kb; }
    }
    return u;
  }
  if (g.tail_per > 0 && unit >= g.tail_from) {
    // unit = tail_from + part * grid + cta: the part-th tile that CTA cta's range of the tail touches
    const long long v = unit - g.tail_from, part = v / grid, cta = v - part * grid;
    const long long all = (g.total_tiles - g.tail_from) * (long long)total_kb;
    const long long start = cta * g.tail_per;
    long long end = start + g.tail_per;
    if (end > all) end = all;
    const long long ti = start / total_kb + part, t0 = ti * (long long)total_kb;
    const long long lo = start > t0 ? start : t0, hi = end < t0 + total_kb ? end : t0 + total_kb;
    u.tile = g.tail_from + ti;
    if (hi <= lo || u.tile >= g.total_tiles) { u.tile = g.tail_from; u.kb_lo = u.kb_hi = 0; }   // nothing of that tile
    else { u.kb_lo = (int)(lo - t0); u.kb_hi = (int)(hi - t0); }
    return u;
  }
  u.tile = unit / g.ksplit;
  const int slice = (int)(unit - u.tile * g.ksplit);
  u.kb_lo = slice * g.kb_per_slice;
  u.kb_hi = u.kb_lo + g.kb_per_slice < total_kb ? u.kb_lo + g.kb_per_slice : total_kb;
  return u;
}
__device__ __forceinline__ Unit decode_unit(const TcArgs& g, long long unit, int total_kb) {
  return decode_unit_on(g, unit, total_kb, (long long)gridDim.x);
}
__device__ __forceinline__ TileCoord decode_tile(const TcArgs& g, long long tile) {
  const long long per_batch = (long long)g.m_tiles * g.n_tiles;
  const long long bt = tile / per_batch;
  const int rem = (int)(tile - bt * per_batch);
  TileCoord t;
  if (g.n_fast) { t.nt = rem % g.n_tiles; t.mt = rem / g.n_tiles; }
  else { t.mt = rem % g.m_tiles; t.nt = rem / g.m_tiles; }
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

}  // namespace tcx
}  // namespace b200
