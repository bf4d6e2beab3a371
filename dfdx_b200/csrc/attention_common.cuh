// Helpers shared by the fused attention kernels (attention.cu: forward, attention_bwd.cu: backward).
#pragma once
#include "tc_device.cuh"
#include <mutex>

namespace b200 {
namespace attn {

using namespace tcx;

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

// Bounded wait whose verdict is the same in every lane of the warp.  The code after it issues warp-collective
// instructions (tcgen05.ld / tcgen05.wait, .sync.aligned): if one lane gave up and the others did not, the warp
// would reach them with a partial mask, which never completes.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag, long long limit) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, limit));
}

// One mbarrier arrival for the whole warp, after every lane has reached this point (each lane has issued its
// own fence before the call).  128 single arrivals per hand-off serialise on the barrier word.
__device__ __forceinline__ void warp_arrive(uint32_t bar, int lane) {
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

inline EncodeTiledFn attn_encode_fn() {
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
inline int encode_bhsd(CUtensorMap* map, const void* base, int64_t d, int64_t s, int64_t h, int64_t b, int64_t ss,
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

inline bool stride_ok(int64_t extent, int64_t stride) { return extent <= 1 || (stride > 0 && stride % 8 == 0); }


}  // namespace attn
}  // namespace b200
