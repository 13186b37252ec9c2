// Device side of k::Shadow: the bf16 copy a producer kernel writes next to its
// f32 output.  Same rounding as the GEMM path's own conversion kernel
// (round to nearest even), the consumer's per-column factor
// applied first when it has one.
#ifndef SEE_CUDA_SHADOW_CUH_
#define SEE_CUDA_SHADOW_CUH_

#include "kernels.h"

namespace see::k {

// The hardware conversion: round to nearest even, NaN to the canonical quiet NaN.
__device__ __forceinline__ uint32_t ShadowBf16(float f) {
  uint16_t r;
  asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(r) : "f"(f));
  return r;
}
__device__ __forceinline__ uint32_t ShadowBf16x2(float lo, float hi) {   // lo in bits 0..15
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// Four consecutive elements of one row: flat index 4 * i4, first column `col`
// (callers know their column; computing it here would cost a 64-bit modulo
// per vector).
__device__ __forceinline__ void ShadowStore4(const Shadow& sh, size_t i4, uint32_t col, float4 v) {
  if (sh.k_scale) {
    const float4 sc = __ldg(reinterpret_cast<const float4*>(sh.k_scale + col));
    v.x *= sc.x; v.y *= sc.y; v.z *= sc.z; v.w *= sc.w;
  }
  uint2 r;
  r.x = ShadowBf16x2(v.x, v.y);
  r.y = ShadowBf16x2(v.z, v.w);
  reinterpret_cast<uint2*>(sh.dst)[i4] = r;
}

// Column bookkeeping for a grid-stride loop over float4 units of a [rows][cols]
// tensor: the column of unit i is kept incrementally instead of recomputed.
struct ShadowCursor {
  uint32_t col4, step4, cols4;
  __device__ __forceinline__ ShadowCursor(const Shadow& sh, size_t first_unit, size_t stride_units) {
    cols4 = sh.dst ? static_cast<uint32_t>(sh.cols / 4) : 1u;
    col4 = static_cast<uint32_t>(first_unit % cols4);
    step4 = static_cast<uint32_t>(stride_units % cols4);
  }
  __device__ __forceinline__ uint32_t col() const { return col4 * 4; }
  __device__ __forceinline__ void advance() {
    col4 += step4;
    if (col4 >= cols4) col4 -= cols4;
  }
};

}  // namespace see::k

#endif  // SEE_CUDA_SHADOW_CUH_
