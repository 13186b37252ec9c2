// The three-way bf16 cut of an f32 value and the order of the six piece products,
// shared by the kernels that prepare a low-rank term's operands (k_lora.cu) and
// the one that produces them straight from its accumulators (k_lora_mma.cu).
#ifndef SEE_CUDA_LORA_SPLIT_CUH_
#define SEE_CUDA_LORA_SPLIT_CUH_

#include <cstdint>

namespace see::k {

__device__ __forceinline__ uint16_t Bf16Rn(float f) {
  uint16_t r;
  asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(r) : "f"(f));
  return r;
}
__device__ __forceinline__ float Bf16ToF32(uint16_t b) { return __uint_as_float(static_cast<uint32_t>(b) << 16); }

// v = p[0] + p[1] + p[2] + (a remainder below 2^-24 |v|); each subtraction is exact.
__device__ __forceinline__ void Split3(float v, uint16_t (&p)[3]) {
  p[0] = Bf16Rn(v);
  const float r1 = v - Bf16ToF32(p[0]);
  p[1] = Bf16Rn(r1);
  const float r2 = r1 - Bf16ToF32(p[1]);
  p[2] = Bf16Rn(r2);
}

// Which piece each of the six K segments takes from the row factor (side 0) and
// from the weight factor (side 1): t2 b0, t1 b1, t0 b2, t1 b0, t0 b1, t0 b0.
__host__ __device__ constexpr int PieceOf(int side, int s) {
  return side == 0 ? (s == 0 ? 2 : (s == 1 || s == 3 ? 1 : 0))
                   : (s == 2 ? 2 : (s == 1 || s == 4 ? 1 : 0));
}

}  // namespace see::k

#endif  // SEE_CUDA_LORA_SPLIT_CUH_
