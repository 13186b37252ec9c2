// Interface of the tensor-core attention kernels (k_attn_umma.cu) to their
// host planner (umma_attn.cc).
#ifndef SEE_CUDA_ATTN_UMMA_H_
#define SEE_CUDA_ATTN_UMMA_H_

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "kernels.h"

namespace see::k {

struct AttnUmmaArgs {
  uint32_t B, S, H, d;
  float inv_sqrt_d;
  float* out;       // O / dQ / dK / dV, f32 [B*S, H*d]
  float* stats;     // f32 [B*H*S, 4]: score max, 1/denominator, delta, start
  DeviceStatus* status;
  Shadow shadow;    // optional bf16 copy of `out` (cols = H*d) for the GEMM that reads it next
  float* out2 = nullptr;   // dK and dV in one walk: dV goes here (out is dK)
  Shadow shadow2;          // and its optional bf16 copy
  // Forward: a second, private copy of O (f32 [B*S, H*d]) kept for the dQ of the same
  // attention (the arena's O is long overwritten by then — its slot usually holds dO).
  float* keep = nullptr;
  // dQ: that copy, and dO's bf16 operand copy ([B*S, H*d], what the tensor core sees).
  // delta_i = sum_j P_ij dP_ij equals dO_i . O_i, so the kernel takes it from one row of
  // each and walks the keys once instead of twice.
  const float* fwd_keep = nullptr;
  const uint16_t* dout_bf16 = nullptr;
};

// f32 [B*S, H*d] -> bf16, same row-major layout (the operand copy the kernels below read).
void PackHeads(const float* x, uint16_t* rows, uint32_t B, uint32_t S, uint32_t H, uint32_t d, cudaStream_t s);

// Maps over that copy: dims {d, S, H, B}, box {64, 128, 1, 1} (a CTA's own 128 rows) or
// {64, 64, 1, 1} (`_half`: the 64 positions of one step); bf16, 128-byte swizzle.  d is 64 or 128.
// A `_half` tile serves both as the K-major operand of a product over the head dimension
// and as the MN-major operand of a product over its 64 positions.
cudaError_t AttnFwdUmma(const CUtensorMap& q, const CUtensorMap& k_half, const CUtensorMap& v_half,
                        const AttnUmmaArgs& a, cudaStream_t s);
cudaError_t AttnDQUmma(const CUtensorMap& q, const CUtensorMap& dout, const CUtensorMap& k_half,
                       const CUtensorMap& v_half, const AttnUmmaArgs& a, cudaStream_t s);
// mode 0: dV (v ignored); 1: dK; 2: both in one walk (a.out = dK, a.out2 = dV; d = 64 only).
cudaError_t AttnDKVUmma(int mode, const CUtensorMap& k, const CUtensorMap& v, const CUtensorMap& q_half,
                        const CUtensorMap& dout_half, const AttnUmmaArgs& a, cudaStream_t s);

}  // namespace see::k

#endif  // SEE_CUDA_ATTN_UMMA_H_
