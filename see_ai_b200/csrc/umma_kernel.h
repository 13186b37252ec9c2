// Interface between the tensor-core GEMM kernel (k_gemm_umma.cu) and its host
// planner (umma_gemm.cc).
#ifndef SEE_CUDA_UMMA_KERNEL_H_
#define SEE_CUDA_UMMA_KERNEL_H_

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "kernels.h"

namespace see::k {

namespace umma_cfg {
constexpr uint32_t kBlockM = 128, kBlockN = 128, kBlockK = 64, kStages = 3;
}

struct UmmaEpilogue {
  float* C;                 // [M, N] f32
  const float* addend;      // [M, N] or null:  v = d + v (before the bias, or after it when addend_last)
  const float* bias;        // [N] or null:     v = v + bias[n]
  const float* col_scale;   // [N] or null:     v = acc * col_scale[n]   (else acc * alpha)
  float alpha;
  int act;
  uint32_t M, N, K;
  DeviceStatus* status;
  // A following activation instruction absorbed into this epilogue.  With v the
  // value above (after scale, addend, bias, act):
  //   kFuseActFwd: g = act(v);          kFuseActBwd: g = act'(dy = v, x = fuse_x[m, n]).
  // g leaves only as the bf16 operand copy of the GEMM that consumes it
  // (shadow_dst, [M, N], times shadow_k_scale[n] when set); v itself is stored to
  // C only when store_c is set.
  int fuse_mode = 0;
  int fuse_act = 0;
  const float* fuse_x = nullptr;
  uint16_t* shadow_dst = nullptr;
  const float* shadow_k_scale = nullptr;
  int store_c = 1;
  int addend_last = 0;
  // A low-rank term folded into the product: after the main operands' K the
  // reduction continues over aux_k_blocks blocks of 64 from a second operand
  // pair, T' [M, 64 * aux_k_blocks] and B' [N, 64 * aux_k_blocks] (bf16, K-major),
  // so the tile holds A W^T + T' B'^T before the epilogue scales it.  With T' and
  // B' the three-way bf16 splits of f32 factors (LoraSplit* in kernels.h) the
  // added term is the f32 product t . b to about 2^-23 of |t| |b|.
  uint32_t aux_k_blocks = 0;
  // The stored value also as bf16 [M, N] (GemmArgs::pack_dst).
  uint16_t* pack_dst = nullptr;
};

size_t UmmaSmemBytes();
// map_a: bf16 [M, K] row-major, box {64, 128}, 128-byte swizzle; map_b: bf16 [N, K] likewise.
cudaError_t UmmaGemmLaunch(const CUtensorMap& map_a, const CUtensorMap& map_b,
                           const UmmaEpilogue& ep, cudaStream_t s, const CUtensorMap* aux_a = nullptr,
                           const CUtensorMap* aux_b = nullptr);
// Large products run on CTA pairs (cta_group::2) by default; off = one CTA per tile.  Process-wide.
void UmmaSetCtaPairs(bool on);
// dst[N][K] (bf16 bits) from src [K][N] (transpose) or [N][K]; int8 and bf16 widen exactly.
// k_scale (or null): dst[n][k] = bf16(src * k_scale[k]).
void WeightToBf16(const void* src, BType type, uint16_t* dst, uint32_t N, uint32_t K,
                  bool transpose, const float* k_scale, cudaStream_t s);

}  // namespace see::k

#endif  // SEE_CUDA_UMMA_KERNEL_H_
