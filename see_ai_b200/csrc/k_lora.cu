// The low-rank (LoRA) side of an adapted projection, engine mode.
//
// An adapted projection is y = x W + s (x A) B with W frozen and A [k_in, r],
// B [r, n_out] trainable, r = 4..16.  The plan spells it as separate rank-r
// products (reference: compiler/analysis/algebra/lora_grafter.cc:170-206); the
// reference's own GPU backend folds the expand product C' = s T B + C into the
// base GEMM (reference: runtime/executor/metal_backend.mm:1155-1316).  Here the
// fold rides the tensor cores: the f32 factors are cut into three bf16 pieces
// each, t = t0 + t1 + t2, b = b0 + b1 + b2 (every piece the bf16 rounding of
// what the earlier pieces left, so the pieces are exact and the remainder is
// below 2^-24 |t|), and the six products with the largest weight
//
//     t0 b0 + t0 b1 + t1 b0 + t0 b2 + t1 b1 + t2 b0
//
// are appended to the base product's reduction as 6 r extra columns of K
// (zero-padded to a multiple of 64).  bf16 x bf16 products are exact in the
// f32 accumulator, so the appended term equals the f32 product t . b to a few
// 2^-24 of |t| |b|: the accuracy class of the exact kernels, at the cost of one
// or two more K blocks on a tensor pipe that is idle most of the time at these
// shapes.  (The dropped products t1 b2, t2 b1, t2 b2 are below 2^-24 |t||b|.)
//
// This file holds the operand preparation: SplitRows turns a [M, r] f32 factor
// into its [M, KX] bf16 row operand, SplitWeights turns every adapter matrix of
// a range into its [N, KX] operand in one launch.  Compiled WITH fused
// multiply-add: nothing here reproduces a CPU rounding sequence bit for bit.
#include "kernels.h"

namespace see::k {

namespace {

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

// Which piece each of the six K segments takes from the row factor (0, 0, 1, 0,
// 1, 2: written out in SplitRowsKernel) and from the weight factor.
__constant__ int kWeightPiece[6] = {0, 1, 0, 2, 1, 0};

// One thread per row: r values in, KX bf16 out (6 r of them pieces, the rest zero).
template <int R>
__global__ void SplitRowsKernel(const float* __restrict__ t, uint16_t* __restrict__ out, uint32_t M, uint32_t KX) {
  const uint32_t row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= M) return;
  uint16_t piece[R][3];
#pragma unroll
  for (int j = 0; j < R; j += 4) {
    const float4 v = *reinterpret_cast<const float4*>(t + static_cast<size_t>(row) * R + j);
    Split3(v.x, piece[j]); Split3(v.y, piece[j + 1]); Split3(v.z, piece[j + 2]); Split3(v.w, piece[j + 3]);
  }
  uint16_t* dst = out + static_cast<size_t>(row) * KX;
#pragma unroll
  for (int s = 0; s < 6; ++s) {
#pragma unroll
    for (int j = 0; j < R; j += 4) {
      const int pc = s == 0 || s == 1 || s == 3 ? 0 : (s == 5 ? 2 : 1);   // kRowPiece, as a compile-time expression
      uint2 w;
      w.x = static_cast<uint32_t>(piece[j][pc]) | (static_cast<uint32_t>(piece[j + 1][pc]) << 16);
      w.y = static_cast<uint32_t>(piece[j + 2][pc]) | (static_cast<uint32_t>(piece[j + 3][pc]) << 16);
      *reinterpret_cast<uint2*>(dst + s * R + j) = w;
    }
  }
  for (uint32_t k = 6 * R; k < KX; k += 4) *reinterpret_cast<uint2*>(dst + k) = make_uint2(0u, 0u);
}

// One thread per (entry, output column n): r values of the adapter matrix,
// scaled, cut and laid out as row n of the [N, KX] operand.
__global__ void SplitWeightsKernel(const LoraWeight* __restrict__ table, int count) {
  const LoraWeight e = table[blockIdx.y];
  const uint32_t n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= e.n_out) return;
  // What the base product's epilogue will multiply the whole tile by has to be
  // divided out of the low-rank term first.
  const float tile_scale = e.col_scale ? e.col_scale[n] : e.tile_alpha;
  uint16_t* dst = e.dst + static_cast<size_t>(n) * e.kx;
  for (uint32_t j = 0; j < e.r; ++j) {
    const float w = e.by_column ? e.src[static_cast<size_t>(n) * e.r + j]       // A [n_out, r]
                                : e.src[static_cast<size_t>(j) * e.n_out + n];  // B [r, n_out]
    uint16_t p[3];
    Split3(e.alpha * w / tile_scale, p);
#pragma unroll
    for (int s = 0; s < 6; ++s) dst[s * e.r + j] = p[kWeightPiece[s]];
  }
  for (uint32_t k = 6 * e.r; k < e.kx; ++k) dst[k] = 0;
}

}  // namespace

uint32_t LoraSplitColumns(uint32_t r) { return (6 * r + 63) / 64 * 64; }

bool LoraSplitRows(const float* t, uint16_t* out, size_t M, uint32_t r, cudaStream_t s) {
  if ((reinterpret_cast<uintptr_t>(t) & 15) != 0 || (reinterpret_cast<uintptr_t>(out) & 15) != 0) return false;
  const uint32_t KX = LoraSplitColumns(r);
  const unsigned blocks = static_cast<unsigned>((M + 127) / 128);
  switch (r) {
    case 4: SplitRowsKernel<4><<<blocks, 128, 0, s>>>(t, out, static_cast<uint32_t>(M), KX); return true;
    case 8: SplitRowsKernel<8><<<blocks, 128, 0, s>>>(t, out, static_cast<uint32_t>(M), KX); return true;
    case 12: SplitRowsKernel<12><<<blocks, 128, 0, s>>>(t, out, static_cast<uint32_t>(M), KX); return true;
    case 16: SplitRowsKernel<16><<<blocks, 128, 0, s>>>(t, out, static_cast<uint32_t>(M), KX); return true;
    default: return false;
  }
}

void LoraSplitWeights(const LoraWeight* table, int count, uint32_t max_n_out, cudaStream_t s) {
  if (count <= 0 || max_n_out == 0) return;
  const dim3 grid((max_n_out + 127) / 128, static_cast<unsigned>(count));
  SplitWeightsKernel<<<grid, 128, 0, s>>>(table, count);
}

}  // namespace see::k
