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
// (zero-padded to a multiple of 64), smallest products first: the tensor core
// adds each 16-term group into its f32 accumulator with truncation, an error of
// up to one unit in the last place of the ACCUMULATOR per group and always
// toward zero, so the many small terms go in while the accumulator is still
// small and only the K/16 groups of t0 b0 meet it at full size (measured at
// K = 8192: 4.7e-6 of sum|a b| with the large products first, against 2e-6 asked).  bf16 x bf16 products are exact in the
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
#include "lora_split.cuh"

namespace see::k {

namespace {

// One thread per (row, four columns of t): 4 values in, their pieces out to the six
// segments; the threads of a row also zero its padding columns [6 R, KX).
template <int R>
__global__ void SplitRowsKernel(const float* __restrict__ t, uint16_t* __restrict__ out, uint32_t M, uint32_t KX) {
  constexpr uint32_t kQuads = R / 4;
  const uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;
  const uint32_t row = idx / kQuads, j = (idx - row * kQuads) * 4;
  if (row >= M) return;
  const float4 v = *reinterpret_cast<const float4*>(t + static_cast<size_t>(row) * R + j);
  uint16_t piece[4][3];
  Split3(v.x, piece[0]); Split3(v.y, piece[1]); Split3(v.z, piece[2]); Split3(v.w, piece[3]);
  uint16_t* dst = out + static_cast<size_t>(row) * KX;
#pragma unroll
  for (int s = 0; s < 6; ++s) {
    const int pc = PieceOf(0, s);
    uint2 w;
    w.x = static_cast<uint32_t>(piece[0][pc]) | (static_cast<uint32_t>(piece[1][pc]) << 16);
    w.y = static_cast<uint32_t>(piece[2][pc]) | (static_cast<uint32_t>(piece[3][pc]) << 16);
    *reinterpret_cast<uint2*>(dst + s * R + j) = w;
  }
  for (uint32_t k = 6 * R + j; k < KX; k += R) *reinterpret_cast<uint2*>(dst + k) = make_uint2(0u, 0u);
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
    for (int s = 0; s < 6; ++s) dst[s * e.r + j] = p[PieceOf(1, s)];
  }
  for (uint32_t k = 6 * e.r; k < e.kx; ++k) dst[k] = 0;
}

// ---- whole matrices: an f32 GEMM on the bf16 tensor cores -------------------------------
// dst [rows][6 * cols] bf16: six K segments of `cols` each, segment s holding
// piece PieceOf(0, s) (the A side of a product) or PieceOf(1, s) (the B side) of
// every element, so that A' B'^T over the long K axis is the six-product sum of
// the header comment (in its order: small products first).  src is [rows][cols], or [cols][rows] when transposed
// (then a 32 x 32 tile goes through shared memory so both sides stay coalesced).
template <int kSide>
__global__ void SplitMatrixKernel(const float* __restrict__ src, uint16_t* __restrict__ dst, uint32_t rows,
                                  uint32_t cols) {
  const size_t quads = static_cast<size_t>(rows) * (cols / 4);
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t q = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; q < quads; q += stride) {
    const uint32_t row = static_cast<uint32_t>(q / (cols / 4)), c4 = static_cast<uint32_t>(q % (cols / 4)) * 4;
    const float4 v = *reinterpret_cast<const float4*>(src + static_cast<size_t>(row) * cols + c4);
    uint16_t p[4][3];
    Split3(v.x, p[0]); Split3(v.y, p[1]); Split3(v.z, p[2]); Split3(v.w, p[3]);
    uint16_t* out = dst + static_cast<size_t>(row) * 6 * cols + c4;
#pragma unroll
    for (int s = 0; s < 6; ++s) {
      const int pc = PieceOf(kSide, s);
      uint2 w;
      w.x = static_cast<uint32_t>(p[0][pc]) | (static_cast<uint32_t>(p[1][pc]) << 16);
      w.y = static_cast<uint32_t>(p[2][pc]) | (static_cast<uint32_t>(p[3][pc]) << 16);
      *reinterpret_cast<uint2*>(out + static_cast<size_t>(s) * cols) = w;
    }
  }
}

// src [cols][rows] -> dst row r, column c = src[c][r].
template <int kSide>
__global__ void SplitMatrixTransposedKernel(const float* __restrict__ src, uint16_t* __restrict__ dst,
                                            uint32_t rows, uint32_t cols) {
  __shared__ float tile[32][33];
  const uint32_t r0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
  for (uint32_t i = threadIdx.y; i < 32; i += blockDim.y) {
    const uint32_t c = c0 + i, r = r0 + threadIdx.x;
    tile[i][threadIdx.x] = c < cols && r < rows ? src[static_cast<size_t>(c) * rows + r] : 0.0f;
  }
  __syncthreads();
  for (uint32_t i = threadIdx.y; i < 32; i += blockDim.y) {
    const uint32_t r = r0 + i, c = c0 + threadIdx.x;
    if (r >= rows || c >= cols) continue;
    uint16_t p[3];
    Split3(tile[threadIdx.x][i], p);
    uint16_t* out = dst + static_cast<size_t>(r) * 6 * cols + c;
#pragma unroll
    for (int s = 0; s < 6; ++s) out[static_cast<size_t>(s) * cols] = p[PieceOf(kSide, s)];
  }
}

}  // namespace

void SplitMatrix(const float* src, uint16_t* dst, size_t rows, size_t cols, bool transposed, int side,
                 cudaStream_t s) {
  if (rows == 0 || cols == 0) return;
  if (transposed) {
    const dim3 grid(static_cast<unsigned>((rows + 31) / 32), static_cast<unsigned>((cols + 31) / 32));
    const dim3 block(32, 8);
    if (side == 0)
      SplitMatrixTransposedKernel<0><<<grid, block, 0, s>>>(src, dst, static_cast<uint32_t>(rows),
                                                            static_cast<uint32_t>(cols));
    else
      SplitMatrixTransposedKernel<1><<<grid, block, 0, s>>>(src, dst, static_cast<uint32_t>(rows),
                                                            static_cast<uint32_t>(cols));
    return;
  }
  size_t blocks = (rows * (cols / 4) + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (side == 0)
    SplitMatrixKernel<0><<<static_cast<unsigned>(blocks), 256, 0, s>>>(src, dst, static_cast<uint32_t>(rows),
                                                                       static_cast<uint32_t>(cols));
  else
    SplitMatrixKernel<1><<<static_cast<unsigned>(blocks), 256, 0, s>>>(src, dst, static_cast<uint32_t>(rows),
                                                                       static_cast<uint32_t>(cols));
}

uint32_t LoraSplitColumns(uint32_t r) { return (6 * r + 63) / 64 * 64; }

bool LoraSplitRows(const float* t, uint16_t* out, size_t M, uint32_t r, cudaStream_t s) {
  if ((reinterpret_cast<uintptr_t>(t) & 15) != 0 || (reinterpret_cast<uintptr_t>(out) & 15) != 0) return false;
  const uint32_t KX = LoraSplitColumns(r);
  const unsigned blocks = static_cast<unsigned>((M * (r / 4) + 255) / 256);
  switch (r) {
    case 4: SplitRowsKernel<4><<<blocks, 256, 0, s>>>(t, out, static_cast<uint32_t>(M), KX); return true;
    case 8: SplitRowsKernel<8><<<blocks, 256, 0, s>>>(t, out, static_cast<uint32_t>(M), KX); return true;
    case 12: SplitRowsKernel<12><<<blocks, 256, 0, s>>>(t, out, static_cast<uint32_t>(M), KX); return true;
    case 16: SplitRowsKernel<16><<<blocks, 256, 0, s>>>(t, out, static_cast<uint32_t>(M), KX); return true;
    default: return false;
  }
}

void LoraSplitWeights(const LoraWeight* table, int count, uint32_t max_n_out, cudaStream_t s) {
  if (count <= 0 || max_n_out == 0) return;
  const dim3 grid((max_n_out + 127) / 128, static_cast<unsigned>(count));
  SplitWeightsKernel<<<grid, 128, 0, s>>>(table, count);
}

}  // namespace see::k
