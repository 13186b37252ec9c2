// The exact GEMM family on CUDA cores: reproduces the CPU executor's two
// reduction contracts bit for bit, for f32, int8 and bf16 weights.
//
//   quad order (NN, TN, AccNN and their narrow-weight forms; reference:
//     runtime/executor/gemm.cc:73-187): per element, from c = 0 (or the
//     existing C for the accumulate form),
//         c += ((a0*b0 + a1*b1) + a2*b2) + a3*b3
//     over consecutive k-quads aligned to k = 0, then one term at a time for
//     the K % 4 tail; alpha (or the per-tensor dequant scale) is multiplied
//     into each A element first, a per-column scale into each widened B element.
//   lane order (NT forms; reference: runtime/executor/gemm.cc:346-527): eight
//     accumulators, product k into lane k mod 8, lanes summed 0..7, the result
//     times alpha; a reduction-axis scale is multiplied into A first.
//
// Epilogue order matches the reference (gemm.cc:536-578): addend `d + s` on
// the finished sum, then bias, then the activation expression.  Compiled with
// -fmad=false; no multiply is ever fused into an add.  This family is the
// parity anchor and the path for the rank-r adapter products, whose outputs are
// 8-16 wide (or tall): the block tile comes in three shapes (64x64, 256x16,
// 16x256 for the quad order; 32x32, 64x16, 16x64 for the lane order) picked
// from the output shape, so a skinny product wastes no lanes.  A tile shape
// changes which thread owns an element, never the element's arithmetic.
// Large frozen-weight products carrying the relaxed permission go to the
// tensor cores instead.
#include "kernels.h"

namespace see::k {

namespace {

constexpr float kGeluC = 0.7978845608028654f;
constexpr float kGeluA = 0.044715f;

__device__ __forceinline__ float ApplyAct(float v, Act act) {
  switch (act) {
    case kActRelu: return v > 0.0f ? v : 0.0f;
    case kActGelu: {
      const float t = tanhf(kGeluC * (v + kGeluA * v * v * v));
      return 0.5f * v * (1.0f + t);
    }
    case kActSilu: return v * (1.0f / (1.0f + expf(-v)));
    default: return v;
  }
}

template <typename T> __device__ __forceinline__ float Widen(T v);
template <> __device__ __forceinline__ float Widen<float>(float v) { return v; }
template <> __device__ __forceinline__ float Widen<int8_t>(int8_t v) { return static_cast<float>(v); }
template <> __device__ __forceinline__ float Widen<uint16_t>(uint16_t v) {
  return __uint_as_float(static_cast<uint32_t>(v) << 16);
}

struct Params {
  const float* A;
  const void* B;
  float* C;
  size_t M, N, K;
  float alpha;
  const float* b_col_scale;
  const float* a_k_scale;
  const float* bias;
  const float* addend;
  Act act;
  bool accumulate;
  // Split-K (long reductions into small outputs): block z reduces k in
  // [z * k_chunk, (z + 1) * k_chunk) with the quad order inside the chunk and
  // writes its raw sums to partials[z][M][N]; a second kernel folds the chunks
  // in chunk order.  k_chunk is a multiple of 16, so quads stay aligned to k = 0.
  size_t k_chunk;
  float* partials;
};

constexpr int BK = 16;
constexpr int kThreads = 256;

template <bool TA>
__device__ __forceinline__ float LoadA(const Params& p, size_t m, size_t k) {
  if (m >= p.M || k >= p.K) return 0.0f;
  return TA ? p.A[k * p.M + m] : p.A[m * p.K + k];
}
template <bool TB, typename BT>
__device__ __forceinline__ float LoadB(const Params& p, size_t k, size_t n) {
  if (n >= p.N || k >= p.K) return 0.0f;
  const BT* B = static_cast<const BT*>(p.B);
  return Widen<BT>(TB ? B[n * p.K + k] : B[k * p.N + n]);
}

// ---- quad order: BM x BN tile (BM * BN = 4096), 256 threads, 4x4 outputs per thread ----
template <bool TA, typename BT, int BM, int BN>
__global__ void __launch_bounds__(kThreads) GemmQuadKernel(Params p) {
  static_assert(BM * BN == 16 * kThreads, "4x4 outputs per thread");
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  const int tx = threadIdx.x % (BN / 4), ty = threadIdx.x / (BN / 4);
  const size_t m0 = static_cast<size_t>(blockIdx.y) * BM, n0 = static_cast<size_t>(blockIdx.x) * BN;
  float c[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const size_t m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
      c[i][j] = (p.accumulate && m < p.M && n < p.N) ? p.C[m * p.N + n] : 0.0f;
    }
  const size_t k_begin = p.k_chunk ? static_cast<size_t>(blockIdx.z) * p.k_chunk : 0;
  const size_t k_end = p.k_chunk ? (k_begin + p.k_chunk < p.K ? k_begin + p.k_chunk : p.K) : p.K;
  for (size_t k0 = k_begin; k0 < k_end; k0 += BK) {
    // Stage the tiles; alpha and the column scale are applied here, once per
    // element, as the reference applies them when an element enters the product.
#pragma unroll
    for (int idx = threadIdx.x; idx < BM * BK; idx += kThreads) {
      int mm, kk;
      if (TA) { kk = idx / BM; mm = idx % BM; } else { mm = idx / BK; kk = idx % BK; }
      As[kk][mm] = p.alpha * LoadA<TA>(p, m0 + mm, k0 + kk);
    }
#pragma unroll
    for (int idx = threadIdx.x; idx < BK * BN; idx += kThreads) {
      const int kb = idx / BN, nb = idx % BN;
      float b = LoadB<false, BT>(p, k0 + kb, n0 + nb);
      if (p.b_col_scale && n0 + nb < p.N) b = b * p.b_col_scale[n0 + nb];
      Bs[kb][nb] = b;
    }
    __syncthreads();
    const int kmax = k_end - k0 < static_cast<size_t>(BK) ? static_cast<int>(k_end - k0) : BK;
    int kk = 0;
    for (; kk + 4 <= kmax; kk += 4) {
      float a[4][4], b[4][4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
#pragma unroll
        for (int i = 0; i < 4; ++i) a[q][i] = As[kk + q][ty * 4 + i];
#pragma unroll
        for (int j = 0; j < 4; ++j) b[q][j] = Bs[kk + q][tx * 4 + j];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float t = a[0][i] * b[0][j];
          t = t + a[1][i] * b[1][j];
          t = t + a[2][i] * b[2][j];
          t = t + a[3][i] * b[3][j];
          c[i][j] = c[i][j] + t;
        }
    }
    for (; kk < kmax; ++kk) {  // the K % 4 tail, one term at a time
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
          c[i][j] = c[i][j] + As[kk][ty * 4 + i] * Bs[kk][tx * 4 + j];
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const size_t m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
      if (m >= p.M || n >= p.N) continue;
      float v = c[i][j];
      if (p.partials) {
        p.partials[(static_cast<size_t>(blockIdx.z) * p.M + m) * p.N + n] = v;
        continue;
      }
      if (p.addend) v = p.addend[m * p.N + n] + v;
      if (p.bias) v = v + p.bias[n];
      p.C[m * p.N + n] = ApplyAct(v, p.act);
    }
}

// Folds split-K partials in chunk order, then the epilogue.
__global__ void SplitKFoldKernel(Params p, size_t chunks) {
  const size_t total = p.M * p.N;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total; i += stride) {
    float v = p.partials[i];
    for (size_t z = 1; z < chunks; ++z) v = v + p.partials[z * total + i];
    if (p.addend) v = p.addend[i] + v;
    if (p.bias) v = v + p.bias[i % p.N];
    p.C[i] = ApplyAct(v, p.act);
  }
}

// ---- lane order: BM x BN tile (BM * BN = 1024), 256 threads, 2x2 outputs x 8 lanes ------
template <typename BT, int BM, int BN>
__global__ void __launch_bounds__(kThreads) GemmLaneKernel(Params p) {
  static_assert(BM * BN == 4 * kThreads, "2x2 outputs per thread");
  __shared__ float As[BK][BM + 2];
  __shared__ float Bs[BK][BN + 2];
  const int tx = threadIdx.x % (BN / 2), ty = threadIdx.x / (BN / 2);
  const size_t m0 = static_cast<size_t>(blockIdx.y) * BM, n0 = static_cast<size_t>(blockIdx.x) * BN;
  float acc[2][2][8];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int l = 0; l < 8; ++l) acc[i][j][l] = 0.0f;
  for (size_t k0 = 0; k0 < p.K; k0 += BK) {
#pragma unroll
    for (int idx = threadIdx.x; idx < BM * BK; idx += kThreads) {
      const int mm = idx / BK, kk = idx % BK;
      float a = LoadA<false>(p, m0 + mm, k0 + kk);
      if (p.a_k_scale && k0 + kk < p.K) a = a * p.a_k_scale[k0 + kk];
      As[kk][mm] = a;
    }
#pragma unroll
    for (int idx = threadIdx.x; idx < BN * BK; idx += kThreads) {
      const int nn = idx / BK, kk = idx % BK;
      Bs[kk][nn] = LoadB<true, BT>(p, k0 + kk, n0 + nn);
    }
    __syncthreads();
    const int kmax = p.K - k0 < static_cast<size_t>(BK) ? static_cast<int>(p.K - k0) : BK;
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      if (kk < kmax) {
        const int l = kk & 7;  // k0 is a multiple of 16, so k mod 8 == kk mod 8
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
          for (int j = 0; j < 2; ++j)
            acc[i][j][l] = acc[i][j][l] + As[kk][ty * 2 + i] * Bs[kk][tx * 2 + j];
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const size_t m = m0 + ty * 2 + i, n = n0 + tx * 2 + j;
      if (m >= p.M || n >= p.N) continue;
      float s = acc[i][j][0];
#pragma unroll
      for (int l = 1; l < 8; ++l) s = s + acc[i][j][l];
      float v = p.alpha * s;
      if (p.addend) v = p.addend[m * p.N + n] + v;
      p.C[m * p.N + n] = v;
    }
}

unsigned Blocks(size_t extent, size_t tile) { return static_cast<unsigned>((extent + tile - 1) / tile); }

template <bool TA, typename BT>
void LaunchQuad(const Params& p, unsigned z, cudaStream_t s) {
  if (p.N <= 16) {
    GemmQuadKernel<TA, BT, 256, 16><<<dim3(Blocks(p.N, 16), Blocks(p.M, 256), z), kThreads, 0, s>>>(p);
  } else if (p.M <= 16) {
    GemmQuadKernel<TA, BT, 16, 256><<<dim3(Blocks(p.N, 256), Blocks(p.M, 16), z), kThreads, 0, s>>>(p);
  } else {
    GemmQuadKernel<TA, BT, 64, 64><<<dim3(Blocks(p.N, 64), Blocks(p.M, 64), z), kThreads, 0, s>>>(p);
  }
}

template <typename BT>
void LaunchLane(const Params& p, cudaStream_t s) {
  if (p.N <= 16) {
    GemmLaneKernel<BT, 64, 16><<<dim3(Blocks(p.N, 16), Blocks(p.M, 64)), kThreads, 0, s>>>(p);
  } else if (p.M <= 16) {
    GemmLaneKernel<BT, 16, 64><<<dim3(Blocks(p.N, 64), Blocks(p.M, 16)), kThreads, 0, s>>>(p);
  } else {
    GemmLaneKernel<BT, 32, 32><<<dim3(Blocks(p.N, 32), Blocks(p.M, 32)), kThreads, 0, s>>>(p);
  }
}

size_t QuadTiles(size_t M, size_t N) {
  if (N <= 16) return static_cast<size_t>(Blocks(M, 256)) * Blocks(N, 16);
  if (M <= 16) return static_cast<size_t>(Blocks(N, 256)) * Blocks(M, 16);
  return static_cast<size_t>(Blocks(M, 64)) * Blocks(N, 64);
}

}  // namespace

size_t SplitKChunks(size_t M, size_t N, size_t K) {
  if (K < 4 * kSplitKChunk || QuadTiles(M, N) >= 148) return 1;
  return (K + kSplitKChunk - 1) / kSplitKChunk;
}

void GemmExact(const GemmArgs& a, cudaStream_t s) {
  if (a.M == 0 || a.N == 0) return;
  Params p{a.A, a.B, a.C, a.M, a.N, a.K, a.alpha, a.b_col_scale, a.a_k_scale,
           a.bias, a.addend, a.act, a.accumulate, 0, nullptr};
  if (a.b_transposed) {
    switch (a.b_type) {
      case BType::kF32: LaunchLane<float>(p, s); break;
      case BType::kI8: LaunchLane<int8_t>(p, s); break;
      case BType::kBf16: LaunchLane<uint16_t>(p, s); break;
    }
    return;
  }
  if (a.a_transposed) {
    // Adapter gradients: a [rank x width] or [width x rank] result reduced over
    // every row of the batch.  With few output tiles and a long K the chunks go
    // to separate blocks (fixed geometry: a pure function of the shape).
    const size_t chunks = SplitKChunks(a.M, a.N, a.K);
    if (chunks > 1 && a.split_scratch && !a.accumulate &&
        chunks * a.M * a.N <= a.split_scratch_floats) {
      p.k_chunk = kSplitKChunk;
      p.partials = a.split_scratch;
      LaunchQuad<true, float>(p, static_cast<unsigned>(chunks), s);
      size_t blocks = (a.M * a.N + 255) / 256;
      if (blocks > 1184) blocks = 1184;
      SplitKFoldKernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(p, chunks);
      return;
    }
    LaunchQuad<true, float>(p, 1, s);
    return;
  }
  switch (a.b_type) {
    case BType::kF32: LaunchQuad<false, float>(p, 1, s); break;
    case BType::kI8: LaunchQuad<false, int8_t>(p, 1, s); break;
    case BType::kBf16: LaunchQuad<false, uint16_t>(p, 1, s); break;
  }
}

}  // namespace see::k
