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
// 16x256 for the quad order; 64x32, 128x16, 16x128 for the lane order) picked
// from the output shape, so a skinny product wastes no lanes.  A tile shape
// changes which thread owns an element, never the element's arithmetic.
// Large frozen-weight products carrying the relaxed permission go to the
// tensor cores instead.
#include "gemm_exact_common.cuh"

namespace see::k {

namespace {

using namespace exact;

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
  __shared__ __align__(16) float As[BK][BM + 4];
  __shared__ __align__(16) float Bs[BK][BN + 4];
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
  const bool a_vec = (reinterpret_cast<uintptr_t>(p.A) & 15) == 0 && ((TA ? p.M : p.K) & 3) == 0;
  const size_t k_begin = p.k_chunk ? static_cast<size_t>(blockIdx.z) * p.k_chunk : 0;
  const size_t k_end = p.k_chunk ? (k_begin + p.k_chunk < p.K ? k_begin + p.k_chunk : p.K) : p.K;
  for (size_t k0 = k_begin; k0 < k_end; k0 += BK) {
    // Stage the tiles; alpha and the column scale are applied here, once per
    // element, as the reference applies them when an element enters the product.
    if (a_vec) {  // 16-byte global loads along A's contiguous axis
#pragma unroll
      for (int idx = threadIdx.x; idx < BM * BK / 4; idx += kThreads) {
        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (TA) {
          const int kk = idx / (BM / 4), mm = (idx % (BM / 4)) * 4;
          if (m0 + mm < p.M && k0 + kk < p.K)
            v = *reinterpret_cast<const float4*>(p.A + (k0 + kk) * p.M + m0 + mm);
          *reinterpret_cast<float4*>(&As[kk][mm]) =
              make_float4(p.alpha * v.x, p.alpha * v.y, p.alpha * v.z, p.alpha * v.w);
        } else {
          const int mm = idx / (BK / 4), kk = (idx % (BK / 4)) * 4;
          if (m0 + mm < p.M && k0 + kk < p.K)
            v = *reinterpret_cast<const float4*>(p.A + (m0 + mm) * p.K + k0 + kk);
          As[kk][mm] = p.alpha * v.x; As[kk + 1][mm] = p.alpha * v.y;
          As[kk + 2][mm] = p.alpha * v.z; As[kk + 3][mm] = p.alpha * v.w;
        }
      }
    } else {
#pragma unroll
      for (int idx = threadIdx.x; idx < BM * BK; idx += kThreads) {
        int mm, kk;
        if (TA) { kk = idx / BM; mm = idx % BM; } else { mm = idx / BK; kk = idx % BK; }
        As[kk][mm] = p.alpha * LoadA<TA>(p, m0 + mm, k0 + kk);
      }
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
      for (int q = 0; q < 4; ++q) {  // one 16-byte shared load per operand row
        const float4 av = *reinterpret_cast<const float4*>(&As[kk + q][ty * 4]);
        const float4 bv = *reinterpret_cast<const float4*>(&Bs[kk + q][tx * 4]);
        a[q][0] = av.x; a[q][1] = av.y; a[q][2] = av.z; a[q][3] = av.w;
        b[q][0] = bv.x; b[q][1] = bv.y; b[q][2] = bv.z; b[q][3] = bv.w;
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
  // Whole 16-byte rows of the thread's 4x4 block when the layout allows it.
  const size_t nq = n0 + tx * 4;
  const bool vec = !p.partials && (p.N & 3) == 0 && nq + 3 < p.N &&
                   (reinterpret_cast<uintptr_t>(p.C) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(p.addend) & 15) == 0;
  if (vec) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const size_t m = m0 + ty * 4 + i;
      if (m >= p.M) continue;
      float v[4] = {c[i][0], c[i][1], c[i][2], c[i][3]};
      if (p.addend) {
        const float4 d = *reinterpret_cast<const float4*>(p.addend + m * p.N + nq);
        v[0] = d.x + v[0]; v[1] = d.y + v[1]; v[2] = d.z + v[2]; v[3] = d.w + v[3];
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (p.bias) v[j] = v[j] + p.bias[nq + j];
        v[j] = ApplyAct(v[j], p.act);
      }
      *reinterpret_cast<float4*>(p.C + m * p.N + nq) = make_float4(v[0], v[1], v[2], v[3]);
    }
    return;
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

// Folds split-K partials, then the epilogue.  Fixed two-level order: the chunks
// are cut into eight consecutive groups; warp w of a block sums group w in chunk
// order (for 32 neighbouring outputs, one per lane, so every load is a full
// 128-byte line), and the eight group sums are then added in group order.  The
// grouping is a function of the chunk count alone.
constexpr int kFoldGroups = 8;
__global__ void __launch_bounds__(32 * kFoldGroups) SplitKFoldKernel(Params p, size_t chunks) {
  __shared__ float group_sum[kFoldGroups][32];
  const size_t total = p.M * p.N;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const size_t i = static_cast<size_t>(blockIdx.x) * 32 + lane;
  const size_t per = (chunks + kFoldGroups - 1) / kFoldGroups;
  const size_t z_begin = w * per, z_end = z_begin + per < chunks ? z_begin + per : chunks;
  float v = 0.0f;
  if (i < total) {
    for (size_t z0 = z_begin; z0 < z_end; z0 += 16) {   // sixteen independent loads at a time
      float part[16];
#pragma unroll
      for (int u = 0; u < 16; ++u)
        part[u] = z0 + u < z_end ? p.partials[(z0 + u) * total + i] : 0.0f;
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        if (z0 + u == z_begin) v = part[u];
        else if (z0 + u < z_end) v = v + part[u];
      }
    }
  }
  group_sum[w][lane] = v;
  __syncthreads();
  if (w != 0 || i >= total) return;
  v = group_sum[0][lane];
  for (int gi = 1; gi < kFoldGroups; ++gi)
    if (static_cast<size_t>(gi) * per < chunks) v = v + group_sum[gi][lane];
  if (p.addend) v = p.addend[i] + v;
  if (p.bias) v = v + p.bias[i % p.N];
  p.C[i] = ApplyAct(v, p.act);
}

// ---- lane order: BM x BN tile (BM * BN = 2048), 256 threads, 4x2 outputs x 8 lanes -----
template <typename BT, int BM, int BN>
__global__ void __launch_bounds__(kThreads) GemmLaneKernel(Params p) {
  static_assert(BM * BN == 8 * kThreads, "4x2 outputs per thread");
  __shared__ __align__(16) float As[BK][BM + 4];
  __shared__ __align__(16) float Bs[BK][BN + 4];
  const int tx = threadIdx.x % (BN / 2), ty = threadIdx.x / (BN / 2);
  const size_t m0 = static_cast<size_t>(blockIdx.y) * BM, n0 = static_cast<size_t>(blockIdx.x) * BN;
  float acc[4][2][8];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int l = 0; l < 8; ++l) acc[i][j][l] = 0.0f;
  const bool a_vec = (p.K & 3) == 0 && (reinterpret_cast<uintptr_t>(p.A) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(p.a_k_scale) & 15) == 0;
  for (size_t k0 = 0; k0 < p.K; k0 += BK) {
    if (a_vec) {  // 16-byte global loads along k
#pragma unroll
      for (int idx = threadIdx.x; idx < BM * BK / 4; idx += kThreads) {
        const int mm = idx / (BK / 4), kk = (idx % (BK / 4)) * 4;
        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (m0 + mm < p.M && k0 + kk < p.K) {
          v = *reinterpret_cast<const float4*>(p.A + (m0 + mm) * p.K + k0 + kk);
          if (p.a_k_scale) {
            const float4 sc = *reinterpret_cast<const float4*>(p.a_k_scale + k0 + kk);
            v.x = v.x * sc.x; v.y = v.y * sc.y; v.z = v.z * sc.z; v.w = v.w * sc.w;
          }
        }
        As[kk][mm] = v.x; As[kk + 1][mm] = v.y; As[kk + 2][mm] = v.z; As[kk + 3][mm] = v.w;
      }
    } else {
#pragma unroll
      for (int idx = threadIdx.x; idx < BM * BK; idx += kThreads) {
        const int mm = idx / BK, kk = idx % BK;
        float a = LoadA<false>(p, m0 + mm, k0 + kk);
        if (p.a_k_scale && k0 + kk < p.K) a = a * p.a_k_scale[k0 + kk];
        As[kk][mm] = a;
      }
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
        const float4 av = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
        const float2 bv = *reinterpret_cast<const float2*>(&Bs[kk][tx * 2]);
        const float a[4] = {av.x, av.y, av.z, av.w};
        const float b[2] = {bv.x, bv.y};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 2; ++j) acc[i][j][l] = acc[i][j][l] + a[i] * b[j];
      }
    }
    __syncthreads();
  }
  const size_t np = n0 + tx * 2;
  if ((p.N & 1) == 0 && np + 1 < p.N && (reinterpret_cast<uintptr_t>(p.C) & 7) == 0 &&
      (reinterpret_cast<uintptr_t>(p.addend) & 7) == 0) {  // 8-byte pairs
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const size_t m = m0 + ty * 4 + i;
      if (m >= p.M) continue;
      float v[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        float s = acc[i][j][0];
#pragma unroll
        for (int l = 1; l < 8; ++l) s = s + acc[i][j][l];
        v[j] = p.alpha * s;
      }
      if (p.addend) {
        const float2 d = *reinterpret_cast<const float2*>(p.addend + m * p.N + np);
        v[0] = d.x + v[0]; v[1] = d.y + v[1];
      }
      *reinterpret_cast<float2*>(p.C + m * p.N + np) = make_float2(v[0], v[1]);
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const size_t m = m0 + ty * 4 + i, n = n0 + tx * 2 + j;
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
    GemmLaneKernel<BT, 128, 16><<<dim3(Blocks(p.N, 16), Blocks(p.M, 128)), kThreads, 0, s>>>(p);
  } else if (p.M <= 16) {
    GemmLaneKernel<BT, 16, 128><<<dim3(Blocks(p.N, 128), Blocks(p.M, 16)), kThreads, 0, s>>>(p);
  } else {
    GemmLaneKernel<BT, 64, 32><<<dim3(Blocks(p.N, 32), Blocks(p.M, 64)), kThreads, 0, s>>>(p);
  }
}

size_t QuadTiles(size_t M, size_t N) {
  if (N <= 16) return static_cast<size_t>(Blocks(M, 256)) * Blocks(N, 16);
  if (M <= 16) return static_cast<size_t>(Blocks(N, 256)) * Blocks(M, 16);
  return static_cast<size_t>(Blocks(M, 64)) * Blocks(N, 64);
}

}  // namespace

size_t SplitKChunkRows(size_t M, size_t N, size_t K) {
  const size_t tiles = QuadTiles(M, N);
  size_t rows = kSplitKChunk;
  while (rows > 32 && ((K + rows - 1) / rows) * tiles < 296) rows /= 2;
  return rows;
}

size_t SplitKChunks(size_t M, size_t N, size_t K) {
  if (K < 4 * kSplitKChunk || QuadTiles(M, N) >= 148) return 1;
  const size_t rows = SplitKChunkRows(M, N, K);
  return (K + rows - 1) / rows;
}

bool GemmExact(const GemmArgs& a, cudaStream_t s) {
  if (a.M == 0 || a.N == 0) return false;
  Params p{a.A, a.B, a.C, a.M, a.N, a.K, a.alpha, a.b_col_scale, a.a_k_scale,
           a.bias, a.addend, a.act, a.accumulate, 0, nullptr};
  // Only the expand kernel takes the tail add; every other path sees none.
  Params pt = p;
  if (a.tail_addend && a.tail_out && Aligned16(a.tail_addend) && Aligned16(a.tail_out)) {
    pt.tail_addend = a.tail_addend;
    pt.tail_out = a.tail_out;
  }
  const auto reduce = a.contract_fma ? fast::SkinnyReduce : exact::SkinnyReduce;
  const auto expand = a.contract_fma ? fast::SkinnyExpand : exact::SkinnyExpand;
  const auto tn_partials = a.contract_fma ? fast::SkinnyTnPartials : exact::SkinnyTnPartials;
  if (a.b_transposed) {
    if (a.b_type == BType::kF32) {
      if (reduce(p, true, s)) return false;
      if (expand(pt, true, s)) return pt.tail_out != nullptr;
    }
    switch (a.b_type) {
      case BType::kF32: LaunchLane<float>(p, s); break;
      case BType::kI8: LaunchLane<int8_t>(p, s); break;
      case BType::kBf16: LaunchLane<uint16_t>(p, s); break;
    }
    return false;
  }
  if (a.a_transposed) {
    // Adapter gradients: a [rank x width] or [width x rank] result reduced over
    // every row of the batch.  With few output tiles and a long K the chunks go
    // to separate blocks (fixed geometry: a pure function of the shape).
    const size_t chunks = SplitKChunks(a.M, a.N, a.K);
    if (chunks > 1 && a.split_scratch && !a.accumulate &&
        chunks * a.M * a.N <= a.split_scratch_floats) {
      p.k_chunk = SplitKChunkRows(a.M, a.N, a.K);
      p.partials = a.split_scratch;
      if (!tn_partials(p, chunks, s)) LaunchQuad<true, float>(p, static_cast<unsigned>(chunks), s);
      const size_t blocks = (a.M * a.N + 31) / 32;
      SplitKFoldKernel<<<static_cast<unsigned>(blocks), 32 * kFoldGroups, 0, s>>>(p, chunks);
      return false;
    }
    LaunchQuad<true, float>(p, 1, s);
    return false;
  }
  if (a.b_type == BType::kF32) {
    if (reduce(p, false, s)) return false;
    if (expand(pt, false, s)) return pt.tail_out != nullptr;
  }
  switch (a.b_type) {
    case BType::kF32: LaunchQuad<false, float>(p, 1, s); break;
    case BType::kI8: LaunchQuad<false, int8_t>(p, 1, s); break;
    case BType::kBf16: LaunchQuad<false, uint16_t>(p, 1, s); break;
  }
  return false;
}

}  // namespace see::k
