// The adapter-side products of a LoRA site that stream a whole activation,
// engine mode:
//
//   forward   t  = x A                    [M, r]   from x [M, K]
//   backward  dT = a1 dY B^T              [M, r]   from dY [M, N]
//             dB = a2 t^T dY              [r, N]
//             dA = a3 x^T dT              [K, r]
//
// The plan spells the backward as three instructions that each stream a
// [M, width] activation through HBM for a rank-r result.  Here ONE kernel reads
// dY and x once each and produces all three: a persistent block takes 16-row
// tiles, forms dT for the tile (the eight warps split the reduction over N and
// fold their partial tiles in warp order), then accumulates the tile's
// contribution to dB and dA in registers; per-block partial sums are folded by
// a second kernel in block order.  The reduction order is a pure function of
// the shape and the grid (one block per SM), so results are identical run to run.
//
// Arithmetic: the products run on the tensor cores as 3xTF32 — each f32 operand
// is cut into its TF32 rounding and the exact remainder, and the three products
// lo*hi, hi*lo, hi*hi are accumulated in f32 (mma.sync.m16n8k8; the legacy tensor
// path is ample for a rank-16 product that is bound by HBM).  The result is the
// f32 product to about 2^-21 of sum|a_k b_k| — inside the bound the reference
// holds its own GEMMs to (2e-6 of 1 + sum|a_k b_k|; reference:
// test/runtime/executor/kernels_test.cc:1803-1822), not the CPU's bits: the
// strict seam keeps the bit-exact kernels.
#include <atomic>

#include "kernels.h"

namespace see::k {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = 8;
constexpr int kTileRows = 16;

__device__ __forceinline__ void CpAsync16(float* smem_dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<unsigned>(
                   __cvta_generic_to_shared(smem_dst))), "l"(src) : "memory");
}
__device__ __forceinline__ void CpAsyncCommit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void CpAsyncWait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory");
}

// x = hi + lo with hi = x cut to TF32 (its low 13 mantissa bits cleared) and lo the
// exact remainder, below 2^-10 |x| (the tensor core reads lo's leading 11 bits, so
// what is lost is below 2^-21 |x|).  A mask and a subtraction: the rounding
// conversion instruction runs on the 16-lane special-function pipe and was 30 % of
// this kernel's issue slots.
__device__ __forceinline__ void SplitTf32(float x, uint32_t* hi, uint32_t* lo) {
  const uint32_t h = __float_as_uint(x) & 0xFFFFE000u;
  *hi = h;
  *lo = __float_as_uint(x - __uint_as_float(h));
}

__device__ __forceinline__ void Mma1688(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// c += a b with both operands given as (hi, lo): the two cross terms first, the
// large product last.
__device__ __forceinline__ void Mma3(float (&c)[4], const uint32_t (&ah)[4], const uint32_t (&al)[4],
                                     const uint32_t (&bh)[2], const uint32_t (&bl)[2]) {
  Mma1688(c, al, bh);
  Mma1688(c, ah, bl);
  Mma1688(c, ah, bh);
}

// Copies rows [row0, row0 + 16) of src [M, W] into tile[16][stride]; rows past M are zeroed.
template <int W>
__device__ __forceinline__ void LoadTile(float* tile, int stride, const float* __restrict__ src, size_t row0,
                                         size_t M) {
  constexpr int kChunks = W / 4;   // 16-byte chunks per row
  for (int idx = threadIdx.x; idx < kTileRows * kChunks; idx += kThreads) {
    const int r = idx / kChunks, c = idx - r * kChunks;
    float* dst = tile + r * stride + 4 * c;
    if (row0 + r < M) CpAsync16(dst, src + (row0 + r) * W + 4 * c);
    else *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

// out[16][R] (+ alpha) = tile[16][W] . w^T, where the weight is read through
// `wf(n, k)`; the warps split k, partial tiles go through `red` and are folded in
// warp order by the first 16 * R threads.  Returns with the block synchronised
// and `out_s[16][out_stride]` holding the result.
template <int W, int R, typename WeightAt>
__device__ __forceinline__ void RowsTimesWeight(const float* tile, int stride, WeightAt wf, float* red,
                                                float* out_s, int out_stride, float alpha) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  constexpr int kPerWarp = W / kWarps;   // a multiple of 8
  float c[R / 8][4];
#pragma unroll
  for (int j = 0; j < R / 8; ++j) c[j][0] = c[j][1] = c[j][2] = c[j][3] = 0.0f;
#pragma unroll 2
  for (int k0 = warp * kPerWarp; k0 < (warp + 1) * kPerWarp; k0 += 8) {
    uint32_t ah[4], al[4];
    SplitTf32(tile[g * stride + k0 + t], &ah[0], &al[0]);
    SplitTf32(tile[(g + 8) * stride + k0 + t], &ah[1], &al[1]);
    SplitTf32(tile[g * stride + k0 + t + 4], &ah[2], &al[2]);
    SplitTf32(tile[(g + 8) * stride + k0 + t + 4], &ah[3], &al[3]);
#pragma unroll
    for (int j = 0; j < R / 8; ++j) {
      uint32_t bh[2], bl[2];
      SplitTf32(wf(8 * j + g, k0 + t), &bh[0], &bl[0]);
      SplitTf32(wf(8 * j + g, k0 + t + 4), &bh[1], &bl[1]);
      Mma3(c[j], ah, al, bh, bl);
    }
  }
  float* mine = red + warp * (kTileRows * R);
#pragma unroll
  for (int j = 0; j < R / 8; ++j) {
    mine[g * R + 8 * j + 2 * t] = c[j][0];
    mine[g * R + 8 * j + 2 * t + 1] = c[j][1];
    mine[(g + 8) * R + 8 * j + 2 * t] = c[j][2];
    mine[(g + 8) * R + 8 * j + 2 * t + 1] = c[j][3];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < kTileRows * R; idx += kThreads) {
    float s = red[idx];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) s += red[w * (kTileRows * R) + idx];
    out_s[(idx / R) * out_stride + (idx % R)] = alpha * s;
  }
  __syncthreads();
}

// ---- forward: t = alpha x A ---------------------------------------------------------------
// Three row tiles of x in flight per block (the kernel is a stream of 48 KB tiles
// with a few hundred tensor instructions each: one tile of lookahead left the SM
// waiting on HBM latency most of the time).
constexpr int kDownStages = 3;

template <int K, int R>
struct DownSmem {
  static constexpr int kXStride = K + 8;
  static constexpr int kAStride = K + 4;     // A^T [R][K]: rows n, so a fragment's eight n land in eight bank groups
  static constexpr int kOutStride = R + 8;
  static constexpr size_t kFloats = kDownStages * kTileRows * kXStride + static_cast<size_t>(R) * kAStride +
                                    kWarps * kTileRows * R + kTileRows * kOutStride;
};

template <int K, int R>
__global__ void __launch_bounds__(kThreads, 1)
LoraDownKernel(const float* __restrict__ x, const float* __restrict__ A, float* __restrict__ out, size_t M,
               float alpha) {
  using S = DownSmem<K, R>;
  extern __shared__ __align__(16) float smem[];
  float* x_s = smem;
  float* a_s = x_s + kDownStages * kTileRows * S::kXStride;
  float* red = a_s + static_cast<size_t>(R) * S::kAStride;
  float* out_s = red + kWarps * kTileRows * R;
  for (int idx = threadIdx.x; idx < K * R; idx += kThreads) {   // A [K][R] -> a_s[n][k]
    const int k = idx / R, n = idx - k * R;
    a_s[n * S::kAStride + k] = A[idx];
  }
  const size_t tiles = (M + kTileRows - 1) / kTileRows;
  // Stage s holds tile blockIdx.x + (i) * gridDim.x for i = s (mod kDownStages); one commit group per tile.
#pragma unroll
  for (int i = 0; i < kDownStages - 1; ++i) {
    const size_t tl = blockIdx.x + static_cast<size_t>(i) * gridDim.x;
    if (tl < tiles) LoadTile<K>(x_s + i * kTileRows * S::kXStride, S::kXStride, x, tl * kTileRows, M);
    CpAsyncCommit();
  }
  int stage = 0;
  for (size_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    // The tile two ahead goes into the stage the previous iteration finished with.
    const size_t ahead = tile + static_cast<size_t>(kDownStages - 1) * gridDim.x;
    const int ahead_stage = (stage + kDownStages - 1) % kDownStages;
    if (ahead < tiles) LoadTile<K>(x_s + ahead_stage * kTileRows * S::kXStride, S::kXStride, x, ahead * kTileRows, M);
    CpAsyncCommit();
    CpAsyncWait<kDownStages - 1>();   // this tile has landed
    __syncthreads();
    const float* xs = x_s + stage * kTileRows * S::kXStride;
    RowsTimesWeight<K, R>(xs, S::kXStride, [&](int n, int k) { return a_s[n * S::kAStride + k]; }, red, out_s,
                          S::kOutStride, alpha);
    const size_t row0 = tile * kTileRows;
    for (int idx = threadIdx.x; idx < kTileRows * R / 4; idx += kThreads) {
      const int r = idx / (R / 4), c = idx - r * (R / 4);
      if (row0 + r < M)
        *reinterpret_cast<float4*>(out + (row0 + r) * R + 4 * c) =
            *reinterpret_cast<const float4*>(out_s + r * S::kOutStride + 4 * c);
    }
    __syncthreads();   // out_s and this stage are rewritten next
    stage = (stage + 1) % kDownStages;
  }
  CpAsyncWait<0>();
}

// ---- backward: dT, and per-block partial sums of dB and dA ------------------------------------
template <int N, int K, int R>
struct BackSmem {
  static constexpr int kDyStride = N + 8, kXStride = K + 8;
  static constexpr int kBStride = N + 4;     // B is [R][N]: rows n, so a fragment's eight n land in eight bank groups
  static constexpr int kSmallStride = R + 8;
  static constexpr size_t kFloats = kTileRows * kDyStride + kTileRows * kXStride + static_cast<size_t>(R) * kBStride +
                                    kWarps * kTileRows * R + 2 * kTileRows * kSmallStride;
};

template <int N, int K, int R>
__global__ void __launch_bounds__(kThreads, 1)
LoraBackwardKernel(const float* __restrict__ dy, const float* __restrict__ x, const float* __restrict__ t,
                   const float* __restrict__ B, float* __restrict__ dt, float* __restrict__ partials, size_t M,
                   float alpha_dt) {
  using S = BackSmem<N, K, R>;
  extern __shared__ __align__(16) float smem[];
  float* dy_s = smem;
  float* x_s = dy_s + kTileRows * S::kDyStride;
  float* b_s = x_s + kTileRows * S::kXStride;
  float* red = b_s + static_cast<size_t>(R) * S::kBStride;
  float* t_s = red + kWarps * kTileRows * R;
  float* dt_s = t_s + kTileRows * S::kSmallStride;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  for (int idx = threadIdx.x; idx < R * N / 4; idx += kThreads) {
    const int n = idx / (N / 4), c = idx - n * (N / 4);
    *reinterpret_cast<float4*>(b_s + n * S::kBStride + 4 * c) = *reinterpret_cast<const float4*>(B + n * N + 4 * c);
  }
  constexpr int kNTiles = N / kWarps / 8;        // dB: this warp's 8-wide column tiles
  constexpr int kMTiles = K / kWarps / 16;       // dA: this warp's 16-tall feature tiles
  float gb[kNTiles][4];
  float ga[kMTiles][R / 8][4];
#pragma unroll
  for (int i = 0; i < kNTiles; ++i) gb[i][0] = gb[i][1] = gb[i][2] = gb[i][3] = 0.0f;
#pragma unroll
  for (int i = 0; i < kMTiles; ++i)
#pragma unroll
    for (int j = 0; j < R / 8; ++j) ga[i][j][0] = ga[i][j][1] = ga[i][j][2] = ga[i][j][3] = 0.0f;

  const size_t tiles = (M + kTileRows - 1) / kTileRows;
  auto load_dy_t = [&](size_t tile) {
    LoadTile<N>(dy_s, S::kDyStride, dy, tile * kTileRows, M);
    LoadTile<R>(t_s, S::kSmallStride, t, tile * kTileRows, M);
  };
  size_t tile = blockIdx.x;
  if (tile < tiles) load_dy_t(tile);
  CpAsyncCommit();   // group "dy"
  if (tile < tiles) LoadTile<K>(x_s, S::kXStride, x, tile * kTileRows, M);
  CpAsyncCommit();   // group "x"
  for (; tile < tiles; tile += gridDim.x) {
    const size_t row0 = tile * kTileRows;
    CpAsyncWait<1>();   // this tile's dY and t have landed (its x may still be in flight)
    __syncthreads();
    // dT tile = alpha dY B^T.
    RowsTimesWeight<N, R>(dy_s, S::kDyStride, [&](int n, int k) { return b_s[n * S::kBStride + k]; }, red, dt_s,
                          S::kSmallStride, alpha_dt);
    for (int idx = threadIdx.x; idx < kTileRows * R / 4; idx += kThreads) {
      const int r = idx / (R / 4), c = idx - r * (R / 4);
      if (row0 + r < M)
        *reinterpret_cast<float4*>(dt + (row0 + r) * R + 4 * c) =
            *reinterpret_cast<const float4*>(dt_s + r * S::kSmallStride + 4 * c);
    }
    // dB += t^T dY over the tile's 16 rows: A(i, k) = t[k][i], B(k, n) = dY[k][n].
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      uint32_t ah[4], al[4];
      const float* tr0 = t_s + (ks * 8 + tq) * S::kSmallStride;
      const float* tr1 = t_s + (ks * 8 + tq + 4) * S::kSmallStride;
      SplitTf32(tr0[g], &ah[0], &al[0]);
      SplitTf32(R > 8 ? tr0[g + 8] : 0.0f, &ah[1], &al[1]);
      SplitTf32(tr1[g], &ah[2], &al[2]);
      SplitTf32(R > 8 ? tr1[g + 8] : 0.0f, &ah[3], &al[3]);
      const float* dr0 = dy_s + (ks * 8 + tq) * S::kDyStride + warp * (N / kWarps) + g;
      const float* dr1 = dy_s + (ks * 8 + tq + 4) * S::kDyStride + warp * (N / kWarps) + g;
#pragma unroll
      for (int i = 0; i < kNTiles; ++i) {
        uint32_t bh[2], bl[2];
        SplitTf32(dr0[8 * i], &bh[0], &bl[0]);
        SplitTf32(dr1[8 * i], &bh[1], &bl[1]);
        Mma3(gb[i], ah, al, bh, bl);
      }
    }
    CpAsyncWait<0>();   // this tile's x
    __syncthreads();    // ... and every warp is done with dy_s and t_s
    if (tile + gridDim.x < tiles) load_dy_t(tile + gridDim.x);
    CpAsyncCommit();
    // dA += x^T dT: A(i, k) = x[k][i], B(k, n) = dT[k][n].
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      uint32_t bh[R / 8][2], bl[R / 8][2];
#pragma unroll
      for (int j = 0; j < R / 8; ++j) {
        SplitTf32(dt_s[(ks * 8 + tq) * S::kSmallStride + 8 * j + g], &bh[j][0], &bl[j][0]);
        SplitTf32(dt_s[(ks * 8 + tq + 4) * S::kSmallStride + 8 * j + g], &bh[j][1], &bl[j][1]);
      }
      const float* xr0 = x_s + (ks * 8 + tq) * S::kXStride + warp * (K / kWarps) + g;
      const float* xr1 = x_s + (ks * 8 + tq + 4) * S::kXStride + warp * (K / kWarps) + g;
#pragma unroll
      for (int i = 0; i < kMTiles; ++i) {
        uint32_t ah[4], al[4];
        SplitTf32(xr0[16 * i], &ah[0], &al[0]);
        SplitTf32(xr0[16 * i + 8], &ah[1], &al[1]);
        SplitTf32(xr1[16 * i], &ah[2], &al[2]);
        SplitTf32(xr1[16 * i + 8], &ah[3], &al[3]);
#pragma unroll
        for (int j = 0; j < R / 8; ++j) Mma3(ga[i][j], ah, al, bh[j], bl[j]);
      }
    }
    __syncthreads();    // every warp is done with x_s and dt_s
    if (tile + gridDim.x < tiles) LoadTile<K>(x_s, S::kXStride, x, (tile + gridDim.x) * kTileRows, M);
    CpAsyncCommit();
  }
  CpAsyncWait<0>();
  // This block's partial sums: dB [R][N], then dA [K][R].
  float* pb = partials + static_cast<size_t>(blockIdx.x) * (static_cast<size_t>(R) * N + static_cast<size_t>(K) * R);
  float* pa = pb + static_cast<size_t>(R) * N;
#pragma unroll
  for (int i = 0; i < kNTiles; ++i) {
    const int n = warp * (N / kWarps) + 8 * i + 2 * tq;
    *reinterpret_cast<float2*>(pb + g * N + n) = make_float2(gb[i][0], gb[i][1]);
    if (R > 8) *reinterpret_cast<float2*>(pb + (g + 8) * N + n) = make_float2(gb[i][2], gb[i][3]);
  }
#pragma unroll
  for (int i = 0; i < kMTiles; ++i) {
    const int f = warp * (K / kWarps) + 16 * i + g;
#pragma unroll
    for (int j = 0; j < R / 8; ++j) {
      *reinterpret_cast<float2*>(pa + f * R + 8 * j + 2 * tq) = make_float2(ga[i][j][0], ga[i][j][1]);
      *reinterpret_cast<float2*>(pa + (f + 8) * R + 8 * j + 2 * tq) = make_float2(ga[i][j][2], ga[i][j][3]);
    }
  }
}

// out[i] = alpha * (partials[0][i] + partials[1][i] + ...), blocks in order.
__global__ void FoldPartialsKernel(const float* __restrict__ partials, size_t stride, int blocks, size_t offset,
                                   size_t n, float alpha, float* __restrict__ out) {
  const size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (i >= n) return;
  float s = partials[offset + i];
  for (int b = 1; b < blocks; ++b) s += partials[static_cast<size_t>(b) * stride + offset + i];
  out[i] = alpha * s;
}

template <typename Kernel>
bool Configure(Kernel kernel, size_t smem_bytes, std::atomic<bool>* flags) {
  int dev = 0;
  cudaGetDevice(&dev);
  const bool tracked = dev >= 0 && dev < 64;
  if (tracked && flags[dev].load(std::memory_order_acquire)) return true;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_bytes)) !=
      cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  if (tracked) flags[dev].store(true, std::memory_order_release);
  return true;
}

int SmCount() {
  static std::atomic<int> cached[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 148;
  int n = cached[dev].load(std::memory_order_acquire);
  if (n == 0) {
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
    cached[dev].store(n, std::memory_order_release);
  }
  return n;
}

template <int K, int R>
bool LaunchDown(const float* x, const float* A, float* out, size_t M, float alpha, cudaStream_t s) {
  static std::atomic<bool> configured[64] = {};
  const size_t smem = DownSmem<K, R>::kFloats * sizeof(float);
  if (!Configure(LoraDownKernel<K, R>, smem, configured)) return false;
  const size_t tiles = (M + kTileRows - 1) / kTileRows;
  const unsigned grid = static_cast<unsigned>(tiles < static_cast<size_t>(SmCount()) ? tiles : SmCount());
  LoraDownKernel<K, R><<<grid, kThreads, smem, s>>>(x, A, out, M, alpha);
  return true;
}

template <int N, int K, int R>
bool LaunchBackward(const LoraBackwardArgs& a, cudaStream_t s) {
  static std::atomic<bool> configured[64] = {};
  const size_t smem = BackSmem<N, K, R>::kFloats * sizeof(float);
  if (!Configure(LoraBackwardKernel<N, K, R>, smem, configured)) return false;
  const size_t tiles = (a.M + kTileRows - 1) / kTileRows;
  const int blocks = static_cast<int>(tiles < static_cast<size_t>(SmCount()) ? tiles : SmCount());
  const size_t stride = static_cast<size_t>(R) * N + static_cast<size_t>(K) * R;
  if (static_cast<size_t>(blocks) * stride > a.partials_floats) return false;
  LoraBackwardKernel<N, K, R><<<blocks, kThreads, smem, s>>>(a.dy, a.x, a.t, a.B, a.dt, a.partials, a.M, a.alpha_dt);
  FoldPartialsKernel<<<static_cast<unsigned>((static_cast<size_t>(R) * N + 255) / 256), 256, 0, s>>>(
      a.partials, stride, blocks, 0, static_cast<size_t>(R) * N, a.alpha_db, a.dB);
  FoldPartialsKernel<<<static_cast<unsigned>((static_cast<size_t>(K) * R + 255) / 256), 256, 0, s>>>(
      a.partials, stride, blocks, static_cast<size_t>(R) * N, static_cast<size_t>(K) * R, a.alpha_da, a.dA);
  return true;
}

bool Aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

size_t LoraBackwardPartialFloats(size_t N, size_t K, size_t r) {
  return static_cast<size_t>(SmCount()) * (r * N + K * r);
}

bool LoraDownSupported(size_t M, size_t K, size_t r) {
  return M >= 64 && ((K == 768 && (r == 16 || r == 8)) || (K == 256 && r == 8));
}

bool LoraDown(const float* x, const float* A, float* out, size_t M, size_t K, size_t r, float alpha, cudaStream_t s) {
  if (!LoraDownSupported(M, K, r) || !Aligned16(x) || !Aligned16(A) || !Aligned16(out)) return false;
  if (K == 768 && r == 16) return LaunchDown<768, 16>(x, A, out, M, alpha, s);
  if (K == 768 && r == 8) return LaunchDown<768, 8>(x, A, out, M, alpha, s);
  return LaunchDown<256, 8>(x, A, out, M, alpha, s);
}

bool LoraBackwardSupported(size_t M, size_t N, size_t K, size_t r) {
  return M >= 64 && ((N == 768 && K == 768 && (r == 16 || r == 8)) || (N == 256 && K == 256 && r == 8));
}

bool LoraBackward(const LoraBackwardArgs& a, cudaStream_t s) {
  if (!LoraBackwardSupported(a.M, a.N, a.K, a.r)) return false;
  if (!Aligned16(a.dy) || !Aligned16(a.x) || !Aligned16(a.t) || !Aligned16(a.B) || !Aligned16(a.dt) ||
      !Aligned16(a.partials))
    return false;
  if (a.N == 768 && a.r == 16) return LaunchBackward<768, 768, 16>(a, s);
  if (a.N == 768 && a.r == 8) return LaunchBackward<768, 768, 8>(a, s);
  return LaunchBackward<256, 256, 8>(a, s);
}

}  // namespace see::k
