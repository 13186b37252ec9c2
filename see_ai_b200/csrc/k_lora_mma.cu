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
//
// Both kernels run at the issue rate of the tensor instruction, not at HBM speed
// (about 5.6 cycles per m16n8k8 and SM).  Two cheaper-looking forms were measured
// on the bench shapes and are not kept: the same products as two-piece bf16
// splits on m16n8k16 (half the instructions, each twice as long: no faster), and
// as register-tiled f32 multiply-adds on the CUDA cores (bound by shared-memory
// operand reads at twice the time).
#include <atomic>

#include "kernels.h"
#include "lora_split.cuh"
#include "lora_umma.h"

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
// A warp owns a 16-row tile over the whole of K: no partial tiles to fold, no
// block-wide barrier after the prologue.  x goes from global memory straight into
// the tensor instruction's row fragments: the reduction index inside a 16-wide
// block of k is permuted (lane t takes columns 4t .. 4t+3: the pairs (4t, 4t+1)
// and (4t+2, 4t+3) are the (t, t+4) elements of two successive instructions), so
// that each lane reads its share as one 16-byte load per row and block, four
// blocks ahead of their use.  A^T sits in shared memory already cut into (hi, lo), read
// with the same permutation.  Every product term keeps its own accumulator
// (lo*hi, hi*lo, hi*hi per 8-column group), so successive instructions do not
// wait on each other; the terms are added small ones first at the end.  With
// `pieces` set the tile also leaves as the three-way bf16 cut that a base
// product's reduction takes as extra K columns (lora_split.cuh), which saves the
// separate pass over t.  (Measured at 32768 x 768, r 16: 30 us, the issue rate of
// the tensor instruction; the same product as register-tiled f32 multiply-adds on
// the CUDA cores was bound by shared-memory reads at twice that.)
constexpr int kDownThreads = 512;
constexpr int kDownWarps = kDownThreads / 32;
constexpr int kDownAhead = 4;   // 16-wide k blocks in flight per lane and row

//
// With fewer tiles than warps on the device (a data-parallel rank's share of the rows) the
// reduction axis is cut instead: `ksplit` warps (a power of two) share a tile, each over its
// own run of k blocks, and the tile's first warp adds their sums in warp order through
// shared memory — a fixed order, so a given row count always gives the same bits.
template <int K, int R>
struct DownSmem {
  static constexpr int kStride = K + 16;   // rows 16 banks apart: a quarter warp's two rows cover all 32
  static constexpr size_t kWeightFloats = 2 * static_cast<size_t>(R) * kStride;
  static constexpr int kLaneFloats = R / 8 * 4;   // one lane's share of a tile's sums
  static constexpr size_t kFloats = kWeightFloats + static_cast<size_t>(kDownThreads) * kLaneFloats;
};

template <int K, int R, bool kSplitK>
__global__ void __launch_bounds__(kDownThreads, 1)
LoraDownKernel(const float* __restrict__ x, const float* __restrict__ A, float* __restrict__ out,
               uint16_t* __restrict__ pieces, uint32_t piece_cols, size_t M, float alpha, int ksplit) {
  using S = DownSmem<K, R>;
  extern __shared__ __align__(16) float smem[];
  uint32_t* a_hi = reinterpret_cast<uint32_t*>(smem);
  uint32_t* a_lo = a_hi + static_cast<size_t>(R) * S::kStride;
  float* part = smem + S::kWeightFloats;   // [warp][lane][kLaneFloats]
  for (int idx = threadIdx.x; idx < K * R; idx += kDownThreads) {   // A [K][R] -> a[n][k], k fastest (bank-free stores)
    const int n = idx / K, k = idx - n * K;
    SplitTf32(__ldg(A + k * R + n), &a_hi[n * S::kStride + k], &a_lo[n * S::kStride + k]);
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  constexpr int kBlocks = K / 16;
  const size_t tiles = (M + kTileRows - 1) / kTileRows;
  // Tile order: group w (a warp, or `ksplit` warps) of block b takes tiles w * gridDim.x + b,
  // + gridDim.x * groups, ...  Every warp makes the same number of trips (the shared-memory
  // hand-over below has block-wide barriers); a trip past the last tile computes nothing.
  const int groups = kSplitK ? kDownWarps / ksplit : kDownWarps;
  const int group = kSplitK ? warp / ksplit : warp;
  const int member = kSplitK ? warp - group * ksplit : 0;
  const int kb0 = kSplitK ? member * (kBlocks / ksplit) : 0;
  const int kb1 = kSplitK ? kb0 + kBlocks / ksplit : kBlocks;
  const size_t stride = static_cast<size_t>(gridDim.x) * groups;
  const size_t trips = kSplitK ? (tiles + stride - 1) / stride : 0;
  size_t trip = 0;
  for (size_t tile = static_cast<size_t>(group) * gridDim.x + blockIdx.x; kSplitK ? trip < trips : tile < tiles;
       tile += stride, ++trip) {
    const bool live = tile < tiles;
    const size_t row_a = tile * kTileRows + g, row_b = row_a + 8;
    const bool in_a = live && row_a < M, in_b = live && row_b < M;
    const float* xa = x + (in_a ? row_a : 0) * K + 4 * t;
    const float* xb = x + (in_b ? row_b : 0) * K + 4 * t;
    float c[R / 8][3][4];
#pragma unroll
    for (int j = 0; j < R / 8; ++j)
#pragma unroll
      for (int term = 0; term < 3; ++term) c[j][term][0] = c[j][term][1] = c[j][term][2] = c[j][term][3] = 0.0f;
    float4 va[kDownAhead], vb[kDownAhead];
#pragma unroll
    for (int p = 0; p < kDownAhead; ++p) {
      if (kSplitK && (!live || kb0 + p >= kb1)) continue;
      va[p] = __ldg(reinterpret_cast<const float4*>(xa + 16 * (kb0 + p)));
      vb[p] = __ldg(reinterpret_cast<const float4*>(xb + 16 * (kb0 + p)));
    }
#pragma unroll 1
    for (int s0 = kb0; s0 < (kSplitK && !live ? kb0 : kb1); s0 += kDownAhead) {
#pragma unroll
      for (int p = 0; p < kDownAhead; ++p) {
        const int s = s0 + p;
        if (kSplitK && s >= kb1) break;
        const float4 ua = va[p], ub = vb[p];
        if (s + kDownAhead < kb1) {
          va[p] = __ldg(reinterpret_cast<const float4*>(xa + 16 * (s + kDownAhead)));
          vb[p] = __ldg(reinterpret_cast<const float4*>(xb + 16 * (s + kDownAhead)));
        }
        uint32_t ah0[4], al0[4], ah1[4], al1[4];   // the block's two instructions' row fragments
        SplitTf32(ua.x, &ah0[0], &al0[0]);
        SplitTf32(ub.x, &ah0[1], &al0[1]);
        SplitTf32(ua.y, &ah0[2], &al0[2]);
        SplitTf32(ub.y, &ah0[3], &al0[3]);
        SplitTf32(ua.z, &ah1[0], &al1[0]);
        SplitTf32(ub.z, &ah1[1], &al1[1]);
        SplitTf32(ua.w, &ah1[2], &al1[2]);
        SplitTf32(ub.w, &ah1[3], &al1[3]);
#pragma unroll
        for (int j = 0; j < R / 8; ++j) {
          const uint4 h = *reinterpret_cast<const uint4*>(a_hi + (8 * j + g) * S::kStride + 16 * s + 4 * t);
          const uint4 l = *reinterpret_cast<const uint4*>(a_lo + (8 * j + g) * S::kStride + 16 * s + 4 * t);
          const uint32_t bh0[2] = {h.x, h.y}, bl0[2] = {l.x, l.y}, bh1[2] = {h.z, h.w}, bl1[2] = {l.z, l.w};
          Mma1688(c[j][0], al0, bh0);
          Mma1688(c[j][1], ah0, bl0);
          Mma1688(c[j][2], ah0, bh0);
          Mma1688(c[j][0], al1, bh1);
          Mma1688(c[j][1], ah1, bl1);
          Mma1688(c[j][2], ah1, bh1);
        }
      }
    }
    // This lane holds rows g and g + 8, columns 8 j + 2 t and + 1.
    if (kSplitK) {
      float* mine = part + (static_cast<size_t>(warp) * 32 + lane) * S::kLaneFloats;
      if (member != 0) {
#pragma unroll
        for (int j = 0; j < R / 8; ++j)
          *reinterpret_cast<float4*>(mine + 4 * j) =
              make_float4((c[j][0][0] + c[j][1][0]) + c[j][2][0], (c[j][0][1] + c[j][1][1]) + c[j][2][1],
                          (c[j][0][2] + c[j][1][2]) + c[j][2][2], (c[j][0][3] + c[j][1][3]) + c[j][2][3]);
      }
      __syncthreads();
      if (member == 0) {
#pragma unroll
        for (int j = 0; j < R / 8; ++j) {
#pragma unroll
          for (int e = 0; e < 4; ++e) c[j][0][e] = (c[j][0][e] + c[j][1][e]) + c[j][2][e];
          for (int w = 1; w < ksplit; ++w) {
            const float4 o = *reinterpret_cast<const float4*>(mine + static_cast<size_t>(w) * 32 * S::kLaneFloats + 4 * j);
            c[j][0][0] += o.x; c[j][0][1] += o.y; c[j][0][2] += o.z; c[j][0][3] += o.w;
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) c[j][1][e] = c[j][2][e] = 0.0f;
        }
      }
      __syncthreads();
      if (member != 0) continue;
    }
#pragma unroll
    for (int j = 0; j < R / 8; ++j) {
      float v[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) v[e] = alpha * ((c[j][0][e] + c[j][1][e]) + c[j][2][e]);
      const int col = 8 * j + 2 * t;
      if (in_a) *reinterpret_cast<float2*>(out + row_a * R + col) = make_float2(v[0], v[1]);
      if (in_b) *reinterpret_cast<float2*>(out + row_b * R + col) = make_float2(v[2], v[3]);
      if (pieces != nullptr) {
        uint16_t p[4][3];
#pragma unroll
        for (int e = 0; e < 4; ++e) Split3(v[e], p[e]);
#pragma unroll
        for (int sgm = 0; sgm < 6; ++sgm) {
          const int pc = PieceOf(0, sgm);
          if (in_a)
            *reinterpret_cast<uint32_t*>(pieces + row_a * piece_cols + sgm * R + col) =
                static_cast<uint32_t>(p[0][pc]) | (static_cast<uint32_t>(p[1][pc]) << 16);
          if (in_b)
            *reinterpret_cast<uint32_t*>(pieces + row_b * piece_cols + sgm * R + col) =
                static_cast<uint32_t>(p[2][pc]) | (static_cast<uint32_t>(p[3][pc]) << 16);
        }
      }
    }
    if (pieces != nullptr) {   // the padding columns [6 R, piece_cols): each lane of a row's four an equal share
      for (uint32_t k = 6 * R + 2 * t; k < piece_cols; k += 8) {
        if (in_a) *reinterpret_cast<uint32_t*>(pieces + row_a * piece_cols + k) = 0u;
        if (in_b) *reinterpret_cast<uint32_t*>(pieces + row_b * piece_cols + k) = 0u;
      }
    }
  }
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
                   float alpha_dt, uint16_t* __restrict__ pieces, uint32_t piece_cols) {
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
    if (pieces != nullptr) {   // dT's three-way bf16 cut, for the product that takes dT A^T into its reduction
      for (int idx = threadIdx.x; idx < kTileRows * R / 2; idx += kThreads) {   // two columns per thread
        const int r = idx / (R / 2), j = 2 * (idx - r * (R / 2));
        if (row0 + r >= M) continue;
        uint16_t p0[3], p1[3];
        Split3(dt_s[r * S::kSmallStride + j], p0);
        Split3(dt_s[r * S::kSmallStride + j + 1], p1);
        uint16_t* dst = pieces + (row0 + r) * piece_cols + j;
#pragma unroll
        for (int sg = 0; sg < 6; ++sg) {
          const int pc = PieceOf(0, sg);
          *reinterpret_cast<uint32_t*>(dst + sg * R) =
              static_cast<uint32_t>(p0[pc]) | (static_cast<uint32_t>(p1[pc]) << 16);
        }
      }
      const int pad_pairs = (static_cast<int>(piece_cols) - 6 * R) / 2;   // the padding columns [6 R, piece_cols)
      for (int idx = threadIdx.x; idx < kTileRows * pad_pairs; idx += kThreads) {
        const int r = idx / pad_pairs, c = idx - r * pad_pairs;
        if (row0 + r < M) *reinterpret_cast<uint32_t*>(pieces + (row0 + r) * piece_cols + 6 * R + 2 * c) = 0u;
      }
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

// dB[i] = alpha_db * sum over blocks of partials[b][i] for i < n_db, dA likewise from the part
// after it.  Four lanes share an output: lane q adds its quarter of the blocks in block
// order (eight loads in flight), then the four sums are added in lane order — a fixed
// order, so the result is the same from run to run.
__global__ void FoldPartialsKernel(const float* __restrict__ partials, size_t stride, int blocks, size_t n_db,
                                   size_t n_da, float alpha_db, float alpha_da, float* __restrict__ dB,
                                   float* __restrict__ dA) {
  const size_t tid = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  const size_t i = tid >> 2;
  const int q = static_cast<int>(tid & 3);
  const bool live = i < n_db + n_da;
  const int per = (blocks + 3) / 4;
  const int b0 = q * per, b1 = b0 + per < blocks ? b0 + per : blocks;
  float s = 0.0f;
  if (live) {
    const float* p = partials + i;
    int b = b0;
    for (; b + 8 <= b1; b += 8) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = __ldg(p + static_cast<size_t>(b + u) * stride);
#pragma unroll
      for (int u = 0; u < 8; ++u) s += v[u];
    }
    for (; b < b1; ++b) s += __ldg(p + static_cast<size_t>(b) * stride);
  }
  // (lanes 4k .. 4k+3 hold one output's four sums)
  const float s1 = __shfl_down_sync(0xFFFFFFFFu, s, 1);
  const float s2 = __shfl_down_sync(0xFFFFFFFFu, s, 2);
  const float s3 = __shfl_down_sync(0xFFFFFFFFu, s, 3);
  if (live && q == 0) {
    const float total = ((s + s1) + s2) + s3;
    if (i < n_db) dB[i] = alpha_db * total;
    else dA[i - n_db] = alpha_da * total;
  }
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
bool LaunchDown(const float* x, const float* A, float* out, uint16_t* pieces, uint32_t piece_cols, size_t M,
                float alpha, cudaStream_t s) {
  static std::atomic<bool> configured[64] = {};
  const size_t smem = DownSmem<K, R>::kFloats * sizeof(float);
  static std::atomic<bool> configured_split[64] = {};
  if (!Configure(LoraDownKernel<K, R, false>, smem, configured)) return false;
  if (!Configure(LoraDownKernel<K, R, true>, smem, configured_split)) return false;
  // One block per SM as soon as there is a tile per SM: the tiles go round the blocks first.
  const size_t tiles = (M + kTileRows - 1) / kTileRows;
  const size_t sms = static_cast<size_t>(SmCount());
  const unsigned grid = static_cast<unsigned>(tiles < sms ? tiles : sms);
  // Warps per tile: the largest power of two that still leaves every tile a group of warps.
  int ksplit = 1;
  while (ksplit < kDownWarps && (K / 16) % (2 * ksplit) == 0 && tiles * (2 * ksplit) <= sms * kDownWarps) ksplit *= 2;
  if (ksplit > 1)
    LoraDownKernel<K, R, true><<<grid, kDownThreads, smem, s>>>(x, A, out, pieces, piece_cols, M, alpha, ksplit);
  else
    LoraDownKernel<K, R, false><<<grid, kDownThreads, smem, s>>>(x, A, out, pieces, piece_cols, M, alpha, 1);
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
  LoraBackwardKernel<N, K, R><<<blocks, kThreads, smem, s>>>(a.dy, a.x, a.t, a.B, a.dt, a.partials, a.M, a.alpha_dt,
                                                             a.dt_pieces, LoraSplitColumns(static_cast<uint32_t>(R)));
  FoldPartialsKernel<<<static_cast<unsigned>((4 * stride + 255) / 256), 256, 0, s>>>(
      a.partials, stride, blocks, static_cast<size_t>(R) * N, static_cast<size_t>(K) * R, a.alpha_db, a.alpha_da, a.dB,
      a.dA);
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

bool LoraDown(const float* x, const float* A, float* out, size_t M, size_t K, size_t r, float alpha, cudaStream_t s,
              uint16_t* pieces) {
  if (!LoraDownSupported(M, K, r) || !Aligned16(x) || !Aligned16(A) || !Aligned16(out) || !Aligned16(pieces))
    return false;
  const uint32_t cols = LoraSplitColumns(static_cast<uint32_t>(r));
  if (K == 768 && r == 16) return LaunchDown<768, 16>(x, A, out, pieces, cols, M, alpha, s);
  if (K == 768 && r == 8) return LaunchDown<768, 8>(x, A, out, pieces, cols, M, alpha, s);
  return LaunchDown<256, 8>(x, A, out, pieces, cols, M, alpha, s);
}

void LoraFoldPartials(const LoraBackwardArgs& a, int blocks, cudaStream_t s) {
  const size_t stride = a.r * a.N + a.K * a.r;
  FoldPartialsKernel<<<static_cast<unsigned>((4 * stride + 255) / 256), 256, 0, s>>>(
      a.partials, stride, blocks, a.r * a.N, a.K * a.r, a.alpha_db, a.alpha_da, a.dB, a.dA);
}

bool LoraBackwardSupported(size_t M, size_t N, size_t K, size_t r) {
  return M >= 64 && ((N == 768 && K == 768 && (r == 16 || r == 8)) || (N == 256 && K == 256 && r == 8));
}

bool LoraBackward(const LoraBackwardArgs& a, cudaStream_t s) {
  if (!LoraBackwardSupported(a.M, a.N, a.K, a.r)) return false;
  if (!Aligned16(a.dy) || !Aligned16(a.x) || !Aligned16(a.t) || !Aligned16(a.B) || !Aligned16(a.dt) ||
      !Aligned16(a.partials) || !Aligned16(a.dt_pieces))
    return false;
  if (a.N == 768 && a.r == 16) return LaunchBackward<768, 768, 16>(a, s);
  if (a.N == 768 && a.r == 8) return LaunchBackward<768, 768, 8>(a, s);
  return LaunchBackward<256, 256, 8>(a, s);
}

}  // namespace see::k
