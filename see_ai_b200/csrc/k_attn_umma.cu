// Causal attention on the tensor cores, for the tiled attention opcodes that
// carry the relaxed permission (reference: source/plan/instruction.h:174-190,
// 356-382; the reference's own relaxed attention is the matrix-tile family of
// runtime/executor/metal_backend.mm:1742-1802).  Same contract as the exact
// tiled family (reference: runtime/executor/attention.cc:448-590): the forward
// writes O and the stats row {score max, 1/denominator, 0, start}; dQ writes
// delta into the stats row and dQ; dK and dV read the stats row.
//
// Blackwell-native: per (sequence, head) the operands are packed once to bf16
// ([S][d] and [d][S]), tiles arrive by TMA (128-byte swizzle), every product
// (Q K^T, P V, dO V^T, dS K, dS^T Q, P^T dO) is a tcgen05.mma with its
// accumulator in tensor memory, and the softmax / softmax-backward arithmetic
// runs in f32 registers on values read with tcgen05.ld; P and dS go back to
// shared memory as bf16 for the second product.  Statistics are exact f32
// reductions of the bf16 products: two passes over the key tiles (first the
// row statistics, then the normalised probabilities), so no accumulator is
// ever rescaled.  128 threads per CTA, one query row (or key row) per thread;
// thread 0 issues TMA and MMA.  Every mbarrier wait is bounded; a wait that
// runs out raises DeviceStatus::wait_timeout and the CTA stores nothing.
//
// Tensor-pipe bound by FLOP count; this first version serialises load, MMA
// and softmax inside a CTA and relies on co-resident CTAs for overlap.
#include <cuda.h>

#include "attn_umma.h"
#include "kernels.h"
#include "umma_device.cuh"

namespace see::k {

using namespace umma_dev;

namespace {

constexpr uint32_t kTile = 128;          // query rows / key rows per tile
constexpr uint32_t kSubTileBytes = 128 * 64 * 2;   // [128 rows][64 bf16], swizzled
constexpr uint32_t kPBytes = 2 * kSubTileBytes;    // P / dS tile: 128 x 128 bf16

// ---- packing: f32 [B*S, H*d] -> bf16 [B*H][S][d] (rows) and [B*H][d][S] (cols) ----
// One block packs 64 positions of one (sequence, head): 16-byte loads of the f32
// rows, 8-byte stores of the bf16 row layout straight from registers, and the
// column layout through a shared-memory transpose, again as 8-byte stores (four
// positions of one feature).  Reads the source once for both layouts.
__device__ __forceinline__ uint32_t Bf16Bits(float f) {   // round to nearest even; NaN stays NaN
  uint32_t u = __float_as_uint(f);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (u >> 16) | 0x0040u;
  u += 0x7FFFu + ((u >> 16) & 1u);
  return u >> 16;
}

constexpr uint32_t kPackPos = 64;

template <int D>
__global__ void __launch_bounds__(256)
PackHeadsKernel(const float* __restrict__ x, uint16_t* __restrict__ rows, uint16_t* __restrict__ cols,
                uint32_t S, uint32_t H) {
  __shared__ uint16_t tile[kPackPos][D + 2];   // odd word stride: conflict-free transpose reads
  const uint32_t bh = blockIdx.y, b = bh / H, h = bh % H;
  const uint32_t s0 = blockIdx.x * kPackPos;
  const size_t HD = static_cast<size_t>(H) * D;
  constexpr uint32_t kVecPerRow = D / 4;
  for (uint32_t idx = threadIdx.x; idx < kPackPos * kVecPerRow; idx += 256) {
    const uint32_t i = idx / kVecPerRow, c = (idx % kVecPerRow) * 4;
    const uint32_t s = s0 + i;
    uint32_t lo = 0, hi = 0;
    if (s < S) {
      const float4 f = *reinterpret_cast<const float4*>(
          x + (static_cast<size_t>(b) * S + s) * HD + static_cast<size_t>(h) * D + c);
      lo = Bf16Bits(f.x) | (Bf16Bits(f.y) << 16);
      hi = Bf16Bits(f.z) | (Bf16Bits(f.w) << 16);
      if (rows)
        *reinterpret_cast<uint2*>(rows + (static_cast<size_t>(bh) * S + s) * D + c) = make_uint2(lo, hi);
    }
    *reinterpret_cast<uint32_t*>(&tile[i][c]) = lo;
    *reinterpret_cast<uint32_t*>(&tile[i][c + 2]) = hi;
  }
  if (!cols) return;
  __syncthreads();
  constexpr uint32_t kGroups = kPackPos / 4;   // groups of four positions
  for (uint32_t idx = threadIdx.x; idx < D * kGroups; idx += 256) {
    const uint32_t c = idx / kGroups, i = (idx % kGroups) * 4;
    const uint32_t s = s0 + i;
    if (s + 4 <= S) {
      const uint32_t lo = tile[i][c] | (static_cast<uint32_t>(tile[i + 1][c]) << 16);
      const uint32_t hi = tile[i + 2][c] | (static_cast<uint32_t>(tile[i + 3][c]) << 16);
      *reinterpret_cast<uint2*>(cols + (static_cast<size_t>(bh) * D + c) * S + s) = make_uint2(lo, hi);
    } else {
      for (uint32_t t = 0; t < 4 && s + t < S; ++t)
        cols[(static_cast<size_t>(bh) * D + c) * S + s + t] = tile[i + t][c];
    }
  }
}

struct Ctl {
  uint64_t load[2];
  uint64_t mma;
  uint32_t tmem_base;
  uint32_t pad;
};

// Loads a [128 rows][D] tile of a row-layout tensor ({d, S, BH} map) as D/64 sub-tiles.
template <int D>
__device__ __forceinline__ void LoadRowTile(uint8_t* dst, const CUtensorMap* map, uint64_t* bar,
                                            uint32_t row0, uint32_t bh) {
#pragma unroll
  for (int kb = 0; kb < D / 64; ++kb)
    TmaLoad3D(dst + kb * kSubTileBytes, map, bar, kb * 64, static_cast<int32_t>(row0),
              static_cast<int32_t>(bh));
}
// Loads a [D rows][128 positions] tile of a column-layout tensor ({S, d, BH} map) as two
// sub-tiles of [D][64].
template <int D>
__device__ __forceinline__ void LoadColTile(uint8_t* dst, const CUtensorMap* map, uint64_t* bar,
                                            uint32_t pos0, uint32_t bh) {
#pragma unroll
  for (int kb = 0; kb < 2; ++kb)
    TmaLoad3D(dst + kb * (D * 128), map, bar, static_cast<int32_t>(pos0 + kb * 64), 0,
              static_cast<int32_t>(bh));
}

// acc[128 x 128] (+)= A[128 rows][D] . B[128 rows][D]^T, both row tiles in shared memory.
template <int D>
__device__ __forceinline__ void MmaRowRow(uint32_t tmem, const uint8_t* a, const uint8_t* b) {
  const uint32_t idesc = MakeInstrDesc(128, 128);
#pragma unroll
  for (int kb = 0; kb < D / 64; ++kb) {
    const uint64_t da = MakeSmemDesc(SmemAddr(a + kb * kSubTileBytes));
    const uint64_t db = MakeSmemDesc(SmemAddr(b + kb * kSubTileBytes));
#pragma unroll
    for (int k = 0; k < 4; ++k) UmmaBf16(tmem, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
  }
}
// acc[128 x D] (+)= P[128 rows][128] . T[D rows][128]^T  (P: two [128][64] sub-tiles;
// T: two [D][64] sub-tiles).  `accumulate` = 0 starts a fresh accumulator.
template <int D>
__device__ __forceinline__ void MmaPT(uint32_t tmem, const uint8_t* p, const uint8_t* t,
                                      uint32_t accumulate) {
  const uint32_t idesc = MakeInstrDesc(128, D);
#pragma unroll
  for (int kb = 0; kb < 2; ++kb) {
    const uint64_t da = MakeSmemDesc(SmemAddr(p + kb * kSubTileBytes));
    const uint64_t db = MakeSmemDesc(SmemAddr(t + kb * (D * 128)));
#pragma unroll
    for (int k = 0; k < 4; ++k)
      UmmaBf16(tmem, da + 2 * k, db + 2 * k, idesc, (accumulate | kb | k) != 0 ? 1u : 0u);
  }
}

// Writes 32 consecutive values of this thread's row (columns c0 .. c0+31 of a 128-wide
// tile) into the swizzled bf16 tile P.
__device__ __forceinline__ void StoreRowChunk(uint8_t* p_tile, uint32_t row, uint32_t c0,
                                              const float (&v)[32]) {
  uint8_t* sub = p_tile + (c0 >> 6) * kSubTileBytes;
  const uint32_t chunk0 = (c0 & 63) >> 3;   // first 16-byte chunk (8 bf16) of the four
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint4 w;
    w.x = PackBf16x2(v[8 * q + 0], v[8 * q + 1]);
    w.y = PackBf16x2(v[8 * q + 2], v[8 * q + 3]);
    w.z = PackBf16x2(v[8 * q + 4], v[8 * q + 5]);
    w.w = PackBf16x2(v[8 * q + 6], v[8 * q + 7]);
    *reinterpret_cast<uint4*>(sub + Sw128Offset(row, chunk0 + q)) = w;
  }
}

__device__ __forceinline__ uint8_t* AlignSmem(uint8_t* raw) {
  return raw + ((1024u - (SmemAddr(raw) & 1023u)) & 1023u);
}

// ---- forward -------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(128)
AttnFwdUmmaKernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                  const __grid_constant__ CUtensorMap map_vt, AttnUmmaArgs a) {
  extern __shared__ uint8_t smem_raw[];
  Ctl* ctl = reinterpret_cast<Ctl*>(smem_raw);             // barriers first, tiles 1024-aligned after
  uint8_t* smem = AlignSmem(smem_raw + sizeof(Ctl));
  constexpr uint32_t kRowTile = 128 * D * 2, kColTile = D * 256;
  uint8_t* q_s = smem;
  uint8_t* stage_s = q_s + kRowTile;                       // 2 x (K row tile + Vt col tile)
  uint8_t* p_s = stage_s + 2 * (kRowTile + kColTile);
  constexpr uint32_t kTmemCols = 256;                      // S: 0..127, O: 128..128+D-1

  const uint32_t tid = threadIdx.x, warp = tid >> 5;
  const uint32_t n_qt = (a.S + kTile - 1) / kTile;
  const uint32_t it = n_qt - 1 - blockIdx.x;               // heaviest tiles first
  const uint32_t bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  const uint32_t n_kt = it + 1;
  const uint32_t total = 2 * n_kt;

  if (tid == 0) {
    MbarInit(&ctl->load[0], 1); MbarInit(&ctl->load[1], 1); MbarInit(&ctl->mma, 1);
    MbarInitFence();
  }
  if (warp == 0) TmemAlloc(&ctl->tmem_base, kTmemCols);
  TcFenceBefore();
  __syncthreads();
  TcFenceAfter();
  const uint32_t tmem = ctl->tmem_base;
  const uint32_t t_s = tmem + ((warp * 32) << 16);
  const uint32_t t_o = t_s + 128;

  auto issue_load = [&](uint32_t ld) {
    const uint32_t jt = ld % n_kt, st = ld & 1;
    const bool second = ld >= n_kt;
    uint8_t* k_dst = stage_s + st * (kRowTile + kColTile);
    uint32_t bytes = kRowTile + (second ? kColTile : 0) + (ld == 0 ? kRowTile : 0);
    MbarExpectTx(&ctl->load[st], bytes);
    if (ld == 0) LoadRowTile<D>(q_s, &map_q, &ctl->load[st], it * kTile, bh);
    LoadRowTile<D>(k_dst, &map_k, &ctl->load[st], jt * kTile, bh);
    if (second) LoadColTile<D>(k_dst + kRowTile, &map_vt, &ctl->load[st], jt * kTile, bh);
  };

  const uint32_t row = it * kTile + tid;                   // this thread's query row
  float m = -INFINITY, l = 0.0f, inv_l = 0.0f;
  uint32_t mma_phase = 0;
  int failed = 0;
  if (tid == 0) issue_load(0);

  for (uint32_t ld = 0; ld < total; ++ld) {
    const uint32_t jt = ld % n_kt, st = ld & 1;
    const bool second = ld >= n_kt;
    uint8_t* k_s = stage_s + st * (kRowTile + kColTile);
    if (tid == 0 && ld + 1 < total) issue_load(ld + 1);
    if (!MbarWait(&ctl->load[st], (ld >> 1) & 1)) failed = 1;
    if (tid == 0) {
      TcFenceAfter();
      MmaRowRow<D>(tmem, q_s, k_s);
      UmmaCommit(&ctl->mma);
    }
    if (!MbarWait(&ctl->mma, mma_phase)) failed = 1;
    mma_phase ^= 1;
    TcFenceAfter();
    if (ld == n_kt) inv_l = 1.0f / l;                      // statistics complete
    const uint32_t key0 = jt * kTile;
#pragma unroll 1
    for (uint32_t c0 = 0; c0 < kTile; c0 += 32) {
      uint32_t r[32];
      TmemLoad32(t_s + c0, r);
      TmemWaitLd();
      float v[32];
      if (!second) {
        float tile_max = -INFINITY;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float s = __uint_as_float(r[j]) * a.inv_sqrt_d;
          v[j] = (key0 + c0 + j <= row) ? s : -INFINITY;
          tile_max = fmaxf(tile_max, v[j]);
        }
        const float m_new = fmaxf(m, tile_max);
        if (m_new > -INFINITY) {
          float sum = 0.0f;
#pragma unroll
          for (int j = 0; j < 32; ++j) sum += __expf(v[j] - m_new);
          l = l * __expf(m - m_new) + sum;
          m = m_new;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float s = __uint_as_float(r[j]) * a.inv_sqrt_d;
          v[j] = (key0 + c0 + j <= row) ? __expf(s - m) * inv_l : 0.0f;
        }
        StoreRowChunk(p_s, tid, c0, v);
      }
    }
    if (second) FenceProxyAsync();
    TcFenceBefore();
    if (__syncthreads_or(failed)) { failed = 1; break; }
    if (second) {
      if (tid == 0) {
        TcFenceAfter();
        MmaPT<D>(tmem + 128, p_s, k_s + kRowTile, jt != 0);
        UmmaCommit(&ctl->mma);
      }
      if (!MbarWait(&ctl->mma, mma_phase)) failed = 1;
      mma_phase ^= 1;
      TcFenceAfter();
    }
  }
  failed = __syncthreads_or(failed);
  if (failed) {
    if (tid == 0) a.status->wait_timeout = 1;
  } else {
    // tcgen05.ld is warp-collective: every thread loads, only rows inside the
    // sequence store.
    const bool live = row < a.S;
    const size_t HD = static_cast<size_t>(a.H) * D;
    float* o = a.out + (static_cast<size_t>(b) * a.S + (live ? row : 0)) * HD + static_cast<size_t>(h) * D;
#pragma unroll 1
    for (uint32_t c0 = 0; c0 < D; c0 += 32) {
      uint32_t r[32];
      TmemLoad32(t_o + c0, r);
      TmemWaitLd();
      if (live) {
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(o + c0 + j) =
              make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                          __uint_as_float(r[j + 3]));
      }
    }
    if (live) {
      float* st = a.stats + (static_cast<size_t>(bh) * a.S + row) * kAttnStatsWidth;
      *reinterpret_cast<float4*>(st) = make_float4(m, inv_l, 0.0f, 0.0f);
    }
  }
  TcFenceBefore();
  __syncthreads();
  if (warp == 0) {
    TcFenceAfter();
    TmemFree(tmem, kTmemCols);
  }
}

// ---- dQ (and delta) --------------------------------------------------------------------
// Per query tile: pass 1 accumulates delta_i = sum_j P_ij dP_ij, pass 2 forms
// dS = P (dP - delta) / sqrt(d) and accumulates dQ = dS K.  NS = shared-memory
// stages for the per-key-tile operands (K rows, V rows, K columns).
template <int D, int NS>
__global__ void __launch_bounds__(128)
AttnDQUmmaKernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                 const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                 const __grid_constant__ CUtensorMap map_kt, AttnUmmaArgs a) {
  extern __shared__ uint8_t smem_raw[];
  Ctl* ctl = reinterpret_cast<Ctl*>(smem_raw);
  uint8_t* smem = AlignSmem(smem_raw + sizeof(Ctl));
  constexpr uint32_t kRowTile = 128 * D * 2, kColTile = D * 256;
  constexpr uint32_t kStage = 2 * kRowTile + kColTile;
  uint8_t* q_s = smem;
  uint8_t* do_s = q_s + kRowTile;
  uint8_t* stage_s = do_s + kRowTile;
  uint8_t* p_s = stage_s + NS * kStage;
  constexpr uint32_t kTmemCols = 512;                      // S 0..127, dP 128..255, dQ 256..

  const uint32_t tid = threadIdx.x, warp = tid >> 5;
  const uint32_t n_qt = (a.S + kTile - 1) / kTile;
  const uint32_t it = n_qt - 1 - blockIdx.x;
  const uint32_t bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  const uint32_t n_kt = it + 1, total = 2 * n_kt;

  if (tid == 0) {
    MbarInit(&ctl->load[0], 1); MbarInit(&ctl->load[1], 1); MbarInit(&ctl->mma, 1);
    MbarInitFence();
  }
  if (warp == 0) TmemAlloc(&ctl->tmem_base, kTmemCols);
  TcFenceBefore();
  __syncthreads();
  TcFenceAfter();
  const uint32_t tmem = ctl->tmem_base;
  const uint32_t t_lane = tmem + ((warp * 32) << 16);

  auto issue_load = [&](uint32_t ld) {
    const uint32_t jt = ld % n_kt, st = ld % NS;
    const bool second = ld >= n_kt;
    uint8_t* dst = stage_s + st * kStage;
    const uint32_t bytes = 2 * kRowTile + (second ? kColTile : 0) + (ld == 0 ? 2 * kRowTile : 0);
    MbarExpectTx(&ctl->load[st], bytes);
    if (ld == 0) {
      LoadRowTile<D>(q_s, &map_q, &ctl->load[st], it * kTile, bh);
      LoadRowTile<D>(do_s, &map_do, &ctl->load[st], it * kTile, bh);
    }
    LoadRowTile<D>(dst, &map_k, &ctl->load[st], jt * kTile, bh);
    LoadRowTile<D>(dst + kRowTile, &map_v, &ctl->load[st], jt * kTile, bh);
    if (second) LoadColTile<D>(dst + 2 * kRowTile, &map_kt, &ctl->load[st], jt * kTile, bh);
  };

  const uint32_t row = it * kTile + tid;
  const bool live = row < a.S;
  float* st_row = a.stats + (static_cast<size_t>(bh) * a.S + (live ? row : 0)) * kAttnStatsWidth;
  const float m = live ? st_row[0] : 0.0f;
  const float inv_l = live ? st_row[1] : 0.0f;
  float delta = 0.0f;
  uint32_t mma_phase = 0;
  int failed = 0;
  if (tid == 0) issue_load(0);

  for (uint32_t ld = 0; ld < total; ++ld) {
    const uint32_t jt = ld % n_kt, st = ld % NS;
    const bool second = ld >= n_kt;
    uint8_t* k_s = stage_s + st * kStage;
    if (NS == 2 && tid == 0 && ld + 1 < total) issue_load(ld + 1);
    if (!MbarWait(&ctl->load[st], (ld / NS) & 1)) failed = 1;
    if (tid == 0) {
      TcFenceAfter();
      MmaRowRow<D>(tmem, q_s, k_s);                        // S  = Q K^T
      MmaRowRow<D>(tmem + 128, do_s, k_s + kRowTile);      // dP = dO V^T
      UmmaCommit(&ctl->mma);
    }
    if (!MbarWait(&ctl->mma, mma_phase)) failed = 1;
    mma_phase ^= 1;
    TcFenceAfter();
    const uint32_t key0 = jt * kTile;
#pragma unroll 1
    for (uint32_t c0 = 0; c0 < kTile; c0 += 32) {
      uint32_t rs[32], rp[32];
      TmemLoad32(t_lane + c0, rs);
      TmemLoad32(t_lane + 128 + c0, rp);
      TmemWaitLd();
      float v[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float s = __uint_as_float(rs[j]) * a.inv_sqrt_d;
        const float p = (key0 + c0 + j <= row) ? __expf(s - m) * inv_l : 0.0f;
        const float dp = __uint_as_float(rp[j]);
        if (!second) delta += p * dp;
        v[j] = p * (dp - delta) * a.inv_sqrt_d;
      }
      if (second) StoreRowChunk(p_s, tid, c0, v);
    }
    if (second) FenceProxyAsync();
    TcFenceBefore();
    if (__syncthreads_or(failed)) { failed = 1; break; }
    if (second) {
      if (tid == 0) {
        TcFenceAfter();
        MmaPT<D>(tmem + 256, p_s, k_s + 2 * kRowTile, jt != 0);   // dQ += dS K
        UmmaCommit(&ctl->mma);
      }
      if (!MbarWait(&ctl->mma, mma_phase)) failed = 1;
      mma_phase ^= 1;
      TcFenceAfter();
    }
    if (NS == 1 && tid == 0 && ld + 1 < total) issue_load(ld + 1);
  }
  failed = __syncthreads_or(failed);
  if (failed) {
    if (tid == 0) a.status->wait_timeout = 1;
  } else {
    const size_t HD = static_cast<size_t>(a.H) * D;
    float* o = a.out + (static_cast<size_t>(b) * a.S + (live ? row : 0)) * HD + static_cast<size_t>(h) * D;
#pragma unroll 1
    for (uint32_t c0 = 0; c0 < D; c0 += 32) {
      uint32_t r[32];
      TmemLoad32(t_lane + 256 + c0, r);
      TmemWaitLd();
      if (live) {
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(o + c0 + j) =
              make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                          __uint_as_float(r[j + 3]));
      }
    }
    if (live) st_row[2] = delta;
  }
  TcFenceBefore();
  __syncthreads();
  if (warp == 0) {
    TcFenceAfter();
    TmemFree(tmem, kTmemCols);
  }
}

// ---- dK / dV ---------------------------------------------------------------------------
// Per key tile, over the query tiles at or below the diagonal, in the
// transposed frame: S^T = K Q^T (one key row per thread, query index along the
// columns), P^T from the stats rows of those queries; dV += P^T dO, or
// dS^T = P^T (dP^T - delta) / sqrt(d) with dP^T = V dO^T and dK += dS^T Q.
template <int D, bool kWantDK, int NS>
__global__ void __launch_bounds__(128)
AttnDKVUmmaKernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                  const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                  const __grid_constant__ CUtensorMap map_t, AttnUmmaArgs a) {
  extern __shared__ uint8_t smem_raw[];
  Ctl* ctl = reinterpret_cast<Ctl*>(smem_raw);
  uint8_t* smem = AlignSmem(smem_raw + sizeof(Ctl));
  constexpr uint32_t kRowTile = 128 * D * 2, kColTile = D * 256;
  constexpr uint32_t kStage = (kWantDK ? 2 : 1) * kRowTile + kColTile;
  uint8_t* k_s = smem;
  uint8_t* v_s = k_s + kRowTile;                            // used by dK only
  uint8_t* stage_s = v_s + (kWantDK ? kRowTile : 0);
  uint8_t* p_s = stage_s + NS * kStage;
  float* stat_s = reinterpret_cast<float*>(p_s + kPBytes);  // m[128], 1/l[128], delta[128]
  constexpr uint32_t kOutCol = kWantDK ? 256 : 128;
  constexpr uint32_t kTmemCols = kWantDK ? 512 : 256;

  const uint32_t tid = threadIdx.x, warp = tid >> 5;
  const uint32_t n_qt = (a.S + kTile - 1) / kTile;
  const uint32_t jt = blockIdx.x;                          // key tile; low tiles have the most work
  const uint32_t bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  const uint32_t total = n_qt - jt;

  if (tid == 0) {
    MbarInit(&ctl->load[0], 1); MbarInit(&ctl->load[1], 1); MbarInit(&ctl->mma, 1);
    MbarInitFence();
  }
  if (warp == 0) TmemAlloc(&ctl->tmem_base, kTmemCols);
  TcFenceBefore();
  __syncthreads();
  TcFenceAfter();
  const uint32_t tmem = ctl->tmem_base;
  const uint32_t t_lane = tmem + ((warp * 32) << 16);

  auto issue_load = [&](uint32_t ld) {
    const uint32_t it = jt + ld, st = ld % NS;
    uint8_t* dst = stage_s + st * kStage;
    const uint32_t bytes = kStage + (ld == 0 ? (kWantDK ? 2 : 1) * kRowTile : 0);
    MbarExpectTx(&ctl->load[st], bytes);
    if (ld == 0) {
      LoadRowTile<D>(k_s, &map_k, &ctl->load[st], jt * kTile, bh);
      if (kWantDK) LoadRowTile<D>(v_s, &map_v, &ctl->load[st], jt * kTile, bh);
    }
    LoadRowTile<D>(dst, &map_q, &ctl->load[st], it * kTile, bh);
    if (kWantDK) LoadRowTile<D>(dst + kRowTile, &map_do, &ctl->load[st], it * kTile, bh);
    LoadColTile<D>(dst + (kWantDK ? 2 : 1) * kRowTile, &map_t, &ctl->load[st], it * kTile, bh);
  };

  const uint32_t key = jt * kTile + tid;                    // this thread's key row
  uint32_t mma_phase = 0;
  int failed = 0;
  if (tid == 0) issue_load(0);

  for (uint32_t ld = 0; ld < total; ++ld) {
    const uint32_t it = jt + ld, st = ld % NS;
    uint8_t* q_s = stage_s + st * kStage;
    if (NS == 2 && tid == 0 && ld + 1 < total) issue_load(ld + 1);
    {  // stats rows of this query tile (zeros past the end of the sequence)
      const uint32_t qi = it * kTile + tid;
      float4 sv = make_float4(0.f, 0.f, 0.f, 0.f);
      if (qi < a.S)
        sv = *reinterpret_cast<const float4*>(a.stats + (static_cast<size_t>(bh) * a.S + qi) * kAttnStatsWidth);
      stat_s[tid] = sv.x; stat_s[128 + tid] = sv.y; stat_s[256 + tid] = sv.z;
    }
    __syncthreads();
    if (!MbarWait(&ctl->load[st], (ld / NS) & 1)) failed = 1;
    if (tid == 0) {
      TcFenceAfter();
      MmaRowRow<D>(tmem, k_s, q_s);                              // S^T  = K Q^T
      if (kWantDK) MmaRowRow<D>(tmem + 128, v_s, q_s + kRowTile); // dP^T = V dO^T
      UmmaCommit(&ctl->mma);
    }
    if (!MbarWait(&ctl->mma, mma_phase)) failed = 1;
    mma_phase ^= 1;
    TcFenceAfter();
    const uint32_t q0 = it * kTile;
#pragma unroll 1
    for (uint32_t c0 = 0; c0 < kTile; c0 += 32) {
      uint32_t rs[32], rp[32];
      TmemLoad32(t_lane + c0, rs);
      if (kWantDK) TmemLoad32(t_lane + 128 + c0, rp);
      TmemWaitLd();
      float v[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const uint32_t qi = q0 + c0 + j;
        const float s = __uint_as_float(rs[j]) * a.inv_sqrt_d;
        const bool ok = key <= qi && qi < a.S;
        const float p = ok ? __expf(s - stat_s[c0 + j]) * stat_s[128 + c0 + j] : 0.0f;
        if (kWantDK) v[j] = p * (__uint_as_float(rp[j]) - stat_s[256 + c0 + j]) * a.inv_sqrt_d;
        else v[j] = p;
      }
      StoreRowChunk(p_s, tid, c0, v);
    }
    FenceProxyAsync();
    TcFenceBefore();
    if (__syncthreads_or(failed)) { failed = 1; break; }
    if (tid == 0) {
      TcFenceAfter();
      MmaPT<D>(tmem + kOutCol, p_s, q_s + (kWantDK ? 2 : 1) * kRowTile, ld != 0);
      UmmaCommit(&ctl->mma);
    }
    if (!MbarWait(&ctl->mma, mma_phase)) failed = 1;
    mma_phase ^= 1;
    TcFenceAfter();
    if (NS == 1 && tid == 0 && ld + 1 < total) issue_load(ld + 1);
  }
  failed = __syncthreads_or(failed);
  if (failed) {
    if (tid == 0) a.status->wait_timeout = 1;
  } else {
    const bool live = key < a.S;
    const size_t HD = static_cast<size_t>(a.H) * D;
    float* o = a.out + (static_cast<size_t>(b) * a.S + (live ? key : 0)) * HD + static_cast<size_t>(h) * D;
#pragma unroll 1
    for (uint32_t c0 = 0; c0 < D; c0 += 32) {
      uint32_t r[32];
      TmemLoad32(t_lane + kOutCol + c0, r);
      TmemWaitLd();
      if (live) {
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(o + c0 + j) =
              make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                          __uint_as_float(r[j + 3]));
      }
    }
  }
  TcFenceBefore();
  __syncthreads();
  if (warp == 0) {
    TcFenceAfter();
    TmemFree(tmem, kTmemCols);
  }
}

}  // namespace


size_t AttnFwdSmem(int d) { return 128 * d * 2 + 2 * (128 * d * 2 + d * 256) + kPBytes + 1024; }
size_t AttnDQSmem(int d, int ns) { return 2 * 128 * d * 2 + ns * (2 * 128 * d * 2 + d * 256) + kPBytes + 1024; }
size_t AttnDKVSmem(int d, bool dk, int ns) {
  const size_t row = 128 * d * 2, col = d * 256;
  return (dk ? 2 : 1) * row + ns * ((dk ? 2 : 1) * row + col) + kPBytes + 3 * 128 * 4 + 1024;
}

template <typename Kernel>
static cudaError_t Configure(Kernel kernel, size_t smem) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
}

void PackHeads(const float* x, uint16_t* rows, uint16_t* cols, uint32_t B, uint32_t S, uint32_t H,
               uint32_t d, cudaStream_t s) {
  const dim3 grid((S + kPackPos - 1) / kPackPos, B * H);
  if (d == 64) PackHeadsKernel<64><<<grid, 256, 0, s>>>(x, rows, cols, S, H);
  else PackHeadsKernel<128><<<grid, 256, 0, s>>>(x, rows, cols, S, H);
}

cudaError_t AttnFwdUmma(const CUtensorMap& q, const CUtensorMap& k, const CUtensorMap& vt,
                        const AttnUmmaArgs& a, cudaStream_t s) {
  dim3 grid((a.S + kTile - 1) / kTile, a.B * a.H);
  const size_t smem = AttnFwdSmem(a.d);
  cudaError_t e;
  if (a.d == 64) {
    if ((e = Configure(AttnFwdUmmaKernel<64>, smem)) != cudaSuccess) return e;
    AttnFwdUmmaKernel<64><<<grid, 128, smem, s>>>(q, k, vt, a);
  } else {
    if ((e = Configure(AttnFwdUmmaKernel<128>, smem)) != cudaSuccess) return e;
    AttnFwdUmmaKernel<128><<<grid, 128, smem, s>>>(q, k, vt, a);
  }
  return cudaGetLastError();
}

cudaError_t AttnDQUmma(const CUtensorMap& q, const CUtensorMap& dout, const CUtensorMap& k,
                       const CUtensorMap& v, const CUtensorMap& kt, const AttnUmmaArgs& a,
                       cudaStream_t s) {
  dim3 grid((a.S + kTile - 1) / kTile, a.B * a.H);
  cudaError_t e;
  if (a.d == 64) {
    const size_t smem = AttnDQSmem(64, 2);
    if ((e = Configure(AttnDQUmmaKernel<64, 2>, smem)) != cudaSuccess) return e;
    AttnDQUmmaKernel<64, 2><<<grid, 128, smem, s>>>(q, dout, k, v, kt, a);
  } else {
    const size_t smem = AttnDQSmem(128, 1);
    if ((e = Configure(AttnDQUmmaKernel<128, 1>, smem)) != cudaSuccess) return e;
    AttnDQUmmaKernel<128, 1><<<grid, 128, smem, s>>>(q, dout, k, v, kt, a);
  }
  return cudaGetLastError();
}

cudaError_t AttnDKVUmma(bool want_dk, const CUtensorMap& k, const CUtensorMap& v, const CUtensorMap& q,
                        const CUtensorMap& dout, const CUtensorMap& t, const AttnUmmaArgs& a,
                        cudaStream_t s) {
  dim3 grid((a.S + kTile - 1) / kTile, a.B * a.H);
  cudaError_t e;
#define SEE_LAUNCH_DKV(D, DK, NS)                                                      \
  do {                                                                                 \
    const size_t smem = AttnDKVSmem(D, DK, NS);                                        \
    if ((e = Configure(AttnDKVUmmaKernel<D, DK, NS>, smem)) != cudaSuccess) return e;  \
    AttnDKVUmmaKernel<D, DK, NS><<<grid, 128, smem, s>>>(k, v, q, dout, t, a);        \
  } while (0)
  if (a.d == 64) {
    if (want_dk) SEE_LAUNCH_DKV(64, true, 2); else SEE_LAUNCH_DKV(64, false, 2);
  } else {
    if (want_dk) SEE_LAUNCH_DKV(128, true, 1); else SEE_LAUNCH_DKV(128, false, 2);
  }
#undef SEE_LAUNCH_DKV
  return cudaGetLastError();
}


}  // namespace see::k
