// Causal attention on the tensor cores, for the tiled attention opcodes that
// carry the relaxed permission (reference: source/plan/instruction.h:174-190,
// 356-382; the reference's own relaxed attention is the matrix-tile family of
// runtime/executor/metal_backend.mm:1742-1802).  Same contract as the exact
// tiled family (reference: runtime/executor/attention.cc:448-590): the forward
// writes O and the stats row {score max, 1/denominator, 0, start}; dQ writes
// delta into the stats row and dQ; dK and dV read the stats row.
//
// Blackwell-native: the operands are held once as bf16 in the tensors' own
// row-major layout [B*S, H*d] (written by the kernel that produces the tensor,
// or converted once), a (sequence, head) tile arrives by one 4-D TMA load
// (128-byte swizzle), every product
// (Q K^T, P V, dO V^T, dS K, dS^T Q, P^T dO) is a tcgen05.mma with its
// accumulator in tensor memory, and the softmax / softmax-backward arithmetic
// runs in f32 registers on values read with tcgen05.ld; P and dS go back to
// shared memory as bf16 for the second product.  Statistics are exact f32
// reductions of the bf16 products: two walks over the keys (first the row
// statistics, then the products), so no accumulator is ever rescaled.
//
// A CTA is 128 threads, one query row (or key row) per thread, and takes the
// other axis 64 positions per step, which keeps its footprint at 48-72 KB of
// shared memory and 128-256 columns of tensor memory: two to four CTAs share an
// SM and fill each other's load, MMA and exp latencies.  Thread 0 issues TMA
// and MMA; one tcgen05.commit per step covers the step's first product(s) and
// the previous step's second product.  Every mbarrier wait is bounded; a wait
// that runs out raises DeviceStatus::wait_timeout and the CTA stores nothing.
#include <cuda.h>

#include "attn_umma.h"
#include "kernels.h"
#include "shadow.cuh"
#include "umma_device.cuh"

namespace see::k {

using namespace umma_dev;

namespace {

constexpr uint32_t kTile = 128;          // query rows / key rows per tile
constexpr uint32_t kSubTileBytes = 128 * 64 * 2;   // [128 rows][64 bf16], swizzled
constexpr uint32_t kPBytes = 2 * kSubTileBytes;    // P / dS tile: 128 x 128 bf16

// ---- operand copies: f32 [B*S, H*d] -> bf16, same layout --------------------------------
// (Every operand tile of the kernels below is cut out of this copy by a 4-D tensor map
// {d, S, H, B}: 64 head-dimension elements x R positions of one head of one sequence land
// as [R][128 bytes] — the K-major tile of a product over the head dimension, and through an
// MN-major descriptor the operand of a product over the positions.)
__device__ __forceinline__ uint32_t Bf16Bits(float f) {   // round to nearest even; NaN stays NaN
  uint32_t u = __float_as_uint(f);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (u >> 16) | 0x0040u;
  u += 0x7FFFu + ((u >> 16) & 1u);
  return u >> 16;
}

__global__ void __launch_bounds__(256)
PackRowsKernel(const float* __restrict__ x, uint16_t* __restrict__ rows, size_t quads) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t q = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; q < quads; q += stride) {
    const float4 f = reinterpret_cast<const float4*>(x)[q];
    reinterpret_cast<uint2*>(rows)[q] =
        make_uint2(Bf16Bits(f.x) | (Bf16Bits(f.y) << 16), Bf16Bits(f.z) | (Bf16Bits(f.w) << 16));
  }
}

struct Ctl {
  uint64_t bar_a;   // operands of the step's first product(s) have landed
  uint64_t bar_b;   // operand of the step's second product has landed
  uint64_t mma;     // the tensor core finished everything issued so far
  uint32_t tmem_base;
  uint32_t pad;
};

constexpr uint32_t kHalf = 64;                    // keys (or queries) per step
constexpr uint32_t kHalfTileBytes = 128 * 64 * 2; // P / dS step tile: [128 rows][64] bf16, swizzled
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float Exp2Approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Loads [R positions][D] of head h of sequence b ({d, S, H, B} map with box {64, R, 1, 1}) as
// D/64 sub-tiles of R * 128 bytes; positions past the end of the sequence arrive as zeros.
template <int D, int R>
__device__ __forceinline__ void LoadRows(uint8_t* dst, const CUtensorMap* map, uint64_t* bar,
                                         uint32_t row0, uint32_t h, uint32_t b) {
#pragma unroll
  for (int kb = 0; kb < D / 64; ++kb)
    TmaLoad4D(dst + kb * (R * 128), map, bar, kb * 64, static_cast<int32_t>(row0), static_cast<int32_t>(h),
              static_cast<int32_t>(b));
}
// acc[128 x NB] = A[128 rows][D] . B[NB rows][D]^T, both row tiles in shared memory.
template <int D, int NB>
__device__ __forceinline__ void MmaRowRow(uint32_t tmem, const uint8_t* a, const uint8_t* b) {
  const uint32_t idesc = MakeInstrDesc(128, NB);
#pragma unroll
  for (int kb = 0; kb < D / 64; ++kb) {
    const uint64_t da = MakeSmemDesc(SmemAddr(a + kb * (128 * 128)));
    const uint64_t db = MakeSmemDesc(SmemAddr(b + kb * (NB * 128)));
#pragma unroll
    for (int k = 0; k < 4; ++k) UmmaBf16(tmem, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
  }
}
// acc[128 x D] (+)= P[128 rows][64] . T with T given as a ROW tile [64 positions][D]
// (the positions are the reduction index: an MN-major B operand), D / 64 sub-tiles of
// [64][64] as LoadRows<D, 64> leaves them.
template <int D>
__device__ __forceinline__ void MmaPRows(uint32_t tmem, const uint8_t* p, const uint8_t* t_rows,
                                         uint32_t accumulate) {
  const uint32_t idesc = MakeInstrDesc(128, D) | kInstrDescBMnMajor;
  const uint64_t da = MakeSmemDesc(SmemAddr(p));
  const uint32_t tb = SmemAddr(t_rows);
#pragma unroll
  for (int k = 0; k < 4; ++k)
    UmmaBf16(tmem, da + 2 * k, MakeSmemDescMn(tb + k * 2048, 64 * 128), idesc, (accumulate | k) != 0 ? 1u : 0u);
}

// Writes 32 consecutive values of this thread's row (columns c0 .. c0+31 of the 64-wide
// step tile) into the swizzled bf16 tile.
__device__ __forceinline__ void StoreRowChunk(uint8_t* p_tile, uint32_t row, uint32_t c0,
                                              const float (&v)[32]) {
  const uint32_t chunk0 = c0 >> 3;   // first 16-byte chunk (8 bf16) of the four
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint4 w;
    w.x = PackBf16x2(v[8 * q + 0], v[8 * q + 1]);
    w.y = PackBf16x2(v[8 * q + 2], v[8 * q + 3]);
    w.z = PackBf16x2(v[8 * q + 4], v[8 * q + 5]);
    w.w = PackBf16x2(v[8 * q + 6], v[8 * q + 7]);
    *reinterpret_cast<uint4*>(p_tile + Sw128Offset(row, chunk0 + q)) = w;
  }
}

__device__ __forceinline__ uint8_t* AlignSmem(uint8_t* raw) {
  return raw + ((1024u - (SmemAddr(raw) & 1023u)) & 1023u);
}

// Stores a warp's 32 output rows (D accumulator columns starting at t_out, one row per
// thread, times the thread's `scale`).  The rows turn through a per-warp slab of shared
// memory (the operand tiles are idle by now) so that HBM sees whole rows: 16-byte chunks
// XOR-swizzled with the row, conflict-free both for the row-per-thread writes and the
// row-per-(half-)warp reads.  `out0` points at (first row, this head's first column) of
// the [B*S, H*d] tensor, `flat0` is that element's index (for the bf16 shadow), `col0`
// its column, `rows_live` how many of the 32 rows exist.
template <int D>
__device__ __forceinline__ void StoreOutRows(uint32_t t_out, float* slab, uint32_t lane, float scale,
                                             float* out0, size_t pitch, uint32_t rows_live,
                                             const Shadow& sh, size_t flat0, uint32_t col0,
                                             float* keep = nullptr) {
  constexpr uint32_t kChunks = D / 4;          // 16-byte chunks per row: 16 or 32
  constexpr uint32_t kRowsPerPass = 32 / kChunks;
#pragma unroll 1
  for (uint32_t c0 = 0; c0 < D; c0 += 32) {
    uint32_t r[32];
    TmemLoad32(t_out + c0, r);
    TmemWaitLd();
#pragma unroll
    for (uint32_t q = 0; q < 8; ++q) {
      const uint32_t chunk = ((c0 >> 2) + q) ^ (lane & (kChunks - 1));
      *reinterpret_cast<float4*>(slab + lane * D + chunk * 4) =
          make_float4(__uint_as_float(r[4 * q]) * scale, __uint_as_float(r[4 * q + 1]) * scale,
                      __uint_as_float(r[4 * q + 2]) * scale, __uint_as_float(r[4 * q + 3]) * scale);
    }
  }
  __syncwarp();
  const uint32_t sub = lane / kChunks, cl = lane % kChunks;
#pragma unroll 4
  for (uint32_t rr = sub; rr < rows_live; rr += kRowsPerPass) {
    const float4 v = *reinterpret_cast<const float4*>(slab + rr * D + ((cl ^ (rr & (kChunks - 1))) * 4));
    *reinterpret_cast<float4*>(out0 + rr * pitch + cl * 4) = v;
    if (sh.dst) ShadowStore4(sh, (flat0 + rr * pitch + cl * 4) / 4, col0 + cl * 4, v);
    if (keep) *reinterpret_cast<float4*>(keep + flat0 + rr * pitch + cl * 4) = v;
  }
}

// After a wait ran out: give copies that may still be in flight towards this CTA's
// shared memory a bounded time to land before the CTA retires.
__device__ __forceinline__ void DrainDelay() {
  for (int i = 0; i < 64; ++i) __nanosleep(2000);
}

constexpr uint32_t TmemColsFor(uint32_t need) { return need <= 128 ? 128 : (need <= 256 ? 256 : 512); }

// ---- forward -------------------------------------------------------------------------
// A CTA owns 128 query rows of one (sequence, head) and walks the keys ONCE, 64 at
// a time.  Per step: S = Q K_h^T (128 x 64, tensor memory columns 0..63), read back
// one row per thread; p = 2^(s c - ref) against a per-row reference exponent, P
// written to shared memory as bf16, O += P V_h (columns 64..64+D) unnormalised.
// The reference follows the running maximum lazily: it moves (and the row's O
// and sum are multiplied by 2^(old - new), a read-modify-write of the row's
// tensor-memory lane) only when a step's maximum exceeds it by more than 2^8, so
// p stays below 256 — exact in f32 sums, the same relative rounding in bf16 —
// and most steps rescale nothing.  The true maximum is tracked beside it and the
// stats row gets {max, 1 / sum relative to that max}, what the backward kernels
// and the exact family expect.  Small footprint on purpose (48 KB of shared
// memory and 128 tensor-memory columns for d = 64): four CTAs share an SM and
// cover each other's waits.
constexpr float kRescaleSlack = 8.0f;   // log2 units

template <int D>
__global__ void __launch_bounds__(128)
AttnFwdUmmaKernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                  const __grid_constant__ CUtensorMap map_v, AttnUmmaArgs a) {
  extern __shared__ uint8_t smem_raw[];
  Ctl* ctl = reinterpret_cast<Ctl*>(smem_raw);             // barriers first, tiles 1024-aligned after
  uint8_t* smem = AlignSmem(smem_raw + sizeof(Ctl));
  constexpr uint32_t kQBytes = 128 * D * 2, kKBytes = 64 * D * 2, kVBytes = D * 128;
  uint8_t* q_s = smem;
  uint8_t* k_s = q_s + kQBytes;
  uint8_t* v_s = k_s + kKBytes;
  uint8_t* p_s = v_s + kVBytes;
  constexpr uint32_t kTmemCols = TmemColsFor(64 + D);

  const uint32_t tid = threadIdx.x, warp = tid >> 5;
  const uint32_t n_qt = (a.S + kTile - 1) / kTile;
  const uint32_t it = n_qt - 1 - blockIdx.x;               // heaviest tiles first
  const uint32_t bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  const uint32_t all_h = (a.S + kHalf - 1) / kHalf;
  const uint32_t total = 2 * (it + 1) < all_h ? 2 * (it + 1) : all_h;   // key steps up to the diagonal

  if (tid == 0) {
    MbarInit(&ctl->bar_a, 1); MbarInit(&ctl->bar_b, 1); MbarInit(&ctl->mma, 1);
    MbarInitFence();
  }
  if (warp == 0) TmemAlloc(&ctl->tmem_base, kTmemCols);
  TcFenceBefore();
  __syncthreads();
  TcFenceAfter();
  const uint32_t tmem = ctl->tmem_base;
  const uint32_t t_s = tmem + ((warp * 32) << 16);
  const uint32_t t_o = t_s + 64;

  auto issue_a = [&](uint32_t t) {
    MbarExpectTx(&ctl->bar_a, kKBytes + (t == 0 ? kQBytes : 0));
    if (t == 0) LoadRows<D, 128>(q_s, &map_q, &ctl->bar_a, it * kTile, h, b);
    LoadRows<D, 64>(k_s, &map_k, &ctl->bar_a, t * kHalf, h, b);
  };
  auto issue_b = [&](uint32_t t) {
    MbarExpectTx(&ctl->bar_b, kVBytes);
    LoadRows<D, 64>(v_s, &map_v, &ctl->bar_b, t * kHalf, h, b);   // V_h as rows: the MN-major operand of P V
  };

  const uint32_t row = it * kTile + tid;                   // this thread's query row
  const float c1 = a.inv_sqrt_d * kLog2e;
  float raw_max = -INFINITY;   // the row's true score maximum so far
  float ref = -INFINITY;       // the exponent (log2 units) its p, sum and O are relative to
  float l = 0.0f;
  int failed = 0;
  if (tid == 0) issue_a(0);

  for (uint32_t t = 0; t < total; ++t) {
    if (tid == 0) {   // only the issuing thread needs the operands' arrival
      if (!MbarWait(&ctl->bar_a, t & 1)) failed = 1;
      TcFenceAfter();
      if (!failed) MmaRowRow<D, 64>(tmem, q_s, k_s);
      UmmaCommit(&ctl->mma);
    }
    // This commit also covers the previous step's O += P V, so p_s, v_s and k_s
    // are all free again once it arrives, and O is at rest.
    if (!MbarWait(&ctl->mma, t & 1)) failed = 1;
    TcFenceAfter();
    if (tid == 0 && !failed) {
      if (t + 1 < total) issue_a(t + 1);
      issue_b(t);
    }
    const uint32_t key0 = t * kHalf;
    const bool diagonal = key0 + kHalf > it * kTile;   // some keys of this step lie above the diagonal
    uint32_t r[64];
    {
      uint32_t lo[32], hi[32];
      TmemLoad32(t_s, lo);
      TmemLoad32(t_s + 32, hi);
      TmemWaitLd();
#pragma unroll
      for (int j = 0; j < 32; ++j) { r[j] = lo[j]; r[32 + j] = hi[j]; }
    }
    float step_max = -INFINITY;
    if (diagonal) {
#pragma unroll
      for (int j = 0; j < 64; ++j)
        if (key0 + j <= row) step_max = fmaxf(step_max, __uint_as_float(r[j]));
    } else {
#pragma unroll
      for (int j = 0; j < 64; ++j) step_max = fmaxf(step_max, __uint_as_float(r[j]));
    }
    raw_max = fmaxf(raw_max, step_max);
    const float step_ref = step_max * c1;
    const bool moves = step_ref > ref + kRescaleSlack;   // always at a row's first live key (ref = -inf)
    float alpha = 1.0f;
    if (moves) {
      alpha = Exp2Approx(ref - step_ref);                // 0 the first time
      l *= alpha;
      ref = step_ref;
    }
    if (t > 0 && __any_sync(0xFFFFFFFFu, moves)) {       // the warp's rows rescale their O lanes together
#pragma unroll 1
      for (uint32_t c0 = 0; c0 < D; c0 += 32) {
        uint32_t o[32];
        TmemLoad32(t_o + c0, o);
        TmemWaitLd();
#pragma unroll
        for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
        TmemStore32(t_o + c0, o);
      }
      TmemWaitSt();
    }
#pragma unroll
    for (uint32_t c0 = 0; c0 < kHalf; c0 += 32) {
      float v[32];
      if (diagonal) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          v[j] = (key0 + c0 + j <= row) ? Exp2Approx(fmaf(__uint_as_float(r[c0 + j]), c1, -ref)) : 0.0f;
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = Exp2Approx(fmaf(__uint_as_float(r[c0 + j]), c1, -ref));
      }
#pragma unroll
      for (int j = 0; j < 32; ++j) l += v[j];
      StoreRowChunk(p_s, tid, c0, v);
    }
    FenceProxyAsync();
    TcFenceBefore();
    if (__syncthreads_or(failed)) { failed = 1; break; }
    if (tid == 0) {
      if (!MbarWait(&ctl->bar_b, t & 1)) failed = 1;
      TcFenceAfter();
      if (!failed) MmaPRows<D>(tmem + 64, p_s, v_s, t != 0);
    }
  }
  if (tid == 0) UmmaCommit(&ctl->mma);
  if (!failed && !MbarWait(&ctl->mma, total & 1)) failed = 1;
  TcFenceAfter();
  failed = __syncthreads_or(failed);
  if (failed) {
    if (tid == 0) a.status->wait_timeout = 1;
    DrainDelay();
  } else {
    const bool live = row < a.S;
    const size_t HD = static_cast<size_t>(a.H) * D;
    const uint32_t row0w = it * kTile + warp * 32;
    const uint32_t rows_live = row0w < a.S ? (a.S - row0w < 32 ? a.S - row0w : 32) : 0;
    const size_t flat0 = (static_cast<size_t>(b) * a.S + row0w) * HD + static_cast<size_t>(h) * D;
    const float inv_l = 1.0f / l;
    StoreOutRows<D>(t_o, reinterpret_cast<float*>(smem) + warp * 32 * D, tid & 31, inv_l,
                    a.out + flat0, HD, rows_live, a.shadow, flat0, h * D, a.keep);
    if (live) {
      // The stats row speaks of the true maximum: the sum relative to it is l 2^(ref - max c).
      const float m = raw_max * a.inv_sqrt_d;
      const float inv_l_at_max = 1.0f / (l * Exp2Approx(ref - raw_max * c1));
      float* st = a.stats + (static_cast<size_t>(bh) * a.S + row) * kAttnStatsWidth;
      *reinterpret_cast<float4*>(st) = make_float4(m, inv_l_at_max, 0.0f, 0.0f);
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
// Per 128 query rows, the keys 64 at a time.  Per step S = Q K_h^T (columns
// 0..63) and dP = dO V_h^T (64..127); dS = P (dP - delta) / sqrt(d) goes to shared
// memory as bf16 and dQ += dS K (columns 128..128+D).  delta_i = sum_j P_ij dP_ij:
// with the forward's kept copy of O at hand it is dO_i . O_i, one row of each read
// by the row's thread before the walk; without it a first walk over the keys sums it.
template <int D>
__global__ void __launch_bounds__(128)
AttnDQUmmaKernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                 const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                 AttnUmmaArgs a) {
  extern __shared__ uint8_t smem_raw[];
  Ctl* ctl = reinterpret_cast<Ctl*>(smem_raw);
  uint8_t* smem = AlignSmem(smem_raw + sizeof(Ctl));
  constexpr uint32_t kFull = 128 * D * 2, kHalfRows = 64 * D * 2;
  uint8_t* q_s = smem;
  uint8_t* do_s = q_s + kFull;
  uint8_t* k_s = do_s + kFull;          // two buffers: step t's K_h also feeds dQ += dS K_h after the softmax,
  uint8_t* v_s = k_s + 2 * kHalfRows;   // while step t + 1's is already on its way
  uint8_t* p_s = v_s + kHalfRows;
  constexpr uint32_t kTmemCols = TmemColsFor(128 + D);

  const uint32_t tid = threadIdx.x, warp = tid >> 5;
  const uint32_t n_qt = (a.S + kTile - 1) / kTile;
  const uint32_t it = n_qt - 1 - blockIdx.x;
  const uint32_t bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  const uint32_t all_h = (a.S + kHalf - 1) / kHalf;
  const uint32_t n_h = 2 * (it + 1) < all_h ? 2 * (it + 1) : all_h;
  const bool one_walk = a.fwd_keep != nullptr;
  const uint32_t total = one_walk ? n_h : 2 * n_h;

  if (tid == 0) {
    MbarInit(&ctl->bar_a, 1); MbarInit(&ctl->bar_b, 1); MbarInit(&ctl->mma, 1);
    MbarInitFence();
  }
  if (warp == 0) TmemAlloc(&ctl->tmem_base, kTmemCols);
  TcFenceBefore();
  __syncthreads();
  TcFenceAfter();
  const uint32_t tmem = ctl->tmem_base;
  const uint32_t t_lane = tmem + ((warp * 32) << 16);

  auto issue_a = [&](uint32_t t) {
    MbarExpectTx(&ctl->bar_a, 2 * kHalfRows + (t == 0 ? 2 * kFull : 0));
    if (t == 0) {
      LoadRows<D, 128>(q_s, &map_q, &ctl->bar_a, it * kTile, h, b);
      LoadRows<D, 128>(do_s, &map_do, &ctl->bar_a, it * kTile, h, b);
    }
    LoadRows<D, 64>(k_s + (t & 1) * kHalfRows, &map_k, &ctl->bar_a, (t % n_h) * kHalf, h, b);
    LoadRows<D, 64>(v_s, &map_v, &ctl->bar_a, (t % n_h) * kHalf, h, b);
  };

  const uint32_t row = it * kTile + tid;
  const bool live = row < a.S;
  float* st_row = a.stats + (static_cast<size_t>(bh) * a.S + (live ? row : 0)) * kAttnStatsWidth;
  const float c1 = a.inv_sqrt_d * kLog2e;
  // P = 2^(s * log2(e)/sqrt(d) - M) with M = max * log2(e) - log2(1/denominator).
  const float m2l = live ? st_row[0] * kLog2e - log2f(st_row[1]) : 0.0f;
  float delta = 0.0f;
  int failed = 0;
  if (tid == 0) issue_a(0);
  if (one_walk && live) {   // (under the first loads' flight)
    const size_t at = (static_cast<size_t>(b) * a.S + row) * (static_cast<size_t>(a.H) * D) + static_cast<size_t>(h) * D;
    const float4* orow = reinterpret_cast<const float4*>(a.fwd_keep + at);
    const uint2* drow = reinterpret_cast<const uint2*>(a.dout_bf16 + at);   // four bf16 per load
#pragma unroll 4
    for (int c = 0; c < D / 4; ++c) {
      const float4 o = orow[c];
      const uint2 g = drow[c];
      delta = fmaf(o.x, __uint_as_float(g.x << 16), delta);
      delta = fmaf(o.y, __uint_as_float(g.x & 0xFFFF0000u), delta);
      delta = fmaf(o.z, __uint_as_float(g.y << 16), delta);
      delta = fmaf(o.w, __uint_as_float(g.y & 0xFFFF0000u), delta);
    }
  }

  for (uint32_t t = 0; t < total; ++t) {
    const uint32_t jh = t % n_h;
    const bool second = one_walk || t >= n_h;
    if (tid == 0) {
      if (!MbarWait(&ctl->bar_a, t & 1)) failed = 1;
      TcFenceAfter();
      if (!failed) {
        MmaRowRow<D, 64>(tmem, q_s, k_s + (t & 1) * kHalfRows);   // S  = Q K_h^T
        MmaRowRow<D, 64>(tmem + 64, do_s, v_s);    // dP = dO V_h^T
      }
      UmmaCommit(&ctl->mma);   // also covers the previous step's dQ += dS K_h
    }
    if (!MbarWait(&ctl->mma, t & 1)) failed = 1;
    TcFenceAfter();
    if (tid == 0 && !failed && t + 1 < total) issue_a(t + 1);
    __syncwarp();
    const uint32_t key0 = jh * kHalf;
    const bool diagonal = key0 + kHalf > it * kTile;
#pragma unroll 1
    for (uint32_t c0 = 0; c0 < kHalf; c0 += 32) {
      uint32_t rs[32], rp[32];
      TmemLoad32(t_lane + c0, rs);
      TmemLoad32(t_lane + 64 + c0, rp);
      TmemWaitLd();
      float pr[32];   // P = exp(s - max) / denominator, zero above the diagonal
      if (diagonal) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          pr[j] = (key0 + c0 + j <= row) ? Exp2Approx(fmaf(__uint_as_float(rs[j]), c1, -m2l)) : 0.0f;
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) pr[j] = Exp2Approx(fmaf(__uint_as_float(rs[j]), c1, -m2l));
      }
      if (!second) {
#pragma unroll
        for (int j = 0; j < 32; ++j) delta = fmaf(pr[j], __uint_as_float(rp[j]), delta);
      } else {
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = pr[j] * (__uint_as_float(rp[j]) - delta) * a.inv_sqrt_d;
        StoreRowChunk(p_s, tid, c0, v);
      }
    }
    if (second) FenceProxyAsync();
    TcFenceBefore();
    if (__syncthreads_or(failed)) { failed = 1; break; }
    if (second && tid == 0) {
      TcFenceAfter();
      MmaPRows<D>(tmem + 128, p_s, k_s + (t & 1) * kHalfRows, jh != 0);   // dQ += dS K_h (K_h as the MN-major operand)
    }
  }
  if (tid == 0) UmmaCommit(&ctl->mma);
  if (!failed && !MbarWait(&ctl->mma, total & 1)) failed = 1;
  TcFenceAfter();
  failed = __syncthreads_or(failed);
  if (failed) {
    if (tid == 0) a.status->wait_timeout = 1;
    DrainDelay();
  } else {
    const size_t HD = static_cast<size_t>(a.H) * D;
    const uint32_t row0w = it * kTile + warp * 32;
    const uint32_t rows_live = row0w < a.S ? (a.S - row0w < 32 ? a.S - row0w : 32) : 0;
    const size_t flat0 = (static_cast<size_t>(b) * a.S + row0w) * HD + static_cast<size_t>(h) * D;
    StoreOutRows<D>(t_lane + 128, reinterpret_cast<float*>(smem) + warp * 32 * D, tid & 31, 1.0f,
                    a.out + flat0, HD, rows_live, a.shadow, flat0, h * D);
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
// Per 128 key rows, over the queries at or below the diagonal 64 at a time, in
// the transposed frame (one key row per thread, query index along the columns):
// S^T = K Q_h^T; P^T from the stats rows of those queries, folded into one
// number per query, M = max * log2(e) - log2(1/denominator), so that
// P^T = 2^(s * log2(e)/sqrt(d) - M).  dV += P^T dO_h, or
// dS^T = P^T (dP^T - delta) / sqrt(d) with dP^T = V dO_h^T and dK += dS^T Q_h.
// kMode 0: dV alone; 1: dK alone; 2: both in one walk (the plan's kAttnDKTiled /
// kAttnDVTiled pair on the same operands): S^T and P^T are formed once, dV's
// product rides the step's second commit, and the second kernel's passes over K,
// Q and the statistics disappear.  Tensor memory: S^T, dP^T, dK, dV = 4 x 64 columns
// at d = 64 (the 256 the dK form occupies anyway).
template <int D, int kMode>
__global__ void __launch_bounds__(128)
AttnDKVUmmaKernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                  const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                  AttnUmmaArgs a) {
  constexpr bool kWantDK = kMode >= 1;
  constexpr bool kBoth = kMode == 2;
  extern __shared__ uint8_t smem_raw[];
  Ctl* ctl = reinterpret_cast<Ctl*>(smem_raw);
  uint8_t* smem = AlignSmem(smem_raw + sizeof(Ctl));
  constexpr uint32_t kFull = 128 * D * 2, kHalfRows = 64 * D * 2;
  uint8_t* k_s = smem;
  uint8_t* v_s = k_s + kFull;                                // dK only
  // Q_h and dO_h are double-buffered: a step's tiles also feed its second products
  // (as MN-major operands) after the softmax, while the next step's are on their way.
  uint8_t* q_s = v_s + (kWantDK ? kFull : 0);
  uint8_t* do_s = q_s + 2 * kHalfRows;
  uint8_t* p_s = do_s + 2 * kHalfRows;
  uint8_t* p2_s = p_s + kHalfTileBytes;                      // both: P^T beside dS^T
  float* stat_s = reinterpret_cast<float*>(p2_s + (kBoth ? kHalfTileBytes : 0));   // M[64], delta[64]
  constexpr uint32_t kOutCol = kWantDK ? 128 : 64;
  constexpr uint32_t kOutCol2 = kOutCol + D;                 // both: dV after dK
  constexpr uint32_t kTmemCols = TmemColsFor(kOutCol + (kBoth ? 2 : 1) * D);

  const uint32_t tid = threadIdx.x, warp = tid >> 5;
  const uint32_t jt = blockIdx.x;                          // key tile; low tiles have the most work
  const uint32_t bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  const uint32_t all_h = (a.S + kHalf - 1) / kHalf;
  const uint32_t h0 = 2 * jt;                              // first query step: the diagonal
  const uint32_t total = all_h - h0;

  if (tid == 0) {
    MbarInit(&ctl->bar_a, 1); MbarInit(&ctl->bar_b, 1); MbarInit(&ctl->mma, 1);
    MbarInitFence();
  }
  if (warp == 0) TmemAlloc(&ctl->tmem_base, kTmemCols);
  TcFenceBefore();
  __syncthreads();
  TcFenceAfter();
  const uint32_t tmem = ctl->tmem_base;
  const uint32_t t_lane = tmem + ((warp * 32) << 16);

  auto issue_a = [&](uint32_t t) {
    constexpr uint32_t kPer = 2 * kHalfRows, kOnce = (kWantDK ? 2 : 1) * kFull;
    MbarExpectTx(&ctl->bar_a, kPer + (t == 0 ? kOnce : 0));
    if (t == 0) {
      LoadRows<D, 128>(k_s, &map_k, &ctl->bar_a, jt * kTile, h, b);
      if (kWantDK) LoadRows<D, 128>(v_s, &map_v, &ctl->bar_a, jt * kTile, h, b);
    }
    LoadRows<D, 64>(q_s + (t & 1) * kHalfRows, &map_q, &ctl->bar_a, (h0 + t) * kHalf, h, b);
    LoadRows<D, 64>(do_s + (t & 1) * kHalfRows, &map_do, &ctl->bar_a, (h0 + t) * kHalf, h, b);
  };

  const uint32_t key = jt * kTile + tid;                    // this thread's key row
  const float c1 = a.inv_sqrt_d * kLog2e;
  int failed = 0;
  if (tid == 0) issue_a(0);

  for (uint32_t t = 0; t < total; ++t) {
    const uint32_t q0 = (h0 + t) * kHalf;
    if (tid < kHalf) {   // this step's queries (the previous step's readers passed a barrier)
      const uint32_t qi = q0 + tid;
      float M = INFINITY, dl = 0.0f;   // past the end of the sequence: P = 2^-inf = 0
      if (qi < a.S) {
        const float4 sv = *reinterpret_cast<const float4*>(
            a.stats + (static_cast<size_t>(bh) * a.S + qi) * kAttnStatsWidth);
        M = sv.x * kLog2e - log2f(sv.y);
        dl = sv.z;
      }
      stat_s[tid] = M;
      stat_s[kHalf + tid] = dl;
    }
    if (tid == 0) {
      if (!MbarWait(&ctl->bar_a, t & 1)) failed = 1;
      TcFenceAfter();
      if (!failed) {
        MmaRowRow<D, 64>(tmem, k_s, q_s + (t & 1) * kHalfRows);                          // S^T  = K Q_h^T
        if (kWantDK) MmaRowRow<D, 64>(tmem + 64, v_s, do_s + (t & 1) * kHalfRows);       // dP^T = V dO_h^T
      }
      UmmaCommit(&ctl->mma);   // also covers the previous step's second product
    }
    __syncthreads();           // stat_s is written
    if (!MbarWait(&ctl->mma, t & 1)) failed = 1;
    TcFenceAfter();
    if (tid == 0 && !failed && t + 1 < total) issue_a(t + 1);
    __syncwarp();
    const bool diagonal = q0 < jt * kTile + kTile;   // some (key, query) pairs are masked
#pragma unroll 1
    for (uint32_t c0 = 0; c0 < kHalf; c0 += 32) {
      uint32_t rs[32], rp[32];
      TmemLoad32(t_lane + c0, rs);
      if (kWantDK) TmemLoad32(t_lane + 64 + c0, rp);
      TmemWaitLd();
      float v[32];
      [[maybe_unused]] float pv[kBoth ? 32 : 1];
#pragma unroll
      for (int j4 = 0; j4 < 32; j4 += 4) {
        const float4 M4 = *reinterpret_cast<const float4*>(&stat_s[c0 + j4]);
        const float Mv[4] = {M4.x, M4.y, M4.z, M4.w};
        float dv[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (kWantDK) {
          const float4 d4 = *reinterpret_cast<const float4*>(&stat_s[kHalf + c0 + j4]);
          dv[0] = d4.x; dv[1] = d4.y; dv[2] = d4.z; dv[3] = d4.w;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int j = j4 + u;
          float p = Exp2Approx(fmaf(__uint_as_float(rs[j]), c1, -Mv[u]));
          if (diagonal && key > q0 + c0 + j) p = 0.0f;
          v[j] = kWantDK ? p * (__uint_as_float(rp[j]) - dv[u]) * a.inv_sqrt_d : p;
          if (kBoth) pv[kBoth ? j : 0] = p;
        }
      }
      StoreRowChunk(p_s, tid, c0, v);
      if constexpr (kBoth) StoreRowChunk(p2_s, tid, c0, pv);
    }
    FenceProxyAsync();
    TcFenceBefore();
    if (__syncthreads_or(failed)) { failed = 1; break; }
    if (tid == 0) {   // the step's own Q_h / dO_h tiles again, now as the MN-major operands
      TcFenceAfter();
      const uint8_t* qh = q_s + (t & 1) * kHalfRows;
      const uint8_t* doh = do_s + (t & 1) * kHalfRows;
      MmaPRows<D>(tmem + kOutCol, p_s, kWantDK ? qh : doh, t != 0);   // dK += dS^T Q_h, or dV += P^T dO_h
      if (kBoth) MmaPRows<D>(tmem + kOutCol2, p2_s, doh, t != 0);     // dV += P^T dO_h
    }
  }
  if (tid == 0) UmmaCommit(&ctl->mma);
  if (!failed && !MbarWait(&ctl->mma, total & 1)) failed = 1;
  TcFenceAfter();
  failed = __syncthreads_or(failed);
  if (failed) {
    if (tid == 0) a.status->wait_timeout = 1;
    DrainDelay();
  } else {
    const size_t HD = static_cast<size_t>(a.H) * D;
    const uint32_t row0w = jt * kTile + warp * 32;
    const uint32_t rows_live = row0w < a.S ? (a.S - row0w < 32 ? a.S - row0w : 32) : 0;
    const size_t flat0 = (static_cast<size_t>(b) * a.S + row0w) * HD + static_cast<size_t>(h) * D;
    StoreOutRows<D>(t_lane + kOutCol, reinterpret_cast<float*>(smem) + warp * 32 * D, tid & 31, 1.0f,
                    a.out + flat0, HD, rows_live, a.shadow, flat0, h * D);
    if constexpr (kBoth) {
      __syncwarp();   // the warp's staging slab is reused
      StoreOutRows<D>(t_lane + kOutCol2, reinterpret_cast<float*>(smem) + warp * 32 * D, tid & 31, 1.0f,
                      a.out2 + flat0, HD, rows_live, a.shadow2, flat0, h * D);
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

size_t AttnFwdSmem(int d) { return 128 * d * 2 + 64 * d * 2 + d * 128 + kHalfTileBytes + 1152; }
size_t AttnDQSmem(int d) { return 2 * 128 * d * 2 + 3 * 64 * d * 2 + kHalfTileBytes + 1152; }
size_t AttnDKVSmem(int d, int mode) {   // 0: dV, 1: dK, 2: both
  const size_t full = 128 * d * 2, half = 64 * d * 2;
  return (mode >= 1 ? 2 : 1) * full + 4 * half + (mode == 2 ? 2 : 1) * kHalfTileBytes + 2 * kHalf * 4 + 1152;
}

template <typename Kernel>
static cudaError_t Configure(Kernel kernel, size_t smem) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
}

void PackHeads(const float* x, uint16_t* rows, uint32_t B, uint32_t S, uint32_t H, uint32_t d, cudaStream_t s) {
  const size_t quads = static_cast<size_t>(B) * S * H * d / 4;
  const size_t blocks = (quads + 255) / 256;
  PackRowsKernel<<<static_cast<unsigned>(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0, s>>>(x, rows, quads);
}

cudaError_t AttnFwdUmma(const CUtensorMap& q, const CUtensorMap& k_half, const CUtensorMap& v_half,
                        const AttnUmmaArgs& a, cudaStream_t s) {
  dim3 grid((a.S + kTile - 1) / kTile, a.B * a.H);
  const size_t smem = AttnFwdSmem(a.d);
  cudaError_t e;
  if (a.d == 64) {
    if ((e = Configure(AttnFwdUmmaKernel<64>, smem)) != cudaSuccess) return e;
    AttnFwdUmmaKernel<64><<<grid, 128, smem, s>>>(q, k_half, v_half, a);
  } else {
    if ((e = Configure(AttnFwdUmmaKernel<128>, smem)) != cudaSuccess) return e;
    AttnFwdUmmaKernel<128><<<grid, 128, smem, s>>>(q, k_half, v_half, a);
  }
  return cudaGetLastError();
}

cudaError_t AttnDQUmma(const CUtensorMap& q, const CUtensorMap& dout, const CUtensorMap& k_half,
                       const CUtensorMap& v_half, const AttnUmmaArgs& a, cudaStream_t s) {
  dim3 grid((a.S + kTile - 1) / kTile, a.B * a.H);
  const size_t smem = AttnDQSmem(a.d);
  cudaError_t e;
  if (a.d == 64) {
    if ((e = Configure(AttnDQUmmaKernel<64>, smem)) != cudaSuccess) return e;
    AttnDQUmmaKernel<64><<<grid, 128, smem, s>>>(q, dout, k_half, v_half, a);
  } else {
    if ((e = Configure(AttnDQUmmaKernel<128>, smem)) != cudaSuccess) return e;
    AttnDQUmmaKernel<128><<<grid, 128, smem, s>>>(q, dout, k_half, v_half, a);
  }
  return cudaGetLastError();
}

cudaError_t AttnDKVUmma(int mode, const CUtensorMap& k, const CUtensorMap& v,
                        const CUtensorMap& q_half, const CUtensorMap& dout_half, const AttnUmmaArgs& a,
                        cudaStream_t s) {
  dim3 grid((a.S + kTile - 1) / kTile, a.B * a.H);
  cudaError_t e;
#define SEE_LAUNCH_DKV(D, MODE)                                                              \
  do {                                                                                       \
    const size_t smem = AttnDKVSmem(D, MODE);                                                \
    if ((e = Configure(AttnDKVUmmaKernel<D, MODE>, smem)) != cudaSuccess) return e;          \
    AttnDKVUmmaKernel<D, MODE><<<grid, 128, smem, s>>>(k, v, q_half, dout_half, a);   \
  } while (0)
  if (a.d == 64) {
    if (mode == 2) SEE_LAUNCH_DKV(64, 2); else if (mode == 1) SEE_LAUNCH_DKV(64, 1); else SEE_LAUNCH_DKV(64, 0);
  } else {   // d = 128: both accumulators would need 384 columns beside S^T and dP^T; not offered
    if (mode == 2) return cudaErrorInvalidValue;
    if (mode == 1) SEE_LAUNCH_DKV(128, 1); else SEE_LAUNCH_DKV(128, 0);
  }
#undef SEE_LAUNCH_DKV
  return cudaGetLastError();
}

}  // namespace see::k
