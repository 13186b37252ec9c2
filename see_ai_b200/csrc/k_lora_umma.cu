// An adapter site's three backward products on the tcgen05 tensor cores:
//   dT = a dY B^T   [M, 16]        dB = t^T dY   [16, N]        dA = x^T dT   [K, 16]
// (k_lora_mma.cu does the same on the legacy tensor instruction, where it is bound by
// that instruction's issue rate: 72 us at 32768 x 768, 61 us here.)
//
// The f32 operands are cut into bf16 pieces (lora_split.cuh): the small ones (B, t, dT) into
// three, v = p0 + p1 + p2 to 2^-24 |v|; the streamed ones (dY, x) into the first two, 16
// bits of mantissa, v = p0 + p1 to 2^-17 |v| with a rounding error of either sign.  A
// streamed piece meets the small operand's three pieces in ONE instruction: the small pieces
// sit side by side along N (48 columns), so the three 16-column groups of an accumulator
// hold sum_i X_i s_0, sum_i X_i s_1, sum_i X_i s_2 and their sum is the product — f32
// accumulation in tensor memory.  Each term a_k b_k is therefore off by at most 2^-17 of
// itself (7.6e-6, inside the 1e-5 the path is held to); the sums measured against float64
// are off by about 1e-7 of sum|a_k b_k|, the errors having no common sign.  (The third
// piece would cost a third more shared-memory traffic, which is what bounds the pass.)
//
// A block walks its 64-row tiles twice.  First over dY: TMA brings 64 rows x 128 columns
// (and the matching 16 x 128 piece of B) into a ring of plain row-major f32 stages;
// worker warps cut each stage into the pieces' tiles ([64 rows][64 columns] bf16 under
// the 128-byte swizzle, two per piece) in a second ring, and one thread then issues
//   - dT += dY_chunk B_chunk^T: A = a piece tile read K-major (64 rows x 16 columns per
//     instruction), B = B's pieces K-major.  A 64-row product leaves row r in tensor-memory
//     lane 32 (r / 16) + r % 16;
//   - dB_chunk += dY_chunk^T t: A = the same piece tiles read MN-major (128 columns x 16
//     rows per instruction), B = t's pieces as [48][64] K-major tiles the workers write.
// dT leaves through the workers (scaled, stored as f32 and as its three-way bf16 cut) one
// tile behind the products, from one of two tensor-memory buffers; dB leaves once as the
// block's partial sums.  Then over x, with the block's own dT rows read back as the small
// operand: dA_chunk += x_chunk^T dT in the same accumulator columns, stored the same way.
// The partial sums have the layout the fold kernel of k_lora_mma.cu adds up in block order.
//
// Every wait is bounded: a wait that runs out raises the status flag, and the block
// stops issuing work and frees its tensor memory.
#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>

#include "kernels.h"
#include "lora_split.cuh"
#include "lora_umma.h"
#include "umma_device.cuh"

namespace see::k {
namespace {
using namespace umma_dev;

constexpr int kR = 16;
constexpr int kWide = 3 * kR;                                   // an accumulator's three column groups
constexpr int kRows = 64;
constexpr int kChunk = 128;
constexpr uint32_t kRawActBytes = kRows * kChunk * 4;           // 32768, [64][128] f32
constexpr uint32_t kRawWBytes = kR * kChunk * 4;                // 8192,  [16][128] f32
constexpr uint32_t kRawBytes = kRawActBytes + kRawWBytes;
constexpr uint32_t kTileBytes = kRows * 128;                    // [64 rows][64 bf16]: 8192
constexpr uint32_t kWTileBytes = kR * 128;                      // [16 rows][64 bf16]: 2048
constexpr int kStreamPieces = 2;                                // pieces kept of dY and x (see above)
constexpr uint32_t kActPieceBytes = 2 * kStreamPieces * kTileBytes;   // piece p, column half h at tile 2 p + h
constexpr uint32_t kPieceBytes = kActPieceBytes + 6 * kWTileBytes;   // B's piece p, half h at tile 3 h + p
constexpr int kStages = 2;      // stages of the pieces' ring
constexpr int kRawStages = 3;   // stages of the f32 ring
constexpr uint32_t kSmallBytes = 3 * kWTileBytes;               // t's or dT's three pieces: [48][64] bf16
constexpr int kWorkerWarps = 12;   // a multiple of four: the warps of a lane quadrant share its chunks
constexpr int kWorkers = kWorkerWarps * 32;
constexpr int kThreads = 64 + kWorkers;
constexpr uint32_t kTmemCols = 512;
constexpr int kMaxChunks = (kTmemCols - 2 * kWide) / kWide;     // 8

struct Bars {
  uint64_t raw_full[kRawStages], raw_empty[kRawStages], pc_full[kStages], pc_empty[kStages];
  uint64_t small_ready[2], dt_full[2], dt_free[2], acc_full, acc_free;
  uint32_t tmem_base;
  volatile uint32_t abort;
};
constexpr size_t kSmemBytes = 1024 + kRawStages * kRawBytes + kStages * kPieceBytes + 2 * kSmallBytes + sizeof(Bars);

constexpr uint32_t kInstrDescAMnMajor = 1u << 15;

__device__ __forceinline__ void TmemLoad16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
// The three column groups of an accumulator row added up, smallest terms first.
__device__ __forceinline__ void LoadSummed(uint32_t taddr, float (&v)[kR]) {
  uint32_t g0[16], g1[16], g2[16];
  TmemLoad16(taddr, g0);
  TmemLoad16(taddr + kR, g1);
  TmemLoad16(taddr + 2 * kR, g2);
  TmemWaitLd();
#pragma unroll
  for (int n = 0; n < kR; ++n) v[n] = (__uint_as_float(g2[n]) + __uint_as_float(g1[n])) + __uint_as_float(g0[n]);
}
__device__ __forceinline__ void MbarArrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(SmemAddr(bar)) : "memory");
}
// A descriptor whose start address lies `bytes` further on (the address field holds bytes / 16).
__device__ __forceinline__ uint64_t Advance(uint64_t desc, uint32_t bytes) { return desc + (bytes >> 4); }
// Two values' three pieces, each as a bf16 pair (a in the low half): what Split3 gives for each.
__device__ __forceinline__ void Split3Pair(float a, float b, uint32_t (&p)[3]) {
  p[0] = PackBf16x2(a, b);
  const float a1 = a - __uint_as_float(p[0] << 16), b1 = b - __uint_as_float(p[0] & 0xFFFF0000u);
  p[1] = PackBf16x2(a1, b1);
  const float a2 = a1 - __uint_as_float(p[1] << 16), b2 = b1 - __uint_as_float(p[1] & 0xFFFF0000u);
  p[2] = PackBf16x2(a2, b2);
}
// Eight consecutive columns of a row: one 16-byte chunk per piece.
__device__ __forceinline__ void Split3Chunk(const float4& lo4, const float4& hi4, uint4 (&out)[3]) {
  uint32_t q[4][3];
  Split3Pair(lo4.x, lo4.y, q[0]);
  Split3Pair(lo4.z, lo4.w, q[1]);
  Split3Pair(hi4.x, hi4.y, q[2]);
  Split3Pair(hi4.z, hi4.w, q[3]);
#pragma unroll
  for (int p = 0; p < 3; ++p) out[p] = make_uint4(q[0][p], q[1][p], q[2][p], q[3][p]);
}
// The same with the first two pieces only (what the streamed operands keep).
__device__ __forceinline__ void Split2Chunk(const float4& lo4, const float4& hi4, uint4 (&out)[2]) {
  const float v[8] = {lo4.x, lo4.y, lo4.z, lo4.w, hi4.x, hi4.y, hi4.z, hi4.w};
  uint32_t p0[4], p1[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    p0[i] = PackBf16x2(v[2 * i], v[2 * i + 1]);
    p1[i] = PackBf16x2(v[2 * i] - __uint_as_float(p0[i] << 16), v[2 * i + 1] - __uint_as_float(p0[i] & 0xFFFF0000u));
  }
  out[0] = make_uint4(p0[0], p0[1], p0[2], p0[3]);
  out[1] = make_uint4(p1[0], p1[1], p1[2], p1[3]);
}
// Byte offset of element (n, k) in a [16][64] bf16 K-major tile under the 128-byte swizzle.
__device__ __forceinline__ uint32_t SmallOffset(uint32_t n, uint32_t k) {
  return Sw128Offset(n, k >> 3) + (k & 7u) * 2u;
}

__global__ void __launch_bounds__(kThreads, 1)
LoraBackwardUmmaKernel(const __grid_constant__ CUtensorMap map_dy, const __grid_constant__ CUtensorMap map_x,
                       const __grid_constant__ CUtensorMap map_b, const float* __restrict__ t,
                       float* dt, float* __restrict__ partials, uint32_t M, uint32_t N, uint32_t K,
                       float alpha_dt, uint16_t* __restrict__ pieces, uint32_t piece_cols, DeviceStatus* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (SmemAddr(smem_raw) & 1023u)) & 1023u);
  uint8_t* pc = smem;                                   // the pieces' ring first: its tiles want 1024-byte alignment
  uint8_t* small = pc + kStages * kPieceBytes;          // two buffers of the small operand's pieces
  uint8_t* raw = small + 2 * kSmallBytes;
  Bars* bars = reinterpret_cast<Bars*>(raw + kRawStages * kRawBytes);

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t nc = N / kChunk, kc = K / kChunk;
  const uint32_t tiles = (M + kRows - 1) / kRows;
  const uint32_t mine = blockIdx.x < tiles ? (tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0u;   // this block's tiles

  if (threadIdx.x == 0) {
    for (int s = 0; s < kRawStages; ++s) {
      MbarInit(&bars->raw_full[s], 1);
      MbarInit(&bars->raw_empty[s], kWorkerWarps);
    }
    for (int s = 0; s < kStages; ++s) {
      MbarInit(&bars->pc_full[s], kWorkerWarps);
      MbarInit(&bars->pc_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      MbarInit(&bars->small_ready[b], kWorkerWarps);
      MbarInit(&bars->dt_full[b], 1);
      MbarInit(&bars->dt_free[b], kWorkerWarps);
    }
    MbarInit(&bars->acc_full, 1);
    MbarInit(&bars->acc_free, kWorkerWarps);
    bars->abort = 0;
    MbarInitFence();
  }
  if (warp == 1) TmemAlloc(&bars->tmem_base, kTmemCols);
  TcFenceBefore();
  __syncthreads();
  TcFenceAfter();
  const uint32_t tmem_base = bars->tmem_base;
  const uint32_t tmem_acc = tmem_base, tmem_dt = tmem_base + kWide * kMaxChunks;   // dT: two buffers of 48 columns

  if (warp == 0) {
    // ---- TMA producer ----
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      auto stage = [&](const CUtensorMap* map, uint32_t c, uint32_t row0, bool with_b) {
        const uint32_t s = it % kRawStages, round = it / kRawStages;
        if (round > 0 && !MbarWait(&bars->raw_empty[s], (round - 1) & 1)) {
          status->wait_timeout = 1;
          bars->abort = 1;
          ok = false;
          return;
        }
        uint8_t* dst = raw + s * kRawBytes;
        MbarExpectTx(&bars->raw_full[s], with_b ? kRawBytes : kRawActBytes);
        TmaLoad2D(dst, map, &bars->raw_full[s], static_cast<int32_t>(c * kChunk), static_cast<int32_t>(row0));
        if (with_b) TmaLoad2D(dst + kRawActBytes, &map_b, &bars->raw_full[s], static_cast<int32_t>(c * kChunk), 0);
        ++it;
      };
      // The ring holds two stages, too little to cover the latency of HBM: position q of the stage
      // stream is asked into L2 kAhead stages before its load.
      constexpr uint32_t kAhead = 8;
      const uint32_t first_walk = mine * nc, total = first_walk + mine * kc;
      auto prefetch = [&](uint32_t q) {
        if (q >= total) return;
        const bool dy = q < first_walk;
        const uint32_t per = dy ? nc : kc, i = dy ? q : q - first_walk;
        const uint32_t v = i / per, c = i - v * per;
        asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];"
                     ::"l"(reinterpret_cast<uint64_t>(dy ? &map_dy : &map_x)), "r"(static_cast<int32_t>(c * kChunk)),
                       "r"(static_cast<int32_t>((blockIdx.x + v * gridDim.x) * kRows))
                     : "memory");
      };
      for (uint32_t q = 0; q < kAhead; ++q) prefetch(q);
      for (uint32_t v = 0; v < mine && ok; ++v)
        for (uint32_t c = 0; c < nc && ok; ++c) {
          prefetch(it + kAhead);
          stage(&map_dy, c, (blockIdx.x + v * gridDim.x) * kRows, true);
        }
      for (uint32_t v = 0; v < mine && ok; ++v)
        for (uint32_t c = 0; c < kc && ok; ++c) {
          prefetch(it + kAhead);
          stage(&map_x, c, (blockIdx.x + v * gridDim.x) * kRows, false);
        }
    }
  } else if (warp == 1) {
    // ---- MMA issue ----
    if (lane == 0) {
      const uint32_t idesc_rows = MakeInstrDesc(kRows, kWide);                      // dT: rows x k
      const uint32_t idesc_cols = MakeInstrDesc(128, kWide) | kInstrDescAMnMajor;   // dB, dA: columns x rows
      uint32_t it = 0;
      bool ok = true;
      auto fail = [&]() {
        status->wait_timeout = 1;
        bars->abort = 1;
        ok = false;
      };
      // D[chunk] += stage^T small, the 64 rows of the tile as the reduction axis.
      auto columns_times_small = [&](uint32_t act, uint32_t small_addr, uint32_t tmem_d, bool first) {
        const uint64_t a0 = MakeSmemDescMn(act, kTileBytes), b0 = MakeSmemDesc(small_addr);
#pragma unroll
        for (uint32_t k16 = 0; k16 < kRows / 16; ++k16) {
#pragma unroll
          for (uint32_t p = 0; p < kStreamPieces; ++p)
            UmmaBf16(tmem_d, Advance(a0, p * 2 * kTileBytes + k16 * 2048u), Advance(b0, k16 * 32u), idesc_cols,
                     (first && k16 == 0 && p == 0) ? 0u : 1u);
        }
      };
      auto wait_small = [&](uint32_t u) { return MbarWait(&bars->small_ready[u & 1], (u >> 1) & 1); };
      // ---- over dY: dT and dB ----
      for (uint32_t v = 0; v < mine && ok; ++v) {
        if (!wait_small(v)) { fail(); break; }
        if (v >= 2 && !MbarWait(&bars->dt_free[v & 1], ((v >> 1) - 1) & 1)) { fail(); break; }
        TcFenceAfter();
        const uint32_t tmem_t = tmem_dt + (v & 1) * kWide;
        for (uint32_t c = 0; c < nc && ok; ++c, ++it) {
          const uint32_t s = it % kStages, round = it / kStages;
          if (!MbarWait(&bars->pc_full[s], round & 1)) { fail(); break; }
          TcFenceAfter();
          const uint32_t act = SmemAddr(pc + s * kPieceBytes), wgt = act + kActPieceBytes;
          const uint64_t a0 = MakeSmemDesc(act), b0 = MakeSmemDesc(wgt);
#pragma unroll
          for (uint32_t kk = 0; kk < kChunk / 16; ++kk) {
            const uint32_t h = kk >> 2, off = (kk & 3u) * 32u;
#pragma unroll
            for (uint32_t p = 0; p < kStreamPieces; ++p)
              UmmaBf16(tmem_t, Advance(a0, (2 * p + h) * kTileBytes + off), Advance(b0, 3 * h * kWTileBytes + off),
                       idesc_rows, (c == 0 && kk == 0 && p == 0) ? 0u : 1u);
          }
          columns_times_small(act, SmemAddr(small + (v & 1) * kSmallBytes), tmem_acc + kWide * c, v == 0);
          UmmaCommit(&bars->pc_empty[s]);
        }
        if (ok) UmmaCommit(&bars->dt_full[v & 1]);
      }
      if (ok && mine > 0) {
        UmmaCommit(&bars->acc_full);
        if (!MbarWait(&bars->acc_free, 0)) fail();   // dB has left the accumulator columns
        TcFenceAfter();
      }
      // ---- over x: dA ----
      for (uint32_t v = 0; v < mine && ok; ++v) {
        if (!wait_small(mine + v)) { fail(); break; }
        TcFenceAfter();
        for (uint32_t c = 0; c < kc && ok; ++c, ++it) {
          const uint32_t s = it % kStages, round = it / kStages;
          if (!MbarWait(&bars->pc_full[s], round & 1)) { fail(); break; }
          TcFenceAfter();
          columns_times_small(SmemAddr(pc + s * kPieceBytes), SmemAddr(small + ((mine + v) & 1) * kSmallBytes),
                              tmem_acc + kWide * c, v == 0);
          UmmaCommit(&bars->pc_empty[s]);
        }
      }
      if (ok && mine > 0) UmmaCommit(&bars->acc_full);
    }
  } else {
    // ---- workers: cut the stages, carry dT out, store the partial sums ----
    const uint32_t w = warp - 2, wt = threadIdx.x - 64;
    const uint32_t quad = warp & 3u;   // the tensor-memory lanes this warp may read: 32 quad .. 32 quad + 31
    uint32_t it = 0;
    bool ok = true;
    auto give_up = [&]() {
      if (lane == 0) { status->wait_timeout = 1; bars->abort = 1; }
      ok = false;
    };
    // An item: eight consecutive columns of a row (32 bytes in, one 16-byte chunk per piece out).  A
    // thread's items are the same in every stage: item wt + j kWorkers, rows 64 .. 79 being B's.
    constexpr int kItemsPerWorker = ((kRows + kR) * (kChunk / 8) + kWorkers - 1) / kWorkers;
    uint32_t item_src[kItemsPerWorker], item_dst[kItemsPerWorker], item_kind[kItemsPerWorker];   // kind: 0 rows, 1 B, 2 none
#pragma unroll
    for (int j = 0; j < kItemsPerWorker; ++j) {
      const uint32_t i = wt + j * kWorkers, r = i >> 4, c8 = i & 15u, h = c8 >> 3, chunk = c8 & 7u;
      item_src[j] = r * (kChunk * 4) + c8 * 32u;
      item_kind[j] = r < kRows ? 0u : (r < kRows + kR ? 1u : 2u);
      item_dst[j] = r < kRows ? h * kTileBytes + Sw128Offset(r, chunk)
                              : kActPieceBytes + 3 * h * kWTileBytes + Sw128Offset(r - kRows, chunk);
    }
    // (the upper half of a quarter warp takes its two 16-byte halves in the other order: eight lanes, eight bank groups)
    const uint32_t flip = (wt >> 2) & 1u;
    auto cut_stage = [&](bool with_b) {
      const uint32_t s = it % kStages, round = it / kStages, rs = it % kRawStages, raw_round = it / kRawStages;
      if (!MbarWait(&bars->raw_full[rs], raw_round & 1)) { give_up(); return; }
      if (round > 0 && !MbarWait(&bars->pc_empty[s], (round - 1) & 1)) { give_up(); return; }
      const uint8_t* src = raw + rs * kRawBytes;
      uint8_t* dst = pc + s * kPieceBytes;
#pragma unroll
      for (int j = 0; j < kItemsPerWorker; ++j) {
        if (item_kind[j] == 2u || (item_kind[j] == 1u && !with_b)) continue;
        const float4* in = reinterpret_cast<const float4*>(src + item_src[j]);
        const float4 in_a = in[flip], in_b = in[flip ^ 1u];
        if (item_kind[j] == 0u) {
          uint4 out[2];
          Split2Chunk(flip ? in_b : in_a, flip ? in_a : in_b, out);
          *reinterpret_cast<uint4*>(dst + item_dst[j]) = out[0];
          *reinterpret_cast<uint4*>(dst + item_dst[j] + 2 * kTileBytes) = out[1];
        } else {
          uint4 out[3];
          Split3Chunk(flip ? in_b : in_a, flip ? in_a : in_b, out);
#pragma unroll
          for (int p = 0; p < 3; ++p) *reinterpret_cast<uint4*>(dst + item_dst[j] + p * kWTileBytes) = out[p];
        }
      }
      FenceProxyAsync();
      __syncwarp();
      if (lane == 0) {
        MbarArrive(&bars->pc_full[s]);
        MbarArrive(&bars->raw_empty[rs]);
      }
      ++it;
    };
    // The rows [row0, row0 + 64) of a [M, 16] f32 matrix as the small operand's pieces, use u of the two
    // buffers; small_load reads them a tile ahead of small_store.  (The products that read this buffer
    // two uses ago have completed: the stage ring's waits since then cover them, a tile being at least
    // two stages long.)
    auto small_load = [&](const float* src, uint32_t row0) {
      const uint32_t r = wt >> 2, n0 = (wt & 3u) * 4u;
      if (wt < 4 * kRows && row0 + r < M)
        return *reinterpret_cast<const float4*>(src + static_cast<size_t>(row0 + r) * kR + n0);
      return make_float4(0.f, 0.f, 0.f, 0.f);
    };
    auto small_store = [&](const float4& v, uint32_t u) {
      uint8_t* dst = small + (u & 1) * kSmallBytes;
      const uint32_t r = wt >> 2, n0 = (wt & 3u) * 4u;
      if (wt < 4 * kRows) {
        const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) {
          uint16_t p[3];
          Split3(e[j], p);
          const uint32_t off = SmallOffset(n0 + j, r);
#pragma unroll
          for (int q = 0; q < 3; ++q) *reinterpret_cast<uint16_t*>(dst + q * kWTileBytes + off) = p[q];
        }
      }
      FenceProxyAsync();
      __syncwarp();
      if (lane == 0) MbarArrive(&bars->small_ready[u & 1]);
    };
    // Tile v's dT out of tensor memory: scaled, stored, cut.
    auto dt_out = [&](uint32_t v) {
      if (!MbarWait(&bars->dt_full[v & 1], (v >> 1) & 1)) { give_up(); return; }
      TcFenceAfter();
      if (w < 4) {   // one warp per lane quadrant: its lanes 0 .. 15 hold rows 16 quad .. 16 quad + 15
        const uint32_t row0 = (blockIdx.x + v * gridDim.x) * kRows;
        float val[kR];
        LoadSummed(tmem_dt + (v & 1) * kWide + ((quad * 32u) << 16), val);
        const uint32_t r = quad * 16u + lane;
        if (lane < 16 && row0 + r < M) {
#pragma unroll
          for (int n = 0; n < kR; ++n) val[n] *= alpha_dt;
          float4* dst = reinterpret_cast<float4*>(dt + static_cast<size_t>(row0 + r) * kR);
#pragma unroll
          for (int q = 0; q < kR / 4; ++q)
            dst[q] = make_float4(val[4 * q], val[4 * q + 1], val[4 * q + 2], val[4 * q + 3]);
          if (pieces != nullptr) {
            uint16_t p[kR][3];
#pragma unroll
            for (int n = 0; n < kR; ++n) Split3(val[n], p[n]);
            uint16_t* out = pieces + static_cast<size_t>(row0 + r) * piece_cols;
#pragma unroll
            for (int sg = 0; sg < 6; ++sg) {
              const int pcs = PieceOf(0, sg);
              uint32_t wds[kR / 2];
#pragma unroll
              for (int n = 0; n < kR / 2; ++n)
                wds[n] = static_cast<uint32_t>(p[2 * n][pcs]) | (static_cast<uint32_t>(p[2 * n + 1][pcs]) << 16);
              uint4* o = reinterpret_cast<uint4*>(out + sg * kR);
              o[0] = make_uint4(wds[0], wds[1], wds[2], wds[3]);
              o[1] = make_uint4(wds[4], wds[5], wds[6], wds[7]);
            }
            for (uint32_t k = 6 * kR; k < piece_cols; k += 8)   // the padding columns
              *reinterpret_cast<uint4*>(out + k) = make_uint4(0u, 0u, 0u, 0u);
          }
        }
      }
      TcFenceBefore();
      __syncwarp();
      if (lane == 0) MbarArrive(&bars->dt_free[v & 1]);
    };
    // The accumulator columns as this block's partial sums; `by_column`: [16][width] (dB), else [width][16] (dA).
    auto store_partials = [&](float* out, uint32_t chunks, uint32_t width, bool by_column) {
      for (uint32_t c = w >> 2; c < chunks; c += kWorkerWarps / 4) {   // the warps of a quadrant take chunks in turn
        float val[kR];
        LoadSummed(tmem_acc + kWide * c + ((quad * 32u) << 16), val);
        const uint32_t f = c * kChunk + quad * 32u + lane;
        if (by_column) {
#pragma unroll
          for (int n = 0; n < kR; ++n) out[static_cast<size_t>(n) * width + f] = val[n];
        } else {
          float4* dst = reinterpret_cast<float4*>(out + static_cast<size_t>(f) * kR);
#pragma unroll
          for (int q = 0; q < kR / 4; ++q)
            dst[q] = make_float4(val[4 * q], val[4 * q + 1], val[4 * q + 2], val[4 * q + 3]);
        }
      }
    };
    float* pb = partials + static_cast<size_t>(blockIdx.x) * (static_cast<size_t>(kR) * N + static_cast<size_t>(K) * kR);
    float* pa = pb + static_cast<size_t>(kR) * N;

    // ---- over dY ----
    float4 ahead = mine > 0 ? small_load(t, blockIdx.x * kRows) : make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t v = 0; v < mine && ok; ++v) {
      const float4 now = ahead;
      if (v + 1 < mine) ahead = small_load(t, (blockIdx.x + (v + 1) * gridDim.x) * kRows);
      small_store(now, v);
      cut_stage(true);
      if (ok && v > 0) dt_out(v - 1);   // one tile behind: its products have had a stage's time to complete
      for (uint32_t c = 1; c < nc && ok; ++c) cut_stage(true);
    }
    if (ok && mine > 0) dt_out(mine - 1);
    if (ok && mine > 0 && !MbarWait(&bars->acc_full, 0)) give_up();
    if (ok && mine > 0) {
      TcFenceAfter();
      store_partials(pb, nc, N, true);
      TcFenceBefore();
      __threadfence_block();   // this block's dT rows, written by two of the warps, are read back by all of them
      __syncwarp();
      if (lane == 0) MbarArrive(&bars->acc_free);
      if (!MbarWait(&bars->acc_free, 0)) give_up();   // every worker warp has stored its rows
    }
    // ---- over x ----
    if (ok && mine > 0) ahead = small_load(dt, blockIdx.x * kRows);
    for (uint32_t v = 0; v < mine && ok; ++v) {
      const float4 now = ahead;
      if (v + 1 < mine) ahead = small_load(dt, (blockIdx.x + (v + 1) * gridDim.x) * kRows);
      small_store(now, mine + v);
      for (uint32_t c = 0; c < kc && ok; ++c) cut_stage(false);
    }
    if (ok && mine > 0 && !MbarWait(&bars->acc_full, 1)) give_up();
    if (ok && mine > 0) {
      TcFenceAfter();
      store_partials(pa, kc, K, false);
    }
  }

  TcFenceBefore();
  __syncthreads();
  if (warp == 1) {
    TcFenceAfter();
    TmemFree(tmem_base, kTmemCols);
  }
}

std::atomic<bool> g_enabled{true};

}  // namespace

void LoraBackwardUmmaSet(bool on) { g_enabled.store(on, std::memory_order_relaxed); }
bool LoraBackwardUmmaEnabled() { return g_enabled.load(std::memory_order_relaxed); }

bool LoraBackwardUmmaSupported(size_t M, size_t N, size_t K, size_t r) {
  return r == kR && M >= kRows && M <= 0x7FFFFFFFull && N % kChunk == 0 && K % kChunk == 0 && N >= 2 * kChunk &&
         K >= 2 * kChunk && N <= kMaxChunks * kChunk && K <= kMaxChunks * kChunk;
}

int LoraBackwardUmmaBlocks(size_t M, int sms) {
  const size_t tiles = (M + kRows - 1) / kRows;
  return static_cast<int>(tiles < static_cast<size_t>(sms) ? tiles : static_cast<size_t>(sms));
}

cudaError_t LoraBackwardUmmaLaunch(const CUtensorMap& map_dy, const CUtensorMap& map_x, const CUtensorMap& map_b,
                                   const LoraBackwardArgs& a, int blocks, DeviceStatus* status, cudaStream_t s) {
  static std::atomic<bool> configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  const bool tracked = dev >= 0 && dev < 64;
  if (!tracked || !configured[dev].load(std::memory_order_acquire)) {
    const cudaError_t e = cudaFuncSetAttribute(LoraBackwardUmmaKernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(kSmemBytes));
    if (e != cudaSuccess) return e;
    if (tracked) configured[dev].store(true, std::memory_order_release);
  }
  LoraBackwardUmmaKernel<<<blocks, kThreads, kSmemBytes, s>>>(
      map_dy, map_x, map_b, a.t, a.dt, a.partials, static_cast<uint32_t>(a.M), static_cast<uint32_t>(a.N),
      static_cast<uint32_t>(a.K), a.alpha_dt, a.dt_pieces, LoraSplitColumns(static_cast<uint32_t>(a.r)), status);
  return cudaGetLastError();
}

}  // namespace see::k
