// The tensor-core GEMM for frozen-weight products that carry the relaxed
// permission (reference: source/plan/instruction.h:356-382; the reference's own
// relaxed kernels are runtime/executor/metal_backend.mm:1385-1449):
//
//     C[M,N] = epilogue( A_bf16[M,K] . B_bf16[N,K]^T )       f32 accumulate
//
// Blackwell-native: operands arrive by TMA (cp.async.bulk.tensor, 128-byte
// swizzle) into a 3-stage shared-memory ring, one elected thread issues
// tcgen05.mma (cta_group::1, kind::f16, M=128 x N=128 x K=16) with the
// accumulator in tensor memory, tcgen05.commit hands ring slots back to the
// producer, and four epilogue warps read the accumulator with tcgen05.ld and
// apply scale / addend / bias / activation on the way to HBM.  One CTA per
// 128x128 output tile, two CTAs resident per SM so one tile's epilogue
// overlaps another's main loop.  Tensor-pipe bound for long K; for K <= 1024
// the f32 output write is a comparable term (the arena is f32 by contract).
//
// Every wait on an mbarrier is bounded; a wait that runs out raises
// DeviceStatus::wait_timeout, the CTA stops issuing work, frees its tensor
// memory and returns, and the host reports the condition at its next flush.
#include <cuda.h>

#include <utility>

#include <atomic>

#include "act_expr.cuh"
#include "kernels.h"
#include "shadow.cuh"
#include "umma_device.cuh"
#include "umma_kernel.h"

namespace see::k {

namespace {

constexpr uint32_t kBlockM = umma_cfg::kBlockM;
constexpr uint32_t kBlockN = umma_cfg::kBlockN;
constexpr uint32_t kBlockK = umma_cfg::kBlockK;   // 64 bf16 = one 128-byte swizzle row
constexpr uint32_t kStages = umma_cfg::kStages;
constexpr uint32_t kUmmaK = 16;
constexpr uint32_t kATileBytes = kBlockM * kBlockK * 2;
constexpr uint32_t kBTileBytes = kBlockN * kBlockK * 2;
constexpr uint32_t kStageBytes = kATileBytes + kBTileBytes;
constexpr uint32_t kTmemCols = kBlockN;           // f32 accumulator columns
constexpr uint32_t kThreads = 192;                // warp 0 TMA, warp 1 MMA, warps 2-5 epilogue


using namespace umma_dev;   // mbarriers with bounded waits, TMA loads, descriptors, MMA issue, TMEM loads

__device__ __forceinline__ float ApplyAct(float v, int act) { return ActFwdExpr(act, v); }

// The tail of both epilogues: four neighbouring columns n.. of row (at / N).
__device__ __forceinline__ void EpilogueStore(const UmmaEpilogue& ep, size_t at, uint32_t n, const float4& acc,
                                              const float4& scale, const float4& bias,
                                              bool has_kscale = false,
                                              float4 kscale = make_float4(1.f, 1.f, 1.f, 1.f),
                                              bool has_side = false,   // the addend / x element, already loaded
                                              float4 side = make_float4(0.f, 0.f, 0.f, 0.f)) {
  float4 v = make_float4(acc.x * scale.x, acc.y * scale.y, acc.z * scale.z, acc.w * scale.w);
  if (ep.addend && !ep.addend_last) {
    const float4 d = has_side ? side : __ldg(reinterpret_cast<const float4*>(ep.addend + at));
    v = make_float4(d.x + v.x, d.y + v.y, d.z + v.z, d.w + v.w);
  }
  if (ep.bias) v = make_float4(v.x + bias.x, v.y + bias.y, v.z + bias.z, v.w + bias.w);
  if (ep.addend && ep.addend_last) {   // an absorbed kAddEW that followed the kAddBias
    const float4 d = has_side ? side : __ldg(reinterpret_cast<const float4*>(ep.addend + at));
    v = make_float4(d.x + v.x, d.y + v.y, d.z + v.z, d.w + v.w);
  }
  if (ep.act != kActNone)
    v = make_float4(ApplyAct(v.x, ep.act), ApplyAct(v.y, ep.act), ApplyAct(v.z, ep.act),
                    ApplyAct(v.w, ep.act));
  if (ep.store_c) *reinterpret_cast<float4*>(ep.C + at) = v;
  if (ep.pack_dst) {   // the bf16 operand copy a tiled attention instruction reads this tensor through
    uint32_t lo, hi;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(lo) : "f"(v.y), "f"(v.x));
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(hi) : "f"(v.w), "f"(v.z));
    *reinterpret_cast<uint2*>(ep.pack_dst + at) = make_uint2(lo, hi);
  }
  if (ep.fuse_mode != kFuseNone) {
    float4 g;
    if (ep.fuse_mode == kFuseActFwd) {
      if (ep.fuse_act == kActGelu) {   // two elements per instruction; the bits of GeluExpr
        UnpackF2(GeluExpr2(PackF2(v.x, v.y)), &g.x, &g.y);
        UnpackF2(GeluExpr2(PackF2(v.z, v.w)), &g.z, &g.w);
      } else {
        g = make_float4(ActFwdExpr(ep.fuse_act, v.x), ActFwdExpr(ep.fuse_act, v.y),
                        ActFwdExpr(ep.fuse_act, v.z), ActFwdExpr(ep.fuse_act, v.w));
      }
    } else {
      const float4 x = has_side ? side : __ldg(reinterpret_cast<const float4*>(ep.fuse_x + at));
      if (ep.fuse_act == kActGelu) {   // likewise, the bits of GeluGrad
        UnpackF2(GeluGrad2(PackF2(v.x, v.y), PackF2(x.x, x.y)), &g.x, &g.y);
        UnpackF2(GeluGrad2(PackF2(v.z, v.w), PackF2(x.z, x.w)), &g.z, &g.w);
      } else {
        g = make_float4(ActBwdExpr(ep.fuse_act, v.x, x.x), ActBwdExpr(ep.fuse_act, v.y, x.y),
                        ActBwdExpr(ep.fuse_act, v.z, x.z), ActBwdExpr(ep.fuse_act, v.w, x.w));
      }
    }
    Shadow sh;
    sh.dst = ep.shadow_dst;
    sh.k_scale = has_kscale ? nullptr : ep.shadow_k_scale;
    sh.cols = ep.N;
    if (has_kscale) g = make_float4(g.x * kscale.x, g.y * kscale.y, g.z * kscale.z, g.w * kscale.w);
    ShadowStore4(sh, at / 4, n, g);
  }
}

// EpilogueStore for the one form in which instruction count bounds the whole kernel: an absorbed GELU
// gradient and nothing else (no addend, bias, activation or attention copy).  The same values, without
// the per-element tests of the general form.
__device__ __forceinline__ bool IsGeluGradOnly(const UmmaEpilogue& ep) {
  return ep.fuse_mode == kFuseActBwd && ep.fuse_act == kActGelu && ep.addend == nullptr && ep.bias == nullptr &&
         ep.act == kActNone && ep.pack_dst == nullptr;
}
__device__ __forceinline__ void EpilogueStoreGeluGrad(const UmmaEpilogue& ep, size_t at, const float4& acc,
                                                      const float4& scale, const float4& kscale, const float4& x) {
  const float4 v = make_float4(acc.x * scale.x, acc.y * scale.y, acc.z * scale.z, acc.w * scale.w);
  if (ep.store_c) *reinterpret_cast<float4*>(ep.C + at) = v;
  float4 g;
  UnpackF2(GeluGrad2(PackF2(v.x, v.y), PackF2(x.x, x.y)), &g.x, &g.y);
  UnpackF2(GeluGrad2(PackF2(v.z, v.w), PackF2(x.z, x.w)), &g.z, &g.w);
  uint2 r;
  r.x = ShadowBf16x2(g.x * kscale.x, g.y * kscale.y);
  r.y = ShadowBf16x2(g.z * kscale.z, g.w * kscale.w);
  reinterpret_cast<uint2*>(ep.shadow_dst)[at >> 2] = r;
}

// Likewise for an addend and nothing else (the accumulating gradient products): C = addend + acc * scale.
__device__ __forceinline__ bool IsAddendOnly(const UmmaEpilogue& ep) {
  return ep.addend != nullptr && ep.bias == nullptr && ep.act == kActNone && ep.pack_dst == nullptr &&
         ep.fuse_mode == kFuseNone && ep.store_c;
}
__device__ __forceinline__ void EpilogueStoreAddend(const UmmaEpilogue& ep, size_t at, const float4& acc,
                                                    const float4& scale, const float4& d) {
  *reinterpret_cast<float4*>(ep.C + at) =
      make_float4(d.x + acc.x * scale.x, d.y + acc.y * scale.y, d.z + acc.z * scale.z, d.w + acc.w * scale.w);
}
// ... for a product that leaves only as the bf16 copy a tiled attention instruction reads (Q, K, V) ...
__device__ __forceinline__ bool IsCopyOnly(const UmmaEpilogue& ep) {
  return ep.addend == nullptr && ep.bias == nullptr && ep.act == kActNone && ep.pack_dst != nullptr &&
         ep.fuse_mode == kFuseNone && !ep.store_c;
}
__device__ __forceinline__ void EpilogueStoreCopy(const UmmaEpilogue& ep, size_t at, const float4& acc,
                                                  const float4& scale) {
  uint32_t lo, hi;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(lo) : "f"(acc.y * scale.y), "f"(acc.x * scale.x));
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(hi) : "f"(acc.w * scale.w), "f"(acc.z * scale.z));
  *reinterpret_cast<uint2*>(ep.pack_dst + at) = make_uint2(lo, hi);
}
// ... for a product stored as it is (the vocabulary head, the gradient products that carry nothing else) ...
__device__ __forceinline__ bool IsPlainStore(const UmmaEpilogue& ep) {
  return ep.addend == nullptr && ep.bias == nullptr && ep.act == kActNone && ep.pack_dst == nullptr &&
         ep.fuse_mode == kFuseNone && ep.store_c;
}
__device__ __forceinline__ void EpilogueStorePlain(const UmmaEpilogue& ep, size_t at, const float4& acc,
                                                   const float4& scale) {
  *reinterpret_cast<float4*>(ep.C + at) =
      make_float4(acc.x * scale.x, acc.y * scale.y, acc.z * scale.z, acc.w * scale.w);
}
// ... and for a bias followed by an absorbed GELU (the feed-forward up product): C = acc * scale + bias,
// the bf16 operand copy of gelu(C) beside it.
__device__ __forceinline__ bool IsBiasGeluOnly(const UmmaEpilogue& ep) {
  return ep.addend == nullptr && ep.bias != nullptr && ep.act == kActNone && ep.pack_dst == nullptr &&
         ep.fuse_mode == kFuseActFwd && ep.fuse_act == kActGelu && ep.store_c;
}
__device__ __forceinline__ void EpilogueStoreBiasGelu(const UmmaEpilogue& ep, size_t at, const float4& acc,
                                                      const float4& scale, const float4& bias, const float4& kscale) {
  float4 v = make_float4(acc.x * scale.x, acc.y * scale.y, acc.z * scale.z, acc.w * scale.w);
  v = make_float4(v.x + bias.x, v.y + bias.y, v.z + bias.z, v.w + bias.w);
  *reinterpret_cast<float4*>(ep.C + at) = v;
  float4 g;
  UnpackF2(GeluExpr2(PackF2(v.x, v.y)), &g.x, &g.y);
  UnpackF2(GeluExpr2(PackF2(v.z, v.w)), &g.z, &g.w);
  uint2 r;
  r.x = ShadowBf16x2(g.x * kscale.x, g.y * kscale.y);
  r.y = ShadowBf16x2(g.z * kscale.z, g.w * kscale.w);
  reinterpret_cast<uint2*>(ep.shadow_dst)[at >> 2] = r;
}

struct __align__(8) Barriers {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmem_full;
  uint32_t tmem_base;
  volatile uint32_t abort;  // set by a role whose wait ran out; the epilogue then stores nothing
};

__global__ void __launch_bounds__(kThreads, 2)
UmmaGemmKernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_a2, const __grid_constant__ CUtensorMap map_b2,
               UmmaEpilogue ep) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: the swizzle pattern and the descriptors' base offset assume it.
  uint8_t* smem = smem_raw + ((1024u - (SmemAddr(smem_raw) & 1023u)) & 1023u);
  Barriers* bars = reinterpret_cast<Barriers*>(smem + kStages * kStageBytes);

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t m0 = blockIdx.y * kBlockM, n0 = blockIdx.x * kBlockN;
  // The reduction runs over the main operands' K and then over aux_k_blocks more
  // 64-wide blocks taken from the second pair of maps (a low-rank term T . B'^T
  // accumulated into the same tile; see UmmaEpilogue::aux_k_blocks).
  const uint32_t main_blocks = (ep.K + kBlockK - 1) / kBlockK;
  const uint32_t k_blocks = main_blocks + ep.aux_k_blocks;

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < kStages; ++s) {
      MbarInit(&bars->full[s], 1);
      MbarInit(&bars->empty[s], 1);
    }
    MbarInit(&bars->tmem_full, 1);
    bars->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(SmemAddr(&bars->tmem_base)), "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ---- TMA producer ----
    if (lane == 0) {
      for (uint32_t kb = 0; kb < k_blocks; ++kb) {
        const uint32_t s = kb % kStages, round = kb / kStages;
        if (round > 0 && !MbarWait(&bars->empty[s], (round - 1) & 1)) {
          ep.status->wait_timeout = 1;
          bars->abort = 1;
          break;
        }
        uint8_t* a_dst = smem + s * kStageBytes;
        uint8_t* b_dst = a_dst + kATileBytes;
        MbarExpectTx(&bars->full[s], kStageBytes);
        const bool aux = kb >= main_blocks;
        const int32_t kx = static_cast<int32_t>((aux ? kb - main_blocks : kb) * kBlockK);
        TmaLoad2D(a_dst, aux ? &map_a2 : &map_a, &bars->full[s], kx, static_cast<int32_t>(m0));
        TmaLoad2D(b_dst, aux ? &map_b2 : &map_b, &bars->full[s], kx, static_cast<int32_t>(n0));
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ----
    if (lane == 0) {
      const uint32_t idesc = MakeInstrDesc(kBlockM, kBlockN);
      bool ok = true;
      for (uint32_t kb = 0; kb < k_blocks && ok; ++kb) {
        const uint32_t s = kb % kStages, round = kb / kStages;
        if (!MbarWait(&bars->full[s], round & 1)) {
          ep.status->wait_timeout = 1;
          bars->abort = 1;
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_addr = SmemAddr(smem + s * kStageBytes);
        const uint64_t desc_a = MakeSmemDesc(a_addr);
        const uint64_t desc_b = MakeSmemDesc(a_addr + kATileBytes);
#pragma unroll
        for (uint32_t k = 0; k < kBlockK / kUmmaK; ++k) {
          // advance 16 bf16 = 32 bytes inside the 128-byte swizzle row: +2 in >>4 units
          UmmaBf16(tmem_base, desc_a + 2 * k, desc_b + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
        }
        UmmaCommit(&bars->empty[s]);  // the slot is free once these MMAs have read it
      }
      UmmaCommit(&bars->tmem_full);   // accumulator complete (or abandoned on timeout)
    }
  } else {
    // ---- epilogue: warps 2..5, TMEM lane quarter = warp % 4 ----
    const uint32_t quarter = warp & 3;
    bool ok = MbarWait(&bars->tmem_full, 0);
    if (!ok && lane == 0) ep.status->wait_timeout = 1;
    if (bars->abort) ok = false;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok && k_blocks > 0) {
      // The accumulator arrives one row per thread; HBM wants one row per warp
      // access.  Each warp turns its 32 x 128 slab through shared memory: the
      // operand ring is idle by now (tmem_full fires after the last MMA has read
      // it), so the slab lives there.  16-byte chunks are XOR-swizzled with the
      // row so both the row-per-thread writes and the row-per-warp reads are
      // bank-conflict free.  Only this warp touches its slab: __syncwarp suffices.
      float* slab = reinterpret_cast<float*>(smem + quarter * (32 * kBlockN * 4));
#pragma unroll 1
      for (uint32_t c0 = 0; c0 < kBlockN; c0 += 32) {
        uint32_t r[32];
        TmemLoad32(tmem_base + ((quarter * 32) << 16) + c0, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (uint32_t q = 0; q < 8; ++q) {
          const uint32_t chunk = ((c0 >> 2) + q) ^ lane;   // 32 chunks of 4 floats per row
          *reinterpret_cast<uint4*>(slab + lane * kBlockN + chunk * 4) =
              make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
        }
      }
      __syncwarp();
      // Lane l owns columns n0 + 4l .. 4l+3 of every row: its scale / bias are loop invariants.
      const uint32_t n = n0 + lane * 4;
      if (n < ep.N) {   // N % 4 == 0: a float4 is all in or all out
        float4 scale = make_float4(ep.alpha, ep.alpha, ep.alpha, ep.alpha);
        if (ep.col_scale) scale = __ldg(reinterpret_cast<const float4*>(ep.col_scale + n));
        float4 bias = make_float4(0.f, 0.f, 0.f, 0.f);
        if (ep.bias) bias = __ldg(reinterpret_cast<const float4*>(ep.bias + n));
        const uint32_t row0 = m0 + quarter * 32;
        const uint32_t rows = row0 < ep.M ? (ep.M - row0 < 32 ? ep.M - row0 : 32) : 0;
#pragma unroll 4
        for (uint32_t rr = 0; rr < rows; ++rr) {
          const float4 acc = *reinterpret_cast<const float4*>(slab + rr * kBlockN + ((lane ^ rr) * 4));
          const size_t at = static_cast<size_t>(row0 + rr) * ep.N + n;
          EpilogueStore(ep, at, n, acc, scale, bias);
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(kTmemCols)
                 : "memory");
  }
}

// ---- persistent form -------------------------------------------------------------------
// One CTA per SM walks 128 x 256 output tiles t = blockIdx.x, blockIdx.x +
// gridDim.x, ... (tiles of one row block are neighbours, so concurrent CTAs
// share A in L2).  The wider tile is what the shared-memory fill rate asks for:
// a 128 x 128 tile moves 32 KB per 128x128x64 block of math (64 FLOP per byte
// from L2), which tops out near 12-13 TB/s of L2 traffic well below the tensor
// peak; 128 x 256 moves 48 KB per twice the math (85 FLOP per byte).  The
// operand ring keeps flowing across tile boundaries, the accumulator is
// double-buffered in tensor memory (2 x 256 columns: all of it), and the
// epilogue warps own a small staging slab, so tile i's epilogue (128 KB of f32) runs
// under tile i+1's main loop.  What the one-tile kernel pays per tile — barrier
// set-up, tensor-memory allocation, the first TMA round trip, CTA launch and
// retirement — is paid once per SM.
// The tile width is a template parameter: 256 columns where the product has tiles
// to spare, 128 where the wide tile would leave SMs without work (a shard of a
// few thousand rows with a 768-wide output: 96 wide tiles for 148 SMs, against
// 192 narrow ones; the narrow tile's shorter stage buys a fourth ring slot).
constexpr uint32_t kPBlockN = 256;                     // the wide tile
constexpr uint32_t kPMaxStages = 5;
constexpr uint32_t kPEpiWarps = 16;
constexpr uint32_t kPThreads = 64 + 32 * kPEpiWarps;   // warp 0 TMA, warp 1 MMA, then the epilogue warps
constexpr uint32_t kSlabCols = 32;
constexpr uint32_t kSlabBytes = 32 * kSlabCols * 4;   // one epilogue warp's 32 x 32 f32
// kPair: two CTAs of a cluster work one 256 x 256 tile (cta_group::2): each loads
// its own 128 rows of A and its own 128 of B's 256 rows (32 KB per k block instead
// of 48 KB for the same 128 x 256 of output per CTA), the even CTA issues one
// 256-row MMA that reads both shared memories, and each CTA's tensor memory
// receives its own 128 rows.  A third less operand traffic from L2 per flop, and
// the smaller stage leaves room for five ring slots: the K = 768 shapes of the
// step were bound by bytes in flight per SM, not by the tensor pipe.
template <uint32_t kTN, bool kPair>
struct PTile {
  static constexpr uint32_t kStages = kPair ? 5 : (kTN == 256 ? 3 : 4);
  static constexpr uint32_t kBRows = kPair ? kTN / 2 : kTN;      // rows of B this CTA loads per k block
  static constexpr uint32_t kBTileBytes = kBRows * kBlockK * 2;
  static constexpr uint32_t kStageBytes = kATileBytes + kBTileBytes;
  static constexpr uint32_t kTmemCols = 2 * kTN;
  static constexpr uint32_t kColsPerEpiWarp = kTN / (kPEpiWarps / 4);
  static constexpr uint32_t kEpiPasses = kColsPerEpiWarp / kSlabCols;
  static constexpr uint32_t kRowsPerTile = kPair ? 2 * kBlockM : kBlockM;
};

// Tile order of the persistent kernel.  Bands of band_blocks row blocks; inside a
// band the row block runs fastest.  With band_blocks = 1 the column tile runs
// fastest: the CTAs of a wave share W (small) and each row block of A is used
// by neighbouring CTAs.  A vocabulary-wide W (dozens of column tiles) does not
// stay in L2 next to the C it produces; with a band of 64 row blocks the CTAs of
// one wave share the band's rows of A and two or three column tiles, and W is
// streamed from HBM once per band rather than once per row block (measured at
// 32768 x 32000 x 768: 1.93 ms -> 1.70 ms; bands of 16 / 32 / 128: 1.83 / 1.76 / 1.82).
constexpr uint32_t kWideBandBlocks = 64;
constexpr uint32_t kWideTilesN = 32;
__device__ __forceinline__ void TileCoord(uint32_t t, uint32_t tiles_m, uint32_t tiles_n, uint32_t band_blocks,
                                          uint32_t* m_block, uint32_t* n_block) {
  const uint32_t per_band = band_blocks * tiles_n;
  const uint32_t band = t / per_band, within = t - band * per_band;
  const uint32_t first = band * band_blocks;
  const uint32_t height = tiles_m - first < band_blocks ? tiles_m - first : band_blocks;
  const uint32_t nb = within / height;
  *m_block = first + (within - nb * height);
  *n_block = nb;
}

struct __align__(8) PBarriers {
  uint64_t full[kPMaxStages];
  uint64_t empty[kPMaxStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  volatile uint32_t abort;
};

// kSideLoads: the epilogue reads a second [M, N] f32 operand beside every output
// (an addend, or the x of an absorbed backward activation).  Those loads are
// then software-pipelined: the four of the NEXT group of rows are in flight
// while this group is converted and stored, across passes and from before the
// wait for the accumulator, so a memory round trip is not paid per group with
// every warp of the CTA waiting on it.
template <bool kSideLoads, uint32_t kTN, bool kPair>
__global__ void __launch_bounds__(kPThreads, 1)
UmmaGemmPersistentKernel(const __grid_constant__ CUtensorMap map_a,
                         const __grid_constant__ CUtensorMap map_b,
                         const __grid_constant__ CUtensorMap map_a2,
                         const __grid_constant__ CUtensorMap map_b2, UmmaEpilogue ep,
                         uint32_t band_blocks) {
  using T = PTile<kTN, kPair>;
  constexpr uint32_t kPStages = T::kStages, kPStageBytes = T::kStageBytes, kPTmemCols = T::kTmemCols;
  constexpr uint32_t kColsPerEpiWarp = T::kColsPerEpiWarp, kEpiPasses = T::kEpiPasses;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (SmemAddr(smem_raw) & 1023u)) & 1023u);
  uint8_t* slabs = smem + kPStages * kPStageBytes;
  PBarriers* bars = reinterpret_cast<PBarriers*>(slabs + kPEpiWarps * kSlabBytes);

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t main_blocks = (ep.K + kBlockK - 1) / kBlockK;
  const uint32_t k_blocks = main_blocks + ep.aux_k_blocks;   // then the low-rank term's blocks
  const uint32_t tiles_n = (ep.N + kTN - 1) / kTN;
  const uint32_t tiles_m = (ep.M + T::kRowsPerTile - 1) / T::kRowsPerTile;
  const uint32_t total_tiles = tiles_m * tiles_n;
  // A work unit is a CTA, or a CTA pair: `unit` walks the tiles, `cta_rank` is this CTA's half of a pair's tile.
  const uint32_t cta_rank = kPair ? ClusterCtaRank() : 0u;
  const uint32_t unit = kPair ? blockIdx.x >> 1 : blockIdx.x, units = kPair ? gridDim.x >> 1 : gridDim.x;

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < kPStages; ++s) {
      MbarInit(&bars->full[s], 1);
      MbarInit(&bars->empty[s], 1);
    }
    for (uint32_t b = 0; b < 2; ++b) {
      MbarInit(&bars->tmem_full[b], 1);
      // one arrival per epilogue warp (of both CTAs of a pair: the even CTA's barrier counts them all)
      MbarInit(&bars->tmem_empty[b], kPair ? 2 * kPEpiWarps : kPEpiWarps);
    }
    bars->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    if constexpr (kPair) {
      TmemAllocPair(const_cast<uint32_t*>(&bars->tmem_base), kPTmemCols);
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                   ::"r"(SmemAddr(&bars->tmem_base)), "r"(kPTmemCols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if constexpr (kPair) ClusterSync();   // the peer's barriers exist before anything signals them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ---- TMA producer ----
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (uint32_t t = unit; t < total_tiles && ok; t += units) {
        uint32_t mb, nb;
        TileCoord(t, tiles_m, tiles_n, band_blocks, &mb, &nb);
        const uint32_t m0 = mb * T::kRowsPerTile + cta_rank * kBlockM, n0 = nb * kTN;
        // Ask L2 for the A rows of this CTA's next tile now, so that its loads
        // find them there instead of paying an HBM round trip inside the ring.
        if (t + units < total_tiles && k_blocks <= 64) {   // (a long K would only thrash L2)
          uint32_t next_mb, next_nb;
          TileCoord(t + units, tiles_m, tiles_n, band_blocks, &next_mb, &next_nb);
          const uint32_t next_m0 = next_mb * T::kRowsPerTile + cta_rank * kBlockM;
          if (next_m0 != m0)
            for (uint32_t kb = 0; kb < main_blocks; ++kb)
              asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];"
                           ::"l"(reinterpret_cast<uint64_t>(&map_a)),
                             "r"(static_cast<int32_t>(kb * kBlockK)), "r"(static_cast<int32_t>(next_m0))
                           : "memory");
        }
        for (uint32_t kb = 0; kb < k_blocks; ++kb, ++it) {
          const uint32_t s = it % kPStages, round = it / kPStages;
          if (round > 0 && !MbarWait(&bars->empty[s], (round - 1) & 1)) {
            ep.status->wait_timeout = 1;
            bars->abort = 1;
            ok = false;
            break;
          }
          uint8_t* a_dst = smem + s * kPStageBytes;
          const bool aux = kb >= main_blocks;
          const CUtensorMap* ma = aux ? &map_a2 : &map_a;
          const CUtensorMap* mb_ = aux ? &map_b2 : &map_b;
          const int32_t kx = static_cast<int32_t>((aux ? kb - main_blocks : kb) * kBlockK);
          if constexpr (kPair) {
            // Both CTAs' bytes are counted on the even CTA's barrier, which alone expects them.
            if (cta_rank == 0) MbarExpectTx(&bars->full[s], 2 * kPStageBytes);
            const uint32_t full_bar = MapToCta(SmemAddr(&bars->full[s]), 0);
            TmaLoad2DPair(a_dst, ma, full_bar, kx, static_cast<int32_t>(m0));
            TmaLoad2DPair(a_dst + kATileBytes, mb_, full_bar, kx, static_cast<int32_t>(n0 + cta_rank * kBlockN));
          } else {
            MbarExpectTx(&bars->full[s], kPStageBytes);
            TmaLoad2D(a_dst, ma, &bars->full[s], kx, static_cast<int32_t>(m0));
            // B's rows as 128-row boxes, back to back: one [kTN][64] tile.
            TmaLoad2D(a_dst + kATileBytes, mb_, &bars->full[s], kx, static_cast<int32_t>(n0));
            if constexpr (kTN == 256)
              TmaLoad2D(a_dst + kATileBytes + kBTileBytes, mb_, &bars->full[s], kx,
                        static_cast<int32_t>(n0 + kBlockN));
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ----
    if (lane == 0 && cta_rank == 0) {   // (a pair's odd CTA issues nothing: its memories are read by the even one's MMAs)
      const uint32_t idesc = MakeInstrDesc(T::kRowsPerTile, kTN);
      uint32_t it = 0, lt = 0;
      bool ok = true;
      for (uint32_t t = unit; t < total_tiles && ok; t += units, ++lt) {
        const uint32_t buf = lt & 1, use = lt >> 1;
        if (use > 0 && !MbarWait(&bars->tmem_empty[buf], (use - 1) & 1)) {
          ep.status->wait_timeout = 1;
          bars->abort = 1;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t acc = tmem_base + buf * kTN;
        for (uint32_t kb = 0; kb < k_blocks; ++kb, ++it) {
          const uint32_t s = it % kPStages, round = it / kPStages;
          if (!MbarWait(&bars->full[s], round & 1)) {
            ep.status->wait_timeout = 1;
            bars->abort = 1;
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = SmemAddr(smem + s * kPStageBytes);
          const uint64_t desc_a = MakeSmemDesc(a_addr);
          const uint64_t desc_b = MakeSmemDesc(a_addr + kATileBytes);
#pragma unroll
          for (uint32_t k = 0; k < kBlockK / kUmmaK; ++k) {
            if constexpr (kPair) UmmaBf16Pair(acc, desc_a + 2 * k, desc_b + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
            else UmmaBf16(acc, desc_a + 2 * k, desc_b + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          if constexpr (kPair) UmmaCommitPair(&bars->empty[s]);
          else UmmaCommit(&bars->empty[s]);
        }
        // accumulator complete (or abandoned on timeout)
        if constexpr (kPair) UmmaCommitPair(&bars->tmem_full[buf]);
        else UmmaCommit(&bars->tmem_full[buf]);
      }
    }
  } else {
    // ---- epilogue warps.  TMEM lane quarter = warp % 4 (the hardware's rule);
    // the warps of a quarter split the tile's 256 columns between them.
    const uint32_t quarter = warp & 3, col_group = (warp - 2) >> 2;
    float* slab = reinterpret_cast<float*>(slabs + (warp - 2) * kSlabBytes);
    constexpr uint32_t kChunks = kSlabCols / 4;          // 16-byte chunks per slab row
    constexpr uint32_t kRowsPerInstr = 32 / kChunks;     // rows one store instruction covers
    const uint32_t sub = lane / kChunks, cl = lane % kChunks;
    uint32_t lt = 0;
    for (uint32_t t = unit; t < total_tiles; t += units, ++lt) {
      const uint32_t buf = lt & 1, use = lt >> 1;
      uint32_t mb, nb;
      TileCoord(t, tiles_m, tiles_n, band_blocks, &mb, &nb);
      const uint32_t m0 = mb * T::kRowsPerTile + cta_rank * kBlockM, n0 = nb * kTN;
      if (ep.fuse_mode == kFuseActBwd) {
        // The absorbed backward activation reads x[m, n] next to every output:
        // ask L2 for this warp's lines of the NEXT tile now (one 128-byte line per
        // lane and pass), a whole tile ahead of the loads that use them.
        auto prefetch_x = [&](uint32_t tile) {
          uint32_t pmb, pnb;
          TileCoord(tile, tiles_m, tiles_n, band_blocks, &pmb, &pnb);
          const uint32_t prow = pmb * T::kRowsPerTile + cta_rank * kBlockM + quarter * 32 + lane;
          if (prow >= ep.M) return;
#pragma unroll
          for (uint32_t pass = 0; pass < kEpiPasses; ++pass) {
            const uint32_t pcol = pnb * kTN + col_group * kColsPerEpiWarp + pass * kSlabCols;
            if (pcol < ep.N)
              asm volatile("prefetch.global.L2 [%0];" ::"l"(ep.fuse_x + static_cast<size_t>(prow) * ep.N + pcol));
          }
        };
        if (lt == 0) prefetch_x(t);
        if (t + units < total_tiles) prefetch_x(t + units);
      }
      const uint32_t row0 = m0 + quarter * 32;
      const uint32_t rows = row0 < ep.M ? (ep.M - row0 < 32 ? ep.M - row0 : 32) : 0;
      [[maybe_unused]] const float* side_ptr = ep.fuse_mode == kFuseActBwd ? ep.fuse_x : ep.addend;
      [[maybe_unused]] const bool gelu_grad_only = IsGeluGradOnly(ep);
      [[maybe_unused]] const bool addend_only = IsAddendOnly(ep);
      [[maybe_unused]] const bool bias_gelu_only = IsBiasGeluOnly(ep);
      [[maybe_unused]] const bool copy_only = IsCopyOnly(ep);
      [[maybe_unused]] const bool plain_store = IsPlainStore(ep);
      [[maybe_unused]] float4 side_a[4], side_b[4];
      if constexpr (kSideLoads) {   // the first group's loads fly during the wait for the accumulator
        const uint32_t n_g = n0 + col_group * kColsPerEpiWarp + cl * 4;
#pragma unroll
        for (uint32_t u = 0; u < 4; ++u) {
          const uint32_t rr = sub + u * kRowsPerInstr;
          side_a[u] = rr < rows && n_g < ep.N
                          ? __ldg(reinterpret_cast<const float4*>(side_ptr + static_cast<size_t>(row0 + rr) * ep.N + n_g))
                          : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
      bool ok = MbarWait(&bars->tmem_full[buf], use & 1);
      if (!ok && lane == 0) { ep.status->wait_timeout = 1; bars->abort = 1; }
      if (bars->abort) ok = false;
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // 32 columns at a time through the slab.  A thread writes its accumulator
      // row as eight 16-byte chunks, chunk index XOR-ed with the row; the warp
      // then reads four rows per instruction (eight lanes each): whole 128-byte
      // lines of C per store instruction.  Conflict-free both ways.
      const uint32_t t_row = tmem_base + ((quarter * 32) << 16) + buf * kTN + col_group * kColsPerEpiWarp;
      if constexpr (!kSideLoads) {
  #pragma unroll 1
        for (uint32_t pass = 0; pass < kEpiPasses; ++pass) {
          uint32_t ra[32];
          TmemLoad32(t_row + pass * kSlabCols, ra);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (pass == kEpiPasses - 1) {
            // The accumulator buffer is read out: hand it back before the slow part.
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
              if constexpr (kPair)
                MbarArriveCluster(MapToCta(SmemAddr(&bars->tmem_empty[buf]), 0));
              else
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];"
                             ::"r"(SmemAddr(&bars->tmem_empty[buf])) : "memory");
            }
          }
  #pragma unroll
          for (uint32_t q = 0; q < kChunks; ++q)
            *reinterpret_cast<uint4*>(slab + lane * kSlabCols + ((q ^ (lane & (kChunks - 1))) * 4)) =
                make_uint4(ra[4 * q], ra[4 * q + 1], ra[4 * q + 2], ra[4 * q + 3]);
          __syncwarp();
          const uint32_t n = n0 + col_group * kColsPerEpiWarp + pass * kSlabCols + cl * 4;
          if (n < ep.N) {   // N % 4 == 0: a float4 is all in or all out
            float4 scale = make_float4(ep.alpha, ep.alpha, ep.alpha, ep.alpha);
            if (ep.col_scale) scale = __ldg(reinterpret_cast<const float4*>(ep.col_scale + n));
            float4 bias = make_float4(0.f, 0.f, 0.f, 0.f);
            if (ep.bias) bias = __ldg(reinterpret_cast<const float4*>(ep.bias + n));
            float4 kscale = make_float4(1.f, 1.f, 1.f, 1.f);   // the consumer's per-column factor (x * 1 == x)
            if (ep.fuse_mode != kFuseNone && ep.shadow_k_scale)
              kscale = __ldg(reinterpret_cast<const float4*>(ep.shadow_k_scale + n));
  #pragma unroll 4
            for (uint32_t rr = sub; rr < rows; rr += kRowsPerInstr) {
              const float4 acc = *reinterpret_cast<const float4*>(
                  slab + rr * kSlabCols + ((cl ^ (rr & (kChunks - 1))) * 4));
              const size_t at = static_cast<size_t>(row0 + rr) * ep.N + n;
              if (plain_store)
                EpilogueStorePlain(ep, at, acc, scale);
              else if (copy_only)
                EpilogueStoreCopy(ep, at, acc, scale);
              else if (bias_gelu_only)
                EpilogueStoreBiasGelu(ep, at, acc, scale, bias, kscale);
              else
                EpilogueStore(ep, at, n, acc, scale, bias, true, kscale);
            }
          }
          __syncwarp();   // the slab is rewritten next
        }
      } else {
        // Groups of four row steps (two per pass); group g + 1's side operands are
        // loaded while group g is converted and stored.
        auto load_group = [&](float4 (&dst)[4], uint32_t grp) {
          const uint32_t n_g = n0 + col_group * kColsPerEpiWarp + (grp >> 1) * kSlabCols + cl * 4;
#pragma unroll
          for (uint32_t u = 0; u < 4; ++u) {
            const uint32_t rr = sub + ((grp & 1) * 4 + u) * kRowsPerInstr;
            dst[u] = rr < rows && n_g < ep.N
                         ? __ldg(reinterpret_cast<const float4*>(side_ptr + static_cast<size_t>(row0 + rr) * ep.N + n_g))
                         : make_float4(0.f, 0.f, 0.f, 0.f);
          }
        };
#pragma unroll
        for (uint32_t pass = 0; pass < kEpiPasses; ++pass) {
          uint32_t ra[32];
          TmemLoad32(t_row + pass * kSlabCols, ra);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (pass == kEpiPasses - 1) {
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
              if constexpr (kPair)
                MbarArriveCluster(MapToCta(SmemAddr(&bars->tmem_empty[buf]), 0));
              else
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];"
                             ::"r"(SmemAddr(&bars->tmem_empty[buf])) : "memory");
            }
          }
#pragma unroll
          for (uint32_t q = 0; q < kChunks; ++q)
            *reinterpret_cast<uint4*>(slab + lane * kSlabCols + ((q ^ (lane & (kChunks - 1))) * 4)) =
                make_uint4(ra[4 * q], ra[4 * q + 1], ra[4 * q + 2], ra[4 * q + 3]);
          __syncwarp();
          const uint32_t n = n0 + col_group * kColsPerEpiWarp + pass * kSlabCols + cl * 4;
          float4 scale = make_float4(ep.alpha, ep.alpha, ep.alpha, ep.alpha);
          float4 bias = make_float4(0.f, 0.f, 0.f, 0.f);
          float4 kscale = make_float4(1.f, 1.f, 1.f, 1.f);
          if (n < ep.N) {
            if (ep.col_scale) scale = __ldg(reinterpret_cast<const float4*>(ep.col_scale + n));
            if (ep.bias) bias = __ldg(reinterpret_cast<const float4*>(ep.bias + n));
            if (ep.fuse_mode != kFuseNone && ep.shadow_k_scale)
              kscale = __ldg(reinterpret_cast<const float4*>(ep.shadow_k_scale + n));
          }
          auto process = [&](const float4 (&sv)[4], uint32_t half) {
#pragma unroll
            for (uint32_t u = 0; u < 4; ++u) {
              const uint32_t rr = sub + (half * 4 + u) * kRowsPerInstr;
              if (rr < rows && n < ep.N) {
                const float4 acc = *reinterpret_cast<const float4*>(
                    slab + rr * kSlabCols + ((cl ^ (rr & (kChunks - 1))) * 4));
                const size_t at = static_cast<size_t>(row0 + rr) * ep.N + n;
                if (gelu_grad_only)
                  EpilogueStoreGeluGrad(ep, at, acc, scale, kscale, sv[u]);
                else if (addend_only)
                  EpilogueStoreAddend(ep, at, acc, scale, sv[u]);
                else
                  EpilogueStore(ep, at, n, acc, scale, bias, true, kscale, true, sv[u]);
              }
            }
          };
          load_group(side_b, 2 * pass + 1);
          process(side_a, 0);
          if (pass + 1 < kEpiPasses) load_group(side_a, 2 * pass + 2);
          process(side_b, 1);
          __syncwarp();   // the slab is rewritten next
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if constexpr (kPair) ClusterSync();   // neither CTA leaves while the other may still read its memories
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if constexpr (kPair) {
      TmemFreePair(tmem_base, kPTmemCols);
    } else {
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                   "r"(kPTmemCols)
                   : "memory");
    }
  }
}

// Weight conversion to the K-major bf16 layout [N][K] the kernel consumes.
// transpose = true: src is [K][N] (the NN forms); false: src is [N][K].
template <typename T> __device__ __forceinline__ uint16_t ToBf16Bits(T v);
template <> __device__ __forceinline__ uint16_t ToBf16Bits<int8_t>(int8_t v) {
  return static_cast<uint16_t>(__float_as_uint(static_cast<float>(v)) >> 16);  // exact
}
template <> __device__ __forceinline__ uint16_t ToBf16Bits<uint16_t>(uint16_t v) { return v; }
template <> __device__ __forceinline__ uint16_t ToBf16Bits<float>(float f) {
  uint32_t b = __float_as_uint(f);
  if ((b & 0x7FFFFFFFu) > 0x7F800000u) return static_cast<uint16_t>((b >> 16) | 0x0040u);
  b += 0x7FFFu + ((b >> 16) & 1u);
  return static_cast<uint16_t>(b >> 16);
}

template <typename T> __device__ __forceinline__ float WidenWeight(T v);
template <> __device__ __forceinline__ float WidenWeight<int8_t>(int8_t v) { return static_cast<float>(v); }
template <> __device__ __forceinline__ float WidenWeight<uint16_t>(uint16_t v) {
  return __uint_as_float(static_cast<uint32_t>(v) << 16);
}
template <> __device__ __forceinline__ float WidenWeight<float>(float v) { return v; }
template <typename T>
__device__ __forceinline__ uint16_t WeightBits(T v, const float* k_scale, uint32_t k) {
  return k_scale ? ToBf16Bits<float>(WidenWeight<T>(v) * k_scale[k]) : ToBf16Bits<T>(v);
}

template <typename T>
__global__ void WeightToBf16Kernel(const T* __restrict__ src, uint16_t* __restrict__ dst, uint32_t N,
                                   uint32_t K, bool transpose, const float* __restrict__ k_scale) {
  __shared__ uint16_t tile[32][33];
  const uint32_t bx = blockIdx.x * 32, by = blockIdx.y * 32;
  if (!transpose) {  // src [N][K] -> dst [N][K]
    for (uint32_t i = threadIdx.y; i < 32; i += blockDim.y) {
      const uint32_t n = by + i, k = bx + threadIdx.x;
      if (n < N && k < K)
        dst[static_cast<size_t>(n) * K + k] = WeightBits<T>(src[static_cast<size_t>(n) * K + k], k_scale, k);
    }
    return;
  }
  // src [K][N]: bx indexes n, by indexes k
  for (uint32_t i = threadIdx.y; i < 32; i += blockDim.y) {
    const uint32_t k = by + i, n = bx + threadIdx.x;
    if (k < K && n < N) tile[i][threadIdx.x] = WeightBits<T>(src[static_cast<size_t>(k) * N + n], k_scale, k);
  }
  __syncthreads();
  for (uint32_t i = threadIdx.y; i < 32; i += blockDim.y) {
    const uint32_t n = bx + i, k = by + threadIdx.x;
    if (k < K && n < N) dst[static_cast<size_t>(n) * K + k] = tile[threadIdx.x][i];
  }
}

}  // namespace

size_t UmmaSmemBytes() { return kStages * kStageBytes + sizeof(Barriers) + 1024; }
template <uint32_t kTN, bool kPair>
static size_t UmmaPersistentSmemBytes() {
  using T = PTile<kTN, kPair>;
  return T::kStages * T::kStageBytes + kPEpiWarps * kSlabBytes + sizeof(PBarriers) + 1024;
}

template <bool kSideLoads, uint32_t kTN, bool kPair>
static cudaError_t ConfigurePersistent() {
  return cudaFuncSetAttribute(UmmaGemmPersistentKernel<kSideLoads, kTN, kPair>,
                              cudaFuncAttributeMaxDynamicSharedMemorySize,
                              static_cast<int>(UmmaPersistentSmemBytes<kTN, kPair>()));
}

// A launch with an optional cluster dimension (2 for the CTA-pair form).
// (Programmatic dependent launches — the next kernel's set-up run beside this
// one's tail — were measured on the whole step and cost 1 %: not used.)
template <typename... KArgs, typename... Args>
static cudaError_t LaunchClustered(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                   unsigned cluster, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = cluster > 1 ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

template <uint32_t kTN>
static cudaError_t LaunchPersistent(uint32_t grid, bool side_loads, const CUtensorMap& map_a, const CUtensorMap& map_b,
                                    const CUtensorMap& map_a2, const CUtensorMap& map_b2, const UmmaEpilogue& ep,
                                    uint32_t band, cudaStream_t s) {
  const size_t smem = UmmaPersistentSmemBytes<kTN, false>();
  if (side_loads)
    return LaunchClustered(UmmaGemmPersistentKernel<true, kTN, false>, dim3(grid), dim3(kPThreads), smem, s, 1u, map_a,
                           map_b, map_a2, map_b2, ep, band);
  return LaunchClustered(UmmaGemmPersistentKernel<false, kTN, false>, dim3(grid), dim3(kPThreads), smem, s, 1u, map_a,
                         map_b, map_a2, map_b2, ep, band);
}

// The CTA-pair form: clusters of two, an even grid.
static cudaError_t LaunchPairs(uint32_t grid, bool side_loads, const CUtensorMap& map_a, const CUtensorMap& map_b,
                               const CUtensorMap& map_a2, const CUtensorMap& map_b2, const UmmaEpilogue& ep,
                               uint32_t band, cudaStream_t s) {
  const size_t smem = UmmaPersistentSmemBytes<256, true>();
  if (side_loads)
    return LaunchClustered(UmmaGemmPersistentKernel<true, 256, true>, dim3(grid & ~1u), dim3(kPThreads), smem, s, 2u,
                           map_a, map_b, map_a2, map_b2, ep, band);
  return LaunchClustered(UmmaGemmPersistentKernel<false, 256, true>, dim3(grid & ~1u), dim3(kPThreads), smem, s, 2u,
                         map_a, map_b, map_a2, map_b2, ep, band);
}

static std::atomic<bool> g_cta_pairs{true};
void UmmaSetCtaPairs(bool on) { g_cta_pairs.store(on, std::memory_order_relaxed); }

cudaError_t UmmaGemmLaunch(const CUtensorMap& map_a, const CUtensorMap& map_b,
                           const UmmaEpilogue& ep, cudaStream_t s, const CUtensorMap* aux_a,
                           const CUtensorMap* aux_b) {
  // Without a low-rank term the second pair of maps is never dereferenced; the
  // main pair stands in so that the parameters are valid descriptors.
  const CUtensorMap& map_a2 = ep.aux_k_blocks && aux_a ? *aux_a : map_a;
  const CUtensorMap& map_b2 = ep.aux_k_blocks && aux_b ? *aux_b : map_b;
  // The shared-memory limit of a kernel is a per-device attribute: one flag per
  // device, so a second backend on another GPU of the same process configures its own.
  static std::atomic<bool> configured_on[64] = {};
  static int sm_count[64] = {};
  const size_t smem = UmmaSmemBytes();
  int dev = 0;
  cudaGetDevice(&dev);
  const bool tracked = dev >= 0 && dev < 64;
  if (!tracked || !configured_on[dev].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(UmmaGemmKernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    if ((e = ConfigurePersistent<false, 256, false>()) != cudaSuccess) return e;
    if ((e = ConfigurePersistent<true, 256, false>()) != cudaSuccess) return e;
    if ((e = ConfigurePersistent<false, 128, false>()) != cudaSuccess) return e;
    if ((e = ConfigurePersistent<true, 128, false>()) != cudaSuccess) return e;
    if ((e = ConfigurePersistent<false, 256, true>()) != cudaSuccess) return e;
    if ((e = ConfigurePersistent<true, 256, true>()) != cudaSuccess) return e;
    if (tracked) configured_on[dev].store(true, std::memory_order_release);
  }
  if (dev >= 0 && dev < 64 && sm_count[dev] == 0)
    cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
  const uint32_t sms = (dev >= 0 && dev < 64 && sm_count[dev] > 0) ? sm_count[dev] : 148;
  const uint32_t tiles_n = (ep.N + kBlockN - 1) / kBlockN, tiles_m = (ep.M + kBlockM - 1) / kBlockM;
  const uint32_t ptiles_n = (ep.N + kPBlockN - 1) / kPBlockN;
  const uint64_t wide = static_cast<uint64_t>(ptiles_n) * tiles_m, narrow = static_cast<uint64_t>(tiles_n) * tiles_m;
  const bool side_loads = ep.addend != nullptr || ep.fuse_mode == kFuseActBwd;
  if (wide > 2ull * sms) {
    // Enough tiles for every SM to amortise its set-up over several.
    const uint32_t band = ptiles_n >= kWideTilesN ? kWideBandBlocks : 1u;
    // CTA pairs where the reduction is long: measured at 32768 rows, K = 3072 and 32000 gain 9-10 % (a third
    // less operand traffic per flop), while at K = 768 the epilogue sets the pace and a pair's two epilogues,
    // which must both finish before the accumulator buffer is free again, cost 5-15 % where they are heavy.
    if (g_cta_pairs.load(std::memory_order_relaxed) && sms >= 2 && ep.K >= 1536)
      return LaunchPairs(sms, side_loads, map_a, map_b, map_a2, map_b2, ep, band > 1 ? band / 2 : 1u, s);
    return LaunchPersistent<256>(sms, side_loads, map_a, map_b, map_a2, map_b2, ep, band, s);
  }
  if (narrow >= sms / 2) {
    // A shard-sized product: the persistent kernel's staged, coalesced epilogue on
    // whichever tile width finishes first, counted in rounds of 128 columns (plus
    // a quarter tile of fixed cost per round).
    const uint64_t wide_cost = ((wide + sms - 1) / sms) * (256 + 32);
    const uint64_t narrow_cost = ((narrow + sms - 1) / sms) * (128 + 32);
    if (wide_cost <= narrow_cost)
      return LaunchPersistent<256>(static_cast<uint32_t>(wide < sms ? wide : sms), side_loads, map_a, map_b, map_a2,
                                   map_b2, ep, 1u, s);
    return LaunchPersistent<128>(static_cast<uint32_t>(narrow < sms ? narrow : sms), side_loads, map_a, map_b, map_a2,
                                 map_b2, ep, 1u, s);
  }
  dim3 grid(tiles_n, tiles_m);
  return LaunchClustered(UmmaGemmKernel, grid, dim3(kThreads), smem, s, 1u, map_a, map_b, map_a2, map_b2, ep);
}

void WeightToBf16(const void* src, BType type, uint16_t* dst, uint32_t N, uint32_t K,
                  bool transpose, const float* k_scale, cudaStream_t s) {
  dim3 block(32, 8);
  dim3 grid = transpose ? dim3((N + 31) / 32, (K + 31) / 32) : dim3((K + 31) / 32, (N + 31) / 32);
  switch (type) {
    case BType::kI8:
      WeightToBf16Kernel<int8_t><<<grid, block, 0, s>>>(static_cast<const int8_t*>(src), dst, N, K, transpose, k_scale);
      break;
    case BType::kBf16:
      WeightToBf16Kernel<uint16_t><<<grid, block, 0, s>>>(static_cast<const uint16_t*>(src), dst, N, K, transpose, k_scale);
      break;
    case BType::kF32:
      WeightToBf16Kernel<float><<<grid, block, 0, s>>>(static_cast<const float*>(src), dst, N, K, transpose, k_scale);
      break;
  }
}

}  // namespace see::k
