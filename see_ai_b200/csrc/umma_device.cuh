// Device-side building blocks shared by the tcgen05 kernels: mbarriers with
// bounded waits, TMA tile loads/stores, shared-memory and instruction
// descriptors for K-major bf16 operands under the 128-byte swizzle, the MMA
// issue / commit wrappers and tensor-memory loads.
#ifndef SEE_CUDA_UMMA_DEVICE_CUH_
#define SEE_CUDA_UMMA_DEVICE_CUH_

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace see::k::umma_dev {

constexpr uint32_t kWaitLimit = 1u << 22;

__device__ __forceinline__ uint32_t SmemAddr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void MbarInit(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(SmemAddr(bar)), "r"(count));
}
__device__ __forceinline__ void MbarInitFence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void MbarExpectTx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(SmemAddr(bar)),
               "r"(bytes)
               : "memory");
}
// Bounded wait: false when the limit ran out (the caller raises the status flag
// and stops issuing work; nothing here spins forever).
__device__ __forceinline__ bool MbarWait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = SmemAddr(bar);
  for (uint32_t it = 0; it < kWaitLimit; ++it) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

__device__ __forceinline__ void TmaLoad2D(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                          int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];"
      ::"r"(SmemAddr(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(SmemAddr(bar)), "r"(x),
      "r"(y)
      : "memory");
}
__device__ __forceinline__ void TmaLoad3D(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                          int32_t x, int32_t y, int32_t z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(SmemAddr(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(SmemAddr(bar)), "r"(x),
      "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void TmaLoad4D(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                          int32_t x, int32_t y, int32_t z, int32_t w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(SmemAddr(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(SmemAddr(bar)), "r"(x),
      "r"(y), "r"(z), "r"(w)
      : "memory");
}
// Tile store shared -> global; rows/columns outside the tensor are clipped.
__device__ __forceinline__ void TmaStore2D(const CUtensorMap* map, const void* smem_src, int32_t x,
                                           int32_t y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(SmemAddr(smem_src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void TmaStoreCommit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void TmaStoreWaitRead() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void TmaStoreWaitAll() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// Make generic-proxy shared-memory writes visible to the async proxy (TMA, tcgen05.mma).
__device__ __forceinline__ void FenceProxyAsync() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Shared-memory matrix descriptor, K-major, 128-byte swizzle: start address
// (>>4), leading byte offset 1 (unused for swizzled K-major), stride byte offset
// 1024 (eight 128-byte rows per swizzle atom), descriptor version 1, layout
// type 2 (SWIZZLE_128B).  Advancing K by 16 bf16 inside a 128-byte row adds 32
// bytes to the start address: +2 in the encoded field.
__device__ __forceinline__ uint64_t MakeSmemDesc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// The same for an MN-major operand under the 128-byte swizzle: the tile is stored
// [k][64 elements of M or N] (128-byte rows, one per k, eight of them per 1024-byte
// swizzle atom) — what a TMA load of a row-major [rows = k][columns = n] tensor
// leaves.  Stride byte offset 1024 (from one group of eight k to the next), leading
// byte offset = the distance between successive 64-element groups along M / N.
// Advancing K by 16 adds 16 rows = 2048 bytes to the start address.
__device__ __forceinline__ uint64_t MakeSmemDescMn(uint32_t smem_addr, uint32_t group_stride_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>((group_stride_bytes >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
constexpr uint32_t kInstrDescBMnMajor = 1u << 16;   // OR into MakeInstrDesc: B is MN-major

// Instruction descriptor for kind::f16: D = f32, A = B = bf16, both K-major.
__device__ __forceinline__ uint32_t MakeInstrDesc(uint32_t m, uint32_t n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

__device__ __forceinline__ void UmmaBf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void UmmaCommit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(SmemAddr(bar))
               : "memory");
}
// ---- CTA pairs (cta_group::2): two CTAs of a cluster, one 256-row tile ---------------------
// The even CTA of the pair (cluster rank 0) issues every MMA; each CTA's shared
// memory holds its own 128 rows of A and its own half of B's rows, each CTA's
// tensor memory receives its own 128 rows of the product.
__device__ __forceinline__ uint32_t ClusterCtaRank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The shared::cluster address of `local` (a shared::cta address) in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t MapToCta(uint32_t local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}
__device__ __forceinline__ void ClusterSync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// A tile load whose completion bytes are counted on a barrier of the pair's even CTA
// (`bar_cluster_addr`: a shared::cluster address); the data lands in the executing
// CTA's own shared memory only.
__device__ __forceinline__ void TmaLoad2DPair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                              int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];"
      ::"r"(SmemAddr(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void UmmaBf16Pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One arrival on the barrier at this shared-memory offset in BOTH CTAs of the pair
// once the MMAs issued so far are complete: one commit per CTA, each naming that
// CTA's barrier by its shared::cluster address.
__device__ __forceinline__ void UmmaCommitPair(uint64_t* bar) {
  const uint32_t local = SmemAddr(bar);
#pragma unroll
  for (uint32_t rank = 0; rank < 2; ++rank)
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(MapToCta(local, rank))
                 : "memory");
}
__device__ __forceinline__ void MbarArriveCluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void TmemAllocPair(uint32_t* smem_slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
               ::"r"(SmemAddr(smem_slot)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void TmemFreePair(uint32_t base, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
}

__device__ __forceinline__ void TcFenceBefore() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void TcFenceAfter() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void TmemWaitLd() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Whole-warp calls.
__device__ __forceinline__ void TmemAlloc(uint32_t* smem_slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
               ::"r"(SmemAddr(smem_slot)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void TmemFree(uint32_t base, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
}

// 32 consecutive f32 columns of this thread's TMEM lane.
__device__ __forceinline__ void TmemLoad32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}

// The inverse: 32 consecutive f32 columns of this thread's TMEM lane written from registers.
__device__ __forceinline__ void TmemStore32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
        "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]),
        "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void TmemWaitSt() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ uint32_t PackBf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// Byte offset of the 16-byte chunk `chunk` (0..7) of row `row` inside a
// [rows][64 bf16] sub-tile stored with the 128-byte swizzle TMA and tcgen05 use.
__device__ __forceinline__ uint32_t Sw128Offset(uint32_t row, uint32_t chunk) {
  return (row >> 3) * 1024u + (row & 7u) * 128u + ((chunk ^ (row & 7u)) << 4);
}

}  // namespace see::k::umma_dev

#endif  // SEE_CUDA_UMMA_DEVICE_CUH_
