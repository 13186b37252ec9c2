#include "umma_gemm.h"

#include <cuda.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <map>
#include <set>
#include <tuple>
#include <vector>

#include "attn_umma.h"
#include "lora_umma.h"
#include "umma_kernel.h"

namespace see::umma {

namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// A cached K-major bf16 copy of a frozen weight: key = (space, byte offset,
// N, K, transposed source, element type, byte offset of the per-k factor
// folded into it or ~0).
using WeightKey = std::tuple<int, uint64_t, uint64_t, uint64_t, bool, int, uint64_t>;

struct ActCopy {   // a bf16 copy of an arena activation [M, K]
  uint64_t a_off = ~0ull, scale_off = ~0ull, M = 0, K = 0;
  bool valid = false;
  bool reserved = false;   // handed to a producer (ReserveShadow) and not yet committed
  uint16_t* buf = nullptr;
  uint64_t capacity = 0;  // elements
  uint64_t last_use = 0;
};

constexpr int kActSlots = 8;

// The bf16 copy of one attention operand (a Q, K, V or dO activation) in the
// tensor's own row-major layout [B*S, H*d], which the kernels' 4-D tensor maps cut
// (sequence, head) tiles out of.  Made
// once, by one kernel, the first time any attention instruction of the range
// reads the operand; the forward's copies serve the backward of the same step
// unless an instruction overwrote the source in between.
struct PackEntry {
  uint16_t* rows = nullptr;
  uint64_t src_off = ~0ull, elems = 0;
  bool valid = false;
  uint64_t last_use = 0;
};

}  // namespace

struct Impl {
  int device = 0;
  EncodeTiledFn encode = nullptr;
  std::map<WeightKey, uint16_t*> weights;
  ActCopy acts[kActSlots];
  uint64_t tick = 0;
  k::DeviceStatus* status = nullptr;  // the backend's device status block (not owned)
  std::vector<PackEntry> packs;
  uint64_t pack_capacity = 0;   // elements per layout of an entry
  cudaEvent_t prof_before = nullptr, prof_after = nullptr;
  bool prof_used = false;
  // bf16 pieces of the operands of exact f32 products (TrySplitGemm)
  uint16_t* split_a = nullptr;
  uint16_t* split_b = nullptr;
  uint64_t split_a_capacity = 0, split_b_capacity = 0;   // elements
  std::map<WeightKey, uint16_t*> split_weights;          // frozen B operands, once per binding
};

std::string Init(Context* ctx, int device, k::DeviceStatus* status) {
  auto* impl = new Impl;
  impl->device = device;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres{};
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) {
    delete impl;
    return "cuda: the driver does not provide cuTensorMapEncodeTiled (TMA descriptors)";
  }
  impl->encode = reinterpret_cast<EncodeTiledFn>(fn);
  impl->status = status;
  ctx->impl = impl;
  return {};
}

void Destroy(Context* ctx) {
  if (!ctx->impl) return;
  InvalidateAll(ctx);
  for (auto& a : ctx->impl->acts) cudaFree(a.buf);
  for (auto& e : ctx->impl->packs) cudaFree(e.rows);
  cudaFree(ctx->impl->split_a);
  cudaFree(ctx->impl->split_b);
  delete ctx->impl;
  ctx->impl = nullptr;
}

void InvalidateAll(Context* ctx) {
  if (!ctx->impl) return;
  for (auto& [key, buf] : ctx->impl->weights) cudaFree(buf);
  ctx->impl->weights.clear();
  for (auto& [key, buf] : ctx->impl->split_weights) cudaFree(buf);
  ctx->impl->split_weights.clear();
  for (auto& a : ctx->impl->acts) a.valid = false;
  for (auto& e : ctx->impl->packs) e.valid = false;
}

void InvalidateRange(Context* ctx, uint64_t off, uint64_t bytes) {
  if (!ctx->impl) return;
  for (auto& a : ctx->impl->acts) {
    if (!a.valid) continue;
    const uint64_t a_bytes = a.M * a.K * 4;
    if (off < a.a_off + a_bytes && a.a_off < off + bytes) a.valid = false;
  }
  for (auto& e : ctx->impl->packs)
    if (e.valid && off < e.src_off + e.elems * 4 && e.src_off < off + bytes) e.valid = false;
}

// Sizes every activation-copy slot for the largest relaxed GEMM of the range
// before the range starts, so no allocation (and no stream drain) can fall
// between its instructions — a requirement for replaying the range as a graph.
void PlanRange(Context* ctx, const Instruction* program, size_t begin, size_t end) {
  Impl* impl = ctx->impl;
  if (!impl) return;
  uint64_t need = 0;
  for (size_t i = begin; i < end; ++i) {
    const Instruction& ins = program[i];
    if (!(ins.flags & kFlagRelaxed)) continue;
    switch (ins.opcode) {
      case kGemmNN: case kGemmNT: case kGemmNNQ8: case kGemmNTQ8: case kGemmNNBF16: case kGemmNTBF16:
        need = std::max(need, ins.out[0] * ins.out[2]);
        break;
      default: break;
    }
  }
  // Attention operands: one pack entry per distinct source of the range, within
  // a budget of one eighth of the device's memory (least recently used entries
  // are recycled beyond that), never fewer than the four one instruction needs.
  uint64_t attn = 0;
  std::set<uint64_t> sources;
  for (size_t i = begin; i < end; ++i) {
    const Instruction& ins = program[i];
    if (!(ins.flags & kFlagRelaxed)) continue;
    if (ins.opcode == kAttnFwdTiled) {
      attn = std::max(attn, Hi32(ins.out[1]) * Lo32(ins.out[1]) * Hi32(ins.out[2]) * Lo32(ins.out[2]));
      for (int j = 0; j < 3; ++j) sources.insert(ins.in[j]);
    }
    if (ins.opcode == kAttnDQTiled || ins.opcode == kAttnDKTiled || ins.opcode == kAttnDVTiled) {
      const AttnGeom g = UnpackAttnGeom(ins.out[2]);
      attn = std::max(attn, g.B * g.S * g.H * g.d);
      for (int j = 0; j < 4; ++j) sources.insert(ins.in[j]);
    }
  }
  if (attn > 0) {
    size_t free_b = 0, total_b = 0;
    cudaMemGetInfo(&free_b, &total_b);
    const uint64_t per_entry = attn * 2;   // bf16
    const uint64_t by_budget = std::max<uint64_t>(4, (total_b / 8) / per_entry);
    const size_t want = static_cast<size_t>(
        std::min<uint64_t>(std::max<uint64_t>(4, sources.size()), by_budget));
    if (attn > impl->pack_capacity || want > impl->packs.size()) {
      cudaDeviceSynchronize();
      const uint64_t cap = std::max(attn, impl->pack_capacity);
      if (attn > impl->pack_capacity) {
        for (auto& e : impl->packs) cudaFree(e.rows);
        impl->packs.clear();
      }
      while (impl->packs.size() < want) {
        PackEntry e;
        void* pr = nullptr;
        if (cudaMalloc(&pr, cap * 2) != cudaSuccess) {
          cudaGetLastError();
          break;
        }
        e.rows = static_cast<uint16_t*>(pr);
        impl->packs.push_back(e);
      }
      impl->pack_capacity = cap;
    }
  }
  if (need == 0) return;
  bool drained = false;
  for (auto& slot : impl->acts) {
    if (slot.capacity >= need) continue;
    if (!drained) { cudaDeviceSynchronize(); drained = true; }
    cudaFree(slot.buf);
    slot.buf = nullptr;
    slot.capacity = 0;
    slot.valid = false;
    void* p = nullptr;
    if (cudaMalloc(&p, need * 2) == cudaSuccess) {
      slot.buf = static_cast<uint16_t*>(p);
      slot.capacity = need;
    }
  }
}

static bool EncodeBf16Map(Impl* impl, CUtensorMap* map, const void* base, uint64_t rows,
                          uint64_t cols, uint32_t box_rows) {
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {k::umma_cfg::kBlockK, box_rows};
  const cuuint32_t elem[2] = {1, 1};
  return impl->encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                      strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static bool EncodeF32Map(Impl* impl, CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                         uint32_t box_rows) {
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 4};
  const cuuint32_t box[2] = {128, box_rows};   // plain row-major in shared memory: the kernel re-tiles it itself
  const cuuint32_t elem[2] = {1, 1};
  return impl->encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, elem,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

std::string TryLoraBackward(Context* ctx, const k::LoraBackwardArgs& a, cudaStream_t stream, int* launches) {
  *launches = 0;
  Impl* impl = ctx->impl;
  if (!impl || !k::LoraBackwardUmmaEnabled() || !k::LoraBackwardUmmaSupported(a.M, a.N, a.K, a.r)) return {};
  auto misaligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; };
  if (misaligned(a.dy) || misaligned(a.x) || misaligned(a.t) || misaligned(a.B) || misaligned(a.dt) ||
      misaligned(a.partials) || misaligned(a.dt_pieces))
    return {};
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) return {};
  const int blocks = k::LoraBackwardUmmaBlocks(a.M, sms);
  if (static_cast<size_t>(blocks) * (a.r * a.N + a.K * a.r) > a.partials_floats) return {};
  CUtensorMap map_dy, map_x, map_b;
  if (!EncodeF32Map(impl, &map_dy, a.dy, a.M, a.N, 64) || !EncodeF32Map(impl, &map_x, a.x, a.M, a.K, 64) ||
      !EncodeF32Map(impl, &map_b, a.B, a.r, a.N, 16))
    return "tensor-core adapter backward: cuTensorMapEncodeTiled refused an operand layout";
  if (k::LoraBackwardUmmaLaunch(map_dy, map_x, map_b, a, blocks, impl->status, stream) != cudaSuccess)
    return "tensor-core adapter backward: launch failed";
  k::LoraFoldPartials(a, blocks, stream);
  *launches = 2;
  return {};
}

std::string TryGemm(Context* ctx, const k::GemmArgs& a, int b_space, uint64_t b_off,
                    uint64_t a_off, uint64_t a_scale_off, cudaStream_t stream, int* launches) {
  *launches = 0;
  Impl* impl = ctx->impl;
  if (!impl) return {};
  // The kernel's domain: K a multiple of 8 (16-byte global strides for TMA), N a
  // multiple of 4 (float4 stores), enough rows to fill a 128-row tile, no
  // transposed A, no accumulate form.  Anything else runs on the exact kernels.
  if (a.a_transposed || a.accumulate) return {};
  if (a.K % 8 != 0 || a.N % 4 != 0 || a.K < 64 || a.N < 16 || a.M < 64) return {};
  if (a.M > 0xFFFFFFFFull || a.N > 0xFFFFFFFFull || a.K > 0xFFFFFFFFull) return {};
  auto misaligned = [](const void* p) { return p && (reinterpret_cast<uintptr_t>(p) & 15) != 0; };
  if (misaligned(a.C) || misaligned(a.addend) || misaligned(a.bias) || misaligned(a.b_col_scale))
    return {};   // the epilogue moves float4s

  // ---- the weight, K-major bf16 [N][K], converted once per binding ----
  // A transposed int8 product's per-k factor (C = (A s_k) W^T) is folded into the
  // weight copy, w[n][k] = bf16(W[n][k] * s[k]), once per binding: the activation
  // copy is then plain bf16(A), which every producer can write without a table
  // look-up per element, and which any other consumer of the tensor can share.
  const WeightKey key{b_space, b_off, a.N, a.K, !a.b_transposed, static_cast<int>(a.b_type),
                      a.a_k_scale ? a_scale_off : ~0ull};
  uint16_t* w = nullptr;
  if (auto it = impl->weights.find(key); it != impl->weights.end()) {
    w = it->second;
  } else {
    void* p = nullptr;
    if (cudaMalloc(&p, a.N * a.K * 2) != cudaSuccess) return "tensor-core path: weight copy allocation failed";
    w = static_cast<uint16_t*>(p);
    k::WeightToBf16(a.B, a.b_type, w, static_cast<uint32_t>(a.N), static_cast<uint32_t>(a.K),
                    /*transpose=*/!a.b_transposed, a.a_k_scale, stream);
    ++*launches;
    impl->weights.emplace(key, w);
  }

  // ---- the activation, bf16 [M][K], reused while its arena range is unwritten ----
  ActCopy* slot = nullptr;
  for (auto& c : impl->acts)
    if (c.valid && c.a_off == a_off && c.scale_off == ~0ull && c.M == a.M && c.K == a.K)
      slot = &c;
  if (!slot) {
    // A slot a producer is writing (this product's own epilogue, when it has
    // absorbed a following activation) is not a candidate.
    for (auto& c : impl->acts) {
      if (c.reserved) continue;
      if (!c.valid) { slot = &c; break; }
      if (!slot || c.last_use < slot->last_use) slot = &c;
    }
    if (!slot) return "tensor-core path: no activation copy slot free";
    const uint64_t need = a.M * a.K;
    if (slot->capacity < need) {
      // Replacing the buffer: queued kernels may still read the old one.
      cudaStreamSynchronize(stream);
      cudaFree(slot->buf);
      slot->buf = nullptr;
      slot->capacity = 0;
      void* p = nullptr;
      if (cudaMalloc(&p, need * 2) != cudaSuccess) return "tensor-core path: activation copy allocation failed";
      slot->buf = static_cast<uint16_t*>(p);
      slot->capacity = need;
    }
    k::ToBf16(a.A, slot->buf, a.M, a.K, nullptr, stream);
    ++*launches;
    slot->a_off = a_off; slot->scale_off = ~0ull; slot->M = a.M; slot->K = a.K;
    slot->valid = true;
  }
  slot->last_use = ++impl->tick;

  CUtensorMap map_a, map_b, aux_a, aux_b;
  if (!EncodeBf16Map(impl, &map_a, slot->buf, a.M, a.K, k::umma_cfg::kBlockM) ||
      !EncodeBf16Map(impl, &map_b, w, a.N, a.K, k::umma_cfg::kBlockN))
    return "tensor-core path: cuTensorMapEncodeTiled refused the operand layout";
  const bool has_aux = a.aux_a && a.aux_b && a.aux_k >= 64 && a.aux_k % 64 == 0;
  if (has_aux && (!EncodeBf16Map(impl, &aux_a, a.aux_a, a.M, a.aux_k, k::umma_cfg::kBlockM) ||
                  !EncodeBf16Map(impl, &aux_b, a.aux_b, a.N, a.aux_k, k::umma_cfg::kBlockN)))
    return "tensor-core path: cuTensorMapEncodeTiled refused the low-rank operand layout";

  k::UmmaEpilogue ep{};
  ep.C = a.C;
  ep.addend = a.addend;
  ep.bias = a.bias;
  ep.col_scale = a.b_col_scale;
  ep.alpha = a.alpha;
  ep.act = static_cast<int>(a.act);
  ep.M = static_cast<uint32_t>(a.M);
  ep.N = static_cast<uint32_t>(a.N);
  ep.K = static_cast<uint32_t>(a.K);
  ep.status = impl->status;
  ep.fuse_mode = a.fuse_mode;
  ep.fuse_act = static_cast<int>(a.fuse_act);
  ep.fuse_x = a.fuse_x;
  ep.shadow_dst = a.fuse_shadow;
  ep.shadow_k_scale = a.fuse_shadow_scale;
  ep.pack_dst = a.pack_dst;
  ep.store_c = a.store_c ? 1 : 0;
  ep.addend_last = a.addend_after_bias ? 1 : 0;
  ep.aux_k_blocks = has_aux ? a.aux_k / 64 : 0;
  if (impl->prof_before) cudaEventRecord(impl->prof_before, stream);
  if (cudaError_t e = k::UmmaGemmLaunch(map_a, map_b, ep, stream, has_aux ? &aux_a : nullptr,
                                        has_aux ? &aux_b : nullptr);
      e != cudaSuccess)
    return std::string("tensor-core GEMM launch: ") + cudaGetErrorString(e);
  if (impl->prof_after) {
    cudaEventRecord(impl->prof_after, stream);
    impl->prof_used = true;
    impl->prof_before = impl->prof_after = nullptr;
  }
  ++*launches;
  return {};
}

bool SplitGemmEligible(const k::GemmArgs& a) {
  if (a.b_type != k::BType::kF32 || a.accumulate || a.b_col_scale || a.a_k_scale) return false;
  if (a.M < 128 || a.N < 64 || a.K < 64 || (a.N & 3) != 0 || (a.K & 3) != 0) return false;
  if (a.M * a.N * a.K < (1ull << 26)) return false;   // below ~0.1 GFLOP a launch is latency either way
  if (a.M > 0x7FFFFFFFull || a.N > 0x7FFFFFFFull || 6 * a.K > 0x7FFFFFFFull) return false;
  auto misaligned = [](const void* p) { return p && (reinterpret_cast<uintptr_t>(p) & 15) != 0; };
  return !(misaligned(a.A) || misaligned(a.B) || misaligned(a.C) || misaligned(a.addend) || misaligned(a.bias));
}

static bool GrowSplit(uint16_t** buf, uint64_t* cap, uint64_t need, cudaStream_t stream, bool whole_device = false) {
  if (need <= *cap) return true;
  // Queued kernels may still read the old buffer.
  if (whole_device) cudaDeviceSynchronize(); else cudaStreamSynchronize(stream);
  cudaFree(*buf);
  *buf = nullptr;
  *cap = 0;
  void* p = nullptr;
  if (cudaMalloc(&p, need * 2) != cudaSuccess) { cudaGetLastError(); return false; }
  *buf = static_cast<uint16_t*>(p);
  *cap = need;
  return true;
}

void PlanSplitGemms(Context* ctx, const Instruction* program, size_t begin, size_t end) {
  Impl* impl = ctx->impl;
  if (!impl) return;
  uint64_t need_a = 0, need_b = 0;
  for (size_t i = begin; i < end; ++i) {
    const Instruction& ins = program[i];
    if (ins.opcode != kGemmNN && ins.opcode != kGemmNT && ins.opcode != kGemmTN) continue;
    const uint64_t M = ins.out[0], N = ins.out[1], K = ins.out[2];
    if (M < 128 || N < 64 || K < 64 || M * N * K < (1ull << 26)) continue;
    need_a = std::max(need_a, M * 6 * K);
    if (RefSpace(ins.in[1]) == kArena) need_b = std::max(need_b, N * 6 * K);
  }
  GrowSplit(&impl->split_a, &impl->split_a_capacity, need_a, nullptr, true);
  GrowSplit(&impl->split_b, &impl->split_b_capacity, need_b, nullptr, true);
}

std::string TrySplitGemm(Context* ctx, const k::GemmArgs& a, int b_space, uint64_t b_off,
                         cudaStream_t stream, int* launches) {
  *launches = 0;
  Impl* impl = ctx->impl;
  if (!impl || !SplitGemmEligible(a)) return {};
  const uint64_t K6 = 6 * a.K;
  if (!GrowSplit(&impl->split_a, &impl->split_a_capacity, a.M * K6, stream))
    return "tensor-core path: operand-piece allocation failed";
  // A: [M, K], or [K, M] for the transposed-A form.
  k::SplitMatrix(a.A, impl->split_a, a.M, a.K, a.a_transposed, 0, stream);
  ++*launches;
  // B: wanted as [N][K]; stored [N, K] (NT) or [K, N] (NN, TN).
  uint16_t* b = nullptr;
  if (b_space != 0) {   // frozen: once per binding
    const WeightKey key{b_space, b_off, a.N, a.K, !a.b_transposed, 100, ~0ull};
    if (auto it = impl->split_weights.find(key); it != impl->split_weights.end()) {
      b = it->second;
    } else {
      void* p = nullptr;
      if (cudaMalloc(&p, a.N * K6 * 2) != cudaSuccess) return "tensor-core path: weight-piece allocation failed";
      b = static_cast<uint16_t*>(p);
      k::SplitMatrix(static_cast<const float*>(a.B), b, a.N, a.K, !a.b_transposed, 1, stream);
      ++*launches;
      impl->split_weights.emplace(key, b);
    }
  } else {
    if (!GrowSplit(&impl->split_b, &impl->split_b_capacity, a.N * K6, stream))
      return "tensor-core path: operand-piece allocation failed";
    b = impl->split_b;
    k::SplitMatrix(static_cast<const float*>(a.B), b, a.N, a.K, !a.b_transposed, 1, stream);
    ++*launches;
  }
  CUtensorMap map_a, map_b;
  if (!EncodeBf16Map(impl, &map_a, impl->split_a, a.M, K6, k::umma_cfg::kBlockM) ||
      !EncodeBf16Map(impl, &map_b, b, a.N, K6, k::umma_cfg::kBlockN))
    return "tensor-core path: cuTensorMapEncodeTiled refused the operand-piece layout";
  k::UmmaEpilogue ep{};
  ep.C = a.C;
  ep.addend = a.addend;
  ep.bias = a.bias;
  ep.col_scale = nullptr;
  ep.alpha = a.alpha;   // (the exact kernels fold alpha into A or the finished dot; here it scales the tile)
  ep.act = static_cast<int>(a.act);
  ep.M = static_cast<uint32_t>(a.M);
  ep.N = static_cast<uint32_t>(a.N);
  ep.K = static_cast<uint32_t>(K6);
  ep.status = impl->status;
  if (impl->prof_before) cudaEventRecord(impl->prof_before, stream);
  if (cudaError_t e = k::UmmaGemmLaunch(map_a, map_b, ep, stream); e != cudaSuccess)
    return std::string("tensor-core GEMM launch: ") + cudaGetErrorString(e);
  if (impl->prof_after) {
    cudaEventRecord(impl->prof_after, stream);
    impl->prof_used = true;
    impl->prof_before = impl->prof_after = nullptr;
  }
  ++*launches;
  return {};
}

bool TouchActCopy(Context* ctx, uint64_t a_off, uint64_t a_scale_off, uint64_t M, uint64_t K) {
  Impl* impl = ctx->impl;
  if (!impl) return false;
  for (auto& c : impl->acts)
    if (c.valid && c.a_off == a_off && c.scale_off == a_scale_off && c.M == M && c.K == K) {
      c.last_use = ++impl->tick;
      return true;
    }
  return false;
}

void ReleaseReservations(Context* ctx) {
  if (!ctx->impl) return;
  for (auto& c : ctx->impl->acts) c.reserved = false;
}

uint16_t* ReserveShadow(Context* ctx, uint64_t elems, bool keep_reserved) {
  Impl* impl = ctx->impl;
  if (!impl) return nullptr;
  ActCopy* slot = nullptr;
  for (auto& c : impl->acts) {
    if (!keep_reserved) c.reserved = false;   // normally one reservation at a time
    if (c.reserved || c.capacity < elems || !c.buf) continue;
    if (!c.valid) { slot = &c; break; }
    if (!slot || c.last_use < slot->last_use) slot = &c;
  }
  if (!slot) return nullptr;
  slot->valid = false;
  slot->reserved = true;
  slot->last_use = ++impl->tick;   // not the next victim while its producer runs
  return slot->buf;
}

void CommitShadow(Context* ctx, uint16_t* buf, uint64_t a_off, uint64_t a_scale_off, uint64_t M,
                  uint64_t K) {
  Impl* impl = ctx->impl;
  if (!impl || !buf) return;
  for (auto& c : impl->acts) {
    if (c.buf != buf) continue;
    c.a_off = a_off; c.scale_off = a_scale_off; c.M = M; c.K = K;
    c.valid = true;
    c.reserved = false;
    c.last_use = ++impl->tick;
  }
}

namespace {

// {d, S, H, B} over a row-major bf16 [B*S, H*d] tensor: a box is 64 head-dimension elements
// of `box_rows` positions of one head of one sequence.
bool EncodeHeads(Impl* impl, CUtensorMap* map, const void* base, uint64_t d, uint64_t S, uint64_t H, uint64_t B,
                 uint32_t box_rows) {
  const cuuint64_t dims[4] = {d, S, H, B};
  const cuuint64_t strides[3] = {H * d * 2, d * 2, S * H * d * 2};
  const cuuint32_t box[4] = {64, box_rows, 1, 1};
  const cuuint32_t elem[4] = {1, 1, 1, 1};
  return impl->encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims,
                      strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

std::string TryAttention(Context* ctx, uint16_t opcode, const AttentionOperands& op,
                         cudaStream_t stream, int* launches, bool* did_second) {
  if (did_second) *did_second = false;
  *launches = 0;
  Impl* impl = ctx->impl;
  if (!impl) return {};
  if ((op.d != 64 && op.d != 128) || op.S % 8 != 0 || op.S < 16 || op.S > 0x7FFFFFFF ||
      op.B * op.H > 65535 || op.B * op.H == 0)
    return {};
  if ((reinterpret_cast<uintptr_t>(op.out) & 15) || (reinterpret_cast<uintptr_t>(op.stats) & 15))
    return {};
  const uint64_t elems = op.B * op.S * op.H * op.d;
  if (elems > impl->pack_capacity) return {};   // executed outside a planned range
  if (impl->packs.size() < 4) return "tensor-core attention: packed-operand allocation failed";
  const bool fwd = opcode == kAttnFwdTiled, dq = opcode == kAttnDQTiled,
             dk = opcode == kAttnDKTiled, dv = opcode == kAttnDVTiled;
  if (!fwd && !dq && !dk && !dv) return {};
  enum { Q = 0, K = 1, V = 2, DO = 3 };
  const float* src[4] = {op.q, op.k, op.v, op.dout};
  const uint64_t off[4] = {op.q_off, op.k_off, op.v_off, op.dout_off};
  bool used[4] = {true, true, true, !fwd};
  if (dv) used[V] = false;
  for (int r = 0; r < 4; ++r)
    if (used[r] && (reinterpret_cast<uintptr_t>(src[r]) & 15)) return {};
  const uint64_t now = ++impl->tick;
  PackEntry* ent[4] = {nullptr, nullptr, nullptr, nullptr};
  for (int r = 0; r < 4; ++r) {
    if (!used[r]) continue;
    for (auto& e : impl->packs)
      if (e.valid && e.src_off == off[r] && e.elems == elems) { ent[r] = &e; break; }
    if (ent[r]) { ent[r]->last_use = now; continue; }
    PackEntry* victim = nullptr;
    for (auto& e : impl->packs) {
      if (e.last_use == now) continue;   // taken by this instruction
      if (!e.valid) { victim = &e; break; }
      if (!victim || e.last_use < victim->last_use) victim = &e;
    }
    if (!victim) return "tensor-core attention: no pack entry free";
    k::PackHeads(src[r], victim->rows, static_cast<uint32_t>(op.B),
                 static_cast<uint32_t>(op.S), static_cast<uint32_t>(op.H),
                 static_cast<uint32_t>(op.d), stream);
    ++*launches;
    victim->valid = true;
    victim->src_off = off[r];
    victim->elems = elems;
    victim->last_use = now;
    ent[r] = victim;
  }
  CUtensorMap mr[4], mh[4];   // rows (box 128), rows (box 64)
  for (int r = 0; r < 4; ++r) {
    if (!used[r]) continue;
    if (!EncodeHeads(impl, &mr[r], ent[r]->rows, op.d, op.S, op.H, op.B, 128) ||
        !EncodeHeads(impl, &mh[r], ent[r]->rows, op.d, op.S, op.H, op.B, 64))
      return "tensor-core attention: cuTensorMapEncodeTiled refused a row layout";
  }
  k::AttnUmmaArgs a{};
  a.B = static_cast<uint32_t>(op.B); a.S = static_cast<uint32_t>(op.S);
  a.H = static_cast<uint32_t>(op.H); a.d = static_cast<uint32_t>(op.d);
  a.inv_sqrt_d = 1.0f / std::sqrt(static_cast<float>(op.d));
  a.out = op.out;
  a.stats = op.stats;
  a.status = impl->status;
  a.shadow = op.shadow;
  cudaError_t e = cudaSuccess;
  if (fwd) {
    a.keep = op.keep;
    e = k::AttnFwdUmma(mr[Q], mh[K], mh[V], a, stream);
    a.keep = nullptr;
  }
  if (dq) {
    if (op.fwd_keep) {
      a.fwd_keep = op.fwd_keep;
      a.dout_bf16 = ent[DO]->rows;
    }
    e = k::AttnDQUmma(mr[Q], mr[DO], mh[K], mh[V], a, stream);
    a.fwd_keep = nullptr;
    a.dout_bf16 = nullptr;
  }
  const bool both = dk && op.out2 != nullptr && op.d == 64 &&
                    (reinterpret_cast<uintptr_t>(op.out2) & 15) == 0;
  if (both) {
    a.out2 = op.out2;
    a.shadow2 = op.shadow2;
  }
  if (dk) e = k::AttnDKVUmma(both ? 2 : 1, mr[K], mr[V], mh[Q], mh[DO], a, stream);
  if (dv) e = k::AttnDKVUmma(0, mr[K], mr[K], mh[Q], mh[DO], a, stream);
  if (both && e == cudaSuccess && did_second) *did_second = true;
  if (e != cudaSuccess) return std::string("tensor-core attention launch: ") + cudaGetErrorString(e);
  ++*launches;
  return {};
}

uint16_t* ReservePack(Context* ctx, uint64_t elems) {
  Impl* impl = ctx->impl;
  if (!impl || elems > impl->pack_capacity) return nullptr;
  PackEntry* victim = nullptr;
  for (auto& e : impl->packs) {
    if (!e.valid) { victim = &e; break; }
    if (!victim || e.last_use < victim->last_use) victim = &e;
  }
  if (!victim) return nullptr;
  victim->valid = false;
  victim->last_use = ++impl->tick;
  return victim->rows;
}

bool TouchPack(Context* ctx, uint64_t src_off, uint64_t elems) {
  Impl* impl = ctx->impl;
  if (!impl) return false;
  for (auto& e : impl->packs)
    if (e.valid && e.src_off == src_off && e.elems == elems) {
      e.last_use = ++impl->tick;
      return true;
    }
  return false;
}

void CommitPack(Context* ctx, uint16_t* rows, uint64_t src_off, uint64_t elems) {
  Impl* impl = ctx->impl;
  if (!impl || !rows) return;
  for (auto& e : impl->packs) {
    if (e.rows == rows) {
      e.valid = true;
      e.src_off = src_off;
      e.elems = elems;
      e.last_use = ++impl->tick;
    } else if (e.valid && e.src_off == src_off) {
      e.valid = false;   // an older copy of the same tensor
    }
  }
}

void SetProfileEvents(Context* ctx, cudaEvent_t before, cudaEvent_t after) {
  if (!ctx->impl) return;
  ctx->impl->prof_before = before;
  ctx->impl->prof_after = after;
  ctx->impl->prof_used = false;
}

bool ProfileEventsUsed(Context* ctx) {
  if (!ctx->impl) return false;
  const bool used = ctx->impl->prof_used;
  ctx->impl->prof_used = false;
  ctx->impl->prof_before = ctx->impl->prof_after = nullptr;
  return used;
}

}  // namespace see::umma
