#include "cuda_backend.h"

#include <algorithm>
#include <cmath>
#include <cstring>

#include "umma_gemm.h"

namespace see {

namespace {

constexpr int kScalarSlots = 64;

std::string CudaErr(cudaError_t e, const char* what) {
  return std::string("cuda: ") + what + ": " + cudaGetErrorString(e);
}

void MergeExtent(std::vector<std::pair<uint64_t, uint64_t>>* list, uint64_t off, uint64_t bytes) {
  if (bytes == 0) return;
  for (auto& r : *list) {
    if (off <= r.first + r.second && r.first <= off + bytes) {  // overlap or touch
      const uint64_t b = std::min(off, r.first);
      const uint64_t e = std::max(off + bytes, r.first + r.second);
      r = {b, e - b};
      return;
    }
  }
  list->push_back({off, bytes});
}

}  // namespace

struct CudaBackend::UmmaState {
  umma::Context ctx;
};

CudaBackend::CudaBackend(int device) : device_(device) {}

std::expected<std::unique_ptr<CudaBackend>, std::string> CudaBackend::Create(int device_ordinal) {
  std::unique_ptr<CudaBackend> b(new CudaBackend(device_ordinal));
  if (auto r = b->Init(); !r) return std::unexpected(r.error());
  return b;
}

Status CudaBackend::Check(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return {};
  return std::unexpected(CudaErr(e, what));
}

Status CudaBackend::Init() {
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0)
    return std::unexpected("cuda: no CUDA device is visible — this backend has no CPU fallback");
  if (device_ < 0 || device_ >= count)
    return std::unexpected("cuda: device ordinal " + std::to_string(device_) + " out of range");
  if (auto r = Check(cudaSetDevice(device_), "cudaSetDevice"); !r) return r;
  cudaDeviceProp prop{};
  if (auto r = Check(cudaGetDeviceProperties(&prop, device_), "cudaGetDeviceProperties"); !r)
    return r;
  if (prop.major != 10)
    return std::unexpected(std::string("cuda: device '") + prop.name +
                           "' is not compute capability 10.x; the kernels are built for sm_100a only");
  device_label_ = std::string(prop.name) + " (sm_" + std::to_string(prop.major) +
                  std::to_string(prop.minor) + ", " + std::to_string(prop.multiProcessorCount) +
                  " SMs), relaxed GEMMs on tcgen05 bf16 tensor cores";
  if (auto r = Check(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking), "stream"); !r)
    return r;
  own_stream_ = true;
  void* p = nullptr;
  const size_t scratch_bytes = 4096 + 256 * sizeof(double);
  if (auto r = Check(cudaMalloc(&p, scratch_bytes), "scratch"); !r) return r;
  if (auto r = Check(cudaMemset(p, 0, scratch_bytes), "scratch memset"); !r) return r;
  uint8_t* base = static_cast<uint8_t*>(p);
  d_status_ = reinterpret_cast<k::DeviceStatus*>(base);
  d_sq_ = reinterpret_cast<double*>(base + 64);
  d_clip_scale_ = reinterpret_cast<float*>(base + 128);
  d_count_ = reinterpret_cast<unsigned long long*>(base + 192);
  d_scalars_ = reinterpret_cast<k::AdamScalars*>(base + 256);
  d_partials_ = reinterpret_cast<double*>(base + 4096);
  if (auto r = Check(cudaMallocHost(reinterpret_cast<void**>(&h_scalars_),
                                    kScalarSlots * sizeof(k::AdamScalars)), "pinned scalars"); !r)
    return r;
  if (auto r = Check(cudaMallocHost(reinterpret_cast<void**>(&h_status_), 64), "pinned status"); !r)
    return r;
  std::memset(h_status_, 0, 64);
  scalar_done_.assign(kScalarSlots, nullptr);
  for (auto& ev : scalar_done_)
    if (auto r = Check(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), "scalar events"); !r) return r;
  umma_ = std::make_unique<UmmaState>();
  if (std::string e = umma::Init(&umma_->ctx, device_, d_status_); !e.empty()) return std::unexpected(e);
  return {};
}

CudaBackend::~CudaBackend() {
  cudaSetDevice(device_);
  if (stream_) cudaStreamSynchronize(stream_);
  for (auto& ev : events_) { cudaEventDestroy(ev.first); cudaEventDestroy(ev.second); }
  for (auto& ev : kernel_events_) { cudaEventDestroy(ev.first); cudaEventDestroy(ev.second); }
  for (auto& ev : scalar_done_) if (ev) cudaEventDestroy(ev);
  if (umma_) umma::Destroy(&umma_->ctx);
  cudaFree(d_arena_);
  cudaFree(d_rodata_);
  cudaFree(d_source_);
  cudaFree(d_status_);  // base of the scratch block
  cudaFree(d_rows_);
  cudaFree(d_gsum_);
  cudaFree(d_colmax_);
  cudaFree(d_split_);
  cudaFree(d_adam_table_);
  FreeLoraRanges();
  cudaFree(d_lora_t_);
  for (float* p : attn_keep_pool_) cudaFree(p);
  cudaFree(d_lora_partials_);
  if (h_scalars_) cudaFreeHost(h_scalars_);
  if (h_status_) cudaFreeHost(h_status_);
  if (own_stream_ && stream_) cudaStreamDestroy(stream_);
}

Status CudaBackend::Bind(uint8_t* arena, uint64_t arena_bytes, const uint8_t* rodata,
                         uint64_t rodata_bytes, uint64_t /*rodata_mapped_bytes*/) {
  if (!arena || arena_bytes == 0) return std::unexpected("cuda: bind: empty arena");
  cudaSetDevice(device_);
  // Allocate the new binding first; only when everything succeeded is the old
  // one released, so a refused Bind leaves the previous plan executable.
  void* new_arena = nullptr;
  void* new_rodata = nullptr;
  if (auto e = cudaMalloc(&new_arena, arena_bytes); e != cudaSuccess)
    return std::unexpected(CudaErr(e, "bind: arena slab"));
  if (rodata_bytes) {
    if (auto e = cudaMalloc(&new_rodata, rodata_bytes + 64); e != cudaSuccess) {
      cudaFree(new_arena);
      return std::unexpected(CudaErr(e, "bind: rodata"));
    }
    if (auto e = cudaMemcpyAsync(new_rodata, rodata, rodata_bytes, cudaMemcpyHostToDevice, stream_);
        e != cudaSuccess) {
      cudaFree(new_arena); cudaFree(new_rodata);
      return std::unexpected(CudaErr(e, "bind: rodata upload"));
    }
  }
  if (auto e = cudaMemcpyAsync(new_arena, arena, arena_bytes, cudaMemcpyHostToDevice, stream_);
      e != cudaSuccess) {
    cudaFree(new_arena); cudaFree(new_rodata);
    return std::unexpected(CudaErr(e, "bind: arena upload"));
  }
  if (auto e = cudaStreamSynchronize(stream_); e != cudaSuccess) {
    cudaFree(new_arena); cudaFree(new_rodata);
    return std::unexpected(CudaErr(e, "bind: sync"));
  }
  cudaFree(d_arena_);
  cudaFree(d_rodata_);
  d_arena_ = static_cast<uint8_t*>(new_arena);
  d_rodata_ = static_cast<uint8_t*>(new_rodata);
  host_arena_ = arena;
  arena_bytes_ = arena_bytes;
  rodata_bytes_ = rodata_bytes;
  counters_.h2d_bytes += arena_bytes + rodata_bytes;
  host_dirty_.clear();
  device_dirty_.clear();
  deferred_error_.clear();
  scalars_valid_ = false;
  umma::InvalidateAll(&umma_->ctx);
  FreeLoraRanges();
  return {};
}

Status CudaBackend::BindDeviceImage(uint64_t arena_bytes, const uint8_t* prefix,
                                    uint64_t prefix_bytes, const uint8_t* rodata,
                                    uint64_t rodata_bytes) {
  if (arena_bytes == 0 || prefix_bytes > arena_bytes)
    return std::unexpected("cuda: bind: bad arena image");
  cudaSetDevice(device_);
  void* new_arena = nullptr;
  void* new_rodata = nullptr;
  auto fail = [&](cudaError_t e, const char* what) -> Status {
    cudaFree(new_arena);
    cudaFree(new_rodata);
    return std::unexpected(CudaErr(e, what));
  };
  if (auto e = cudaMalloc(&new_arena, arena_bytes); e != cudaSuccess) return fail(e, "bind: arena slab");
  if (auto e = cudaMemsetAsync(new_arena, 0, arena_bytes, stream_); e != cudaSuccess)
    return fail(e, "bind: arena clear");
  if (prefix_bytes)
    if (auto e = cudaMemcpyAsync(new_arena, prefix, prefix_bytes, cudaMemcpyHostToDevice, stream_);
        e != cudaSuccess)
      return fail(e, "bind: persistent image upload");
  if (rodata_bytes) {
    if (auto e = cudaMalloc(&new_rodata, rodata_bytes + 64); e != cudaSuccess) return fail(e, "bind: rodata");
    if (auto e = cudaMemcpyAsync(new_rodata, rodata, rodata_bytes, cudaMemcpyHostToDevice, stream_);
        e != cudaSuccess)
      return fail(e, "bind: rodata upload");
  }
  if (auto e = cudaStreamSynchronize(stream_); e != cudaSuccess) return fail(e, "bind: sync");
  cudaFree(d_arena_);
  cudaFree(d_rodata_);
  d_arena_ = static_cast<uint8_t*>(new_arena);
  d_rodata_ = static_cast<uint8_t*>(new_rodata);
  host_arena_ = nullptr;
  arena_bytes_ = arena_bytes;
  rodata_bytes_ = rodata_bytes;
  coherence_ = Coherence::kLazy;
  counters_.h2d_bytes += prefix_bytes + rodata_bytes;
  host_dirty_.clear();
  device_dirty_.clear();
  deferred_error_.clear();
  scalars_valid_ = false;
  umma::InvalidateAll(&umma_->ctx);
  FreeLoraRanges();
  return {};
}

Status CudaBackend::ReadArena(uint64_t off, uint64_t bytes, void* dst) {
  if (!d_arena_) return std::unexpected("cuda: nothing is bound");
  if (off > arena_bytes_ || bytes > arena_bytes_ - off)
    return std::unexpected("cuda: read: range outside the arena");
  cudaSetDevice(device_);
  if (auto r = Check(cudaMemcpyAsync(dst, d_arena_ + off, bytes, cudaMemcpyDeviceToHost, stream_),
                     "read"); !r)
    return r;
  counters_.d2h_bytes += bytes;
  return Check(cudaStreamSynchronize(stream_), "read sync");
}

Status CudaBackend::WriteArena(uint64_t off, uint64_t bytes, const void* src) {
  if (!d_arena_) return std::unexpected("cuda: nothing is bound");
  if (off > arena_bytes_ || bytes > arena_bytes_ - off)
    return std::unexpected("cuda: write: range outside the arena");
  cudaSetDevice(device_);
  if (auto r = Check(cudaMemcpyAsync(d_arena_ + off, src, bytes, cudaMemcpyHostToDevice, stream_),
                     "write"); !r)
    return r;
  counters_.h2d_bytes += bytes;
  umma::InvalidateRange(&umma_->ctx, off, bytes);
  return {};
}

Status CudaBackend::BindSource(const uint8_t* data, uint64_t bytes) {
  cudaSetDevice(device_);
  cudaStreamSynchronize(stream_);
  cudaFree(d_source_);
  d_source_ = nullptr;
  source_bytes_ = 0;
  // Every bf16 weight copy made from the old source model is stale now (they are
  // keyed by offset, and a second model has the same offsets).
  umma::InvalidateAll(&umma_->ctx);
  if (!data || bytes == 0) return {};
  void* p = nullptr;
  if (auto r = Check(cudaMalloc(&p, bytes), "bind source"); !r) return r;
  if (auto r = Check(cudaMemcpy(p, data, bytes, cudaMemcpyHostToDevice), "source upload"); !r) {
    cudaFree(p);
    return r;
  }
  d_source_ = static_cast<uint8_t*>(p);
  source_bytes_ = bytes;
  counters_.h2d_bytes += bytes;
  return {};
}

void CudaBackend::HostWrote(uint64_t off, uint64_t bytes) {
  if (off >= arena_bytes_) return;
  bytes = std::min(bytes, arena_bytes_ - off);
  MergeExtent(&host_dirty_, off, bytes);
}

Status CudaBackend::UploadDirty() {
  for (const auto& [off, bytes] : host_dirty_) {
    if (auto r = Check(cudaMemcpyAsync(d_arena_ + off, host_arena_ + off, bytes,
                                       cudaMemcpyHostToDevice, stream_), "upload"); !r)
      return r;
    counters_.h2d_bytes += bytes;
  }
  host_dirty_.clear();
  return {};
}

Status CudaBackend::HostNeeds(uint64_t off, uint64_t bytes) {
  if (!d_arena_) return std::unexpected("cuda: nothing is bound");
  if (off > arena_bytes_ || bytes > arena_bytes_ - off)
    return std::unexpected("cuda: host_needs: range outside the arena");
  cudaSetDevice(device_);
  if (auto r = Check(cudaMemcpyAsync(host_arena_ + off, d_arena_ + off, bytes,
                                     cudaMemcpyDeviceToHost, stream_), "download"); !r)
    return r;
  counters_.d2h_bytes += bytes;
  return Check(cudaStreamSynchronize(stream_), "download sync");
}

void CudaBackend::SetGradientGather(int ranks, const void* gathered, uint64_t block_off,
                                    uint64_t block_bytes) {
  gather_ranks_ = ranks > 1 ? ranks : 1;
  d_gathered_ = ranks > 1 ? static_cast<const uint8_t*>(gathered) : nullptr;
  gather_off_ = block_off;
  gather_bytes_ = block_bytes;
  fold_gather_ = gather_folded_ = false;
}

Status CudaBackend::QuantizeColumns(const float* w, uint64_t K, uint64_t N, int8_t* levels, float* scales) {
  if (!w || !levels || !scales || K == 0 || N == 0) return std::unexpected("cuda: quantize: empty operand");
  cudaSetDevice(device_);
  if (N > colmax_capacity_) {
    cudaStreamSynchronize(stream_);
    cudaFree(d_colmax_);
    d_colmax_ = nullptr;
    colmax_capacity_ = 0;
    void* p = nullptr;
    if (auto r = Check(cudaMalloc(&p, N * sizeof(unsigned int)), "quantize scratch"); !r) return r;
    d_colmax_ = static_cast<unsigned int*>(p);
    colmax_capacity_ = N;
  }
  k::QuantizeColumns(w, K, N, levels, scales, d_colmax_, stream_);
  counters_.kernel_launches += 3;
  return Check(cudaPeekAtLastError(), "quantize");
}

void CudaBackend::SetProfiling(bool on) { profiling_ = on; }

std::vector<ProfileRecord> CudaBackend::TakeProfile() {
  cudaSetDevice(device_);
  cudaStreamSynchronize(stream_);
  for (size_t i = 0; i < pending_profile_.size(); ++i) {
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, events_[i].first, events_[i].second);
    pending_profile_[i].ms = ms;
    if (pending_profile_[i].has_kernel) {
      float kms = 0.0f;
      cudaEventElapsedTime(&kms, kernel_events_[i].first, kernel_events_[i].second);
      pending_profile_[i].kernel_ms = kms;
    }
  }
  std::vector<ProfileRecord> out;
  out.swap(pending_profile_);
  return out;
}

Status CudaBackend::EnsureScratch(uint64_t row_doubles) {
  if (row_doubles <= rows_capacity_) return {};
  // Growing scratch replaces the buffer: drain the stream first so no queued
  // kernel still reads the old one.
  if (auto r = Check(cudaStreamSynchronize(stream_), "scratch sync"); !r) return r;
  cudaFree(d_rows_);
  d_rows_ = nullptr;
  rows_capacity_ = 0;
  void* p = nullptr;
  if (auto r = Check(cudaMalloc(&p, row_doubles * sizeof(double)), "row scratch"); !r) return r;
  d_rows_ = static_cast<double*>(p);
  rows_capacity_ = row_doubles;
  return {};
}

void CudaBackend::BeginRange(std::span<const Instruction> program, size_t begin, size_t end) {
  // Size every scratch buffer the range needs up front, so no allocation (and
  // no stream drain) happens between its instructions.
  uint64_t rows = 0, gsum = 0, split = 0;
  fold_gather_ = gather_folded_ = false;
  range_error_.clear();
  if (gather_ranks_ > 1) {
    bool clip = false;
    for (size_t i = begin; i < end && i < program.size(); ++i) {
      const uint16_t op = program[i].opcode;
      clip = clip || op == kClipNorm || op == kSqNormAccum || op == kClipGlobal;
    }
    if (clip) {
      fold_gather_ = true;
      // The optimizer steps that consume the clipped gradient must be in this
      // range too: a later range would go back to the gathered, unclipped copies.
      for (size_t i = std::min(end, program.size()); i < program.size(); ++i)
        if (program[i].opcode == kAdamWStep || program[i].opcode == kSgdStep)
          range_error_ = "cuda: data parallel: a range with a standalone clip instruction must also hold "
                         "the optimizer steps that follow it";
    }
  }
  for (size_t i = begin; i < end && i < program.size(); ++i) {
    const Instruction& ins = program[i];
    switch (ins.opcode) {
      case kGemmTN: {
        const uint64_t chunks = k::SplitKChunks(ins.out[0], ins.out[1], ins.out[2]);
        if (chunks > 1) split = std::max(split, chunks * ins.out[0] * ins.out[1]);
        break;
      }
      case kSoftmaxXEntFwd: case kSoftmaxXEntMaskedFwd: rows = std::max(rows, ins.out[0]); break;
      case kKLDistillFwd: rows = std::max(rows, Hi32(ins.out[1])); break;
      case kMseFwd: rows = std::max<uint64_t>(rows, 256); break;
      case kAdamWStep: case kSgdStep:
        if (gather_ranks_ > 1 && !fold_gather_ && BitsToF32(ins.out[1]) > 0.0f) gsum = std::max(gsum, ins.out[0]);
        break;
      default: break;
    }
  }
  if (rows) (void)EnsureScratch(rows);
  if (split > split_capacity_) {
    cudaStreamSynchronize(stream_);
    cudaFree(d_split_);
    d_split_ = nullptr;
    split_capacity_ = 0;
    void* p = nullptr;
    if (cudaMalloc(&p, split * sizeof(float)) == cudaSuccess) {
      d_split_ = static_cast<float*>(p);
      split_capacity_ = split;
    }
  }
  if (gsum > gsum_capacity_) {
    cudaStreamSynchronize(stream_);
    cudaFree(d_gsum_);
    d_gsum_ = nullptr;
    gsum_capacity_ = 0;
    void* p = nullptr;
    if (cudaMalloc(&p, gsum * sizeof(float)) == cudaSuccess) {
      d_gsum_ = static_cast<float*>(p);
      gsum_capacity_ = gsum;
    }
  }
  umma::PlanRange(&umma_->ctx, program.data(), begin, std::min(end, program.size()));
  if (SplitGemmOn()) umma::PlanSplitGemms(&umma_->ctx, program.data(), begin, std::min(end, program.size()));
  // Cached bf16 activation copies do not outlive a range: a range replayed as a
  // CUDA graph must contain every conversion it depends on.
  umma::InvalidateRange(&umma_->ctx, 0, arena_bytes_);
  range_index_ = 0;
  lora_rows_tag_.valid = false;
  PlanAdamGroups(program, begin, std::min(end, program.size()));
  PlanAttentionKeeps(program, begin, std::min(end, program.size()));
  auto plan_fusions = [&] {
    PlanShadows(program, begin, std::min(end, program.size()));
    PlanBiasFusions(program, begin, std::min(end, program.size()));
    PlanActFusions(program, begin, std::min(end, program.size()));
    PlanAttentionPacks(program, begin, std::min(end, program.size()));
  };
  plan_fusions();
  uint64_t partial_floats = 0;
  for (size_t i = 0; i < adapter_bwd_.size(); ++i)
    if (adapter_bwd_[i].fuse)
      partial_floats = std::max<uint64_t>(partial_floats,
                                          k::LoraBackwardPartialFloats(program[begin + i].out[2], adapter_bwd_[i].da.out[0],
                                                                       program[begin + i].out[1]));
  if (partial_floats > lora_partials_capacity_) {
    cudaStreamSynchronize(stream_);
    cudaFree(d_lora_partials_);
    d_lora_partials_ = nullptr;
    lora_partials_capacity_ = 0;
    void* p = nullptr;
    if (cudaMalloc(&p, partial_floats * sizeof(float)) == cudaSuccess) {
      d_lora_partials_ = static_cast<float*>(p);
      lora_partials_capacity_ = partial_floats;
    } else {   // no scratch: the three products stay three instructions
      cudaGetLastError();
      for (size_t i = 0; i < adapter_bwd_.size(); ++i)
        if (adapter_bwd_[i].fuse) {
          adapter_bwd_[i].fuse = false;
          for (size_t q = i + 1; q < lora_skip_.size() && q <= i + 3; ++q)
            if (lora_skip_[q] == 1 && (program[begin + q].opcode == kGemmTN)) lora_skip_[q] = 0;
        }
    }
  }
  uint64_t fold_rows = 0;
  for (size_t i = 0; i < lora_fold_.size(); ++i)
    if (lora_fold_[i].fuse) fold_rows = std::max<uint64_t>(fold_rows, program[begin + i].out[0]);
  if (auto r = PrepareLoraFolds(program.data(), begin, fold_rows); !r) {   // no memory for the operands: run the plan as written
    cudaGetLastError();
    const bool enabled = lora_fold_enabled_;
    lora_fold_enabled_ = false;
    plan_fusions();   // again, without the folds (they had taken over some of the add fusions)
    lora_fold_enabled_ = enabled;
  }
}

// Device buffers and the weight table of the folds just planned.
Status CudaBackend::PrepareLoraFolds(const Instruction* program, size_t begin, uint64_t max_rows) {
  d_lora_table_ = nullptr;
  d_lora_w_ = nullptr;
  if (lora_weights_.empty()) return {};
  LoraRangeBuffers& rb = lora_ranges_[{program, begin}];
  const uint64_t w_need = static_cast<uint64_t>(lora_weights_.size()) * lora_max_n_ * lora_max_kx_;
  const uint64_t t_need = max_rows * lora_max_kx_;
  if (w_need > rb.weights_capacity || t_need > lora_t_capacity_ || lora_weights_.size() > rb.table_capacity)
    cudaStreamSynchronize(stream_);   // queued kernels may still read the old buffers
  auto grow = [&](void** buf, uint64_t* cap, uint64_t need, size_t elem) -> Status {
    if (need <= *cap) return {};
    cudaFree(*buf);
    *buf = nullptr;
    *cap = 0;
    if (auto r = Check(cudaMalloc(buf, need * elem), "low-rank fold operands"); !r) return r;
    *cap = need;
    return {};
  };
  uint64_t table_cap = rb.table_capacity;
  if (auto r = grow(reinterpret_cast<void**>(&rb.weights), &rb.weights_capacity, w_need, 2); !r) return r;
  if (auto r = grow(reinterpret_cast<void**>(&d_lora_t_), &lora_t_capacity_, t_need, 2); !r) return r;
  if (auto r = grow(reinterpret_cast<void**>(&rb.table), &table_cap, lora_weights_.size(), sizeof(k::LoraWeight));
      !r)
    return r;
  rb.table_capacity = table_cap;
  d_lora_table_ = rb.table;
  d_lora_w_ = rb.weights;
  for (size_t i = 0; i < lora_weights_.size(); ++i)
    lora_weights_[i].dst = d_lora_w_ + static_cast<uint64_t>(i) * lora_max_n_ * lora_max_kx_;
  // An earlier pass over this range may still be reading the table.
  cudaStreamSynchronize(stream_);
  return Check(cudaMemcpy(d_lora_table_, lora_weights_.data(), lora_weights_.size() * sizeof(k::LoraWeight),
                          cudaMemcpyHostToDevice), "low-rank fold table");
}

void CudaBackend::FreeLoraRanges() {
  for (auto& [key, rb] : lora_ranges_) {
    cudaFree(rb.table);
    cudaFree(rb.weights);
  }
  lora_ranges_.clear();
  d_lora_table_ = nullptr;
  d_lora_w_ = nullptr;
}

void CudaBackend::EndRange() {
  adapter_bwd_.clear();
  lora_fold_.clear();
  lora_skip_.clear();
  lora_weights_.clear();
  fold_gather_ = gather_folded_ = false;
  range_error_.clear();
  bias_fusion_.clear();
  skip_next_add_bias_ = false;
  act_fusion_.clear();
  loss_fusion_.clear();
  add_fusion_.clear();
  skip_add_at_ = -1;
  attn_dv_out_.clear();
  attn_dv_shadow_.clear();
  skip_attn_dv_at_ = -1;
  skip_act_at_ = -1;
  elided_.clear();
  pending_elided_.clear();
  deferred_elided_.clear();
  lora_rows_tag_.valid = false;
  pack_plan_.clear();
  pending_pack_ = PendingPack{};
  shadow_plan_.clear();
  adam_group_of_.clear();
  adam_groups_.clear();
}

// Consecutive AdamW instructions without a fused clip become one launch over a
// table of their tensors; the table is uploaded here, before the range (and any
// graph capture of it) starts.
void CudaBackend::PlanAdamGroups(std::span<const Instruction> program, size_t begin, size_t end) {
  adam_group_of_.assign(end > begin ? end - begin : 0, -1);
  adam_groups_.clear();
  if (coherence_ == Coherence::kStrict || end <= begin) return;
  std::vector<k::AdamTensor> table;
  for (size_t i = begin; i < end;) {
    size_t j = i;
    while (j < end && program[j].opcode == kAdamWStep && BitsToF32(program[j].out[1]) <= 0.0f &&
           program[j].out[0] > 0)
      ++j;
    if (j - i < 2) { i = j > i ? j : i + 1; continue; }
    AdamGroup grp;
    grp.table_begin = table.size();
    grp.count = static_cast<int>(j - i);
    for (size_t t = i; t < j; ++t) {
      const Instruction& ins = program[t];
      Extents ext;
      if (!DescribeInstruction(ins, arena_bytes_, rodata_bytes_, source_bytes_, &ext).empty()) {
        grp.count = 0;   // a malformed member: leave the run to the per-instruction path
        break;
      }
      k::AdamTensor e{};
      e.p = Wr(ins.in[0]); e.g = Rd(ins.in[1]); e.m = Wr(ins.in[2]); e.v = Wr(ins.in[3]);
      e.n = ins.out[0];
      e.g_copies = 1;
      const uint64_t g_off = RefOffset(ins.in[1]);
      if (gather_ranks_ > 1 && !fold_gather_ && RefSpace(ins.in[1]) == kArena && g_off >= gather_off_ &&
          g_off + e.n * 4 <= gather_off_ + gather_bytes_) {
        e.g = reinterpret_cast<const float*>(d_gathered_ + (g_off - gather_off_));
        e.g_copies = gather_ranks_;
        e.copy_stride = gather_bytes_ / 4;
      }
      grp.max_n = std::max<uint64_t>(grp.max_n, e.n);
      table.push_back(e);
    }
    if (grp.count >= 2) {
      adam_group_of_[i - begin] = static_cast<int32_t>(adam_groups_.size());
      for (size_t t = i + 1; t < j; ++t) adam_group_of_[t - begin] = -2;
      adam_groups_.push_back(grp);
    } else {
      table.resize(grp.table_begin);
    }
    i = j;
  }
  if (table.empty()) return;
  if (table.size() > adam_table_capacity_) {
    cudaStreamSynchronize(stream_);
    cudaFree(d_adam_table_);
    d_adam_table_ = nullptr;
    adam_table_capacity_ = 0;
    void* p = nullptr;
    if (cudaMalloc(&p, table.size() * sizeof(k::AdamTensor)) != cudaSuccess) {
      cudaGetLastError();
      adam_group_of_.assign(adam_group_of_.size(), -1);
      adam_groups_.clear();
      return;
    }
    d_adam_table_ = static_cast<k::AdamTensor*>(p);
    adam_table_capacity_ = table.size();
  }
  // The previous range's launches may still be reading the table.
  cudaStreamSynchronize(stream_);
  cudaMemcpy(d_adam_table_, table.data(), table.size() * sizeof(k::AdamTensor), cudaMemcpyHostToDevice);
}

namespace {

bool IsShadowProducer(uint16_t op) {
  switch (op) {
    case kAddEW: case kReluFwd: case kGeluFwd: case kSiluFwd: case kReluBwd: case kGeluBwd:
    case kSiluBwd: case kLayerNormFwd: case kSoftmaxXEntBwd: case kSoftmaxXEntMaskedBwd:
    case kAttnFwdTiled: case kAttnDQTiled: case kAttnDKTiled: case kAttnDVTiled:
      return true;
    default:
      return false;
  }
}

}  // namespace

// For every relaxed GEMM of the range whose A operand is an arena tensor, finds
// the instruction that last writes that tensor; if it writes exactly that
// tensor and can emit a bf16 copy, marks it.  Only an optimisation hint: the
// copy is published under the usual key and dies with any later write into the
// range (InvalidateRange), so a missed or spurious mark cannot change a result.
void CudaBackend::PlanShadows(std::span<const Instruction> program, size_t begin, size_t end) {
  shadow_plan_.assign(end > begin ? end - begin : 0, ShadowPlan{});
  if (!relaxed_allowed_ || end <= begin) return;
  std::vector<Extents> ext(end - begin);
  for (size_t i = begin; i < end; ++i)
    if (!DescribeInstruction(program[i], arena_bytes_, rodata_bytes_, source_bytes_, &ext[i - begin]).empty())
      ext[i - begin].count = 0;
  for (size_t j = begin; j < end; ++j) {
    const Instruction& g = program[j];
    const uint16_t op = g.opcode;
    const bool gemm = op == kGemmNN || op == kGemmNT || op == kGemmNNQ8 || op == kGemmNTQ8 ||
                      op == kGemmNNBF16 || op == kGemmNTBF16;
    if (!gemm || !(g.flags & kFlagRelaxed) || RefSpace(g.in[1]) == kArena ||
        RefSpace(g.in[0]) != kArena)
      continue;
    const uint64_t M = g.out[0], N = g.out[1], K = g.out[2];
    if (K % 8 != 0 || N % 4 != 0 || K < 64 || N < 16 || M < 64) continue;   // TryGemm's domain
    ShadowPlan want;
    want.want = true;
    want.a_off = RefOffset(g.in[0]);
    want.M = M;
    want.K = K;
    const uint64_t bytes = M * K * 4;
    for (size_t i = j; i-- > begin;) {
      const Extents& e = ext[i - begin];
      bool touches = false, exact = false;
      for (size_t x = 0; x < e.count; ++x) {
        if (!e.e[x].write) continue;
        if (e.e[x].off < want.a_off + bytes && want.a_off < e.e[x].off + e.e[x].bytes) {
          touches = true;
          exact = e.e[x].off == want.a_off && e.e[x].bytes == bytes;
        }
      }
      if (!touches) continue;
      ShadowPlan& slot = shadow_plan_[i - begin];
      if (exact && IsShadowProducer(program[i].opcode) && !slot.want) slot = want;
      break;
    }
  }
}

// Marks GEMM i / kAddBias i+1 pairs whose intermediate tensor R (the GEMM's
// output, the kAddBias input) nobody needs: every byte of R is overwritten by a
// later instruction of the range before any instruction reads it.  Proven on
// the operand extents; a range that ends with part of R unaccounted for keeps
// the pair as it is.
void CudaBackend::PlanBiasFusions(std::span<const Instruction> program, size_t begin, size_t end) {
  bias_fusion_.assign(end > begin ? end - begin : 0, BiasFusion{});
  if (coherence_ == Coherence::kStrict || !relaxed_allowed_ || !epilogue_fusion_ || end < begin + 2) return;
  std::vector<Extents> ext(end - begin);
  for (size_t i = begin; i < end; ++i)
    if (!DescribeInstruction(program[i], arena_bytes_, rodata_bytes_, source_bytes_, &ext[i - begin]).empty())
      return;   // a malformed instruction: leave everything as it is
  using Interval = std::pair<uint64_t, uint64_t>;   // [lo, hi)
  for (size_t i = begin; i + 1 < end; ++i) {
    const Instruction& g = program[i];
    const Instruction& ab = program[i + 1];
    const uint16_t op = g.opcode;
    const bool gemm = op == kGemmNN || op == kGemmNT || op == kGemmNNQ8 || op == kGemmNTQ8 ||
                      op == kGemmNNBF16 || op == kGemmNTBF16;
    if (!gemm || !(g.flags & kFlagRelaxed) || ab.opcode != kAddBias) continue;
    if ((g.flags & (kFlagEpilogueBias | kFlagGemmAddend)) || ActOf(g.flags) != kActNone) continue;
    if (RefSpace(g.in[1]) == kArena || RefSpace(g.in[0]) != kArena || RefSpace(g.in[2]) != kArena ||
        RefSpace(ab.in[2]) != kArena)
      continue;
    const uint64_t M = g.out[0], N = g.out[1], K = g.out[2];
    if (K % 8 != 0 || N % 4 != 0 || K < 64 || N < 16 || M < 64) continue;   // TryGemm's domain
    if (ab.in[0] != g.in[2] || ab.out[0] != M || ab.out[1] != N) continue;
    const uint64_t r_lo = RefOffset(g.in[2]), r_hi = r_lo + M * N * 4;
    const uint64_t z_lo = RefOffset(ab.in[2]), z_hi = z_lo + M * N * 4;
    if (z_lo < r_hi && r_lo < z_hi && z_lo != r_lo) continue;   // partial overlap: not a case we take
    if ((RefOffset(ab.in[1]) & 15) != 0 || (z_lo & 15) != 0) continue;   // the epilogue moves float4s
    bool dead = z_lo == r_lo;   // in place: R is Z, nothing to prove
    if (!dead) {
      std::vector<Interval> unknown{{r_lo, r_hi}};
      bool read_first = false;
      for (size_t j = i + 2; j < end && !unknown.empty() && !read_first; ++j) {
        const Extents& e = ext[j - begin];
        for (size_t x = 0; x < e.count && !read_first; ++x) {
          if (e.e[x].space != kArena) continue;
          const uint64_t lo = e.e[x].off, hi = lo + e.e[x].bytes;
          if (!e.e[x].write || e.e[x].read)
            for (const Interval& u : unknown)
              if (lo < u.second && u.first < hi) { read_first = true; break; }
        }
        if (read_first) break;
        for (size_t x = 0; x < e.count; ++x) {
          if (e.e[x].space != kArena || !e.e[x].write) continue;
          const uint64_t lo = e.e[x].off, hi = lo + e.e[x].bytes;
          std::vector<Interval> rest;
          for (const Interval& u : unknown) {
            if (hi <= u.first || u.second <= lo) { rest.push_back(u); continue; }
            if (u.first < lo) rest.push_back({u.first, lo});
            if (hi < u.second) rest.push_back({hi, u.second});
          }
          unknown.swap(rest);
        }
      }
      dead = !read_first && unknown.empty();
    }
    if (!dead) continue;
    BiasFusion& f = bias_fusion_[i - begin];
    f.fuse = true;
    f.bias_ref = ab.in[1];
    f.out_ref = ab.in[2];
  }
}

namespace {

bool IsRelaxedFrozenGemm(const Instruction& g) {
  const uint16_t op = g.opcode;
  const bool gemm = op == kGemmNN || op == kGemmNT || op == kGemmNNQ8 || op == kGemmNTQ8 ||
                    op == kGemmNNBF16 || op == kGemmNTBF16;
  if (!gemm || !(g.flags & kFlagRelaxed) || RefSpace(g.in[1]) == kArena || RefSpace(g.in[0]) != kArena)
    return false;
  const uint64_t M = g.out[0], N = g.out[1], K = g.out[2];
  return K % 8 == 0 && N % 4 == 0 && K >= 64 && N >= 16 && M >= 64;   // TryGemm's domain
}

uint64_t GemmScaleKey(const Instruction& g) {
  (void)g;   // the per-k factor of a transposed int8 product lives in its weight copy, not in the operand copy
  return ~0ull;
}

}  // namespace

// True when every byte of arena range [lo, hi) is overwritten before anything
// reads it, walking instructions start, start + 1, ... to the end of `ext`
// (the range, or the whole program under the step-program promise, in which
// case the walk then wraps to instruction 0 and stops at `wrap_stop`, the
// instruction that defines the range again in the next pass).  Exception, when
// `allow_consumers`: relaxed GEMMs of the current range (index < range_end)
// whose A operand is exactly that range under that copy key — they take the
// bf16 copy — and only while nothing has written into the range yet.
struct DeadQuery {
  uint64_t lo, hi;
  bool allow_consumers;
  uint64_t key_scale, M, K;
  // Reads of the whole tensor by relaxed tiled attention instructions of the range do not
  // count: they take the bf16 copy its producer wrote.
  bool allow_attention = false;
};

// A relaxed tiled attention instruction whose geometry the tensor-core kernels take, reading
// the tensor at `off` as one of its operands.
static bool IsAttentionCopyReader(const Instruction& ins, uint64_t off) {
  const bool fwd = ins.opcode == kAttnFwdTiled;
  const bool bwd = ins.opcode == kAttnDQTiled || ins.opcode == kAttnDKTiled || ins.opcode == kAttnDVTiled;
  if (!(fwd || bwd) || !(ins.flags & kFlagRelaxed)) return false;
  AttnGeom g;
  if (fwd) { g.B = Hi32(ins.out[1]); g.S = Lo32(ins.out[1]); g.H = Hi32(ins.out[2]); g.d = Lo32(ins.out[2]); }
  else g = UnpackAttnGeom(ins.out[2]);
  if ((g.d != 64 && g.d != 128) || g.S % 8 != 0 || g.S < 16 || g.B * g.H > 65535 || g.B * g.H == 0) return false;
  for (int r = 0; r < (fwd ? 3 : 4); ++r)
    if (RefSpace(ins.in[r]) == kArena && RefOffset(ins.in[r]) == off) return true;
  return false;
}
static bool DeadFrom(std::span<const Instruction> program, const std::vector<Extents>& ext, size_t ext_base,
                     size_t range_end, size_t start, bool wrap, size_t wrap_stop, const DeadQuery& q) {
  using Interval = std::pair<uint64_t, uint64_t>;
  std::vector<Interval> unknown{{q.lo, q.hi}};
  bool written = false;
  auto step = [&](size_t j, bool in_range) -> int {   // -1 read, 1 all overwritten, 0 go on
    const Extents& e = ext[j - ext_base];
    const Instruction& ins = program[j];
    for (size_t x = 0; x < e.count; ++x) {
      if (e.e[x].space != kArena) continue;
      const uint64_t elo = e.e[x].off, ehi = elo + e.e[x].bytes;
      if (e.e[x].write && !e.e[x].read) continue;
      bool hits = false;
      for (const Interval& u : unknown)
        if (elo < u.second && u.first < ehi) { hits = true; break; }
      if (!hits) continue;
      const bool consumer = q.allow_consumers && in_range && !written && !e.e[x].write &&
                            IsRelaxedFrozenGemm(ins) && RefOffset(ins.in[0]) == q.lo && elo == q.lo &&
                            ehi == q.hi && ins.out[0] == q.M && ins.out[2] == q.K &&
                            GemmScaleKey(ins) == q.key_scale;
      const bool copy_reader = q.allow_attention && in_range && !written && !e.e[x].write && elo == q.lo &&
                               ehi == q.hi && IsAttentionCopyReader(ins, q.lo);
      if (!consumer && !copy_reader) return -1;
    }
    for (size_t x = 0; x < e.count; ++x) {
      if (e.e[x].space != kArena || !e.e[x].write) continue;
      const uint64_t elo = e.e[x].off, ehi = elo + e.e[x].bytes;
      if (elo < q.hi && q.lo < ehi) written = true;
      std::vector<Interval> rest;
      for (const Interval& u : unknown) {
        if (ehi <= u.first || u.second <= elo) { rest.push_back(u); continue; }
        if (u.first < elo) rest.push_back({u.first, elo});
        if (ehi < u.second) rest.push_back({ehi, u.second});
      }
      unknown.swap(rest);
    }
    return unknown.empty() ? 1 : 0;
  };
  const size_t stop = ext_base + ext.size();
  for (size_t j = start; j < stop; ++j)
    if (const int r = step(j, j < range_end); r != 0) return r > 0;
  if (!wrap) return false;   // the range ended with bytes unaccounted for
  for (size_t j = ext_base; j < wrap_stop; ++j)
    if (const int r = step(j, false); r != 0) return r > 0;
  return true;   // reached the instruction that defines the range again
}

// Pairs each relaxed kAttnDQTiled of the range with the kAttnFwdTiled of the same
// attention earlier in the range (same q, k, v and stats row) and gives the pair a
// buffer for the forward's kept copy of O.  Buffers are allocated here, before any
// capture; a failed allocation just leaves the pair on the two-walk kernel.
void CudaBackend::PlanAttentionKeeps(std::span<const Instruction> program, size_t begin, size_t end) {
  attn_keep_slot_.assign(end > begin ? end - begin : 0, -1);
  if (coherence_ == Coherence::kStrict || !relaxed_allowed_ || !attn_one_walk_) return;
  int slots = 0;
  uint64_t elems = 0;
  for (size_t i = begin; i < end && i < program.size(); ++i) {
    const Instruction& dq = program[i];
    if (dq.opcode != kAttnDQTiled || !(dq.flags & kFlagRelaxed)) continue;
    const AttnGeom g = UnpackAttnGeom(dq.out[2]);
    for (size_t j = i; j-- > begin;) {
      const Instruction& fw = program[j];
      if (fw.opcode != kAttnFwdTiled || fw.out[0] != dq.out[0]) continue;
      if ((fw.flags & kFlagRelaxed) && fw.in[0] == dq.in[0] && fw.in[1] == dq.in[1] && fw.in[2] == dq.in[2] &&
          Hi32(fw.out[1]) == g.B && Lo32(fw.out[1]) == g.S && Hi32(fw.out[2]) == g.H && Lo32(fw.out[2]) == g.d &&
          attn_keep_slot_[j - begin] < 0) {
        attn_keep_slot_[j - begin] = attn_keep_slot_[i - begin] = slots++;
        elems = std::max(elems, g.B * g.S * g.H * g.d);
      }
      break;
    }
  }
  if (slots == 0) return;
  if (elems > attn_keep_elems_) {   // grow: every buffer anew
    cudaStreamSynchronize(stream_);
    for (float* p : attn_keep_pool_) cudaFree(p);
    attn_keep_pool_.clear();
    attn_keep_elems_ = elems;
  }
  while (static_cast<int>(attn_keep_pool_.size()) < slots) {
    void* p = nullptr;
    if (cudaMalloc(&p, attn_keep_elems_ * sizeof(float)) != cudaSuccess) {
      cudaGetLastError();
      break;
    }
    attn_keep_pool_.push_back(static_cast<float*>(p));
  }
  for (int& slot : attn_keep_slot_)
    if (slot >= static_cast<int>(attn_keep_pool_.size())) slot = -1;
  attn_keep_written_.assign(attn_keep_pool_.size(), 0);
}

// After the fusions are planned: for every relaxed GEMM of the range that will run as one
// tensor-core dispatch, where does its result finally land (its own output, the sum of an
// absorbed add, the output of a folded low-rank term), and is that tensor read, before
// anything overwrites it, by a relaxed tiled attention instruction as one of its operands?
void CudaBackend::PlanAttentionPacks(std::span<const Instruction> program, size_t begin, size_t end) {
  pack_plan_.assign(end > begin ? end - begin : 0, PackPlan{});
  if (coherence_ == Coherence::kStrict || !relaxed_allowed_ || !epilogue_fusion_) return;
  // Liveness of the f32 forms, as PlanActFusions decides it: on the whole program under the step-program promise.
  const bool whole = step_program_ != nullptr && program.data() == step_program_;
  const size_t ext_base = whole ? 0 : begin, ext_end = whole ? program.size() : end;
  std::vector<Extents> ext(ext_end - ext_base);
  bool have_ext = true;
  for (size_t i = ext_base; i < ext_end && have_ext; ++i)
    have_ext = DescribeInstruction(program[i], arena_bytes_, rodata_bytes_, source_bytes_, &ext[i - ext_base]).empty();
  auto unobserved = [&](uint64_t lo, uint64_t hi) {
    for (const auto& [off, bytes] : observed_)
      if (lo < off + bytes && off < hi) return false;
    return !(gather_ranks_ > 1 && lo < gather_off_ + gather_bytes_ && gather_off_ < hi);
  };
  for (size_t i = begin; i < end; ++i) {
    const Instruction& g = program[i];
    const bool gemm = g.opcode == kGemmNN || g.opcode == kGemmNT || g.opcode == kGemmNNQ8 || g.opcode == kGemmNTQ8 ||
                      g.opcode == kGemmNNBF16 || g.opcode == kGemmNTBF16;
    if (!gemm || !(g.flags & kFlagRelaxed)) continue;
    const size_t ri = i - begin;
    if (ri < act_fusion_.size() && act_fusion_[ri].mode != 0) continue;   // its stored value is not the consumer's operand
    if (ri < lora_skip_.size() && lora_skip_[ri] != 0) continue;
    uint64_t out = g.in[2];
    size_t last = i;   // the last instruction this dispatch stands for
    if (ri < add_fusion_.size() && add_fusion_[ri].fuse) {
      out = add_fusion_[ri].out_ref;
      last = std::max(last, begin + add_fusion_[ri].add_index);
    }
    if (ri < lora_fold_.size() && lora_fold_[ri].fuse) {
      out = lora_fold_[ri].out_ref;
      // The instructions this dispatch stands for follow it directly (the down product, the expand
      // product, an absorbed add): the last of them is the last skipped one before anything else runs.
      for (size_t j = i + 1; j < end && j - begin < lora_skip_.size() && lora_skip_[j - begin] != 0; ++j)
        last = std::max(last, j);
    }
    if (RefSpace(out) != kArena) continue;
    const uint64_t o_lo = RefOffset(out), o_hi = o_lo + g.out[0] * g.out[1] * 4;
    for (size_t j = last + 1; j < end; ++j) {
      const Instruction& at = program[j];
      const bool fwd = at.opcode == kAttnFwdTiled;
      const bool bwd = at.opcode == kAttnDQTiled || at.opcode == kAttnDKTiled || at.opcode == kAttnDVTiled;
      if ((fwd || bwd) && (at.flags & kFlagRelaxed)) {
        bool reads = false;
        for (int r = 0; r < (fwd ? 3 : 4); ++r) reads = reads || at.in[r] == out;
        if (reads) {
          AttnGeom geo;
          if (fwd) { geo.B = Hi32(at.out[1]); geo.S = Lo32(at.out[1]); geo.H = Hi32(at.out[2]); geo.d = Lo32(at.out[2]); }
          else geo = UnpackAttnGeom(at.out[2]);
          if (geo.B * geo.S == g.out[0] && geo.H * geo.d == g.out[1] && IsAttentionCopyReader(at, o_lo)) {
            pack_plan_[ri] = PackPlan{out, static_cast<uint32_t>(geo.S), static_cast<uint32_t>(geo.H),
                                      static_cast<uint32_t>(geo.d), false, last - begin};
            // Is the f32 form read by anything else before it is written again?
            DeadQuery q{o_lo, o_hi, false, 0, 0, 0, true};
            if (have_ext) {
              const bool wrap = whole && unobserved(o_lo, o_hi);
              if (whole && !wrap) {
                std::vector<Extents> in_range(ext.begin() + static_cast<long>(begin), ext.begin() + static_cast<long>(end));
                pack_plan_[ri].copy_only = DeadFrom(program, in_range, begin, end, last + 1, false, 0, q);
              } else {
                pack_plan_[ri].copy_only = DeadFrom(program, ext, ext_base, end, last + 1, wrap, i, q);
              }
            }
          }
          break;
        }
      }
      Extents ex;
      if (!DescribeInstruction(at, arena_bytes_, rodata_bytes_, source_bytes_, &ex).empty()) break;
      bool overwritten = false;
      for (size_t e = 0; e < ex.count; ++e)
        if (ex.e[e].write && ex.e[e].space == kArena && ex.e[e].off < o_hi && o_lo < ex.e[e].off + ex.e[e].bytes)
          overwritten = true;
      if (overwritten) break;
    }
  }
}

void CudaBackend::PlanActFusions(std::span<const Instruction> program, size_t begin, size_t end) {
  act_fusion_.assign(end > begin ? end - begin : 0, ActFusion{});
  loss_fusion_.assign(end > begin ? end - begin : 0, LossFusion{});
  add_fusion_.assign(end > begin ? end - begin : 0, AddFusion{});
  attn_dv_out_.assign(end > begin ? end - begin : 0, kNullRef);
  attn_dv_shadow_.assign(end > begin ? end - begin : 0, ShadowPlan{});
  lora_fold_.assign(end > begin ? end - begin : 0, LoraFold{});
  adapter_bwd_.assign(end > begin ? end - begin : 0, AdapterBackward{});
  lora_skip_.assign(end > begin ? end - begin : 0, 0);
  lora_weights_.clear();
  lora_max_n_ = lora_max_kx_ = 0;
  if (coherence_ == Coherence::kStrict || !relaxed_allowed_ || !epilogue_fusion_ || end < begin + 3) return;
  // Under the step-program promise liveness is decided on the whole program.
  const bool whole = step_program_ != nullptr && program.data() == step_program_;
  const size_t ext_base = whole ? 0 : begin, ext_end = whole ? program.size() : end;
  std::vector<Extents> ext(ext_end - ext_base);
  for (size_t i = ext_base; i < ext_end; ++i)
    if (!DescribeInstruction(program[i], arena_bytes_, rodata_bytes_, source_bytes_, &ext[i - ext_base]).empty())
      return;   // a malformed instruction: leave everything as it is
  auto disjoint = [](uint64_t alo, uint64_t ahi, uint64_t blo, uint64_t bhi) { return ahi <= blo || bhi <= alo; };
  auto unobserved = [&](uint64_t lo, uint64_t hi) {
    for (const auto& [off, bytes] : observed_)
      if (lo < off + bytes && off < hi) return false;
    return !(gather_ranks_ > 1 && lo < gather_off_ + gather_bytes_ && gather_off_ < hi);
  };
  // Is the range dead after instruction `def` (which defines it)?  The walk may
  // leave the range (and wrap) only for bytes nothing outside the program looks at.
  // `last` is the last instruction allowed to read it, `def` the one that defines
  // it (where a wrapped walk stops: the next pass writes it again there).
  auto dead_after = [&](size_t last, const DeadQuery& q, size_t def = ~size_t{0}) {
    if (def == ~size_t{0}) def = last;
    const bool wrap = whole && unobserved(q.lo, q.hi);
    if (whole && !wrap) {   // observed bytes: the proof must close inside the range
      std::vector<Extents> in_range(ext.begin() + static_cast<long>(begin), ext.begin() + static_cast<long>(end));
      return DeadFrom(program, in_range, begin, end, last + 1, false, 0, q);
    }
    return DeadFrom(program, ext, ext_base, end, last + 1, wrap, def, q);
  };
  // Producers that can write the bf16 copy alone: the loss gradient, whose f32
  // form (rows x vocabulary) is the largest tensor of a step.
  for (size_t i = begin; i < end; ++i) {
    ShadowPlan& sp = shadow_plan_[i - begin];
    const uint16_t op = program[i].opcode;
    if (!sp.want || (op != kSoftmaxXEntBwd && op != kSoftmaxXEntMaskedBwd)) continue;
    if (sp.scale_ref != kNullRef && (sp.scale_off & 15) != 0) continue;
    sp.only = dead_after(i, DeadQuery{sp.a_off, sp.a_off + sp.M * sp.K * 4, true, sp.scale_off, sp.M, sp.K});
  }
  // dK and dV of the same attention in one walk over the queries.
  for (size_t i = begin; i + 1 < end; ++i) {
    const Instruction& dk = program[i];
    const Instruction& dv = program[i + 1];
    if (dk.opcode != kAttnDKTiled || dv.opcode != kAttnDVTiled || !(dk.flags & kFlagRelaxed) ||
        !(dv.flags & kFlagRelaxed))
      continue;
    if (dk.in[0] != dv.in[0] || dk.in[1] != dv.in[1] || dk.in[2] != dv.in[2] || dk.in[3] != dv.in[3] ||
        dk.out[0] != dv.out[0] || dk.out[2] != dv.out[2] || RefSpace(dk.out[1]) != kArena ||
        RefSpace(dv.out[1]) != kArena)
      continue;
    const AttnGeom g = UnpackAttnGeom(dk.out[2]);
    const uint64_t bytes = g.B * g.S * g.H * g.d * 4;
    if (g.d != 64 || !disjoint(RefOffset(dk.out[1]), RefOffset(dk.out[1]) + bytes, RefOffset(dv.out[1]),
                               RefOffset(dv.out[1]) + bytes))
      continue;
    // Neither output may lie over an operand the other instruction still reads.
    bool clash = false;
    for (int op = 0; op < 4; ++op)
      if (RefSpace(dk.in[op]) == kArena &&
          (!disjoint(RefOffset(dk.in[op]), RefOffset(dk.in[op]) + bytes, RefOffset(dk.out[1]),
                     RefOffset(dk.out[1]) + bytes) ||
           !disjoint(RefOffset(dk.in[op]), RefOffset(dk.in[op]) + bytes, RefOffset(dv.out[1]),
                     RefOffset(dv.out[1]) + bytes)))
        clash = true;
    if (clash) continue;
    attn_dv_out_[i - begin] = dv.out[1];
    attn_dv_shadow_[i - begin] = shadow_plan_[i + 1 - begin];   // the pair's kernel makes dV's copy too
    shadow_plan_[i + 1 - begin].want = false;
  }
  // Forward loss, seed fill, backward loss: one row pass when the gradient leaves
  // as a copy only.
  for (size_t i = begin; i + 2 < end; ++i) {
    const Instruction& f = program[i];
    const Instruction& fill = program[i + 1];
    const Instruction& b = program[i + 2];
    if (f.opcode != kSoftmaxXEntFwd || fill.opcode != kFill || fill.out[0] != 1 || b.opcode != kSoftmaxXEntBwd)
      continue;
    if (b.in[0] != f.in[3] || b.in[1] != f.in[1] || b.in[2] != fill.in[0] || b.out[0] != f.out[0] ||
        b.out[1] != f.out[1] || RefSpace(f.in[3]) != kArena)
      continue;
    ShadowPlan& sp = shadow_plan_[i + 2 - begin];
    if (!sp.want || !sp.only || shadow_plan_[i - begin].want) continue;
    LossFusion lf;
    lf.fuse = true;
    lf.seed = BitsToF32(fill.in[1]);
    lf.bwd_index = static_cast<uint32_t>(i + 2 - begin);
    lf.probs_lo = RefOffset(f.in[3]);
    lf.probs_hi = lf.probs_lo + f.out[0] * f.out[1] * 4;
    lf.store_probs = !dead_after(i + 2, DeadQuery{lf.probs_lo, lf.probs_hi, false, ~0ull, 0, 0}, i);
    loss_fusion_[i - begin] = lf;
    shadow_plan_[i - begin] = sp;   // the forward is now the copy's producer
    sp.want = false;
  }
  for (size_t i = begin; i + 1 < end; ++i) {
    const Instruction& g = program[i];
    if (!IsRelaxedFrozenGemm(g) || RefSpace(g.in[2]) != kArena) continue;
    if ((g.flags & (kFlagEpilogueBias | kFlagGemmAddend)) || ActOf(g.flags) != kActNone) continue;
    const uint64_t M = g.out[0], N = g.out[1], bytes = M * N * 4;
    size_t next = i + 1;
    uint64_t z_ref = g.in[2];
    if (bias_fusion_[i - begin].fuse) {
      z_ref = bias_fusion_[i - begin].out_ref;
      next = i + 2;
    }
    if (next >= end) continue;
    const Instruction& act = program[next];
    const uint16_t aop = act.opcode;
    const bool fwd = aop == kReluFwd || aop == kGeluFwd || aop == kSiluFwd;
    const bool bwd = aop == kReluBwd || aop == kGeluBwd || aop == kSiluBwd;
    if ((!fwd && !bwd) || act.in[0] != z_ref || act.out[0] != M * N) continue;
    const uint64_t out_ref = fwd ? act.in[1] : act.in[2];
    if (RefSpace(out_ref) != kArena) continue;
    const ShadowPlan& sp = shadow_plan_[next - begin];
    if (!sp.want || sp.a_off != RefOffset(out_ref) || sp.M != M || sp.K != N) continue;
    if (sp.scale_ref != kNullRef && (sp.scale_off & 15) != 0) continue;
    const uint64_t z_lo = RefOffset(z_ref), z_hi = z_lo + bytes;
    const uint64_t o_lo = RefOffset(out_ref), o_hi = o_lo + bytes;
    auto dead = [&](uint64_t lo, uint64_t hi, bool consumers) {
      return dead_after(next, DeadQuery{lo, hi, consumers, sp.scale_off, M, N});
    };
    ActFusion f;
    f.act = aop == kReluFwd || aop == kReluBwd ? kActRelu : aop == kGeluFwd || aop == kGeluBwd ? kActGelu : kActSilu;
    f.act_index = static_cast<uint32_t>(next - begin);
    if (fwd) {
      if (!disjoint(z_lo, z_hi, o_lo, o_hi)) continue;
      if (!dead(o_lo, o_hi, true)) continue;
      f.mode = k::kFuseActFwd;
      f.store_c = true;
      f.elided[0][0] = o_lo; f.elided[0][1] = o_hi;
      f.elided_count = 1;
    } else {
      if (RefSpace(act.in[1]) != kArena || (RefOffset(act.in[1]) & 15) != 0) continue;
      const uint64_t x_lo = RefOffset(act.in[1]), x_hi = x_lo + bytes;
      if (!disjoint(x_lo, x_hi, z_lo, z_hi) || !disjoint(x_lo, x_hi, o_lo, o_hi)) continue;
      const bool in_place = o_lo == z_lo;
      if (!in_place && !disjoint(z_lo, z_hi, o_lo, o_hi)) continue;
      if (!dead(o_lo, o_hi, true)) continue;
      f.mode = k::kFuseActBwd;
      f.x_ref = act.in[1];
      f.elided[0][0] = o_lo; f.elided[0][1] = o_hi;
      f.elided_count = 1;
      if (in_place) {
        f.store_c = false;
      } else {
        f.store_c = !dead(z_lo, z_hi, false);
        if (!f.store_c) {
          f.elided[1][0] = z_lo; f.elided[1][1] = z_hi;
          f.elided_count = 2;
        }
      }
    }
    act_fusion_[i - begin] = f;
    // The GEMM is now the producer of the copy the activation would have made.
    shadow_plan_[i - begin] = sp;
    shadow_plan_[next - begin].want = false;
  }
  // A following kAddEW as the epilogue's addend.
  for (size_t i = begin; i + 1 < end; ++i) {
    const Instruction& g = program[i];
    if (!IsRelaxedFrozenGemm(g) || RefSpace(g.in[2]) != kArena || act_fusion_[i - begin].mode != 0) continue;
    if ((g.flags & (kFlagEpilogueBias | kFlagGemmAddend)) || ActOf(g.flags) != kActNone) continue;
    const uint64_t M = g.out[0], N = g.out[1], bytes = M * N * 4;
    size_t next = i + 1;
    uint64_t z_ref = g.in[2];
    if (bias_fusion_[i - begin].fuse) {
      z_ref = bias_fusion_[i - begin].out_ref;
      next = i + 2;
    }
    if (next >= end) continue;
    const Instruction& add = program[next];
    if (add.opcode != kAddEW || add.out[0] != M * N || shadow_plan_[next - begin].want) continue;
    uint64_t x_ref;
    if (add.in[0] == z_ref && add.in[1] != z_ref) x_ref = add.in[1];
    else if (add.in[1] == z_ref && add.in[0] != z_ref) x_ref = add.in[0];
    else continue;
    const uint64_t out_ref = add.in[2];
    if (RefSpace(x_ref) != kArena || RefSpace(out_ref) != kArena || (RefOffset(x_ref) & 15) != 0 ||
        (RefOffset(out_ref) & 15) != 0)
      continue;
    const uint64_t z_lo = RefOffset(z_ref), z_hi = z_lo + bytes;
    const uint64_t x_lo = RefOffset(x_ref), x_hi = x_lo + bytes;
    const uint64_t o_lo = RefOffset(out_ref), o_hi = o_lo + bytes;
    if (!disjoint(x_lo, x_hi, z_lo, z_hi)) continue;
    if (o_lo != x_lo && !disjoint(o_lo, o_hi, x_lo, x_hi)) continue;   // in place over x, or apart from it
    if (o_lo != z_lo && !disjoint(o_lo, o_hi, z_lo, z_hi)) continue;   // likewise for the product
    if (o_lo != z_lo && !dead_after(next, DeadQuery{z_lo, z_hi, false, ~0ull, 0, 0}, i)) continue;
    AddFusion af;
    af.fuse = true;
    af.x_ref = x_ref;
    af.out_ref = out_ref;
    af.add_index = static_cast<uint32_t>(next - begin);
    if (o_lo != z_lo) { af.z_lo = z_lo; af.z_hi = z_hi; }
    add_fusion_[i - begin] = af;
  }
  // The same for the rank-r expand product of an adapter (exact kernels): the
  // residual add after the adapted projection.
  for (size_t i = begin; i + 1 < end; ++i) {
    const Instruction& g = program[i];
    const Instruction& add = program[i + 1];
    if ((g.opcode != kGemmNN && g.opcode != kGemmNT) || (g.flags & kFlagRelaxed) || add.opcode != kAddEW) continue;
    if (RefSpace(g.in[2]) != kArena || shadow_plan_[i + 1 - begin].want) continue;
    const uint64_t M = g.out[0], N = g.out[1], K = g.out[2], bytes = M * N * 4;
    if ((K != 4 && K != 8 && K != 12 && K != 16) || (N & 3) != 0 || N < 64 || M < 64) continue;   // the expand kernel's shapes
    if (add.out[0] != M * N) continue;
    const uint64_t z_ref = g.in[2];
    uint64_t x_ref;
    if (add.in[0] == z_ref && add.in[1] != z_ref) x_ref = add.in[1];
    else if (add.in[1] == z_ref && add.in[0] != z_ref) x_ref = add.in[0];
    else continue;
    const uint64_t out_ref = add.in[2];
    if (RefSpace(x_ref) != kArena || RefSpace(out_ref) != kArena) continue;
    const uint64_t z_lo = RefOffset(z_ref), z_hi = z_lo + bytes;
    const uint64_t x_lo = RefOffset(x_ref), x_hi = x_lo + bytes;
    const uint64_t o_lo = RefOffset(out_ref), o_hi = o_lo + bytes;
    if (!disjoint(x_lo, x_hi, z_lo, z_hi) || !disjoint(o_lo, o_hi, z_lo, z_hi)) continue;
    if (o_lo != x_lo && !disjoint(o_lo, o_hi, x_lo, x_hi)) continue;
    // The product's own operands must not be overwritten by the sum while other
    // blocks still read them (the addend it accumulates onto may be the sum's place
    // exactly: each element is read, then written, by the same thread).
    bool clash = false;
    const uint64_t srcs[2] = {g.in[0], (g.flags & kFlagGemmAddend) ? g.in[3] : kNullRef};
    const uint64_t src_bytes[2] = {M * K * 4, bytes};
    for (int op = 0; op < 2; ++op)
      if (srcs[op] != kNullRef && RefSpace(srcs[op]) == kArena &&
          !disjoint(o_lo, o_hi, RefOffset(srcs[op]), RefOffset(srcs[op]) + src_bytes[op]) &&
          !(op == 1 && RefOffset(srcs[op]) == o_lo))   // exactly over the addend: read, then written, per element
        clash = true;
    if (RefSpace(g.in[1]) == kArena && !disjoint(o_lo, o_hi, RefOffset(g.in[1]), RefOffset(g.in[1]) + K * N * 4))
      clash = true;
    if (clash) continue;
    if (!dead_after(i + 1, DeadQuery{z_lo, z_hi, false, ~0ull, 0, 0}, i)) continue;
    AddFusion af;
    af.fuse = true;
    af.x_ref = x_ref;
    af.out_ref = out_ref;
    af.add_index = static_cast<uint32_t>(i + 1 - begin);
    af.z_lo = z_lo; af.z_hi = z_hi;
    add_fusion_[i - begin] = af;
  }
  // The same for a LayerNorm backward whose dx is only one term of a sum.
  for (size_t i = begin; i + 1 < end; ++i) {
    const Instruction& ln = program[i];
    const Instruction& add = program[i + 1];
    if (ln.opcode != kLayerNormBwd || add.opcode != kAddEW || RefSpace(ln.in[3]) != kArena) continue;
    const uint64_t elems = static_cast<uint64_t>(Hi32(ln.out[2])) * Lo32(ln.out[2]), bytes = elems * 4;
    if (add.out[0] != elems || shadow_plan_[i - begin].want) continue;
    const uint64_t z_ref = ln.in[3];
    uint64_t x_ref;
    if (add.in[0] == z_ref && add.in[1] != z_ref) x_ref = add.in[1];
    else if (add.in[1] == z_ref && add.in[0] != z_ref) x_ref = add.in[0];
    else continue;
    const uint64_t out_ref = add.in[2];
    if (RefSpace(x_ref) != kArena || RefSpace(out_ref) != kArena) continue;
    const uint64_t z_lo = RefOffset(z_ref), z_hi = z_lo + bytes;
    const uint64_t x_lo = RefOffset(x_ref), x_hi = x_lo + bytes;
    const uint64_t o_lo = RefOffset(out_ref), o_hi = o_lo + bytes;
    if (!disjoint(x_lo, x_hi, z_lo, z_hi)) continue;
    if (o_lo != x_lo && !disjoint(o_lo, o_hi, x_lo, x_hi)) continue;
    if (o_lo != z_lo && !disjoint(o_lo, o_hi, z_lo, z_hi)) continue;
    // The kernel reads whole rows of dy and x before it writes the row of the sum:
    // the sum may lie over either, but not partly.
    bool partial = false;
    for (int op = 0; op < 2; ++op) {
      const uint64_t s_lo = RefOffset(ln.in[op]), s_hi = s_lo + bytes;
      if (RefSpace(ln.in[op]) == kArena && s_lo != o_lo && !disjoint(o_lo, o_hi, s_lo, s_hi)) partial = true;
    }
    if (partial) continue;
    if (o_lo != z_lo && !dead_after(i + 1, DeadQuery{z_lo, z_hi, false, ~0ull, 0, 0}, i)) continue;
    AddFusion af;
    af.fuse = true;
    af.x_ref = x_ref;
    af.out_ref = out_ref;
    af.add_index = static_cast<uint32_t>(i + 1 - begin);
    if (o_lo != z_lo) { af.z_lo = z_lo; af.z_hi = z_hi; }
    add_fusion_[i - begin] = af;
    if (shadow_plan_[i + 1 - begin].want) {   // the kernel makes the sum's copy too
      shadow_plan_[i - begin] = shadow_plan_[i + 1 - begin];
      shadow_plan_[i + 1 - begin].want = false;
    }
  }

  // ---- the adapter's expand product folded into the frozen product (LoraFold) ----
  const bool folds = lora_fold_enabled_;
  auto overlap = [](uint64_t alo, uint64_t ahi, uint64_t blo, uint64_t bhi) { return alo < bhi && blo < ahi; };
  auto touches = [&](size_t j, uint64_t lo, uint64_t hi, bool want_write) {   // does instruction j write (read) [lo, hi)?
    const Extents& e = ext[j - ext_base];
    for (size_t x = 0; x < e.count; ++x) {
      if (e.e[x].space != kArena || !overlap(e.e[x].off, e.e[x].off + e.e[x].bytes, lo, hi)) continue;
      if (want_write ? e.e[x].write : (!e.e[x].write || e.e[x].read)) return true;
    }
    return false;
  };
  auto rank_ok = [](uint64_t r) { return r == 4 || r == 8 || r == 12 || r == 16; };
  auto aligned = [](uint64_t ref) { return RefSpace(ref) == kArena && (RefOffset(ref) & 15) == 0; };
  auto plain_frozen = [&](size_t i) {
    const Instruction& g = program[i];
    return IsRelaxedFrozenGemm(g) && RefSpace(g.in[2]) == kArena &&
           !(g.flags & (kFlagEpilogueBias | kFlagGemmAddend)) && ActOf(g.flags) == kActNone &&
           !bias_fusion_[i - begin].fuse && act_fusion_[i - begin].mode == 0 && lora_skip_[i - begin] == 0 &&
           !shadow_plan_[i - begin].want;
  };
  // The adapter matrix must hold the same values when the range starts (where its
  // split copy is made) as where the plan multiplies by it.
  auto unwritten_before = [&](size_t i, uint64_t lo, uint64_t hi) {
    for (size_t j = begin; j < i; ++j)
      if (touches(j, lo, hi, true)) return false;
    return true;
  };
  auto add_weight = [&](const Instruction& g, uint64_t w_ref, uint32_t r, uint32_t n_out, float alpha, bool by_column) {
    const k::GemmArgs ga = GemmArgsOf(g);
    k::LoraWeight w{};
    w.src = Rd(w_ref);
    w.col_scale = ga.b_col_scale;
    w.tile_alpha = ga.alpha;
    w.alpha = alpha;
    w.n_out = n_out;
    w.r = r;
    w.kx = k::LoraSplitColumns(r);
    w.by_column = by_column ? 1u : 0u;
    lora_weights_.push_back(w);
    lora_max_n_ = std::max(lora_max_n_, n_out);
    lora_max_kx_ = std::max(lora_max_kx_, w.kx);
    return static_cast<uint32_t>(lora_weights_.size() - 1);
  };
  // A kAddEW planned to ride the expand kernel (add_fusion_ at the expand's
  // position) moves to the frozen product's epilogue, or back to its own kernel.
  auto take_add = [&](size_t e_abs, LoraFold* f, uint64_t e_out_lo, uint64_t e_out_hi, uint64_t keep_lo[3],
                      uint64_t keep_hi[3], int keeps) {
    AddFusion& af = add_fusion_[e_abs - begin];
    if (!af.fuse) return;
    bool ok = aligned(af.x_ref) && aligned(af.out_ref) && !shadow_plan_[af.add_index].want;
    const uint64_t o_lo = RefOffset(af.out_ref), o_hi = o_lo + (e_out_hi - e_out_lo);
    for (int q = 0; q < keeps && ok; ++q)   // the sum must not land on anything the product still reads
      if (overlap(o_lo, o_hi, keep_lo[q], keep_hi[q])) ok = false;
    // ... and lies exactly over, or apart from, each range the fold leaves unwritten
    // (the plan often puts the sum where the un-adapted product was).
    for (int q = 0; q < f->dead_count && ok; ++q)
      if (overlap(o_lo, o_hi, f->dead[q][0], f->dead[q][1]) && o_lo != f->dead[q][0]) ok = false;
    if (ok) {
      f->out_ref = af.out_ref;
      f->addend_ref = af.x_ref;
      ++f->absorbed;
      lora_skip_[af.add_index] = 1;                       // the sum is written by the product
      lora_skip_[e_abs - begin] = 2;                      // the expand's own output never is
      int kept = 0;
      for (int q = 0; q < f->dead_count; ++q)             // a range the sum lands on is written after all
        if (f->dead[q][0] != o_lo) { f->dead[kept][0] = f->dead[q][0]; f->dead[kept][1] = f->dead[q][1]; ++kept; }
      f->dead_count = kept;
      if (e_out_lo != o_lo) {
        f->dead[f->dead_count][0] = e_out_lo; f->dead[f->dead_count][1] = e_out_hi; ++f->dead_count;
      }
    }
    af = AddFusion{};   // either way the expand kernel no longer runs
  };
  for (size_t i = begin; i < end && folds; ++i) {
    if (!plain_frozen(i) || add_fusion_[i - begin].fuse) continue;
    const Instruction& g = program[i];
    const uint64_t M = g.out[0], N = g.out[1];
    const uint64_t b_lo = RefOffset(g.in[2]), b_hi = b_lo + M * N * 4;
    const uint64_t x_lo = RefOffset(g.in[0]), x_hi = x_lo + M * g.out[2] * 4;
    // kind 1: G; D: t = x A; E: out = G.out + s t B
    if (i + 2 < end) {
      const Instruction& d = program[i + 1];
      const Instruction& e = program[i + 2];
      const uint64_t r = d.out[1];
      if (d.opcode == kGemmNN && d.flags == 0 && e.opcode == kGemmNN && e.flags == kFlagGemmAddend && rank_ok(r) &&
          d.out[0] == M && e.out[0] == M && e.out[1] == N && e.out[2] == r && e.in[0] == d.in[2] &&
          e.in[3] == g.in[2] && aligned(d.in[2]) && aligned(e.in[2]) && RefSpace(e.in[1]) == kArena &&
          RefSpace(d.in[0]) == kArena && lora_skip_[i + 1 - begin] == 0 && lora_skip_[i + 2 - begin] == 0 &&
          !shadow_plan_[i + 1 - begin].want && !shadow_plan_[i + 2 - begin].want) {
        const uint64_t t_lo = RefOffset(d.in[2]), t_hi = t_lo + M * r * 4;
        const uint64_t dx_lo = RefOffset(d.in[0]), dx_hi = dx_lo + M * d.out[2] * 4;
        const uint64_t a_lo = RefOffset(d.in[1]), a_hi = a_lo + d.out[2] * r * 4;
        const uint64_t w_lo = RefOffset(e.in[1]), w_hi = w_lo + r * N * 4;
        const uint64_t o_lo = RefOffset(e.in[2]), o_hi = o_lo + M * N * 4;
        const bool a_in_arena = RefSpace(d.in[1]) == kArena;
        bool ok = !overlap(b_lo, b_hi, dx_lo, dx_hi) && !(a_in_arena && overlap(b_lo, b_hi, a_lo, a_hi)) &&
                  !overlap(t_lo, t_hi, x_lo, x_hi) && !overlap(t_lo, t_hi, b_lo, b_hi) &&
                  !overlap(o_lo, o_hi, t_lo, t_hi) &&
                  !overlap(o_lo, o_hi, w_lo, w_hi) && (o_lo == b_lo || !overlap(o_lo, o_hi, b_lo, b_hi)) &&
                  unwritten_before(i + 2, w_lo, w_hi);
        if (ok && o_lo != b_lo) ok = dead_after(i + 2, DeadQuery{b_lo, b_hi, false, ~0ull, 0, 0}, i);
        if (ok) {
          LoraFold f;
          f.fuse = true;
          f.kind = 1;
          f.down = d;
          f.t_ref = d.in[2];
          f.r = static_cast<uint32_t>(r);
          f.out_ref = e.in[2];
          f.absorbed = 2;
          f.weight_slot = add_weight(g, e.in[1], f.r, static_cast<uint32_t>(N), GemmAlphaOf(e.imm), false);
          if (o_lo != b_lo) { f.dead[0][0] = b_lo; f.dead[0][1] = b_hi; f.dead_count = 1; }
          lora_skip_[i + 1 - begin] = 1;
          lora_skip_[i + 2 - begin] = 1;
          // (The sum may land on the product's own f32 operand: the product reads its bf16 copy,
          // made before the kernel starts.  Not on t, which the backward sweep reads.)
          uint64_t keep_lo[3] = {t_lo, w_lo, 0}, keep_hi[3] = {t_hi, w_hi, 0};
          take_add(i + 2, &f, o_lo, o_hi, keep_lo, keep_hi, 2);
          lora_fold_[i - begin] = f;
          continue;
        }
      }
    }
    // kind 2: G; E: out = G.out + dT A^T
    if (i + 1 < end) {
      const Instruction& e = program[i + 1];
      const uint64_t r = e.out[2];
      if (e.opcode == kGemmNT && e.flags == kFlagGemmAddend && rank_ok(r) && e.out[0] == M && e.out[1] == N &&
          e.in[3] == g.in[2] && aligned(e.in[0]) && aligned(e.in[2]) && RefSpace(e.in[1]) == kArena &&
          lora_skip_[i + 1 - begin] == 0 && !shadow_plan_[i + 1 - begin].want) {
        const uint64_t t_lo = RefOffset(e.in[0]), t_hi = t_lo + M * r * 4;
        const uint64_t w_lo = RefOffset(e.in[1]), w_hi = w_lo + N * r * 4;
        const uint64_t o_lo = RefOffset(e.in[2]), o_hi = o_lo + M * N * 4;
        // The sum may reuse the slot of dY or of dT (the plans do): both are read through copies
        // made before the kernel starts, and the plan's own expand kernel wrote the sum there too.
        bool ok = !overlap(o_lo, o_hi, w_lo, w_hi) && !overlap(b_lo, b_hi, t_lo, t_hi) &&
                  (o_lo == b_lo || !overlap(o_lo, o_hi, b_lo, b_hi)) && unwritten_before(i + 1, w_lo, w_hi);
        if (ok && o_lo != b_lo) ok = dead_after(i + 1, DeadQuery{b_lo, b_hi, false, ~0ull, 0, 0}, i);
        if (ok) {
          LoraFold f;
          f.fuse = true;
          f.kind = 2;
          f.t_ref = e.in[0];
          f.r = static_cast<uint32_t>(r);
          f.out_ref = e.in[2];
          f.absorbed = 1;
          f.weight_slot = add_weight(g, e.in[1], f.r, static_cast<uint32_t>(N), GemmAlphaOf(e.imm), true);
          if (o_lo != b_lo) { f.dead[0][0] = b_lo; f.dead[0][1] = b_hi; f.dead_count = 1; }
          lora_skip_[i + 1 - begin] = 1;
          uint64_t keep_lo[3] = {w_lo, 0, 0}, keep_hi[3] = {w_hi, 0, 0};
          take_add(i + 1, &f, o_lo, o_hi, keep_lo, keep_hi, 1);
          lora_fold_[i - begin] = f;
          continue;
        }
      }
    }
  }
  // kind 3: E: part = acc + dT A^T; (up to two instructions); G; kAddEW: part + G.out, already planned as G's
  // epilogue addend: the addend becomes acc and the expand rides the reduction.
  for (size_t i = begin; i < end && folds; ++i) {
    AddFusion& af = add_fusion_[i - begin];
    const Instruction& g = program[i];
    if (!af.fuse || !IsRelaxedFrozenGemm(g) || RefSpace(g.in[2]) != kArena || lora_fold_[i - begin].fuse ||
        bias_fusion_[i - begin].fuse || act_fusion_[i - begin].mode != 0 || lora_skip_[i - begin] != 0)
      continue;
    if ((g.flags & (kFlagEpilogueBias | kFlagGemmAddend)) || ActOf(g.flags) != kActNone) continue;
    const uint64_t M = g.out[0], N = g.out[1];
    const size_t add_abs = begin + af.add_index;
    for (size_t back = 1; back <= 3 && i >= begin + back; ++back) {
      const size_t ea = i - back;
      const Instruction& e = program[ea];
      const uint64_t r = e.out[2];
      if (e.opcode != kGemmNT || e.flags != kFlagGemmAddend || !rank_ok(r) || e.out[0] != M || e.out[1] != N ||
          e.in[2] != af.x_ref || !aligned(e.in[0]) || !aligned(e.in[3]) || RefSpace(e.in[1]) != kArena ||
          lora_skip_[ea - begin] != 0 || add_fusion_[ea - begin].fuse || shadow_plan_[ea - begin].want)
        continue;
      const uint64_t p_lo = RefOffset(e.in[2]), p_hi = p_lo + M * N * 4;       // part
      const uint64_t t_lo = RefOffset(e.in[0]), t_hi = t_lo + M * r * 4;       // dT
      const uint64_t w_lo = RefOffset(e.in[1]), w_hi = w_lo + N * r * 4;       // A
      const uint64_t c_lo = RefOffset(e.in[3]), c_hi = c_lo + M * N * 4;       // acc
      const uint64_t o_lo = RefOffset(af.out_ref), o_hi = o_lo + M * N * 4;    // the sum
      const uint64_t x_lo = RefOffset(g.in[0]), x_hi = x_lo + M * g.out[2] * 4;
      bool ok = true;
      for (size_t j = ea + 1; j < i && ok; ++j)   // nothing in between looks at part or changes the expand's operands
        ok = !touches(j, p_lo, p_hi, false) && !touches(j, p_lo, p_hi, true) && !touches(j, t_lo, t_hi, true) &&
             !touches(j, w_lo, w_hi, true) && !touches(j, c_lo, c_hi, true);
      ok = ok && !overlap(o_lo, o_hi, w_lo, w_hi) && (o_lo == c_lo || !overlap(o_lo, o_hi, c_lo, c_hi)) &&
           !overlap(p_lo, p_hi, c_lo, c_hi) && !overlap(p_lo, p_hi, x_lo, x_hi) && unwritten_before(i, w_lo, w_hi);
      if (ok && o_lo != p_lo) ok = dead_after(add_abs, DeadQuery{p_lo, p_hi, false, ~0ull, 0, 0}, ea);
      if (!ok) continue;
      LoraFold f;
      f.fuse = true;
      f.kind = 3;
      f.t_ref = e.in[0];
      f.r = static_cast<uint32_t>(r);
      f.out_ref = af.out_ref;
      f.addend_ref = e.in[3];
      f.absorbed = 1;   // (the kAddEW is counted by the add fusion it already is)
      f.weight_slot = add_weight(g, e.in[1], f.r, static_cast<uint32_t>(N), GemmAlphaOf(e.imm), true);
      lora_skip_[ea - begin] = 2;
      lora_fold_[i - begin] = f;
      break;
    }
  }
  // ---- the three activation-streaming backward products of an adapter site in one pass ----
  //   [j] dT = a dY B^T   [j+1] dB = a t^T dY   [j+2 or j+3] dA = x^T dT
  if (!adapter_fma_) return;
  for (size_t j = begin; j + 2 < end; ++j) {
    const Instruction& dt = program[j];
    const Instruction& db = program[j + 1];
    if (dt.opcode != kGemmNT || dt.flags != 0 || db.opcode != kGemmTN || db.flags != 0) continue;
    if (lora_skip_[j - begin] != 0 || lora_skip_[j + 1 - begin] != 0) continue;
    const uint64_t M = dt.out[0], r = dt.out[1], N = dt.out[2];
    if (db.out[0] != r || db.out[1] != N || db.out[2] != M || db.in[1] != dt.in[0]) continue;
    size_t ja = 0;
    for (size_t q = j + 2; q < end && q <= j + 3; ++q) {
      const Instruction& c = program[q];
      if (c.opcode == kGemmTN && c.flags == 0 && c.out[1] == r && c.out[2] == M && c.in[1] == dt.in[2] &&
          lora_skip_[q - begin] == 0) {
        ja = q;
        break;
      }
    }
    if (ja == 0) continue;
    const Instruction& da = program[ja];
    const uint64_t K = da.out[0];
    if (!k::LoraBackwardSupported(M, N, K, r)) continue;
    const uint64_t refs[7] = {dt.in[0], da.in[0], db.in[0], dt.in[1], dt.in[2], db.in[2], da.in[2]};
    const uint64_t bytes[7] = {M * N * 4, M * K * 4, M * r * 4, r * N * 4, M * r * 4, r * N * 4, K * r * 4};
    bool ok = true;
    for (int q = 0; q < 7; ++q) ok = ok && aligned(refs[q]);
    // the three outputs apart from each other and from every operand
    for (int o = 4; o < 7 && ok; ++o)
      for (int q = 0; q < 7 && ok; ++q)
        if (q != o && overlap(RefOffset(refs[o]), RefOffset(refs[o]) + bytes[o], RefOffset(refs[q]),
                              RefOffset(refs[q]) + bytes[q]))
          ok = false;
    // what the plan runs between dT and dA (an expand product, at most) neither changes an operand nor
    // looks at dB / dA, which exist early now
    for (size_t q = j + 1; q < ja && ok; ++q) {
      if (q == j + 1) continue;
      for (int w = 0; w < 5 && ok; ++w)
        if (touches(q, RefOffset(refs[w]), RefOffset(refs[w]) + bytes[w], true)) ok = false;
      for (int o = 5; o < 7 && ok; ++o)
        if (touches(q, RefOffset(refs[o]), RefOffset(refs[o]) + bytes[o], true) ||
            touches(q, RefOffset(refs[o]), RefOffset(refs[o]) + bytes[o], false))
          ok = false;
    }
    if (!ok) continue;
    AdapterBackward ab;
    ab.fuse = true;
    ab.db = db;
    ab.da = da;
    adapter_bwd_[j - begin] = ab;
    lora_skip_[j + 1 - begin] = 1;
    lora_skip_[ja - begin] = 1;
  }
}

const k::Shadow* CudaBackend::ShadowFor(uint64_t out_ref, uint64_t elems) const {
  if (!cur_shadow_.dst || RefSpace(out_ref) != kArena || RefOffset(out_ref) != cur_plan_.a_off ||
      elems != cur_plan_.M * cur_plan_.K)
    return nullptr;
  return &cur_shadow_;
}

Status CudaBackend::Flush() {
  if (!d_arena_) return {};
  cudaSetDevice(device_);
  if (coherence_ == Coherence::kStrict) {
    for (const auto& [off, bytes] : device_dirty_) {
      if (auto r = Check(cudaMemcpyAsync(host_arena_ + off, d_arena_ + off, bytes,
                                         cudaMemcpyDeviceToHost, stream_), "flush download"); !r)
        return r;
      counters_.d2h_bytes += bytes;
    }
  }
  device_dirty_.clear();
  if (auto r = Check(cudaMemcpyAsync(h_status_, d_status_, sizeof(k::DeviceStatus),
                                     cudaMemcpyDeviceToHost, stream_), "status"); !r)
    return r;
  // Completion is an error or a success, never a silent fallback.
  if (auto r = Check(cudaStreamSynchronize(stream_), "flush: device work did not complete"); !r)
    return r;
  if (auto e = cudaGetLastError(); e != cudaSuccess) return std::unexpected(CudaErr(e, "flush"));
  if (!deferred_error_.empty()) {
    std::string e;
    e.swap(deferred_error_);
    return std::unexpected(e);
  }
  if (h_status_[0] || h_status_[1]) {
    const bool refused = h_status_[0] != 0;
    cudaMemsetAsync(d_status_, 0, sizeof(k::DeviceStatus), stream_);
    cudaStreamSynchronize(stream_);
    h_status_[0] = h_status_[1] = 0;
    return std::unexpected(refused ? std::string(kNonFiniteNormRefusal)
                                   : std::string("cuda: a bounded device-side wait ran out"));
  }
  return {};
}

Status CudaBackend::Execute(const Instruction& ins, const StepParams& params) {
  if (!d_arena_) return std::unexpected("cuda: execute before bind");
  cudaSetDevice(device_);
  Extents ext;
  if (std::string e = DescribeInstruction(ins, arena_bytes_, rodata_bytes_, source_bytes_, &ext);
      !e.empty())
    return std::unexpected("cuda: " + e);
  if (!range_error_.empty()) return std::unexpected(range_error_);
  if (!host_dirty_.empty())
    if (auto r = UploadDirty(); !r) return r;
  if (fold_gather_ && !gather_folded_ &&
      (ins.opcode == kClipNorm || ins.opcode == kSqNormAccum || ins.opcode == kClipGlobal ||
       ins.opcode == kAdamWStep || ins.opcode == kSgdStep))
    if (auto r = FoldGatheredIntoArena(); !r) return r;

  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  if (profiling_) {
    const size_t slot = pending_profile_.size();
    if (slot >= events_.size()) {
      cudaEvent_t a, b;
      cudaEventCreate(&a);
      cudaEventCreate(&b);
      events_.push_back({a, b});
      cudaEvent_t c, d;
      cudaEventCreate(&c);
      cudaEventCreate(&d);
      kernel_events_.push_back({c, d});
    }
    umma::SetProfileEvents(&umma_->ctx, kernel_events_[slot].first, kernel_events_[slot].second);
    ev0 = events_[slot].first;
    ev1 = events_[slot].second;
    cudaEventRecord(ev0, stream_);
  }

  if (ins.opcode != kAddBias) skip_next_add_bias_ = false;
  cur_shadow_ = k::Shadow{};
  shadow_written_ = false;
  umma::ReleaseReservations(&umma_->ctx);
  // An activation absorbed by the preceding product: nothing runs and nothing is
  // written, so the copy the product published under this output's key stays.
  const uint8_t lora_skip = range_index_ < lora_skip_.size() ? lora_skip_[range_index_] : 0;
  const bool absorbed = skip_act_at_ == static_cast<int64_t>(range_index_) || lora_skip == 2;
  if (skip_act_at_ == static_cast<int64_t>(range_index_)) skip_act_at_ = -1;
  if (lora_skip == 2)   // an expand product deferred into a later frozen product: its output stays unwritten
    for (size_t i = 0; i < ext.count; ++i)
      if (ext.e[i].space == kArena && ext.e[i].write) elided_.push_back({ext.e[i].off, ext.e[i].off + ext.e[i].bytes});
  // (A kAddBias done by the preceding product's epilogue reads nothing either.)
  // (A kAddEW done by the kernel before it: that kernel's dispatch has already
  // dropped older copies of the sum's range and may have published the new one.)
  const bool add_done = skip_add_at_ == static_cast<int64_t>(range_index_) ||
                        skip_attn_dv_at_ == static_cast<int64_t>(range_index_) || lora_skip == 1;
  const bool bias_done = (skip_next_add_bias_ && ins.opcode == kAddBias) || add_done;
  if (!elided_.empty() && !absorbed && !bias_done) {
    for (size_t i = 0; i < ext.count; ++i) {
      const Extent& e = ext.e[i];
      if (e.space != kArena || (e.write && !e.read)) continue;
      bool hits = false;
      for (const auto& [lo, hi] : elided_)
        if (e.off < hi && lo < e.off + e.bytes) hits = true;
      if (!hits) continue;
      const bool gemm_a = (ins.flags & kFlagRelaxed) && relaxed_allowed_ && RefSpace(ins.in[0]) == kArena &&
                          RefOffset(ins.in[0]) == e.off && !e.write &&
                          (ins.opcode == kGemmNN || ins.opcode == kGemmNT || ins.opcode == kGemmNNQ8 ||
                           ins.opcode == kGemmNTQ8 || ins.opcode == kGemmNNBF16 || ins.opcode == kGemmNTBF16) &&
                          umma::TouchActCopy(&umma_->ctx, e.off,
                                             ~0ull,
                                             ins.out[0], ins.out[2]);
      const bool attn_copy = !e.write && IsAttentionCopyReader(ins, e.off) && relaxed_allowed_ &&
                             umma::TouchPack(&umma_->ctx, e.off, e.bytes / 4);
      if (!gemm_a && !attn_copy)
        return std::unexpected(std::string("cuda: ") + OpName(ins.opcode) +
                               " reads an activation whose f32 form an epilogue fusion left unwritten");
    }
  }
  if (range_index_ < shadow_plan_.size() && shadow_plan_[range_index_].want) {
    cur_plan_ = shadow_plan_[range_index_];
    if (range_index_ < act_fusion_.size() && act_fusion_[range_index_].mode != 0)
      // The product reads one copy and writes another: keep its operand's slot.
      umma::TouchActCopy(&umma_->ctx, RefOffset(ins.in[0]),
                         ~0ull,
                         ins.out[0], ins.out[2]);
    if (uint16_t* buf = umma::ReserveShadow(&umma_->ctx, cur_plan_.M * cur_plan_.K)) {
      cur_shadow_.dst = buf;
      cur_shadow_.k_scale = cur_plan_.scale_ref == kNullRef ? nullptr : Rd(cur_plan_.scale_ref);
      cur_shadow_.cols = cur_plan_.K;
      cur_shadow_.only = cur_plan_.only;
    }
  }

  if (range_index_ == 0 && !lora_weights_.empty()) {   // every adapter matrix of the range, cut once
    k::LoraSplitWeights(d_lora_table_, static_cast<int>(lora_weights_.size()), lora_max_n_, stream_);
    ++counters_.kernel_launches;
  }
  const uint64_t fused_before = counters_.fused_dispatches;
  if (!absorbed && lora_skip != 1)
    if (auto r = Dispatch(ins, params, ext); !r) return r;
  ++counters_.instructions;

  if (profiling_) {
    cudaEventRecord(ev1, stream_);
    ProfileRecord rec{ins.opcode, range_index_, 0.0f, 0, 0, 0};
    rec.has_kernel = umma::ProfileEventsUsed(&umma_->ctx);
    rec.absorbed = static_cast<uint16_t>(counters_.fused_dispatches - fused_before);
    if (ins.opcode <= kGemmAccNN || ins.opcode == kGemmNNQ8 || ins.opcode == kGemmNTQ8 ||
        ins.opcode == kGemmNNBF16 || ins.opcode == kGemmNTBF16) {
      rec.m = ins.out[0]; rec.n = ins.out[1]; rec.k = ins.out[2];
    }
    pending_profile_.push_back(rec);
  }
  ++range_index_;

  for (size_t i = 0; i < ext.count && !absorbed; ++i) {
    const Extent& e = ext.e[i];
    if (!e.write) continue;
    if (lora_rows_tag_.valid && lora_rows_tag_.producer + 1 != range_index_ && e.space == kArena &&
        e.off < lora_rows_tag_.off + lora_rows_tag_.M * lora_rows_tag_.r * 4 && lora_rows_tag_.off < e.off + e.bytes)
      lora_rows_tag_.valid = false;
    if (!add_done) umma::InvalidateRange(&umma_->ctx, e.off, e.bytes);
    if (coherence_ == Coherence::kStrict) MergeExtent(&device_dirty_, e.off, e.bytes);
    if (!elided_.empty() && e.space == kArena) {   // written for real: no longer stale
      std::vector<std::pair<uint64_t, uint64_t>> rest;
      for (const auto& [lo, hi] : elided_) {
        if (e.off + e.bytes <= lo || hi <= e.off) { rest.push_back({lo, hi}); continue; }
        if (lo < e.off) rest.push_back({lo, e.off});
        if (e.off + e.bytes < hi) rest.push_back({e.off + e.bytes, hi});
      }
      elided_.swap(rest);
    }
  }
  if (shadow_written_ && cur_shadow_.only && (ins.opcode == kSoftmaxXEntBwd || ins.opcode == kSoftmaxXEntMaskedBwd))
    elided_.push_back({cur_plan_.a_off, cur_plan_.a_off + cur_plan_.M * cur_plan_.K * 4});
  elided_.insert(elided_.end(), pending_elided_.begin(), pending_elided_.end());
  pending_elided_.clear();
  if (shadow_written_)   // after the instruction's own writes have invalidated the range
    umma::CommitShadow(&umma_->ctx, cur_shadow_.dst, cur_plan_.a_off, cur_plan_.scale_off,
                       cur_plan_.M, cur_plan_.K);
  if (pending_pack_.rows) {
    umma::CommitPack(&umma_->ctx, pending_pack_.rows, pending_pack_.off, pending_pack_.elems);
    pending_pack_ = PendingPack{};
  }
  for (size_t i = 0; i < deferred_elided_.size();) {   // (range_index_ has moved past this instruction)
    if (deferred_elided_[i].after + 1 == range_index_) {
      elided_.push_back({deferred_elided_[i].lo, deferred_elided_[i].hi});
      deferred_elided_.erase(deferred_elided_.begin() + static_cast<long>(i));
    } else {
      ++i;
    }
  }
  if (auto e = cudaPeekAtLastError(); e != cudaSuccess) {
    cudaGetLastError();
    return std::unexpected(CudaErr(e, OpName(ins.opcode)));
  }
  return {};
}

k::GemmArgs CudaBackend::GemmArgsOf(const Instruction& ins) const {
  k::GemmArgs a;
  a.A = Rd(ins.in[0]);
  a.B = Rd<uint8_t>(ins.in[1]);
  a.C = Wr(ins.in[2]);
  a.M = ins.out[0]; a.N = ins.out[1]; a.K = ins.out[2];
  const uint16_t op = ins.opcode;
  a.b_transposed = op == kGemmNT || op == kGemmNTQ8 || op == kGemmNTBF16;
  a.a_transposed = op == kGemmTN;
  a.b_type = (op == kGemmNNQ8 || op == kGemmNTQ8) ? k::BType::kI8
             : (op == kGemmNNBF16 || op == kGemmNTBF16) ? k::BType::kBf16 : k::BType::kF32;
  a.act = ActOf(ins.flags);
  if (ins.flags & kFlagEpilogueBias) a.bias = Rd(ins.in[3]);
  if (ins.flags & kFlagGemmAddend) a.addend = Rd(ins.in[3]);
  if (op == kGemmNN || op == kGemmNT || op == kGemmTN) a.alpha = GemmAlphaOf(ins.imm);
  if (op == kGemmAccNN) { a.alpha = BitsToF32(ins.in[3]); a.accumulate = true; }
  if (op == kGemmNNQ8 || op == kGemmNTQ8) {
    if (ins.flags & kFlagQ8ColScale) {
      if (a.b_transposed) a.a_k_scale = Rd(ins.in[3]); else a.b_col_scale = Rd(ins.in[3]);
    } else {
      a.alpha = BitsToF32(ins.in[3]);
    }
  }
  return a;
}

Status CudaBackend::DispatchGemm(const Instruction& ins) {
  k::GemmArgs a = GemmArgsOf(ins);
  // The relaxed permission: frozen-weight products may run on the bf16 tensor
  // cores (activation rounded to bf16 once, weight exact, f32 accumulate).
  if ((ins.flags & kFlagRelaxed) && relaxed_allowed_ && !a.a_transposed && !a.accumulate &&
      RefSpace(ins.in[1]) != kArena) {
    const BiasFusion* fuse = range_index_ < bias_fusion_.size() && bias_fusion_[range_index_].fuse
                                 ? &bias_fusion_[range_index_] : nullptr;
    if (fuse) {   // the following kAddBias, done in this product's epilogue
      a.bias = Rd(fuse->bias_ref);
      a.C = Wr(fuse->out_ref);
    }
    const AddFusion* adf = range_index_ < add_fusion_.size() && add_fusion_[range_index_].fuse
                               ? &add_fusion_[range_index_] : nullptr;
    if (adf) {   // the kAddEW after it (after the fused kAddBias, if any): the epilogue's addend
      a.addend = Rd(adf->x_ref);
      a.addend_after_bias = true;
      a.C = Wr(adf->out_ref);
    }
    const ActFusion* af = range_index_ < act_fusion_.size() && act_fusion_[range_index_].mode != 0 &&
                                  cur_shadow_.dst ? &act_fusion_[range_index_] : nullptr;
    if (af) {   // and the activation after it: its result leaves as the consumer's bf16 operand
      a.fuse_mode = af->mode;
      a.fuse_act = af->act;
      a.fuse_x = af->x_ref == kNullRef ? nullptr : Rd(af->x_ref);
      a.fuse_shadow = cur_shadow_.dst;
      a.fuse_shadow_scale = cur_shadow_.k_scale;
      a.store_c = af->store_c;
    }
    const LoraFold* lf = range_index_ < lora_fold_.size() && lora_fold_[range_index_].fuse
                             ? &lora_fold_[range_index_] : nullptr;
    if (lf) {   // the adapter's expand product rides this product's reduction
      bool pieces_made = false;
      if (lf->kind == 1) {   // its down product t = x A first (the plan has it after this instruction)
        k::GemmArgs d = GemmArgsOf(lf->down);
        d.contract_fma = adapter_fma_;
        // (the tensor-core form of it leaves t's bf16 cut in the same launch)
        pieces_made = adapter_fma_ && lf->down.flags == 0 && d.N == lf->r && k::LoraDownSupported(d.M, d.K, d.N) &&
                      k::LoraDown(d.A, static_cast<const float*>(d.B), d.C, d.M, d.K, d.N, d.alpha, stream_,
                                  d_lora_t_);
        if (!pieces_made) k::GemmExact(d, stream_);
        ++counters_.kernel_launches;
        umma::InvalidateRange(&umma_->ctx, RefOffset(lf->down.in[2]), d.M * d.N * 4);
      }
      if (!pieces_made && lf->kind != 1 && lora_rows_tag_.valid && lora_rows_tag_.off == RefOffset(lf->t_ref) &&
          lora_rows_tag_.M == a.M && lora_rows_tag_.r == lf->r)
        pieces_made = true;   // the adapter backward left dT's cut in the scratch
      else
        lora_rows_tag_.valid = false;   // the scratch is rewritten below (or was, by the down product)
      if (!pieces_made) {
        if (!k::LoraSplitRows(Rd(lf->t_ref), d_lora_t_, a.M, lf->r, stream_))
          return std::unexpected("cuda: low-rank fold: the factor cannot be split (rank or alignment)");
        ++counters_.kernel_launches;
      }
      const uint32_t kx = k::LoraSplitColumns(lf->r);
      a.aux_a = d_lora_t_;
      a.aux_b = d_lora_w_ + static_cast<uint64_t>(lf->weight_slot) * lora_max_n_ * lora_max_kx_;
      a.aux_k = kx;
      a.C = Wr(lf->out_ref);
      if (lf->addend_ref != kNullRef) {
        a.addend = Rd(lf->addend_ref);
        a.addend_after_bias = true;
      }
    }
    uint16_t* pack_rows = nullptr;
    if (range_index_ < pack_plan_.size() && pack_plan_[range_index_].S != 0 && !af &&
        RefOffset(pack_plan_[range_index_].out_ref) == static_cast<uint64_t>(reinterpret_cast<uint8_t*>(a.C) - d_arena_)) {
      pack_rows = umma::ReservePack(&umma_->ctx, a.M * a.N);
      if (pack_rows) {
        a.pack_dst = pack_rows;
        if (pack_plan_[range_index_].copy_only) a.store_c = false;
      }
    }
    int launches = 0;
    const std::string err = umma::TryGemm(&umma_->ctx, a, RefSpace(ins.in[1]) == kRodata ? 1 : 2,
                                          RefOffset(ins.in[1]), RefOffset(ins.in[0]),
                                          a.a_k_scale ? ins.in[3] : ~0ull,   // the whole ref: its address space is part of the key
                                          stream_,
                                          &launches);
    if (err.empty() && launches > 0) {
      ++counters_.relaxed_executions;
      counters_.kernel_launches += launches;
      skip_next_add_bias_ = fuse != nullptr;
      if (fuse) ++counters_.fused_dispatches;
      if (adf) {
        ++counters_.fused_dispatches;
        skip_add_at_ = static_cast<int64_t>(adf->add_index);
        umma::InvalidateRange(&umma_->ctx, RefOffset(adf->out_ref), a.M * a.N * 4);
        if (adf->z_hi > adf->z_lo) pending_elided_.push_back({adf->z_lo, adf->z_hi});
      }
      if (af) {
        ++counters_.fused_dispatches;
        shadow_written_ = true;
        skip_act_at_ = static_cast<int64_t>(af->act_index);
        for (int e = 0; e < af->elided_count; ++e)
          pending_elided_.push_back({af->elided[e][0], af->elided[e][1]});
      }
      if (lf) {
        counters_.fused_dispatches += lf->absorbed;
        umma::InvalidateRange(&umma_->ctx, RefOffset(lf->out_ref), a.M * a.N * 4);
        for (int e = 0; e < lf->dead_count; ++e) pending_elided_.push_back({lf->dead[e][0], lf->dead[e][1]});
      }
      if (pack_rows) {   // published once this instruction's own write extents have dropped older copies
        const uint64_t c_off = static_cast<uint64_t>(reinterpret_cast<uint8_t*>(a.C) - d_arena_);
        pending_pack_ = PendingPack{pack_rows, c_off, a.M * a.N};
        if (!a.store_c) deferred_elided_.push_back({pack_plan_[range_index_].last, c_off, c_off + a.M * a.N * 4});
      }
      return {};
    }
    a.pack_dst = nullptr;
    if (!err.empty()) return std::unexpected("cuda: " + err);
    if (lf) return std::unexpected("cuda: low-rank fold: the tensor-core path refused a product it was planned on");
    // launches == 0: the shape is outside the tensor-core kernel's domain.
    if (fuse) {
      a.bias = nullptr;
      a.C = Wr(ins.in[2]);
    }
    if (adf) {
      a.addend = nullptr;
      a.addend_after_bias = false;
      a.C = Wr(ins.in[2]);
    }
    a.fuse_mode = 0;
    a.fuse_x = nullptr;
    a.fuse_shadow = nullptr;
    a.fuse_shadow_scale = nullptr;
    a.store_c = true;
  }
  // An adapter site's three backward products in one pass (this is the first of them).
  if (range_index_ < adapter_bwd_.size() && adapter_bwd_[range_index_].fuse) {
    const AdapterBackward& ab = adapter_bwd_[range_index_];
    k::LoraBackwardArgs b;
    b.dy = Rd(ins.in[0]); b.B = Rd(ins.in[1]); b.dt = Wr(ins.in[2]);
    b.t = Rd(ab.db.in[0]); b.dB = Wr(ab.db.in[2]);
    b.x = Rd(ab.da.in[0]); b.dA = Wr(ab.da.in[2]);
    b.partials = d_lora_partials_;
    b.partials_floats = lora_partials_capacity_;
    b.M = ins.out[0]; b.r = ins.out[1]; b.N = ins.out[2]; b.K = ab.da.out[0];
    b.alpha_dt = GemmAlphaOf(ins.imm); b.alpha_db = GemmAlphaOf(ab.db.imm); b.alpha_da = GemmAlphaOf(ab.da.imm);
    // dT's bf16 cut in the same pass, for the fold that takes dT A^T a few instructions on.
    const bool cut = lora_fold_enabled_ && d_lora_t_ != nullptr &&
                     b.M * k::LoraSplitColumns(static_cast<uint32_t>(b.r)) <= lora_t_capacity_;
    if (cut) b.dt_pieces = d_lora_t_;
    lora_rows_tag_.valid = false;
    int tensor_launches = 0;
    if (const std::string err = umma::TryLoraBackward(&umma_->ctx, b, stream_, &tensor_launches); !err.empty())
      return std::unexpected("cuda: " + err);
    if (tensor_launches == 0 && !k::LoraBackward(b, stream_))
      return std::unexpected("cuda: the fused adapter backward refused a site it was planned on");
    if (cut) lora_rows_tag_ = LoraRowsTag{true, RefOffset(ins.in[2]), b.M, static_cast<uint32_t>(b.r), range_index_};
    counters_.kernel_launches += 3;
    counters_.fused_dispatches += 2;
    umma::InvalidateRange(&umma_->ctx, RefOffset(ab.db.in[2]), b.r * b.N * 4);
    umma::InvalidateRange(&umma_->ctx, RefOffset(ab.da.in[2]), b.K * b.r * 4);
    return {};
  }
  // The forward's down product t = x A on the tensor cores (3xTF32) where the bits are not observed.
  if (coherence_ == Coherence::kLazy && adapter_fma_ && ins.opcode == kGemmNN && ins.flags == 0 &&
      RefSpace(ins.in[1]) == kArena && k::LoraDownSupported(a.M, a.K, a.N) &&
      k::LoraDown(a.A, static_cast<const float*>(a.B), a.C, a.M, a.K, a.N, a.alpha, stream_)) {
    ++counters_.kernel_launches;
    return {};
  }
  // Large exact f32 products: bf16 pieces on the tensor cores where the bits are not observed.
  if (SplitGemmOn() && (ins.opcode == kGemmNN || ins.opcode == kGemmNT || ins.opcode == kGemmTN) &&
      umma::SplitGemmEligible(a)) {
    int launches = 0;
    const std::string err = umma::TrySplitGemm(&umma_->ctx, a,
                                               RefSpace(ins.in[1]) == kArena ? 0 : (RefSpace(ins.in[1]) == kRodata ? 1 : 2),
                                               RefOffset(ins.in[1]), stream_, &launches);
    if (!err.empty()) return std::unexpected("cuda: " + err);
    if (launches > 0) {
      counters_.kernel_launches += launches;
      ++counters_.split_executions;
      return {};
    }
  }
  // The split-K scratch is sized per range (BeginRange); an instruction executed
  // outside any range simply runs unsplit.
  a.split_scratch = d_split_;
  a.split_scratch_floats = split_capacity_;
  const AddFusion* tail = !(ins.flags & kFlagRelaxed) && range_index_ < add_fusion_.size() &&
                                  add_fusion_[range_index_].fuse ? &add_fusion_[range_index_] : nullptr;
  if (tail) {   // the kAddEW after a rank-r expand product rides its kernel
    a.tail_addend = Rd(tail->x_ref);
    a.tail_out = Wr(tail->out_ref);
  }
  // The engine does not observe whether a rank-r product rounded once or twice per term.
  a.contract_fma = coherence_ == Coherence::kLazy && adapter_fma_;
  const bool tail_done = k::GemmExact(a, stream_);
  ++counters_.kernel_launches;
  if (tail && tail_done) {
    ++counters_.fused_dispatches;
    skip_add_at_ = static_cast<int64_t>(tail->add_index);
    umma::InvalidateRange(&umma_->ctx, RefOffset(tail->out_ref), a.M * a.N * 4);
    if (tail->z_hi > tail->z_lo) pending_elided_.push_back({tail->z_lo, tail->z_hi});
  }
  return {};
}

k::AdamScalars CudaBackend::ScalarsOf(const StepParams& params) {
  k::AdamScalars sc{};
  sc.lr = params.lr; sc.beta1 = params.beta1; sc.beta2 = params.beta2; sc.eps = params.eps;
  sc.weight_decay = params.weight_decay;
  sc.inv_bc1 = 1.0f / (1.0f - std::pow(params.beta1, static_cast<float>(params.step)));
  sc.inv_bc2 = 1.0f / (1.0f - std::pow(params.beta2, static_cast<float>(params.step)));
  return sc;
}

void CudaBackend::SetCapturing(bool on) { capturing_ = on; }

Status CudaBackend::UploadStepScalars(const StepParams& params) {
  cudaSetDevice(device_);
  scalar_slot_ = (scalar_slot_ + 1) % kScalarSlots;
  // The slot's previous upload may still be queued behind device work when the
  // host runs many steps ahead: its bytes must not change until that copy ran.
  if (auto r = Check(cudaEventSynchronize(scalar_done_[scalar_slot_]), "step scalars: slot"); !r) return r;
  h_scalars_[scalar_slot_] = ScalarsOf(params);
  if (auto r = Check(cudaMemcpyAsync(d_scalars_, &h_scalars_[scalar_slot_], sizeof(k::AdamScalars),
                                     cudaMemcpyHostToDevice, stream_), "step scalars"); !r)
    return r;
  if (auto r = Check(cudaEventRecord(scalar_done_[scalar_slot_], stream_), "step scalars: event"); !r) return r;
  last_params_ = params;
  scalars_valid_ = true;
  return {};
}

// The rank-ordered mean of the gathered gradient copies, written over this
// rank's own block in the arena (what a host-side exchange leaves there), for
// ranges whose clip instructions work on the arena in place.
Status CudaBackend::FoldGatheredIntoArena() {
  if (!d_gathered_ || gather_bytes_ == 0 || gather_off_ + gather_bytes_ > arena_bytes_)
    return std::unexpected("cuda: data parallel: the gathered gradient block is not set");
  const size_t n = gather_bytes_ / 4;
  k::SumCopies(reinterpret_cast<const float*>(d_gathered_), reinterpret_cast<float*>(d_arena_ + gather_off_), n,
               gather_ranks_, n, 1.0f / static_cast<float>(gather_ranks_), stream_);
  ++counters_.kernel_launches;
  umma::InvalidateRange(&umma_->ctx, gather_off_, gather_bytes_);
  if (coherence_ == Coherence::kStrict) MergeExtent(&device_dirty_, gather_off_, gather_bytes_);
  gather_folded_ = true;
  return {};
}

Status CudaBackend::DispatchOptimizer(const Instruction& ins, const StepParams& params) {
  // Per-range scalars, computed with the host libm exactly as the CPU executor
  // computes them (reference: runtime/executor/optimizer.cc:113-118), uploaded
  // once per distinct StepParams.
  if (!scalars_valid_ || std::memcmp(&params, &last_params_, sizeof(StepParams)) != 0) {
    // A range being captured must not contain the upload (a replay would re-read
    // the pinned slot with whatever the host has put there since).
    if (capturing_)
      return std::unexpected("cuda: step scalars must be uploaded before a range is captured");
    if (auto r = UploadStepScalars(params); !r) return r;
  }
  if (range_index_ < adam_group_of_.size() && adam_group_of_[range_index_] != -1) {
    const int32_t gi = adam_group_of_[range_index_];
    if (gi == -2) return {};   // done by the run's first instruction
    const AdamGroup& grp = adam_groups_[gi];
    k::AdamWStepMulti(d_adam_table_ + grp.table_begin, grp.count, grp.max_n, d_scalars_, d_status_,
                      gather_ranks_ > 1 && !fold_gather_ ? 1.0f / static_cast<float>(gather_ranks_) : 1.0f,
                      stream_);
    ++counters_.kernel_launches;
    return {};
  }
  const uint64_t n = ins.out[0];
  const float clip = BitsToF32(ins.out[1]);
  const uint64_t g_off = RefOffset(ins.in[1]);
  const float* g = Rd(ins.in[1]);
  int copies = 1;
  size_t cstride = 0;
  float inv = 1.0f;
  if (gather_ranks_ > 1 && !fold_gather_ && RefSpace(ins.in[1]) == kArena && g_off >= gather_off_ &&
      g_off + n * 4 <= gather_off_ + gather_bytes_) {
    g = reinterpret_cast<const float*>(d_gathered_ + (g_off - gather_off_));
    copies = gather_ranks_;
    cstride = gather_bytes_ / 4;
    inv = 1.0f / static_cast<float>(gather_ranks_);
  }
  const float* clip_scale = nullptr;
  if (clip > 0.0f) {
    const float* norm_src = g;
    if (copies > 1) {  // the clip norm is taken on the summed gradient
      if (n > gsum_capacity_) return std::unexpected("cuda: gradient-sum scratch not sized");
      k::SumCopies(g, d_gsum_, n, copies, cstride, inv, stream_);
      norm_src = d_gsum_;
      ++counters_.kernel_launches;
    }
    k::L2Squared(norm_src, n, d_partials_, d_sq_, stream_);
    k::ClipScaleFromSq(d_sq_, clip, d_clip_scale_, d_status_, stream_);
    counters_.kernel_launches += 3;
    clip_scale = d_clip_scale_;
  }
  if (ins.opcode == kAdamWStep)
    k::AdamWStep(Wr(ins.in[0]), g, Wr(ins.in[2]), Wr(ins.in[3]), n, d_scalars_, clip_scale,
                 d_status_, copies, cstride, inv, stream_);
  else
    k::SgdStep(Wr(ins.in[0]), g, n, d_scalars_, clip_scale, d_status_, copies, cstride, inv,
               stream_);
  ++counters_.kernel_launches;
  return {};
}

Status CudaBackend::Dispatch(const Instruction& ins, const StepParams& params, const Extents&) {
  cudaStream_t s = stream_;
  auto launched = [&](int n = 1) { counters_.kernel_launches += n; };
  switch (static_cast<Op>(ins.opcode)) {
    case kNop: break;
    case kGemmNN: case kGemmNT: case kGemmTN: case kGemmAccNN: case kGemmNNQ8: case kGemmNTQ8:
    case kGemmNNBF16: case kGemmNTBF16:
      return DispatchGemm(ins);
    case kAddEW:
      if (skip_add_at_ == static_cast<int64_t>(range_index_)) {   // done as the preceding product's addend
        skip_add_at_ = -1;
        break;
      }
      shadow_written_ = k::AddEW(Rd(ins.in[0]), Rd(ins.in[1]), Wr(ins.in[2]), ins.out[0], s,
                                 ShadowFor(ins.in[2], ins.out[0]));
      launched();
      break;
    case kMulEW: k::MulEW(Rd(ins.in[0]), Rd(ins.in[1]), Wr(ins.in[2]), ins.out[0], s); launched(); break;
    case kAddBias:
      if (skip_next_add_bias_) {   // the preceding product's epilogue already wrote this output
        skip_next_add_bias_ = false;
        break;
      }
      k::AddBias(Rd(ins.in[0]), Rd(ins.in[1]), Wr(ins.in[2]), ins.out[0], ins.out[1], s); launched(); break;
    case kReluFwd:
      shadow_written_ = k::ActFwd(kActRelu, Rd(ins.in[0]), Wr(ins.in[1]), ins.out[0], s,
                                  ShadowFor(ins.in[1], ins.out[0]));
      launched();
      break;
    case kGeluFwd:
      shadow_written_ = k::ActFwd(kActGelu, Rd(ins.in[0]), Wr(ins.in[1]), ins.out[0], s,
                                  ShadowFor(ins.in[1], ins.out[0]));
      launched();
      break;
    case kSiluFwd:
      shadow_written_ = k::ActFwd(kActSilu, Rd(ins.in[0]), Wr(ins.in[1]), ins.out[0], s,
                                  ShadowFor(ins.in[1], ins.out[0]));
      launched();
      break;
    case kReluBwd:
      shadow_written_ = k::ActBwd(kActRelu, Rd(ins.in[0]), Rd(ins.in[1]), Wr(ins.in[2]), ins.out[0], s,
                                  ShadowFor(ins.in[2], ins.out[0]));
      launched();
      break;
    case kGeluBwd:
      shadow_written_ = k::ActBwd(kActGelu, Rd(ins.in[0]), Rd(ins.in[1]), Wr(ins.in[2]), ins.out[0], s,
                                  ShadowFor(ins.in[2], ins.out[0]));
      launched();
      break;
    case kSiluBwd:
      shadow_written_ = k::ActBwd(kActSilu, Rd(ins.in[0]), Rd(ins.in[1]), Wr(ins.in[2]), ins.out[0], s,
                                  ShadowFor(ins.in[2], ins.out[0]));
      launched();
      break;
    case kScale:
      k::Scale(Rd(ins.in[0]), Wr(ins.in[1]), BitsToF32(ins.in[2]), ins.out[0], s); launched(); break;
    case kFill: k::Fill(Wr(ins.in[0]), BitsToF32(ins.in[1]), ins.out[0], s); launched(); break;
    case kCopy: k::Copy(Rd(ins.in[0]), Wr(ins.in[1]), ins.out[0], s); launched(); break;
    case kAccumulate: k::Accumulate(Wr(ins.in[0]), Rd(ins.in[1]), ins.out[0], s); launched(); break;
    case kReduceRows:
      k::ReduceRows(Rd(ins.in[0]), Wr(ins.in[1]), ins.out[0], ins.out[1], s); launched(); break;
    case kFusedMap:
      k::FusedMap(Rd(ins.in[0]), ins.in[1] == kNullRef ? nullptr : Rd(ins.in[1]),
                  ins.in[2] == kNullRef ? nullptr : Rd(ins.in[2]), Wr(ins.in[3]), ins.out[0],
                  static_cast<uint32_t>(ins.out[1]), BitsToF32(ins.out[2]),
                  BitsToF32(ins.out[2] >> 32), s);
      launched();
      break;
    case kEmbedFwd:
      k::EmbedFwd(Rd<int32_t>(ins.in[0]), Rd(ins.in[1]), Wr(ins.in[2]), ins.out[0],
                  Lo32(ins.out[1]), Hi32(ins.out[1]), s);
      launched();
      break;
    case kLayerNormFwd:
      shadow_written_ = k::LayerNormFwd(
          Rd(ins.in[0]), Rd(ins.in[1]), Rd(ins.in[2]), Wr(ins.in[3]), Wr(ins.out[1]), Wr(ins.out[2]),
          Hi32(ins.out[0]), Lo32(ins.out[0]), NormEpsOf(ins.imm), s,
          ShadowFor(ins.in[3], Hi32(ins.out[0]) * Lo32(ins.out[0])));
      launched();
      break;
    case kLayerNormBwd: {
      const AddFusion* adf = range_index_ < add_fusion_.size() && add_fusion_[range_index_].fuse
                                 ? &add_fusion_[range_index_] : nullptr;
      const int fused = k::LayerNormBwd(Rd(ins.in[0]), Rd(ins.in[1]), Rd(ins.in[2]), Rd(ins.out[0]),
                                         Rd(ins.out[1]), Wr(ins.in[3]), Hi32(ins.out[2]), Lo32(ins.out[2]), s,
                                         adf ? Rd(adf->x_ref) : nullptr, adf ? Wr(adf->out_ref) : nullptr,
                                         adf ? ShadowFor(adf->out_ref, static_cast<uint64_t>(Hi32(ins.out[2])) *
                                                                           Lo32(ins.out[2])) : nullptr);
      launched();
      if (fused) {   // the kAddEW after it has been done
        shadow_written_ = fused == 2;
        umma::InvalidateRange(&umma_->ctx, RefOffset(adf->out_ref),
                              static_cast<uint64_t>(Hi32(ins.out[2])) * Lo32(ins.out[2]) * 4);
        ++counters_.fused_dispatches;
        skip_add_at_ = static_cast<int64_t>(adf->add_index);
        if (adf->z_hi > adf->z_lo) pending_elided_.push_back({adf->z_lo, adf->z_hi});
      }
      break;
    }
    case kRmsNormFwd:
      k::RmsNormFwd(Rd(ins.in[0]), Rd(ins.in[1]), Wr(ins.in[2]), Wr(ins.in[3]), Hi32(ins.out[0]),
                    Lo32(ins.out[0]), NormEpsOf(ins.imm), s);
      launched();
      break;
    case kRmsNormBwd:
      k::RmsNormBwd(Rd(ins.in[0]), Rd(ins.in[1]), Rd(ins.in[2]), Rd(ins.out[0]), Wr(ins.in[3]),
                    Hi32(ins.out[1]), Lo32(ins.out[1]), s);
      launched();
      break;
    case kSoftmaxXEntFwd: case kSoftmaxXEntMaskedFwd:
    {
      if (auto r = EnsureScratch(ins.out[0]); !r) return r;
      const LossFusion* lf = range_index_ < loss_fusion_.size() && loss_fusion_[range_index_].fuse &&
                                     cur_shadow_.dst ? &loss_fusion_[range_index_] : nullptr;
      k::XEntFusedBwd fb;
      if (lf) {
        fb.shadow = cur_shadow_;
        fb.seed = lf->seed;
        fb.store_probs = lf->store_probs;
      }
      const bool fused = k::SoftmaxXEntFwd(ins.opcode == kSoftmaxXEntMaskedFwd, Rd(ins.in[0]),
                                           Rd<int32_t>(ins.in[1]), Wr(ins.in[2]), Wr(ins.in[3]), ins.out[0],
                                           ins.out[1], d_rows_, d_count_, s, lf ? &fb : nullptr);
      launched(2);
      if (fused) {   // the backward instruction two places on has been done
        shadow_written_ = true;
        skip_act_at_ = static_cast<int64_t>(lf->bwd_index);
        ++counters_.fused_dispatches;
        pending_elided_.push_back({cur_plan_.a_off, cur_plan_.a_off + cur_plan_.M * cur_plan_.K * 4});
        if (!lf->store_probs) pending_elided_.push_back({lf->probs_lo, lf->probs_hi});
      }
      break;
    }
    case kSoftmaxXEntBwd: case kSoftmaxXEntMaskedBwd:
      shadow_written_ = k::SoftmaxXEntBwd(
          ins.opcode == kSoftmaxXEntMaskedBwd, Rd(ins.in[0]), Rd<int32_t>(ins.in[1]), Rd(ins.in[2]),
          Wr(ins.in[3]), ins.out[0], ins.out[1], d_count_, s, ShadowFor(ins.in[3], ins.out[0] * ins.out[1]));
      launched(ins.opcode == kSoftmaxXEntMaskedBwd ? 2 : 1);
      break;
    case kMseFwd:
      if (auto r = EnsureScratch(256); !r) return r;
      k::MseFwd(Rd(ins.in[0]), Rd(ins.in[1]), Wr(ins.in[2]), ins.out[0], d_rows_, s);
      launched(2);
      break;
    case kMseBwd:
      k::MseBwd(Rd(ins.in[0]), Rd(ins.in[1]), Rd(ins.in[2]), Wr(ins.in[3]), ins.out[0], s);
      launched();
      break;
    case kKLDistillFwd: {
      const float T = BitsToF32(ins.out[2]);
      const uint64_t hi = ins.out[2] >> 32;
      if (!std::isfinite(T) || !(T > 0.0f)) return std::unexpected("cuda: kl.fwd: temperature");
      if (auto r = EnsureScratch(Hi32(ins.out[1])); !r) return r;
      k::KLDistillFwd(Rd(ins.in[0]), Rd(ins.in[1]), Wr(ins.in[2]), Wr(ins.in[3]), Wr(ins.out[0]),
                      Hi32(ins.out[1]), Lo32(ins.out[1]), T, hi == 0 ? 1.0f : BitsToF32(hi),
                      d_rows_, s);
      launched(2);
      break;
    }
    case kKLDistillBwd: {
      const float T = BitsToF32(ins.out[1]);
      const uint64_t hi = ins.out[1] >> 32;
      if (!std::isfinite(T) || !(T > 0.0f)) return std::unexpected("cuda: kl.bwd: temperature");
      k::KLDistillBwd(Rd(ins.in[0]), Rd(ins.in[1]), Rd(ins.in[2]), Wr(ins.in[3]), Hi32(ins.out[0]),
                      Lo32(ins.out[0]), T, hi == 0 ? 1.0f : BitsToF32(hi), s);
      launched();
      break;
    }
    case kSgdStep: case kAdamWStep:
      return DispatchOptimizer(ins, params);
    case kClipNorm: {
      const float cap = BitsToF32(ins.in[1]);
      if (!std::isfinite(cap) || !(cap > 0.0f)) return std::unexpected(kClipThresholdRefusal);
      k::L2Squared(Rd(ins.in[0]), ins.out[0], d_partials_, d_sq_, s);
      k::ClipScaleFromSq(d_sq_, cap, d_clip_scale_, d_status_, s);
      k::ScaleInPlaceBy(Wr(ins.in[0]), ins.out[0], d_clip_scale_, d_status_, s);
      launched(4);
      break;
    }
    case kSqNormAccum:
      k::L2Squared(Rd(ins.in[0]), ins.out[0], d_partials_, d_sq_, s);
      k::SqNormAccum(d_sq_, Wr(ins.in[1]), s);
      launched(3);
      break;
    case kClipGlobal: {
      const float cap = BitsToF32(ins.in[2]);
      if (!std::isfinite(cap) || !(cap > 0.0f)) return std::unexpected(kClipThresholdRefusal);
      k::ClipGlobalScale(Rd(ins.in[1]), cap, d_clip_scale_, d_status_, s);
      k::ScaleInPlaceBy(Wr(ins.in[0]), ins.out[0], d_clip_scale_, d_status_, s);
      launched(2);
      break;
    }
    case kRopeTable: {
      const uint64_t S = Hi32(ins.out[0]), d = Lo32(ins.out[0]);
      const float step = std::pow(BitsToF32(ins.out[1]), -2.0f / static_cast<float>(d));
      k::RopeTable(Wr(ins.in[0]), S, d, step, s);
      launched();
      break;
    }
    case kRopeFwd: case kRopeBwd: {
      const uint64_t d = Lo32(ins.out[1]);
      const float step = std::pow(BitsToF32(ins.out[2]), -2.0f / static_cast<float>(d));
      k::Rope(ins.opcode == kRopeBwd, Rd(ins.in[0]), Wr(ins.in[1]), Hi32(ins.out[0]),
              Lo32(ins.out[0]), Hi32(ins.out[1]), d, step,
              ins.in[2] == kNullRef ? nullptr : Rd(ins.in[2]), s);
      launched();
      break;
    }
    case kSegmentStarts:
      k::SegmentStarts(Rd<int32_t>(ins.in[0]), Wr<int32_t>(ins.in[1]), Hi32(ins.out[0]),
                       Lo32(ins.out[0]), static_cast<int32_t>(ins.out[1]), s);
      launched();
      break;
    case kAttnFwd:
      k::AttnFwd(Rd(ins.in[0]), Rd(ins.in[1]), Rd(ins.in[2]), Wr(ins.in[3]), Wr(ins.out[0]), nullptr,
                 Hi32(ins.out[1]), Lo32(ins.out[1]), Hi32(ins.out[2]), Lo32(ins.out[2]), nullptr, s);
      launched();
      break;
    case kAttnFwdSeg: {
      const AttnGeom g = UnpackAttnGeom(ins.out[1]);
      k::AttnFwd(Rd(ins.in[0]), Rd(ins.in[1]), Rd(ins.in[2]), Wr(ins.in[3]), Wr(ins.out[0]), nullptr,
                 g.B, g.S, g.H, g.d, Rd<int32_t>(ins.out[2]), s);
      launched();
      break;
    }
    case kAttnFwdTiled:
      if ((ins.flags & kFlagRelaxed) && relaxed_allowed_) {
        umma::AttentionOperands op{Rd(ins.in[0]), Rd(ins.in[1]), Rd(ins.in[2]), nullptr,
                                   RefOffset(ins.in[0]), RefOffset(ins.in[1]), RefOffset(ins.in[2]), 0,
                                   Wr(ins.out[0]), Wr(ins.in[3]),
                                   Hi32(ins.out[1]), Lo32(ins.out[1]), Hi32(ins.out[2]), Lo32(ins.out[2]),
                                   k::Shadow{}};
        const uint64_t elems = op.B * op.S * op.H * op.d;
        const k::Shadow* sh = ShadowFor(ins.in[3], elems);
        if (sh && sh->cols == op.H * op.d && k::ShadowUsable(sh, op.out, elems)) op.shadow = *sh;
        const int keep = range_index_ < attn_keep_slot_.size() ? attn_keep_slot_[range_index_] : -1;
        if (keep >= 0) {
          op.keep = attn_keep_pool_[static_cast<size_t>(keep)];
          attn_keep_written_[static_cast<size_t>(keep)] = 0;
        }
        int n = 0;
        if (std::string e = umma::TryAttention(&umma_->ctx, ins.opcode, op, s, &n); !e.empty())
          return std::unexpected("cuda: " + e);
        if (n > 0) {
          if (keep >= 0) attn_keep_written_[static_cast<size_t>(keep)] = 1;
          shadow_written_ = op.shadow.dst != nullptr;
          ++counters_.relaxed_executions;
          launched(n);
          break;
        }
      }
      k::AttnFwd(Rd(ins.in[0]), Rd(ins.in[1]), Rd(ins.in[2]), Wr(ins.in[3]), nullptr, Wr(ins.out[0]),
                 Hi32(ins.out[1]), Lo32(ins.out[1]), Hi32(ins.out[2]), Lo32(ins.out[2]), nullptr, s);
      launched();
      break;
    case kAttnFwdTiledSeg: {
      const AttnGeom g = UnpackAttnGeom(ins.out[1]);
      k::AttnFwd(Rd(ins.in[0]), Rd(ins.in[1]), Rd(ins.in[2]), Wr(ins.in[3]), nullptr, Wr(ins.out[0]),
                 g.B, g.S, g.H, g.d, Rd<int32_t>(ins.out[2]), s);
      launched();
      break;
    }
    case kAttnDP:
      k::AttnDP(Rd(ins.in[0]), Rd(ins.in[1]), Wr(ins.in[2]), Hi32(ins.out[0]), Lo32(ins.out[0]),
                Hi32(ins.out[1]), Lo32(ins.out[1]), s);
      launched();
      break;
    case kAttnDV:
      k::AttnDV(Rd(ins.in[0]), Rd(ins.in[1]), Wr(ins.in[2]), Hi32(ins.out[0]), Lo32(ins.out[0]),
                Hi32(ins.out[1]), Lo32(ins.out[1]), s);
      launched();
      break;
    case kSoftmaxRowsBwd:
      k::SoftmaxRowsBwd(Rd(ins.in[0]), Rd(ins.in[1]), Wr(ins.in[2]), Hi32(ins.out[0]),
                        Lo32(ins.out[0]), s);
      launched();
      break;
    case kAttnDQ:
      k::AttnDQ(Rd(ins.in[0]), Rd(ins.in[1]), Wr(ins.in[2]), Hi32(ins.out[0]), Lo32(ins.out[0]),
                Hi32(ins.out[1]), Lo32(ins.out[1]), s);
      launched();
      break;
    case kAttnDK:
      k::AttnDK(Rd(ins.in[0]), Rd(ins.in[1]), Wr(ins.in[2]), Hi32(ins.out[0]), Lo32(ins.out[0]),
                Hi32(ins.out[1]), Lo32(ins.out[1]), s);
      launched();
      break;
    case kAttnDQTiled: case kAttnDKTiled: case kAttnDVTiled: {
      const AttnGeom g = UnpackAttnGeom(ins.out[2]);
      if ((ins.flags & kFlagRelaxed) && relaxed_allowed_) {
        umma::AttentionOperands op{Rd(ins.in[0]), Rd(ins.in[1]), Rd(ins.in[2]), Rd(ins.in[3]),
                                   RefOffset(ins.in[0]), RefOffset(ins.in[1]), RefOffset(ins.in[2]),
                                   RefOffset(ins.in[3]), Wr(ins.out[0]), Wr(ins.out[1]),
                                   g.B, g.S, g.H, g.d, k::Shadow{}};
        const uint64_t elems = g.B * g.S * g.H * g.d;
        if (ins.opcode == kAttnDVTiled && skip_attn_dv_at_ == static_cast<int64_t>(range_index_)) {
          skip_attn_dv_at_ = -1;   // done by the dK kernel before it
          ++counters_.relaxed_executions;
          break;
        }
        const k::Shadow* sh = ShadowFor(ins.out[1], elems);
        if (sh && sh->cols == g.H * g.d && k::ShadowUsable(sh, op.out, elems)) op.shadow = *sh;
        if (ins.opcode == kAttnDKTiled && range_index_ < attn_dv_out_.size() &&
            attn_dv_out_[range_index_] != kNullRef)
          op.out2 = Wr(attn_dv_out_[range_index_]);
        if (ins.opcode == kAttnDQTiled && range_index_ < attn_keep_slot_.size() && attn_keep_slot_[range_index_] >= 0 &&
            attn_keep_written_[static_cast<size_t>(attn_keep_slot_[range_index_])])
          op.fwd_keep = attn_keep_pool_[static_cast<size_t>(attn_keep_slot_[range_index_])];
        uint16_t* dv_copy = nullptr;
        if (op.out2 && attn_dv_shadow_[range_index_].want && attn_dv_shadow_[range_index_].scale_ref == kNullRef) {
          const ShadowPlan& sp2 = attn_dv_shadow_[range_index_];
          if (sp2.M * sp2.K == elems && sp2.K == g.H * g.d && sp2.a_off == RefOffset(attn_dv_out_[range_index_]))
            dv_copy = umma::ReserveShadow(&umma_->ctx, elems, /*keep_reserved=*/true);
          if (dv_copy) {
            op.shadow2.dst = dv_copy;
            op.shadow2.cols = sp2.K;
            if (!k::ShadowUsable(&op.shadow2, op.out2, elems)) { op.shadow2 = k::Shadow{}; dv_copy = nullptr; }
          }
        }
        int n = 0;
        bool did_second = false;
        if (std::string e = umma::TryAttention(&umma_->ctx, ins.opcode, op, s, &n, &did_second); !e.empty())
          return std::unexpected("cuda: " + e);
        if (n > 0) {
          shadow_written_ = op.shadow.dst != nullptr;
          ++counters_.relaxed_executions;
          launched(n);
          if (did_second) {
            ++counters_.fused_dispatches;
            skip_attn_dv_at_ = static_cast<int64_t>(range_index_) + 1;
            // dV's range is written now: older copies of it go, the new one is published
            // (the skipped instruction's own bookkeeping must then leave it alone).
            const ShadowPlan& sp2 = attn_dv_shadow_[range_index_];
            umma::InvalidateRange(&umma_->ctx, RefOffset(attn_dv_out_[range_index_]), elems * 4);
            if (dv_copy) umma::CommitShadow(&umma_->ctx, dv_copy, sp2.a_off, sp2.scale_off, sp2.M, sp2.K);
          } else if (dv_copy) {
            umma::ReleaseReservations(&umma_->ctx);
          }
          break;
        }
      }
      if (g.d > 256 && ins.opcode != kAttnDQTiled)
        return std::unexpected("cuda: tiled attention backward supports head widths up to 256");
      if (ins.opcode == kAttnDQTiled)
        k::AttnDQTiled(Rd(ins.in[0]), Rd(ins.in[1]), Rd(ins.in[2]), Rd(ins.in[3]), Wr(ins.out[0]),
                       Wr(ins.out[1]), g.B, g.S, g.H, g.d, s);
      else
        k::AttnDKVTiled(ins.opcode == kAttnDKTiled, Rd(ins.in[0]), Rd(ins.in[1]), Rd(ins.in[2]),
                        Rd(ins.in[3]), Rd(ins.out[0]), Wr(ins.out[1]), g.B, g.S, g.H, g.d, s);
      launched();
      break;
    }
    case kOpCount:
      return std::unexpected("cuda: unknown opcode");
  }
  return {};
}

}  // namespace see
