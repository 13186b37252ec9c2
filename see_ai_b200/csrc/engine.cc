#include "engine.h"

#include <algorithm>
#include <cmath>
#include <cstddef>
#include <cstring>

#include "extents.h"

namespace see {

// ---- the seal -------------------------------------------------------------------
namespace {

constexpr uint64_t kFnvOffset = 0xcbf29ce484222325ull;
constexpr uint64_t kFnvPrime = 0x100000001b3ull;
constexpr size_t kHashChunk = size_t{1} << 20;
constexpr size_t kMaxChunks = 256;

uint64_t MixWord(uint64_t state, uint64_t word) {
  for (int b = 0; b < 8; ++b) {
    state ^= (word >> (8 * b)) & 0xff;
    state *= kFnvPrime;
  }
  return state;
}

// Eight interleaved FNV-1a lanes; byte i feeds lane i mod 8; bytes inside
// [skip_begin, skip_end) are read as zero.
uint64_t StripedFnv(const uint8_t* data, size_t size, size_t base, size_t skip_begin,
                    size_t skip_end) {
  uint64_t lane[8];
  for (size_t l = 0; l < 8; ++l) lane[l] = kFnvOffset ^ (0x9E3779B97F4A7C15ull * (l + 1));
  for (size_t i = 0; i < size; ++i) {
    const size_t at = base + i;
    const uint8_t byte = (at >= skip_begin && at < skip_end) ? 0 : data[i];
    lane[i % 8] ^= byte;
    lane[i % 8] *= kFnvPrime;
  }
  uint64_t h = kFnvOffset;
  for (size_t l = 0; l < 8; ++l) h = MixWord(h, lane[l]);
  return MixWord(h, size);
}

}  // namespace

uint64_t PlanSelfHash(const uint8_t* plan, size_t size, size_t hash_offset) {
  const size_t cap = (size + kMaxChunks - 1) / kMaxChunks;
  const size_t grain = std::max(kHashChunk, std::max<size_t>(cap, 1));
  uint64_t h = kFnvOffset;
  if (size == 0) {
    h = MixWord(h, StripedFnv(plan, 0, 0, hash_offset, hash_offset + 8));
  } else {
    for (size_t b = 0; b < size; b += grain) {
      const size_t e = std::min(b + grain, size);
      h = MixWord(h, StripedFnv(plan + b, e - b, b, hash_offset, hash_offset + 8));
    }
  }
  return MixWord(h, size);
}

PhaseBoundaries ScanPhases(const std::vector<Instruction>& train) {
  PhaseBoundaries p{train.size(), train.size()};
  for (size_t i = 0; i < train.size(); ++i) {
    const uint16_t op = train[i].opcode;
    if (op == kSoftmaxXEntFwd || op == kSoftmaxXEntMaskedFwd || op == kMseFwd || op == kKLDistillFwd)
      p.bwd_begin = i + 1;
    if ((op == kClipNorm || op == kSqNormAccum || op == kClipGlobal || op == kSgdStep ||
         op == kAdamWStep) && p.opt_begin == train.size())
      p.opt_begin = i;
  }
  if (p.opt_begin < p.bwd_begin) p.opt_begin = p.bwd_begin;
  return p;
}

// ---- lifecycle ---------------------------------------------------------------------

std::expected<std::unique_ptr<UpdateEngine>, std::string> UpdateEngine::Create(int device) {
  auto backend = CudaBackend::Create(device);
  if (!backend) return std::unexpected(backend.error());
  std::unique_ptr<UpdateEngine> e(new UpdateEngine);
  e->backend_ = std::move(*backend);
  for (auto& ev : e->ev_)
    if (cudaEventCreate(&ev) != cudaSuccess) return std::unexpected("cuda: event creation failed");
  for (auto& ev : e->staged_)
    if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess)
      return std::unexpected("cuda: event creation failed");
  void* p = nullptr;
  if (cudaMalloc(&p, 4 * sizeof(unsigned long long)) != cudaSuccess)
    return std::unexpected("cuda: tally allocation failed");
  e->d_tally_ = static_cast<unsigned long long*>(p);
  if (cudaMalloc(&p, 2 * sizeof(double)) != cudaSuccess)
    return std::unexpected("cuda: eval scratch allocation failed");
  e->d_eval_out_ = static_cast<double*>(p);
  return e;
}

void UpdateEngine::DropGraphs() {
  for (GraphSlot* g : {&g_fwdbwd_, &g_opt_, &g_eval_, &g_step_}) {
    if (g->exec) cudaGraphExecDestroy(g->exec);
    g->exec = nullptr;
    g->runs = 0;
  }
}

UpdateEngine::~UpdateEngine() {
  if (backend_) cudaStreamSynchronize(backend_->stream());
  DropGraphs();
  for (auto& ev : ev_) if (ev) cudaEventDestroy(ev);
  for (auto& ev : staged_) if (ev) cudaEventDestroy(ev);
  if (pinned_) cudaFreeHost(pinned_);
  cudaFree(d_tally_);
  cudaFree(d_eval_out_);
  cudaFree(d_eval_terms_);
  if (copy_stream_) {
    cudaStreamSynchronize(copy_stream_);
    cudaStreamDestroy(copy_stream_);
    cudaEventDestroy(snap_taken_);
    cudaEventDestroy(snap_done_);
  }
  cudaFree(d_snap_);
  if (h_snap_) cudaFreeHost(h_snap_);
}

const std::vector<Instruction>& UpdateEngine::program(int which) const {
  switch (which) {
    case 1: return eval_;
    case 2: return merge_;
    case 3: return step_prog_;
    default: return train_;
  }
}

Status UpdateEngine::LoadFromMemory(const uint8_t* plan, uint64_t size) {
  if (size < sizeof(PlanHeader)) return std::unexpected("engine: plan is truncated");
  PlanHeader h;
  std::memcpy(&h, plan, sizeof(h));
  if (h.magic != kSeeuMagic) return std::unexpected("engine: not a .seeu plan");
  if (h.version < kSeeuOldestReadable || h.version > kSeeuVersion)
    return std::unexpected("engine: unsupported plan version " + std::to_string(h.version));
  if (PlanSelfHash(plan, size, offsetof(PlanHeader, plan_hash)) != h.plan_hash)
    return std::unexpected("engine: plan integrity check failed (plan_hash)");
  auto range_ok = [&](uint64_t off, uint64_t bytes) { return off <= size && bytes <= size - off; };
  auto decode = [&](uint64_t off, uint64_t count, std::vector<Instruction>* out) -> bool {
    if (count > size / sizeof(Instruction) || !range_ok(off, count * sizeof(Instruction))) return false;
    out->resize(count);
    if (count) std::memcpy(out->data(), plan + off, count * sizeof(Instruction));
    return true;
  };
  std::vector<Instruction> train, eval, merge, step;
  if (!decode(h.train_instr_offset, h.train_instr_count, &train) ||
      !decode(h.eval_instr_offset, h.eval_instr_count, &eval) ||
      !decode(h.merge_instr_offset, h.merge_instr_count, &merge) ||
      !decode(h.step_instr_offset, h.step_instr_count, &step) ||
      !range_ok(h.rodata_offset, h.rodata_size) ||
      !range_ok(h.persist_init_offset, h.persist_init_size) ||
      h.emit_count > size / sizeof(EmitEntry) ||
      !range_ok(h.emit_table_offset, h.emit_count * sizeof(EmitEntry)))
    return std::unexpected("engine: a plan section lies outside the file");
  if (h.persist_init_size != h.persistent_size || h.persistent_size > h.arena_size)
    return std::unexpected("engine: persistent image does not match the header");
  if (h.arena_size == 0) return std::unexpected("engine: empty arena");
  auto slot_ok = [&](uint64_t ref, uint64_t bytes) {
    return ref == kNullRef || (RefSpace(ref) == kArena && ref % 4 == 0 && ref <= h.arena_size &&
                               bytes <= h.arena_size - ref);
  };
  if (!slot_ok(h.input_ref, h.input_floats * 4) || !slot_ok(h.label_ref, h.label_bytes) ||
      !slot_ok(h.loss_ref, 4))
    return std::unexpected("engine: an I/O slot lies outside the arena");
  // Every operand of every instruction is proven inside its address space once,
  // here; source refs are checked again at execution against the bound file.
  const uint64_t arena_alloc = (h.arena_size + kArenaAlignment - 1) / kArenaAlignment * kArenaAlignment;
  const std::pair<const char*, const std::vector<Instruction>*> sections[] = {
      {"train", &train}, {"eval", &eval}, {"merge", &merge}, {"step", &step}};
  for (const auto& [name, prog] : sections) {
    for (size_t i = 0; i < prog->size(); ++i) {
      Extents ext;
      const std::string e = DescribeInstruction((*prog)[i], h.arena_size, h.rodata_size,
                                                /*source_bytes=*/uint64_t{1} << 48, &ext);
      if (!e.empty())
        return std::unexpected(std::string("engine: ") + name + " instruction " + std::to_string(i) +
                               ": " + e);
    }
  }
  // The optimizer steps' gradient operands, as one block.
  uint64_t g_lo = ~0ull, g_hi = 0;
  const auto& opt_prog = step.empty() ? train : step;
  for (const Instruction& ins : opt_prog)
    if (ins.opcode == kAdamWStep || ins.opcode == kSgdStep) {
      g_lo = std::min(g_lo, RefOffset(ins.in[1]));
      g_hi = std::max(g_hi, RefOffset(ins.in[1]) + ins.out[0] * 4);
    }

  if (auto r = backend_->BindDeviceImage(arena_alloc, plan + h.persist_init_offset,
                                         h.persist_init_size, plan + h.rodata_offset, h.rodata_size);
      !r)
    return r;  // the previous plan, if any, stays bound

  DropGraphs();
  header_ = h;
  train_ = std::move(train);
  eval_ = std::move(eval);
  merge_ = std::move(merge);
  step_prog_ = std::move(step);
  emit_.resize(h.emit_count);
  if (h.emit_count) std::memcpy(emit_.data(), plan + h.emit_table_offset, h.emit_count * sizeof(EmitEntry));
  phases_ = ScanPhases(train_);
  grad_off_ = g_lo == ~0ull ? 0 : g_lo;
  grad_bytes_ = g_lo == ~0ull ? 0 : g_hi - g_lo;
  // The train program is a complete step that this engine only runs from its
  // first instruction, pass after pass; outside it only these arena ranges are
  // ever looked at (checkpoints and the merge / eval programs read the persistent
  // prefix, ReadLoss the loss slot, the data-parallel exchange and a separate
  // step program the gradient block).
  {
    std::vector<std::pair<uint64_t, uint64_t>> observed;
    if (header_.persistent_size) observed.push_back({0, header_.persistent_size});
    if (header_.loss_ref != kNullRef) observed.push_back({RefOffset(header_.loss_ref), 4});
    if (grad_bytes_) observed.push_back({grad_off_, grad_bytes_});
    backend_->DeclareStepProgram(train_.data(), std::move(observed));
  }
  step_ = 0;
  horizon_ = h.default_steps;
  eval_probs_ref_ = eval_labels_ref_ = kNullRef;
  eval_tail_ = EvalTail{};
  uint64_t terms = 0;
  for (const Instruction& ins : eval_) {
    if (ins.opcode == kSoftmaxXEntFwd || ins.opcode == kSoftmaxXEntMaskedFwd) {
      eval_probs_ref_ = ins.in[3];
      eval_labels_ref_ = ins.in[1];
      eval_rows_ = ins.out[0];
      eval_cols_ = ins.out[1];
      // Row-separable only when it is the instruction that writes the plan's loss
      // slot over exactly one batch of rows.
      if (ins.in[2] == h.loss_ref && ins.out[0] == h.batch) {
        eval_tail_ = {ins.opcode == kSoftmaxXEntFwd ? EvalTail::kXent : EvalTail::kXentMasked, ins.in[3],
                      ins.in[1], ins.out[1]};
        terms = std::max<uint64_t>(terms, h.batch);
      }
    } else if (ins.opcode == kMseFwd && ins.in[2] == h.loss_ref && h.batch > 0 && ins.out[0] % h.batch == 0) {
      eval_tail_ = {EvalTail::kMse, ins.in[0], ins.in[1], ins.out[0] / h.batch};
      terms = std::max<uint64_t>(terms, ins.out[0]);
    }
  }
  if (terms > eval_terms_capacity_) {
    cudaStreamSynchronize(backend_->stream());
    cudaFree(d_eval_terms_);
    d_eval_terms_ = nullptr;
    eval_terms_capacity_ = 0;
    void* p = nullptr;
    if (cudaMalloc(&p, terms * sizeof(double)) != cudaSuccess)
      return std::unexpected("engine: eval scratch allocation failed");
    d_eval_terms_ = static_cast<double*>(p);
    eval_terms_capacity_ = terms;
  }
  const uint64_t stage = (h.input_ref == kNullRef ? 0 : h.input_floats * 4) +
                         (h.label_ref == kNullRef ? 0 : h.label_bytes);
  if (stage > pinned_bytes_) {
    if (pinned_) cudaFreeHost(pinned_);
    pinned_ = nullptr;
    pinned_bytes_ = 0;
    void* p = nullptr;
    if (cudaMallocHost(&p, 2 * stage) != cudaSuccess)
      return std::unexpected("engine: pinned staging allocation failed");
    pinned_ = static_cast<uint8_t*>(p);
    pinned_bytes_ = stage;
  }
  // A communicator joined for the previous plan's gradient block does not fit this one.
  if (exchange_) {
    exchange_.reset();
    exchange_pending_ = false;
    backend_->SetGradientGather(1, nullptr, 0, 0);
  }
  loaded_ = true;
  return {};
}

Status UpdateEngine::BindSourceModel(const uint8_t* data, uint64_t bytes) {
  // Captured ranges hold the old source model's device addresses.
  if (backend_) cudaStreamSynchronize(backend_->stream());
  DropGraphs();
  return backend_->BindSource(data, bytes);
}

// The scheduled learning rate of the current timestep, in f32 with the host's
// cosf, operation for operation as the reference engine computes it (reference:
// runtime/dispatcher/update_engine.cc:370-391): schedule 1 is a linear ramp over
// the plan's warm-up steps, then half a cosine from the plan's rate down to
// rate * min_lr_factor over the rest of the RUN's length, and that floor beyond.
float UpdateEngine::EffectiveLr() const {
  const float peak = header_.lr;
  constexpr uint32_t kCosineWithWarmup = 1;
  if (header_.lr_schedule != kCosineWithWarmup) return peak;
  const uint64_t warm = header_.warmup_steps;
  if (warm > 0 && step_ <= warm) return peak * static_cast<float>(step_) / static_cast<float>(warm);
  const float lowest = peak * header_.min_lr_factor;
  const uint64_t decay_steps = horizon_ > warm ? horizon_ - warm : 0;
  const uint64_t into_decay = step_ - warm;
  if (decay_steps == 0 || into_decay >= decay_steps) return lowest;
  const float progress = static_cast<float>(into_decay) / static_cast<float>(decay_steps);
  const float pi = 3.14159265358979323846f;
  return lowest + (peak - lowest) * 0.5f * (1.0f + std::cos(pi * progress));
}

StepParams UpdateEngine::MakeParams() const {
  StepParams p;
  p.lr = EffectiveLr();
  p.beta1 = header_.beta1; p.beta2 = header_.beta2; p.eps = header_.eps;
  p.weight_decay = header_.weight_decay;
  p.step = step_;
  return p;
}

Status UpdateEngine::StageBatch(const void* input, uint64_t input_bytes, const void* labels,
                                uint64_t label_bytes) {
  if (!loaded_) return std::unexpected("engine: no plan is loaded");
  const uint64_t want_in = header_.input_ref == kNullRef ? 0 : header_.input_floats * 4;
  const uint64_t want_lab = header_.label_ref == kNullRef ? 0 : header_.label_bytes;
  if (input_bytes != want_in || label_bytes != want_lab)
    return std::unexpected("engine: batch size does not match the plan's I/O slots");
  // Double-buffered pinned staging: wait until the copy that last used this
  // half has been consumed, fill it, enqueue the async upload.
  uint8_t* buf = pinned_ + static_cast<uint64_t>(pinned_slot_) * pinned_bytes_;
  cudaEventSynchronize(staged_[pinned_slot_]);
  if (want_in) std::memcpy(buf, input, want_in);
  if (want_lab) std::memcpy(buf + want_in, labels, want_lab);
  if (want_in)
    if (auto r = backend_->WriteArena(RefOffset(header_.input_ref), want_in, buf); !r) return r;
  if (want_lab)
    if (auto r = backend_->WriteArena(RefOffset(header_.label_ref), want_lab, buf + want_in); !r)
      return r;
  cudaEventRecord(staged_[pinned_slot_], backend_->stream());
  pinned_slot_ ^= 1;
  return {};
}

Status UpdateEngine::RunRange(const std::vector<Instruction>& prog, size_t begin, size_t end,
                              GraphSlot* slot, float* phase_ms) {
  if (!loaded_) return std::unexpected("engine: no plan is loaded");
  if (begin >= end) return {};
  const StepParams params = MakeParams();
  cudaStream_t s = backend_->stream();
  if (phase_ms) cudaEventRecord(ev_[0], s);
  const std::span<const Instruction> span(prog.data(), prog.size());
  Status result{};
  bool has_opt = false;
  for (size_t i = begin; i < end; ++i) has_opt = has_opt || prog[i].opcode == kAdamWStep || prog[i].opcode == kSgdStep;
  if (use_graphs_ && slot && slot->exec) {
    if (has_opt)
      if (auto r = backend_->UploadStepScalars(params); !r) return r;
    if (auto e = cudaGraphLaunch(slot->exec, s); e != cudaSuccess)
      return std::unexpected(std::string("engine: graph launch: ") + cudaGetErrorString(e));
  } else {
    backend_->BeginRange(span, begin, end);
    const bool capture = use_graphs_ && slot && slot->runs >= 1;
    cudaGraph_t graph = nullptr;
    if (capture) {
      if (has_opt)
        if (auto r = backend_->UploadStepScalars(params); !r) { backend_->EndRange(); return r; }
      backend_->SetCapturing(true);
      if (auto e = cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal); e != cudaSuccess) {
        backend_->SetCapturing(false);
        return std::unexpected(std::string("engine: begin capture: ") + cudaGetErrorString(e));
      }
    }
    for (size_t i = begin; i < end; ++i) {
      if (auto r = backend_->Execute(prog[i], params); !r) {
        result = std::unexpected("instruction " + std::to_string(i) + ": " + r.error());
        break;
      }
    }
    if (capture) {
      const cudaError_t e = cudaStreamEndCapture(s, &graph);
      backend_->SetCapturing(false);
      if (e != cudaSuccess || !graph) {
        if (result) result = std::unexpected(std::string("engine: end capture: ") + cudaGetErrorString(e));
      } else if (result) {
        cudaGraphExec_t exec = nullptr;
        if (auto ie = cudaGraphInstantiate(&exec, graph, 0); ie != cudaSuccess) {
          result = std::unexpected(std::string("engine: graph instantiate: ") + cudaGetErrorString(ie));
        } else {
          slot->exec = exec;
          if (auto le = cudaGraphLaunch(exec, s); le != cudaSuccess)
            result = std::unexpected(std::string("engine: graph launch: ") + cudaGetErrorString(le));
        }
      }
      if (graph) cudaGraphDestroy(graph);
    }
    if (slot) ++slot->runs;
    backend_->EndRange();
  }
  if (phase_ms) {
    cudaEventRecord(ev_[1], s);
    cudaEventSynchronize(ev_[1]);
    cudaEventElapsedTime(phase_ms, ev_[0], ev_[1]);
  }
  return result;
}

bool UpdateEngine::has_masked_loss() const {
  for (const Instruction& ins : train_)
    if (ins.opcode == kSoftmaxXEntMaskedFwd || ins.opcode == kSoftmaxXEntMaskedBwd) return true;
  return false;
}

Status UpdateEngine::AttachExchange(int world, int rank, const uint8_t* id) {
  if (!loaded_) return std::unexpected("engine: no plan is loaded");
  if (world <= 1) {
    DetachExchange();
    return {};
  }
  // The masked loss divides each shard's gradient by that shard's own target
  // count, so the plain 1/N mean of shard gradients is the global masked mean
  // only when every shard holds the same number of targets: not promised here.
  if (has_masked_loss())
    return std::unexpected("engine: data parallel: plans with a masked cross-entropy are not supported "
                           "(shards would need a target-count-weighted mean)");
  if (!id) return std::unexpected("engine: data parallel: no communicator id");
  auto x = GradientExchange::Join(world, rank, id, grad_bytes_);
  if (!x) return std::unexpected(x.error());
  DropGraphs();   // the optimizer kernels now read the gathered copies
  exchange_ = std::move(*x);
  backend_->SetGradientGather(world, exchange_->gathered(), grad_off_, grad_bytes_);
  exchange_pending_ = false;
  return {};
}

void UpdateEngine::DetachExchange() {
  if (!exchange_) return;
  cudaStreamSynchronize(backend_->stream());
  DropGraphs();
  backend_->SetGradientGather(1, nullptr, 0, 0);
  exchange_.reset();
  exchange_pending_ = false;
}

Status UpdateEngine::Exchange() {
  if (!exchange_ || !exchange_pending_) return {};
  exchange_pending_ = false;
  const uint8_t* local = static_cast<const uint8_t*>(backend_->device_arena()) + grad_off_;
  return exchange_->AllGather(local, backend_->stream());
}

Status UpdateEngine::TrainForwardBackward(bool advance) {
  if (advance) ++step_;
  if (step_ == 0) step_ = 1;  // AdamW's timestep is 1-indexed
  exchange_pending_ = exchange_ != nullptr;
  if (!phase_timing_) return RunRange(train_, 0, phases_.opt_begin, &g_fwdbwd_, nullptr);
  // Phase timing splits forward from backward at the loss (two ranges, no graph).
  float f = 0, b = 0;
  if (auto r = RunRange(train_, 0, phases_.bwd_begin, nullptr, &f); !r) return r;
  if (auto r = RunRange(train_, phases_.bwd_begin, phases_.opt_begin, nullptr, &b); !r) return r;
  timings_.forward += f;
  timings_.backward += b;
  return {};
}

Status UpdateEngine::TrainOptimizer() {
  if (auto x = Exchange(); !x) return x;
  float o = 0;
  auto r = RunRange(train_, phases_.opt_begin, train_.size(), phase_timing_ ? nullptr : &g_opt_,
                    phase_timing_ ? &o : nullptr);
  if (phase_timing_) {
    timings_.optimizer += o;
    if (step_prog_.empty()) ++timings_.steps;
  }
  return r;
}

Status UpdateEngine::StepProgram() {
  if (auto x = Exchange(); !x) return x;
  float o = 0;
  auto r = RunRange(step_prog_, 0, step_prog_.size(), phase_timing_ ? nullptr : &g_step_,
                    phase_timing_ ? &o : nullptr);
  if (phase_timing_) {
    timings_.optimizer += o;
    ++timings_.steps;
  }
  return r;
}

StepTimings UpdateEngine::TakeTimings() {
  StepTimings t = timings_;
  timings_ = StepTimings{};
  return t;
}

Status UpdateEngine::ReadLoss(float* loss) {
  if (header_.loss_ref == kNullRef) return std::unexpected("engine: the plan has no loss slot");
  if (auto r = backend_->ReadArena(RefOffset(header_.loss_ref), 4, loss); !r) return r;
  return backend_->Flush();  // surfaces a refusal raised on the device
}

Status UpdateEngine::Evaluate(EvalResult* out, uint64_t real_rows) {
  if (!loaded_) return std::unexpected("engine: no plan is loaded");
  if (eval_.empty()) return std::unexpected("engine: the plan carries no eval program");
  if (auto r = RunRange(eval_, 0, eval_.size(), &g_eval_, nullptr); !r) return r;
  const uint64_t real = std::min<uint64_t>(real_rows, header_.batch);
  cudaStream_t s = backend_->stream();
  cudaMemsetAsync(d_tally_, 0, 4 * sizeof(unsigned long long), s);
  cudaMemsetAsync(d_eval_out_, 0, 2 * sizeof(double), s);
  auto at = [&](uint64_t ref) { return backend_->device_arena() + RefOffset(ref); };
  // Accuracy needs class labels in the label slot and a softmax whose rows cover
  // the batch (reference: update_engine.cc:458-466); real rows only, each once.
  const bool track_accuracy = header_.label_kind == 1 && header_.label_ref != kNullRef &&
                              eval_probs_ref_ != kNullRef && eval_cols_ > 0 && eval_rows_ >= header_.batch;
  const int32_t* label_slot = header_.label_ref == kNullRef
                                  ? nullptr : reinterpret_cast<const int32_t*>(at(header_.label_ref));
  if (track_accuracy)
    k::ArgmaxTally(reinterpret_cast<const float*>(at(eval_probs_ref_)), label_slot, real, eval_cols_, d_tally_, s);
  bool row_loss = true;
  switch (eval_tail_.kind) {
    case EvalTail::kXent: case EvalTail::kXentMasked:
      if (!label_slot) return std::unexpected("engine: a cross-entropy eval tail needs the label slot");
      k::XentRealRowLoss(reinterpret_cast<const float*>(at(eval_tail_.a)), label_slot, real, eval_tail_.width,
                         d_eval_terms_, d_eval_out_, d_tally_, s);
      break;
    case EvalTail::kMse:
      k::MseRealRowLoss(reinterpret_cast<const float*>(at(eval_tail_.a)),
                        reinterpret_cast<const float*>(at(eval_tail_.b)), real, eval_tail_.width, d_eval_terms_,
                        d_eval_out_, d_tally_, s);
      break;
    case EvalTail::kWeighted: row_loss = false; break;
  }
  unsigned long long tally[4] = {0, 0, 0, 0};
  double sums[2] = {0, 0};
  if (auto e = cudaMemcpyAsync(tally, d_tally_, sizeof(tally), cudaMemcpyDeviceToHost, s); e != cudaSuccess)
    return std::unexpected(std::string("engine: tally read: ") + cudaGetErrorString(e));
  if (auto e = cudaMemcpyAsync(sums, d_eval_out_, sizeof(sums), cudaMemcpyDeviceToHost, s); e != cudaSuccess)
    return std::unexpected(std::string("engine: row-loss read: ") + cudaGetErrorString(e));
  if (auto r = ReadLoss(&out->loss); !r) return r;   // synchronises the stream
  out->rows = tally[0];
  out->correct = tally[1];
  out->has_accuracy = track_accuracy;
  if (row_loss) {
    out->real_row_loss = sums[0];
    out->loss_rows = eval_tail_.kind == EvalTail::kMse ? real : tally[3];
  } else {
    // A composite loss keeps no per-row values: the batch mean stands for each real row.
    out->real_row_loss = static_cast<double>(out->loss) * static_cast<double>(real);
    out->loss_rows = real;
  }
  return {};
}

Status UpdateEngine::RunMerge(bool* all_finite) {
  if (auto r = RunRange(merge_, 0, merge_.size(), nullptr, nullptr); !r) return r;
  cudaStream_t s = backend_->stream();
  cudaMemsetAsync(d_tally_, 0, 4 * sizeof(unsigned long long), s);
  for (const EmitEntry& e : emit_) {
    if (e.arena_offset > header_.arena_size || e.byte_size > header_.arena_size - e.arena_offset)
      return std::unexpected("engine: an emit entry lies outside the arena");
    k::CountNonFinite(reinterpret_cast<const float*>(backend_->device_arena() + e.arena_offset),
                      e.byte_size / 4, d_tally_, s);
  }
  unsigned long long tally[4] = {0, 0, 0, 0};
  if (auto e = cudaMemcpyAsync(tally, d_tally_, sizeof(tally), cudaMemcpyDeviceToHost, s); e != cudaSuccess)
    return std::unexpected(std::string("engine: tally read: ") + cudaGetErrorString(e));
  if (auto r = backend_->Flush(); !r) return r;
  if (all_finite) *all_finite = tally[2] == 0;
  return {};
}

Status UpdateEngine::WriteArena(uint64_t off, uint64_t bytes, const void* src) {
  if (auto r = backend_->WriteArena(off, bytes, src); !r) return r;
  // The source is the caller's (pageable) memory: finish the copy before returning.
  if (auto e = cudaStreamSynchronize(backend_->stream()); e != cudaSuccess)
    return std::unexpected(std::string("engine: write: ") + cudaGetErrorString(e));
  return {};
}

Status UpdateEngine::WritePersistent(const void* src) {
  return WriteArena(0, header_.persistent_size, src);
}

Status UpdateEngine::SnapshotBegin() {
  if (!loaded_) return std::unexpected("engine: no plan is loaded");
  const uint64_t bytes = header_.persistent_size;
  if (bytes == 0) return std::unexpected("engine: the plan has no persistent state");
  auto fail = [](const char* what, cudaError_t e) -> Status {
    return std::unexpected(std::string("engine: snapshot: ") + what + ": " + cudaGetErrorString(e));
  };
  if (snap_pending_) cudaEventSynchronize(snap_done_);   // the buffers are reused
  if (bytes > snap_bytes_) {
    cudaFree(d_snap_);
    if (h_snap_) cudaFreeHost(h_snap_);
    d_snap_ = nullptr; h_snap_ = nullptr; snap_bytes_ = 0;
    void* p = nullptr;
    if (auto e = cudaMalloc(&p, bytes); e != cudaSuccess) return fail("device buffer", e);
    d_snap_ = static_cast<uint8_t*>(p);
    if (auto e = cudaMallocHost(&p, bytes); e != cudaSuccess) return fail("pinned buffer", e);
    h_snap_ = static_cast<uint8_t*>(p);
    snap_bytes_ = bytes;
  }
  if (!copy_stream_) {
    if (auto e = cudaStreamCreateWithFlags(&copy_stream_, cudaStreamNonBlocking); e != cudaSuccess)
      return fail("copy stream", e);
    if (auto e = cudaEventCreateWithFlags(&snap_taken_, cudaEventDisableTiming); e != cudaSuccess)
      return fail("event", e);
    if (auto e = cudaEventCreateWithFlags(&snap_done_, cudaEventDisableTiming); e != cudaSuccess)
      return fail("event", e);
  }
  cudaStream_t s = backend_->stream();
  if (auto e = cudaMemcpyAsync(d_snap_, backend_->device_arena(), bytes, cudaMemcpyDeviceToDevice, s);
      e != cudaSuccess)
    return fail("copy aside", e);
  cudaEventRecord(snap_taken_, s);
  cudaStreamWaitEvent(copy_stream_, snap_taken_, 0);
  if (auto e = cudaMemcpyAsync(h_snap_, d_snap_, bytes, cudaMemcpyDeviceToHost, copy_stream_);
      e != cudaSuccess)
    return fail("download", e);
  cudaEventRecord(snap_done_, copy_stream_);
  snap_pending_ = true;
  return {};
}

Status UpdateEngine::SnapshotWait(void* dst, uint64_t bytes) {
  if (!snap_pending_) return std::unexpected("engine: no snapshot was begun");
  if (bytes != header_.persistent_size)
    return std::unexpected("engine: a snapshot is persistent_size bytes");
  if (auto e = cudaEventSynchronize(snap_done_); e != cudaSuccess)
    return std::unexpected(std::string("engine: snapshot: ") + cudaGetErrorString(e));
  std::memcpy(dst, h_snap_, bytes);
  snap_pending_ = false;
  return {};
}

Status UpdateEngine::Restore(const void* src, uint64_t bytes, uint64_t step) {
  if (!loaded_) return std::unexpected("engine: no plan is loaded");
  if (bytes != header_.persistent_size)
    return std::unexpected("engine: a restore is persistent_size bytes");
  if (auto r = WritePersistent(src); !r) return r;
  step_ = step;
  return {};
}

}  // namespace see
