// extern "C" face of CudaBackend and UpdateEngine: one forwarding function per
// member of the seam it mirrors.
#include "../../include/see_cuda.h"

#include <cstring>
#include <memory>
#include <span>
#include <string>

#include "cuda_backend.h"
#include "engine.h"
#include "lora_umma.h"
#include "umma_kernel.h"

struct see_cuda_backend {
  see::CudaBackend* backend = nullptr;          // borrowed when owned is empty
  std::unique_ptr<see::CudaBackend> owned;
  std::string error;
  std::string device;
};

struct see_engine {
  std::unique_ptr<see::UpdateEngine> engine;
  see_cuda_backend backend_view;                // a borrowed view of the engine's backend
  std::string error;
};

namespace {

thread_local std::string g_create_error;

static_assert(sizeof(see_step_params) == sizeof(see::StepParams));
static_assert(sizeof(see_cuda_counters) == sizeof(see::Counters));

see::StepParams ToParams(const see_step_params* p) {
  see::StepParams s;
  if (p) std::memcpy(&s, p, sizeof(s));
  return s;
}

int CodeOf(const std::string& msg) {
  // A refusal may arrive prefixed with the failing instruction's index.
  const bool refused = msg.find(see::kNonFiniteNormRefusal) != std::string::npos ||
                       msg.find(see::kClipThresholdRefusal) != std::string::npos;
  return refused ? SEE_REFUSED : SEE_ERROR;
}
int Fail(see_cuda_backend* h, const std::string& msg) {
  h->error = msg;
  return CodeOf(msg);
}
int Fail(see_engine* h, const std::string& msg) {
  h->error = msg;
  return CodeOf(msg);
}
int Done(see_engine* h, const see::Status& r) { return r ? SEE_OK : Fail(h, r.error()); }

}  // namespace

extern "C" {

int see_cuda_create(int device_ordinal, see_cuda_backend** out) {
  if (!out) return SEE_ERROR;
  *out = nullptr;
  auto b = see::CudaBackend::Create(device_ordinal);
  if (!b) {
    g_create_error = b.error();
    return SEE_ERROR;
  }
  auto* h = new see_cuda_backend;
  h->owned = std::move(*b);
  h->backend = h->owned.get();
  h->device = h->backend->device();
  *out = h;
  return SEE_OK;
}

const char* see_cuda_create_error(void) { return g_create_error.c_str(); }

void see_cuda_destroy(see_cuda_backend* h) {
  if (h && h->owned) delete h;  // a borrowed view belongs to its engine
}

const char* see_cuda_name(see_cuda_backend* h) { return h->backend->name(); }
const char* see_cuda_device(see_cuda_backend* h) { return h->device.c_str(); }
const char* see_cuda_last_error(see_cuda_backend* h) { return h->error.c_str(); }

int see_cuda_bind(see_cuda_backend* h, uint8_t* arena, uint64_t arena_bytes,
                  const uint8_t* rodata, uint64_t rodata_bytes) {
  auto r = h->backend->Bind(arena, arena_bytes, rodata, rodata_bytes, rodata_bytes);
  return r ? SEE_OK : Fail(h, r.error());
}

int see_cuda_bind_source(see_cuda_backend* h, const uint8_t* data, uint64_t bytes) {
  auto r = h->backend->BindSource(data, bytes);
  return r ? SEE_OK : Fail(h, r.error());
}

int see_cuda_begin_range(see_cuda_backend* h, const void* instructions, uint64_t count,
                         uint64_t begin, uint64_t end) {
  if (begin > end || end > count) return Fail(h, "cuda: begin_range: bad range");
  h->backend->BeginRange(
      std::span<const see::Instruction>(static_cast<const see::Instruction*>(instructions), count),
      begin, end);
  return SEE_OK;
}

int see_cuda_execute(see_cuda_backend* h, const void* instruction, const see_step_params* params) {
  see::Instruction ins;
  std::memcpy(&ins, instruction, sizeof(ins));
  auto r = h->backend->Execute(ins, ToParams(params));
  return r ? SEE_OK : Fail(h, r.error());
}

int see_cuda_end_range(see_cuda_backend* h) {
  h->backend->EndRange();
  return SEE_OK;
}

int see_cuda_set_lora_fold(see_cuda_backend* h, int enabled) {
  h->backend->SetLoraFold(enabled != 0);
  return SEE_OK;
}

int see_cuda_set_attention_one_walk(see_cuda_backend* h, int enabled) {
  h->backend->SetAttentionOneWalk(enabled != 0);
  return SEE_OK;
}

int see_cuda_set_adapter_fma(see_cuda_backend* h, int enabled) {
  h->backend->SetAdapterFma(enabled != 0);
  return SEE_OK;
}

int see_cuda_set_split_gemm(see_cuda_backend* h, int mode) {
  h->backend->SetSplitGemm(mode);
  return SEE_OK;
}

int see_cuda_set_cta_pairs(int enabled) {
  see::k::UmmaSetCtaPairs(enabled != 0);
  return SEE_OK;
}

int see_cuda_set_adapter_tensor_backward(int enabled) {
  see::k::LoraBackwardUmmaSet(enabled != 0);
  return SEE_OK;
}

int see_cuda_quantize_columns(see_cuda_backend* h, const float* w, uint64_t K, uint64_t N,
                              int8_t* levels, float* scales) {
  auto r = h->backend->QuantizeColumns(w, K, N, levels, scales);
  return r ? SEE_OK : Fail(h, r.error());
}

int see_cuda_flush(see_cuda_backend* h) {
  auto r = h->backend->Flush();
  return r ? SEE_OK : Fail(h, r.error());
}

int see_cuda_run_range(see_cuda_backend* h, const void* instructions, uint64_t count,
                       uint64_t begin, uint64_t end, const see_step_params* params,
                       uint64_t* failed_index) {
  if (begin > end || end > count) return Fail(h, "cuda: run_range: bad range");
  const auto* prog = static_cast<const see::Instruction*>(instructions);
  const see::StepParams sp = ToParams(params);
  h->backend->BeginRange(std::span<const see::Instruction>(prog, count), begin, end);
  for (uint64_t i = begin; i < end; ++i) {
    see::Instruction ins;
    std::memcpy(&ins, prog + i, sizeof(ins));
    if (auto r = h->backend->Execute(ins, sp); !r) {
      if (failed_index) *failed_index = i;
      (void)h->backend->Flush();
      h->backend->EndRange();
      return Fail(h, "instruction " + std::to_string(i) + ": " + r.error());
    }
  }
  auto r = h->backend->Flush();
  h->backend->EndRange();
  if (!r) {
    if (failed_index) *failed_index = end;
    return Fail(h, r.error());
  }
  return SEE_OK;
}

int see_cuda_set_coherence(see_cuda_backend* h, int mode) {
  h->backend->SetCoherence(mode == SEE_COHERENCE_LAZY ? see::Coherence::kLazy
                                                      : see::Coherence::kStrict);
  return SEE_OK;
}

int see_cuda_host_wrote(see_cuda_backend* h, uint64_t offset, uint64_t bytes) {
  h->backend->HostWrote(offset, bytes);
  return SEE_OK;
}

int see_cuda_host_needs(see_cuda_backend* h, uint64_t offset, uint64_t bytes) {
  auto r = h->backend->HostNeeds(offset, bytes);
  return r ? SEE_OK : Fail(h, r.error());
}

int see_cuda_counters_get(see_cuda_backend* h, see_cuda_counters* out) {
  std::memcpy(out, &h->backend->counters(), sizeof(*out));
  return SEE_OK;
}

int see_cuda_set_stream(see_cuda_backend* h, void* cuda_stream) {
  h->backend->SetStream(static_cast<cudaStream_t>(cuda_stream));
  return SEE_OK;
}

void* see_cuda_device_arena(see_cuda_backend* h) { return h->backend->device_arena(); }

int see_cuda_set_relaxed_allowed(see_cuda_backend* h, int allowed) {
  h->backend->SetRelaxedAllowed(allowed != 0);
  return SEE_OK;
}

int see_cuda_set_epilogue_fusion(see_cuda_backend* h, int enabled) {
  h->backend->SetEpilogueFusion(enabled != 0);
  return SEE_OK;
}

int see_cuda_set_gradient_gather(see_cuda_backend* h, int ranks, const void* gathered_device,
                                 uint64_t block_offset, uint64_t block_bytes) {
  h->backend->SetGradientGather(ranks, gathered_device, block_offset, block_bytes);
  return SEE_OK;
}

int see_cuda_set_profiling(see_cuda_backend* h, int on) {
  h->backend->SetProfiling(on != 0);
  return SEE_OK;
}

int64_t see_cuda_take_profile(see_cuda_backend* h, see_profile_record* out, uint64_t capacity) {
  const auto recs = h->backend->TakeProfile();
  uint64_t n = 0;
  for (const auto& r : recs) {
    if (n >= capacity) break;
    out[n] = see_profile_record{r.opcode, r.absorbed, r.index, r.ms, r.kernel_ms, r.m, r.n, r.k};
    ++n;
  }
  return static_cast<int64_t>(n);
}

// ---- the engine ---------------------------------------------------------------------

int see_engine_create(int device_ordinal, see_engine** out) {
  if (!out) return SEE_ERROR;
  *out = nullptr;
  auto e = see::UpdateEngine::Create(device_ordinal);
  if (!e) {
    g_create_error = e.error();
    return SEE_ERROR;
  }
  auto* h = new see_engine;
  h->engine = std::move(*e);
  h->backend_view.backend = &h->engine->backend();
  h->backend_view.device = h->engine->backend().device();
  *out = h;
  return SEE_OK;
}

void see_engine_destroy(see_engine* h) { delete h; }
const char* see_engine_last_error(see_engine* h) { return h->error.c_str(); }
see_cuda_backend* see_engine_backend(see_engine* h) { return &h->backend_view; }

int see_engine_load(see_engine* h, const uint8_t* plan, uint64_t bytes) {
  return Done(h, h->engine->LoadFromMemory(plan, bytes));
}
int see_engine_bind_source(see_engine* h, const uint8_t* data, uint64_t bytes) {
  return Done(h, h->engine->BindSourceModel(data, bytes));
}
int see_engine_header(see_engine* h, void* out_320_bytes) {
  std::memcpy(out_320_bytes, &h->engine->header(), sizeof(see::PlanHeader));
  return SEE_OK;
}
int see_engine_stage_batch(see_engine* h, const void* input, uint64_t input_bytes,
                           const void* labels, uint64_t label_bytes) {
  return Done(h, h->engine->StageBatch(input, input_bytes, labels, label_bytes));
}
int see_engine_train_forward_backward(see_engine* h, int advance_step) {
  return Done(h, h->engine->TrainForwardBackward(advance_step != 0));
}
int see_engine_train_optimizer(see_engine* h) { return Done(h, h->engine->TrainOptimizer()); }
int see_engine_step_program(see_engine* h) { return Done(h, h->engine->StepProgram()); }
int see_engine_read_loss(see_engine* h, float* loss) { return Done(h, h->engine->ReadLoss(loss)); }
int see_engine_evaluate(see_engine* h, float* loss, uint64_t* rows, uint64_t* correct) {
  see::EvalResult r;
  if (auto s = h->engine->Evaluate(&r); !s) return Fail(h, s.error());
  if (loss) *loss = r.loss;
  if (rows) *rows = r.rows;
  if (correct) *correct = r.correct;
  return SEE_OK;
}
int see_engine_evaluate_rows(see_engine* h, uint64_t real_rows, see_eval_result* out) {
  see::EvalResult r;
  if (auto s = h->engine->Evaluate(&r, real_rows); !s) return Fail(h, s.error());
  if (out) {
    out->loss = r.loss;
    out->has_accuracy = r.has_accuracy ? 1u : 0u;
    out->rows = r.rows;
    out->correct = r.correct;
    out->real_row_loss = r.real_row_loss;
    out->loss_rows = r.loss_rows;
  }
  return SEE_OK;
}
int see_engine_run_merge(see_engine* h, int* all_finite) {
  bool finite = false;
  if (auto s = h->engine->RunMerge(&finite); !s) return Fail(h, s.error());
  if (all_finite) *all_finite = finite ? 1 : 0;
  return SEE_OK;
}
int see_engine_read_arena(see_engine* h, uint64_t offset, uint64_t bytes, void* dst) {
  return Done(h, h->engine->ReadArena(offset, bytes, dst));
}
int see_engine_write_arena(see_engine* h, uint64_t offset, uint64_t bytes, const void* src) {
  return Done(h, h->engine->WriteArena(offset, bytes, src));
}
uint64_t see_engine_step(see_engine* h) { return h->engine->step(); }
int see_engine_set_step(see_engine* h, uint64_t step) { h->engine->SetStep(step); return SEE_OK; }
int see_engine_set_horizon(see_engine* h, uint64_t steps) { h->engine->SetHorizon(steps); return SEE_OK; }
float see_engine_effective_lr(see_engine* h) { return h->engine->EffectiveLr(); }
int see_engine_set_use_graphs(see_engine* h, int on) { h->engine->SetUseGraphs(on != 0); return SEE_OK; }
int see_engine_set_phase_timing(see_engine* h, int on) { h->engine->SetPhaseTiming(on != 0); return SEE_OK; }
int see_engine_take_timings(see_engine* h, float* forward_ms, float* backward_ms,
                            float* optimizer_ms, uint64_t* steps) {
  const see::StepTimings t = h->engine->TakeTimings();
  if (forward_ms) *forward_ms = t.forward;
  if (backward_ms) *backward_ms = t.backward;
  if (optimizer_ms) *optimizer_ms = t.optimizer;
  if (steps) *steps = t.steps;
  return SEE_OK;
}
int see_engine_gradient_block(see_engine* h, uint64_t* offset, uint64_t* bytes) {
  h->engine->GradientBlock(offset, bytes);
  return SEE_OK;
}
int see_cuda_exchange_id(uint8_t* out128) {
  if (!out128) return SEE_ERROR;
  if (auto r = see::MakeExchangeId(out128); !r) {
    g_create_error = r.error();
    return SEE_ERROR;
  }
  return SEE_OK;
}
int see_engine_attach_exchange(see_engine* h, int world, int rank, const uint8_t* id128) {
  return Done(h, h->engine->AttachExchange(world, rank, id128));
}
int see_engine_detach_exchange(see_engine* h) {
  h->engine->DetachExchange();
  return SEE_OK;
}
int see_engine_exchange(see_engine* h) { return Done(h, h->engine->Exchange()); }
int see_engine_snapshot_begin(see_engine* h) { return Done(h, h->engine->SnapshotBegin()); }
int see_engine_snapshot_wait(see_engine* h, void* dst, uint64_t bytes) {
  return Done(h, h->engine->SnapshotWait(dst, bytes));
}
int see_engine_restore(see_engine* h, const void* src, uint64_t bytes, uint64_t step) {
  return Done(h, h->engine->Restore(src, bytes, step));
}

}  // extern "C"
