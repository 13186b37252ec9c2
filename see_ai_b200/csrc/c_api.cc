// extern "C" face of CudaBackend: one forwarding function per seam member.
#include "../../include/see_cuda.h"

#include <cstring>
#include <memory>
#include <span>
#include <string>

#include "cuda_backend.h"

struct see_cuda_backend {
  std::unique_ptr<see::CudaBackend> backend;
  std::string error;
  std::string device;
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

int Fail(see_cuda_backend* h, const std::string& msg) {
  h->error = msg;
  // A refusal may arrive prefixed with the failing instruction's index.
  const bool refused = msg.find(see::kNonFiniteNormRefusal) != std::string::npos ||
                       msg.find(see::kClipThresholdRefusal) != std::string::npos;
  return refused ? SEE_REFUSED : SEE_ERROR;
}

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
  h->backend = std::move(*b);
  h->device = h->backend->device();
  *out = h;
  return SEE_OK;
}

const char* see_cuda_create_error(void) { return g_create_error.c_str(); }

void see_cuda_destroy(see_cuda_backend* h) { delete h; }

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
    out[n] = see_profile_record{r.opcode, 0, r.index, r.ms, 0, r.m, r.n, r.k};
    ++n;
  }
  return static_cast<int64_t>(n);
}

}  // extern "C"
