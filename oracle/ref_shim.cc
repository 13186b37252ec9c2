// TEST INFRASTRUCTURE — not part of the product.
//
// A C-ABI shim around the reference's own CPU executor, so tests (and the
// bench's CPU-baseline leg) can run instruction programs through the real
// reference kernels via ctypes.  It is compiled TOGETHER WITH the reference's
// source files where they lie (see the Makefile beside this file); the result
// lives in oracle/_ref/ and is never committed.  Only this shim is ours: it
// includes the reference's backend seam (runtime/executor/backend.h) and calls
// CreateCpuBackend / Bind / BindSource / Execute / Flush, nothing else.
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <memory>
#include <string>

#include "runtime/executor/backend.h"
#include "source/parallel/parallel_for.h"
#include "source/plan/instruction.h"

namespace rt = seeml::update_rt;
namespace up = seeml::update;

struct SeeRefStepParams {
  float lr, beta1, beta2, eps, weight_decay;
  uint32_t pad;
  uint64_t step;
};

struct SeeRef {
  std::unique_ptr<rt::ExecutorBackend> backend;
  std::string error;
};

extern "C" {

void* seeref_create(void) {
  auto* h = new SeeRef;
  h->backend = rt::CreateCpuBackend();
  return h;
}

void seeref_destroy(void* handle) { delete static_cast<SeeRef*>(handle); }

const char* seeref_last_error(void* handle) {
  return static_cast<SeeRef*>(handle)->error.c_str();
}

void seeref_set_threads(uint64_t n) { up::SetParallelThreadCount(n); }
uint64_t seeref_threads(void) { return up::ParallelThreadCount(); }

int seeref_bind(void* handle, uint8_t* arena, uint64_t arena_bytes,
                const uint8_t* rodata, uint64_t rodata_bytes) {
  auto* h = static_cast<SeeRef*>(handle);
  auto r = h->backend->Bind(arena, arena_bytes, rodata, rodata_bytes, rodata_bytes);
  if (!r) { h->error = r.error(); return 1; }
  h->backend->Configure(rt::kernels::KernelPolicy{});
  return 0;
}

int seeref_bind_source(void* handle, const uint8_t* data, uint64_t bytes) {
  auto* h = static_cast<SeeRef*>(handle);
  auto r = h->backend->BindSource(data, bytes);
  if (!r) { h->error = r.error(); return 1; }
  return 0;
}

// Executes instrs[begin, end) in order, then Flush.  Returns 0, or 1 + the
// failing instruction's index with the reference's message in last_error.
int64_t seeref_run(void* handle, const void* instrs, uint64_t begin, uint64_t end,
                   const SeeRefStepParams* sp) {
  auto* h = static_cast<SeeRef*>(handle);
  static_assert(sizeof(up::UpdateInstruction) == 64);
  const auto* prog = static_cast<const up::UpdateInstruction*>(instrs);
  rt::StepParams p;
  p.lr = sp->lr; p.beta1 = sp->beta1; p.beta2 = sp->beta2; p.eps = sp->eps;
  p.weight_decay = sp->weight_decay; p.step = sp->step;
  for (uint64_t i = begin; i < end; ++i) {
    auto r = h->backend->Execute(prog[i], p);
    if (!r) { h->error = r.error(); return 1 + static_cast<int64_t>(i); }
  }
  auto r = h->backend->Flush();
  if (!r) { h->error = r.error(); return 1 + static_cast<int64_t>(end); }
  return 0;
}

}  // extern "C"
