// The reference-side binding: a subclass of seeml::update_rt::ExecutorBackend
// (runtime/executor/backend.h:82-166) whose every virtual is one call into
// libsee_cuda.so's C functions (see_cuda.h). A maintainer drops this file into
// the reference tree as runtime/executor/cuda_backend.cc and adds one case to
// CreateBackend (runtime/executor/backend.cc:26-60). It is compiled here only
// by a test that has the reference's headers; the library itself never sees it.
#include "runtime/executor/backend.h"

#include <cstring>
#include <expected>
#include <memory>
#include <span>
#include <string>

#include "see_cuda.h"

namespace seeml::update_rt {
namespace {

static_assert(sizeof(seeml::update::UpdateInstruction) == 64,
              "the C functions take the plan's 64-byte instruction word as it is");

class CudaBackend final : public ExecutorBackend {
 public:
  explicit CudaBackend(see_cuda_backend* handle) : handle_(handle) {}
  ~CudaBackend() override { see_cuda_destroy(handle_); }

  const char* name() const override { return "cuda"; }
  std::string device() const override { return see_cuda_device(handle_); }

  std::expected<void, std::string> Bind(uint8_t* arena, uint64_t arena_bytes, const uint8_t* rodata,
                                        uint64_t rodata_bytes, uint64_t /*rodata_mapped_bytes*/) override {
    return Done(see_cuda_bind(handle_, arena, arena_bytes, rodata, rodata_bytes));
  }
  std::expected<void, std::string> BindSource(const uint8_t* data, uint64_t bytes) override {
    return Done(see_cuda_bind_source(handle_, data, bytes));
  }
  std::expected<void, std::string> Execute(const seeml::update::UpdateInstruction& ins,
                                           const StepParams& p) override {
    see_step_params sp;
    std::memset(&sp, 0, sizeof(sp));
    sp.lr = p.lr;
    sp.beta1 = p.beta1;
    sp.beta2 = p.beta2;
    sp.eps = p.eps;
    sp.weight_decay = p.weight_decay;
    sp.step = p.step;
    return Done(see_cuda_execute(handle_, &ins, &sp));
  }
  void BeginRange(std::span<const seeml::update::UpdateInstruction> program, size_t begin,
                  size_t end) override {
    see_cuda_begin_range(handle_, program.data(), program.size(), begin, end);
  }
  void EndRange() override { see_cuda_end_range(handle_); }
  std::expected<void, std::string> Flush() override { return Done(see_cuda_flush(handle_)); }

  uint64_t relaxed_executions() const override { return Counters().relaxed_executions; }
  uint64_t fused_dispatches() const override { return Counters().fused_dispatches; }

  /// The host's own writes into the arena (a staged batch, a restored
  /// checkpoint) must be announced before the next Execute.
  void HostWrote(uint64_t offset, uint64_t bytes) { see_cuda_host_wrote(handle_, offset, bytes); }

 private:
  see_cuda_counters Counters() const {
    see_cuda_counters c;
    std::memset(&c, 0, sizeof(c));
    see_cuda_counters_get(handle_, &c);
    return c;
  }
  std::expected<void, std::string> Done(int rc) {
    if (rc == SEE_OK) return {};
    return std::unexpected(std::string(see_cuda_last_error(handle_)));
  }
  see_cuda_backend* handle_;
};

}  // namespace

/// What the new `case BackendKind::kCuda:` of CreateBackend calls. There is no
/// CPU fallback behind it: without a usable device the error comes back as is.
std::expected<std::unique_ptr<ExecutorBackend>, std::string> CreateCudaBackend(int device_index) {
  see_cuda_backend* handle = nullptr;
  if (see_cuda_create(device_index, &handle) != SEE_OK) {
    return std::unexpected(std::string(see_cuda_create_error()));
  }
  return std::make_unique<CudaBackend>(handle);
}

}  // namespace seeml::update_rt
