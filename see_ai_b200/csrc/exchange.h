// The data-parallel gradient exchange: one NCCL all-gather per optimizer step of
// the contiguous gradient block, enqueued on the engine's stream between the
// backward range and the optimizer range.  The reference has no distributed
// path (its only parallelism is threads inside one process); what shards is the
// batch, and the trainable gradients sit back to back in the arena (reference:
// compiler/backend/allocation/arena_binder.cc:56-77), so one collective per step
// is the whole data path.  The gathered copies are summed in rank order inside
// the optimizer kernel (k_optim.cu), which a ring all-reduce's order would not
// reproduce from run to run.
//
// NCCL is resolved at run time from the process (libnccl.so.2): a single-GPU
// user of the library needs no NCCL installed.
#ifndef SEE_CUDA_EXCHANGE_H_
#define SEE_CUDA_EXCHANGE_H_

#include <cuda_runtime.h>

#include <cstdint>
#include <expected>
#include <memory>
#include <string>

namespace see {

constexpr int kExchangeIdBytes = 128;   // an ncclUniqueId

// Fills `out` with a fresh communicator id (rank 0 makes it; the host hands it to
// every rank by whatever channel it has).
std::expected<void, std::string> MakeExchangeId(uint8_t out[kExchangeIdBytes]);

class GradientExchange {
 public:
  // Collective over all ranks: every rank calls it with the same id.  `bytes` is
  // the gradient block's size; the gather buffer holds world copies of it.
  static std::expected<std::unique_ptr<GradientExchange>, std::string> Join(int world, int rank,
                                                                            const uint8_t id[kExchangeIdBytes],
                                                                            uint64_t bytes);
  ~GradientExchange();
  int world() const { return world_; }
  int rank() const { return rank_; }
  void* gathered() const { return gathered_; }
  // gathered[r] = rank r's `local` block, for every r, on stream `s`.
  std::expected<void, std::string> AllGather(const void* local, cudaStream_t s);

 private:
  GradientExchange() = default;
  int world_ = 1, rank_ = 0;
  uint64_t bytes_ = 0;
  void* comm_ = nullptr;
  void* gathered_ = nullptr;
};

}  // namespace see

#endif  // SEE_CUDA_EXCHANGE_H_
