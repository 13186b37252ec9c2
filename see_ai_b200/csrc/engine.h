// UpdateEngine — the dispatcher over the CUDA executor: loads a sealed plan,
// owns the device slab, runs the plan's programs as ranges through
// CudaBackend exactly as the reference engine runs them through its backend,
// and keeps the host-side scalars (timestep, scheduled learning rate) the
// way the reference does.  Mirrors the hot-path surface of
// seeml::update_rt::UpdateEngine (reference: runtime/dispatcher/update_engine.h:211-367;
// ExecuteRange update_engine.cc:325-364; EffectiveLr :370-391; the train loop
// :817-924; Evaluate :432-580; RunMerge :1028-1063).  What the reference does
// on the host over unified memory — the accuracy argmax over the probabilities,
// the finiteness scan of the merged deltas — runs here on the device, so only
// scalars cross the bus.
#ifndef SEE_CUDA_ENGINE_H_
#define SEE_CUDA_ENGINE_H_

#include <cuda_runtime.h>

#include <cstdint>
#include <expected>
#include <memory>
#include <string>
#include <vector>

#include "cuda_backend.h"
#include "exchange.h"
#include "plan_abi.h"

namespace see {

// Chunked, striped FNV-1a over a plan blob with its own hash field read as
// zero (reference: source/identity/hash.h:80-161).
uint64_t PlanSelfHash(const uint8_t* plan, size_t size, size_t hash_offset);

struct PhaseBoundaries { size_t bwd_begin = 0, opt_begin = 0; };
// reference: runtime/profiler/step_timings.h:37-59
PhaseBoundaries ScanPhases(const std::vector<Instruction>& train);

struct StepTimings {   // milliseconds on the device, by CUDA events
  float forward = 0, backward = 0, optimizer = 0;
  uint64_t steps = 0;
};

struct EvalResult {
  float loss = 0;         // the eval program's own loss: the mean over the whole fixed-shape batch
  uint64_t rows = 0;      // rows judged for accuracy: real rows whose label is >= 0
  uint64_t correct = 0;   // argmax == label among them (first maximum wins)
  // The batch's loss over its real rows alone (a validation set's last batch
  // wraps; a masked plan is always scored over its target rows): the row-order
  // double sum of the per-row losses and the number of rows it is over
  // (reference: runtime/dispatcher/update_engine.cc:977-1026).
  double real_row_loss = 0;
  uint64_t loss_rows = 0;
  bool has_accuracy = false;
};

// What the eval program's loss instruction lets the engine recompute per row
// (reference: runtime/loader/plan_loader.cc:165-181).
struct EvalTail {
  enum Kind { kWeighted = 0, kXent = 1, kXentMasked = 2, kMse = 3 } kind = kWeighted;
  uint64_t a = kNullRef, b = kNullRef, width = 0;
};

class UpdateEngine {
 public:
  static std::expected<std::unique_ptr<UpdateEngine>, std::string> Create(int device);
  ~UpdateEngine();

  // Decodes and verifies the plan (seal, version window, section bounds, every
  // instruction's operands), creates the slab — zeroed, persistent image at
  // offset 0 — and uploads the frozen weights.  A refused load keeps the
  // previously loaded plan bound and usable.
  Status LoadFromMemory(const uint8_t* plan, uint64_t size);
  Status BindSourceModel(const uint8_t* data, uint64_t bytes);

  const PlanHeader& header() const { return header_; }
  CudaBackend& backend() { return *backend_; }
  uint64_t step() const { return step_; }
  void SetStep(uint64_t s) { step_ = s; }
  void SetHorizon(uint64_t steps) { horizon_ = steps; }
  float EffectiveLr() const;

  // Copies one batch into the plan's I/O slots (host -> device, asynchronous
  // from an internal pinned double buffer).
  Status StageBatch(const void* input, uint64_t input_bytes, const void* labels,
                    uint64_t label_bytes);
  // One execution of the train program.  With grad accumulation the caller
  // runs it G times and then StepProgram().  `advance` moves the 1-indexed
  // timestep first (once per optimizer step).
  Status TrainForwardBackward(bool advance);   // [0, opt_begin)
  Status TrainOptimizer();                     // [opt_begin, end)
  Status StepProgram();
  Status ReadLoss(float* loss);
  // Evaluation of the staged batch: the eval program, its loss, and on the
  // device the accuracy tally and the real-row loss over the batch's first
  // `real_rows` rows (the whole batch when real_rows >= the plan's batch).
  Status Evaluate(EvalResult* out, uint64_t real_rows = ~0ull);
  // Merge: every adapter's delta, then a device-side finiteness scan.
  Status RunMerge(bool* all_finite);

  Status ReadArena(uint64_t off, uint64_t bytes, void* dst) { return backend_->ReadArena(off, bytes, dst); }
  Status WriteArena(uint64_t off, uint64_t bytes, const void* src);
  Status ReadPersistent(void* dst) { return backend_->ReadArena(0, header_.persistent_size, dst); }
  Status WritePersistent(const void* src);

  // Checkpoint / gate snapshot of the persistent prefix (adapters and optimizer
  // moments) without stalling training (reference: runtime/gating/gate.h:20-49
  // keeps the best state; runtime/storage/checkpoint.h saves it).
  // SnapshotBegin copies the prefix aside on the compute stream — a device-to-
  // device copy at the current point of the step sequence, so later steps may
  // overwrite the arena — and moves that copy to pinned host memory on a second
  // stream while training continues.  SnapshotWait blocks until the bytes are
  // on the host and copies them to `dst`.  Restore is the inverse for a resume:
  // the prefix back into the arena, the timestep set.
  Status SnapshotBegin();
  Status SnapshotWait(void* dst, uint64_t bytes);
  Status Restore(const void* src, uint64_t bytes, uint64_t step);

  // Replays each phase as a CUDA graph after its first eager execution.
  void SetUseGraphs(bool on) { use_graphs_ = on; }
  void SetPhaseTiming(bool on) { phase_timing_ = on; }
  StepTimings TakeTimings();
  // The contiguous arena block holding every optimizer step's gradient
  // operand (what data parallelism exchanges between backward and optimizer).
  void GradientBlock(uint64_t* off, uint64_t* bytes) const { *off = grad_off_; *bytes = grad_bytes_; }
  // Data parallelism: joins the ranks' communicator (a collective call, same id
  // on every rank) and from then on all-gathers the gradient block on the step
  // stream between the backward range and the optimizer range; the optimizer
  // kernels fold the copies in rank order.  Plans with a masked loss are refused
  // (each shard's gradient is a mean over its own target count).  Exchange()
  // enqueues the step's all-gather now (a host that wants to time it); otherwise
  // TrainOptimizer / StepProgram do it when a backward has run since the last one.
  Status AttachExchange(int world, int rank, const uint8_t* id);
  void DetachExchange();
  Status Exchange();
  bool has_masked_loss() const;
  uint64_t train_instructions() const { return train_.size(); }
  const std::vector<Instruction>& program(int which) const;  // 0 train, 1 eval, 2 merge, 3 step

 private:
  UpdateEngine() = default;
  struct GraphSlot {
    cudaGraphExec_t exec = nullptr;
    int runs = 0;
  };
  Status RunRange(const std::vector<Instruction>& prog, size_t begin, size_t end, GraphSlot* slot,
                  float* phase_ms);
  StepParams MakeParams() const;
  void DropGraphs();

  std::unique_ptr<CudaBackend> backend_;
  PlanHeader header_{};
  std::vector<Instruction> train_, eval_, merge_, step_prog_;
  std::vector<EmitEntry> emit_;
  PhaseBoundaries phases_;
  uint64_t step_ = 0, horizon_ = 0;
  uint64_t grad_off_ = 0, grad_bytes_ = 0;
  bool use_graphs_ = false, phase_timing_ = false;
  GraphSlot g_fwdbwd_, g_opt_, g_eval_, g_step_;
  uint8_t* pinned_ = nullptr;        // staging double buffer
  uint64_t pinned_bytes_ = 0;
  int pinned_slot_ = 0;
  cudaEvent_t staged_[2] = {nullptr, nullptr};
  cudaEvent_t ev_[4] = {nullptr, nullptr, nullptr, nullptr};
  StepTimings timings_;
  unsigned long long* d_tally_ = nullptr;  // {rows, correct, nonfinite, loss rows}
  double* d_eval_out_ = nullptr;           // the real-row loss sum
  double* d_eval_terms_ = nullptr;         // per-row (per-element) loss terms
  uint64_t eval_terms_capacity_ = 0;
  EvalTail eval_tail_;
  // snapshot path
  uint8_t* d_snap_ = nullptr;
  uint8_t* h_snap_ = nullptr;
  uint64_t snap_bytes_ = 0;
  cudaStream_t copy_stream_ = nullptr;
  cudaEvent_t snap_taken_ = nullptr, snap_done_ = nullptr;
  bool snap_pending_ = false;
  // where the eval program's loss-forward leaves its probabilities
  uint64_t eval_probs_ref_ = kNullRef, eval_labels_ref_ = kNullRef, eval_rows_ = 0, eval_cols_ = 0;
  std::unique_ptr<GradientExchange> exchange_;
  bool exchange_pending_ = false;
  bool loaded_ = false;
};

}  // namespace see

#endif  // SEE_CUDA_ENGINE_H_
