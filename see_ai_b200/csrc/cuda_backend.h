// CudaBackend — the B200 executor behind the reference's backend seam.  The
// method set, argument meaning and error behaviour mirror
// seeml::update_rt::ExecutorBackend (reference: runtime/executor/backend.h:82-166):
// Bind / BindSource / Configure / Execute / BeginRange / EndRange / Flush,
// relaxed_executions(), fused_dispatches().  Host-only header (C++23).
//
// What differs from a unified-memory backend is coherence.  The compiler's
// arena lives in ONE cudaMalloc'd slab at the compiler-decided offsets; the
// caller's host arena is a mirror.  Two modes:
//   strict (default)  Flush copies every range written since the last Flush
//                     back into the host arena, so the seam's promise — after
//                     Flush the arena's bytes are what the instructions
//                     computed — holds byte for byte.
//   lazy              nothing is copied back unless asked (HostNeeds); the
//                     engine asks for the loss slot each step and for the
//                     persistent prefix or deltas when it checkpoints/merges.
// In both modes the host announces its own writes (HostWrote) and they are
// uploaded before the next instruction runs; Bind uploads the whole arena.
#ifndef SEE_CUDA_BACKEND_H_
#define SEE_CUDA_BACKEND_H_

#include <cuda_runtime.h>

#include <cstdint>
#include <expected>
#include <map>
#include <memory>
#include <span>
#include <string>
#include <utility>
#include <vector>

#include "extents.h"
#include "kernels.h"
#include "plan_abi.h"

namespace see {

using Status = std::expected<void, std::string>;

// The two refusal verdicts, worded as the reference words them (reference:
// runtime/executor/backend.h:72-80) so a twin test can compare strings.
inline constexpr const char* kNonFiniteNormRefusal =
    "gradient norm is not finite — the step was refused with the parameters "
    "and optimizer state untouched";
inline constexpr const char* kClipThresholdRefusal =
    "clip threshold is not a finite positive float — the instruction was "
    "refused with the gradient untouched";

enum class Coherence : int { kStrict = 0, kLazy = 1 };

struct Counters {
  uint64_t relaxed_executions = 0;   // instructions run on the tensor-core (bf16) path
  uint64_t fused_dispatches = 0;     // instruction pairs run as one launch
  uint64_t kernel_launches = 0;      // device kernels enqueued since creation
  uint64_t h2d_bytes = 0, d2h_bytes = 0;
  uint64_t instructions = 0;
  uint64_t split_executions = 0;     // exact f32 products run as bf16 pieces on the tensor cores
};

// One timed instruction (profile mode): opcode, index in the range, milliseconds.
// kernel_ms > 0 only for instructions that ran on the tensor-core GEMM: the
// kernel alone, without the operand conversions that ms also covers.
struct ProfileRecord {
  uint16_t opcode; uint32_t index; float ms; uint64_t m, n, k; float kernel_ms = 0.0f; bool has_kernel = false;
  uint16_t absorbed = 0;   // following instructions this one also did
};

class CudaBackend {
 public:
  static std::expected<std::unique_ptr<CudaBackend>, std::string> Create(int device_ordinal);
  ~CudaBackend();
  CudaBackend(const CudaBackend&) = delete;
  CudaBackend& operator=(const CudaBackend&) = delete;

  const char* name() const { return "cuda"; }
  std::string device() const { return device_label_; }

  // A refused Bind leaves the previous binding intact and executable.
  Status Bind(uint8_t* arena, uint64_t arena_bytes, const uint8_t* rodata, uint64_t rodata_bytes,
              uint64_t rodata_mapped_bytes);
  Status BindSource(const uint8_t* data, uint64_t bytes);
  // The engine's form of Bind: the slab is created on the device as the
  // runtime's arena is created on the host — zeroed, then the persistent image
  // copied to offset 0 (reference: runtime/loader/plan_loader.cc:251-288) — with
  // no host mirror at all.  Coherence is then lazy by construction: the engine
  // moves bytes with ReadArena / WriteArena.
  Status BindDeviceImage(uint64_t arena_bytes, const uint8_t* prefix, uint64_t prefix_bytes,
                         const uint8_t* rodata, uint64_t rodata_bytes);
  // Synchronous device -> dst.  Orders after everything enqueued so far.
  Status ReadArena(uint64_t off, uint64_t bytes, void* dst);
  // Asynchronous src -> device on the backend's stream; `src` must stay valid
  // until the stream has passed the copy (pinned memory for true overlap).
  Status WriteArena(uint64_t off, uint64_t bytes, const void* src);
  void Configure() {}  // the CPU tile policy is throughput-only on its own backend; ignored here

  Status Execute(const Instruction& ins, const StepParams& params);

  // The caller's promise that `program` (the span later passed to BeginRange) is
  // a complete update step that it only ever runs from instruction 0 onwards,
  // pass after pass, and that arena bytes outside `observed` ([offset, bytes)
  // ranges: persistent state, loss, the gradient block ...) are read by nothing
  // but that program's instructions.  Scratch tensors of such a program that no
  // instruction reads before the next pass rewrites them may then be left
  // unwritten by the epilogue fusions (lazy coherence only).
  void DeclareStepProgram(const Instruction* program, std::vector<std::pair<uint64_t, uint64_t>> observed) {
    step_program_ = program;
    observed_ = std::move(observed);
  }
  void BeginRange(std::span<const Instruction> program, size_t begin, size_t end);
  void EndRange();
  Status Flush();

  uint64_t relaxed_executions() const { return counters_.relaxed_executions; }
  uint64_t fused_dispatches() const { return counters_.fused_dispatches; }
  const Counters& counters() const { return counters_; }

  // ---- coherence ----
  void SetCoherence(Coherence mode) { coherence_ = mode; }
  void HostWrote(uint64_t off, uint64_t bytes);
  Status HostNeeds(uint64_t off, uint64_t bytes);  // synchronous device -> host arena

  // ---- stream / device memory access for the engine and the data-parallel driver ----
  void SetStream(cudaStream_t s) { stream_ = s; }
  cudaStream_t stream() const { return stream_; }
  uint8_t* device_arena() const { return d_arena_; }
  uint64_t arena_bytes() const { return arena_bytes_; }
  int device_ordinal() const { return device_; }

  // Data parallelism: optimizer steps whose gradient operand lies inside
  // [block_off, block_off + block_bytes) of the arena read it instead as the
  // rank-ordered sum of `ranks` gathered copies at `gathered` (device memory,
  // copy r at gathered + r * block_bytes), times 1/ranks.  ranks <= 1 clears it.
  void SetGradientGather(int ranks, const void* gathered, uint64_t block_off, uint64_t block_bytes);

  // Allow / forbid the tensor-core path for instructions carrying the relaxed
  // permission (default: allowed).  The exact kernels are always a valid
  // execution of a relaxed instruction.
  void SetRelaxedAllowed(bool allowed) { relaxed_allowed_ = allowed; }
  // Off: no kAddBias or activation is absorbed into a product's epilogue (takes
  // effect at the next BeginRange).
  void SetEpilogueFusion(bool enabled) { epilogue_fusion_ = enabled; }

  // Off: the rank-r expand product of an adapter stays its own kernel instead of
  // riding the frozen product's reduction (takes effect at the next BeginRange).
  void SetLoraFold(bool enabled) { lora_fold_enabled_ = enabled; }
  void SetAttentionOneWalk(bool enabled) { attn_one_walk_ = enabled; }

  // Off: the rank-r adapter products keep the CPU's one-rounding-per-operation
  // arithmetic even in lazy coherence (default on: fused multiply-adds there).
  void SetAdapterFma(bool enabled) { adapter_fma_ = enabled; }

  // Exact f32 products (kGemmNN / NT / TN without the relaxed permission) above a
  // size threshold on the tensor cores as six bf16 piece products (umma::TrySplitGemm):
  // f32-class accuracy, not the CPU's bits.  -1 (default): in lazy coherence only;
  // 0: never; 1: in strict coherence too.
  void SetSplitGemm(int mode) { split_gemm_mode_ = mode; }

  // CUDA-graph support for the engine.  The optimizer kernels read the step's
  // learning rate and bias corrections from a small device block.  A captured
  // range contains no upload of that block: before it captures or replays a range
  // with optimizer instructions the engine calls UploadStepScalars, an ordinary
  // stream-ordered copy from a ring of pinned slots (a slot is rewritten only
  // after the copy that last read it has completed), so every replay sees its own
  // step's values however far the host runs ahead of the device.
  void SetCapturing(bool on);
  Status UploadStepScalars(const StepParams& params);
  static k::AdamScalars ScalarsOf(const StepParams& params);

  // Per-column int8 quantisation of W [K, N] (device pointers), the compiler's
  // arithmetic bit for bit (reference: compiler/backend/allocation/arena_binder.cc:129-190).
  Status QuantizeColumns(const float* w, uint64_t K, uint64_t N, int8_t* levels, float* scales);

  // Profile mode: every instruction is bracketed by CUDA events on the stream.
  void SetProfiling(bool on);
  std::vector<ProfileRecord> TakeProfile();

 private:
  explicit CudaBackend(int device);
  Status Init();
  Status Check(cudaError_t e, const char* what);
  Status UploadDirty();
  Status EnsureScratch(uint64_t row_doubles);
  Status EnsureBf16(uint64_t a_elems);
  Status Dispatch(const Instruction& ins, const StepParams& params, const Extents& ext);
  Status DispatchGemm(const Instruction& ins);
  Status DispatchOptimizer(const Instruction& ins, const StepParams& params);

  template <typename T = float>
  const T* Rd(uint64_t ref) const {
    const uint64_t off = RefOffset(ref);
    switch (RefSpace(ref)) {
      case kRodata: return reinterpret_cast<const T*>(d_rodata_ + off);
      case kSource: return reinterpret_cast<const T*>(d_source_ + off);
      default: return reinterpret_cast<const T*>(d_arena_ + off);
    }
  }
  template <typename T = float>
  T* Wr(uint64_t ref) const { return reinterpret_cast<T*>(d_arena_ + RefOffset(ref)); }

  int device_ = 0;
  std::string device_label_;
  cudaStream_t stream_ = nullptr;
  bool own_stream_ = false;

  uint8_t* host_arena_ = nullptr;
  uint64_t arena_bytes_ = 0;
  uint8_t* d_arena_ = nullptr;
  uint8_t* d_rodata_ = nullptr;
  uint64_t rodata_bytes_ = 0;
  uint8_t* d_source_ = nullptr;
  uint64_t source_bytes_ = 0;

  // device scratch
  k::DeviceStatus* d_status_ = nullptr;
  double* d_partials_ = nullptr;  // 256 doubles
  double* d_sq_ = nullptr;
  float* d_clip_scale_ = nullptr;
  unsigned long long* d_count_ = nullptr;
  double* d_rows_ = nullptr;
  uint64_t rows_capacity_ = 0;
  float* d_split_ = nullptr;      // split-K partial sums of the adapter-gradient GEMMs
  uint64_t split_capacity_ = 0;   // floats
  unsigned int* d_colmax_ = nullptr;   // the quantiser's per-column maxima
  uint64_t colmax_capacity_ = 0;
  float* d_gsum_ = nullptr;       // summed gradient for fused clips under data parallelism
  uint64_t gsum_capacity_ = 0;
  k::AdamScalars* d_scalars_ = nullptr;
  k::AdamScalars* h_scalars_ = nullptr;  // pinned ring
  std::vector<cudaEvent_t> scalar_done_; // per slot: the upload that last read it
  int scalar_slot_ = 0;
  StepParams last_params_{};
  bool scalars_valid_ = false;
  bool capturing_ = false;
  int* h_status_ = nullptr;  // pinned mirror of the status words

  Coherence coherence_ = Coherence::kStrict;
  std::vector<std::pair<uint64_t, uint64_t>> host_dirty_;
  std::vector<std::pair<uint64_t, uint64_t>> device_dirty_;
  std::string deferred_error_;

  int gather_ranks_ = 1;
  const uint8_t* d_gathered_ = nullptr;
  uint64_t gather_off_ = 0, gather_bytes_ = 0;
  // A range with a standalone clip instruction (kClipNorm / kSqNormAccum /
  // kClipGlobal) reads and scales the gradient where it lies in the arena, so
  // under data parallelism the rank-ordered mean of the gathered copies is
  // written into the arena block once, at the range's first optimizer-phase
  // instruction, and every instruction after it uses the arena.
  bool fold_gather_ = false;    // this range needs the fold
  bool gather_folded_ = false;  // ... and it has been done
  std::string range_error_;     // a range BeginRange found it cannot run; reported by Execute
  Status FoldGatheredIntoArena();

  bool relaxed_allowed_ = true;
  bool epilogue_fusion_ = true;
  bool profiling_ = false;
  std::vector<std::pair<cudaEvent_t, cudaEvent_t>> events_;
  std::vector<std::pair<cudaEvent_t, cudaEvent_t>> kernel_events_;
  std::vector<ProfileRecord> pending_profile_;
  uint32_t range_index_ = 0;

  // Runs of AdamW instructions issued as one launch (engine / lazy coherence
  // only: in strict mode every instruction's effect must be visible on its own).
  struct AdamGroup { size_t table_begin = 0; int count = 0; uint64_t max_n = 0; };
  void PlanAdamGroups(std::span<const Instruction> program, size_t begin, size_t end);
  std::vector<int32_t> adam_group_of_;   // per range position: -1 none, -2 member, else group index
  std::vector<AdamGroup> adam_groups_;
  k::AdamTensor* d_adam_table_ = nullptr;
  size_t adam_table_capacity_ = 0;

  // A relaxed GEMM followed by the kAddBias that consumes its output, when the
  // un-biased product is provably dead afterwards: the GEMM's epilogue adds the
  // bias and writes the kAddBias output directly; the kAddBias becomes a no-op.
  // Engine / lazy coherence only.
  struct BiasFusion { bool fuse = false; uint64_t bias_ref = kNullRef, out_ref = kNullRef; };
  void PlanBiasFusions(std::span<const Instruction> program, size_t begin, size_t end);
  std::vector<BiasFusion> bias_fusion_;   // per range position (of the GEMM)
  bool skip_next_add_bias_ = false;

  // Producer-side bf16 conversion (k::Shadow): for each instruction of the
  // current range, whether its output is the A operand of a later relaxed GEMM,
  // and under which key that GEMM will look the copy up.
  struct ShadowPlan {
    bool want = false;
    bool only = false;   // the f32 tensor itself is dead: the producer may write the copy alone
    uint64_t a_off = 0, M = 0, K = 0, scale_off = ~0ull, scale_ref = kNullRef;
  };
  void PlanShadows(std::span<const Instruction> program, size_t begin, size_t end);
  const k::Shadow* ShadowFor(uint64_t out_ref, uint64_t elems) const;
  std::vector<ShadowPlan> shadow_plan_;
  ShadowPlan cur_plan_;
  k::Shadow cur_shadow_;
  bool shadow_written_ = false;

  // An activation instruction that follows a relaxed GEMM (directly, or after
  // the kAddBias fused above) and reads its output, done in the GEMM's epilogue
  // when the activation's f32 output is read by nothing but the relaxed GEMM(s)
  // that take its bf16 operand copy before every byte of it is overwritten: the
  // epilogue writes that copy and the f32 tensor is never materialised.  For a
  // backward activation the GEMM's own output (dy) is left unwritten too when it
  // is dead.  Engine / lazy coherence only.  elided_ lists the f32 ranges left
  // stale; any other read of them is refused (a guard behind the static proof).
  struct ActFusion {
    int mode = 0;                 // k::kFuseNone / kFuseActFwd / kFuseActBwd
    Act act = kActNone;
    uint32_t act_index = 0;       // range position of the absorbed instruction
    uint64_t x_ref = kNullRef;    // backward: the forward input
    bool store_c = true;
    uint64_t elided[2][2] = {{0, 0}, {0, 0}};   // [lo, hi) byte ranges
    int elided_count = 0;
  };
  void PlanActFusions(std::span<const Instruction> program, size_t begin, size_t end);
  const Instruction* step_program_ = nullptr;   // see DeclareStepProgram
  std::vector<std::pair<uint64_t, uint64_t>> observed_;
  std::vector<ActFusion> act_fusion_;   // per range position (of the GEMM)
  int64_t skip_act_at_ = -1;
  std::vector<std::pair<uint64_t, uint64_t>> elided_;
  std::vector<std::pair<uint64_t, uint64_t>> pending_elided_;   // joins elided_ once the instruction's own writes are accounted

  // kSoftmaxXEntFwd, the one-element kFill of the seed, kSoftmaxXEntBwd: when only
  // the bf16 copy of the loss gradient is needed, the forward's row pass
  // produces it (the backward instruction launches nothing); the probabilities
  // are stored only if something else reads them.
  struct LossFusion {
    bool fuse = false;
    float seed = 1.0f;
    bool store_probs = true;
    uint32_t bwd_index = 0;
    uint64_t probs_lo = 0, probs_hi = 0;
  };
  std::vector<LossFusion> loss_fusion_;   // per range position (of the forward)

  // A kAddEW that follows a relaxed GEMM (directly, or after the kAddBias fused
  // above) and adds another tensor to its output: done as the epilogue's addend
  // (same f32 add) when the un-summed product is dead afterwards.
  struct AddFusion {
    bool fuse = false;
    uint64_t x_ref = kNullRef, out_ref = kNullRef;
    uint32_t add_index = 0;
    uint64_t z_lo = 0, z_hi = 0;   // the product's own range when it stays unwritten
  };
  std::vector<AddFusion> add_fusion_;   // per range position (of the GEMM)

  // kAttnDKTiled directly followed by kAttnDVTiled on the same operands (relaxed,
  // head width 64): one kernel walks the queries once for both.  Per range
  // position of the dK instruction: the dV output reference, or kNullRef.
  std::vector<uint64_t> attn_dv_out_;
  // Relaxed tiled attention: the forward keeps a private f32 copy of its output for the dQ of the
  // same attention (per instruction of the range: the pool slot, or -1); a slot is usable by dQ
  // once the tensor-core forward of this pass has written it.
  std::vector<int> attn_keep_slot_;
  std::vector<float*> attn_keep_pool_;
  std::vector<uint8_t> attn_keep_written_;
  uint64_t attn_keep_elems_ = 0;
  void PlanAttentionKeeps(std::span<const Instruction> program, size_t begin, size_t end);
  // A tensor-core GEMM whose result a relaxed tiled attention instruction reads as q, k, v or dO
  // writes that operand's packed bf16 rows in its own epilogue (per instruction of the range:
  // the attention geometry, S == 0 when not wanted).
  struct PackPlan {
    uint64_t out_ref = kNullRef;
    uint32_t S = 0, H = 0, d = 0;
    // Nothing but attention instructions of this range (which take the copy) reads the
    // tensor's f32 form before it is written again: the epilogue stores the copy alone.
    bool copy_only = false;
    size_t last = 0;   // range index of the last instruction the dispatch stands for
  };
  // Ranges whose f32 form a dispatch left unwritten, recorded as stale once the instruction
  // at the given range index (the last one the dispatch stood for) has passed.
  struct DeferredElision { size_t after; uint64_t lo, hi; };
  std::vector<DeferredElision> deferred_elided_;
  // What the shared row-operand scratch of the low-rank folds (d_lora_t_) holds: the bf16 cut of the
  // [M, r] tensor at `off`, written by the instruction at range index `producer`; any other
  // instruction that writes into that tensor, or reuses the scratch, ends it.
  struct LoraRowsTag { bool valid = false; uint64_t off = 0, M = 0; uint32_t r = 0; size_t producer = 0; } lora_rows_tag_;
  std::vector<PackPlan> pack_plan_;
  struct PendingPack {
    uint16_t* rows = nullptr;
    uint64_t off = 0, elems = 0;
  } pending_pack_;
  void PlanAttentionPacks(std::span<const Instruction> program, size_t begin, size_t end);
  std::vector<ShadowPlan> attn_dv_shadow_;   // the dV instruction's copy plan, made by the pair's kernel
  int64_t skip_attn_dv_at_ = -1;
  int64_t skip_add_at_ = -1;            // the absorbed kAddEW (its output IS written, by the product)

  // The rank-r expand product of an adapter, C' = C + s T B, folded into the
  // frozen product that makes C (the reference's own GPU backend folds the same
  // pair: runtime/executor/metal_backend.mm:1155-1316): T and the adapter matrix
  // are cut into bf16 pieces and appended to the tensor-core reduction
  // (k_lora.cu), so the expand kernel's read-modify-write of C disappears.  Three
  // instruction patterns, per range position of the frozen product G:
  //   kind 1 (forward)   G; D: t = x A; E: out = G.out + s t B      D runs early, inside G's dispatch
  //   kind 2 (backward)  G; E: out = G.out + dT A^T
  //   kind 3 (backward)  E: part = acc + dT A^T; ...; G; kAddEW: part + G.out    E never runs
  // each optionally followed by a kAddEW that the epilogue absorbs as well.
  // Engine / lazy coherence only; every intermediate left unwritten is proven dead.
  struct LoraFold {
    bool fuse = false;
    int kind = 0;
    Instruction down{};             // kind 1: the down product, executed by the fold
    uint64_t t_ref = kNullRef;      // the [M, r] factor whose split copy feeds the reduction
    uint32_t r = 0;
    uint32_t weight_slot = 0;       // entry of the range's split-weight table
    uint64_t out_ref = kNullRef;    // where the sum is written
    uint64_t addend_ref = kNullRef; // epilogue addend (the absorbed kAddEW's other operand, or kind 3's acc)
    uint32_t absorbed = 0;          // instructions this dispatch stands for besides G
    uint64_t dead[3][2] = {{0, 0}, {0, 0}, {0, 0}};   // f32 ranges left unwritten
    int dead_count = 0;
  };
  std::vector<LoraFold> lora_fold_;          // per range position (of G)
  std::vector<uint8_t> lora_skip_;           // per range position: 1 done by an earlier dispatch, 2 never runs
  std::vector<k::LoraWeight> lora_weights_;  // the range's adapter matrices (host copy of the table)
  uint32_t lora_max_n_ = 0, lora_max_kx_ = 0;
  // The table and the split weights belong to ONE range (a captured range keeps
  // reading them at every replay), so each (program, begin) has its own pair,
  // kept until the next Bind; the row operand is scratch shared by all.
  struct LoraRangeBuffers {
    k::LoraWeight* table = nullptr;
    size_t table_capacity = 0;
    uint16_t* weights = nullptr;   // [entries][max n_out][max kx] bf16
    uint64_t weights_capacity = 0;
  };
  std::map<std::pair<const Instruction*, size_t>, LoraRangeBuffers> lora_ranges_;
  k::LoraWeight* d_lora_table_ = nullptr;    // the current range's
  uint16_t* d_lora_w_ = nullptr;
  uint16_t* d_lora_t_ = nullptr;             // [rows][kx] bf16, reused by every fold
  uint64_t lora_t_capacity_ = 0;
  bool lora_fold_enabled_ = true;
  bool attn_one_walk_ = true;
  bool adapter_fma_ = true;
  // The three backward products of an adapter site (dT = a dY B^T, dB = a t^T dY,
  // dA = x^T dT), which the plan spells as three instructions that each stream a
  // whole activation, as ONE pass over dY and x (k::LoraBackward).  Per range
  // position of the dT instruction; the other two are marked done in lora_skip_.
  struct AdapterBackward {
    bool fuse = false;
    Instruction db{}, da{};
  };
  std::vector<AdapterBackward> adapter_bwd_;
  float* d_lora_partials_ = nullptr;
  uint64_t lora_partials_capacity_ = 0;   // floats
  int split_gemm_mode_ = -1;
  bool SplitGemmOn() const { return split_gemm_mode_ > 0 || (split_gemm_mode_ < 0 && coherence_ == Coherence::kLazy); }
  Status PrepareLoraFolds(const Instruction* program, size_t begin, uint64_t max_rows);
  void FreeLoraRanges();
  k::GemmArgs GemmArgsOf(const Instruction& ins) const;

  Counters counters_;
  struct UmmaState;
  std::unique_ptr<UmmaState> umma_;
};

}  // namespace see

#endif  // SEE_CUDA_BACKEND_H_
