/* see_cuda.h — the C ABI of the B200 executor backend (libsee_cuda.so).
 *
 * The reference has no C ABI: its executor backends are C++ classes behind
 * `seeml::update_rt::ExecutorBackend` (reference: runtime/executor/backend.h:82-166),
 * chosen by `CreateBackend` (reference: runtime/executor/backend.cc:26-60).
 * Each entry point below is the C spelling of one member of that seam, so a
 * maintainer's `CudaBackend : ExecutorBackend` adapter is one forwarding line
 * per method.  Plain pointers and sizes only.
 *
 * Every function returns 0 on success and a nonzero code on failure;
 * see_cuda_last_error(h) then holds a one-line "<unit>: <message>" diagnostic.
 * A handle is not thread-safe; use one handle per GPU.  There is no CPU
 * fallback: with no sm_100 device see_cuda_create fails.
 */
#ifndef SEE_CUDA_H_
#define SEE_CUDA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct see_cuda_backend see_cuda_backend;

/* Per-range scalars (reference: runtime/executor/backend.h:56-63, StepParams). */
typedef struct see_step_params {
  float lr, beta1, beta2, eps, weight_decay;
  uint32_t pad;
  uint64_t step; /* 1-indexed AdamW timestep */
} see_step_params;

typedef struct see_cuda_counters {
  uint64_t relaxed_executions; /* reference: backend.h:149-161 */
  uint64_t fused_dispatches;   /* reference: backend.h:162-165 */
  uint64_t kernel_launches;
  uint64_t h2d_bytes, d2h_bytes;
  uint64_t instructions;
  uint64_t split_executions; /* exact f32 products run as bf16 pieces on the tensor cores */
} see_cuda_counters;

enum { SEE_OK = 0, SEE_ERROR = 1, SEE_REFUSED = 2 };
enum { SEE_COHERENCE_STRICT = 0, SEE_COHERENCE_LAZY = 1 };

/* CreateBackend(kCuda) — reference: runtime/executor/backend.cc:26-60.  On
 * failure *out is NULL and see_cuda_create_error() names the reason. */
int see_cuda_create(int device_ordinal, see_cuda_backend** out);
const char* see_cuda_create_error(void);
void see_cuda_destroy(see_cuda_backend* h);

/* name() / device() — reference: backend.h:86-87. */
const char* see_cuda_name(see_cuda_backend* h);
const char* see_cuda_device(see_cuda_backend* h);
const char* see_cuda_last_error(see_cuda_backend* h);

/* Bind — reference: backend.h:89-101.  `arena` stays the caller's; the device
 * slab is a mirror at the same offsets.  A refused bind keeps the previous one. */
int see_cuda_bind(see_cuda_backend* h, uint8_t* arena, uint64_t arena_bytes,
                  const uint8_t* rodata, uint64_t rodata_bytes);
/* BindSource — reference: backend.h:103-109.  NULL unbinds. */
int see_cuda_bind_source(see_cuda_backend* h, const uint8_t* data, uint64_t bytes);

/* BeginRange / Execute / EndRange / Flush — reference: backend.h:119-147.
 * `instructions` points at 64-byte instruction words (the plan's own bytes). */
int see_cuda_begin_range(see_cuda_backend* h, const void* instructions, uint64_t count,
                         uint64_t begin, uint64_t end);
int see_cuda_execute(see_cuda_backend* h, const void* instruction, const see_step_params* params);
int see_cuda_end_range(see_cuda_backend* h);
int see_cuda_flush(see_cuda_backend* h);

/* Convenience over the three calls above: BeginRange, Execute each of
 * [begin, end), Flush, EndRange — the engine's ExecuteRange (reference:
 * runtime/dispatcher/update_engine.cc:325-364).  On an Execute failure
 * *failed_index (if not NULL) is the instruction's index. */
int see_cuda_run_range(see_cuda_backend* h, const void* instructions, uint64_t count,
                       uint64_t begin, uint64_t end, const see_step_params* params,
                       uint64_t* failed_index);

/* Coherence between the caller's host arena and the device slab (the seam's
 * "after Flush the arena is readable by the CPU", backend.h:144-147, made
 * explicit for discrete memory).  Strict (default): Flush downloads every
 * range written since the previous Flush.  Lazy: only see_cuda_host_needs
 * downloads.  The host announces its own writes in either mode. */
int see_cuda_set_coherence(see_cuda_backend* h, int mode);
int see_cuda_host_wrote(see_cuda_backend* h, uint64_t offset, uint64_t bytes);
int see_cuda_host_needs(see_cuda_backend* h, uint64_t offset, uint64_t bytes);

int see_cuda_counters_get(see_cuda_backend* h, see_cuda_counters* out);

/* Knobs with no counterpart in the reference seam. */
int see_cuda_set_stream(see_cuda_backend* h, void* cuda_stream);     /* run on the caller's stream */
void* see_cuda_device_arena(see_cuda_backend* h);                      /* device address of offset 0 */
int see_cuda_set_relaxed_allowed(see_cuda_backend* h, int allowed);  /* 0: always the exact kernels */
/* 0: every instruction is its own kernel(s) even in lazy coherence (no bias add or
 * activation absorbed into a product's epilogue); default 1. */
int see_cuda_set_epilogue_fusion(see_cuda_backend* h, int enabled);
/* 0: an adapter's rank-r expand product stays its own kernel instead of riding the
 * frozen product's tensor-core reduction (lazy coherence only); default 1. */
int see_cuda_set_lora_fold(see_cuda_backend* h, int enabled);
/* 0: the rank-r adapter products keep one rounding per operation (the CPU's
 * arithmetic, bit for bit) in lazy coherence too; default 1: fused multiply-adds
 * there.  Strict coherence is always bit-exact. */
int see_cuda_set_adapter_fma(see_cuda_backend* h, int enabled);
/* Lazy coherence: the relaxed attention forward keeps a private f32 copy of its output, and the dQ
 * instruction of the same attention takes delta_i = sum_j P_ij dP_ij as dO_i . O_i from it and walks
 * the keys once instead of twice.  Same quantity, another rounding (tolerance class, like every relaxed
 * attention result).  Default on; 0 keeps the two-walk kernel. */
int see_cuda_set_attention_one_walk(see_cuda_backend* h, int enabled);
/* Exact f32 products (kGemmNN / kGemmNT / kGemmTN without the relaxed permission)
 * of at least 2^26 multiply-adds on the tensor cores: both operands cut into
 * three bf16 pieces, six piece products over a K axis six times as long, f32
 * accumulation.  The result is the f32 product to a few 2^-24 of sum|a_k b_k|
 * (the reference holds its own GEMMs to 2e-6 of that: test/runtime/executor/
 * kernels_test.cc:1803-1822), not the CPU's bits.  mode -1 (default): in lazy
 * coherence only; 0: never; 1: in strict coherence too. */
int see_cuda_set_split_gemm(see_cuda_backend* h, int mode);
/* Large tensor-core products run on CTA pairs (two SMs per 256 x 256 tile, each loading half of the
 * weight tile).  Default on; 0 = one CTA per 128 x 256 tile.  Results are identical either way (the same
 * products in the same order).  Process-wide, not per handle. */
int see_cuda_set_cta_pairs(int enabled);
/* In lazy coherence an adapter site's three backward products (dT = a dY B^T, dB = a t^T dY,
 * dA = x^T dT) run as 3xTF32 on the tcgen05 tensor cores where the site's shape allows (rank 16,
 * widths multiples of 128).  Default on; 0 = the legacy tensor instruction's kernel for every site.
 * Both hold the reference's bound for its own GEMMs (2e-6 of 1 + sum|a_k b_k|,
 * test/runtime/executor/kernels_test.cc:1803-1822); their bits differ.  Process-wide, not per handle.
 * No counterpart in the reference. */
int see_cuda_set_adapter_tensor_backward(int enabled);
/* Data parallelism: optimizer steps read gradients inside [block_offset,
 * block_offset + block_bytes) as the rank-ordered sum of `ranks` gathered
 * copies (device memory, copy r at gathered + r * block_bytes) times 1/ranks. */
int see_cuda_set_gradient_gather(see_cuda_backend* h, int ranks, const void* gathered_device,
                                 uint64_t block_offset, uint64_t block_bytes);
/* Symmetric per-column int8 quantisation of a frozen weight W [K, N] on the
 * device, with the compiler's own arithmetic, so a weight patched by a
 * committed update can be re-packed where it lies: scale[n] = max_k |w[k,n]| /
 * 127 (an all-zero column takes 1; never below FLT_MIN), level = round half
 * away from zero of w / scale, clamped to +-127 (reference:
 * compiler/backend/allocation/arena_binder.cc:129-190).  All three are DEVICE
 * pointers; levels [K, N] int8, scales [N] f32; bit-identical to the reference. */
int see_cuda_quantize_columns(see_cuda_backend* h, const float* w, uint64_t K, uint64_t N,
                              int8_t* levels, float* scales);
/* Profile mode: CUDA-event pairs around every instruction (the profiler hook,
 * reference: runtime/profiler/kernel_profile.h:25-72).  take_profile fills up
 * to `capacity` records and returns the count. */
typedef struct see_profile_record {
  uint16_t opcode;
  uint16_t absorbed; /* following instructions this one also did (epilogue fusion) */
  uint32_t index;
  float ms;        /* the whole instruction */
  float kernel_ms; /* the tensor-core GEMM kernel alone, 0 when the instruction did not use it */
  uint64_t m, n, k;
} see_profile_record;
int see_cuda_set_profiling(see_cuda_backend* h, int on);
int64_t see_cuda_take_profile(see_cuda_backend* h, see_profile_record* out, uint64_t capacity);

/* ---- Softmax cross-entropy forward without any allocation ----------------------
 * No counterpart in the reference (its CPU kernel keeps its partial sums on the
 * stack; reference: runtime/executor/loss.cc:35-57).  For callers that may not
 * call cudaMalloc — a plugin inside a host whose pool already owns the device's
 * memory, a loop where allocation after start-up is forbidden, or the caller's
 * own stream capture.  Same arithmetic and kernels as the kSoftmaxXEntFwd
 * instruction; the per-row scratch is a fixed array inside the library, so
 * `rows` is limited to see_cuda_static_max_rows() (65536) and larger batches are
 * refused with SEE_ERROR.  logits [rows, classes], labels [rows] (i32), loss [1]
 * and probs [rows, classes] are DEVICE pointers; the work is enqueued on
 * `cuda_stream`.  The first call on a device looks up the array's address — make
 * it before any stream capture (and one first call per row-width class: rows of
 * 4096..32768 classes use a kernel whose first launch configures it).  All calls share the array: calls that can
 * overlap on the GPU race.  masked != 0 selects the form that ignores labels of -1. */
int see_cuda_xent_forward_static(const float* logits, const int32_t* labels, float* loss,
                                 float* probs, uint64_t rows, uint64_t classes, int masked,
                                 void* cuda_stream);
uint64_t see_cuda_static_max_rows(void);
const char* see_cuda_static_last_error(void);

/* ---- The dispatcher: UpdateEngine over the CUDA backend ----------------------
 * Mirrors the hot-path surface of seeml::update_rt::UpdateEngine (reference:
 * runtime/dispatcher/update_engine.h:211-367).  The engine owns the device slab
 * (zeroed, persistent image at offset 0 — reference: runtime/loader/
 * plan_loader.cc:251-288); the host moves bytes only through the calls below. */
typedef struct see_engine see_engine;

int see_engine_create(int device_ordinal, see_engine** out); /* error: see_cuda_create_error() */
void see_engine_destroy(see_engine* h);
const char* see_engine_last_error(see_engine* h);
/* The engine's backend, for the see_cuda_* knobs (stream, counters, gradient
 * gather, profiling).  Borrowed: do not destroy it. */
see_cuda_backend* see_engine_backend(see_engine* h);

/* LoadFromMemory — reference: update_engine.h:227-243, update_engine.cc:211-301:
 * seal, version window, section bounds, every instruction's operand extents.
 * A refused load keeps the previous plan bound. */
int see_engine_load(see_engine* h, const uint8_t* plan, uint64_t bytes);
/* BindSourceModel — reference: update_engine.h:245-252. */
int see_engine_bind_source(see_engine* h, const uint8_t* data, uint64_t bytes);
/* Copies the decoded 320-byte plan header (reference: source/plan/schema.h:298-386). */
int see_engine_header(see_engine* h, void* out_320_bytes);

/* One batch into the I/O slots — what BatchPipeline::NextBatch's memcpy does
 * (reference: runtime/pipeline/batch_pipeline.h:43-57, update_engine.cc:853),
 * here a pinned double-buffered host->device copy. */
int see_engine_stage_batch(see_engine* h, const void* input, uint64_t input_bytes,
                           const void* labels, uint64_t label_bytes);
/* ExecuteTrainProgram as two ranges split where the optimizer phase begins
 * (reference: update_engine.cc:318-364; runtime/profiler/step_timings.h:37-59),
 * so a data-parallel driver can exchange gradients between them.
 * advance_step != 0 moves the 1-indexed AdamW timestep first. */
int see_engine_train_forward_backward(see_engine* h, int advance_step);
int see_engine_train_optimizer(see_engine* h);
/* ExecuteStepProgram (gradient accumulation) — reference: update_engine.cc:318-323. */
int see_engine_step_program(see_engine* h);
/* LossValue — reference: update_engine.cc:366-368.  Also surfaces a refusal. */
int see_engine_read_loss(see_engine* h, float* loss);
/* Evaluate one staged batch: eval program, loss, and the accuracy tally
 * (rows judged, argmax hits; reference: update_engine.cc:432-580) on device. */
int see_engine_evaluate(see_engine* h, float* loss, uint64_t* rows, uint64_t* correct);
/* The same with the batch's first `real_rows` rows as its real rows — a
 * validation set's last batch wraps, and its duplicate rows count neither for
 * accuracy nor for the loss (reference: update_engine.cc:486-564).  Also
 * returns the real-row loss: the row-order double sum of each real row's loss
 * and the number of rows it is over (under a masked loss: the real TARGET
 * rows), computed on the device from the loss instruction's own operands
 * (reference: update_engine.cc:977-1026; runtime/executor/loss.cc:78-105).
 * The integer tallies equal the reference's host scan. */
typedef struct see_eval_result {
  float loss;            /* the eval program's loss slot (mean over the whole batch) */
  uint32_t has_accuracy; /* class labels + a softmax covering the batch */
  uint64_t rows;         /* rows judged for accuracy */
  uint64_t correct;      /* argmax == label among them; the first maximum wins */
  double real_row_loss;  /* sum of per-row losses over the real rows */
  uint64_t loss_rows;    /* rows that sum is over */
} see_eval_result;
int see_engine_evaluate_rows(see_engine* h, uint64_t real_rows, see_eval_result* out);
/* RunMerge + the finiteness scan of every delta — reference: update_engine.cc:1028-1063. */
int see_engine_run_merge(see_engine* h, int* all_finite);
/* Arena access for checkpoints, gate snapshots and commit (reference:
 * update_engine.cc:763, 1148-1159, 1172-1235). */
int see_engine_read_arena(see_engine* h, uint64_t offset, uint64_t bytes, void* dst);
int see_engine_write_arena(see_engine* h, uint64_t offset, uint64_t bytes, const void* src);

uint64_t see_engine_step(see_engine* h);
int see_engine_set_step(see_engine* h, uint64_t step);      /* resume */
int see_engine_set_horizon(see_engine* h, uint64_t steps);  /* the run's length, for the schedule */
/* EffectiveLr — reference: update_engine.cc:370-391. */
float see_engine_effective_lr(see_engine* h);
/* Replay each range as a CUDA graph after its first eager execution. */
int see_engine_set_use_graphs(see_engine* h, int on);
/* StepProfiler — reference: runtime/profiler/step_timings.h:69-131 — with CUDA
 * events: forward / backward / optimizer milliseconds accumulated per step. */
int see_engine_set_phase_timing(see_engine* h, int on);
int see_engine_take_timings(see_engine* h, float* forward_ms, float* backward_ms,
                            float* optimizer_ms, uint64_t* steps);
/* The contiguous arena block holding every optimizer step's gradient operand
 * (reference: compiler/backend/allocation/arena_binder.cc:56-77 binds them back to back). */
int see_engine_gradient_block(see_engine* h, uint64_t* offset, uint64_t* bytes);

/* Data parallelism, one engine per GPU and process.  No counterpart in the reference (it has no
 * distributed path); what is exchanged is the gradient block above, once per optimizer step.
 * see_cuda_exchange_id: a fresh 128-byte communicator id (ncclGetUniqueId; NCCL is resolved from the
 *   process at run time, error text in see_cuda_create_error()).  One rank makes it and the host hands it
 *   to the others by whatever channel it has.
 * see_engine_attach_exchange: a COLLECTIVE call (every rank, same id): joins the communicator and allocates
 *   the gather buffer.  From then on the step's all-gather runs on the engine's stream between the backward
 *   range and the optimizer range (inside see_engine_train_optimizer / see_engine_step_program, or earlier
 *   through see_engine_exchange for a host that wants to time it), and the optimizer kernels sum the
 *   gathered copies in rank order and scale by 1/world: the same bits on every rank and every run.
 *   Refused for plans with a masked loss (shards would need a target-count-weighted mean).  world <= 1
 *   detaches. */
int see_cuda_exchange_id(uint8_t* out128);
int see_engine_attach_exchange(see_engine* h, int world, int rank, const uint8_t* id128);
int see_engine_detach_exchange(see_engine* h);
int see_engine_exchange(see_engine* h);

/* Checkpoint / gate snapshot of the persistent prefix (adapters + optimizer moments) without stalling
 * training; replaces the host copies the reference engine makes of the persistent segment for its gate and
 * checkpoints (reference: runtime/gating/gate.h:20-49, runtime/storage/checkpoint.h, runtime/dispatcher/update_engine.cc:763).
 * `begin` takes the copy at the current point of the step sequence (device to device on the compute stream)
 * and downloads it on a second stream while later steps run; `wait` blocks until it is on the host and
 * copies it to dst (bytes must equal the header's persistent_size).  `restore` is the resume path: the
 * prefix back into the arena and the optimizer timestep set. */
int see_engine_snapshot_begin(see_engine* h);
int see_engine_snapshot_wait(see_engine* h, void* dst, uint64_t bytes);
int see_engine_restore(see_engine* h, const void* src, uint64_t bytes, uint64_t step);

#ifdef __cplusplus
}
#endif

#endif /* SEE_CUDA_H_ */
