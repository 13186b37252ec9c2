// The tensor-core path for GEMMs that carry the relaxed permission: the f32
// activation is rounded once to bf16 (round to nearest even), the frozen
// weight is widened exactly to bf16 (int8 and bf16 weights) or rounded to it
// (f32 weights), products accumulate in f32 in tensor memory (tcgen05 / TMEM),
// operands arrive through TMA.  Host-side planning lives here; the kernel in
// k_gemm_umma.cu.
#ifndef SEE_CUDA_UMMA_GEMM_H_
#define SEE_CUDA_UMMA_GEMM_H_

#include <cuda_runtime.h>

#include <cstdint>
#include <string>

#include "kernels.h"
#include "plan_abi.h"

namespace see::umma {

struct Impl;
struct Context {
  Impl* impl = nullptr;
};

// Returns an empty string, or why the tensor-core path cannot be set up.
// `status` is the backend's device status block; a bounded wait that runs out is raised there.
std::string Init(Context* ctx, int device, k::DeviceStatus* status);
void Destroy(Context* ctx);

// Cached operand conversions: frozen weights are converted once per binding;
// an activation's bf16 copy is reused by every GEMM that reads the same arena
// range until an instruction writes into that range.
void InvalidateAll(Context* ctx);
void InvalidateRange(Context* ctx, uint64_t arena_off, uint64_t bytes);
void PlanRange(Context* ctx, const Instruction* program, size_t begin, size_t end);

// Runs C = epilogue(A @ B) on the tensor cores when the shape is inside the
// kernel's domain.  *launches is the number of kernels enqueued; 0 with an
// empty return value means "not applicable — use the exact kernel".
// b_space: 1 = rodata, 2 = source model; offsets identify operands for caching.
std::string TryGemm(Context* ctx, const k::GemmArgs& args, int b_space, uint64_t b_off,
                    uint64_t a_off, uint64_t a_scale_off, cudaStream_t stream, int* launches);

// An adapter site's three backward products (k::LoraBackwardArgs) as 3xTF32 on the tcgen05
// tensor cores, one pass over dY and x, when the shape is inside that kernel's domain.
// *launches == 0 with an empty return value: not applicable, use k::LoraBackward.
std::string TryLoraBackward(Context* ctx, const k::LoraBackwardArgs& args, cudaStream_t stream, int* launches);

// An EXACT f32 product on the tensor cores: both operands cut into three bf16
// pieces, the six largest piece products summed over a K axis six times as long
// (k::SplitMatrix), f32 accumulation in tensor memory.  The result is the f32
// product to a few 2^-24 of sum|a_k b_k| — the accuracy the exact CUDA-core
// kernels have against a float64 sum, not their bits — at a sixth of the bf16
// tensor rate instead of the FP32 pipe's.  Takes NN, NT and TN forms with f32
// operands in any address space; epilogue addend / bias / activation as usual.
// *launches == 0 with an empty return value: outside the domain (small or odd
// shapes, narrow outputs), use the exact kernels.
bool SplitGemmEligible(const k::GemmArgs& args);
std::string TrySplitGemm(Context* ctx, const k::GemmArgs& args, int b_space, uint64_t b_off,
                         cudaStream_t stream, int* launches);
// Sizes the two operand buffers for the largest eligible product of a range
// (called with the other per-range sizing, before any capture).
void PlanSplitGemms(Context* ctx, const Instruction* program, size_t begin, size_t end);

// Producer-side conversion: the instruction that writes a tensor a relaxed GEMM
// reads next can emit the bf16 copy itself (k::Shadow) and spare the GEMM's
// conversion pass the f32 re-read.  ReserveShadow picks an activation slot and
// returns its buffer (null when none can hold M x K); after the producing
// instruction's own write extents have gone through InvalidateRange, CommitShadow
// publishes the slot under the key TryGemm looks up (arena offset, scale offset,
// M, K).  A reservation that is not committed is simply reused later.
// keep_reserved: a second reservation beside the one already held (an instruction
// that writes two tensors).
uint16_t* ReserveShadow(Context* ctx, uint64_t elems, bool keep_reserved = false);
// True when a valid copy with this key exists; marks it most recently used (so
// the next ReserveShadow does not take its slot).
bool TouchActCopy(Context* ctx, uint64_t a_off, uint64_t a_scale_off, uint64_t M, uint64_t K);
// Drops a reservation that was never committed.
void ReleaseReservations(Context* ctx);
void CommitShadow(Context* ctx, uint16_t* buf, uint64_t a_off, uint64_t a_scale_off, uint64_t M,
                  uint64_t K);

// Runs one tiled attention opcode (kAttnFwdTiled / kAttnDQTiled / kAttnDKTiled /
// kAttnDVTiled) on the tensor cores when the geometry is inside the kernels'
// domain (head width 64 or 128, sequence length a multiple of 8).  Operands are
// device pointers into the arena; the *_off arguments are their arena offsets,
// used to reuse packed bf16 copies between the backward opcodes of one layer.
// *launches == 0 with an empty return value means "not applicable".
struct AttentionOperands {
  const float* q; const float* k; const float* v; const float* dout;
  uint64_t q_off, k_off, v_off, dout_off;
  float* stats; float* out;
  uint64_t B, S, H, d;
  k::Shadow shadow;   // optional bf16 copy of `out`
  // kAttnDKTiled only: the kAttnDVTiled that follows on the same operands, done in
  // the same walk (its output; head width 64 only — TryAttention ignores it otherwise
  // and reports through *did_second).
  float* out2 = nullptr;
  k::Shadow shadow2;   // optional bf16 copy of `out2`
  // kAttnFwdTiled: where to keep a private f32 copy of the output for the dQ of the same
  // attention; kAttnDQTiled: that copy (one walk over the keys instead of two).
  float* keep = nullptr;
  const float* fwd_keep = nullptr;
};
// A producer (a tensor-core GEMM epilogue) can write an attention operand's packed rows
// itself: ReservePack hands out an entry's buffer (null when none fits `elems`), CommitPack
// publishes it under the tensor's arena offset once the producing instruction's own write
// extents have gone through InvalidateRange; TryAttention then finds it and packs nothing.
uint16_t* ReservePack(Context* ctx, uint64_t elems);
void CommitPack(Context* ctx, uint16_t* rows, uint64_t src_off, uint64_t elems);
// True when a valid copy of the tensor at `src_off` exists; marks it most recently used.
bool TouchPack(Context* ctx, uint64_t src_off, uint64_t elems);
std::string TryAttention(Context* ctx, uint16_t opcode, const AttentionOperands& op,
                         cudaStream_t stream, int* launches, bool* did_second = nullptr);

// Profile mode: the next tensor-core launch records `before` / `after` around
// the kernel itself (not the operand conversions).  Returns whether a launch
// consumed them since the last call.
void SetProfileEvents(Context* ctx, cudaEvent_t before, cudaEvent_t after);
bool ProfileEventsUsed(Context* ctx);

}  // namespace see::umma

#endif  // SEE_CUDA_UMMA_GEMM_H_
