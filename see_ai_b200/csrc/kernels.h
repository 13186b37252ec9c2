// Launchers of the device kernels.  Every function enqueues on `stream` and
// returns; pointers are device pointers.  Arithmetic contracts are stated at
// each definition (which reference kernel's expression it evaluates, and
// whether the result is bit-identical to the CPU executor's or within
// floating-point tolerance of it).
#ifndef SEE_CUDA_KERNELS_H_
#define SEE_CUDA_KERNELS_H_

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "plan_abi.h"

namespace see::k {

// Device-side status block shared by all kernels of one backend.
struct DeviceStatus {
  int refused;        // 1 = a clip saw a non-finite gradient norm; parameter
                      // writers skip their stores while it is set
  int wait_timeout;   // 1 = a bounded device-side wait ran out
  int pad[2];
};

// An optional second output of a producer kernel: a bf16 copy of the tensor it
// writes, laid out [rows][cols] like the tensor, for the tensor-core GEMM that
// reads the tensor next (it would otherwise re-read the f32 values just to
// round them).  dst[i] = bf16_rne(v[i] * (k_scale ? k_scale[i % cols] : 1)) —
// the rounding the GEMM's own conversion pass applies.  Producers honour it on
// their 16-byte vector paths only (ShadowUsable), and ignore it otherwise.
struct Shadow {
  uint16_t* dst = nullptr;
  const float* k_scale = nullptr;   // per-column factor of the consumer (or null)
  size_t cols = 0;
  // The f32 output itself is read by nobody (proven by the caller): a producer
  // that supports it writes the copy alone.  Others ignore the flag.
  bool only = false;
};
inline bool ShadowUsable(const Shadow* sh, const void* out, size_t n) {
  return sh && sh->dst && sh->cols != 0 && sh->cols % 4 == 0 && n % sh->cols == 0 &&
         (reinterpret_cast<uintptr_t>(out) & 15) == 0 &&
         (reinterpret_cast<uintptr_t>(sh->dst) & 7) == 0 &&
         (reinterpret_cast<uintptr_t>(sh->k_scale) & 15) == 0;
}

// ---- elementwise / broadcast / gather -------------------------------------
// Launchers that take a Shadow return true when they wrote it.
bool AddEW(const float* x, const float* y, float* out, size_t n, cudaStream_t s,
           const Shadow* shadow = nullptr);
void MulEW(const float* x, const float* y, float* out, size_t n, cudaStream_t s);
void AddBias(const float* x, const float* b, float* out, size_t rows, size_t cols, cudaStream_t s);
void Accumulate(float* dst, const float* src, size_t n, cudaStream_t s);
void Scale(const float* x, float* out, float alpha, size_t n, cudaStream_t s);
void Fill(float* dst, float value, size_t n, cudaStream_t s);
void Copy(const float* src, float* dst, size_t n, cudaStream_t s);
bool ActFwd(Act act, const float* x, float* out, size_t n, cudaStream_t s,
            const Shadow* shadow = nullptr);
bool ActBwd(Act act, const float* dy, const float* x, float* dx, size_t n, cudaStream_t s,
            const Shadow* shadow = nullptr);
void FusedMap(const float* x, const float* o1, const float* o2, float* out, size_t n,
              uint32_t stages, float imm0, float imm1, cudaStream_t s);
void EmbedFwd(const int32_t* tokens, const float* table, float* out, size_t rows, size_t dim,
              size_t vocab, cudaStream_t s);
void ReduceRows(const float* dy, float* db, size_t rows, size_t cols, cudaStream_t s);
void SegmentStarts(const int32_t* tokens, int32_t* starts, size_t B, size_t S, int32_t eos,
                   cudaStream_t s);
void RopeTable(float* table, size_t S, size_t d, float step, cudaStream_t s);
void Rope(bool backward, const float* x, float* y, size_t B, size_t S, size_t H, size_t d,
          float step, const float* table, cudaStream_t s);
// f32 -> bf16 (round to nearest even), optionally scaling column k by
// col_scale[k] first (the int8 dX GEMM's reduction-axis scales).
void ToBf16(const float* x, uint16_t* out, size_t rows, size_t cols, const float* col_scale,
            cudaStream_t s);

// ---- normalization ----------------------------------------------------------
bool LayerNormFwd(const float* x, const float* gamma, const float* beta, float* y, float* mean,
                  float* rstd, size_t rows, size_t cols, float eps, cudaStream_t s,
                  const Shadow* shadow = nullptr);
// With addend and sum_out both given, a following kAddEW rides along: the kernel
// writes sum_out = addend + dx instead of dx (sum_out may alias addend).  Returns
// 0: dx was written as usual (the kAddEW still has to run); 1: the sum was
// written; 2: the sum and its bf16 copy.
int LayerNormBwd(const float* dy, const float* x, const float* gamma, const float* mean,
                  const float* rstd, float* dx, size_t rows, size_t cols, cudaStream_t s,
                  const float* addend = nullptr, float* sum_out = nullptr,
                  const Shadow* sum_shadow = nullptr);   // the copy the kAddEW would have made of the sum
void RmsNormFwd(const float* x, const float* gamma, float* y, float* rstd, size_t rows,
                size_t cols, float eps, cudaStream_t s);
void RmsNormBwd(const float* dy, const float* x, const float* gamma, const float* rstd,
                float* dx, size_t rows, size_t cols, cudaStream_t s);

// ---- losses -----------------------------------------------------------------
// `row_scratch` holds N doubles (per-row -log p) and `count_scratch` one
// uint64 (the masked forms' target count).
// The backward instruction that follows (dlogits = seed / N * (p - onehot)) can ride
// the forward's row pass when only its bf16 operand copy is needed: XEntFusedBwd
// carries the seed the plan fills in between, the copy, and whether the
// probabilities themselves still have to be stored.  Returns true when the
// backward was done here (wide rows only); false leaves it to SoftmaxXEntBwd.
struct XEntFusedBwd {
  Shadow shadow;
  float seed = 1.0f;
  bool store_probs = true;
};
bool SoftmaxXEntFwd(bool masked, const float* logits, const int32_t* labels, float* loss,
                    float* probs, size_t N, size_t C, double* row_scratch,
                    unsigned long long* count_scratch, cudaStream_t s,
                    const XEntFusedBwd* fused_bwd = nullptr);
bool SoftmaxXEntBwd(bool masked, const float* probs, const int32_t* labels, const float* seed,
                    float* dlogits, size_t N, size_t C, unsigned long long* count_scratch,
                    cudaStream_t s, const Shadow* shadow = nullptr);
void MseFwd(const float* pred, const float* target, float* loss, size_t n, double* scratch,
            cudaStream_t s);
void MseBwd(const float* pred, const float* target, const float* seed, float* dpred, size_t n,
            cudaStream_t s);
void KLDistillFwd(const float* s_logits, const float* t_logits, float* loss, float* p_s,
                  float* p_t, size_t N, size_t C, float T, float loss_scale, double* row_scratch,
                  cudaStream_t s);
void KLDistillBwd(const float* p_s, const float* p_t, const float* seed, float* dlogits,
                  size_t N, size_t C, float T, float loss_scale, cudaStream_t s);

// ---- optimizer / clipping ---------------------------------------------------
// Sum of squares of g in double, per shape-derived chunk then in chunk order;
// result in *sq (device).  `partials` holds 256 doubles.
void L2Squared(const float* g, size_t n, double* partials, double* sq, cudaStream_t s);
// scale = clip factor for threshold `max_norm` from *sq (1 when max_norm <= 0);
// raises status->refused when the norm is not finite.
void ClipScaleFromSq(const double* sq, float max_norm, float* scale, DeviceStatus* status,
                     cudaStream_t s);
void ScaleInPlaceBy(float* g, size_t n, const float* scale, const DeviceStatus* status,
                    cudaStream_t s);
void SqNormAccum(const double* sq, float* acc, cudaStream_t s);
void ClipGlobalScale(const float* acc, float max_norm, float* scale, DeviceStatus* status,
                     cudaStream_t s);
struct AdamScalars {
  float lr, beta1, beta2, eps, weight_decay, inv_bc1, inv_bc2;
};
// g_copies > 1: the gradient is the sum, in copy order, of g_copies blocks
// spaced copy_stride floats apart starting at g, times inv_copies.
// `a` points at device memory (the backend's per-range scalar block), so a
// captured launch picks up each step's learning rate and bias corrections.
void AdamWStep(float* p, const float* g, float* m, float* v, size_t n, const AdamScalars* a,
               const float* clip_scale, const DeviceStatus* status, int g_copies,
               size_t copy_stride, float inv_copies, cudaStream_t s);
// A run of AdamW instructions as one launch: blockIdx.y picks the tensor.  Each
// tensor's arithmetic is AdamWStep's, element for element.
struct AdamTensor {
  float* p; const float* g; float* m; float* v;
  uint64_t n;
  int32_t g_copies; uint32_t pad;
  uint64_t copy_stride;
};
void AdamWStepMulti(const AdamTensor* table, int count, uint64_t max_n, const AdamScalars* a,
                    const DeviceStatus* status, float inv_copies, cudaStream_t s);
void SgdStep(float* p, const float* g, size_t n, const AdamScalars* a,
             const float* clip_scale, const DeviceStatus* status, int g_copies,
             size_t copy_stride, float inv_copies, cudaStream_t s);
// out = (sum over copies in order) * inv_copies, for norms taken on a summed gradient.
void SumCopies(const float* g, float* out, size_t n, int g_copies, size_t copy_stride,
               float inv_copies, cudaStream_t s);

// ---- attention (exact family; scores in double like the CPU executor) --------
void AttnFwd(const float* q, const float* k, const float* v, float* o, float* probs,
             float* stats, size_t B, size_t S, size_t H, size_t d, const int32_t* starts,
             cudaStream_t s);  // probs != null: cached family; stats != null: tiled family
void AttnDP(const float* dout, const float* v, float* dp, size_t B, size_t S, size_t H, size_t d,
            cudaStream_t s);
void AttnDV(const float* probs, const float* dout, float* dv, size_t B, size_t S, size_t H,
            size_t d, cudaStream_t s);
void SoftmaxRowsBwd(const float* probs, const float* dp, float* ds, size_t rows, size_t cols,
                    cudaStream_t s);
void AttnDQ(const float* ds, const float* k, float* dq, size_t B, size_t S, size_t H, size_t d,
            cudaStream_t s);
void AttnDK(const float* ds, const float* q, float* dk, size_t B, size_t S, size_t H, size_t d,
            cudaStream_t s);
void AttnDQTiled(const float* q, const float* k, const float* v, const float* dout, float* stats,
                 float* dq, size_t B, size_t S, size_t H, size_t d, cudaStream_t s);
void AttnDKVTiled(bool want_dk, const float* q, const float* k, const float* v, const float* dout,
                  const float* stats, float* out, size_t B, size_t S, size_t H, size_t d,
                  cudaStream_t s);

// ---- evaluation / merge tails (integer tallies, exact) -------------------------
// tally[0] += rows with label >= 0, tally[1] += those whose argmax == label.
void ArgmaxTally(const float* probs, const int32_t* labels, size_t N, size_t C,
                 unsigned long long* tally, cudaStream_t s);
// tally[2] += count of non-finite elements.
void CountNonFinite(const float* x, size_t n, unsigned long long* tally, cudaStream_t s);
// The real-row loss of the batch just evaluated: out[0] = the sum over the first
// real_rows rows of each row's loss (-log max(p[label], 1e-12), NaN kept; rows
// with label < 0 skipped), added in row order in double; tally[3] = the rows it
// is over.  `terms` holds real_rows doubles.  The MSE form sums the squared
// differences of real_rows * width elements in element order and divides by width.
void XentRealRowLoss(const float* probs, const int32_t* labels, size_t real_rows, size_t width,
                     double* terms, double* out, unsigned long long* tally, cudaStream_t s);
void MseRealRowLoss(const float* pred, const float* target, size_t real_rows, size_t width, double* terms,
                    double* out, unsigned long long* tally, cudaStream_t s);
// Symmetric per-column int8 quantisation of W [K, N] with the compiler's own
// arithmetic: levels [K, N] int8 and scales [N] f32, bit for bit.
// `maxbits_scratch` holds N 32-bit words.
void QuantizeColumns(const float* w, size_t K, size_t N, int8_t* levels, float* scales,
                     unsigned int* maxbits_scratch, cudaStream_t s);

// ---- low-rank (adapter) term folded into a tensor-core GEMM --------------------
// The f32 factors of s * T * B are cut into three bf16 pieces each and laid out
// as extra K columns of the base product (k_lora.cu).  LoraSplitColumns(r) is the
// width of both operands: 6 r rounded up to a multiple of 64.
uint32_t LoraSplitColumns(uint32_t r);
// out [M, LoraSplitColumns(r)] bf16 from t [M, r] f32, r in {4, 8, 12, 16}.
// False (nothing launched) for another rank or a misaligned pointer.
bool LoraSplitRows(const float* t, uint16_t* out, size_t M, uint32_t r, cudaStream_t s);
struct LoraWeight {
  const float* src;         // the adapter matrix: B [r, n_out], or A [n_out, r] when by_column
  uint16_t* dst;            // [n_out, kx] bf16
  const float* col_scale;   // the base product's per-column epilogue scale, or null
  float tile_alpha;         // ... or its scalar scale
  float alpha;              // the low-rank term's own factor
  uint32_t n_out, r, kx;
  uint32_t by_column;
};
// Every entry of a device-resident table in one launch.
void LoraSplitWeights(const LoraWeight* table, int count, uint32_t max_n_out, cudaStream_t s);

// ---- the activation-streaming adapter products on the tensor cores (k_lora_mma.cu) -----
// t = alpha x A for x [M, K], A [K, r]; 3xTF32 (f32-class accuracy, not the CPU's
// bits).  With `pieces` ([M, LoraSplitColumns(r)] bf16) the same launch also writes
// what LoraSplitRows would make of t.  False (nothing launched) outside the shapes
// it is built for.
bool LoraDownSupported(size_t M, size_t K, size_t r);
bool LoraDown(const float* x, const float* A, float* out, size_t M, size_t K, size_t r, float alpha, cudaStream_t s,
              uint16_t* pieces = nullptr);
// The three backward products of one adapter site in one pass over dY and x:
// dT = alpha_dt dY B^T, dB = alpha_db t^T dY, dA = alpha_da x^T dT.  `partials`
// holds LoraBackwardPartialFloats(N, K, r) floats of scratch.
struct LoraBackwardArgs {
  const float* dy = nullptr;   // [M, N]
  const float* x = nullptr;    // [M, K]
  const float* t = nullptr;    // [M, r]
  const float* B = nullptr;    // [r, N]
  float* dt = nullptr;         // [M, r]
  float* dB = nullptr;         // [r, N]
  float* dA = nullptr;         // [K, r]
  float* partials = nullptr;
  size_t partials_floats = 0;
  size_t M = 0, N = 0, K = 0, r = 0;
  float alpha_dt = 1.0f, alpha_db = 1.0f, alpha_da = 1.0f;
  uint16_t* dt_pieces = nullptr;   // optional: what LoraSplitRows would make of dt ([M, LoraSplitColumns(r)] bf16)
};
bool LoraBackwardSupported(size_t M, size_t N, size_t K, size_t r);
size_t LoraBackwardPartialFloats(size_t N, size_t K, size_t r);
bool LoraBackward(const LoraBackwardArgs& args, cudaStream_t s);

// A whole f32 matrix as its bf16 pieces, dst [rows][6 * cols] (six K segments of
// `cols`): the operand layout that makes an f32 GEMM a bf16 tensor-core GEMM over
// K' = 6 K (k_lora.cu).  side 0: the A operand's piece order; 1: the B operand's.
// src is [rows][cols], or [cols][rows] when `transposed`.  cols % 4 == 0 and 16-byte
// aligned pointers for the untransposed form.
void SplitMatrix(const float* src, uint16_t* dst, size_t rows, size_t cols, bool transposed, int side,
                 cudaStream_t s);

// ---- GEMM -------------------------------------------------------------------
enum class BType : uint8_t { kF32 = 0, kI8 = 1, kBf16 = 2 };
constexpr int kFuseNone = 0, kFuseActFwd = 1, kFuseActBwd = 2;   // GemmArgs::fuse_mode
struct GemmArgs {
  const float* A = nullptr;    // [M,K], or [K,M] when a_transposed
  const void* B = nullptr;     // [K,N], or [N,K] when b_transposed
  float* C = nullptr;          // [M,N]
  size_t M = 0, N = 0, K = 0;
  bool a_transposed = false, b_transposed = false;
  BType b_type = BType::kF32;
  float alpha = 1.0f;               // NN/TN: folded into A; NT: applied to the dot
  const float* b_col_scale = nullptr;  // NN q8: scale per output column n (joins B's widening)
  const float* a_k_scale = nullptr;    // NT q8: scale per reduction index k (joins A)
  const float* bias = nullptr;
  const float* addend = nullptr;
  Act act = kActNone;
  bool accumulate = false;  // C += (the merge program's form)
  // Tensor-core path only: a following activation instruction done in the
  // epilogue (see UmmaEpilogue); its result leaves as the bf16 operand copy
  // fuse_shadow of the product that consumes it.
  int fuse_mode = 0;
  Act fuse_act = kActNone;
  const float* fuse_x = nullptr;
  uint16_t* fuse_shadow = nullptr;
  const float* fuse_shadow_scale = nullptr;
  // Tensor-core path only: the result (what goes to C) also leaves as bf16 in the same
  // [M, N] layout: the operand copy a tiled attention instruction reads it through, which
  // saves that instruction's conversion pass.
  uint16_t* pack_dst = nullptr;
  bool store_c = true;
  bool addend_after_bias = false;   // tensor-core path: v = addend + (product + bias)
  // Tensor-core path only: a low-rank term appended to the reduction (see
  // UmmaEpilogue::aux_k_blocks): aux_a [M, aux_k] and aux_b [N, aux_k], bf16.
  const uint16_t* aux_a = nullptr;
  const uint16_t* aux_b = nullptr;
  uint32_t aux_k = 0;
  // Exact path, rank-r expand kernel only: a following kAddEW rides along
  // (tail_out = tail_addend + result; C is not written).  GemmExact returns whether
  // it did.
  const float* tail_addend = nullptr;
  float* tail_out = nullptr;
  // Exact path: the shape-specialised rank-r kernels may contract multiply-adds
  // (same reduction order, one rounding per term instead of two).  Set by the
  // engine; never through the strict seam.
  bool contract_fma = false;
  // Scratch for the split-K form of the transposed-A product (optional).
  float* split_scratch = nullptr;
  size_t split_scratch_floats = 0;
};
// The transposed-A product is cut along K when it has fewer output tiles than
// SMs and K is long: chunks of SplitKChunkRows rows (256, halved down to 32
// while the partial-sum grid would hold fewer than 296 blocks), a pure function
// of the shape, so a shape always reduces in the same order.  SplitKChunks is
// the chunk count; 1 means "not split".
constexpr size_t kSplitKChunk = 256;   // the largest chunk
size_t SplitKChunkRows(size_t M, size_t N, size_t K);
size_t SplitKChunks(size_t M, size_t N, size_t K);
// The reference's reduction orders on CUDA cores, without fused multiply-adds:
// bit-identical to the CPU executor for f32 / int8 / bf16 weights.
bool GemmExact(const GemmArgs& a, cudaStream_t s);

}  // namespace see::k

#endif  // SEE_CUDA_KERNELS_H_
