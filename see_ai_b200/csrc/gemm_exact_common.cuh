// Pieces shared by the exact (CUDA-core) GEMM kernels: the parameter block, the
// activation expressions as the CPU executor writes them (reference:
// runtime/executor/gemm.cc:536-578) and the narrow-weight widenings.  Every
// file that includes this is compiled with -fmad=false.
#ifndef SEE_CUDA_GEMM_EXACT_COMMON_CUH_
#define SEE_CUDA_GEMM_EXACT_COMMON_CUH_

#include "kernels.h"

namespace see::k::exact {

constexpr float kGeluC = 0.7978845608028654f;
constexpr float kGeluA = 0.044715f;

__device__ __forceinline__ float ApplyAct(float v, Act act) {
  switch (act) {
    case kActRelu: return v > 0.0f ? v : 0.0f;
    case kActGelu: {
      const float t = tanhf(kGeluC * (v + kGeluA * v * v * v));
      return 0.5f * v * (1.0f + t);
    }
    case kActSilu: return v * (1.0f / (1.0f + expf(-v)));
    default: return v;
  }
}

template <typename T> __device__ __forceinline__ float Widen(T v);
template <> __device__ __forceinline__ float Widen<float>(float v) { return v; }
template <> __device__ __forceinline__ float Widen<int8_t>(int8_t v) { return static_cast<float>(v); }
template <> __device__ __forceinline__ float Widen<uint16_t>(uint16_t v) {
  return __uint_as_float(static_cast<uint32_t>(v) << 16);
}

struct Params {
  const float* A;
  const void* B;
  float* C;
  size_t M, N, K;
  float alpha;
  const float* b_col_scale;
  const float* a_k_scale;
  const float* bias;
  const float* addend;
  Act act;
  bool accumulate;
  // Split-K (long reductions into small outputs): block z reduces k in
  // [z * k_chunk, (z + 1) * k_chunk) with the quad order inside the chunk and
  // writes its raw sums to partials[z][M][N]; a second kernel folds the chunks
  // in chunk order.  k_chunk is a multiple of 16, so quads stay aligned to k = 0.
  size_t k_chunk;
  float* partials;
  // A following kAddEW done by the expand kernel: tail_out = tail_addend + (what C
  // would have received); C itself is then not written.
  const float* tail_addend = nullptr;
  float* tail_out = nullptr;
};

inline bool Aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Shape-specialised kernels for the rank-r adapter products.  Each returns
// false (and launches nothing) when the shape or layout is not one it covers;
// the caller then uses the general tile kernels.  Same arithmetic per element
// as the general kernels, so the choice never changes a bit of the result.
//   Reduce : C[M, N] with N in {4, 8, 16} over a long K (t = x*A, dT = dY*B^T).
//   Expand : C[M, N] with K in {4, 8, 12, 16} (y += t*B, dX += dT*A^T).
//   TnPartials : the per-chunk partial sums of a transposed-A product whose
//     output is at most 16 wide or 16 tall (dA = x^T*dT, dB = t^T*dY);
//     p.k_chunk and p.partials are set, the caller folds.
bool SkinnyReduce(const Params& p, bool lane_order, cudaStream_t s);
bool SkinnyExpand(const Params& p, bool lane_order, cudaStream_t s);
bool SkinnyTnPartials(const Params& p, size_t chunks, cudaStream_t s);

}  // namespace see::k::exact

// The same three with multiply-adds contracted (see k_gemm_skinny.cu).
namespace see::k::fast {
bool SkinnyReduce(const exact::Params& p, bool lane_order, cudaStream_t s);
bool SkinnyExpand(const exact::Params& p, bool lane_order, cudaStream_t s);
bool SkinnyTnPartials(const exact::Params& p, size_t chunks, cudaStream_t s);
}  // namespace see::k::fast

#endif  // SEE_CUDA_GEMM_EXACT_COMMON_CUH_
