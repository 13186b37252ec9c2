// Activation expressions shared by the elementwise kernels and the GEMM
// epilogue that can absorb a following activation instruction: one definition,
// so both produce the same bits (both files are compiled with -fmad=false).
// Reference: runtime/executor/kernel_policy.h:122-136,
// runtime/executor/activation.cc:22-75.
#ifndef SEE_CUDA_ACT_EXPR_CUH_
#define SEE_CUDA_ACT_EXPR_CUH_

#include "kernels.h"

namespace see::k {

constexpr float kGeluExprC = 0.7978845608028654f;
constexpr float kGeluExprA = 0.044715f;

__device__ __forceinline__ float SigmoidExpr(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float ReluExpr(float x) { return x > 0.0f ? x : 0.0f; }
__device__ __forceinline__ float GeluExpr(float x) {
  const float t = tanhf(kGeluExprC * (x + kGeluExprA * x * x * x));
  return 0.5f * x * (1.0f + t);
}
__device__ __forceinline__ float SiluExpr(float x) { return x * SigmoidExpr(x); }
__device__ __forceinline__ float ReluGrad(float dy, float x) { return x > 0.0f ? dy : 0.0f; }
__device__ __forceinline__ float GeluGrad(float dy, float v) {
  const float u = kGeluExprC * (v + kGeluExprA * v * v * v);
  const float t = tanhf(u);
  const float one_minus_t2 = 1.0f - t * t;
  const float tail = one_minus_t2 == 0.0f
                         ? 0.0f
                         : 0.5f * v * one_minus_t2 * (kGeluExprC * (1.0f + 3.0f * kGeluExprA * v * v));
  return dy * (0.5f * (1.0f + t) + tail);
}
__device__ __forceinline__ float SiluGrad(float dy, float x) {
  const float s = SigmoidExpr(x);
  return dy * (s * (1.0f + x * (1.0f - s)));
}

__device__ __forceinline__ float ActFwdExpr(int act, float x) {
  switch (act) {
    case kActRelu: return ReluExpr(x);
    case kActGelu: return GeluExpr(x);
    case kActSilu: return SiluExpr(x);
    default: return x;
  }
}
__device__ __forceinline__ float ActBwdExpr(int act, float dy, float x) {
  switch (act) {
    case kActRelu: return ReluGrad(dy, x);
    case kActGelu: return GeluGrad(dy, x);
    case kActSilu: return SiluGrad(dy, x);
    default: return dy;
  }
}

}  // namespace see::k

#endif  // SEE_CUDA_ACT_EXPR_CUH_
