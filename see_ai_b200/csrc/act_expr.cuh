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

// GELU (tanh form) through the hardware exponential and reciprocal.  With
// u = c (x + a x^3) and r = 1 / (1 + e^{2u}):  tanh u = 1 - 2r, so
// 0.5 x (1 + tanh u) = x - x r.  Absolute error a few 1e-7 of |x| (the reference
// differ's bound for these rows is 1e-5 of the tensor's magnitude); saturates
// exactly, keeps NaN.  About a dozen instructions, explicit FMAs (these rows are
// tolerance class, not bit-exact class): what lets a GEMM epilogue absorb the
// activation without becoming the kernel's critical path.
__device__ __forceinline__ float Ex2Approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float RcpApprox(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
constexpr float kTwoLog2E = 2.885390081777927f;   // e^{2u} = 2^{u * 2 log2 e}

__device__ __forceinline__ float SigmoidExpr(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float ReluExpr(float x) { return x > 0.0f ? x : 0.0f; }
__device__ __forceinline__ float GeluExpr(float x) {
  const float u = x * __fmaf_rn(x * x, kGeluExprC * kGeluExprA, kGeluExprC);
  const float r = RcpApprox(1.0f + Ex2Approx(u * kTwoLog2E));
  return __fmaf_rn(-x, r, x);
}
__device__ __forceinline__ float SiluExpr(float x) { return x * SigmoidExpr(x); }
__device__ __forceinline__ float ReluGrad(float dy, float x) { return x > 0.0f ? dy : 0.0f; }
__device__ __forceinline__ float GeluGrad(float dy, float v) {
  const float v2 = v * v;
  const float u = v * __fmaf_rn(v2, kGeluExprC * kGeluExprA, kGeluExprC);
  const float r = RcpApprox(1.0f + Ex2Approx(u * kTwoLog2E));
  const float t = __fmaf_rn(-2.0f, r, 1.0f);             // tanh u
  const float one_minus_t2 = __fmaf_rn(-t, t, 1.0f);
  const float du = __fmaf_rn(v2, 3.0f * kGeluExprC * kGeluExprA, kGeluExprC);
  // Saturated: the reference drops the tail rather than multiply 0 by a huge du.
  const float tail = one_minus_t2 == 0.0f ? 0.0f : (0.5f * v) * one_minus_t2 * du;
  return dy * (__fmaf_rn(0.5f, t, 0.5f) + tail);
}
__device__ __forceinline__ float SiluGrad(float dy, float x) {
  const float s = SigmoidExpr(x);
  return dy * (s * (1.0f + x * (1.0f - s)));
}

// ---- the same GELU expressions on two elements at once ---------------------------------
// Packed FP32 instructions (`fma/mul/add.rn.f32x2`) round each half exactly as
// their scalar forms do, so a pair computed here has the bits GeluExpr /
// GeluGrad give each element: the operation sequence below is theirs, one
// packed instruction per two scalar ones (the exponential and the reciprocal
// stay per element).  For the GEMM epilogue, where instruction count is the
// limit.
using f32x2 = unsigned long long;
__device__ __forceinline__ f32x2 PackF2(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void UnpackF2(f32x2 v, float* lo, float* hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(*lo), "=f"(*hi) : "l"(v));
}
__device__ __forceinline__ f32x2 Mul2(f32x2 a, f32x2 b) {
  f32x2 r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ f32x2 AddF2(f32x2 a, f32x2 b) {
  f32x2 r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ f32x2 Fma2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ f32x2 Splat2(float v) { return PackF2(v, v); }

// r = 1 / (1 + e^{2u}) for both halves, u = v (c + c a v^2); also returns v^2.
__device__ __forceinline__ f32x2 GeluRcp2(f32x2 v, f32x2* v2_out) {
  const f32x2 v2 = Mul2(v, v);
  const f32x2 u = Mul2(v, Fma2(v2, Splat2(kGeluExprC * kGeluExprA), Splat2(kGeluExprC)));
  float a0, a1;
  UnpackF2(Mul2(u, Splat2(kTwoLog2E)), &a0, &a1);
  float d0, d1;
  UnpackF2(AddF2(Splat2(1.0f), PackF2(Ex2Approx(a0), Ex2Approx(a1))), &d0, &d1);
  *v2_out = v2;
  return PackF2(RcpApprox(d0), RcpApprox(d1));
}
__device__ __forceinline__ f32x2 GeluExpr2(f32x2 x) {
  f32x2 x2;
  const f32x2 r = GeluRcp2(x, &x2);
  // fma(-x, r, x): the negation is exact, and rounding is sign-symmetric.
  return Fma2(Mul2(x, Splat2(-1.0f)), r, x);
}
__device__ __forceinline__ f32x2 GeluGrad2(f32x2 dy, f32x2 v) {
  f32x2 v2;
  const f32x2 r = GeluRcp2(v, &v2);
  const f32x2 t = Fma2(Splat2(-2.0f), r, Splat2(1.0f));    // tanh u
  const f32x2 nt = Fma2(Splat2(2.0f), r, Splat2(-1.0f));   // -tanh u, the same bits negated
  const f32x2 one_minus_t2 = Fma2(nt, t, Splat2(1.0f));
  const f32x2 du = Fma2(v2, Splat2(3.0f * kGeluExprC * kGeluExprA), Splat2(kGeluExprC));
  const f32x2 tail0 = Mul2(Mul2(Mul2(Splat2(0.5f), v), one_minus_t2), du);
  float s0, s1, t0, t1;
  UnpackF2(one_minus_t2, &s0, &s1);
  UnpackF2(tail0, &t0, &t1);
  const f32x2 tail = PackF2(s0 == 0.0f ? 0.0f : t0, s1 == 0.0f ? 0.0f : t1);
  return Mul2(dy, AddF2(Fma2(Splat2(0.5f), t, Splat2(0.5f)), tail));
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
