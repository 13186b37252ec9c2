// Optimizer steps and gradient clipping.  HBM-bound elementwise kernels; the
// AdamW update evaluates the reference's expression term by term without
// fused multiply-adds (-fmad=false), with the bias corrections and the
// learning rate computed on the host by the same libm calls the CPU executor
// makes, so p / m / v are bit-identical to the CPU's for an identical gradient
// (reference: runtime/executor/optimizer.cc:104-132).
//
// A clip's squared norm is a double sum over shape-derived chunks folded in
// chunk order (reference: runtime/executor/optimizer.cc:22-35).  A non-finite
// norm raises DeviceStatus::refused; every parameter-writing kernel checks the
// flag first and writes nothing, so a refused step leaves parameters and
// moments untouched and the host reports the refusal at its next flush.
//
// Data-parallel form: the gradient may be given as `g_copies` blocks (one per
// rank, gathered into local memory) that are summed in rank order and scaled
// by 1 / copies before the update — identical bits on every rank.
#include "kernels.h"

namespace see::k {

namespace {

constexpr size_t kMaxChunks = 256;
constexpr size_t kGrainCheap = 32768;

inline size_t ChunkGrain(size_t n, size_t grain) {
  const size_t cap = (n + kMaxChunks - 1) / kMaxChunks;
  return grain < cap ? cap : grain;
}

__device__ __forceinline__ double WarpSumD(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}

__global__ void SqPartialKernel(const float* __restrict__ g, size_t n, size_t grain,
                                double* __restrict__ partials) {
  __shared__ double smem[8];
  const size_t b = blockIdx.x * grain;
  const size_t e = b + grain < n ? b + grain : n;
  double sq = 0.0;
  for (size_t i = b + threadIdx.x; i < e; i += blockDim.x)
    sq += static_cast<double>(g[i]) * static_cast<double>(g[i]);
  sq = WarpSumD(sq);
  if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = sq;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < (blockDim.x >> 5); ++w) t += smem[w];
    partials[blockIdx.x] = t;
  }
}

__global__ void SqFoldKernel(const double* __restrict__ partials, size_t chunks,
                             double* __restrict__ sq) {
  double t = 0.0;
  for (size_t c = 0; c < chunks; ++c) t += partials[c];
  *sq = t;
}

// reference: runtime/executor/optimizer.cc:42-50 (ClipScale)
__global__ void ClipScaleKernel(const double* __restrict__ sq, float max_norm,
                                float* __restrict__ scale, DeviceStatus* status) {
  float s = 1.0f;
  if (max_norm > 0.0f) {
    const double norm = sqrt(*sq);
    if (!isfinite(norm)) {
      status->refused = 1;
    } else if (!(norm <= static_cast<double>(max_norm) || norm == 0.0)) {
      s = static_cast<float>(static_cast<double>(max_norm) / norm);
    }
  }
  *scale = s;
}

// reference: runtime/executor/optimizer.cc:70-85 (ClipGlobal's factor)
__global__ void ClipGlobalScaleKernel(const float* __restrict__ acc, float max_norm,
                                      float* __restrict__ scale, DeviceStatus* status) {
  float s = 1.0f;
  const double norm = sqrt(static_cast<double>(acc[0]));
  if (!isfinite(norm)) {
    status->refused = 1;
  } else if (!(norm <= static_cast<double>(max_norm) || norm == 0.0)) {
    s = static_cast<float>(static_cast<double>(max_norm) / norm);
  }
  *scale = s;
}

__global__ void SqNormAccumKernel(const double* __restrict__ sq, float* __restrict__ acc) {
  acc[0] = static_cast<float>(static_cast<double>(acc[0]) + *sq);
}

// g *= s only when s != 1 (the reference leaves g untouched below the threshold).
__global__ void ScaleInPlaceKernel(float* __restrict__ g, size_t n, const float* __restrict__ scale,
                                   const DeviceStatus* __restrict__ status) {
  if (status->refused) return;
  const float s = *scale;
  if (s == 1.0f) return;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += stride)
    g[i] *= s;
}

__device__ __forceinline__ float GatherGrad(const float* __restrict__ g, size_t i, int copies,
                                            size_t stride, float inv_copies) {
  if (copies <= 1) return g[i];
  float sum = g[i];
  for (int r = 1; r < copies; ++r) sum += g[i + static_cast<size_t>(r) * stride];
  return sum * inv_copies;
}

__global__ void AdamWKernel(float* __restrict__ p, const float* __restrict__ g,
                            float* __restrict__ m, float* __restrict__ v, size_t n,
                            const AdamScalars* __restrict__ scalars,
                            const float* __restrict__ clip_scale,
                            const DeviceStatus* __restrict__ status, int copies, size_t cstride,
                            float inv_copies) {
  if (status->refused) return;
  const AdamScalars a = *scalars;
  const float s = clip_scale ? *clip_scale : 1.0f;
  const float om_b1 = 1.0f - a.beta1;
  const float om_b2 = 1.0f - a.beta2;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += stride) {
    const float gi = GatherGrad(g, i, copies, cstride, inv_copies) * s;
    const float mi = a.beta1 * m[i] + om_b1 * gi;
    const float vi = a.beta2 * v[i] + om_b2 * gi * gi;
    m[i] = mi;
    v[i] = vi;
    const float m_hat = mi * a.inv_bc1;
    const float v_hat = vi * a.inv_bc2;
    p[i] -= a.lr * (m_hat / (sqrtf(v_hat) + a.eps) + a.weight_decay * p[i]);
  }
}

// The same update for a table of tensors (one optimizer phase in one launch).
__global__ void AdamWMultiKernel(const AdamTensor* __restrict__ table,
                                 const AdamScalars* __restrict__ scalars,
                                 const DeviceStatus* __restrict__ status, float inv_copies) {
  if (status->refused) return;
  const AdamTensor t = table[blockIdx.y];
  const AdamScalars a = *scalars;
  const float om_b1 = 1.0f - a.beta1;
  const float om_b2 = 1.0f - a.beta2;
  const float inv = t.g_copies > 1 ? inv_copies : 1.0f;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < t.n; i += stride) {
    const float gi = GatherGrad(t.g, i, t.g_copies, t.copy_stride, inv) * 1.0f;
    const float mi = a.beta1 * t.m[i] + om_b1 * gi;
    const float vi = a.beta2 * t.v[i] + om_b2 * gi * gi;
    t.m[i] = mi;
    t.v[i] = vi;
    const float m_hat = mi * a.inv_bc1;
    const float v_hat = vi * a.inv_bc2;
    t.p[i] -= a.lr * (m_hat / (sqrtf(v_hat) + a.eps) + a.weight_decay * t.p[i]);
  }
}

// reference: runtime/executor/optimizer.cc:91-102
__global__ void SgdKernel(float* __restrict__ p, const float* __restrict__ g, size_t n,
                          const AdamScalars* __restrict__ scalars,
                          const float* __restrict__ clip_scale,
                          const DeviceStatus* __restrict__ status, int copies, size_t cstride,
                          float inv_copies) {
  if (status->refused) return;
  const float lr = scalars->lr, weight_decay = scalars->weight_decay;
  const float s = clip_scale ? *clip_scale : 1.0f;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += stride) {
    const float gi = GatherGrad(g, i, copies, cstride, inv_copies) * s;
    p[i] -= lr * (gi + weight_decay * p[i]);
  }
}

__global__ void SumCopiesKernel(const float* __restrict__ g, float* __restrict__ out, size_t n,
                                int copies, size_t cstride, float inv_copies) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += stride)
    out[i] = GatherGrad(g, i, copies, cstride, inv_copies);
}

inline unsigned GridFor(size_t n) {
  size_t b = (n + 255) / 256;
  if (b < 1) b = 1;
  if (b > 148 * 8) b = 148 * 8;
  return static_cast<unsigned>(b);
}

}  // namespace

void L2Squared(const float* g, size_t n, double* partials, double* sq, cudaStream_t s) {
  const size_t grain = ChunkGrain(n, kGrainCheap);
  const size_t chunks = n == 0 ? 0 : (n + grain - 1) / grain;
  if (chunks)
    SqPartialKernel<<<static_cast<unsigned>(chunks), 256, 0, s>>>(g, n, grain, partials);
  SqFoldKernel<<<1, 1, 0, s>>>(partials, chunks, sq);
}

void ClipScaleFromSq(const double* sq, float max_norm, float* scale, DeviceStatus* status,
                     cudaStream_t s) {
  ClipScaleKernel<<<1, 1, 0, s>>>(sq, max_norm, scale, status);
}

void ScaleInPlaceBy(float* g, size_t n, const float* scale, const DeviceStatus* status,
                    cudaStream_t s) {
  if (n == 0) return;
  ScaleInPlaceKernel<<<GridFor(n), 256, 0, s>>>(g, n, scale, status);
}

void SqNormAccum(const double* sq, float* acc, cudaStream_t s) {
  SqNormAccumKernel<<<1, 1, 0, s>>>(sq, acc);
}

void ClipGlobalScale(const float* acc, float max_norm, float* scale, DeviceStatus* status,
                     cudaStream_t s) {
  ClipGlobalScaleKernel<<<1, 1, 0, s>>>(acc, max_norm, scale, status);
}

void AdamWStep(float* p, const float* g, float* m, float* v, size_t n, const AdamScalars* a,
               const float* clip_scale, const DeviceStatus* status, int g_copies,
               size_t copy_stride, float inv_copies, cudaStream_t s) {
  if (n == 0) return;
  AdamWKernel<<<GridFor(n), 256, 0, s>>>(p, g, m, v, n, a, clip_scale, status, g_copies,
                                         copy_stride, inv_copies);
}

void AdamWStepMulti(const AdamTensor* table, int count, uint64_t max_n, const AdamScalars* a,
                    const DeviceStatus* status, float inv_copies, cudaStream_t s) {
  if (count <= 0 || max_n == 0) return;
  size_t bx = (max_n + 255) / 256;
  if (bx > 64) bx = 64;
  AdamWMultiKernel<<<dim3(static_cast<unsigned>(bx), static_cast<unsigned>(count)), 256, 0, s>>>(
      table, a, status, inv_copies);
}

void SgdStep(float* p, const float* g, size_t n, const AdamScalars* a,
             const float* clip_scale, const DeviceStatus* status, int g_copies,
             size_t copy_stride, float inv_copies, cudaStream_t s) {
  if (n == 0) return;
  SgdKernel<<<GridFor(n), 256, 0, s>>>(p, g, n, a, clip_scale, status, g_copies,
                                       copy_stride, inv_copies);
}

void SumCopies(const float* g, float* out, size_t n, int g_copies, size_t copy_stride,
               float inv_copies, cudaStream_t s) {
  if (n == 0) return;
  SumCopiesKernel<<<GridFor(n), 256, 0, s>>>(g, out, n, g_copies, copy_stride, inv_copies);
}

}  // namespace see::k
