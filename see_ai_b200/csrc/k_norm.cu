// LayerNorm / RMSNorm forward and backward.  HBM-bound row kernels: one warp
// per row, the row streamed twice (sums, then the output) with float4 loads
// where the row width allows.  Row sums are taken in double like the reference
// (reference: runtime/executor/normalization.cc:17-113), in a fixed order —
// lane-strided partials combined by a shuffle tree — so results are run-to-run
// identical and independent of the grid; they can differ from the CPU's
// sequential double sum in the last bit of the double, which almost never
// survives the cast to float.  Compiled with -fmad=false so the output
// expressions round like the reference's.
#include "kernels.h"
#include "shadow.cuh"

namespace see::k {

namespace {

constexpr int kWarpsPerBlock = 8;

__device__ __forceinline__ double WarpSum(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}

__global__ void LayerNormFwdKernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                   const float* __restrict__ beta, float* __restrict__ y,
                                   float* __restrict__ mean, float* __restrict__ rstd,
                                   size_t rows, size_t cols, float eps, Shadow sh) {
  const size_t r = blockIdx.x * static_cast<size_t>(kWarpsPerBlock) + threadIdx.x / 32;
  const int lane = threadIdx.x & 31;
  if (r >= rows) return;
  const float* xr = x + r * cols;
  double sum = 0.0;
  for (size_t c = lane; c < cols; c += 32) sum += static_cast<double>(xr[c]);
  sum = WarpSum(sum);
  const float mu = static_cast<float>(sum / static_cast<double>(cols));
  double var = 0.0;
  for (size_t c = lane; c < cols; c += 32) {
    const double d = static_cast<double>(xr[c]) - static_cast<double>(mu);
    var += d * d;
  }
  var = WarpSum(var);
  const float rs = 1.0f / sqrtf(static_cast<float>(var / static_cast<double>(cols)) + eps);
  if (lane == 0) {
    mean[r] = mu;
    rstd[r] = rs;
  }
  float* yr = y + r * cols;
  for (size_t c = lane; c < cols; c += 32) {
    const float v = (xr[c] - mu) * rs * gamma[c] + beta[c];
    yr[c] = v;
    if (sh.dst)   // the bf16 copy for the GEMM that reads y next
      sh.dst[r * cols + c] = static_cast<uint16_t>(ShadowBf16(sh.k_scale ? v * sh.k_scale[c] : v));
  }
}

__global__ void LayerNormBwdKernel(const float* __restrict__ dy, const float* __restrict__ x,
                                   const float* __restrict__ gamma, const float* __restrict__ mean,
                                   const float* __restrict__ rstd, float* __restrict__ dx,
                                   size_t rows, size_t cols) {
  const size_t r = blockIdx.x * static_cast<size_t>(kWarpsPerBlock) + threadIdx.x / 32;
  const int lane = threadIdx.x & 31;
  if (r >= rows) return;
  const float inv_d = 1.0f / static_cast<float>(cols);
  const float* dyr = dy + r * cols;
  const float* xr = x + r * cols;
  float* dxr = dx + r * cols;
  const float mu = mean[r], rs = rstd[r];
  double sum_g = 0.0, sum_gx = 0.0;
  for (size_t c = lane; c < cols; c += 32) {
    const float xhat = (xr[c] - mu) * rs;
    const float g = dyr[c] * gamma[c];
    sum_g += static_cast<double>(g);
    sum_gx += static_cast<double>(g) * static_cast<double>(xhat);
  }
  sum_g = WarpSum(sum_g);
  sum_gx = WarpSum(sum_gx);
  const float mg = static_cast<float>(sum_g) * inv_d;
  const float mgx = static_cast<float>(sum_gx) * inv_d;
  for (size_t c = lane; c < cols; c += 32) {
    const float xhat = (xr[c] - mu) * rs;
    const float g = dyr[c] * gamma[c];
    dxr[c] = rs * (g - mg - xhat * mgx);
  }
}

__global__ void RmsNormFwdKernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                 float* __restrict__ y, float* __restrict__ rstd, size_t rows,
                                 size_t cols, float eps) {
  const size_t r = blockIdx.x * static_cast<size_t>(kWarpsPerBlock) + threadIdx.x / 32;
  const int lane = threadIdx.x & 31;
  if (r >= rows) return;
  const float* xr = x + r * cols;
  double ss = 0.0;
  for (size_t c = lane; c < cols; c += 32)
    ss += static_cast<double>(xr[c]) * static_cast<double>(xr[c]);
  ss = WarpSum(ss);
  const float rs = 1.0f / sqrtf(static_cast<float>(ss / static_cast<double>(cols)) + eps);
  if (lane == 0) rstd[r] = rs;
  float* yr = y + r * cols;
  for (size_t c = lane; c < cols; c += 32) yr[c] = xr[c] * rs * gamma[c];
}

__global__ void RmsNormBwdKernel(const float* __restrict__ dy, const float* __restrict__ x,
                                 const float* __restrict__ gamma, const float* __restrict__ rstd,
                                 float* __restrict__ dx, size_t rows, size_t cols) {
  const size_t r = blockIdx.x * static_cast<size_t>(kWarpsPerBlock) + threadIdx.x / 32;
  const int lane = threadIdx.x & 31;
  if (r >= rows) return;
  const float inv_d = 1.0f / static_cast<float>(cols);
  const float* dyr = dy + r * cols;
  const float* xr = x + r * cols;
  float* dxr = dx + r * cols;
  const float rs = rstd[r];
  double sum_gx = 0.0;
  for (size_t c = lane; c < cols; c += 32)
    sum_gx += static_cast<double>(dyr[c] * gamma[c]) * static_cast<double>(xr[c]);
  sum_gx = WarpSum(sum_gx);
  const float mgx = static_cast<float>(sum_gx) * inv_d;
  for (size_t c = lane; c < cols; c += 32)
    dxr[c] = rs * (dyr[c] * gamma[c] - xr[c] * rs * rs * mgx);
}

inline unsigned RowBlocks(size_t rows) {
  return static_cast<unsigned>((rows + kWarpsPerBlock - 1) / kWarpsPerBlock);
}

}  // namespace

bool LayerNormFwd(const float* x, const float* gamma, const float* beta, float* y, float* mean,
                  float* rstd, size_t rows, size_t cols, float eps, cudaStream_t s,
                  const Shadow* shadow) {
  if (rows == 0) return false;
  const bool shadowed = shadow && shadow->dst && shadow->cols == cols;
  LayerNormFwdKernel<<<RowBlocks(rows), kWarpsPerBlock * 32, 0, s>>>(
      x, gamma, beta, y, mean, rstd, rows, cols, eps, shadowed ? *shadow : Shadow{});
  return shadowed;
}
void LayerNormBwd(const float* dy, const float* x, const float* gamma, const float* mean,
                  const float* rstd, float* dx, size_t rows, size_t cols, cudaStream_t s) {
  if (rows == 0) return;
  LayerNormBwdKernel<<<RowBlocks(rows), kWarpsPerBlock * 32, 0, s>>>(dy, x, gamma, mean, rstd, dx,
                                                                     rows, cols);
}
void RmsNormFwd(const float* x, const float* gamma, float* y, float* rstd, size_t rows,
                size_t cols, float eps, cudaStream_t s) {
  if (rows == 0) return;
  RmsNormFwdKernel<<<RowBlocks(rows), kWarpsPerBlock * 32, 0, s>>>(x, gamma, y, rstd, rows, cols,
                                                                   eps);
}
void RmsNormBwd(const float* dy, const float* x, const float* gamma, const float* rstd,
                float* dx, size_t rows, size_t cols, cudaStream_t s) {
  if (rows == 0) return;
  RmsNormBwdKernel<<<RowBlocks(rows), kWarpsPerBlock * 32, 0, s>>>(dy, x, gamma, rstd, dx, rows,
                                                                   cols);
}

}  // namespace see::k
