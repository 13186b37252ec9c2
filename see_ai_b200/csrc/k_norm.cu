// LayerNorm / RMSNorm forward and backward.  HBM-bound row kernels: one warp
// per row; LayerNorm rows of 128..1024 floats (a multiple of 128) are held in
// registers and read once with 16-byte loads, other widths are streamed twice.  Row sums are taken in double like the reference
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
  const float row_mean = static_cast<float>(sum / static_cast<double>(cols));
  double var = 0.0;
  for (size_t c = lane; c < cols; c += 32) {
    const double d = static_cast<double>(xr[c]) - static_cast<double>(row_mean);
    var += d * d;
  }
  var = WarpSum(var);
  const float inv_sigma = 1.0f / sqrtf(static_cast<float>(var / static_cast<double>(cols)) + eps);
  if (lane == 0) {
    mean[r] = row_mean;
    rstd[r] = inv_sigma;
  }
  float* yr = y + r * cols;
  for (size_t c = lane; c < cols; c += 32) {
    const float v = (xr[c] - row_mean) * inv_sigma * gamma[c] + beta[c];
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
  const float per_col = 1.0f / static_cast<float>(cols);
  const float* dyr = dy + r * cols;
  const float* xr = x + r * cols;
  float* dxr = dx + r * cols;
  const float row_mean = mean[r], inv_sigma = rstd[r];
  double acc_g = 0.0, acc_gu = 0.0;
  for (size_t c = lane; c < cols; c += 32) {
    const float unit = (xr[c] - row_mean) * inv_sigma;
    const float g = dyr[c] * gamma[c];
    acc_g += static_cast<double>(g);
    acc_gu += static_cast<double>(g) * static_cast<double>(unit);
  }
  acc_g = WarpSum(acc_g);
  acc_gu = WarpSum(acc_gu);
  const float avg_g = static_cast<float>(acc_g) * per_col;
  const float avg_gu = static_cast<float>(acc_gu) * per_col;
  for (size_t c = lane; c < cols; c += 32) {
    const float unit = (xr[c] - row_mean) * inv_sigma;
    const float g = dyr[c] * gamma[c];
    dxr[c] = inv_sigma * (g - avg_g - unit * avg_gu);
  }
}

// Rows of 128 * V floats (V <= 8) held in registers: each lane owns V float4
// chunks (chunk index lane + 32 i), so the row is read from memory once, with
// 16-byte accesses.  Same expressions per element as the scalar kernels; the
// double sums run over a lane's chunks in ascending order, then the shuffle tree.
template <int V>
__global__ void __launch_bounds__(kWarpsPerBlock * 32, 4)
LayerNormFwdVecKernel(const float* __restrict__ x, const float* __restrict__ gamma,
                      const float* __restrict__ beta, float* __restrict__ y,
                      float* __restrict__ mean, float* __restrict__ rstd, size_t rows, float eps,
                      Shadow sh) {
  constexpr size_t cols = 128 * V;
  const size_t r = blockIdx.x * static_cast<size_t>(kWarpsPerBlock) + threadIdx.x / 32;
  const int lane = threadIdx.x & 31;
  if (r >= rows) return;
  const float4* xr = reinterpret_cast<const float4*>(x + r * cols);
  float4 xv[V];
  double sum = 0.0;
#pragma unroll
  for (int i = 0; i < V; ++i) {
    xv[i] = xr[lane + 32 * i];
    sum += static_cast<double>(xv[i].x);
    sum += static_cast<double>(xv[i].y);
    sum += static_cast<double>(xv[i].z);
    sum += static_cast<double>(xv[i].w);
  }
  sum = WarpSum(sum);
  const float row_mean = static_cast<float>(sum / static_cast<double>(cols));
  double var = 0.0;
#pragma unroll
  for (int i = 0; i < V; ++i) {
    const float e[4] = {xv[i].x, xv[i].y, xv[i].z, xv[i].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const double d = static_cast<double>(e[j]) - static_cast<double>(row_mean);
      var += d * d;
    }
  }
  var = WarpSum(var);
  const float inv_sigma = 1.0f / sqrtf(static_cast<float>(var / static_cast<double>(cols)) + eps);
  if (lane == 0) {
    mean[r] = row_mean;
    rstd[r] = inv_sigma;
  }
  float4* yr = reinterpret_cast<float4*>(y + r * cols);
#pragma unroll
  for (int i = 0; i < V; ++i) {
    const int c4 = lane + 32 * i;
    const float4 g = __ldg(reinterpret_cast<const float4*>(gamma) + c4);
    const float4 b = __ldg(reinterpret_cast<const float4*>(beta) + c4);
    float4 v;
    v.x = (xv[i].x - row_mean) * inv_sigma * g.x + b.x;
    v.y = (xv[i].y - row_mean) * inv_sigma * g.y + b.y;
    v.z = (xv[i].z - row_mean) * inv_sigma * g.z + b.z;
    v.w = (xv[i].w - row_mean) * inv_sigma * g.w + b.w;
    yr[c4] = v;
    if (sh.dst) ShadowStore4(sh, r * (cols / 4) + c4, static_cast<uint32_t>(c4 * 4), v);
  }
}

template <int V>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
LayerNormBwdVecKernel(const float* __restrict__ dy, const float* __restrict__ x,
                      const float* __restrict__ gamma, const float* __restrict__ mean,
                      const float* __restrict__ rstd, float* dx, size_t rows, const float* addend, Shadow sh) {
  constexpr size_t cols = 128 * V;
  const size_t r = blockIdx.x * static_cast<size_t>(kWarpsPerBlock) + threadIdx.x / 32;
  const int lane = threadIdx.x & 31;
  if (r >= rows) return;
  const float per_col = 1.0f / static_cast<float>(cols);
  const float4* dyr = reinterpret_cast<const float4*>(dy + r * cols);
  const float4* xr = reinterpret_cast<const float4*>(x + r * cols);
  const float row_mean = mean[r], inv_sigma = rstd[r];
  float unit[V][4], g[V][4];
  double acc_g = 0.0, acc_gu = 0.0;
#pragma unroll
  for (int i = 0; i < V; ++i) {
    const int c4 = lane + 32 * i;
    const float4 xv = xr[c4], dv = dyr[c4];
    const float4 gm = __ldg(reinterpret_cast<const float4*>(gamma) + c4);
    const float xe[4] = {xv.x, xv.y, xv.z, xv.w}, de[4] = {dv.x, dv.y, dv.z, dv.w},
                ge[4] = {gm.x, gm.y, gm.z, gm.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      unit[i][j] = (xe[j] - row_mean) * inv_sigma;
      g[i][j] = de[j] * ge[j];
      acc_g += static_cast<double>(g[i][j]);
      acc_gu += static_cast<double>(g[i][j]) * static_cast<double>(unit[i][j]);
    }
  }
  acc_g = WarpSum(acc_g);
  acc_gu = WarpSum(acc_gu);
  const float avg_g = static_cast<float>(acc_g) * per_col;
  const float avg_gu = static_cast<float>(acc_gu) * per_col;
  float4* dxr = reinterpret_cast<float4*>(dx + r * cols);
  const float4* adr = addend ? reinterpret_cast<const float4*>(addend + r * cols) : nullptr;
#pragma unroll
  for (int i = 0; i < V; ++i) {
    float4 v = make_float4(inv_sigma * (g[i][0] - avg_g - unit[i][0] * avg_gu), inv_sigma * (g[i][1] - avg_g - unit[i][1] * avg_gu),
                           inv_sigma * (g[i][2] - avg_g - unit[i][2] * avg_gu), inv_sigma * (g[i][3] - avg_g - unit[i][3] * avg_gu));
    if (adr) {   // an absorbed kAddEW: the sum it would have written (dx may alias the addend)
      const float4 a = adr[lane + 32 * i];
      v = make_float4(a.x + v.x, a.y + v.y, a.z + v.z, a.w + v.w);
    }
    dxr[lane + 32 * i] = v;
    if (sh.dst) ShadowStore4(sh, r * (cols / 4) + lane + 32 * i, static_cast<uint32_t>((lane + 32 * i) * 4), v);
  }
}

inline bool Vec16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

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
  const float inv_sigma = 1.0f / sqrtf(static_cast<float>(ss / static_cast<double>(cols)) + eps);
  if (lane == 0) rstd[r] = inv_sigma;
  float* yr = y + r * cols;
  for (size_t c = lane; c < cols; c += 32) yr[c] = xr[c] * inv_sigma * gamma[c];
}

__global__ void RmsNormBwdKernel(const float* __restrict__ dy, const float* __restrict__ x,
                                 const float* __restrict__ gamma, const float* __restrict__ rstd,
                                 float* __restrict__ dx, size_t rows, size_t cols) {
  const size_t r = blockIdx.x * static_cast<size_t>(kWarpsPerBlock) + threadIdx.x / 32;
  const int lane = threadIdx.x & 31;
  if (r >= rows) return;
  const float per_col = 1.0f / static_cast<float>(cols);
  const float* dyr = dy + r * cols;
  const float* xr = x + r * cols;
  float* dxr = dx + r * cols;
  const float inv_sigma = rstd[r];
  double acc_gu = 0.0;
  for (size_t c = lane; c < cols; c += 32)
    acc_gu += static_cast<double>(dyr[c] * gamma[c]) * static_cast<double>(xr[c]);
  acc_gu = WarpSum(acc_gu);
  const float avg_gu = static_cast<float>(acc_gu) * per_col;
  for (size_t c = lane; c < cols; c += 32)
    dxr[c] = inv_sigma * (dyr[c] * gamma[c] - xr[c] * inv_sigma * inv_sigma * avg_gu);
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
  const Shadow sh = shadowed ? *shadow : Shadow{};
  if (cols % 128 == 0 && cols <= 1024 && Vec16(x) && Vec16(y) && Vec16(gamma) && Vec16(beta) &&
      (!shadowed || ShadowUsable(shadow, y, rows * cols))) {
    const unsigned blocks = RowBlocks(rows);
#define SEE_LN_FWD(V) \
    case V: LayerNormFwdVecKernel<V><<<blocks, kWarpsPerBlock * 32, 0, s>>>(x, gamma, beta, y, mean, rstd, rows, eps, sh); break
    switch (cols / 128) {
      SEE_LN_FWD(1); SEE_LN_FWD(2); SEE_LN_FWD(3); SEE_LN_FWD(4);
      SEE_LN_FWD(5); SEE_LN_FWD(6); SEE_LN_FWD(7); SEE_LN_FWD(8);
    }
#undef SEE_LN_FWD
    return shadowed;
  }
  LayerNormFwdKernel<<<RowBlocks(rows), kWarpsPerBlock * 32, 0, s>>>(x, gamma, beta, y, mean, rstd,
                                                                     rows, cols, eps, sh);
  return shadowed;
}
int LayerNormBwd(const float* dy, const float* x, const float* gamma, const float* mean,
                  const float* rstd, float* dx, size_t rows, size_t cols, cudaStream_t s,
                  const float* addend, float* sum_out, const Shadow* sum_shadow) {
  if (rows == 0) return 0;
  if (cols % 128 == 0 && cols <= 1024 && Vec16(dy) && Vec16(x) && Vec16(gamma) && Vec16(dx) && Vec16(addend) &&
      Vec16(sum_out)) {
    const unsigned blocks = RowBlocks(rows);
    const bool fused = addend != nullptr && sum_out != nullptr;
    if (fused) dx = sum_out;
    else addend = nullptr;
    const Shadow sh = fused && ShadowUsable(sum_shadow, sum_out, rows * cols) && sum_shadow->cols == cols
                          ? *sum_shadow : Shadow{};
#define SEE_LN_BWD(V) \
    case V: LayerNormBwdVecKernel<V><<<blocks, kWarpsPerBlock * 32, 0, s>>>(dy, x, gamma, mean, rstd, dx, rows, addend, sh); break
    switch (cols / 128) {
      SEE_LN_BWD(1); SEE_LN_BWD(2); SEE_LN_BWD(3); SEE_LN_BWD(4);
      SEE_LN_BWD(5); SEE_LN_BWD(6); SEE_LN_BWD(7); SEE_LN_BWD(8);
    }
#undef SEE_LN_BWD
    return fused ? (sh.dst ? 2 : 1) : 0;
  }
  LayerNormBwdKernel<<<RowBlocks(rows), kWarpsPerBlock * 32, 0, s>>>(dy, x, gamma, mean, rstd, dx,
                                                                     rows, cols);
  return 0;
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
