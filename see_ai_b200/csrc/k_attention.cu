// Causal attention, exact family: the cached opcodes (probabilities kept in
// the arena) and the tiled opcodes (four statistics per query row, every
// probability recomputed) evaluated with the CPU executor's own expressions —
// dot products accumulated in double in ascending feature order (a product of
// two floats is exact in double, so the fused and unfused forms coincide),
// the 1/sqrt(d) scale and the softmax in f32, output sums in f32 in ascending
// key (or query) order without fused multiply-adds (-fmad=false)
// (reference: runtime/executor/attention.cc:187-343 cached, :448-590 tiled).
// What is not sequential here are the two per-row double sums (softmax
// denominator, the backward's rowsum): lane partials folded by a shuffle
// tree, a fixed order that can differ from the CPU's in the last bit of the
// double.  One warp owns one (batch, head, row) unit; activations are
// [B*S, H*d] row-major with heads interleaved along the row.
#include "kernels.h"

namespace see::k {

namespace {

constexpr int kWarps = 4;

__device__ __forceinline__ double WarpSumD(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}
__device__ __forceinline__ float WarpMaxF(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
  return v;
}

// a (in shared memory) . row (global), accumulated in double, ascending c.
__device__ __forceinline__ double DotD(const float* a, const float* __restrict__ row, size_t d) {
  double acc = 0.0;
  for (size_t c = 0; c < d; ++c) acc += static_cast<double>(a[c]) * static_cast<double>(row[c]);
  return acc;
}

__device__ __forceinline__ size_t StatsStart(float stored, size_t i) {
  if (!(stored > 0.0f)) return 0;
  const float cap = static_cast<float>(i);
  return stored >= cap ? i : static_cast<size_t>(stored);
}

struct Unit { size_t b, h, i; };
__device__ __forceinline__ Unit UnitOf(size_t u, size_t H, size_t S) {
  return {u / (H * S), (u / S) % H, u % S};
}

// Shared memory per warp: d floats (the unit's query-side row) then `rows`
// rows of S floats.
__device__ __forceinline__ float* WarpSmem(float* base, size_t d, size_t S, int rows) {
  return base + (threadIdx.x >> 5) * (d + static_cast<size_t>(rows) * S);
}

__global__ void AttnFwdKernel(const float* __restrict__ q, const float* __restrict__ k,
                              const float* __restrict__ v, float* __restrict__ o,
                              float* __restrict__ probs, float* __restrict__ stats, size_t B,
                              size_t S, size_t H, size_t d, const int32_t* __restrict__ starts,
                              float inv_sqrt_d) {
  extern __shared__ float smem[];
  float* qs = WarpSmem(smem, d, S, 1);
  float* prow = qs + d;
  const int lane = threadIdx.x & 31;
  const size_t D = H * d, units = B * H * S;
  for (size_t u = blockIdx.x * static_cast<size_t>(kWarps) + (threadIdx.x >> 5); u < units;
       u += static_cast<size_t>(gridDim.x) * kWarps) {
    const Unit un = UnitOf(u, H, S);
    const size_t b = un.b, h = un.h, i = un.i;
    const float* qi = q + (b * S + i) * D + h * d;
    for (size_t c = lane; c < d; c += 32) qs[c] = qi[c];
    __syncwarp();
    size_t j0 = 0;
    if (starts) {
      const int32_t s0 = starts[b * S + i];
      j0 = s0 <= 0 ? 0 : (static_cast<size_t>(s0) < i ? static_cast<size_t>(s0) : i);
    }
    const float* kb = k + b * S * D + h * d;
    float row_max = -INFINITY;
    for (size_t j = j0 + lane; j <= i; j += 32) {
      const float sc = static_cast<float>(DotD(qs, kb + j * D, d)) * inv_sqrt_d;
      prow[j] = sc;
      row_max = fmaxf(row_max, sc);
    }
    row_max = WarpMaxF(row_max);
    double denom = 0.0;
    for (size_t j = j0 + lane; j <= i; j += 32) {
      const float e = expf(prow[j] - row_max);
      prow[j] = e;
      denom += static_cast<double>(e);
    }
    denom = WarpSumD(denom);
    const float inv_denom = 1.0f / static_cast<float>(denom);
    for (size_t j = j0 + lane; j <= i; j += 32) prow[j] *= inv_denom;
    __syncwarp();
    if (probs) {
      float* grow = probs + u * S;
      for (size_t j = lane; j < S; j += 32) grow[j] = (j >= j0 && j <= i) ? prow[j] : 0.0f;
    }
    const float* vb = v + b * S * D + h * d;
    float* oi = o + (b * S + i) * D + h * d;
    for (size_t c = lane; c < d; c += 32) {
      float acc = 0.0f;
      for (size_t j = j0; j <= i; ++j) acc += prow[j] * vb[j * D + c];
      oi[c] = acc;
    }
    if (stats && lane == 0) {
      float* st = stats + u * kAttnStatsWidth;
      st[0] = row_max;
      st[1] = inv_denom;
      st[2] = 0.0f;
      st[3] = static_cast<float>(j0);
    }
    __syncwarp();
  }
}

// dP[u, j] = dO_i . v_j for j <= i, zero above the diagonal.
__global__ void AttnDPKernel(const float* __restrict__ dout, const float* __restrict__ v,
                             float* __restrict__ dp, size_t B, size_t S, size_t H, size_t d) {
  extern __shared__ float smem[];
  float* as = WarpSmem(smem, d, S, 0);
  const int lane = threadIdx.x & 31;
  const size_t D = H * d, units = B * H * S;
  for (size_t u = blockIdx.x * static_cast<size_t>(kWarps) + (threadIdx.x >> 5); u < units;
       u += static_cast<size_t>(gridDim.x) * kWarps) {
    const Unit un = UnitOf(u, H, S);
    const float* doi = dout + (un.b * S + un.i) * D + un.h * d;
    for (size_t c = lane; c < d; c += 32) as[c] = doi[c];
    __syncwarp();
    const float* vb = v + un.b * S * D + un.h * d;
    float* row = dp + u * S;
    for (size_t j = lane; j < S; j += 32)
      row[j] = j <= un.i ? static_cast<float>(DotD(as, vb + j * D, d)) : 0.0f;
    __syncwarp();
  }
}

// out_j[c] = sum over i >= j of w[(bh*S + i)*S + j] * scale * x_i[c]  (dV with
// w = P, x = dO, scale absent; dK with w = dS, x = Q, scale = 1/sqrt(d)).
template <bool kScaled>
__global__ void AttnColKernel(const float* __restrict__ w, const float* __restrict__ x,
                              float* __restrict__ out, size_t B, size_t S, size_t H, size_t d,
                              float inv_sqrt_d) {
  const int lane = threadIdx.x & 31;
  const size_t D = H * d, units = B * H * S;
  for (size_t u = blockIdx.x * static_cast<size_t>(kWarps) + (threadIdx.x >> 5); u < units;
       u += static_cast<size_t>(gridDim.x) * kWarps) {
    const Unit un = UnitOf(u, H, S);
    const size_t j = un.i;
    const float* wcol = w + (un.b * H + un.h) * S * S + j;
    const float* xb = x + un.b * S * D + un.h * d;
    float* oj = out + (un.b * S + j) * D + un.h * d;
    for (size_t c = lane; c < d; c += 32) {
      float acc = 0.0f;
      for (size_t i = j; i < S; ++i) {
        float g = wcol[i * S];
        if (kScaled) g = g * inv_sqrt_d;
        acc += g * xb[i * D + c];
      }
      oj[c] = acc;
    }
  }
}

// dQ_i[c] = sum over j <= i of (dS[u, j] / sqrt(d)) * k_j[c].
__global__ void AttnDQKernel(const float* __restrict__ ds, const float* __restrict__ k,
                             float* __restrict__ dq, size_t B, size_t S, size_t H, size_t d,
                             float inv_sqrt_d) {
  const int lane = threadIdx.x & 31;
  const size_t D = H * d, units = B * H * S;
  for (size_t u = blockIdx.x * static_cast<size_t>(kWarps) + (threadIdx.x >> 5); u < units;
       u += static_cast<size_t>(gridDim.x) * kWarps) {
    const Unit un = UnitOf(u, H, S);
    const float* dsrow = ds + u * S;
    const float* kb = k + un.b * S * D + un.h * d;
    float* dqi = dq + (un.b * S + un.i) * D + un.h * d;
    for (size_t c = lane; c < d; c += 32) {
      float acc = 0.0f;
      for (size_t j = 0; j <= un.i; ++j) acc += (dsrow[j] * inv_sqrt_d) * kb[j * D + c];
      dqi[c] = acc;
    }
  }
}

// dS = P * (dP - rowsum(dP * P)), the rowsum in double.
__global__ void SoftmaxRowsBwdKernel(const float* __restrict__ probs, const float* __restrict__ dp,
                                     float* __restrict__ ds, size_t rows, size_t cols) {
  const int lane = threadIdx.x & 31;
  for (size_t r = blockIdx.x * static_cast<size_t>(kWarps) + (threadIdx.x >> 5); r < rows;
       r += static_cast<size_t>(gridDim.x) * kWarps) {
    const float* pr = probs + r * cols;
    const float* dpr = dp + r * cols;
    float* dsr = ds + r * cols;
    double dot = 0.0;
    for (size_t c = lane; c < cols; c += 32)
      dot += static_cast<double>(dpr[c]) * static_cast<double>(pr[c]);
    const float sum = static_cast<float>(WarpSumD(dot));
    for (size_t c = lane; c < cols; c += 32) dsr[c] = pr[c] * (dpr[c] - sum);
  }
}

// Tiled dQ: recomputes the row's probabilities and dP, writes delta into the
// stats row, then dQ (reference: runtime/executor/attention.cc:492-531).
__global__ void AttnDQTiledKernel(const float* __restrict__ q, const float* __restrict__ k,
                                  const float* __restrict__ v, const float* __restrict__ dout,
                                  float* __restrict__ stats, float* __restrict__ dq, size_t B,
                                  size_t S, size_t H, size_t d, float inv_sqrt_d) {
  extern __shared__ float smem[];
  // per warp: q row (d), dO row (d) packed as 2d, then prow (S), dprow (S)
  float* base = smem + (threadIdx.x >> 5) * (2 * d + 2 * S);
  float* qs = base;
  float* dos = base + d;
  float* prow = base + 2 * d;
  float* dprow = prow + S;
  const int lane = threadIdx.x & 31;
  const size_t D = H * d, units = B * H * S;
  for (size_t u = blockIdx.x * static_cast<size_t>(kWarps) + (threadIdx.x >> 5); u < units;
       u += static_cast<size_t>(gridDim.x) * kWarps) {
    const Unit un = UnitOf(u, H, S);
    const size_t b = un.b, h = un.h, i = un.i;
    const float* qi = q + (b * S + i) * D + h * d;
    const float* doi = dout + (b * S + i) * D + h * d;
    for (size_t c = lane; c < d; c += 32) {
      qs[c] = qi[c];
      dos[c] = doi[c];
    }
    float* st = stats + u * kAttnStatsWidth;
    const float m = st[0], inv_denom = st[1];
    const size_t j0 = StatsStart(st[3], i);
    __syncwarp();
    const float* kb = k + b * S * D + h * d;
    const float* vb = v + b * S * D + h * d;
    double dot = 0.0;
    for (size_t j = j0 + lane; j <= i; j += 32) {
      const float sc = static_cast<float>(DotD(qs, kb + j * D, d)) * inv_sqrt_d;
      const float p = expf(sc - m) * inv_denom;
      const float dpv = static_cast<float>(DotD(dos, vb + j * D, d));
      prow[j] = p;
      dprow[j] = dpv;
      dot += static_cast<double>(dpv) * static_cast<double>(p);
    }
    const float delta = static_cast<float>(WarpSumD(dot));
    __syncwarp();
    if (lane == 0) st[2] = delta;
    float* dqi = dq + (b * S + i) * D + h * d;
    for (size_t c = lane; c < d; c += 32) {
      float acc = 0.0f;
      for (size_t j = j0; j <= i; ++j) {
        const float dsv = prow[j] * (dprow[j] - delta);
        acc += (dsv * inv_sqrt_d) * kb[j * D + c];
      }
      dqi[c] = acc;
    }
    __syncwarp();
  }
}

// Tiled dK (kWantDK) or dV over the query rows i >= j of key j (reference:
// runtime/executor/attention.cc:533-590).  Thirty-two query rows at a time:
// each lane recomputes one row's weight, then the warp folds the rows in
// ascending order with lanes across the head width.
template <bool kWantDK>
__global__ void AttnDKVTiledKernel(const float* __restrict__ q, const float* __restrict__ k,
                                   const float* __restrict__ v, const float* __restrict__ dout,
                                   const float* __restrict__ stats, float* __restrict__ out,
                                   size_t B, size_t S, size_t H, size_t d, float inv_sqrt_d) {
  extern __shared__ float smem[];
  float* ks = smem + (threadIdx.x >> 5) * (2 * d);
  float* vs = ks + d;
  const int lane = threadIdx.x & 31;
  const size_t D = H * d, units = B * H * S;
  for (size_t u = blockIdx.x * static_cast<size_t>(kWarps) + (threadIdx.x >> 5); u < units;
       u += static_cast<size_t>(gridDim.x) * kWarps) {
    const Unit un = UnitOf(u, H, S);
    const size_t b = un.b, h = un.h, j = un.i;
    const float* kj = k + (b * S + j) * D + h * d;
    const float* vj = v + (b * S + j) * D + h * d;
    for (size_t c = lane; c < d; c += 32) {
      ks[c] = kj[c];
      vs[c] = vj[c];
    }
    __syncwarp();
    const float* qb = q + b * S * D + h * d;
    const float* dob = dout + b * S * D + h * d;
    const float* stb = stats + (b * H + h) * S * kAttnStatsWidth;
    // Up to 8 output features per lane (d <= 256).
    float acc[8];
#pragma unroll
    for (int t = 0; t < 8; ++t) acc[t] = 0.0f;
    for (size_t i0 = j; i0 < S; i0 += 32) {
      const size_t i = i0 + lane;
      float g = 0.0f;
      bool live = false;
      if (i < S) {
        const float* st = stb + i * kAttnStatsWidth;
        if (!(j < StatsStart(st[3], i))) {
          live = true;
          const float sc = static_cast<float>(DotD(ks, qb + i * D, d)) * inv_sqrt_d;
          const float p = expf(sc - st[0]) * st[1];
          if (kWantDK) {
            const float dsv = p * (static_cast<float>(DotD(vs, dob + i * D, d)) - st[2]);
            g = dsv * inv_sqrt_d;
          } else {
            g = p;
          }
        }
      }
      const unsigned live_mask = __ballot_sync(0xFFFFFFFFu, live);
      const size_t rows = S - i0 < 32 ? S - i0 : 32;
      const float* xb = kWantDK ? qb : dob;
      for (size_t r = 0; r < rows; ++r) {
        const float gr = __shfl_sync(0xFFFFFFFFu, g, static_cast<int>(r));
        if (!((live_mask >> r) & 1u)) continue;
        const float* xr = xb + (i0 + r) * D;
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          const size_t c = lane + 32 * static_cast<size_t>(t);
          if (c < d) acc[t] += gr * xr[c];
        }
      }
    }
    float* oj = out + (b * S + j) * D + h * d;
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      const size_t c = lane + 32 * static_cast<size_t>(t);
      if (c < d) oj[c] = acc[t];
    }
    __syncwarp();
  }
}

inline unsigned UnitBlocks(size_t units) {
  size_t b = (units + kWarps - 1) / kWarps;
  if (b < 1) b = 1;
  if (b > 148 * 16) b = 148 * 16;
  return static_cast<unsigned>(b);
}

template <typename Kernel>
inline bool AllowSmem(Kernel kernel, size_t bytes) {
  if (bytes <= 48 * 1024) return true;
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              static_cast<int>(bytes)) == cudaSuccess;
}

}  // namespace

// The dot-product identity a.b = b.a holds bit for bit here (each product is
// exact in double and the order over c is the same), so the tiled backward may
// keep the key row in shared memory and stream the query rows.

void AttnFwd(const float* q, const float* k, const float* v, float* o, float* probs,
             float* stats, size_t B, size_t S, size_t H, size_t d, const int32_t* starts,
             cudaStream_t s) {
  const size_t units = B * H * S;
  if (units == 0) return;
  const size_t bytes = kWarps * (d + S) * sizeof(float);
  AllowSmem(AttnFwdKernel, bytes);
  const float inv_sqrt_d = 1.0f / sqrtf(static_cast<float>(d));
  AttnFwdKernel<<<UnitBlocks(units), kWarps * 32, bytes, s>>>(q, k, v, o, probs, stats, B, S, H, d,
                                                             starts, inv_sqrt_d);
}

void AttnDP(const float* dout, const float* v, float* dp, size_t B, size_t S, size_t H, size_t d,
            cudaStream_t s) {
  const size_t units = B * H * S;
  if (units == 0) return;
  const size_t bytes = kWarps * d * sizeof(float);
  AllowSmem(AttnDPKernel, bytes);
  AttnDPKernel<<<UnitBlocks(units), kWarps * 32, bytes, s>>>(dout, v, dp, B, S, H, d);
}

void AttnDV(const float* probs, const float* dout, float* dv, size_t B, size_t S, size_t H,
            size_t d, cudaStream_t s) {
  const size_t units = B * H * S;
  if (units == 0) return;
  AttnColKernel<false><<<UnitBlocks(units), kWarps * 32, 0, s>>>(probs, dout, dv, B, S, H, d, 1.0f);
}

void AttnDK(const float* ds, const float* q, float* dk, size_t B, size_t S, size_t H, size_t d,
            cudaStream_t s) {
  const size_t units = B * H * S;
  if (units == 0) return;
  const float inv_sqrt_d = 1.0f / sqrtf(static_cast<float>(d));
  AttnColKernel<true><<<UnitBlocks(units), kWarps * 32, 0, s>>>(ds, q, dk, B, S, H, d, inv_sqrt_d);
}

void AttnDQ(const float* ds, const float* k, float* dq, size_t B, size_t S, size_t H, size_t d,
            cudaStream_t s) {
  const size_t units = B * H * S;
  if (units == 0) return;
  const float inv_sqrt_d = 1.0f / sqrtf(static_cast<float>(d));
  AttnDQKernel<<<UnitBlocks(units), kWarps * 32, 0, s>>>(ds, k, dq, B, S, H, d, inv_sqrt_d);
}

void SoftmaxRowsBwd(const float* probs, const float* dp, float* ds, size_t rows, size_t cols,
                    cudaStream_t s) {
  if (rows == 0) return;
  SoftmaxRowsBwdKernel<<<UnitBlocks(rows), kWarps * 32, 0, s>>>(probs, dp, ds, rows, cols);
}

void AttnDQTiled(const float* q, const float* k, const float* v, const float* dout, float* stats,
                 float* dq, size_t B, size_t S, size_t H, size_t d, cudaStream_t s) {
  const size_t units = B * H * S;
  if (units == 0) return;
  const size_t bytes = kWarps * (2 * d + 2 * S) * sizeof(float);
  AllowSmem(AttnDQTiledKernel, bytes);
  const float inv_sqrt_d = 1.0f / sqrtf(static_cast<float>(d));
  AttnDQTiledKernel<<<UnitBlocks(units), kWarps * 32, bytes, s>>>(q, k, v, dout, stats, dq, B, S, H,
                                                                 d, inv_sqrt_d);
}

void AttnDKVTiled(bool want_dk, const float* q, const float* k, const float* v, const float* dout,
                  const float* stats, float* out, size_t B, size_t S, size_t H, size_t d,
                  cudaStream_t s) {
  const size_t units = B * H * S;
  if (units == 0) return;
  const size_t bytes = kWarps * 2 * d * sizeof(float);
  const float inv_sqrt_d = 1.0f / sqrtf(static_cast<float>(d));
  if (want_dk) {
    AllowSmem(AttnDKVTiledKernel<true>, bytes);
    AttnDKVTiledKernel<true><<<UnitBlocks(units), kWarps * 32, bytes, s>>>(q, k, v, dout, stats, out,
                                                                          B, S, H, d, inv_sqrt_d);
  } else {
    AllowSmem(AttnDKVTiledKernel<false>, bytes);
    AttnDKVTiledKernel<false><<<UnitBlocks(units), kWarps * 32, bytes, s>>>(q, k, v, dout, stats,
                                                                           out, B, S, H, d,
                                                                           inv_sqrt_d);
  }
}

}  // namespace see::k
