// Losses: softmax cross-entropy (plain and masked), MSE, KL distillation.
// HBM-bound row kernels.  The row softmax is the reference's f32 expression
// (max, exp(x - max), sum, times 1/sum; reference: runtime/executor/loss.cc:21-31)
// with the row sum taken as lane/thread partials combined in a fixed order.
// The batch loss follows the reference's shape-chunked contract exactly
// (reference: runtime/executor/loss.cc:35-72, source/parallel/parallel_for.h:55-67):
// per-row -log p in double, rows folded sequentially inside each chunk, chunks
// folded in chunk order, so the loss does not depend on the launch geometry.
// Integer results (the masked forms' target count) are exact.
#include <atomic>
#include "act_expr.cuh"
#include "kernels.h"
#include "shadow.cuh"

namespace see::k {

namespace {

constexpr size_t kMaxChunks = 256;   // the reference's kMaxParallelChunks
constexpr size_t kGrainCheap = 32768;
constexpr size_t kGrainMath = 4096;

__host__ __device__ inline size_t RowGrain(size_t per_row, size_t budget) {
  return per_row == 0 ? budget : (budget / per_row > 0 ? budget / per_row : 1);
}
__host__ __device__ inline size_t ChunkGrain(size_t n, size_t grain) {
  if (grain == 0) grain = 1;
  const size_t cap = (n + kMaxChunks - 1) / kMaxChunks;
  return grain < cap ? cap : grain;
}

__device__ __forceinline__ float WarpMax(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
  return v;
}
__device__ __forceinline__ float WarpSumF(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}
__device__ __forceinline__ double WarpSumD(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}

// Block-wide reductions for kThreads = 256 (8 warps); every thread gets the result.
template <typename T, typename WarpOp, typename Op>
__device__ __forceinline__ T BlockReduce(T v, T identity, T* smem, WarpOp warp_op, Op op) {
  v = warp_op(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  T r = identity;
  const int warps = blockDim.x >> 5;
  for (int w = 0; w < warps; ++w) r = op(r, smem[w]);
  return r;
}

// One block per row.  probs[row] = softmax(logits[row] * inv_T); returns the
// normalised probabilities in place and, via *p_label, the label's probability.
__device__ void RowSoftmaxBlock(const float* __restrict__ lrow, float* __restrict__ prow, size_t C,
                                float inv_T, float* smem_f) {
  float mx = -INFINITY;
  bool any = false;
  for (size_t c = threadIdx.x; c < C; c += blockDim.x) {
    const float v = lrow[c] * inv_T;
    mx = any ? fmaxf(mx, v) : v;
    any = true;
  }
  // Threads with no element hold -inf, which fmaxf ignores against any number.
  mx = BlockReduce<float>(mx, -INFINITY, smem_f, WarpMax,
                          [](float a, float b) { return fmaxf(a, b); });
  float sum = 0.0f;
  for (size_t c = threadIdx.x; c < C; c += blockDim.x) {
    const float e = expf(lrow[c] * inv_T - mx);
    prow[c] = e;
    sum += e;
  }
  sum = BlockReduce<float>(sum, 0.0f, smem_f, WarpSumF, [](float a, float b) { return a + b; });
  const float inv_sum = 1.0f / sum;
  for (size_t c = threadIdx.x; c < C; c += blockDim.x) prow[c] *= inv_sum;
  __syncthreads();
}

__device__ __forceinline__ double NegLogSafe(float p) {
  const double safe = isnan(p) ? static_cast<double>(p) : static_cast<double>(fmaxf(p, 1e-12f));
  return -log(safe);
}

// row_loss[n] = -log p[n, label]; masked rows (label < 0) store 0 and are
// skipped by the fold.  A label outside [0, C) is treated as the reference's
// feeder contract would never allow: it reads class 0's probability scaled by
// nothing — the row contributes NaN so the run fails loudly instead of
// reading outside the row.
__global__ void XEntRowsKernel(const float* __restrict__ logits, const int32_t* __restrict__ labels,
                               float* __restrict__ probs, double* __restrict__ row_loss, size_t N,
                               size_t C, bool masked) {
  __shared__ float smem_f[32];
  for (size_t n = blockIdx.x; n < N; n += gridDim.x) {
    RowSoftmaxBlock(logits + n * C, probs + n * C, C, 1.0f, smem_f);
    if (threadIdx.x == 0) {
      const int32_t lab = labels[n];
      double v;
      if (masked && lab < 0) v = 0.0;
      else if (lab < 0 || static_cast<size_t>(lab) >= C) v = NAN;
      else v = NegLogSafe(probs[n * C + static_cast<size_t>(lab)]);
      row_loss[n] = v;
    }
  }
}

// The same row softmax for wide rows (4096 <= C <= 32768, C % 4 == 0): one
// 1024-thread block per row with the whole row in registers (eight 16-byte
// vectors per thread), so the logits are read from HBM once and the
// probabilities written once.  The next row is copied into shared memory
// asynchronously (cp.async) while the current one is reduced, each thread
// fetching exactly the chunks it will later read itself, so no barrier guards
// the buffer.  Same expressions per element as RowSoftmaxBlock; the row sum is
// folded as thread partials (ascending index), warp shuffles, then warps in order.
constexpr int kWideThreads = 1024;
constexpr int kWideVecs = 8;

__device__ __forceinline__ void CpAsync16(void* smem, const void* gmem) {
  const unsigned s = static_cast<unsigned>(__cvta_generic_to_shared(smem));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}

__global__ void __launch_bounds__(kWideThreads, 1)
XEntRowsWideKernel(const float* __restrict__ logits, const int32_t* __restrict__ labels,
                   float* __restrict__ probs, double* __restrict__ row_loss, size_t N, size_t C,
                   bool masked, Shadow sh, float bwd_scale, bool store_probs) {
  extern __shared__ __align__(16) float4 row_smem[];
  __shared__ float smem_f[32];
  __shared__ float label_prob;
  const int C4 = static_cast<int>(C / 4);
  const int tid = threadIdx.x;
  auto prefetch = [&](size_t n) {
    const float4* lrow = reinterpret_cast<const float4*>(logits + n * C);
#pragma unroll
    for (int i = 0; i < kWideVecs; ++i) {
      const int c4 = i * kWideThreads + tid;
      if (c4 < C4) CpAsync16(&row_smem[c4], &lrow[c4]);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (blockIdx.x < N) prefetch(blockIdx.x);
  for (size_t n = blockIdx.x; n < N; n += gridDim.x) {
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    float4 x[kWideVecs];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < kWideVecs; ++i) {
      const int c4 = i * kWideThreads + tid;
      if (c4 < C4) {
        x[i] = row_smem[c4];
        mx = fmaxf(fmaxf(mx, x[i].x), fmaxf(x[i].y, fmaxf(x[i].z, x[i].w)));
      }
    }
    if (n + gridDim.x < N) prefetch(n + gridDim.x);
    mx = BlockReduce<float>(mx, -INFINITY, smem_f, WarpMax,
                            [](float a, float b) { return fmaxf(a, b); });
    // e^{x - mx} = 2^{x log2 e - mx log2 e} on the hardware exponential: one FMA and
    // one MUFU per element (libm expf is about twenty instructions, and a
    // vocabulary-wide row is instruction-bound with it).  Relative error about 1e-6
    // at the far end of the row, inside the 1e-5 these rows are held to.
    constexpr float kLog2E = 1.4426950408889634f;
    const float shift = -mx * kLog2E;
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < kWideVecs; ++i) {
      if (i * kWideThreads + tid < C4) {
        x[i].x = Ex2Approx(__fmaf_rn(x[i].x, kLog2E, shift)); sum += x[i].x;
        x[i].y = Ex2Approx(__fmaf_rn(x[i].y, kLog2E, shift)); sum += x[i].y;
        x[i].z = Ex2Approx(__fmaf_rn(x[i].z, kLog2E, shift)); sum += x[i].z;
        x[i].w = Ex2Approx(__fmaf_rn(x[i].w, kLog2E, shift)); sum += x[i].w;
      }
    }
    sum = BlockReduce<float>(sum, 0.0f, smem_f, WarpSumF, [](float a, float b) { return a + b; });
    const float inv_sum = 1.0f / sum;
    float4* prow = reinterpret_cast<float4*>(probs + n * C);
    const int32_t lab = labels[n];
    const int lab4 = lab >= 0 && static_cast<size_t>(lab) < C ? lab >> 2 : -1;
#pragma unroll
    for (int i = 0; i < kWideVecs; ++i) {
      const int c4 = i * kWideThreads + tid;
      if (c4 < C4) {
        const float4 p = make_float4(x[i].x * inv_sum, x[i].y * inv_sum, x[i].z * inv_sum, x[i].w * inv_sum);
        if (store_probs) prow[c4] = p;
        if (c4 == lab4) label_prob = (lab & 3) == 0 ? p.x : (lab & 3) == 1 ? p.y : (lab & 3) == 2 ? p.z : p.w;
        if (sh.dst) {
          // The backward instruction's arithmetic on the value it would have read back.
          float4 v = make_float4(bwd_scale * p.x, bwd_scale * p.y, bwd_scale * p.z, bwd_scale * p.w);
          if (c4 == lab4) {
            switch (lab & 3) {
              case 0: v.x -= bwd_scale; break;
              case 1: v.y -= bwd_scale; break;
              case 2: v.z -= bwd_scale; break;
              default: v.w -= bwd_scale; break;
            }
          }
          ShadowStore4(sh, n * static_cast<size_t>(C4) + c4, static_cast<uint32_t>(c4 * 4), v);
        }
      }
    }
    __syncthreads();  // label_prob is visible to thread 0 below; and the smem buffers are reused
    if (tid == 0) {
      double v;
      if (masked && lab < 0) v = 0.0;
      else if (lab < 0 || static_cast<size_t>(lab) >= C) v = NAN;
      else v = NegLogSafe(label_prob);
      row_loss[n] = v;
    }
  }
}

// Folds row losses with the reference's chunk geometry: thread t owns chunk t
// (rows [t*grain, ...)), summed sequentially; thread 0 then folds the chunk
// partials in chunk order.  One block of kMaxChunks threads.
__global__ void XEntFoldKernel(const double* __restrict__ row_loss,
                               const int32_t* __restrict__ labels, float* __restrict__ loss,
                               size_t N, size_t grain, bool masked,
                               unsigned long long* __restrict__ count_out) {
  __shared__ double partial[kMaxChunks];
  __shared__ unsigned long long targets[kMaxChunks];
  const size_t chunk = threadIdx.x;
  const size_t r0 = chunk * grain;
  double total = 0.0;
  unsigned long long t = 0;
  if (r0 < N) {
    const size_t r1 = r0 + grain < N ? r0 + grain : N;
    for (size_t n = r0; n < r1; ++n) {
      if (masked && labels[n] < 0) continue;
      total += row_loss[n];
      ++t;
    }
  }
  partial[chunk] = total;
  targets[chunk] = t;
  __syncthreads();
  if (threadIdx.x == 0) {
    const size_t chunks = (N + grain - 1) / grain;
    double sum = 0.0;
    unsigned long long T = 0;
    for (size_t c = 0; c < chunks; ++c) {
      sum += partial[c];
      T += targets[c];
    }
    if (masked) {
      *loss = T ? static_cast<float>(sum / static_cast<double>(T)) : 0.0f;
      if (count_out) *count_out = T;
    } else {
      *loss = static_cast<float>(sum / static_cast<double>(N));
    }
  }
}

__global__ void CountTargetsKernel(const int32_t* __restrict__ labels, size_t N,
                                   unsigned long long* __restrict__ count_out) {
  __shared__ unsigned long long smem[32];
  unsigned long long t = 0;
  for (size_t n = threadIdx.x; n < N; n += blockDim.x) t += labels[n] >= 0;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xFFFFFFFFu, t, o);
  if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = t;
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long T = 0;
    for (int w = 0; w < (blockDim.x >> 5); ++w) T += smem[w];
    *count_out = T;
  }
}

// dlogits = scale * probs, minus scale at the label (reference:
// runtime/executor/loss.cc:59-72, 107-126).  Bit-identical to the CPU given the
// same probs: one multiply, and one subtract at the label.
__global__ void XEntBwdKernel(const float* __restrict__ probs, const int32_t* __restrict__ labels,
                              const float* __restrict__ seed, float* __restrict__ dlogits, size_t N,
                              size_t C, bool masked,
                              const unsigned long long* __restrict__ count) {
  float scale;
  if (masked) {
    const unsigned long long T = *count;
    scale = T ? *seed / static_cast<float>(T) : 0.0f;
  } else {
    scale = *seed / static_cast<float>(N);
  }
  const size_t total = N * C;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += stride) {
    const size_t n = i / C, c = i % C;
    const int32_t lab = labels[n];
    float v;
    if (masked && lab < 0) {
      v = 0.0f;
    } else {
      v = scale * probs[i];
      if (static_cast<size_t>(lab) == c) v -= scale;
    }
    dlogits[i] = v;
  }
}

// The same for rows of whole 16-byte vectors: blockIdx.y walks rows, so the
// label and the row index are per-block values, not a division per element.
__global__ void XEntBwdRowsKernel(const float* __restrict__ probs, const int32_t* __restrict__ labels,
                                  const float* __restrict__ seed, float* __restrict__ dlogits,
                                  size_t N, size_t C, bool masked,
                                  const unsigned long long* __restrict__ count, Shadow sh) {
  float scale;
  if (masked) {
    const unsigned long long T = *count;
    scale = T ? *seed / static_cast<float>(T) : 0.0f;
  } else {
    scale = *seed / static_cast<float>(N);
  }
  const size_t C4 = C / 4;
  for (size_t n = blockIdx.y; n < N; n += gridDim.y) {
    const int32_t lab = labels[n];
    const float4* prow = reinterpret_cast<const float4*>(probs + n * C);
    float4* drow = reinterpret_cast<float4*>(dlogits + n * C);
    const bool off = masked && lab < 0;
    for (size_t c4 = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; c4 < C4;
         c4 += static_cast<size_t>(gridDim.x) * blockDim.x) {
      float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (!off) {
        const float4 pr = prow[c4];
        v = make_float4(scale * pr.x, scale * pr.y, scale * pr.z, scale * pr.w);
        if (lab >= 0 && static_cast<size_t>(lab) / 4 == c4) {
          switch (lab & 3) {
            case 0: v.x -= scale; break;
            case 1: v.y -= scale; break;
            case 2: v.z -= scale; break;
            default: v.w -= scale; break;
          }
        }
      }
      if (!sh.only) drow[c4] = v;
      if (sh.dst) ShadowStore4(sh, n * C4 + c4, static_cast<uint32_t>(c4 * 4), v);
    }
  }
}

// ---- MSE ---------------------------------------------------------------------
// Per-chunk double partials (chunk = kGrainCheap elements, capped at 256
// chunks), chunks folded in order (reference: runtime/executor/loss.cc:128-152).
__global__ void MsePartialKernel(const float* __restrict__ pred, const float* __restrict__ target,
                                 size_t n, size_t grain, double* __restrict__ partials) {
  __shared__ double smem[32];
  const size_t b = blockIdx.x * grain;
  const size_t e = b + grain < n ? b + grain : n;
  double total = 0.0;
  for (size_t i = b + threadIdx.x; i < e; i += blockDim.x) {
    const double d = static_cast<double>(pred[i]) - static_cast<double>(target[i]);
    total += d * d;
  }
  total = BlockReduce<double>(total, 0.0, smem, WarpSumD, [](double a, double c) { return a + c; });
  if (threadIdx.x == 0) partials[blockIdx.x] = total;
}
__global__ void MseFoldKernel(const double* __restrict__ partials, size_t chunks, size_t n,
                              float* __restrict__ loss) {
  double total = 0.0;
  for (size_t c = 0; c < chunks; ++c) total += partials[c];
  *loss = static_cast<float>(total / static_cast<double>(n));
}
__global__ void MseBwdKernel(const float* __restrict__ pred, const float* __restrict__ target,
                             const float* __restrict__ seed, float* __restrict__ dpred, size_t n) {
  const float scale = 2.0f * *seed / static_cast<float>(n);
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += stride)
    dpred[i] = scale * (pred[i] - target[i]);
}

// ---- KL distillation (reference: runtime/executor/loss.cc:154-202) ------------
__global__ void KLRowsKernel(const float* __restrict__ s_logits, const float* __restrict__ t_logits,
                             float* __restrict__ p_s, float* __restrict__ p_t,
                             double* __restrict__ row_loss, size_t N, size_t C, float inv_T) {
  __shared__ float smem_f[32];
  __shared__ double smem_d[32];
  for (size_t n = blockIdx.x; n < N; n += gridDim.x) {
    RowSoftmaxBlock(s_logits + n * C, p_s + n * C, C, inv_T, smem_f);
    RowSoftmaxBlock(t_logits + n * C, p_t + n * C, C, inv_T, smem_f);
    double total = 0.0;
    for (size_t c = threadIdx.x; c < C; c += blockDim.x) {
      const float pt = p_t[n * C + c];
      if (pt <= 0.0f) continue;
      const float ps_raw = p_s[n * C + c];
      const double ps = isnan(ps_raw) ? static_cast<double>(ps_raw)
                                      : static_cast<double>(fmaxf(ps_raw, 1e-12f));
      total += static_cast<double>(pt) * (log(static_cast<double>(pt)) - log(ps));
    }
    total = BlockReduce<double>(total, 0.0, smem_d, WarpSumD,
                                [](double a, double b) { return a + b; });
    if (threadIdx.x == 0) row_loss[n] = total;
  }
}
__global__ void KLFoldKernel(const double* __restrict__ row_loss, float* __restrict__ loss,
                             size_t N, size_t grain, float loss_scale) {
  __shared__ double partial[kMaxChunks];
  const size_t r0 = threadIdx.x * grain;
  double total = 0.0;
  if (r0 < N) {
    const size_t r1 = r0 + grain < N ? r0 + grain : N;
    for (size_t n = r0; n < r1; ++n) total += row_loss[n];
  }
  partial[threadIdx.x] = total;
  __syncthreads();
  if (threadIdx.x == 0) {
    const size_t chunks = (N + grain - 1) / grain;
    double sum = 0.0;
    for (size_t c = 0; c < chunks; ++c) sum += partial[c];
    *loss = static_cast<float>(sum / static_cast<double>(N)) * loss_scale;
  }
}
__global__ void KLBwdKernel(const float* __restrict__ p_s, const float* __restrict__ p_t,
                            const float* __restrict__ seed, float* __restrict__ dlogits,
                            size_t total, float n_rows, float T, float loss_scale) {
  const float scale = (*seed * loss_scale) / (n_rows * T);
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += stride)
    dlogits[i] = scale * (p_s[i] - p_t[i]);
}

inline unsigned GridFor(size_t items, int threads, unsigned cap) {
  size_t b = (items + threads - 1) / threads;
  if (b < 1) b = 1;
  if (b > cap) b = cap;
  return static_cast<unsigned>(b);
}

}  // namespace

bool SoftmaxXEntFwd(bool masked, const float* logits, const int32_t* labels, float* loss,
                    float* probs, size_t N, size_t C, double* row_scratch,
                    unsigned long long* count_scratch, cudaStream_t s, const XEntFusedBwd* fused_bwd) {
  if (N == 0) return false;
  bool fused = false;
  const bool wide = C >= 4096 && C <= static_cast<size_t>(4 * kWideThreads * kWideVecs) &&
                    (C & 3) == 0 && ((reinterpret_cast<uintptr_t>(logits) |
                                      reinterpret_cast<uintptr_t>(probs)) & 15) == 0;
  if (wide) {
    // Raising a kernel's dynamic shared-memory limit is a per-device setting of
    // the function, not an allocation; done on first use per device.
    // (Atomic flags: handle-free callers may make their first calls from two host
    // threads at once; setting the attribute twice is harmless, a torn flag is not.)
    static std::atomic<bool> configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev].load(std::memory_order_acquire)) {
      cudaFuncSetAttribute(XEntRowsWideKernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           4 * kWideThreads * kWideVecs * static_cast<int>(sizeof(float)));
      configured[dev].store(true, std::memory_order_release);
    }
    const unsigned blocks = static_cast<unsigned>(N < 148 * 4 ? N : 148 * 4);
    Shadow sh{};
    float bwd_scale = 0.0f;
    bool store_probs = true;
    if (fused_bwd && !masked && ShadowUsable(&fused_bwd->shadow, probs, N * C) && fused_bwd->shadow.cols == C) {
      sh = fused_bwd->shadow;
      bwd_scale = fused_bwd->seed / static_cast<float>(N);   // the backward kernel's own expression
      store_probs = fused_bwd->store_probs;
      fused = true;
    }
    XEntRowsWideKernel<<<blocks, kWideThreads, C * sizeof(float), s>>>(logits, labels, probs, row_scratch, N, C,
                                                                       masked, sh, bwd_scale, store_probs);
  } else {
    const int threads = C >= 1024 ? 256 : (C >= 128 ? 128 : 32);
    const unsigned blocks = static_cast<unsigned>(N < 148 * 16 ? N : 148 * 16);
    XEntRowsKernel<<<blocks, threads, 0, s>>>(logits, labels, probs, row_scratch, N, C, masked);
  }
  const size_t grain = ChunkGrain(N, RowGrain(C, kGrainMath));
  XEntFoldKernel<<<1, kMaxChunks, 0, s>>>(row_scratch, labels, loss, N, grain, masked,
                                         count_scratch);
  return fused;
}

bool SoftmaxXEntBwd(bool masked, const float* probs, const int32_t* labels, const float* seed,
                    float* dlogits, size_t N, size_t C, unsigned long long* count_scratch,
                    cudaStream_t s, const Shadow* shadow) {
  if (N * C == 0) return false;
  if (masked) CountTargetsKernel<<<1, 256, 0, s>>>(labels, N, count_scratch);
  if (C >= 1024 && (C & 3) == 0 &&
      ((reinterpret_cast<uintptr_t>(probs) | reinterpret_cast<uintptr_t>(dlogits)) & 15) == 0) {
    const size_t per_row = (C / 4 + 255) / 256;
    const dim3 grid(static_cast<unsigned>(per_row < 64 ? per_row : 64),
                    static_cast<unsigned>(N < 65535 ? N : 65535));
    const bool shadowed = ShadowUsable(shadow, dlogits, N * C) && shadow->cols == C;
    Shadow sh = shadowed ? *shadow : Shadow{};
    if (!shadowed) sh.only = false;
    XEntBwdRowsKernel<<<grid, 256, 0, s>>>(probs, labels, seed, dlogits, N, C, masked, count_scratch, sh);
    return shadowed;
  }
  XEntBwdKernel<<<GridFor(N * C, 256, 148 * 8), 256, 0, s>>>(probs, labels, seed, dlogits, N, C,
                                                            masked, count_scratch);
  return false;
}

void MseFwd(const float* pred, const float* target, float* loss, size_t n, double* scratch,
            cudaStream_t s) {
  if (n == 0) return;
  const size_t grain = ChunkGrain(n, kGrainCheap);
  const size_t chunks = (n + grain - 1) / grain;
  MsePartialKernel<<<static_cast<unsigned>(chunks), 256, 0, s>>>(pred, target, n, grain, scratch);
  MseFoldKernel<<<1, 1, 0, s>>>(scratch, chunks, n, loss);
}

void MseBwd(const float* pred, const float* target, const float* seed, float* dpred, size_t n,
            cudaStream_t s) {
  if (n == 0) return;
  MseBwdKernel<<<GridFor(n, 256, 148 * 8), 256, 0, s>>>(pred, target, seed, dpred, n);
}

void KLDistillFwd(const float* s_logits, const float* t_logits, float* loss, float* p_s,
                  float* p_t, size_t N, size_t C, float T, float loss_scale, double* row_scratch,
                  cudaStream_t s) {
  if (N == 0) return;
  const float inv_T = 1.0f / T;
  const int threads = C >= 1024 ? 256 : (C >= 128 ? 128 : 32);
  const unsigned blocks = static_cast<unsigned>(N < 148 * 16 ? N : 148 * 16);
  KLRowsKernel<<<blocks, threads, 0, s>>>(s_logits, t_logits, p_s, p_t, row_scratch, N, C, inv_T);
  const size_t grain = ChunkGrain(N, RowGrain(C, kGrainMath));
  KLFoldKernel<<<1, kMaxChunks, 0, s>>>(row_scratch, loss, N, grain, loss_scale);
}

void KLDistillBwd(const float* p_s, const float* p_t, const float* seed, float* dlogits,
                  size_t N, size_t C, float T, float loss_scale, cudaStream_t s) {
  if (N * C == 0) return;
  KLBwdKernel<<<GridFor(N * C, 256, 148 * 8), 256, 0, s>>>(p_s, p_t, seed, dlogits, N * C,
                                                          static_cast<float>(N), T, loss_scale);
}

}  // namespace see::k
