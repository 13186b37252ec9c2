// Device-side tails of evaluation and merge: the accuracy tally over the
// softmax probabilities and the finiteness scan of merged deltas.  The
// reference computes both on the host over its arena (reference:
// runtime/dispatcher/update_engine.cc:535-564 and :1051-1060); with discrete
// memory that would move the whole probability tensor over the bus, so the
// same integer results are produced here and only three counters come back.
// Integer tallies: exact whatever the order of the atomic adds.
#include "kernels.h"

namespace see::k {

namespace {

// One warp per row.  argmax as the sequential scan defines it: start at column
// 0, move to column c only when row[c] > row[argmax] — the first maximum wins,
// a NaN never wins, and a NaN in column 0 is never displaced.
__global__ void ArgmaxTallyKernel(const float* __restrict__ probs, const int32_t* __restrict__ labels,
                                  size_t N, size_t C, unsigned long long* __restrict__ tally) {
  const int lane = threadIdx.x & 31;
  const size_t warps = (static_cast<size_t>(gridDim.x) * blockDim.x) >> 5;
  unsigned long long rows = 0, hits = 0;
  for (size_t r = (blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x) >> 5; r < N;
       r += warps) {
    const int32_t lab = labels[r];
    if (lab < 0) continue;
    const float* row = probs + r * C;
    const float first = row[0];
    size_t arg = 0;
    if (!isnan(first)) {
      float best = first;
      size_t idx = 0;
      for (size_t c = lane; c < C; c += 32) {
        const float v = row[c];
        if (v > best || (v == best && c < idx)) { best = v; idx = c; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
        const unsigned long long oi = __shfl_xor_sync(0xFFFFFFFFu, static_cast<unsigned long long>(idx), o);
        if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
      }
      arg = idx;
    }
    if (lane == 0) {
      ++rows;
      if (static_cast<size_t>(lab) == arg) ++hits;
    }
  }
  if (lane == 0 && rows) {
    atomicAdd(&tally[0], rows);
    atomicAdd(&tally[1], hits);
  }
}

__global__ void CountNonFiniteKernel(const float* __restrict__ x, size_t n,
                                     unsigned long long* __restrict__ tally) {
  unsigned long long bad = 0;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += stride)
    bad += !isfinite(x[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) bad += __shfl_xor_sync(0xFFFFFFFFu, bad, o);
  if ((threadIdx.x & 31) == 0 && bad) atomicAdd(&tally[2], bad);
}

// ---- the real-row loss of an evaluated batch -------------------------------------------
// The engine scores a validation set whose last batch wraps (or any masked
// plan) over its real rows alone: the sum, in row order and in double, of each
// row's loss evaluated with the loss kernel's own expression (reference:
// runtime/dispatcher/update_engine.cc:977-1026).  Two kernels: every row's
// term in parallel, then ONE thread adds the terms in row order, so the double
// sum has the reference's association.  The count of rows the sum is over (the
// real rows, or the real TARGET rows under a masked loss) is an integer tally.
__global__ void XentRowTermsKernel(const float* __restrict__ probs, const int32_t* __restrict__ labels,
                                   size_t rows, size_t width, double* __restrict__ terms) {
  const size_t r = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (r >= rows) return;
  const int32_t lab = labels[r];
  if (lab < 0) { terms[r] = 0.0; return; }   // skipped by the fold (it tests the label too)
  const float p = probs[r * width + static_cast<size_t>(lab)];
  const double safe = isnan(p) ? static_cast<double>(p) : static_cast<double>(fmaxf(p, 1e-12f));
  terms[r] = log(safe);
}

__global__ void SquaredDiffTermsKernel(const float* __restrict__ pred, const float* __restrict__ target,
                                       size_t n, double* __restrict__ terms) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += stride) {
    const double d = static_cast<double>(pred[i]) - target[i];
    terms[i] = d * d;
  }
}

// out[0] = sum (sign = -1: minus the terms; +1: plus), out[1] = divisor applied
// (MSE: the row width), tally[3] = rows counted.
__global__ void OrderedFoldKernel(const double* __restrict__ terms, const int32_t* __restrict__ labels,
                                  size_t n, double sign, double divisor, double* __restrict__ out,
                                  unsigned long long* __restrict__ tally) {
  if (blockIdx.x != 0 || threadIdx.x != 0) return;
  double sum = 0.0;
  unsigned long long counted = 0;
  for (size_t i = 0; i < n; ++i) {
    if (labels && labels[i] < 0) continue;
    ++counted;
    sum += sign * terms[i];   // x + (-t) and x - t are the same IEEE operation
  }
  out[0] = divisor != 0.0 ? sum / divisor : sum;
  tally[3] = counted;
}

// ---- per-column int8 quantiser ----------------------------------------------------------
// scale[n] = max_k |w[k, n]| / 127, an all-zero column takes 1, and the scale
// never falls below the smallest normal float; level = round-half-away(w /
// scale) clamped to +-127, by a true division (reference:
// compiler/backend/allocation/arena_binder.cc:129-190).  A maximum does not
// depend on the order it is taken in, so atomics on the bit pattern of |w|
// (non-negative floats order like their bits) give the reference's scales exactly.
__global__ void ColumnAbsMaxKernel(const float* __restrict__ w, size_t K, size_t N,
                                   unsigned int* __restrict__ maxbits) {
  const size_t n = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (n >= N) return;
  const size_t rows_per = (K + gridDim.y - 1) / gridDim.y;
  const size_t k0 = blockIdx.y * rows_per, k1 = k0 + rows_per < K ? k0 + rows_per : K;
  float m = 0.0f;
  for (size_t k = k0; k < k1; ++k) {
    const float a = fabsf(w[k * N + n]);
    if (m < a) m = a;   // std::max(m, a): a NaN never replaces m
  }
  atomicMax(&maxbits[n], __float_as_uint(m));
}

__global__ void ColumnScaleKernel(const unsigned int* __restrict__ maxbits, size_t N, float* __restrict__ scales) {
  const size_t n = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (n >= N) return;
  const float m = __uint_as_float(maxbits[n]);
  const float q = __fdiv_rn(m, 127.0f);
  scales[n] = m == 0.0f ? 1.0f : (q < 1.17549435e-38f ? 1.17549435e-38f : q);
}

__global__ void QuantizeLevelsKernel(const float* __restrict__ w, const float* __restrict__ scales, size_t count,
                                     size_t N, int8_t* __restrict__ q) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < count; i += stride) {
    float r = roundf(__fdiv_rn(w[i], scales[i % N]));   // roundf: halves away from zero, as std::round
    r = r < -127.0f ? -127.0f : (r > 127.0f ? 127.0f : r);
    q[i] = static_cast<int8_t>(r);
  }
}

}  // namespace

void XentRealRowLoss(const float* probs, const int32_t* labels, size_t real_rows, size_t width,
                     double* terms, double* out, unsigned long long* tally, cudaStream_t s) {
  if (real_rows)
    XentRowTermsKernel<<<static_cast<unsigned>((real_rows + 255) / 256), 256, 0, s>>>(probs, labels, real_rows,
                                                                                     width, terms);
  OrderedFoldKernel<<<1, 32, 0, s>>>(terms, labels, real_rows, -1.0, 0.0, out, tally);
}

void MseRealRowLoss(const float* pred, const float* target, size_t real_rows, size_t width, double* terms,
                    double* out, unsigned long long* tally, cudaStream_t s) {
  const size_t n = real_rows * width;
  if (n) {
    size_t blocks = (n + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    SquaredDiffTermsKernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(pred, target, n, terms);
  }
  OrderedFoldKernel<<<1, 32, 0, s>>>(terms, nullptr, n, 1.0, static_cast<double>(width), out, tally);
}

void QuantizeColumns(const float* w, size_t K, size_t N, int8_t* levels, float* scales,
                     unsigned int* maxbits_scratch, cudaStream_t s) {
  if (K == 0 || N == 0) return;
  cudaMemsetAsync(maxbits_scratch, 0, N * sizeof(unsigned int), s);
  unsigned slices = static_cast<unsigned>((K + 63) / 64);
  if (slices > 1024) slices = 1024;
  const dim3 grid(static_cast<unsigned>((N + 127) / 128), slices);
  ColumnAbsMaxKernel<<<grid, 128, 0, s>>>(w, K, N, maxbits_scratch);
  ColumnScaleKernel<<<static_cast<unsigned>((N + 127) / 128), 128, 0, s>>>(maxbits_scratch, N, scales);
  size_t blocks = (K * N + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  QuantizeLevelsKernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(w, scales, K * N, N, levels);
}

void ArgmaxTally(const float* probs, const int32_t* labels, size_t N, size_t C,
                 unsigned long long* tally, cudaStream_t s) {
  if (N == 0) return;
  size_t blocks = (N + 7) / 8;
  if (blocks > 148 * 8) blocks = 148 * 8;
  ArgmaxTallyKernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(probs, labels, N, C, tally);
}

void CountNonFinite(const float* x, size_t n, unsigned long long* tally, cudaStream_t s) {
  if (n == 0) return;
  size_t blocks = (n + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  CountNonFiniteKernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(x, n, tally);
}

}  // namespace see::k
