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

}  // namespace

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
