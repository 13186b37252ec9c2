// Shape-specialised exact kernels for the rank-r adapter products of a LoRA
// update.  A decoder step runs six of them per adapted projection, each moving
// one [rows x width] activation through HBM for a few hundred MFLOP, so they
// are streaming kernels: the wide operand is read once with 16-byte loads
// straight into registers, the rank-r operand lives in shared memory or
// registers, and there is no block-wide barrier inside the stream.
//
// Arithmetic per output element is the CPU executor's, operation for operation
// (reference: runtime/executor/gemm.cc:73-187 quad order, :346-527 lane
// order); compiled with -fmad=false.  Only the assignment of elements to
// threads differs from the general tile kernels.
//
// This file is compiled twice.  As see::k::exact (with -fmad=false) it is the
// bit-exact form the strict seam uses.  As see::k::fast (through
// k_gemm_skinny_fast.cu, multiply-adds contracted) it is the form the engine
// uses where the plan does not observe the bits: the same kernels, the same
// fixed reduction orders — so still identical run to run — at one instruction
// per multiply-add instead of two, and within a few 2^-24 of the exact form.
#include <atomic>

#include "gemm_exact_common.cuh"

#ifndef SEE_SKINNY_NAMESPACE
#define SEE_SKINNY_NAMESPACE exact
#endif

namespace see::k::SEE_SKINNY_NAMESPACE {

using namespace see::k::exact;   // Params, ApplyAct, Aligned16 (a no-op in the exact build)

namespace {

// Two-wide FP32 adds.  `add.rn.f32x2` rounds each half exactly as `add.rn.f32`
// does, and ptxas does not contract a SCALAR multiply into a packed add (it does
// contract a packed multiply feeding a packed add into a packed FMA, even with
// -fmad=false, which would break the reference's rounding: so products stay
// scalar).  Two neighbouring columns then cost two multiplies and one add per k
// instead of two and two.
__device__ __forceinline__ unsigned long long Pack2(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void Unpack2(unsigned long long v, float* lo, float* hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(*lo), "=f"(*hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long Add2(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

// One quad of the quad order for four neighbouring columns:
//   c[j] += ((a0*w0[j] + a1*w1[j]) + a2*w2[j]) + a3*w3[j]
__device__ __forceinline__ void QuadStep(float (&c)[4], float a0, float a1, float a2, float a3,
                                         const float4& w0, const float4& w1, const float4& w2,
                                         const float4& w3) {
  const float b0[4] = {w0.x, w0.y, w0.z, w0.w};
  const float b1[4] = {w1.x, w1.y, w1.z, w1.w};
  const float b2[4] = {w2.x, w2.y, w2.z, w2.w};
  const float b3[4] = {w3.x, w3.y, w3.z, w3.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float t = a0 * b0[j];
    t = t + a1 * b1[j];
    t = t + a2 * b2[j];
    t = t + a3 * b3[j];
    c[j] = c[j] + t;
  }
}

// ---- reduce: C[M, N = 4G] = A[M, K] * W, K long --------------------------------------
// A warp owns R * 32 / G rows; lane = (row slot, column group g) holds the outputs
// C[row, 4g .. 4g+3] of R rows, so every 16 bytes of W read from shared memory
// feed R rows.  The lanes of a row read the same 16 bytes of A (one broadcast
// load).  A row is consumed 16 k at a time from one of two register buffers, the
// next 16 k already in flight while these are multiplied.  All of W sits in
// shared memory (dynamic, K <= kReduceMaxK), in the layout it has in memory:
// [k][N] for the quad order (W is [K, N]); [n][k] for the lane order (W is
// [N, K]), where row n starts at n * (K + 16) + 4 * (n / 4) floats so that the
// four column groups of a warp read four different bank groups.
constexpr size_t kReduceMaxK = 3072;

template <int G, bool kLane, int R, int Q, int kReduceThreads>
__global__ void __launch_bounds__(kReduceThreads) ReduceKernel(Params p) {
  constexpr int N = 4 * G;
  constexpr int kRowsPerWarp = 32 / G;  // per row slot; a warp covers R of these
  constexpr int kRowsPerBlock = R * kRowsPerWarp * (kReduceThreads / 32);
  extern __shared__ __align__(16) float Wsm[];
  const int K = static_cast<int>(p.K);
  const int wn_stride = K + 16;
  auto wn_row = [&](int n) { return n * wn_stride + 4 * (n >> 2); };
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane % G;
  const float* B = static_cast<const float*>(p.B);
  size_t row[R];
  bool live[R];
  const float* xrow[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    row[r] = static_cast<size_t>(blockIdx.x) * kRowsPerBlock + (warp * R + r) * kRowsPerWarp + lane / G;
    live[r] = row[r] < p.M;
    xrow[r] = p.A + (live[r] ? row[r] : 0) * p.K;
  }

  // Stage W, eight 16-byte loads in flight per thread (the copy is latency-bound
  // otherwise: every block fetches all of W from L2).
  {
    const int per_row = K / 4, total = N * per_row;   // in float4 units; [n][k] and [k][n] alike
    for (int base = threadIdx.x; base < total; base += 8 * kReduceThreads) {
      float4 tmp[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int idx = base + u * kReduceThreads;
        if (idx < total) tmp[u] = reinterpret_cast<const float4*>(B)[idx];
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int idx = base + u * kReduceThreads;
        if (idx >= total) continue;
        if (kLane) {   // W is [N][K]: float4 unit idx is (n, kq) = (idx / per_row, idx % per_row)
          const int n = idx / per_row, kq = idx - n * per_row;
          *reinterpret_cast<float4*>(&Wsm[wn_row(n) + 4 * kq]) = tmp[u];
        } else {
          reinterpret_cast<float4*>(Wsm)[idx] = tmp[u];
        }
      }
    }
  }
  __syncthreads();
  if (!live[0]) return;  // rows ascend with r: a dead first row means a dead thread

  float c[R][4];       // quad order
  float acc[R][4][8];  // lane order
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      c[r][j] = 0.0f;
#pragma unroll
      for (int l = 0; l < 8; ++l) acc[r][j][l] = 0.0f;
    }

  auto load = [&](float4 (&buf)[R][Q], int k) {
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int q = 0; q < Q; ++q) buf[r][q] = *reinterpret_cast<const float4*>(xrow[r] + k + 4 * q);
  };
  auto consume = [&](const float4 (&buf)[R][Q], int k) {
#pragma unroll
    for (int q = 0; q < Q; ++q) {
      const int kq = k + 4 * q;
      if (kLane) {
        // Product k goes to accumulator k mod 8; k is a multiple of 8.
        const int l0 = (q & 1) * 4;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float4 w = *reinterpret_cast<const float4*>(&Wsm[wn_row(4 * g + j) + kq]);
#pragma unroll
          for (int r = 0; r < R; ++r) {
            acc[r][j][l0 + 0] = acc[r][j][l0 + 0] + buf[r][q].x * w.x;
            acc[r][j][l0 + 1] = acc[r][j][l0 + 1] + buf[r][q].y * w.y;
            acc[r][j][l0 + 2] = acc[r][j][l0 + 2] + buf[r][q].z * w.z;
            acc[r][j][l0 + 3] = acc[r][j][l0 + 3] + buf[r][q].w * w.w;
          }
        }
      } else {
        const float4 w0 = *reinterpret_cast<const float4*>(&Wsm[(kq + 0) * N + 4 * g]);
        const float4 w1 = *reinterpret_cast<const float4*>(&Wsm[(kq + 1) * N + 4 * g]);
        const float4 w2 = *reinterpret_cast<const float4*>(&Wsm[(kq + 2) * N + 4 * g]);
        const float4 w3 = *reinterpret_cast<const float4*>(&Wsm[(kq + 3) * N + 4 * g]);
#pragma unroll
        for (int r = 0; r < R; ++r) {
          if (p.alpha == 1.0f)   // 1.0f * x == x: the multiply changes no bit
            QuadStep(c[r], buf[r][q].x, buf[r][q].y, buf[r][q].z, buf[r][q].w, w0, w1, w2, w3);
          else
            QuadStep(c[r], p.alpha * buf[r][q].x, p.alpha * buf[r][q].y, p.alpha * buf[r][q].z,
                     p.alpha * buf[r][q].w, w0, w1, w2, w3);
        }
      }
    }
  };
  constexpr int kStep = 4 * Q;   // k per register buffer (8 or 16; K % 16 == 0)
  float4 xa[R][Q], xb[R][Q];
  load(xa, 0);
  for (int k = 0; k < K; k += 2 * kStep) {
    if (k + kStep < K) load(xb, k + kStep);
    consume(xa, k);
    if (k + kStep < K) {
      if (k + 2 * kStep < K) load(xa, k + 2 * kStep);
      consume(xb, k + kStep);
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    if (!live[r]) continue;
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (kLane) {
        float s = acc[r][j][0];
#pragma unroll
        for (int l = 1; l < 8; ++l) s = s + acc[r][j][l];
        v[j] = p.alpha * s;
      } else {
        v[j] = c[r][j];
      }
    }
    const size_t o = row[r] * N + 4 * g;
    if (p.addend) {
      const float4 d = *reinterpret_cast<const float4*>(p.addend + o);
      v[0] = d.x + v[0]; v[1] = d.y + v[1]; v[2] = d.z + v[2]; v[3] = d.w + v[3];
    }
    if (!kLane) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (p.bias) v[j] = v[j] + p.bias[4 * g + j];
        v[j] = ApplyAct(v[j], p.act);
      }
    }
    *reinterpret_cast<float4*>(p.C + o) = make_float4(v[0], v[1], v[2], v[3]);
  }
}

template <int G, bool kLane, int R, int Q, int kReduceThreads>
bool LaunchReduceAs(const Params& p, cudaStream_t s) {
  constexpr int N = 4 * G;
  constexpr int kRowsPerBlock = R * (32 / G) * (kReduceThreads / 32);
  const size_t smem = (kLane ? N * (p.K + 16) + 16 : p.K * N) * sizeof(float);
  static std::atomic<bool> configured_on[64] = {};   // per instantiation and device
  int dev = 0;
  cudaGetDevice(&dev);
  const bool tracked = dev >= 0 && dev < 64;
  if (!tracked || !configured_on[dev].load(std::memory_order_acquire)) {
    if (cudaFuncSetAttribute(ReduceKernel<G, kLane, R, Q, kReduceThreads>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(kReduceMaxK * N * sizeof(float) + 2048)) != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    if (tracked) configured_on[dev].store(true, std::memory_order_release);
  }
  const unsigned blocks = static_cast<unsigned>((p.M + kRowsPerBlock - 1) / kRowsPerBlock);
  ReduceKernel<G, kLane, R, Q, kReduceThreads><<<blocks, kReduceThreads, smem, s>>>(p);
  return true;
}

// ---- reduce, few rows: the block's rows of A staged in shared memory ------------------
// With a few thousand rows per GPU there are only a few warps per SM, and a
// thread that keeps two 16-k register buffers of its row in flight pays one
// DRAM round trip per 16 k: the kernel above is latency-bound there.  This one
// issues ALL of the block's traffic at once with 16-byte asynchronous copies
// (its rows of A and W, in four k chunks, one commit group each) and computes
// chunk c while chunks c+1.. are still landing, so the round trip is paid once.
// Rows of A sit at a stride of K + 4 floats: the row slots of a warp then read
// distinct bank groups.  Arithmetic per element is the same as above.
__device__ __forceinline__ void CpAsync16(float* smem_dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<unsigned>(
                   __cvta_generic_to_shared(smem_dst))), "l"(src) : "memory");
}
__device__ __forceinline__ void CpAsyncCommit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void CpAsyncWait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory");
}

constexpr int kStagedChunks = 4;
constexpr size_t kStagedMaxSmem = 112 * 1024;   // two blocks per SM

template <int G>
struct StagedShape {
  static constexpr int kThreads = G == 4 ? 64 : 32;
  static constexpr int kRows = (32 / G) * (kThreads / 32);
};

template <int G, bool kLane>
__host__ __device__ inline size_t StagedSmemFloats(size_t K) {
  constexpr int N = 4 * G;
  return StagedShape<G>::kRows * (K + 4) + (kLane ? N * (K + 16) + 16 : K * N);
}

template <int G, bool kLane>
__global__ void __launch_bounds__(StagedShape<G>::kThreads) ReduceStagedKernel(Params p) {
  constexpr int N = 4 * G;
  constexpr int kThreads = StagedShape<G>::kThreads, kRows = StagedShape<G>::kRows;
  constexpr int kRowsPerWarp = 32 / G;
  extern __shared__ __align__(16) float smem[];
  const int K = static_cast<int>(p.K);
  const int xs_stride = K + 4, wn_stride = K + 16;
  float* Xs = smem;
  float* Wsm = smem + kRows * xs_stride;
  auto wn_row = [&](int n) { return n * wn_stride + 4 * (n >> 2); };
  const float* B = static_cast<const float*>(p.B);
  const size_t row0 = static_cast<size_t>(blockIdx.x) * kRows;
  const int rows_live = p.M - row0 < static_cast<size_t>(kRows) ? static_cast<int>(p.M - row0) : kRows;
  const int ck = ((K / 16 + kStagedChunks - 1) / kStagedChunks) * 16;   // chunk length, a multiple of 16

  {
    const int sub = threadIdx.x >> 4, seg = threadIdx.x & 15;   // 16 threads copy 256 contiguous bytes
    constexpr int kSubs = kThreads / 16;
    for (int c = 0; c < kStagedChunks; ++c) {
      const int k0 = c * ck;
      const int len = K - k0 < ck ? (K - k0 > 0 ? K - k0 : 0) : ck;
      const int per = len / 4;
      for (int r = sub; r < rows_live; r += kSubs)
        for (int kq = seg; kq < per; kq += 16)
          CpAsync16(&Xs[r * xs_stride + k0 + 4 * kq], p.A + (row0 + r) * p.K + k0 + 4 * kq);
      if (kLane) {
        for (int n = sub; n < N; n += kSubs)
          for (int kq = seg; kq < per; kq += 16)
            CpAsync16(&Wsm[wn_row(n) + k0 + 4 * kq], B + static_cast<size_t>(n) * p.K + k0 + 4 * kq);
      } else {
        for (int i = threadIdx.x; i < per * N; i += kThreads)   // rows k0.. of [K][N]: one contiguous run
          CpAsync16(&Wsm[k0 * N + 4 * i], B + static_cast<size_t>(k0) * N + 4 * i);
      }
      CpAsyncCommit();
    }
  }

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane % G;
  const int slot = warp * kRowsPerWarp + lane / G;
  const bool live = slot < rows_live;
  const float* xs = Xs + slot * xs_stride;
  float c[4];
  float acc[4][8];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    c[j] = 0.0f;
#pragma unroll
    for (int l = 0; l < 8; ++l) acc[j][l] = 0.0f;
  }
  auto chunk = [&](int k0) {
    const int k1 = k0 + ck < K ? k0 + ck : K;
    if (!live) return;
#pragma unroll 2
    for (int k = k0; k < k1; k += 8) {
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int kq = k + 4 * q;
        const float4 x = *reinterpret_cast<const float4*>(xs + kq);
        if (kLane) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float4 w = *reinterpret_cast<const float4*>(&Wsm[wn_row(4 * g + j) + kq]);
            acc[j][4 * q + 0] = acc[j][4 * q + 0] + x.x * w.x;   // product k into accumulator k mod 8
            acc[j][4 * q + 1] = acc[j][4 * q + 1] + x.y * w.y;
            acc[j][4 * q + 2] = acc[j][4 * q + 2] + x.z * w.z;
            acc[j][4 * q + 3] = acc[j][4 * q + 3] + x.w * w.w;
          }
        } else {
          const float4 w0 = *reinterpret_cast<const float4*>(&Wsm[(kq + 0) * N + 4 * g]);
          const float4 w1 = *reinterpret_cast<const float4*>(&Wsm[(kq + 1) * N + 4 * g]);
          const float4 w2 = *reinterpret_cast<const float4*>(&Wsm[(kq + 2) * N + 4 * g]);
          const float4 w3 = *reinterpret_cast<const float4*>(&Wsm[(kq + 3) * N + 4 * g]);
          if (p.alpha == 1.0f)   // 1.0f * x == x: the multiply changes no bit
            QuadStep(c, x.x, x.y, x.z, x.w, w0, w1, w2, w3);
          else
            QuadStep(c, p.alpha * x.x, p.alpha * x.y, p.alpha * x.z, p.alpha * x.w, w0, w1, w2, w3);
        }
      }
    }
  };
  CpAsyncWait<3>(); __syncthreads(); chunk(0);
  CpAsyncWait<2>(); __syncthreads(); chunk(ck);
  CpAsyncWait<1>(); __syncthreads(); chunk(2 * ck);
  CpAsyncWait<0>(); __syncthreads(); chunk(3 * ck);
  static_assert(kStagedChunks == 4, "the waits above are written out for four chunks");
  if (!live) return;

  float v[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (kLane) {
      float s = acc[j][0];
#pragma unroll
      for (int l = 1; l < 8; ++l) s = s + acc[j][l];
      v[j] = p.alpha * s;
    } else {
      v[j] = c[j];
    }
  }
  const size_t o = (row0 + slot) * N + 4 * g;
  if (p.addend) {
    const float4 d = *reinterpret_cast<const float4*>(p.addend + o);
    v[0] = d.x + v[0]; v[1] = d.y + v[1]; v[2] = d.z + v[2]; v[3] = d.w + v[3];
  }
  if (!kLane) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (p.bias) v[j] = v[j] + p.bias[4 * g + j];
      v[j] = ApplyAct(v[j], p.act);
    }
  }
  *reinterpret_cast<float4*>(p.C + o) = make_float4(v[0], v[1], v[2], v[3]);
}

template <int G, bool kLane>
bool LaunchReduceStaged(const Params& p, cudaStream_t s) {
  const size_t smem = StagedSmemFloats<G, kLane>(p.K) * sizeof(float);
  static std::atomic<bool> configured_on[64] = {};   // per instantiation and device
  int dev = 0;
  cudaGetDevice(&dev);
  const bool tracked = dev >= 0 && dev < 64;
  if (!tracked || !configured_on[dev].load(std::memory_order_acquire)) {
    if (cudaFuncSetAttribute(ReduceStagedKernel<G, kLane>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(kStagedMaxSmem)) != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    if (tracked) configured_on[dev].store(true, std::memory_order_release);
  }
  constexpr int kRows = StagedShape<G>::kRows;
  const unsigned blocks = static_cast<unsigned>((p.M + kRows - 1) / kRows);
  ReduceStagedKernel<G, kLane><<<blocks, StagedShape<G>::kThreads, smem, s>>>(p);
  return true;
}

// Eight-warp streaming blocks when there are enough rows to fill the GPU with
// them; otherwise (a per-GPU batch of a few thousand rows) the staged kernel,
// or two-warp streaming blocks when K is too long for its shared memory.
template <int G, bool kLane>
bool LaunchReduceSized(const Params& p, cudaStream_t s) {
  constexpr int kBigRows = 2 * (32 / G) * 8;
  if ((p.M + kBigRows - 1) / kBigRows >= 148) return LaunchReduceAs<G, kLane, 2, 2, 256>(p, s);
  if (StagedSmemFloats<G, kLane>(p.K) * sizeof(float) <= kStagedMaxSmem) return LaunchReduceStaged<G, kLane>(p, s);
  return LaunchReduceAs<G, kLane, 1, 2, 64>(p, s);
}

template <int G>
bool LaunchReduce(const Params& p, bool lane_order, cudaStream_t s) {
  return lane_order ? LaunchReduceSized<G, true>(p, s) : LaunchReduceSized<G, false>(p, s);
}

}  // namespace

bool SkinnyReduce(const exact::Params& p, bool lane_order, cudaStream_t s) {
  if (p.N != 4 && p.N != 8 && p.N != 16) return false;
  if (p.K < 64 || (p.K & 15) != 0 || p.K > kReduceMaxK || p.M < 256) return false;
  if (p.accumulate || p.b_col_scale || p.a_k_scale || p.partials) return false;
  if (lane_order && (p.bias || p.act != kActNone)) return false;
  if (!Aligned16(p.A) || !Aligned16(p.B) || !Aligned16(p.C) || !Aligned16(p.addend)) return false;
  switch (p.N) {
    case 4: return LaunchReduce<1>(p, lane_order, s);
    case 8: return LaunchReduce<2>(p, lane_order, s);
    default: return LaunchReduce<4>(p, lane_order, s);
  }
}

namespace {

// ---- expand: C[M, N] = addend + A[M, K] * W with K = rank (4..16) ---------------------
// A thread owns four neighbouring columns for kExpandRows consecutive rows and
// keeps its K x 4 slice of W in registers.  The block's rows of A (kExpandRows x
// K floats) are staged in shared memory once and read back as broadcasts.  Rows
// go four at a time: the four 16-byte addend loads are issued before any
// arithmetic, so each thread keeps 64 bytes of the stream in flight.  The kernel
// moves 32 bytes per 2K multiply-adds.
constexpr int kExpandThreads = 64;
constexpr int kExpandRows = 32;
constexpr int kExpandBatch = 4;

template <int K, bool kLane, bool kTail>
__global__ void __launch_bounds__(kExpandThreads) ExpandKernel(Params p) {
  __shared__ __align__(16) float As[kExpandRows][K];
  const size_t r0 = static_cast<size_t>(blockIdx.y) * kExpandRows;
  const int rows = p.M - r0 < static_cast<size_t>(kExpandRows) ? static_cast<int>(p.M - r0) : kExpandRows;
  {
    const float4* src = reinterpret_cast<const float4*>(p.A + r0 * K);
    for (int idx = threadIdx.x; idx < rows * K / 4; idx += kExpandThreads)
      reinterpret_cast<float4*>(&As[0][0])[idx] = src[idx];
  }
  __syncthreads();
  const size_t n = (static_cast<size_t>(blockIdx.x) * kExpandThreads + threadIdx.x) * 4;
  if (n >= p.N) return;
  const float* B = static_cast<const float*>(p.B);
  float w[K][4];
  if (kLane) {  // W is [N, K]
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int kq = 0; kq < K; kq += 4) {
        const float4 t = *reinterpret_cast<const float4*>(B + (n + j) * K + kq);
        w[kq][j] = t.x; w[kq + 1][j] = t.y; w[kq + 2][j] = t.z; w[kq + 3][j] = t.w;
      }
  } else {      // W is [K, N]
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const float4 t = *reinterpret_cast<const float4*>(B + static_cast<size_t>(k) * p.N + n);
      w[k][0] = t.x; w[k][1] = t.y; w[k][2] = t.z; w[k][3] = t.w;
    }
  }
  float bias[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  if (p.bias) {
#pragma unroll
    for (int j = 0; j < 4; ++j) bias[j] = p.bias[n + j];
  }
  for (int mb = 0; mb < rows; mb += kExpandBatch) {
    float4 d[kExpandBatch];
#pragma unroll
    for (int u = 0; u < kExpandBatch; ++u)
      d[u] = (p.addend && mb + u < rows)
                 ? *reinterpret_cast<const float4*>(p.addend + (r0 + mb + u) * p.N + n)
                 : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float4 tail[kTail ? kExpandBatch : 1];   // the absorbed add's other operand, fetched with the addend
    if (kTail) {
#pragma unroll
      for (int u = 0; u < kExpandBatch; ++u)
        tail[kTail ? u : 0] = mb + u < rows
                                  ? *reinterpret_cast<const float4*>(p.tail_addend + (r0 + mb + u) * p.N + n)
                                  : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
#pragma unroll
    for (int u = 0; u < kExpandBatch; ++u) {
      if (mb + u >= rows) break;
      float a[K];
#pragma unroll
      for (int kq = 0; kq < K; kq += 4) {
        const float4 t = *reinterpret_cast<const float4*>(&As[mb + u][kq]);
        a[kq] = t.x; a[kq + 1] = t.y; a[kq + 2] = t.z; a[kq + 3] = t.w;
      }
      float v[4];
      if (kLane) {
        // Product k into accumulator k mod 8, from zero; accumulators summed 0..7.
#pragma unroll
        for (int j = 0; j < 4; j += 2) {   // columns j and j + 1 share each packed add
          unsigned long long acc[8];
#pragma unroll
          for (int l = 0; l < 8; ++l) acc[l] = Pack2(0.0f, 0.0f);
#pragma unroll
          for (int k = 0; k < K; ++k) acc[k & 7] = Add2(acc[k & 7], Pack2(a[k] * w[k][j], a[k] * w[k][j + 1]));
          unsigned long long s = acc[0];
#pragma unroll
          for (int l = 1; l < 8; ++l) s = Add2(s, acc[l]);
          float s0, s1;
          Unpack2(s, &s0, &s1);
          v[j] = p.alpha * s0;
          v[j + 1] = p.alpha * s1;
        }
      } else {
#pragma unroll
        for (int kq = 0; kq < K; ++kq) a[kq] = p.alpha * a[kq];
#pragma unroll
        for (int j = 0; j < 4; j += 2) {   // columns j and j + 1 share each packed add
          unsigned long long c = Pack2(0.0f, 0.0f);
#pragma unroll
          for (int kq = 0; kq < K; kq += 4) {
            unsigned long long t = Pack2(a[kq] * w[kq][j], a[kq] * w[kq][j + 1]);
            t = Add2(t, Pack2(a[kq + 1] * w[kq + 1][j], a[kq + 1] * w[kq + 1][j + 1]));
            t = Add2(t, Pack2(a[kq + 2] * w[kq + 2][j], a[kq + 2] * w[kq + 2][j + 1]));
            t = Add2(t, Pack2(a[kq + 3] * w[kq + 3][j], a[kq + 3] * w[kq + 3][j + 1]));
            c = Add2(c, t);
          }
          Unpack2(c, &v[j], &v[j + 1]);
        }
      }
      if (p.addend) {
        v[0] = d[u].x + v[0]; v[1] = d[u].y + v[1]; v[2] = d[u].z + v[2]; v[3] = d[u].w + v[3];
      }
      if (!kLane) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (p.bias) v[j] = v[j] + bias[j];
          v[j] = ApplyAct(v[j], p.act);
        }
      }
      const size_t at = (r0 + mb + u) * p.N + n;
      if (kTail) {   // the kAddEW that follows, done here (tail_out may alias tail_addend or the addend)
        const float4 t = tail[kTail ? u : 0];
        *reinterpret_cast<float4*>(p.tail_out + at) = make_float4(t.x + v[0], t.y + v[1], t.z + v[2], t.w + v[3]);
      } else {
        *reinterpret_cast<float4*>(p.C + at) = make_float4(v[0], v[1], v[2], v[3]);
      }
    }
  }
}

template <int K>
void LaunchExpand(const Params& p, bool lane_order, cudaStream_t s) {
  const dim3 grid(static_cast<unsigned>((p.N / 4 + kExpandThreads - 1) / kExpandThreads),
                  static_cast<unsigned>((p.M + kExpandRows - 1) / kExpandRows));
  if (p.tail_out) {
    if (lane_order) ExpandKernel<K, true, true><<<grid, kExpandThreads, 0, s>>>(p);
    else ExpandKernel<K, false, true><<<grid, kExpandThreads, 0, s>>>(p);
  } else {
    if (lane_order) ExpandKernel<K, true, false><<<grid, kExpandThreads, 0, s>>>(p);
    else ExpandKernel<K, false, false><<<grid, kExpandThreads, 0, s>>>(p);
  }
}

}  // namespace

bool SkinnyExpand(const exact::Params& p, bool lane_order, cudaStream_t s) {
  if (p.K != 4 && p.K != 8 && p.K != 12 && p.K != 16) return false;
  if ((p.N & 3) != 0 || p.N < 64 || p.M < 64) return false;
  if (p.M > 65535u * static_cast<size_t>(kExpandRows)) return false;
  if (p.accumulate || p.b_col_scale || p.a_k_scale || p.partials) return false;
  if (lane_order && (p.bias || p.act != kActNone)) return false;
  if (!Aligned16(p.A) || !Aligned16(p.B) || !Aligned16(p.C) || !Aligned16(p.addend)) return false;
  switch (p.K) {
    case 4: LaunchExpand<4>(p, lane_order, s); break;
    case 8: LaunchExpand<8>(p, lane_order, s); break;
    case 12: LaunchExpand<12>(p, lane_order, s); break;
    default: LaunchExpand<16>(p, lane_order, s); break;
  }
  return true;
}

namespace {

// ---- transposed-A partials: C = A^T * B over one K chunk, output <= 16 wide or tall ----
// C[i, j] = sum_k (alpha * A[k, i]) * B[k, j].  One operand is `wide` (its rows
// are W floats, streamed once with 8-byte loads), the other `narrow` (rows of
// R floats, R in {4, 8, 12, 16}).  A block takes one chunk of p.k_chunk reduction
// rows and one segment of 2 * kTnThreads wide columns; the chunk's narrow rows
// are staged in shared memory transposed, Ns[r][k], so the four k of a quad
// come back in one 16-byte broadcast load.  Each thread holds the R x 2 partial
// sums of its two wide columns and walks the chunk in quad order, exactly as
// the general kernel does.  Wide rows are fetched sixteen at a time into one of
// two register buffers, the next sixteen in flight while these are consumed.
constexpr int kTnThreads = 128;
constexpr int kTnChunk = 256;
constexpr int kTnStage = 16;
static_assert(kTnChunk == kSplitKChunk, "the staging buffer holds the largest chunk");

template <bool kWideA, int R, int kChunk>
__global__ void __launch_bounds__(kTnThreads) TnPartialKernel(Params p) {
  __shared__ __align__(16) float Ns[R][kChunk + 4];
  const size_t W = kWideA ? p.M : p.N;
  const float* wide = kWideA ? p.A : static_cast<const float*>(p.B);
  const float* narrow = kWideA ? static_cast<const float*>(p.B) : p.A;
  const size_t k0 = static_cast<size_t>(blockIdx.z) * kChunk;   // kChunk == p.k_chunk
  const int len = p.K - k0 < static_cast<size_t>(kChunk) ? static_cast<int>(p.K - k0) : kChunk;
  for (int idx = threadIdx.x; idx < len * R; idx += kTnThreads) {
    const int m = idx / R, r = idx % R;
    const float v = narrow[(k0 + m) * R + r];
    Ns[r][m] = kWideA ? v : p.alpha * v;
  }
  __syncthreads();
  const size_t w0 = (static_cast<size_t>(blockIdx.x) * kTnThreads + threadIdx.x) * 2;
  if (w0 >= W) return;
  float acc[R][2];
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r][0] = acc[r][1] = 0.0f;
  const float* wp = wide + k0 * W + w0;

  auto load = [&](float2 (&buf)[kTnStage], int m0) {
#pragma unroll
    for (int u = 0; u < kTnStage; ++u) {
      buf[u] = m0 + u < len ? *reinterpret_cast<const float2*>(wp + static_cast<size_t>(m0 + u) * W)
                            : make_float2(0.0f, 0.0f);
      if (kWideA) { buf[u].x = p.alpha * buf[u].x; buf[u].y = p.alpha * buf[u].y; }
    }
  };
  auto consume = [&](const float2 (&buf)[kTnStage], int m0) {
#pragma unroll
    for (int q = 0; q < kTnStage / 4; ++q) {
      const int m = m0 + 4 * q;
      if (m + 4 <= len) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const float4 nv = *reinterpret_cast<const float4*>(&Ns[r][m]);
          float t = nv.x * buf[4 * q].x;
          t = t + nv.y * buf[4 * q + 1].x;
          t = t + nv.z * buf[4 * q + 2].x;
          t = t + nv.w * buf[4 * q + 3].x;
          acc[r][0] = acc[r][0] + t;
          float u = nv.x * buf[4 * q].y;
          u = u + nv.y * buf[4 * q + 1].y;
          u = u + nv.z * buf[4 * q + 2].y;
          u = u + nv.w * buf[4 * q + 3].y;
          acc[r][1] = acc[r][1] + u;
        }
      } else {  // the K % 4 tail (last chunk only), one term at a time
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (m + i < len) {
#pragma unroll
            for (int r = 0; r < R; ++r) {
              acc[r][0] = acc[r][0] + Ns[r][m + i] * buf[4 * q + i].x;
              acc[r][1] = acc[r][1] + Ns[r][m + i] * buf[4 * q + i].y;
            }
          }
        }
      }
    }
  };
  float2 buf0[kTnStage], buf1[kTnStage];
  load(buf0, 0);
  for (int m0 = 0; m0 < len; m0 += 2 * kTnStage) {
    if (m0 + kTnStage < len) load(buf1, m0 + kTnStage);
    consume(buf0, m0);
    if (m0 + kTnStage < len) {
      if (m0 + 2 * kTnStage < len) load(buf0, m0 + 2 * kTnStage);
      consume(buf1, m0 + kTnStage);
    }
  }
  float* out = p.partials + static_cast<size_t>(blockIdx.z) * p.M * p.N;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    if (kWideA) {
      out[w0 * p.N + r] = acc[r][0];
      out[(w0 + 1) * p.N + r] = acc[r][1];
    } else {
      *reinterpret_cast<float2*>(out + static_cast<size_t>(r) * p.N + w0) =
          make_float2(acc[r][0], acc[r][1]);
    }
  }
}

template <bool kWideA, int kChunk>
bool LaunchTnChunk(const Params& p, int R, dim3 grid, cudaStream_t s) {
  switch (R) {
    case 4: TnPartialKernel<kWideA, 4, kChunk><<<grid, kTnThreads, 0, s>>>(p); return true;
    case 8: TnPartialKernel<kWideA, 8, kChunk><<<grid, kTnThreads, 0, s>>>(p); return true;
    case 12: TnPartialKernel<kWideA, 12, kChunk><<<grid, kTnThreads, 0, s>>>(p); return true;
    case 16: TnPartialKernel<kWideA, 16, kChunk><<<grid, kTnThreads, 0, s>>>(p); return true;
    default: return false;
  }
}

template <bool kWideA>
bool LaunchTn(const Params& p, int R, dim3 grid, cudaStream_t s) {
  switch (p.k_chunk) {
    case 256: return LaunchTnChunk<kWideA, 256>(p, R, grid, s);
    case 128: return LaunchTnChunk<kWideA, 128>(p, R, grid, s);
    case 64: return LaunchTnChunk<kWideA, 64>(p, R, grid, s);
    case 32: return LaunchTnChunk<kWideA, 32>(p, R, grid, s);
    default: return false;
  }
}

}  // namespace

bool SkinnyTnPartials(const exact::Params& p, size_t chunks, cudaStream_t s) {
  if (p.k_chunk == 0 || p.k_chunk > static_cast<size_t>(kTnChunk) || (p.k_chunk & 15) != 0 ||
      !p.partials || chunks > 65535)
    return false;
  const bool wide_a = p.N <= 16;
  if (!wide_a && p.M > 16) return false;
  const size_t W = wide_a ? p.M : p.N;
  const int R = static_cast<int>(wide_a ? p.N : p.M);
  if ((W & 1) != 0 || W < 64) return false;
  const void* wide = wide_a ? static_cast<const void*>(p.A) : p.B;
  if ((reinterpret_cast<uintptr_t>(wide) & 7) != 0 || (reinterpret_cast<uintptr_t>(p.partials) & 7) != 0)
    return false;
  const dim3 grid(static_cast<unsigned>((W / 2 + kTnThreads - 1) / kTnThreads), 1,
                  static_cast<unsigned>(chunks));
  return wide_a ? LaunchTn<true>(p, R, grid, s) : LaunchTn<false>(p, R, grid, s);
}

}  // namespace see::k::SEE_SKINNY_NAMESPACE
