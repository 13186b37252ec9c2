// Elementwise, broadcast and gather kernels.  HBM-bound: float4 accesses on a
// grid-stride loop sized to the SM count, scalar path for unaligned operands.
// Compiled with -fmad=false: every expression below rounds exactly as the
// reference's x86 build does (one rounding per written operation), so the
// add / mul / bias / scale / relu / accumulate / fill / copy / gather results
// are bit-identical to the CPU executor's; tanh / exp based activations agree
// to libm-vs-CUDA-libm differences (a few ulp).
#include "act_expr.cuh"
#include "kernels.h"
#include "shadow.cuh"

namespace see::k {

namespace {

constexpr int kThreads = 256;
constexpr int kSmCount = 148;
constexpr int kMaxBlocks = kSmCount * 8;

inline int BlocksFor(size_t work_items) {
  size_t b = (work_items + kThreads - 1) / kThreads;
  if (b < 1) b = 1;
  if (b > static_cast<size_t>(kMaxBlocks)) b = kMaxBlocks;
  return static_cast<int>(b);
}

inline bool Aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ---- generic maps -------------------------------------------------------------
template <typename F>
__global__ void Map1(const float* __restrict__ x, float* __restrict__ out, size_t n, bool vec, F f,
                     Shadow sh) {
  const size_t tid = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  if (vec) {
    const size_t n4 = n / 4;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    float4* o4 = reinterpret_cast<float4*>(out);
    ShadowCursor cur(sh, tid, stride);
    for (size_t i = tid; i < n4; i += stride) {
      float4 a = x4[i];
      a.x = f(a.x); a.y = f(a.y); a.z = f(a.z); a.w = f(a.w);
      o4[i] = a;
      if (sh.dst) { ShadowStore4(sh, i, cur.col(), a); cur.advance(); }
    }
    for (size_t i = n4 * 4 + tid; i < n; i += stride) out[i] = f(x[i]);
  } else {
    for (size_t i = tid; i < n; i += stride) out[i] = f(x[i]);
  }
}

// out may alias x or y exactly (in-place accumulate); never partially.
template <typename F>
__global__ void Map2(const float* x, const float* y, float* out, size_t n, bool vec, F f, Shadow sh) {
  const size_t tid = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  if (vec) {
    const size_t n4 = n / 4;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    const float4* y4 = reinterpret_cast<const float4*>(y);
    float4* o4 = reinterpret_cast<float4*>(out);
    ShadowCursor cur(sh, tid, stride);
    for (size_t i = tid; i < n4; i += stride) {
      const float4 a = x4[i], b = y4[i];
      float4 r;
      r.x = f(a.x, b.x); r.y = f(a.y, b.y); r.z = f(a.z, b.z); r.w = f(a.w, b.w);
      o4[i] = r;
      if (sh.dst) { ShadowStore4(sh, i, cur.col(), r); cur.advance(); }
    }
    for (size_t i = n4 * 4 + tid; i < n; i += stride) out[i] = f(x[i], y[i]);
  } else {
    for (size_t i = tid; i < n; i += stride) out[i] = f(x[i], y[i]);
  }
}

struct AddF { __device__ float operator()(float a, float b) const { return a + b; } };
struct MulF { __device__ float operator()(float a, float b) const { return a * b; } };
struct ScaleF { float alpha; __device__ float operator()(float a) const { return alpha * a; } };
struct IdF { __device__ float operator()(float a) const { return a; } };
struct ReluF { __device__ float operator()(float a) const { return ReluExpr(a); } };
struct GeluF { __device__ float operator()(float a) const { return GeluExpr(a); } };
struct SiluF { __device__ float operator()(float a) const { return SiluExpr(a); } };
struct ReluBwdF { __device__ float operator()(float dy, float x) const { return ReluGrad(dy, x); } };
struct GeluBwdF { __device__ float operator()(float dy, float x) const { return GeluGrad(dy, x); } };
struct SiluBwdF { __device__ float operator()(float dy, float x) const { return SiluGrad(dy, x); } };

template <typename F>
bool LaunchMap1(const float* x, float* out, size_t n, cudaStream_t s, F f,
                const Shadow* shadow = nullptr) {
  if (n == 0) return false;
  const bool vec = Aligned16(x) && Aligned16(out);
  const bool shadowed = vec && ShadowUsable(shadow, out, n);
  Map1<<<BlocksFor(vec ? (n + 3) / 4 : n), kThreads, 0, s>>>(x, out, n, vec, f,
                                                              shadowed ? *shadow : Shadow{});
  return shadowed;
}
template <typename F>
bool LaunchMap2(const float* x, const float* y, float* out, size_t n, cudaStream_t s, F f,
                const Shadow* shadow = nullptr) {
  if (n == 0) return false;
  const bool vec = Aligned16(x) && Aligned16(y) && Aligned16(out);
  const bool shadowed = vec && ShadowUsable(shadow, out, n);
  Map2<<<BlocksFor(vec ? (n + 3) / 4 : n), kThreads, 0, s>>>(x, y, out, n, vec, f,
                                                              shadowed ? *shadow : Shadow{});
  return shadowed;
}

__global__ void FillKernel(float* __restrict__ dst, float value, size_t n, bool vec) {
  const size_t tid = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  if (vec) {
    const size_t n4 = n / 4;
    float4* d4 = reinterpret_cast<float4*>(dst);
    const float4 v = make_float4(value, value, value, value);
    for (size_t i = tid; i < n4; i += stride) d4[i] = v;
    for (size_t i = n4 * 4 + tid; i < n; i += stride) dst[i] = value;
  } else {
    for (size_t i = tid; i < n; i += stride) dst[i] = value;
  }
}

// out[r, c] = x[r, c] + b[c]   (reference: runtime/executor/elementwise.cc:28-36)
__global__ void AddBiasKernel(const float* __restrict__ x, const float* __restrict__ b,
                              float* __restrict__ out, size_t rows, size_t cols, bool vec) {
  const size_t tid = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  if (vec) {  // cols % 4 == 0
    const size_t c4 = cols / 4, n4 = rows * c4;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    const float4* b4 = reinterpret_cast<const float4*>(b);
    float4* o4 = reinterpret_cast<float4*>(out);
    for (size_t i = tid; i < n4; i += stride) {
      const float4 a = x4[i], bb = b4[i % c4];
      o4[i] = make_float4(a.x + bb.x, a.y + bb.y, a.z + bb.z, a.w + bb.w);
    }
  } else {
    const size_t n = rows * cols;
    for (size_t i = tid; i < n; i += stride) out[i] = x[i] + b[i % cols];
  }
}

// The fused chain: up to four stages over a running value, each stage one
// separately rounded expression (reference: runtime/executor/elementwise.cc:59-149).
__device__ __forceinline__ float RunStages(float v, float y1, float y2, uint32_t stages,
                                           float imm0, float imm1) {
#pragma unroll
  for (int sidx = 0; sidx < 4; ++sidx) {
    const uint32_t st = (stages >> (8 * sidx)) & 0xFF;
    const uint32_t kind = st & 0x0F;
    if (kind == kFEnd) break;
    const uint32_t arg = (st >> 4) & 3;
    // IEEE add and mul commute in value; operand order only selects a NaN payload.
    const float other = arg == 1 ? y1 : y2;
    switch (kind) {
      case kFAdd: v = (st & 0x80) ? other + v : v + other; break;
      case kFMul: v = (st & 0x80) ? other * v : v * other; break;
      case kFScale: v = (arg == 0 ? imm0 : imm1) * v; break;
      case kFRelu: v = ReluExpr(v); break;
      case kFGelu: v = GeluExpr(v); break;
      case kFSilu: v = SiluExpr(v); break;
      default: break;
    }
  }
  return v;
}

__global__ void FusedMapKernel(const float* __restrict__ x, const float* __restrict__ o1,
                               const float* __restrict__ o2, float* __restrict__ out, size_t n,
                               uint32_t stages, float imm0, float imm1) {
  const size_t tid = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = tid; i < n; i += stride) {
    const float y1 = o1 ? o1[i] : 0.0f;
    const float y2 = o2 ? o2[i] : 0.0f;
    out[i] = RunStages(x[i], y1, y2, stages, imm0, imm1);
  }
}

// out[t, :] = table[tokens[t], :]; a token outside [0, vocab) writes zeros
// rather than reading outside the table (the reference leaves that bound to
// its data feeder; the device must not fault on a bad id).
__global__ void EmbedKernel(const int32_t* __restrict__ tokens, const float* __restrict__ table,
                            float* __restrict__ out, size_t rows, size_t dim, size_t vocab,
                            bool vec) {
  const size_t tid = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  if (vec) {
    const size_t d4 = dim / 4, n4 = rows * d4;
    const float4* t4 = reinterpret_cast<const float4*>(table);
    float4* o4 = reinterpret_cast<float4*>(out);
    for (size_t i = tid; i < n4; i += stride) {
      const size_t r = i / d4, c = i % d4;
      const int32_t tok = tokens[r];
      o4[i] = (tok >= 0 && static_cast<size_t>(tok) < vocab)
                  ? t4[static_cast<size_t>(tok) * d4 + c]
                  : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  } else {
    const size_t n = rows * dim;
    for (size_t i = tid; i < n; i += stride) {
      const size_t r = i / dim, c = i % dim;
      const int32_t tok = tokens[r];
      out[i] = (tok >= 0 && static_cast<size_t>(tok) < vocab)
                   ? table[static_cast<size_t>(tok) * dim + c] : 0.0f;
    }
  }
}

// db[c] = sum over rows of dy[r, c], rows in order (reference:
// runtime/executor/elementwise.cc:162-187): one thread per column.
__global__ void ReduceRowsKernel(const float* __restrict__ dy, float* __restrict__ db,
                                 size_t rows, size_t cols) {
  const size_t c = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (c >= cols) return;
  float acc = 0.0f;
  for (size_t r = 0; r < rows; ++r) acc += dy[r * cols + c];
  db[c] = acc;
}

// starts[b, t] = one past the last EOS strictly before t (reference:
// runtime/executor/attention.cc:176-185): integer, bit-exact.
__global__ void SegmentStartsKernel(const int32_t* __restrict__ tokens,
                                    int32_t* __restrict__ starts, size_t B, size_t S,
                                    int32_t eos) {
  const size_t b = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (b >= B) return;
  int32_t start = 0;
  for (size_t t = 0; t < S; ++t) {
    starts[b * S + t] = start;
    if (tokens[b * S + t] == eos) start = static_cast<int32_t>(t + 1);
  }
}

// table[s, c, 0..1] = cos, sin(s * freq_c), freq by the f32 recurrence
// freq *= step (reference: runtime/executor/attention.cc:157-174).
__global__ void RopeTableKernel(float* __restrict__ table, size_t S, size_t half, float step) {
  const size_t s = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (s >= S) return;
  float* row = table + s * half * 2;
  float freq = 1.0f;
  for (size_t c = 0; c < half; ++c) {
    const float theta = static_cast<float>(s) * freq;
    row[2 * c] = cosf(theta);
    row[2 * c + 1] = sinf(theta);
    freq *= step;
  }
}

// Rotation of interleaved pairs within each head (reference:
// runtime/executor/attention.cc:103-155); one thread per (row, head).
template <bool kBackward>
__global__ void RopeKernel(const float* __restrict__ x, float* __restrict__ y, size_t units,
                           size_t S, size_t H, size_t d, float step,
                           const float* __restrict__ table) {
  const size_t u = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (u >= units) return;
  const size_t D = H * d, half = d / 2;
  const size_t s = (u / H) % S;
  const float* xr = x + (u / H) * D + (u % H) * d;
  float* yr = y + (u / H) * D + (u % H) * d;
  const float* row = table ? table + s * half * 2 : nullptr;
  float freq = 1.0f;
  for (size_t c = 0; c + 1 < d; c += 2) {
    float cs, sn;
    if (row) {
      cs = row[c];
      sn = row[c + 1];
    } else {
      const float theta = static_cast<float>(s) * freq;
      cs = cosf(theta);
      sn = sinf(theta);
      freq *= step;
    }
    const float a = xr[c], b2 = xr[c + 1];
    if (kBackward) {
      yr[c] = a * cs + b2 * sn;
      yr[c + 1] = -a * sn + b2 * cs;
    } else {
      yr[c] = a * cs - b2 * sn;
      yr[c + 1] = a * sn + b2 * cs;
    }
  }
}

__device__ __forceinline__ uint16_t Bf16Rne(float f) { return static_cast<uint16_t>(ShadowBf16(f)); }

__global__ void ToBf16Kernel(const float* __restrict__ x, uint16_t* __restrict__ out, size_t rows,
                             size_t cols, const float* __restrict__ col_scale, bool vec) {
  const size_t tid = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  const size_t n = rows * cols;
  if (vec) {  // cols % 4 == 0 and every pointer aligned for its vector type
    const float4* x4 = reinterpret_cast<const float4*>(x);
    uint2* o2 = reinterpret_cast<uint2*>(out);
    const size_t c4 = cols / 4;
    for (size_t i = tid; i < n / 4; i += stride) {
      float4 a = x4[i];
      if (col_scale) {
        const float4 sc = reinterpret_cast<const float4*>(col_scale)[i % c4];
        a.x *= sc.x; a.y *= sc.y; a.z *= sc.z; a.w *= sc.w;
      }
      uint2 r;
      r.x = ShadowBf16x2(a.x, a.y);
      r.y = ShadowBf16x2(a.z, a.w);
      o2[i] = r;
    }
  } else {
    for (size_t i = tid; i < n; i += stride) {
      float a = x[i];
      if (col_scale) a *= col_scale[i % cols];
      out[i] = Bf16Rne(a);
    }
  }
}

}  // namespace

bool AddEW(const float* x, const float* y, float* out, size_t n, cudaStream_t s,
           const Shadow* shadow) {
  return LaunchMap2(x, y, out, n, s, AddF{}, shadow);
}
void MulEW(const float* x, const float* y, float* out, size_t n, cudaStream_t s) {
  LaunchMap2(x, y, out, n, s, MulF{});
}
void Accumulate(float* dst, const float* src, size_t n, cudaStream_t s) {
  LaunchMap2(dst, src, dst, n, s, AddF{});
}
void Scale(const float* x, float* out, float alpha, size_t n, cudaStream_t s) {
  LaunchMap1(x, out, n, s, ScaleF{alpha});
}
void Copy(const float* src, float* dst, size_t n, cudaStream_t s) {
  LaunchMap1(src, dst, n, s, IdF{});
}
void Fill(float* dst, float value, size_t n, cudaStream_t s) {
  if (n == 0) return;
  const bool vec = Aligned16(dst);
  FillKernel<<<BlocksFor(vec ? (n + 3) / 4 : n), kThreads, 0, s>>>(dst, value, n, vec);
}
void AddBias(const float* x, const float* b, float* out, size_t rows, size_t cols,
             cudaStream_t s) {
  if (rows * cols == 0) return;
  const bool vec = (cols % 4 == 0) && Aligned16(x) && Aligned16(b) && Aligned16(out);
  AddBiasKernel<<<BlocksFor(vec ? rows * cols / 4 : rows * cols), kThreads, 0, s>>>(
      x, b, out, rows, cols, vec);
}
bool ActFwd(Act act, const float* x, float* out, size_t n, cudaStream_t s, const Shadow* shadow) {
  switch (act) {
    case kActRelu: return LaunchMap1(x, out, n, s, ReluF{}, shadow);
    case kActGelu: return LaunchMap1(x, out, n, s, GeluF{}, shadow);
    case kActSilu: return LaunchMap1(x, out, n, s, SiluF{}, shadow);
    case kActNone: return LaunchMap1(x, out, n, s, IdF{}, shadow);
  }
  return false;
}
bool ActBwd(Act act, const float* dy, const float* x, float* dx, size_t n, cudaStream_t s,
            const Shadow* shadow) {
  switch (act) {
    case kActRelu: return LaunchMap2(dy, x, dx, n, s, ReluBwdF{}, shadow);
    case kActGelu: return LaunchMap2(dy, x, dx, n, s, GeluBwdF{}, shadow);
    case kActSilu: return LaunchMap2(dy, x, dx, n, s, SiluBwdF{}, shadow);
    case kActNone: break;
  }
  return false;
}
void FusedMap(const float* x, const float* o1, const float* o2, float* out, size_t n,
              uint32_t stages, float imm0, float imm1, cudaStream_t s) {
  if (n == 0) return;
  FusedMapKernel<<<BlocksFor(n), kThreads, 0, s>>>(x, o1, o2, out, n, stages, imm0, imm1);
}
void EmbedFwd(const int32_t* tokens, const float* table, float* out, size_t rows, size_t dim,
              size_t vocab, cudaStream_t s) {
  if (rows * dim == 0) return;
  const bool vec = (dim % 4 == 0) && Aligned16(table) && Aligned16(out);
  EmbedKernel<<<BlocksFor(vec ? rows * dim / 4 : rows * dim), kThreads, 0, s>>>(
      tokens, table, out, rows, dim, vocab, vec);
}
void ReduceRows(const float* dy, float* db, size_t rows, size_t cols, cudaStream_t s) {
  if (cols == 0) return;
  ReduceRowsKernel<<<static_cast<unsigned>((cols + 127) / 128), 128, 0, s>>>(dy, db, rows, cols);
}
void SegmentStarts(const int32_t* tokens, int32_t* starts, size_t B, size_t S, int32_t eos,
                   cudaStream_t s) {
  if (B == 0) return;
  SegmentStartsKernel<<<static_cast<unsigned>((B + 63) / 64), 64, 0, s>>>(tokens, starts, B, S, eos);
}
void RopeTable(float* table, size_t S, size_t d, float step, cudaStream_t s) {
  if (S == 0) return;
  RopeTableKernel<<<static_cast<unsigned>((S + 127) / 128), 128, 0, s>>>(table, S, d / 2, step);
}
void Rope(bool backward, const float* x, float* y, size_t B, size_t S, size_t H, size_t d,
          float step, const float* table, cudaStream_t s) {
  const size_t units = B * S * H;
  if (units == 0) return;
  const unsigned blocks = static_cast<unsigned>((units + 127) / 128);
  if (backward)
    RopeKernel<true><<<blocks, 128, 0, s>>>(x, y, units, S, H, d, step, table);
  else
    RopeKernel<false><<<blocks, 128, 0, s>>>(x, y, units, S, H, d, step, table);
}
void ToBf16(const float* x, uint16_t* out, size_t rows, size_t cols, const float* col_scale,
            cudaStream_t s) {
  if (rows * cols == 0) return;
  const bool vec = (cols % 4 == 0) && Aligned16(x) &&
                   (reinterpret_cast<uintptr_t>(out) & 7) == 0 &&
                   (!col_scale || Aligned16(col_scale));
  ToBf16Kernel<<<BlocksFor((rows * cols + 3) / 4), kThreads, 0, s>>>(x, out, rows, cols, col_scale,
                                                                     vec);
}

}  // namespace see::k
