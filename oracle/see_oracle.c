/* TEST INFRASTRUCTURE — a plain-C restatement of the reference CPU executor's
 * arithmetic, used only as a checker by tests, the smoke check and the bench's
 * CPU-baseline leg.  Nothing the product ships calls into this file.
 *
 * Parity is PINNED: tests/test_oracle_pinned.py holds this restatement bit for
 * bit to (a) the write traces the reference's own probe produced for eight
 * plans compiled by the reference compiler (tests/golden), and (b) the
 * reference executor itself (oracle/_ref) on seeded instruction programs, and
 * to the reference's known-answer vectors (tests/test_oracle_known_answers.py).
 *
 * Everything is serial; reductions that the reference folds per parallel chunk
 * are folded here in the same shape-derived chunk geometry, so the bits do not
 * depend on a thread count on either side.  Build: -O2 -ffp-contract=off (no
 * fused multiply-add may appear; the reference's x86 build has none).
 *
 * Each function cites the reference lines it follows.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

typedef struct {
  uint16_t opcode, flags;
  uint32_t imm;
  uint64_t in[4];
  uint64_t out[3];
} __attribute__((packed)) Instr;

typedef struct {
  float lr, beta1, beta2, eps, weight_decay;
  uint32_t pad;
  uint64_t step;
} StepParams;

typedef struct {
  uint8_t* arena;
  const uint8_t* rodata;
  const uint8_t* source;
  char error[256];
} Oracle;

#define RODATA_BIT (1ull << 63)
#define SOURCE_BIT (1ull << 62)
#define NULL_REF (~0ull)
#define MAX_CHUNKS 256u /* source/parallel/parallel_for.h:50 */
#define GRAIN_CHEAP 32768u /* runtime/executor/kernel_policy.h:42 */
#define GRAIN_MATH 4096u   /* runtime/executor/kernel_policy.h:43 */

enum { FLAG_BIAS = 1, FLAG_ACT_SHIFT = 1, FLAG_ACT_MASK = 6, FLAG_ADDEND = 8, FLAG_COLSCALE = 16 };

/* ---- reference decoding: runtime/executor/cpu_backend.cc:221-240 ------------ */
static const void* rd(const Oracle* o, uint64_t ref) {
  const uint64_t off = ref & ~(RODATA_BIT | SOURCE_BIT);
  if (ref & RODATA_BIT) return o->rodata + off;
  if (ref & SOURCE_BIT) return o->source + off;
  return o->arena + off;
}
static void* wr(const Oracle* o, uint64_t ref) { return o->arena + (ref & ~(RODATA_BIT | SOURCE_BIT)); }
static float bits_f32(uint64_t b) { uint32_t u = (uint32_t)b; float f; memcpy(&f, &u, 4); return f; }

/* ---- chunk geometry: source/parallel/parallel_for.h:55-67, kernel_policy.h:46-48 */
static size_t row_grain(size_t per_row, size_t budget) {
  return per_row == 0 ? budget : (budget / per_row > 0 ? budget / per_row : 1);
}
static size_t chunk_grain(size_t n, size_t grain) {
  if (grain == 0) grain = 1;
  const size_t cap = (n + MAX_CHUNKS - 1) / MAX_CHUNKS;
  return grain < cap ? cap : grain;
}

/* ---- activation expressions: runtime/executor/kernel_policy.h:122-136 --------- */
static const float kGeluC = 0.7978845608028654f;
static const float kGeluA = 0.044715f;
static float sigmoid_expr(float x) { return 1.0f / (1.0f + expf(-x)); }
static float relu_expr(float x) { return x > 0.0f ? x : 0.0f; }
static float gelu_expr(float x) {
  const float t = tanhf(kGeluC * (x + kGeluA * x * x * x));
  return 0.5f * x * (1.0f + t);
}
static float silu_expr(float x) { return x * sigmoid_expr(x); }
static float act_expr(int act, float v) {
  switch (act) {
    case 1: return relu_expr(v);
    case 2: return gelu_expr(v);
    case 3: return silu_expr(v);
    default: return v;
  }
}

/* ---- GEMM: runtime/executor/gemm.cc ----------------------------------------------
 * b_type: 0 f32, 1 int8, 2 bf16 (widening exact: source/plan/bf16.h:26-36). */
static float widen(const void* B, int b_type, size_t idx) {
  if (b_type == 1) return (float)((const int8_t*)B)[idx];
  if (b_type == 2) {
    uint32_t u = (uint32_t)((const uint16_t*)B)[idx] << 16;
    float f; memcpy(&f, &u, 4); return f;
  }
  return ((const float*)B)[idx];
}

/* Quad order (gemm.cc:73-187): c += ((a0b0 + a1b1) + a2b2) + a3b3 over k-quads
 * from k = 0, then single terms; alpha folded into each A element, a column
 * scale into each widened B element.  a_t: A is [K, M]. */
static void gemm_quad(const float* A, const void* B, int b_type, float* C, size_t M, size_t N,
                      size_t K, float alpha, int a_t, const float* col_scale, int accumulate) {
  for (size_t m = 0; m < M; ++m) {
    for (size_t n = 0; n < N; ++n) {
      float c = accumulate ? C[m * N + n] : 0.0f;
      size_t k = 0;
      for (; k + 4 <= K; k += 4) {
        float a[4], b[4];
        for (int q = 0; q < 4; ++q) {
          a[q] = alpha * (a_t ? A[(k + q) * M + m] : A[m * K + k + q]);
          b[q] = widen(B, b_type, (k + q) * N + n);
          if (col_scale) b[q] = b[q] * col_scale[n];
        }
        c += a[0] * b[0] + a[1] * b[1] + a[2] * b[2] + a[3] * b[3];
      }
      for (; k < K; ++k) {
        const float a = alpha * (a_t ? A[k * M + m] : A[m * K + k]);
        float b = widen(B, b_type, k * N + n);
        if (col_scale) b = b * col_scale[n];
        c += a * b;
      }
      C[m * N + n] = c;
    }
  }
}

/* Lane order (gemm.cc:346-527): product k into lane k mod 8, lanes summed
 * 0..7, times alpha; a reduction-axis scale multiplies A first (gemm.cc:652-674). */
static void gemm_lane(const float* A, const void* B, int b_type, float* C, size_t M, size_t N,
                      size_t K, float alpha, const float* k_scale) {
  for (size_t m = 0; m < M; ++m) {
    for (size_t n = 0; n < N; ++n) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (size_t k = 0; k < K; ++k) {
        float a = A[m * K + k];
        if (k_scale) a = a * k_scale[k];
        acc[k % 8] += a * widen(B, b_type, n * K + k);
      }
      float s = acc[0];
      for (int l = 1; l < 8; ++l) s += acc[l];
      C[m * N + n] = alpha * s;
    }
  }
}

/* Epilogues (gemm.cc:536-578): addend d + s, then bias, then activation. */
static void gemm_epilogue(float* C, size_t M, size_t N, const float* addend, const float* bias,
                          int act) {
  if (addend)
    for (size_t i = 0; i < M * N; ++i) C[i] = addend[i] + C[i];
  if (bias || act)
    for (size_t m = 0; m < M; ++m)
      for (size_t n = 0; n < N; ++n) {
        const float v = bias ? C[m * N + n] + bias[n] : C[m * N + n];
        C[m * N + n] = act_expr(act, v);
      }
}

/* ---- normalization: runtime/executor/normalization.cc:17-113 ------------------- */
static void layernorm_fwd(const float* x, const float* gamma, const float* beta, float* y,
                          float* mean, float* rstd, size_t rows, size_t cols, float eps) {
  for (size_t r = 0; r < rows; ++r) {
    const float* xr = x + r * cols;
    double sum = 0.0;
    for (size_t c = 0; c < cols; ++c) sum += xr[c];
    const float mu = (float)(sum / (double)cols);
    double var = 0.0;
    for (size_t c = 0; c < cols; ++c) {
      const double d = (double)xr[c] - mu;
      var += d * d;
    }
    const float rs = 1.0f / sqrtf((float)(var / (double)cols) + eps);
    mean[r] = mu;
    rstd[r] = rs;
    float* yr = y + r * cols;
    for (size_t c = 0; c < cols; ++c) yr[c] = (xr[c] - mu) * rs * gamma[c] + beta[c];
  }
}
static void layernorm_bwd(const float* dy, const float* x, const float* gamma, const float* mean,
                          const float* rstd, float* dx, size_t rows, size_t cols) {
  const float inv_d = 1.0f / (float)cols;
  for (size_t r = 0; r < rows; ++r) {
    const float* dyr = dy + r * cols;
    const float* xr = x + r * cols;
    float* dxr = dx + r * cols;
    const float mu = mean[r], rs = rstd[r];
    double sum_g = 0.0, sum_gx = 0.0;
    for (size_t c = 0; c < cols; ++c) {
      const float xhat = (xr[c] - mu) * rs;
      const float g = dyr[c] * gamma[c];
      sum_g += g;
      sum_gx += (double)g * xhat;
    }
    const float mg = (float)sum_g * inv_d;
    const float mgx = (float)sum_gx * inv_d;
    for (size_t c = 0; c < cols; ++c) {
      const float xhat = (xr[c] - mu) * rs;
      const float g = dyr[c] * gamma[c];
      dxr[c] = rs * (g - mg - xhat * mgx);
    }
  }
}
static void rmsnorm_fwd(const float* x, const float* gamma, float* y, float* rstd, size_t rows,
                        size_t cols, float eps) {
  for (size_t r = 0; r < rows; ++r) {
    const float* xr = x + r * cols;
    double ss = 0.0;
    for (size_t c = 0; c < cols; ++c) ss += (double)xr[c] * xr[c];
    const float rs = 1.0f / sqrtf((float)(ss / (double)cols) + eps);
    rstd[r] = rs;
    float* yr = y + r * cols;
    for (size_t c = 0; c < cols; ++c) yr[c] = xr[c] * rs * gamma[c];
  }
}
static void rmsnorm_bwd(const float* dy, const float* x, const float* gamma, const float* rstd,
                        float* dx, size_t rows, size_t cols) {
  const float inv_d = 1.0f / (float)cols;
  for (size_t r = 0; r < rows; ++r) {
    const float* dyr = dy + r * cols;
    const float* xr = x + r * cols;
    float* dxr = dx + r * cols;
    const float rs = rstd[r];
    double sum_gx = 0.0;
    for (size_t c = 0; c < cols; ++c) sum_gx += (double)(dyr[c] * gamma[c]) * xr[c];
    const float mgx = (float)sum_gx * inv_d;
    for (size_t c = 0; c < cols; ++c) dxr[c] = rs * (dyr[c] * gamma[c] - xr[c] * rs * rs * mgx);
  }
}

/* ---- losses: runtime/executor/loss.cc ------------------------------------------- */
static void row_softmax(const float* logits, float* probs, size_t C, float inv_T) { /* :21-31 */
  float max_v = logits[0] * inv_T;
  for (size_t c = 1; c < C; ++c) max_v = fmaxf(max_v, logits[c] * inv_T);
  float sum = 0.0f;
  for (size_t c = 0; c < C; ++c) {
    probs[c] = expf(logits[c] * inv_T - max_v);
    sum += probs[c];
  }
  const float inv_sum = 1.0f / sum;
  for (size_t c = 0; c < C; ++c) probs[c] *= inv_sum;
}
static double neg_log_safe(float p) { /* :44-51 */
  const double safe = isnan(p) ? (double)p : (double)fmaxf(p, 1e-12f);
  return log(safe);
}
static void xent_fwd(int masked, const float* logits, const int32_t* labels, float* loss,
                     float* probs, size_t N, size_t C) { /* :35-57, :74-105 */
  const size_t grain = chunk_grain(N, row_grain(C, GRAIN_MATH));
  double total = 0.0;
  uint64_t T = 0;
  for (size_t r0 = 0; r0 < N; r0 += grain) {
    const size_t r1 = r0 + grain < N ? r0 + grain : N;
    double part = 0.0;
    for (size_t n = r0; n < r1; ++n) {
      row_softmax(logits + n * C, probs + n * C, C, 1.0f);
      if (masked && labels[n] < 0) continue;
      part -= neg_log_safe(probs[n * C + (size_t)labels[n]]);
      ++T;
    }
    total += part;
  }
  if (masked) *loss = T ? (float)(total / (double)T) : 0.0f;
  else *loss = (float)(total / (double)N);
}
static void xent_bwd(int masked, const float* probs, const int32_t* labels, const float* seed,
                     float* dlogits, size_t N, size_t C) { /* :59-72, :107-126 */
  float scale;
  if (masked) {
    uint64_t T = 0;
    for (size_t n = 0; n < N; ++n) T += labels[n] >= 0;
    scale = T ? *seed / (float)T : 0.0f;
  } else {
    scale = *seed / (float)N;
  }
  for (size_t n = 0; n < N; ++n) {
    if (masked && labels[n] < 0) {
      for (size_t c = 0; c < C; ++c) dlogits[n * C + c] = 0.0f;
      continue;
    }
    for (size_t c = 0; c < C; ++c) dlogits[n * C + c] = scale * probs[n * C + c];
    dlogits[n * C + (size_t)labels[n]] -= scale;
  }
}
static void mse_fwd(const float* pred, const float* target, float* loss, size_t n) { /* :128-145 */
  const size_t grain = chunk_grain(n, GRAIN_CHEAP);
  double total = 0.0;
  for (size_t b = 0; b < n; b += grain) {
    const size_t e = b + grain < n ? b + grain : n;
    double part = 0.0;
    for (size_t i = b; i < e; ++i) {
      const double d = (double)pred[i] - target[i];
      part += d * d;
    }
    total += part;
  }
  *loss = (float)(total / (double)n);
}
static void mse_bwd(const float* pred, const float* target, const float* seed, float* dpred,
                    size_t n) { /* :147-153 */
  const float scale = 2.0f * *seed / (float)n;
  for (size_t i = 0; i < n; ++i) dpred[i] = scale * (pred[i] - target[i]);
}
static void kl_fwd(const float* s_logits, const float* t_logits, float* loss, float* p_s,
                   float* p_t, size_t N, size_t C, float T, float loss_scale) { /* :155-190 */
  const float inv_T = 1.0f / T;
  const size_t grain = chunk_grain(N, row_grain(C, GRAIN_MATH));
  double total = 0.0;
  for (size_t r0 = 0; r0 < N; r0 += grain) {
    const size_t r1 = r0 + grain < N ? r0 + grain : N;
    double part = 0.0;
    for (size_t n = r0; n < r1; ++n) {
      row_softmax(s_logits + n * C, p_s + n * C, C, inv_T);
      row_softmax(t_logits + n * C, p_t + n * C, C, inv_T);
      for (size_t c = 0; c < C; ++c) {
        const float pt = p_t[n * C + c];
        if (pt <= 0.0f) continue;
        const float ps_raw = p_s[n * C + c];
        const double ps = isnan(ps_raw) ? (double)ps_raw : (double)fmaxf(ps_raw, 1e-12f);
        part += (double)pt * (log((double)pt) - log(ps));
      }
    }
    total += part;
  }
  *loss = (float)(total / (double)N) * loss_scale;
}
static void kl_bwd(const float* p_s, const float* p_t, const float* seed, float* dlogits,
                   size_t N, size_t C, float T, float loss_scale) { /* :192-200 */
  const float scale = (*seed * loss_scale) / ((float)N * T);
  for (size_t i = 0; i < N * C; ++i) dlogits[i] = scale * (p_s[i] - p_t[i]);
}

/* ---- optimizer: runtime/executor/optimizer.cc -------------------------------------- */
static double l2_squared(const float* g, size_t n) { /* :22-35 */
  const size_t grain = chunk_grain(n, GRAIN_CHEAP);
  double sq = 0.0;
  for (size_t b = 0; b < n; b += grain) {
    const size_t e = b + grain < n ? b + grain : n;
    double part = 0.0;
    for (size_t i = b; i < e; ++i) part += (double)g[i] * (double)g[i];
    sq += part;
  }
  return sq;
}
static int clip_scale(const float* g, size_t n, float max_norm, float* scale) { /* :42-50 */
  *scale = 1.0f;
  if (!(max_norm > 0.0f)) return 1;
  const double norm = sqrt(l2_squared(g, n));
  if (!isfinite(norm)) return 0;
  if (norm <= (double)max_norm || norm == 0.0) return 1;
  *scale = (float)((double)max_norm / norm);
  return 1;
}
static int clip_norm(float* g, size_t n, float max_norm) { /* :54-64 */
  if (!isfinite(max_norm) || !(max_norm > 0.0f)) return 0;
  const double norm = sqrt(l2_squared(g, n));
  if (!isfinite(norm)) return 0;
  if (norm <= (double)max_norm || norm == 0.0) return 1;
  const float s = (float)((double)max_norm / norm);
  for (size_t i = 0; i < n; ++i) g[i] *= s;
  return 1;
}
static int clip_global(float* g, size_t n, const float* acc, float max_norm) { /* :70-85 */
  if (!isfinite(max_norm) || !(max_norm > 0.0f)) return 0;
  const double norm = sqrt((double)acc[0]);
  if (!isfinite(norm)) return 0;
  if (norm <= (double)max_norm || norm == 0.0) return 1;
  const float s = (float)((double)max_norm / norm);
  for (size_t i = 0; i < n; ++i) g[i] *= s;
  return 1;
}
static int sgd_step(float* p, const float* g, size_t n, float lr, float wd, float clip) { /* :91-102 */
  float s = 1.0f;
  if (!clip_scale(g, n, clip, &s)) return 0;
  for (size_t i = 0; i < n; ++i) {
    const float gi = g[i] * s;
    p[i] -= lr * (gi + wd * p[i]);
  }
  return 1;
}
static int adamw_step(float* p, const float* g, float* m, float* v, size_t n, const StepParams* sp,
                      float clip) { /* :104-132 */
  float s = 1.0f;
  if (!clip_scale(g, n, clip, &s)) return 0;
  const float inv_bc1 = 1.0f / (1.0f - powf(sp->beta1, (float)sp->step));
  const float inv_bc2 = 1.0f / (1.0f - powf(sp->beta2, (float)sp->step));
  const float om_b1 = 1.0f - sp->beta1;
  const float om_b2 = 1.0f - sp->beta2;
  for (size_t i = 0; i < n; ++i) {
    const float gi = g[i] * s;
    const float mi = sp->beta1 * m[i] + om_b1 * gi;
    const float vi = sp->beta2 * v[i] + om_b2 * gi * gi;
    m[i] = mi;
    v[i] = vi;
    const float m_hat = mi * inv_bc1;
    const float v_hat = vi * inv_bc2;
    p[i] -= sp->lr * (m_hat / (sqrtf(v_hat) + sp->eps) + sp->weight_decay * p[i]);
  }
  return 1;
}

/* ---- fused map: runtime/executor/elementwise.cc:59-149 ------------------------------ */
static void fused_map(const float* x, const float* o1, const float* o2, float* out, size_t n,
                      uint64_t stages, float imm0, float imm1) {
  for (size_t i = 0; i < n; ++i) {
    float v = x[i];
    for (int s = 0; s < 4; ++s) {
      const uint8_t st = (uint8_t)(stages >> (8 * s));
      const int kind = st & 0x0F, arg = (st >> 4) & 3;
      if (kind == 0) break;
      const float other = arg == 1 ? (o1 ? o1[i] : 0.0f) : (o2 ? o2[i] : 0.0f);
      switch (kind) {
        case 1: v = (st & 0x80) ? other + v : v + other; break;
        case 2: v = (st & 0x80) ? other * v : v * other; break;
        case 3: v = (arg == 0 ? imm0 : imm1) * v; break;
        case 4: v = relu_expr(v); break;
        case 5: v = gelu_expr(v); break;
        case 6: v = silu_expr(v); break;
        default: break;
      }
    }
    out[i] = v;
  }
}

/* ---- RoPE: runtime/executor/attention.cc:103-174 --------------------------------------- */
static void rope(int backward, const float* x, float* y, size_t B, size_t S, size_t H, size_t d,
                 float base, const float* table) {
  const size_t D = H * d, half = d / 2;
  const float step = powf(base, -2.0f / (float)d);
  for (size_t u = 0; u < B * S * H; ++u) {
    const size_t s = (u / H) % S;
    const float* xr = x + (u / H) * D + (u % H) * d;
    float* yr = y + (u / H) * D + (u % H) * d;
    const float* row = table ? table + s * half * 2 : NULL;
    float freq = 1.0f;
    for (size_t c = 0; c + 1 < d; c += 2) {
      float cs, sn;
      if (row) { cs = row[c]; sn = row[c + 1]; }
      else {
        const float theta = (float)s * freq;
        cs = cosf(theta); sn = sinf(theta);
        freq *= step;
      }
      const float a = xr[c], b2 = xr[c + 1];
      if (backward) { yr[c] = a * cs + b2 * sn; yr[c + 1] = -a * sn + b2 * cs; }
      else { yr[c] = a * cs - b2 * sn; yr[c + 1] = a * sn + b2 * cs; }
    }
  }
}
static void rope_table(float* table, size_t S, size_t d, float base) {
  const size_t half = d / 2;
  const float step = powf(base, -2.0f / (float)d);
  for (size_t s = 0; s < S; ++s) {
    float* row = table + s * half * 2;
    float freq = 1.0f;
    for (size_t c = 0; c < half; ++c) {
      const float theta = (float)s * freq;
      row[2 * c] = cosf(theta);
      row[2 * c + 1] = sinf(theta);
      freq *= step;
    }
  }
}

/* ---- attention: runtime/executor/attention.cc:187-343 (cached), :448-590 (tiled) ------- */
static double dot_d(const float* a, const float* b, size_t d) {
  double acc = 0.0;
  for (size_t c = 0; c < d; ++c) acc += (double)a[c] * (double)b[c];
  return acc;
}
static size_t stats_start(float stored, size_t i) { /* source/plan/instruction.h:245-249 */
  if (!(stored > 0.0f)) return 0;
  const float cap = (float)i;
  return stored >= cap ? i : (size_t)stored;
}
/* probs != NULL: cached family (row written with exact zeros outside [j0, i]);
 * stats != NULL: tiled family (row kept in scratch). */
static void attn_fwd(const float* q, const float* k, const float* v, float* o, float* probs,
                     float* stats, size_t B, size_t S, size_t H, size_t d, const int32_t* starts) {
  const size_t D = H * d;
  const float inv_sqrt_d = 1.0f / sqrtf((float)d);
  float* scratch = (float*)malloc(S * sizeof(float));
  for (size_t u = 0; u < B * H * S; ++u) {
    const size_t b = u / (H * S), h = (u / S) % H, i = u % S;
    const float* qi = q + (b * S + i) * D + h * d;
    float* prow = probs ? probs + u * S : scratch;
    size_t j0 = 0;
    if (starts) {
      const int32_t s0 = starts[b * S + i];
      j0 = s0 <= 0 ? 0 : ((size_t)s0 < i ? (size_t)s0 : i);
    }
    if (probs) for (size_t j = 0; j < j0; ++j) prow[j] = 0.0f;
    float row_max = -INFINITY;
    for (size_t j = j0; j <= i; ++j) {
      const float s = (float)dot_d(qi, k + (b * S + j) * D + h * d, d) * inv_sqrt_d;
      prow[j] = s;
      if (s > row_max) row_max = s;
    }
    double denom = 0.0;
    for (size_t j = j0; j <= i; ++j) {
      const float e = expf(prow[j] - row_max);
      prow[j] = e;
      denom += e;
    }
    const float inv_denom = 1.0f / (float)denom;
    for (size_t j = j0; j <= i; ++j) prow[j] *= inv_denom;
    if (probs) for (size_t j = i + 1; j < S; ++j) prow[j] = 0.0f;
    float* oi = o + (b * S + i) * D + h * d;
    for (size_t c = 0; c < d; ++c) oi[c] = 0.0f;
    for (size_t j = j0; j <= i; ++j) {
      const float p = prow[j];
      const float* vj = v + (b * S + j) * D + h * d;
      for (size_t c = 0; c < d; ++c) oi[c] += p * vj[c];
    }
    if (stats) {
      float* st = stats + u * 4;
      st[0] = row_max; st[1] = inv_denom; st[2] = 0.0f; st[3] = (float)j0;
    }
  }
  free(scratch);
}
static void attn_dp(const float* dout, const float* v, float* dp, size_t B, size_t S, size_t H,
                    size_t d) {
  const size_t D = H * d;
  for (size_t u = 0; u < B * H * S; ++u) {
    const size_t b = u / (H * S), h = (u / S) % H, i = u % S;
    const float* doi = dout + (b * S + i) * D + h * d;
    float* row = dp + u * S;
    for (size_t j = 0; j <= i; ++j) row[j] = (float)dot_d(doi, v + (b * S + j) * D + h * d, d);
    for (size_t j = i + 1; j < S; ++j) row[j] = 0.0f;
  }
}
/* out_j = sum_{i>=j} (w[i, j] [* scale]) * x_i : dV (w = P, x = dO) and dK (w = dS, x = Q). */
static void attn_col(const float* w, const float* x, float* out, size_t B, size_t S, size_t H,
                     size_t d, int scaled) {
  const size_t D = H * d;
  const float inv_sqrt_d = 1.0f / sqrtf((float)d);
  for (size_t u = 0; u < B * H * S; ++u) {
    const size_t b = u / (H * S), h = (u / S) % H, j = u % S;
    float* oj = out + (b * S + j) * D + h * d;
    for (size_t c = 0; c < d; ++c) oj[c] = 0.0f;
    for (size_t i = j; i < S; ++i) {
      float g = w[((b * H + h) * S + i) * S + j];
      if (scaled) g = g * inv_sqrt_d;
      const float* xi = x + (b * S + i) * D + h * d;
      for (size_t c = 0; c < d; ++c) oj[c] += g * xi[c];
    }
  }
}
static void attn_dq(const float* ds, const float* k, float* dq, size_t B, size_t S, size_t H,
                    size_t d) {
  const size_t D = H * d;
  const float inv_sqrt_d = 1.0f / sqrtf((float)d);
  for (size_t u = 0; u < B * H * S; ++u) {
    const size_t b = u / (H * S), h = (u / S) % H, i = u % S;
    float* dqi = dq + (b * S + i) * D + h * d;
    for (size_t c = 0; c < d; ++c) dqi[c] = 0.0f;
    for (size_t j = 0; j <= i; ++j) {
      const float g = ds[u * S + j] * inv_sqrt_d;
      const float* kj = k + (b * S + j) * D + h * d;
      for (size_t c = 0; c < d; ++c) dqi[c] += g * kj[c];
    }
  }
}
static void softmax_rows_bwd(const float* probs, const float* dp, float* ds, size_t rows,
                             size_t cols) {
  for (size_t r = 0; r < rows; ++r) {
    const float* pr = probs + r * cols;
    const float* dpr = dp + r * cols;
    float* dsr = ds + r * cols;
    double dot = 0.0;
    for (size_t c = 0; c < cols; ++c) dot += (double)dpr[c] * pr[c];
    const float sum = (float)dot;
    for (size_t c = 0; c < cols; ++c) dsr[c] = pr[c] * (dpr[c] - sum);
  }
}
static float prob_of(const float* qi, const float* kj, size_t d, float inv_sqrt_d, float m,
                     float inv_denom) {
  const float s = (float)dot_d(qi, kj, d) * inv_sqrt_d;
  return expf(s - m) * inv_denom;
}
static void attn_dq_tiled(const float* q, const float* k, const float* v, const float* dout,
                          float* stats, float* dq, size_t B, size_t S, size_t H, size_t d) {
  const size_t D = H * d;
  const float inv_sqrt_d = 1.0f / sqrtf((float)d);
  float* prow = (float*)malloc(2 * S * sizeof(float));
  float* dprow = prow + S;
  for (size_t u = 0; u < B * H * S; ++u) {
    const size_t b = u / (H * S), h = (u / S) % H, i = u % S;
    const float* qi = q + (b * S + i) * D + h * d;
    const float* doi = dout + (b * S + i) * D + h * d;
    float* st = stats + u * 4;
    const size_t j0 = stats_start(st[3], i);
    double dot = 0.0;
    for (size_t j = j0; j <= i; ++j)
      prow[j] = prob_of(qi, k + (b * S + j) * D + h * d, d, inv_sqrt_d, st[0], st[1]);
    for (size_t j = j0; j <= i; ++j) {
      dprow[j] = (float)dot_d(doi, v + (b * S + j) * D + h * d, d);
      dot += (double)dprow[j] * prow[j];
    }
    const float delta = (float)dot;
    st[2] = delta;
    float* dqi = dq + (b * S + i) * D + h * d;
    for (size_t c = 0; c < d; ++c) dqi[c] = 0.0f;
    for (size_t j = j0; j <= i; ++j) {
      const float dsv = prow[j] * (dprow[j] - delta);
      const float g = dsv * inv_sqrt_d;
      const float* kj = k + (b * S + j) * D + h * d;
      for (size_t c = 0; c < d; ++c) dqi[c] += g * kj[c];
    }
  }
  free(prow);
}
static void attn_dkv_tiled(int want_dk, const float* q, const float* k, const float* v,
                           const float* dout, const float* stats, float* out, size_t B, size_t S,
                           size_t H, size_t d) {
  const size_t D = H * d;
  const float inv_sqrt_d = 1.0f / sqrtf((float)d);
  for (size_t u = 0; u < B * H * S; ++u) {
    const size_t b = u / (H * S), h = (u / S) % H, j = u % S;
    const float* kj = k + (b * S + j) * D + h * d;
    const float* vj = v + (b * S + j) * D + h * d;
    float* oj = out + (b * S + j) * D + h * d;
    for (size_t c = 0; c < d; ++c) oj[c] = 0.0f;
    for (size_t i = j; i < S; ++i) {
      const float* qi = q + (b * S + i) * D + h * d;
      const float* doi = dout + (b * S + i) * D + h * d;
      const float* st = stats + ((b * H + h) * S + i) * 4;
      if (j < stats_start(st[3], i)) continue;
      const float p = prob_of(qi, kj, d, inv_sqrt_d, st[0], st[1]);
      if (want_dk) {
        const float dsv = p * ((float)dot_d(doi, vj, d) - st[2]);
        const float g = dsv * inv_sqrt_d;
        for (size_t c = 0; c < d; ++c) oj[c] += g * qi[c];
      } else {
        for (size_t c = 0; c < d; ++c) oj[c] += p * doi[c];
      }
    }
  }
}

/* ---- dispatch: runtime/executor/cpu_backend.cc:260-646 -------------------------------- */
#define HI(w) ((size_t)((w) >> 32))
#define LO(w) ((size_t)((w) & 0xFFFFFFFFull))
#define RF(i) ((const float*)rd(o, ins->in[i]))
#define WF(i) ((float*)wr(o, ins->in[i]))

static int execute(Oracle* o, const Instr* ins, const StepParams* sp) {
  const uint64_t d0 = ins->out[0], d1 = ins->out[1], d2 = ins->out[2];
  const int act = (ins->flags & FLAG_ACT_MASK) >> FLAG_ACT_SHIFT;
  const float alpha = ins->imm == 0 ? 1.0f : bits_f32(ins->imm);
  const float eps = ins->imm == 0 ? 1e-5f : bits_f32(ins->imm);
  const float* in3 = ins->in[3] == NULL_REF ? NULL : (const float*)rd(o, ins->in[3]);
  switch (ins->opcode) {
    case 0: break;
    case 1: /* gemm.nn */
      gemm_quad(RF(0), rd(o, ins->in[1]), 0, WF(2), d0, d1, d2, alpha, 0, NULL, 0);
      gemm_epilogue(WF(2), d0, d1, (ins->flags & FLAG_ADDEND) ? in3 : NULL,
                    (ins->flags & FLAG_BIAS) ? in3 : NULL, act);
      break;
    case 2: /* gemm.nt */
      gemm_lane(RF(0), rd(o, ins->in[1]), 0, WF(2), d0, d1, d2, alpha, NULL);
      gemm_epilogue(WF(2), d0, d1, (ins->flags & FLAG_ADDEND) ? in3 : NULL, NULL, 0);
      break;
    case 3: /* gemm.tn */
      gemm_quad(RF(0), rd(o, ins->in[1]), 0, WF(2), d0, d1, d2, alpha, 1, NULL, 0);
      gemm_epilogue(WF(2), d0, d1, (ins->flags & FLAG_ADDEND) ? in3 : NULL, NULL, 0);
      break;
    case 4: /* gemm.acc.nn */
      gemm_quad(RF(0), rd(o, ins->in[1]), 0, WF(2), d0, d1, d2, bits_f32(ins->in[3]), 0, NULL, 1);
      break;
    case 29: { /* gemm.nn.q8 */
      const int cs = (ins->flags & FLAG_COLSCALE) != 0;
      gemm_quad(RF(0), rd(o, ins->in[1]), 1, WF(2), d0, d1, d2, cs ? 1.0f : bits_f32(ins->in[3]), 0,
                cs ? in3 : NULL, 0);
      gemm_epilogue(WF(2), d0, d1, NULL, NULL, act);
      break;
    }
    case 30: { /* gemm.nt.q8 */
      const int cs = (ins->flags & FLAG_COLSCALE) != 0;
      gemm_lane(RF(0), rd(o, ins->in[1]), 1, WF(2), d0, d1, d2, cs ? 1.0f : bits_f32(ins->in[3]),
                cs ? in3 : NULL);
      break;
    }
    case 43: /* gemm.nn.bf16 */
      gemm_quad(RF(0), rd(o, ins->in[1]), 2, WF(2), d0, d1, d2, 1.0f, 0, NULL, 0);
      gemm_epilogue(WF(2), d0, d1, NULL, (ins->flags & FLAG_BIAS) ? in3 : NULL, act);
      break;
    case 44: /* gemm.nt.bf16 */
      gemm_lane(RF(0), rd(o, ins->in[1]), 2, WF(2), d0, d1, d2, 1.0f, NULL);
      break;
    case 5: { const float *x = RF(0), *y = RF(1); float* out = WF(2);
      for (size_t i = 0; i < d0; ++i) out[i] = x[i] + y[i]; break; }
    case 21: { const float *x = RF(0), *y = RF(1); float* out = WF(2);
      for (size_t i = 0; i < d0; ++i) out[i] = x[i] * y[i]; break; }
    case 6: { const float *x = RF(0), *b = RF(1); float* out = WF(2);
      for (size_t r = 0; r < d0; ++r) for (size_t c = 0; c < d1; ++c) out[r * d1 + c] = x[r * d1 + c] + b[c];
      break; }
    case 7: { const float* x = RF(0); float* out = WF(1);
      for (size_t i = 0; i < d0; ++i) out[i] = relu_expr(x[i]); break; }
    case 22: { const float* x = RF(0); float* out = WF(1);
      for (size_t i = 0; i < d0; ++i) out[i] = gelu_expr(x[i]); break; }
    case 24: { const float* x = RF(0); float* out = WF(1);
      for (size_t i = 0; i < d0; ++i) out[i] = silu_expr(x[i]); break; }
    case 8: { const float *dy = RF(0), *x = RF(1); float* dx = WF(2); /* activation.cc:28-32 */
      for (size_t i = 0; i < d0; ++i) dx[i] = x[i] > 0.0f ? dy[i] : 0.0f; break; }
    case 23: { const float *dy = RF(0), *x = RF(1); float* dx = WF(2); /* activation.cc:40-60 */
      for (size_t i = 0; i < d0; ++i) {
        const float v = x[i];
        const float u = kGeluC * (v + kGeluA * v * v * v);
        const float t = tanhf(u);
        const float one_minus_t2 = 1.0f - t * t;
        const float tail = one_minus_t2 == 0.0f ? 0.0f
            : 0.5f * v * one_minus_t2 * (kGeluC * (1.0f + 3.0f * kGeluA * v * v));
        dx[i] = dy[i] * (0.5f * (1.0f + t) + tail);
      }
      break; }
    case 25: { const float *dy = RF(0), *x = RF(1); float* dx = WF(2); /* activation.cc:68-75 */
      for (size_t i = 0; i < d0; ++i) {
        const float s = sigmoid_expr(x[i]);
        dx[i] = dy[i] * (s * (1.0f + x[i] * (1.0f - s)));
      }
      break; }
    case 9: { const float* x = RF(0); float* out = WF(1); const float a = bits_f32(ins->in[2]);
      for (size_t i = 0; i < d0; ++i) out[i] = a * x[i]; break; }
    case 10: { const float* dy = RF(0); float* db = WF(1); /* elementwise.cc:162-187 */
      for (size_t c = 0; c < d1; ++c) { float acc = 0.0f;
        for (size_t r = 0; r < d0; ++r) acc += dy[r * d1 + c]; db[c] = acc; }
      break; }
    case 11: xent_fwd(0, RF(0), (const int32_t*)rd(o, ins->in[1]), WF(2), WF(3), d0, d1); break;
    case 51: xent_fwd(1, RF(0), (const int32_t*)rd(o, ins->in[1]), WF(2), WF(3), d0, d1); break;
    case 12: xent_bwd(0, RF(0), (const int32_t*)rd(o, ins->in[1]), RF(2), WF(3), d0, d1); break;
    case 52: xent_bwd(1, RF(0), (const int32_t*)rd(o, ins->in[1]), RF(2), WF(3), d0, d1); break;
    case 13: mse_fwd(RF(0), RF(1), WF(2), d0); break;
    case 14: mse_bwd(RF(0), RF(1), RF(2), WF(3), d0); break;
    case 15: kl_fwd(RF(0), RF(1), WF(2), WF(3), (float*)wr(o, d0), HI(d1), LO(d1), bits_f32(d2),
                    (d2 >> 32) == 0 ? 1.0f : bits_f32(d2 >> 32)); break;
    case 16: kl_bwd(RF(0), RF(1), RF(2), WF(3), HI(d0), LO(d0), bits_f32(d1),
                    (d1 >> 32) == 0 ? 1.0f : bits_f32(d1 >> 32)); break;
    case 17:
      if (!sgd_step(WF(0), RF(1), d0, sp->lr, sp->weight_decay, bits_f32(d1))) return 2;
      break;
    case 18:
      if (!adamw_step(WF(0), RF(1), WF(2), WF(3), d0, sp, bits_f32(d1))) return 2;
      break;
    case 19: { float* dst = WF(0); const float v = bits_f32(ins->in[1]);
      for (size_t i = 0; i < d0; ++i) dst[i] = v; break; }
    case 20: memcpy(WF(1), RF(0), d0 * sizeof(float)); break;
    case 42: { float* dst = WF(0); const float* src = RF(1);
      for (size_t i = 0; i < d0; ++i) dst[i] += src[i]; break; }
    case 26: layernorm_fwd(RF(0), RF(1), RF(2), WF(3), (float*)wr(o, d1), (float*)wr(o, d2),
                           HI(d0), LO(d0), eps); break;
    case 27: layernorm_bwd(RF(0), RF(1), RF(2), (const float*)rd(o, d0), (const float*)rd(o, d1),
                           WF(3), HI(d2), LO(d2)); break;
    case 31: rmsnorm_fwd(RF(0), RF(1), WF(2), WF(3), HI(d0), LO(d0), eps); break;
    case 32: rmsnorm_bwd(RF(0), RF(1), RF(2), (const float*)rd(o, d0), WF(3), HI(d1), LO(d1)); break;
    case 28: { const float cap = bits_f32(ins->in[1]);
      if (!isfinite(cap) || !(cap > 0.0f)) return 3;
      if (!clip_norm(WF(0), d0, cap)) return 2;
      break; }
    case 53: { float* acc = WF(1); /* optimizer.cc:66-68 */
      acc[0] = (float)((double)acc[0] + l2_squared(RF(0), d0)); break; }
    case 54: { const float cap = bits_f32(ins->in[2]);
      if (!isfinite(cap) || !(cap > 0.0f)) return 3;
      if (!clip_global(WF(0), d0, RF(1), cap)) return 2;
      break; }
    case 33: case 34:
      rope(ins->opcode == 34, RF(0), WF(1), HI(d0), LO(d0), HI(d1), LO(d1), bits_f32(d2),
           ins->in[2] == NULL_REF ? NULL : RF(2));
      break;
    case 45: rope_table(WF(0), HI(d0), LO(d0), bits_f32(d1)); break;
    case 46:
      fused_map(RF(0), ins->in[1] == NULL_REF ? NULL : RF(1), ins->in[2] == NULL_REF ? NULL : RF(2),
                WF(3), d0, d1, bits_f32(d2), bits_f32(d2 >> 32));
      break;
    case 35: attn_fwd(RF(0), RF(1), RF(2), WF(3), (float*)wr(o, d0), NULL, HI(d1), LO(d1), HI(d2),
                      LO(d2), NULL); break;
    case 56: attn_fwd(RF(0), RF(1), RF(2), WF(3), (float*)wr(o, d0), NULL, d1 >> 48,
                      (d1 >> 32) & 0xFFFF, (d1 >> 16) & 0xFFFF, d1 & 0xFFFF,
                      (const int32_t*)rd(o, d2)); break;
    case 47: attn_fwd(RF(0), RF(1), RF(2), WF(3), NULL, (float*)wr(o, d0), HI(d1), LO(d1), HI(d2),
                      LO(d2), NULL); break;
    case 57: attn_fwd(RF(0), RF(1), RF(2), WF(3), NULL, (float*)wr(o, d0), d1 >> 48,
                      (d1 >> 32) & 0xFFFF, (d1 >> 16) & 0xFFFF, d1 & 0xFFFF,
                      (const int32_t*)rd(o, d2)); break;
    case 36: attn_dp(RF(0), RF(1), WF(2), HI(d0), LO(d0), HI(d1), LO(d1)); break;
    case 37: attn_col(RF(0), RF(1), WF(2), HI(d0), LO(d0), HI(d1), LO(d1), 0); break;
    case 38: softmax_rows_bwd(RF(0), RF(1), WF(2), HI(d0), LO(d0)); break;
    case 39: attn_dq(RF(0), RF(1), WF(2), HI(d0), LO(d0), HI(d1), LO(d1)); break;
    case 40: attn_col(RF(0), RF(1), WF(2), HI(d0), LO(d0), HI(d1), LO(d1), 1); break;
    case 48:
      attn_dq_tiled(RF(0), RF(1), RF(2), RF(3), (float*)wr(o, d0), (float*)wr(o, d1), d2 >> 48,
                    (d2 >> 32) & 0xFFFF, (d2 >> 16) & 0xFFFF, d2 & 0xFFFF);
      break;
    case 49: case 50:
      attn_dkv_tiled(ins->opcode == 49, RF(0), RF(1), RF(2), RF(3), (const float*)rd(o, d0),
                     (float*)wr(o, d1), d2 >> 48, (d2 >> 32) & 0xFFFF, (d2 >> 16) & 0xFFFF,
                     d2 & 0xFFFF);
      break;
    case 41: { /* elementwise.cc:151-160 */
      const int32_t* tok = (const int32_t*)rd(o, ins->in[0]);
      const float* table = RF(1);
      float* out = WF(2);
      const size_t dim = LO(d1);
      for (size_t r = 0; r < d0; ++r)
        memcpy(out + r * dim, table + (size_t)tok[r] * dim, dim * sizeof(float));
      break; }
    case 55: { /* attention.cc:176-185 */
      const int32_t* tok = (const int32_t*)rd(o, ins->in[0]);
      int32_t* starts = (int32_t*)wr(o, ins->in[1]);
      const size_t B = HI(d0), S = LO(d0);
      for (size_t b = 0; b < B; ++b) { int32_t start = 0;
        for (size_t t = 0; t < S; ++t) { starts[b * S + t] = start;
          if (tok[b * S + t] == (int32_t)d1) start = (int32_t)(t + 1); } }
      break; }
    default:
      return 1;
  }
  return 0;
}

/* ---- C face, same shape as the reference shim's ------------------------------------------ */
void* seeo_create(void) { return calloc(1, sizeof(Oracle)); }
void seeo_destroy(void* h) { free(h); }
const char* seeo_last_error(void* h) { return ((Oracle*)h)->error; }
int seeo_bind(void* h, uint8_t* arena, uint64_t arena_bytes, const uint8_t* rodata,
              uint64_t rodata_bytes) {
  Oracle* o = (Oracle*)h;
  (void)arena_bytes; (void)rodata_bytes;
  o->arena = arena;
  o->rodata = rodata;
  return 0;
}
int seeo_bind_source(void* h, const uint8_t* data, uint64_t bytes) {
  (void)bytes;
  ((Oracle*)h)->source = data;
  return 0;
}
int64_t seeo_run(void* h, const void* instrs, uint64_t begin, uint64_t end, const StepParams* sp) {
  Oracle* o = (Oracle*)h;
  const Instr* prog = (const Instr*)instrs;
  for (uint64_t i = begin; i < end; ++i) {
    const int rc = execute(o, &prog[i], sp);
    if (rc) {
      snprintf(o->error, sizeof(o->error), "%s",
               rc == 2 ? "gradient norm is not finite — the step was refused with the parameters "
                         "and optimizer state untouched"
               : rc == 3 ? "clip threshold is not a finite positive float — the instruction was "
                           "refused with the gradient untouched"
                         : "unknown opcode");
      return 1 + (int64_t)i;
    }
  }
  return 0;
}
