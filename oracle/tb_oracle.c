/*
 * CPU oracle: a C restatement of torchburn's quantized decode hot path.
 *
 * TEST INFRASTRUCTURE ONLY - see tb_oracle.h.  The scalar functions are the
 * semantic definition (they follow the reference's scalar branches statement
 * by statement and are compiled with floating-point contraction off, as Rust
 * never contracts a*b+c).  The AVX2 / AVX-512 functions restate the
 * reference's SIMD tiers (same lane layout and accumulation order) and are the
 * timed CPU baseline; tests hold them within the reference's own bar (1e-3 of
 * scalar, in practice ~1e-6).  The reference's AVX-512-VNNI tier is W4A8
 * (activations rounded to 8 bits) and is lossy; it is intentionally absent.
 *
 * Threading: one task per output row chunk, chunk = max(n / (threads*4), 8),
 * as the reference's rayon `with_min_len` (src/quantization/gemv.rs:1535-1572).
 */
#include "tb_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#if defined(__x86_64__)
#include <immintrin.h>
#define TBO_X86 1
#else
#define TBO_X86 0
#endif

/* ------------------------------------------------------------------ tiers */

static int g_forced_tier = TBO_TIER_AUTO;
static int g_threads = 0;

int tbo_best_tier(void) {
#if TBO_X86
  __builtin_cpu_init();
  if (__builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw")) return TBO_TIER_AVX512;
  if (__builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma")) return TBO_TIER_AVX2;
#endif
  return TBO_TIER_SCALAR;
}

static int active_tier(void) {
  int best = tbo_best_tier();
  if (g_forced_tier == TBO_TIER_AUTO) return best;
  return g_forced_tier <= best ? g_forced_tier : best;
}

int tbo_force_tier(int tier) {
  g_forced_tier = tier;
  return active_tier();
}

void tbo_set_threads(int n) { g_threads = n; }

int tbo_get_threads(void) {
  if (g_threads > 0) return g_threads;
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

static int64_t row_chunk(int64_t n) {
  int64_t c = n / ((int64_t)tbo_get_threads() * 4);
  return c < 8 ? 8 : c;
}

/* -------------------------------------------------------------- quantizer */

/* python/torchburn/quantization.py:85-96.
 *   max_val = |w|.amax over the group
 *   scales  = clamp(max_val / 7.0, min=1e-8)          (fp32 division)
 *   q       = clamp(round(w / scales), -8, 7)          (fp32 division, torch.round = half-to-even)
 *   u       = q + 8 ; byte j = u[2j] | (u[2j+1] << 4)
 * rintf() under the default rounding mode is round-half-to-even. */
int tbo_quantize_int4_grouped(const float* w, int64_t n, int64_t k, int group_size,
                              uint8_t* packed, float* scales) {
  if (group_size <= 0 || k % group_size != 0) return -1; /* quantization.py:75-79 */
  const int64_t ng = k / group_size;
  const int64_t pc = (k + 1) / 2;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < n; ++r) {
    const float* wr = w + r * k;
    uint8_t* pr = packed + r * pc;
    memset(pr, 0, (size_t)pc);
    for (int64_t g = 0; g < ng; ++g) {
      const float* wg = wr + g * group_size;
      float mx = 0.0f;
      for (int i = 0; i < group_size; ++i) {
        float a = fabsf(wg[i]);
        if (a > mx || a != a) mx = a; /* amax propagates NaN */
      }
      float s = mx / 7.0f;
      if (s < 1e-8f) s = 1e-8f; /* clamp(min=1e-8); NaN stays NaN like torch.clamp */
      scales[r * ng + g] = s;
      for (int i = 0; i < group_size; ++i) {
        float q = rintf(wg[i] / s);
        if (q < -8.0f) q = -8.0f;
        if (q > 7.0f) q = 7.0f;
        int qi = (q != q) ? 0 : (int)q; /* NaN -> int8 conversion is undefined in torch; use 0 */
        uint8_t u = (uint8_t)(qi + 8) & 0x0F;
        int64_t idx = g * group_size + i;
        if ((idx & 1) == 0)
          pr[idx >> 1] |= u;
        else
          pr[idx >> 1] |= (uint8_t)(u << 4);
      }
    }
  }
  return 0;
}

/* src/quantization/gemv.rs:1491-1499: element i of a row lives in byte i/2,
 * low nibble when i is even, high nibble when odd; code = nibble - 8. */
static inline int code_at(const uint8_t* row, int64_t i) {
  uint8_t b = row[i >> 1];
  return ((i & 1) == 0) ? (int)(b & 0x0F) - 8 : (int)((b >> 4) & 0x0F) - 8;
}

void tbo_unpack_codes(const uint8_t* packed, int64_t n, int64_t k, int8_t* codes) {
  const int64_t pc = (k + 1) / 2;
  for (int64_t r = 0; r < n; ++r)
    for (int64_t i = 0; i < k; ++i) codes[r * k + i] = (int8_t)code_at(packed + r * pc, i);
}

/* tests/test_parity.py:51-64: w[j,i] = float(code) * scales[j, i / G]. */
void tbo_dequant_int4_grouped(const uint8_t* packed, const float* scales, int64_t n, int64_t k,
                              int group_size, float* w_out) {
  const int64_t ng = (k + group_size - 1) / group_size;
  const int64_t pc = (k + 1) / 2;
  for (int64_t r = 0; r < n; ++r)
    for (int64_t i = 0; i < k; ++i)
      w_out[r * k + i] = (float)code_at(packed + r * pc, i) * scales[r * ng + i / group_size];
}

/* ------------------------------------------------------------- row kernels */

/* src/quantization/gemv.rs:1486-1502 dot_f32_u4_group_scalar. */
static float dot_group_scalar(const float* x, const uint8_t* wp, int len) {
  float total = 0.0f;
  for (int i = 0; i < len; ++i) {
    uint8_t byte = wp[i / 2];
    int q = ((i % 2) == 0) ? (int)(byte & 0x0F) - 8 : (int)((byte >> 4) & 0x0F) - 8;
    total += x[i] * (float)q;
  }
  return total;
}

/* src/quantization/gemv.rs:1669-1679 (scalar branch; tail group clamped). */
static float row_scalar(const float* x, const uint8_t* w_row, const float* s_row, int64_t k,
                        int group_size) {
  const int64_t ng = (k + group_size - 1) / group_size;
  const int bpg = group_size / 2;
  float s = 0.0f;
  for (int64_t g = 0; g < ng; ++g) {
    int64_t rem = k - g * group_size;
    int cur = rem < group_size ? (int)rem : group_size;
    s += dot_group_scalar(x + g * group_size, w_row + g * bpg, cur) * s_row[g];
  }
  return s;
}

#if TBO_X86
/* src/quantization/gemv.rs:1190-1211 unpack_and_fma_32_avx512: 16 bytes ->
 * 32 codes in element order (unpacklo/hi interleave low and high nibbles),
 * widened to fp32; returns wf1*xf1 + (wf0*xf0) lane-wise. */
__attribute__((target("avx512f,avx512bw"))) static inline __m512 unpack_fma32_avx512(
    const float* x, const uint8_t* w) {
  const __m128i mask = _mm_set1_epi8(0x0F);
  const __m128i sub8 = _mm_set1_epi8(8);
  __m128i raw = _mm_loadu_si128((const __m128i*)w);
  __m128i lo = _mm_and_si128(raw, mask);
  __m128i hi = _mm_and_si128(_mm_srli_epi16(raw, 4), mask);
  __m128i s_lo = _mm_sub_epi8(_mm_unpacklo_epi8(lo, hi), sub8);
  __m128i s_hi = _mm_sub_epi8(_mm_unpackhi_epi8(lo, hi), sub8);
  __m512 wf0 = _mm512_cvtepi32_ps(_mm512_cvtepi8_epi32(s_lo));
  __m512 xf0 = _mm512_loadu_ps(x);
  __m512 wf1 = _mm512_cvtepi32_ps(_mm512_cvtepi8_epi32(s_hi));
  __m512 xf1 = _mm512_loadu_ps(x + 16);
  return _mm512_fmadd_ps(wf1, xf1, _mm512_mul_ps(wf0, xf0));
}

/* gemv.rs:1279-1299 (G=32) and :1253-1275 (G=64): lane-wise accumulation
 * acc = fma(group_sum, scale, acc), one horizontal add per row. */
__attribute__((target("avx512f,avx512bw"))) static float row_avx512(const float* x,
                                                                    const uint8_t* w_row,
                                                                    const float* s_row, int64_t ng,
                                                                    int group_size) {
  __m512 acc = _mm512_setzero_ps();
  if (group_size == 32) {
    for (int64_t g = 0; g < ng; ++g) {
      __m512 sum0 = unpack_fma32_avx512(x + g * 32, w_row + g * 16);
      acc = _mm512_fmadd_ps(sum0, _mm512_set1_ps(s_row[g]), acc);
    }
  } else { /* 64 */
    for (int64_t g = 0; g < ng; ++g) {
      __m512 sum0 = unpack_fma32_avx512(x + g * 64, w_row + g * 32);
      __m512 sum1 = unpack_fma32_avx512(x + g * 64 + 32, w_row + g * 32 + 16);
      acc = _mm512_fmadd_ps(_mm512_add_ps(sum0, sum1), _mm512_set1_ps(s_row[g]), acc);
    }
  }
  return _mm512_reduce_add_ps(acc);
}

/* src/quantization/gemv/swiglu.rs:205-255: gate and up rows share the x loads. */
__attribute__((target("avx512f,avx512bw"))) static void swiglu_pair_avx512(
    const float* x, const uint8_t* gw, const float* gs, const uint8_t* uw, const float* us,
    int64_t ng, int group_size, float* g_out, float* u_out) {
  __m512 ga = _mm512_setzero_ps(), ua = _mm512_setzero_ps();
  const int halves = group_size / 32;
  for (int64_t g = 0; g < ng; ++g) {
    __m512 gsum = _mm512_setzero_ps(), usum = _mm512_setzero_ps();
    for (int h = 0; h < halves; ++h) {
      const float* xp = x + g * group_size + h * 32;
      __m512 a = unpack_fma32_avx512(xp, gw + g * (group_size / 2) + h * 16);
      __m512 b = unpack_fma32_avx512(xp, uw + g * (group_size / 2) + h * 16);
      gsum = h == 0 ? a : _mm512_add_ps(gsum, a);
      usum = h == 0 ? b : _mm512_add_ps(usum, b);
    }
    ga = _mm512_fmadd_ps(gsum, _mm512_set1_ps(gs[g]), ga);
    ua = _mm512_fmadd_ps(usum, _mm512_set1_ps(us[g]), ua);
  }
  *g_out = _mm512_reduce_add_ps(ga);
  *u_out = _mm512_reduce_add_ps(ua);
}

/* gemv.rs hsum256_ps_avx equivalent. */
__attribute__((target("avx2,fma"))) static inline float hsum256(__m256 v) {
  __m128 lo = _mm256_castps256_ps128(v);
  __m128 hi = _mm256_extractf128_ps(v, 1);
  lo = _mm_add_ps(lo, hi);
  __m128 sh = _mm_movehdup_ps(lo);
  __m128 sums = _mm_add_ps(lo, sh);
  sh = _mm_movehl_ps(sh, sums);
  sums = _mm_add_ss(sums, sh);
  return _mm_cvtss_f32(sums);
}

/* src/quantization/gemv.rs:1215-1249 unpack_and_fma_32_avx2. */
__attribute__((target("avx2,fma"))) static inline __m256 unpack_fma32_avx2(const float* x,
                                                                           const uint8_t* w) {
  const __m128i mask = _mm_set1_epi8(0x0F);
  const __m128i sub8 = _mm_set1_epi8(8);
  __m128i raw = _mm_loadu_si128((const __m128i*)w);
  __m128i lo = _mm_and_si128(raw, mask);
  __m128i hi = _mm_and_si128(_mm_srli_epi16(raw, 4), mask);
  __m128i s_lo = _mm_sub_epi8(_mm_unpacklo_epi8(lo, hi), sub8);
  __m128i s_hi = _mm_sub_epi8(_mm_unpackhi_epi8(lo, hi), sub8);
  __m256 wf0 = _mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(s_lo));
  __m256 sum0 = _mm256_mul_ps(wf0, _mm256_loadu_ps(x));
  __m256 wf1 = _mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(_mm_unpackhi_epi64(s_lo, s_lo)));
  sum0 = _mm256_fmadd_ps(wf1, _mm256_loadu_ps(x + 8), sum0);
  __m256 wf2 = _mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(s_hi));
  __m256 sum1 = _mm256_mul_ps(wf2, _mm256_loadu_ps(x + 16));
  __m256 wf3 = _mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(_mm_unpackhi_epi64(s_hi, s_hi)));
  sum1 = _mm256_fmadd_ps(wf3, _mm256_loadu_ps(x + 24), sum1);
  return _mm256_add_ps(sum0, sum1);
}

/* gemv.rs:1303-1349. */
__attribute__((target("avx2,fma"))) static float row_avx2(const float* x, const uint8_t* w_row,
                                                          const float* s_row, int64_t ng,
                                                          int group_size) {
  __m256 acc = _mm256_setzero_ps();
  if (group_size == 32) {
    for (int64_t g = 0; g < ng; ++g) {
      __m256 sum0 = unpack_fma32_avx2(x + g * 32, w_row + g * 16);
      acc = _mm256_fmadd_ps(sum0, _mm256_set1_ps(s_row[g]), acc);
    }
  } else {
    for (int64_t g = 0; g < ng; ++g) {
      __m256 sum0 = unpack_fma32_avx2(x + g * 64, w_row + g * 32);
      __m256 sum1 = unpack_fma32_avx2(x + g * 64 + 32, w_row + g * 32 + 16);
      acc = _mm256_fmadd_ps(_mm256_add_ps(sum0, sum1), _mm256_set1_ps(s_row[g]), acc);
    }
  }
  return hsum256(acc);
}

__attribute__((target("avx2,fma"))) static void swiglu_pair_avx2(
    const float* x, const uint8_t* gw, const float* gs, const uint8_t* uw, const float* us,
    int64_t ng, int group_size, float* g_out, float* u_out) {
  *g_out = row_avx2(x, gw, gs, ng, group_size);
  *u_out = row_avx2(x, uw, us, ng, group_size);
}

/* src/quantization/fused_ops.rs:646-665 dot_f32_f32 (AVX-512 branch). */
__attribute__((target("avx512f"))) static float dot_avx512(const float* a, const float* b,
                                                           int len) {
  __m512 acc = _mm512_setzero_ps();
  int i = 0;
  for (; i + 16 <= len; i += 16)
    acc = _mm512_fmadd_ps(_mm512_loadu_ps(a + i), _mm512_loadu_ps(b + i), acc);
  float sum = _mm512_reduce_add_ps(acc);
  for (; i < len; ++i) sum += a[i] * b[i];
  return sum;
}

/* src/quantization/fused_ops.rs:666-681 (AVX2 branch). */
__attribute__((target("avx2,fma"))) static float dot_avx2(const float* a, const float* b, int len) {
  __m256 acc = _mm256_setzero_ps();
  int i = 0;
  for (; i + 8 <= len; i += 8)
    acc = _mm256_fmadd_ps(_mm256_loadu_ps(a + i), _mm256_loadu_ps(b + i), acc);
  float sum = hsum256(acc);
  for (; i < len; ++i) sum += a[i] * b[i];
  return sum;
}

/* fast_vector_fma: dst += src * w (fused on the SIMD tiers). */
__attribute__((target("avx512f"))) static void vfma_avx512(float* dst, const float* src, float w,
                                                           int n) {
  __m512 wv = _mm512_set1_ps(w);
  int i = 0;
  for (; i + 16 <= n; i += 16)
    _mm512_storeu_ps(dst + i, _mm512_fmadd_ps(_mm512_loadu_ps(src + i), wv, _mm512_loadu_ps(dst + i)));
  for (; i < n; ++i) dst[i] += src[i] * w;
}

__attribute__((target("avx2,fma"))) static void vfma_avx2(float* dst, const float* src, float w,
                                                          int n) {
  __m256 wv = _mm256_set1_ps(w);
  int i = 0;
  for (; i + 8 <= n; i += 8)
    _mm256_storeu_ps(dst + i, _mm256_fmadd_ps(_mm256_loadu_ps(src + i), wv, _mm256_loadu_ps(dst + i)));
  for (; i < n; ++i) dst[i] += src[i] * w;
}

/* src/quantization/fused_ops.rs:1063-1090 fast_rms_norm_avx512. */
__attribute__((target("avx512f"))) static void rms_norm_avx512(const float* x, const float* w,
                                                               float* out, int64_t n, float eps) {
  __m512 sum_sq = _mm512_setzero_ps();
  int64_t chunks = n / 16;
  for (int64_t c = 0; c < chunks; ++c) {
    __m512 v = _mm512_loadu_ps(x + c * 16);
    sum_sq = _mm512_fmadd_ps(v, v, sum_sq);
  }
  float total = _mm512_reduce_add_ps(sum_sq);
  for (int64_t i = chunks * 16; i < n; ++i) total += x[i] * x[i];
  float rms = sqrtf(total / (float)n + eps);
  __m512 inv = _mm512_set1_ps(1.0f / rms);
  for (int64_t c = 0; c < chunks; ++c) {
    __m512 v = _mm512_loadu_ps(x + c * 16);
    __m512 wt = _mm512_loadu_ps(w + c * 16);
    _mm512_storeu_ps(out + c * 16, _mm512_mul_ps(_mm512_mul_ps(v, inv), wt));
  }
  for (int64_t i = chunks * 16; i < n; ++i) out[i] = (x[i] / rms) * w[i];
}
#endif /* TBO_X86 */

static float row_dispatch(int tier, const float* x, const uint8_t* w_row, const float* s_row,
                          int64_t k, int group_size) {
#if TBO_X86
  /* The SIMD rows assume whole groups of 32 or 64 (gemv.rs:1579-1600); any
   * other group size takes the scalar group loop on every tier. */
  if ((group_size == 32 || group_size == 64) && k % group_size == 0) {
    if (tier == TBO_TIER_AVX512) return row_avx512(x, w_row, s_row, k / group_size, group_size);
    if (tier == TBO_TIER_AVX2) return row_avx2(x, w_row, s_row, k / group_size, group_size);
  }
#endif
  (void)tier;
  return row_scalar(x, w_row, s_row, k, group_size);
}

/* ------------------------------------------------------------ GEMV / GEMM */

void tbo_gemv_w4a32_grouped(const float* x, const uint8_t* w, const float* scales,
                            const float* bias, float* out, int64_t n, int64_t k, int group_size) {
  const int64_t ng = (k + group_size - 1) / group_size;
  const int64_t bpr = (k + 1) / 2;
  const int tier = active_tier();
  const int64_t chunk = row_chunk(n);
  const int nt = tbo_get_threads();
#pragma omp parallel for schedule(dynamic, chunk) num_threads(nt) if (nt > 1)
  for (int64_t j = 0; j < n; ++j) {
    float row_sum = row_dispatch(tier, x, w + j * bpr, scales + j * ng, k, group_size);
    float b = bias ? bias[j] : 0.0f;
    out[j] = row_sum + b; /* gemv.rs:1681-1682 */
  }
}

/* gemv.rs:1717-1724: M independent GEMVs. */
void tbo_gemm_w4a32_grouped(const float* x, const uint8_t* w, const float* scales,
                            const float* bias, float* out, int64_t m, int64_t n, int64_t k,
                            int group_size) {
  for (int64_t i = 0; i < m; ++i)
    tbo_gemv_w4a32_grouped(x + i * k, w, scales, bias, out + i * n, n, k, group_size);
}

void tbo_gemm_w4a32_f64(const float* x, const uint8_t* w, const float* scales, const float* bias,
                        double* out, int64_t m, int64_t n, int64_t k, int group_size) {
  const int64_t ng = (k + group_size - 1) / group_size;
  const int64_t bpr = (k + 1) / 2;
#pragma omp parallel for schedule(static)
  for (int64_t j = 0; j < n; ++j) {
    for (int64_t i = 0; i < m; ++i) {
      double acc = 0.0;
      for (int64_t c = 0; c < k; ++c)
        acc += (double)x[i * k + c] * (double)code_at(w + j * bpr, c) *
               (double)scales[j * ng + c / group_size];
      out[i * n + j] = acc + (bias ? (double)bias[j] : 0.0);
    }
  }
}

/* ----------------------------------------------------------------- RMSNorm */

void tbo_rms_norm(const float* x, const float* w, float* out, int64_t n, float eps) {
#if TBO_X86
  if (active_tier() == TBO_TIER_AVX512) {
    rms_norm_avx512(x, w, out, n, eps);
    return;
  }
#endif
  /* fused_ops.rs:1107-1116 (scalar). */
  float total = 0.0f;
  for (int64_t i = 0; i < n; ++i) total += x[i] * x[i];
  float rms = sqrtf(total / (float)n + eps);
  float inv = 1.0f / rms;
  for (int64_t i = 0; i < n; ++i) out[i] = x[i] * inv * w[i];
}

/* -------------------------------------------------------------------- RoPE */

void tbo_rope_tables(int64_t max_seq_len, int head_dim, double theta, float* cos_t, float* sin_t) {
  const int half = head_dim / 2;
  for (int64_t pos = 0; pos < max_seq_len; ++pos) {
    for (int i = 0; i < half; ++i) {
      double freq = 1.0 / pow(theta, (2.0 * (double)i) / (double)head_dim);
      double val = (double)pos * freq;
      float c = (float)cos(val), s = (float)sin(val);
      cos_t[pos * head_dim + i] = c;
      cos_t[pos * head_dim + i + half] = c;
      sin_t[pos * head_dim + i] = s;
      sin_t[pos * head_dim + i + half] = s;
    }
  }
}

/* decoder.rs:28-68: products are rounded separately (no fused multiply-add). */
void tbo_rope_apply_head(float* head, const float* cos_p, const float* sin_p, int half_dim) {
  for (int i = 0; i < half_dim; ++i) {
    float q1 = head[i], q2 = head[i + half_dim];
    float a = q1 * cos_p[i];
    float b = q2 * sin_p[i];
    float c = q2 * cos_p[i + half_dim];
    float d = q1 * sin_p[i + half_dim];
    head[i] = a - b;
    head[i + half_dim] = c + d;
  }
}

/* --------------------------------------------------------------- attention */

static float dot_f32(int tier, const float* a, const float* b, int len) {
#if TBO_X86
  if (tier == TBO_TIER_AVX512 && len >= 16) return dot_avx512(a, b, len);
  if (tier >= TBO_TIER_AVX2 && len >= 8) return dot_avx2(a, b, len);
#endif
  (void)tier;
  float s = 0.0f;
  for (int i = 0; i < len; ++i) s += a[i] * b[i];
  return s;
}

static void vec_fma(int tier, float* dst, const float* src, float w, int n) {
#if TBO_X86
  if (tier == TBO_TIER_AVX512) { vfma_avx512(dst, src, w, n); return; }
  if (tier == TBO_TIER_AVX2) { vfma_avx2(dst, src, w, n); return; }
#endif
  (void)tier;
  for (int i = 0; i < n; ++i) dst[i] += src[i] * w;
}

/* decoder.rs:1148-1213: per q head, kv_h = h / (Hq/Hkv); scores scaled by
 * 1/sqrt(d); two-pass softmax (max, exp(s-max), sum, inv = 1/max(sum,1e-30));
 * out = sum_t (e_t*inv) * v_t.  seq_len == 1 copies v.  seq_len capped at 32768. */
void tbo_attention_decode(const float* q, const float* k_cache, const float* v_cache, float* out,
                          int num_heads, int num_kv_heads, int head_dim, int64_t max_seq_len,
                          int64_t seq_len) {
  const int64_t head_stride = max_seq_len * head_dim;
  const float scale = 1.0f / sqrtf((float)head_dim);
  int hpk = num_heads / (num_kv_heads > 0 ? num_kv_heads : 1);
  if (hpk < 1) hpk = 1;
  const int tier = active_tier();
  const int nt = tbo_get_threads();
#pragma omp parallel for schedule(dynamic, 1) num_threads(nt) if (nt > 1)
  for (int h = 0; h < num_heads; ++h) {
    float* out_h = out + (int64_t)h * head_dim;
    memset(out_h, 0, sizeof(float) * (size_t)head_dim);
    const int kv_h = h / hpk;
    const float* qh = q + (int64_t)h * head_dim;
    const float* kb = k_cache + kv_h * head_stride;
    const float* vb = v_cache + kv_h * head_stride;
    if (seq_len == 1) {
      memcpy(out_h, vb, sizeof(float) * (size_t)head_dim);
      continue;
    }
    int64_t capped = seq_len < 32768 ? seq_len : 32768;
    float* scores = (float*)malloc(sizeof(float) * (size_t)capped);
    float max_score = -INFINITY;
    for (int64_t t = 0; t < capped; ++t) {
      float sc = dot_f32(tier, qh, kb + t * head_dim, head_dim) * scale;
      scores[t] = sc;
      if (sc > max_score) max_score = sc;
    }
    float exp_sum = 0.0f;
    for (int64_t t = 0; t < capped; ++t) {
      float ex = expf(scores[t] - max_score);
      scores[t] = ex;
      exp_sum += ex;
    }
    float inv_sum = 1.0f / (exp_sum > 1e-30f ? exp_sum : 1e-30f);
    for (int64_t t = 0; t < capped; ++t)
      vec_fma(tier, out_h, vb + t * head_dim, scores[t] * inv_sum, head_dim);
    free(scores);
  }
}

/* ------------------------------------------------------------------ SwiGLU */

void tbo_swiglu_gemv(const float* x, const uint8_t* gw, const float* gs, const float* gb,
                     const uint8_t* uw, const float* us, const float* ub, float* h, int64_t n,
                     int64_t k, int group_size) {
  const int64_t ng = (k + group_size - 1) / group_size;
  const int64_t bpr = (k + 1) / 2;
  const int tier = active_tier();
  const int64_t chunk = row_chunk(n);
  const int nt = tbo_get_threads();
#pragma omp parallel for schedule(dynamic, chunk) num_threads(nt) if (nt > 1)
  for (int64_t j = 0; j < n; ++j) {
    float g_sum, u_sum;
    const uint8_t* gr = gw + j * bpr;
    const uint8_t* ur = uw + j * bpr;
    const float* gsr = gs + j * ng;
    const float* usr = us + j * ng;
    int simd_ok = (group_size == 32 || group_size == 64) && k % group_size == 0;
#if TBO_X86
    if (simd_ok && tier == TBO_TIER_AVX512)
      swiglu_pair_avx512(x, gr, gsr, ur, usr, ng, group_size, &g_sum, &u_sum);
    else if (simd_ok && tier == TBO_TIER_AVX2)
      swiglu_pair_avx2(x, gr, gsr, ur, usr, ng, group_size, &g_sum, &u_sum);
    else
#endif
    {
      (void)simd_ok;
      g_sum = row_scalar(x, gr, gsr, k, group_size);
      u_sum = row_scalar(x, ur, usr, k, group_size);
    }
    /* decoder.rs:1316-1322 */
    float g = g_sum + (gb ? gb[j] : 0.0f);
    float u = u_sum + (ub ? ub[j] : 0.0f);
    float silu_g = g / (1.0f + expf(-g));
    h[j] = silu_g * u;
  }
}

void tbo_fused_swiglu_mlp(const float* x, int64_t m, const uint8_t* gw, const float* gs,
                          const float* gb, const uint8_t* uw, const float* us, const float* ub,
                          const uint8_t* dw, const float* ds, const float* db, float* out,
                          int64_t hidden, int64_t inter, int group_size) {
  float* h = (float*)malloc(sizeof(float) * (size_t)(m * inter));
  if (m == 1) {
    tbo_swiglu_gemv(x, gw, gs, gb, uw, us, ub, h, inter, hidden, group_size);
  } else {
    /* fused_ops.rs:1297-1313: two linears then elementwise SwiGLU. */
    float* u = (float*)malloc(sizeof(float) * (size_t)(m * inter));
    tbo_gemm_w4a32_grouped(x, gw, gs, gb, h, m, inter, hidden, group_size);
    tbo_gemm_w4a32_grouped(x, uw, us, ub, u, m, inter, hidden, group_size);
    for (int64_t i = 0; i < m * inter; ++i) {
      float gv = h[i];
      h[i] = (gv / (1.0f + expf(-gv))) * u[i];
    }
    free(u);
  }
  tbo_gemm_w4a32_grouped(h, dw, ds, db, out, m, hidden, inter, group_size);
  free(h);
}

/* ----------------------------------------------------------------- decoder */

struct tbo_decoder {
  tbo_model_config cfg;
  const float* embed;
  tbo_layer_weights* layers;
  const float* final_norm_w;
  const uint8_t* lm_w;
  const float* lm_s;
  float **k_caches, **v_caches;
  int64_t kv_used;
  float *cos_t, *sin_t;
  float *x, *normed, *qkv, *attn, *o_out, *h, *down_out, *logits;
  /* layer-0 snapshots */
  float *dbg_embed, *dbg_normed, *dbg_qkv, *dbg_attn, *dbg_x_attn, *dbg_h, *dbg_x_out;
};

static float* falloc(int64_t n) { return (float*)calloc((size_t)(n > 0 ? n : 1), sizeof(float)); }

tbo_decoder* tbo_decoder_create(const tbo_model_config* c, const float* embed_tokens,
                                const tbo_layer_weights* layers, const float* final_norm_w,
                                const uint8_t* lm_head_w, const float* lm_head_s) {
  /* decoder.rs:214-233 */
  if (c->hidden_size % 4 != 0) return NULL;
  if (c->group_size <= 0 || c->hidden_size % c->group_size != 0) return NULL;
  if (c->head_dim % 2 != 0) return NULL;
  if (c->num_kv_heads <= 0 || c->num_heads % c->num_kv_heads != 0) return NULL;
  tbo_decoder* d = (tbo_decoder*)calloc(1, sizeof(tbo_decoder));
  d->cfg = *c;
  d->embed = embed_tokens;
  d->layers = (tbo_layer_weights*)malloc(sizeof(tbo_layer_weights) * (size_t)c->num_layers);
  memcpy(d->layers, layers, sizeof(tbo_layer_weights) * (size_t)c->num_layers);
  d->final_norm_w = final_norm_w;
  d->lm_w = lm_head_w;
  d->lm_s = lm_head_s;
  const int64_t hd = c->head_dim;
  d->cos_t = falloc(c->max_seq_len * hd);
  d->sin_t = falloc(c->max_seq_len * hd);
  tbo_rope_tables(c->max_seq_len, c->head_dim, c->rope_theta, d->cos_t, d->sin_t);
  const int64_t kv_len = (int64_t)c->num_kv_heads * c->max_seq_len * hd; /* decoder.rs:353-359 */
  d->k_caches = (float**)malloc(sizeof(float*) * (size_t)c->num_layers);
  d->v_caches = (float**)malloc(sizeof(float*) * (size_t)c->num_layers);
  for (int l = 0; l < c->num_layers; ++l) {
    d->k_caches[l] = falloc(kv_len);
    d->v_caches[l] = falloc(kv_len);
  }
  const int64_t q_dim = (int64_t)c->num_heads * hd, kv_dim = (int64_t)c->num_kv_heads * hd;
  const int64_t total_qkv = q_dim + 2 * kv_dim;
  d->x = falloc(c->hidden_size);
  d->normed = falloc(c->hidden_size);
  d->qkv = falloc(total_qkv);
  d->attn = falloc(q_dim);
  d->o_out = falloc(c->hidden_size);
  d->h = falloc(c->intermediate_size);
  d->down_out = falloc(c->hidden_size);
  d->logits = falloc(c->vocab_size);
  d->dbg_embed = falloc(c->hidden_size);
  d->dbg_normed = falloc(c->hidden_size);
  d->dbg_qkv = falloc(total_qkv);
  d->dbg_attn = falloc(q_dim);
  d->dbg_x_attn = falloc(c->hidden_size);
  d->dbg_h = falloc(c->intermediate_size);
  d->dbg_x_out = falloc(c->hidden_size);
  return d;
}

void tbo_decoder_destroy(tbo_decoder* d) {
  if (!d) return;
  for (int l = 0; l < d->cfg.num_layers; ++l) {
    free(d->k_caches[l]);
    free(d->v_caches[l]);
  }
  free(d->k_caches); free(d->v_caches); free(d->layers);
  free(d->cos_t); free(d->sin_t);
  free(d->x); free(d->normed); free(d->qkv); free(d->attn); free(d->o_out); free(d->h);
  free(d->down_out); free(d->logits);
  free(d->dbg_embed); free(d->dbg_normed); free(d->dbg_qkv); free(d->dbg_attn);
  free(d->dbg_x_attn); free(d->dbg_h); free(d->dbg_x_out);
  free(d);
}

void tbo_decoder_step(tbo_decoder* d, int64_t token_id, int64_t offset) {
  const tbo_model_config* c = &d->cfg;
  const int64_t H = c->hidden_size, I = c->intermediate_size;
  const int hd = c->head_dim, nh = c->num_heads, nkv = c->num_kv_heads;
  const int64_t q_dim = (int64_t)nh * hd, kv_dim = (int64_t)nkv * hd, total_qkv = q_dim + 2 * kv_dim;
  const int G = c->group_size;
  const int64_t head_stride = c->max_seq_len * hd;
  const int half = hd / 2;

  /* 1. embedding lookup; out-of-range token or offset -> zeroed step (decoder.rs:1066-1092) */
  if (token_id < 0 || token_id >= c->vocab_size || offset < 0 || offset >= c->max_seq_len) {
    memset(d->x, 0, sizeof(float) * (size_t)H);
    memset(d->logits, 0, sizeof(float) * (size_t)c->vocab_size);
    return;
  }
  memcpy(d->x, d->embed + token_id * H, sizeof(float) * (size_t)H);
  const float* cos_p = d->cos_t + offset * hd;
  const float* sin_p = d->sin_t + offset * hd;
  if (offset + 1 > d->kv_used) d->kv_used = offset + 1;

  for (int l = 0; l < c->num_layers; ++l) {
    const tbo_layer_weights* L = &d->layers[l];
    if (l == 0) memcpy(d->dbg_embed, d->x, sizeof(float) * (size_t)H);
    /* A */
    tbo_rms_norm(d->x, L->input_norm_w, d->normed, H, c->rms_norm_eps);
    if (l == 0) memcpy(d->dbg_normed, d->normed, sizeof(float) * (size_t)H);
    /* B */
    tbo_gemv_w4a32_grouped(d->normed, L->qkv_w, L->qkv_s, L->qkv_b, d->qkv, total_qkv, H, G);
    float* q = d->qkv;
    float* k = d->qkv + q_dim;
    float* v = k + kv_dim;
    /* C */
    for (int h = 0; h < nh; ++h) tbo_rope_apply_head(q + (int64_t)h * hd, cos_p, sin_p, half);
    for (int h = 0; h < nkv; ++h) tbo_rope_apply_head(k + (int64_t)h * hd, cos_p, sin_p, half);
    if (l == 0) memcpy(d->dbg_qkv, d->qkv, sizeof(float) * (size_t)total_qkv);
    /* D */
    for (int kh = 0; kh < nkv; ++kh) {
      int64_t dst = kh * head_stride + offset * hd;
      memcpy(d->k_caches[l] + dst, k + (int64_t)kh * hd, sizeof(float) * (size_t)hd);
      memcpy(d->v_caches[l] + dst, v + (int64_t)kh * hd, sizeof(float) * (size_t)hd);
    }
    /* E */
    tbo_attention_decode(q, d->k_caches[l], d->v_caches[l], d->attn, nh, nkv, hd, c->max_seq_len,
                         offset + 1);
    if (l == 0) memcpy(d->dbg_attn, d->attn, sizeof(float) * (size_t)q_dim);
    /* F, G */
    tbo_gemv_w4a32_grouped(d->attn, L->o_w, L->o_s, NULL, d->o_out, H, q_dim, G);
    for (int64_t i = 0; i < H; ++i) d->x[i] += d->o_out[i];
    if (l == 0) memcpy(d->dbg_x_attn, d->x, sizeof(float) * (size_t)H);
    /* H */
    tbo_rms_norm(d->x, L->post_norm_w, d->normed, H, c->rms_norm_eps);
    /* I */
    tbo_swiglu_gemv(d->normed, L->gate_w, L->gate_s, NULL, L->up_w, L->up_s, NULL, d->h, I, H, G);
    if (l == 0) memcpy(d->dbg_h, d->h, sizeof(float) * (size_t)I);
    tbo_gemv_w4a32_grouped(d->h, L->down_w, L->down_s, NULL, d->down_out, H, I, G);
    /* J */
    for (int64_t i = 0; i < H; ++i) d->x[i] += d->down_out[i];
    if (l == 0) memcpy(d->dbg_x_out, d->x, sizeof(float) * (size_t)H);
  }
  /* 3, 4 */
  tbo_rms_norm(d->x, d->final_norm_w, d->normed, H, c->rms_norm_eps);
  tbo_gemv_w4a32_grouped(d->normed, d->lm_w, d->lm_s, NULL, d->logits, c->vocab_size, H, G);
}

int64_t tbo_decoder_prefill_tokens(tbo_decoder* d, const int64_t* tokens, int64_t n,
                                   int64_t start_offset) {
  if (n == 0) return start_offset;
  if (start_offset + n > d->cfg.max_seq_len) return -1;
  for (int64_t i = 0; i < n; ++i) tbo_decoder_step(d, tokens[i], start_offset + i);
  return start_offset + n;
}

void tbo_decoder_reset_kv_cache(tbo_decoder* d) {
  const tbo_model_config* c = &d->cfg;
  int64_t used = d->kv_used < c->max_seq_len ? d->kv_used : c->max_seq_len;
  if (used == 0) return;
  const int64_t stride = c->max_seq_len * c->head_dim;
  for (int l = 0; l < c->num_layers; ++l)
    for (int kh = 0; kh < c->num_kv_heads; ++kh) {
      memset(d->k_caches[l] + kh * stride, 0, sizeof(float) * (size_t)(used * c->head_dim));
      memset(d->v_caches[l] + kh * stride, 0, sizeof(float) * (size_t)(used * c->head_dim));
    }
  d->kv_used = 0;
}

int64_t tbo_decoder_kv_len(const tbo_decoder* d) { return d->kv_used; }
const float* tbo_decoder_logits(const tbo_decoder* d) { return d->logits; }
float* tbo_decoder_k_cache(tbo_decoder* d, int layer) { return d->k_caches[layer]; }
float* tbo_decoder_v_cache(tbo_decoder* d, int layer) { return d->v_caches[layer]; }
void tbo_decoder_set_kv_len(tbo_decoder* d, int64_t n) { d->kv_used = n; }

int64_t tbo_decoder_debug_stage(const tbo_decoder* d, const char* name, const float** data) {
  const tbo_model_config* c = &d->cfg;
  const int64_t q_dim = (int64_t)c->num_heads * c->head_dim;
  const int64_t total_qkv = q_dim + 2 * (int64_t)c->num_kv_heads * c->head_dim;
  if (!strcmp(name, "embed")) { *data = d->dbg_embed; return c->hidden_size; }
  if (!strcmp(name, "normed")) { *data = d->dbg_normed; return c->hidden_size; }
  if (!strcmp(name, "qkv")) { *data = d->dbg_qkv; return total_qkv; }
  if (!strcmp(name, "attn")) { *data = d->dbg_attn; return q_dim; }
  if (!strcmp(name, "x_attn")) { *data = d->dbg_x_attn; return c->hidden_size; }
  if (!strcmp(name, "h")) { *data = d->dbg_h; return c->intermediate_size; }
  if (!strcmp(name, "x_out")) { *data = d->dbg_x_out; return c->hidden_size; }
  return -1;
}

int64_t tbo_argmax(const float* logits, int64_t n) {
  if (n <= 0) return 0;
  int64_t best = 0;
  float bv = logits[0];
  for (int64_t i = 1; i < n; ++i)
    if (logits[i] > bv) { bv = logits[i]; best = i; }
  return best;
}

/* ---------------------------------------------------------------- sampling */

/* src/llm/decoder.rs:878-899: each distinct in-vocabulary token once. */
void tbo_apply_repetition_penalty(float* logits, int64_t vocab, const int64_t* recent, int64_t n_recent,
                                  float penalty) {
  if (penalty <= 1.0f || n_recent <= 0) return;
  for (int64_t i = 0; i < n_recent; ++i) {
    int64_t t = recent[i];
    if (t < 0 || t >= vocab) continue;
    int dup = 0;
    for (int64_t j = 0; j < i; ++j)
      if (recent[j] == t) { dup = 1; break; }
    if (dup) continue;
    float l = logits[t];
    logits[t] = l > 0.0f ? l / penalty : l * penalty;
  }
}

/* src/llm/decoder.rs:908-1020 with the random draw passed in as `u` in [0,1).
 * Branches restated: greedy; k >= vocab; running top-k for k <= 1024.  (The k > 1024 branch
 * uses an unstable selection whose order is unspecified; callers compare sets there.) */
int64_t tbo_sample_logits(const float* logits, int64_t vocab, float temperature, int64_t top_k, float top_p,
                          float u) {
  if (vocab == 0) return 0;
  if (!isfinite(temperature) || temperature <= 0.0f || top_k == 1) return tbo_argmax(logits, vocab);
  int64_t k = top_k < vocab ? top_k : vocab;
  if (k < 1) k = 1;
  int64_t* idx = (int64_t*)malloc(sizeof(int64_t) * (size_t)k);
  float* val = (float*)malloc(sizeof(float) * (size_t)k);
  int64_t cnt = 0;
  if (k >= vocab) {
    for (int64_t i = 0; i < vocab; ++i) { idx[i] = i; val[i] = isfinite(logits[i]) ? logits[i] : -INFINITY; }
    cnt = vocab;
  } else {
    float min_val = -INFINITY;
    int64_t min_pos = 0;
    for (int64_t i = 0; i < vocab; ++i) {
      float v = isfinite(logits[i]) ? logits[i] : -INFINITY;
      if (cnt < k) {
        idx[cnt] = i; val[cnt] = v; ++cnt;
        if (v < min_val || cnt == 1) { min_val = v; min_pos = cnt - 1; }
      } else if (v > min_val) {
        idx[min_pos] = i; val[min_pos] = v;
        float nm = val[0]; int64_t np = 0;
        for (int64_t j = 0; j < cnt; ++j) if (val[j] < nm) { nm = val[j]; np = j; }
        min_val = nm; min_pos = np;
      }
    }
  }
  float mx = -INFINITY;
  for (int64_t j = 0; j < cnt; ++j) if (val[j] > mx) mx = val[j];
  float inv_temp = 1.0f / temperature;
  for (int64_t j = 0; j < cnt; ++j) val[j] = expf((val[j] - mx) * inv_temp);
  float pre = 0.f;
  for (int64_t j = 0; j < cnt; ++j) pre += val[j];
  int64_t kept = cnt;
  if (top_p > 0.0f && top_p < 1.0f && kept > 1 && pre > 0.0f) {
    /* descending by probability (insertion sort keeps equal items in order) */
    for (int64_t a = 1; a < cnt; ++a) {
      float v = val[a]; int64_t id = idx[a]; int64_t b = a - 1;
      while (b >= 0 && val[b] < v) { val[b + 1] = val[b]; idx[b + 1] = idx[b]; --b; }
      val[b + 1] = v; idx[b + 1] = id;
    }
    float inv = 1.0f / pre, cum = 0.f;
    for (int64_t j = 0; j < cnt; ++j) {
      if (cum > top_p) { kept = j; break; }
      cum += val[j] * inv;
    }
  }
  float ks = 0.f;
  for (int64_t j = 0; j < kept; ++j) ks += val[j];
  float r = u * ks, acc = 0.f;
  int64_t out = idx[0];
  for (int64_t j = 0; j < kept; ++j) {
    acc += val[j];
    if (acc >= r) { out = idx[j]; break; }
  }
  free(idx); free(val);
  return out;
}

/* ---------------------------------------------------- speculative acceptance */

/* splitmix64 -> [0,1), src/llm/decoder.rs:643-650. */
static double tbo_splitmix_u01(uint64_t* st) {
  *st += 0x9E3779B97F4A7C15ull;
  uint64_t z = *st;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return (double)(z >> 11) / 9007199254740992.0;
}

/* src/llm/decoder.rs:616-634. */
static void tbo_softmax_row(const float* logits, int64_t v, float temp, float* out) {
  float t = (isfinite(temp) && temp > 0.0f) ? temp : 1.0f;
  float m = -INFINITY;
  for (int64_t j = 0; j < v; ++j) {
    float b = isfinite(logits[j]) ? logits[j] : -INFINITY;
    if (b > m) m = b;
  }
  float s = 0.f;
  for (int64_t j = 0; j < v; ++j) {
    float x = isfinite(logits[j]) ? logits[j] : -INFINITY;
    out[j] = expf((x - m) / t);
    s += out[j];
  }
  float inv = 1.0f / (s > 1e-30f ? s : 1e-30f);
  for (int64_t j = 0; j < v; ++j) out[j] *= inv;
}

/* src/llm/decoder.rs:651-726 on given target logits [k, v]; returns accepted, *bonus set.
 * The final sort is a selection in descending order that keeps equal items in index order. */
int64_t tbo_speculative_accept_rows(const float* target_logits, int64_t v, const int64_t* draft_tokens, int64_t k,
                                    const float* draft_probs, float temperature, float top_p, uint64_t* rng,
                                    int64_t* bonus) {
  *bonus = v - 1;
  if (k == 0) return 0;
  if (*rng == 0) *rng = 1;
  float* tp = (float*)malloc(sizeof(float) * (size_t)v);
  int64_t accepted = 0;
  for (int64_t i = 0; i < k; ++i) {
    tbo_softmax_row(target_logits + i * v, v, temperature, tp);
    const float* dp = draft_probs + i * v;
    int64_t tok = draft_tokens[i] < v - 1 ? draft_tokens[i] : v - 1;
    if (tok < 0) tok = 0;
    float p_target = tp[tok];
    float p_draft = dp[tok] > 0.0f ? dp[tok] : 0.0f;
    float accept = p_target / (p_draft + 1e-12f);
    if (accept > 1.0f) accept = 1.0f;
    if (tbo_splitmix_u01(rng) <= (double)accept) { ++accepted; continue; }
    float s = 0.f;
    for (int64_t j = 0; j < v; ++j) { float c = tp[j] - dp[j]; s += c > 0.0f ? c : 0.0f; }
    if (s > 1e-12f) {
      float r = (float)tbo_splitmix_u01(rng) * s, acc = 0.f;
      for (int64_t j = 0; j < v; ++j) {
        float c = tp[j] - dp[j];
        acc += c > 0.0f ? c : 0.0f;
        if (acc >= r) { *bonus = j; break; }
      }
    } else {
      int64_t b = 0;
      for (int64_t j = 1; j < v; ++j) if (tp[j] >= tp[b]) b = j;
      *bonus = b;
    }
    free(tp);
    return accepted;
  }
  tbo_softmax_row(target_logits + (k - 1) * v, v, temperature, tp);
  /* walk the probabilities in descending order without sorting: repeated selection is O(v*kept),
   * fine for the test sizes this oracle runs at */
  char* used = (char*)calloc((size_t)v, 1);
  int64_t* order = (int64_t*)malloc(sizeof(int64_t) * (size_t)v);
  for (int64_t i = 0; i < v; ++i) {
    int64_t best = -1;
    for (int64_t j = 0; j < v; ++j) if (!used[j] && (best < 0 || tp[j] > tp[best])) best = j;
    used[best] = 1; order[i] = best;
  }
  int64_t kept = v;
  if (top_p > 0.0f && top_p < 1.0f) {
    float cum = 0.f;
    for (int64_t i = 0; i < v; ++i) { if (cum > top_p) { kept = i; break; } cum += tp[order[i]]; }
    if (kept < 1) kept = 1;
  }
  float mass = 0.f;
  for (int64_t i = 0; i < kept; ++i) mass += tp[order[i]];
  float r = (float)tbo_splitmix_u01(rng) * (mass > 1e-30f ? mass : 1e-30f), acc = 0.f;
  *bonus = order[kept - 1];
  for (int64_t i = 0; i < kept; ++i) { acc += tp[order[i]]; if (acc >= r) { *bonus = order[i]; break; } }
  free(used); free(order); free(tp);
  return accepted;
}


/* ------------------------------------------------------------ v2 layout */

/* src/quantization/packed_v2.rs:67-112 (round to nearest even). */
uint16_t tbo_f32_to_f16(float v) {
  uint32_t x;
  memcpy(&x, &v, 4);
  uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
  int exp_abs = (int)((x >> 23) & 0xFF);
  uint32_t mant = x & 0x007FFFFFu;
  if (exp_abs == 0xFF) return (uint16_t)(mant == 0 ? (sign | 0x7C00u) : (sign | 0x7E00u));
  int e = exp_abs - 127;
  if (e > 15) return (uint16_t)(sign | 0x7C00u);
  if (e >= -14) {
    uint32_t h_exp = (uint32_t)(e + 15), h_mant = mant >> 13, rem = mant & 0x1FFFu;
    uint32_t h = (h_exp << 10) | h_mant;
    if (rem > 0x1000u || (rem == 0x1000u && (h_mant & 1u) == 1u)) h += 1;
    return (uint16_t)(sign | h);
  }
  if (e < -25) return sign;
  uint32_t full = mant | 0x00800000u;
  uint32_t shift = (uint32_t)(-e - 1);
  uint32_t h_mant = full >> shift, rem = full & ((1u << shift) - 1u), round = 1u << (shift - 1);
  uint32_t m = h_mant;
  if (rem > round || (rem == round && (h_mant & 1u) == 1u)) m += 1;
  return (uint16_t)(sign | m);
}

/* src/quantization/packed_v2.rs:30-57. */
float tbo_f16_to_f32(uint16_t bits) {
  uint32_t sign = (bits >> 15) & 1u, exp = (bits >> 10) & 0x1Fu, mant = bits & 0x3FFu;
  if (exp == 0) {
    if (mant == 0) return sign ? -0.0f : 0.0f;
    float v = ((float)mant / 1024.0f) * ldexpf(1.0f, -14);
    return sign ? -v : v;
  }
  if (exp == 0x1F) return mant == 0 ? (sign ? -INFINITY : INFINITY) : NAN;
  uint32_t o = (sign << 31) | ((exp + 112u) << 23) | (mant << 13);
  float f;
  memcpy(&f, &o, 4);
  return f;
}

/* src/quantization/packed_v2.rs:120-143. */
void tbo_pack_v1_to_v2(const uint8_t* w_packed, const float* scales, int64_t n, int64_t k, uint8_t* out) {
  int64_t ng = k / 64, src_row = (k + 1) / 2;
  for (int64_t row = 0; row < n; ++row)
    for (int64_t g = 0; g < ng; ++g) {
      uint8_t* dst = out + row * ng * 34 + g * 34;
      memcpy(dst, w_packed + row * src_row + g * 32, 32);
      uint16_t h = tbo_f32_to_f16(scales[row * ng + g]);
      dst[32] = (uint8_t)(h & 0xFF);
      dst[33] = (uint8_t)(h >> 8);
    }
}

/* src/quantization/packed_v2.rs:145-203 (scalar v2 row kernel): per group, dot of x with the
 * codes times the binary16 scale. */
void tbo_gemv_w4a32_v2(const float* x, const uint8_t* blocks, const float* bias, float* out, int64_t n, int64_t k) {
  int64_t ng = k / 64;
  for (int64_t row = 0; row < n; ++row) {
    float s = 0.0f;
    for (int64_t g = 0; g < ng; ++g) {
      const uint8_t* b = blocks + (row * ng + g) * 34;
      s += dot_group_scalar(x + g * 64, b, 64) * tbo_f16_to_f32((uint16_t)(b[32] | (b[33] << 8)));
    }
    out[row] = s + (bias ? bias[row] : 0.0f);
  }
}
