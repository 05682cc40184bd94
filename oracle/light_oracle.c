/*
 * light_oracle.c -- CPU restatement of the reference's quantized-weight matmul path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA kernels are compared
 * with and the timed CPU baseline; nothing in the product package may call it.
 *
 * Parity: pinned.  tests/test_oracle_*.py check every function here against the
 * reference's own known-answer tests (quant/q4_k_test.go:48-127, quant/q6_k_test.go:61-147,
 * quant/others_test.go:30-51, quant/quantize_test.go:13-45, ops/fp8_block_test.go:16-106,
 * ops/int4_test.go) re-expressed as data, and against independent codecs (numpy float16,
 * torch bfloat16 / float8_e4m3fn).  The one piece with nothing to pin against is the
 * K-quant ENCODER used to make synthetic weights: the reference has none
 * (quant/quantize.go:14-20), so that encoder lives in the test helpers, not here.
 *
 * Each function cites the reference file:line whose arithmetic it follows.  The
 * reference CPU path is Go + Plan 9 AVX2 assembly (no Go toolchain is available), so
 * this is a C restatement, not a build of the reference.  The reference's AVX2 row
 * decoders are bit-identical to its scalar Go decoders (kernels/cpu/qdecode_test.go:38-89),
 * so the scalar decoders below ARE the decode oracle, and the AVX2 row decoders restated
 * further down (with intrinsics) are what the timed matmul uses, as the reference's does;
 * compile with -ffp-contract=off so that `a*b - c` stays a separate multiply and subtract
 * exactly as Go on amd64 does.
 */
#define _GNU_SOURCE
#include <malloc.h>
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <immintrin.h>

#define LO_API __attribute__((visibility("default")))

/* ggml on-disk type codes (gguf/types.go:39-58). */
enum { LO_Q4_0 = 2, LO_Q5_0 = 6, LO_Q8_0 = 8, LO_Q4_K = 12, LO_Q5_K = 13, LO_Q6_K = 14 };

/* ------------------------------------------------------------------ codecs */

/* dtype/half.go:85-113 (Half.ToF32). */
LO_API float lo_f16_to_f32(uint16_t h) {
  uint32_t sign = (h >> 15) & 1u, exp = (h >> 10) & 0x1fu, mant = h & 0x3ffu, out;
  if (exp == 0) {
    if (mant == 0) {
      out = sign << 31;
    } else {
      float v = (float)mant * (1.0f / 16777216.0f); /* mant * 2^-24 */
      return sign ? -v : v;
    }
  } else if (exp == 0x1f) {
    out = mant == 0 ? (sign << 31 | 0x7f800000u) : (sign << 31 | 0x7fc00000u);
  } else {
    out = sign << 31 | (exp + 127 - 15) << 23 | mant << 13;
  }
  float f;
  memcpy(&f, &out, 4);
  return f;
}

/* dtype/half.go:15-83 (HalfFromF32, round to nearest even). */
LO_API uint16_t lo_f32_to_f16(float f) {
  uint32_t bits;
  memcpy(&bits, &f, 4);
  uint16_t sign = (uint16_t)((bits >> 31) & 1u);
  int32_t exp32 = (int32_t)((bits >> 23) & 0xffu);
  uint32_t mant32 = bits & 0x7fffffu;
  if (exp32 == 0xff) {
    if (mant32 == 0) return (uint16_t)(sign << 15 | 0x7c00);
    return (uint16_t)(sign << 15 | 0x7c00 | (uint16_t)(mant32 >> 13) | 0x200);
  }
  if (exp32 == 0) return (uint16_t)(sign << 15);
  int32_t e = exp32 - 127;
  if (e > 15) return (uint16_t)(sign << 15 | 0x7c00);
  if (e < -24) return (uint16_t)(sign << 15);
  if (e < -14) {
    uint32_t mant = mant32 | 0x800000u;
    uint32_t shift = (uint32_t)(-e - 14 + 13);
    uint32_t h = mant >> shift;
    uint32_t rem = mant & ((1u << shift) - 1u), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (h & 1u))) h++;
    return (uint16_t)(sign << 15 | (uint16_t)h);
  }
  uint32_t hexp = (uint32_t)(e + 15), hmant = mant32 >> 13, rem = mant32 & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (hmant & 1u))) {
    hmant++;
    if (hmant > 0x3ffu) {
      hmant = 0;
      hexp++;
      if (hexp >= 31) return (uint16_t)(sign << 15 | 0x7c00);
    }
  }
  return (uint16_t)(sign << 15 | (uint16_t)(hexp << 10) | (uint16_t)hmant);
}

/* dtype/half.go:115-133 (BF16FromF32, RNE with quiet-NaN guard; BFloat16.ToF32). */
LO_API uint16_t lo_f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7f800000u) == 0x7f800000u && (u & 0x7fffffu) != 0) return (uint16_t)((u >> 16) | 0x0040u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
LO_API float lo_bf16_to_f32(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* dtype/f8.go:57-71 (Float8.ToF32, e4m3fn: bias 7, no inf, NaN = 0x7F/0xFF). */
LO_API float lo_e4m3_to_f32(uint8_t x) {
  float sign = (x & 0x80) ? -1.0f : 1.0f;
  if ((x & 0x7F) == 0x7F) return NAN;
  int exp = (x >> 3) & 0xF;
  float m = (float)(x & 7);
  if (exp == 0) return sign * m * (1.0f / 512.0f);
  return sign * (1.0f + m / 8.0f) * ldexpf(1.0f, exp - 7);
}

/* dtype/f8.go:21-55 (F8FromF32, RNE, saturating to +-448). */
LO_API uint8_t lo_f32_to_e4m3(float f) {
  if (f != f) return 0x7F;
  uint8_t sign = 0;
  double v = (double)f;
  if (signbit(v)) {
    sign = 0x80;
    v = -v;
  }
  if (v >= 448.0) return (uint8_t)(sign | 0x7E);
  if (v < 1.0 / 64) {
    double m = nearbyint(v / (1.0 / 512)); /* default rounding mode: to nearest even */
    if (m >= 8) return (uint8_t)(sign | 0x08);
    return (uint8_t)(sign | (uint8_t)m);
  }
  double e = floor(log2(v));
  double mant = v / ldexp(1.0, (int)e) - 1.0;
  double m = nearbyint(mant * 8);
  if (m >= 8) {
    m = 0;
    e += 1;
  }
  int exp = (int)e + 7;
  if (exp >= 16 || (exp == 15 && m >= 7)) return (uint8_t)(sign | 0x7E);
  return (uint8_t)(sign | (uint8_t)(exp << 3) | (uint8_t)m);
}

/* ------------------------------------------------------- block geometry */

/* dtype/dtype.go:53-60 (blockInfo). */
LO_API int lo_block_elems(int dt) {
  switch (dt) {
    case LO_Q4_0: case LO_Q5_0: case LO_Q8_0: return 32;
    case LO_Q4_K: case LO_Q5_K: case LO_Q6_K: return 256;
  }
  return 0;
}
LO_API int lo_block_bytes(int dt) {
  switch (dt) {
    case LO_Q4_0: return 18;
    case LO_Q5_0: return 22;
    case LO_Q8_0: return 34;
    case LO_Q4_K: return 144;
    case LO_Q5_K: return 176;
    case LO_Q6_K: return 210;
  }
  return 0;
}

/* ------------------------------------------------------------ decoders */

static inline float f16le(const uint8_t *p) { return lo_f16_to_f32((uint16_t)(p[0] | p[1] << 8)); }

/* quant/q4_k.go:82-89 (getScaleMinK4). */
static inline void scale_min_k4(int j, const uint8_t *q, uint8_t *sc, uint8_t *m) {
  if (j < 4) {
    *sc = q[j] & 63;
    *m = q[j + 4] & 63;
  } else {
    *sc = (uint8_t)((q[j + 4] & 0x0F) | ((q[j - 4] >> 6) << 4));
    *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
  }
}

/* kernels/cpu/quant_matmul.go:30-35 / quant/q8_0.go:46-53: y = d * q. */
static void dec_q8_0(const uint8_t *b, float *dst) {
  float d = f16le(b);
  for (int i = 0; i < 32; i++) dst[i] = d * (float)(int8_t)b[2 + i];
}
/* kernels/cpu/quant_matmul.go:36-43: y = d * (nibble - 8). */
static void dec_q4_0(const uint8_t *b, float *dst) {
  float d = f16le(b);
  for (int j = 0; j < 16; j++) {
    uint8_t q = b[2 + j];
    dst[j] = d * (float)((int)(q & 15) - 8);
    dst[j + 16] = d * (float)((int)(q >> 4) - 8);
  }
}
/* kernels/cpu/quant_matmul.go:44-54: fifth bit from qh, y = d * (q - 16). */
static void dec_q5_0(const uint8_t *b, float *dst) {
  float d = f16le(b);
  uint32_t qh = (uint32_t)b[2] | (uint32_t)b[3] << 8 | (uint32_t)b[4] << 16 | (uint32_t)b[5] << 24;
  for (int j = 0; j < 16; j++) {
    uint8_t q = b[6 + j];
    int lo = (int)(q & 15) | (int)((qh >> j) & 1u) << 4;
    int hi = (int)(q >> 4) | (int)((qh >> (j + 16)) & 1u) << 4;
    dst[j] = d * (float)(lo - 16);
    dst[j + 16] = d * (float)(hi - 16);
  }
}
/* kernels/cpu/quant_matmul.go:55-69 / quant/q4_k.go:55-76: y = (d*sc)*q - (dmin*m),
 * three separately rounded f32 operations. */
static void dec_q4_k(const uint8_t *b, float *dst) {
  float d = f16le(b), dmin = f16le(b + 2);
  const uint8_t *scales = b + 4, *qs = b + 16;
  for (int p = 0; p < 4; p++) {
    uint8_t sc0, m0, sc1, m1;
    scale_min_k4(2 * p, scales, &sc0, &m0);
    scale_min_k4(2 * p + 1, scales, &sc1, &m1);
    float d1 = d * (float)sc0, mo1 = dmin * (float)m0;
    float d2 = d * (float)sc1, mo2 = dmin * (float)m1;
    for (int l = 0; l < 32; l++) {
      uint8_t q = qs[p * 32 + l];
      dst[p * 64 + l] = d1 * (float)(q & 15) - mo1;
      dst[p * 64 + 32 + l] = d2 * (float)(q >> 4) - mo2;
    }
  }
}
/* kernels/cuda/src/matmul_q.cu:200-228 and dequant.cu (Q5_K): Q4_K plus a fifth bit
 * from qh[32]; bit 2p for the low-nibble half, 2p+1 for the high-nibble half. */
static void dec_q5_k(const uint8_t *b, float *dst) {
  float d = f16le(b), dmin = f16le(b + 2);
  const uint8_t *scales = b + 4, *qh = b + 16, *qs = b + 48;
  for (int p = 0; p < 4; p++) {
    uint8_t sc0, m0, sc1, m1;
    scale_min_k4(2 * p, scales, &sc0, &m0);
    scale_min_k4(2 * p + 1, scales, &sc1, &m1);
    float d1 = d * (float)sc0, mo1 = dmin * (float)m0;
    float d2 = d * (float)sc1, mo2 = dmin * (float)m1;
    unsigned bit0 = 1u << (2 * p), bit1 = 1u << (2 * p + 1);
    for (int l = 0; l < 32; l++) {
      uint8_t q = qs[p * 32 + l];
      unsigned h = qh[l];
      unsigned lo = (unsigned)(q & 15) | ((h & bit0) ? 16u : 0u);
      unsigned hi = (unsigned)(q >> 4) | ((h & bit1) ? 16u : 0u);
      dst[p * 64 + l] = d1 * (float)lo - mo1;
      dst[p * 64 + 32 + l] = d2 * (float)hi - mo2;
    }
  }
}
/* kernels/cpu/quant_matmul.go:70-88 / quant/q6_k.go:65-93: y = (d*sc)*(q-32). */
static void dec_q6_k(const uint8_t *b, float *dst) {
  const uint8_t *ql = b, *qh = b + 128;
  const int8_t *sc = (const int8_t *)(b + 192);
  float d = f16le(b + 208);
  for (int half = 0; half < 2; half++) {
    int qlB = half * 64, qhB = half * 32, scB = half * 8, y = half * 128;
    for (int l = 0; l < 32; l++) {
      int is = l >> 4;
      uint8_t h = qh[qhB + l];
      int q1 = ((int)(ql[qlB + l] & 15) | (int)(h & 3) << 4) - 32;
      int q2 = ((int)(ql[qlB + l + 32] & 15) | (int)((h >> 2) & 3) << 4) - 32;
      int q3 = ((int)(ql[qlB + l] >> 4) | (int)((h >> 4) & 3) << 4) - 32;
      int q4 = ((int)(ql[qlB + l + 32] >> 4) | (int)((h >> 6) & 3) << 4) - 32;
      dst[y + l] = d * (float)sc[scB + is] * (float)q1;
      dst[y + l + 32] = d * (float)sc[scB + 2 + is] * (float)q2;
      dst[y + l + 64] = d * (float)sc[scB + 4 + is] * (float)q3;
      dst[y + l + 96] = d * (float)sc[scB + 6 + is] * (float)q4;
    }
  }
}

typedef void (*block_dec)(const uint8_t *, float *);
static block_dec decoder_for(int dt) {
  switch (dt) {
    case LO_Q4_0: return dec_q4_0;
    case LO_Q5_0: return dec_q5_0;
    case LO_Q8_0: return dec_q8_0;
    case LO_Q4_K: return dec_q4_k;
    case LO_Q5_K: return dec_q5_k;
    case LO_Q6_K: return dec_q6_k;
  }
  return 0;
}

/* quant.Dequantize for the fused formats: blocks -> f32.  Returns 0, or -1 on a bad
 * dtype / element count (quant/q4_k.go:29-36: n must be a whole number of blocks). */
LO_API int lo_dequant(int dt, const uint8_t *src, float *dst, int64_t n) {
  block_dec dec = decoder_for(dt);
  int be = lo_block_elems(dt), bb = lo_block_bytes(dt);
  if (!dec || n < 0 || n % be) return -1;
  for (int64_t b = 0; b < n / be; b++) dec(src + b * bb, dst + b * be);
  return 0;
}

/* quant/quantize.go:70-86 (encodeQ8_0): d = amax/127, q = RoundToEven(v * (1/d)). */
LO_API int lo_quantize_q8_0(const float *src, uint8_t *dst, int64_t n) {
  if (n < 0 || n % 32) return -1;
  for (int64_t b = 0; b < n / 32; b++) {
    const float *blk = src + b * 32;
    uint8_t *o = dst + b * 34;
    float amax = 0;
    for (int i = 0; i < 32; i++) {
      float a = fabsf(blk[i]);
      if (a > amax) amax = a;
    }
    float d = amax / 127, id = d != 0 ? 1 / d : 0;
    uint16_t h = lo_f32_to_f16(d);
    o[0] = (uint8_t)h;
    o[1] = (uint8_t)(h >> 8);
    for (int i = 0; i < 32; i++) o[2 + i] = (uint8_t)(int8_t)nearbyint((double)(blk[i] * id));
  }
  return 0;
}

/* --------------------------------------------------- f32 tile arithmetic */

/* internal/simd/simd_amd64.s:6-56 (dotAVX2): four 8-lane FMA accumulators over 32-float
 * strides, single-accumulator 8-float steps, (Y0+Y1)+(Y2+Y3), 128-bit halves, two
 * horizontal adds, scalar FMA tail. */
__attribute__((target("avx2,fma"))) static float dot_avx2(const float *a, const float *b, int n) {
  __m256 y0 = _mm256_setzero_ps(), y1 = y0, y2 = y0, y3 = y0;
  while (n >= 32) {
    y0 = _mm256_fmadd_ps(_mm256_loadu_ps(a), _mm256_loadu_ps(b), y0);
    y1 = _mm256_fmadd_ps(_mm256_loadu_ps(a + 8), _mm256_loadu_ps(b + 8), y1);
    y2 = _mm256_fmadd_ps(_mm256_loadu_ps(a + 16), _mm256_loadu_ps(b + 16), y2);
    y3 = _mm256_fmadd_ps(_mm256_loadu_ps(a + 24), _mm256_loadu_ps(b + 24), y3);
    a += 32, b += 32, n -= 32;
  }
  while (n >= 8) {
    y0 = _mm256_fmadd_ps(_mm256_loadu_ps(a), _mm256_loadu_ps(b), y0);
    a += 8, b += 8, n -= 8;
  }
  y0 = _mm256_add_ps(_mm256_add_ps(y0, y1), _mm256_add_ps(y2, y3));
  __m128 x = _mm_add_ps(_mm256_castps256_ps128(y0), _mm256_extractf128_ps(y0, 1));
  x = _mm_hadd_ps(x, x);
  x = _mm_hadd_ps(x, x);
  float s = _mm_cvtss_f32(x);
  for (; n > 0; n--) s = fmaf(*a++, *b++, s);
  return s;
}

/* internal/simd/simd.go:41-54 (dotGo), used when AVX2+FMA is absent. */
static float dot_scalar(const float *a, const float *b, int n) {
  float s0 = 0, s1 = 0, s2 = 0, s3 = 0;
  int i = 0;
  for (; i + 4 <= n; i += 4) {
    s0 += a[i] * b[i];
    s1 += a[i + 1] * b[i + 1];
    s2 += a[i + 2] * b[i + 2];
    s3 += a[i + 3] * b[i + 3];
  }
  for (; i < n; i++) s0 += a[i] * b[i];
  return (s0 + s1) + (s2 + s3);
}

static int g_avx2 = -1;
static int have_avx2(void) {
  if (g_avx2 < 0) g_avx2 = __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma");
  return g_avx2;
}
static float dot(const float *a, const float *b, int n) { return have_avx2() ? dot_avx2(a, b, n) : dot_scalar(a, b, n); }

__attribute__((target("avx2,fma"))) static inline float hsum256(__m256 y) {
  __m128 x = _mm_add_ps(_mm256_castps256_ps128(y), _mm256_extractf128_ps(y, 1));
  x = _mm_hadd_ps(x, x);
  x = _mm_hadd_ps(x, x);
  return _mm_cvtss_f32(x);
}

/* internal/simd/simd_amd64.s:127-205 (dot4x3AVX2): 4 activation rows x 3 weight rows,
 * one accumulator per output, k a multiple of 8. */
__attribute__((target("avx2,fma"))) static void dot4x3_avx2(const float *a, int lda, const float *w, int ldw, int k,
                                                           float *out) {
  __m256 c[12];
  for (int i = 0; i < 12; i++) c[i] = _mm256_setzero_ps();
  for (int t = 0; t < k; t += 8) {
    __m256 w0 = _mm256_loadu_ps(w + t), w1 = _mm256_loadu_ps(w + ldw + t), w2 = _mm256_loadu_ps(w + 2 * ldw + t);
    for (int r = 0; r < 4; r++) {
      __m256 av = _mm256_loadu_ps(a + (size_t)r * lda + t);
      c[3 * r] = _mm256_fmadd_ps(av, w0, c[3 * r]);
      c[3 * r + 1] = _mm256_fmadd_ps(av, w1, c[3 * r + 1]);
      c[3 * r + 2] = _mm256_fmadd_ps(av, w2, c[3 * r + 2]);
    }
  }
  for (int i = 0; i < 12; i++) out[i] = hsum256(c[i]);
}

/* internal/simd/simd.go:56-90 (MatTB): out[i*ldo+j] = sum_t a[i*lda+t] * w[j*ldw+t]. */
static void mat_tb(const float *a, int lda, const float *w, int ldw, float *out, int ldo, int m, int n, int k) {
  int i = 0;
  if (have_avx2() && k % 8 == 0 && k > 0) {
    float t[12];
    for (; i + 4 <= m; i += 4) {
      int j = 0;
      for (; j + 3 <= n; j += 3) {
        dot4x3_avx2(a + (size_t)i * lda, lda, w + (size_t)j * ldw, ldw, k, t);
        for (int r = 0; r < 4; r++) {
          float *o = out + (size_t)(i + r) * ldo + j;
          o[0] = t[3 * r], o[1] = t[3 * r + 1], o[2] = t[3 * r + 2];
        }
      }
      for (; j < n; j++)
        for (int r = 0; r < 4; r++) out[(size_t)(i + r) * ldo + j] = dot(a + (size_t)(i + r) * lda, w + (size_t)j * ldw, k);
    }
  }
  for (; i < m; i++)
    for (int j = 0; j < n; j++) out[(size_t)i * ldo + j] = dot(a + (size_t)i * lda, w + (size_t)j * ldw, k);
}

/* --------------------------------------------------------- parallel.For */

typedef void (*range_fn)(int lo, int hi, void *ctx);
typedef struct {
  range_fn fn;
  void *ctx;
  int lo, hi;
} par_job;
static void *par_tramp(void *p) {
  par_job *j = (par_job *)p;
  j->fn(j->lo, j->hi, j->ctx);
  return 0;
}

/* internal/parallel/parallel.go:11-37 (For): static contiguous chunks, at least `grain`
 * items each, `threads` workers standing in for GOMAXPROCS. */
static void parallel_for(int n, int grain, int threads, range_fn fn, void *ctx) {
  if (n <= 0) return;
  int workers = threads < 1 ? 1 : threads;
  if (grain < 1) grain = 1;
  if (n / grain < workers) workers = n / grain;
  if (workers <= 1) {
    fn(0, n, ctx);
    return;
  }
  int chunk = (n + workers - 1) / workers, cnt = 0;
  pthread_t *th = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)workers);
  par_job *jobs = (par_job *)malloc(sizeof(par_job) * (size_t)workers);
  for (int lo = 0; lo < n; lo += chunk, cnt++) {
    jobs[cnt] = (par_job){fn, ctx, lo, lo + chunk < n ? lo + chunk : n};
    pthread_create(&th[cnt], 0, par_tramp, &jobs[cnt]);
  }
  for (int i = 0; i < cnt; i++) pthread_join(th[i], 0);
  free(th);
  free(jobs);
}

/* ------------------------------------------------ AVX2 row decoders
 *
 * kernels/cpu/qdecode_amd64.s:33-285 with its driver decodeRowAVX2 (kernels/cpu/quant_matmul.go:208-250):
 * the reference's CPU matmul decodes Q8_0 / Q4_0 / Q5_0 / Q4_K / Q6_K rows (and int4 rows) eight lanes at
 * a time -- the integer code is formed per lane, converted to f32 and scaled with the same operations in
 * the same order as the scalar decoders, so the floats are identical (the reference asserts this in
 * kernels/cpu/qdecode_test.go:38-89; tests/test_oracle_avx2.py asserts it for this restatement).  These
 * are what lo_matmul_q times when the host has AVX2 + FMA + F16C, as the reference's matmulQCPU does. */

#define LO_AVX2 __attribute__((target("avx2,fma,f16c")))

LO_AVX2 static inline __m256i ld8_u8(const uint8_t *p) { return _mm256_cvtepu8_epi32(_mm_loadl_epi64((const __m128i *)p)); }
LO_AVX2 static inline __m256i ld8_s8(const uint8_t *p) { return _mm256_cvtepi8_epi32(_mm_loadl_epi64((const __m128i *)p)); }

/* qdecode_amd64.s:33-68 (q8_0RowAVX2): d * float(int8). */
LO_AVX2 static void row_q8_0_avx2(const uint8_t *raw, float *dst, int K) {
  for (int b = 0; b < K / 32; b++, raw += 34, dst += 32) {
    const __m256 d = _mm256_set1_ps(f16le(raw));
    for (int i = 0; i < 4; i++) _mm256_storeu_ps(dst + 8 * i, _mm256_mul_ps(_mm256_cvtepi32_ps(ld8_s8(raw + 2 + 8 * i)), d));
  }
}
/* qdecode_amd64.s:70-114 (q4_0RowAVX2): d * float(nibble - 8); low nibbles are elements 0..15, high 16..31. */
LO_AVX2 static void row_q4_0_avx2(const uint8_t *raw, float *dst, int K) {
  const __m256i m15 = _mm256_set1_epi32(15), off = _mm256_set1_epi32(8);
  for (int b = 0; b < K / 32; b++, raw += 18, dst += 32) {
    const __m256 d = _mm256_set1_ps(f16le(raw));
    for (int h = 0; h < 2; h++) {
      const __m256i v = ld8_u8(raw + 2 + 8 * h);
      const __m256i lo = _mm256_sub_epi32(_mm256_and_si256(v, m15), off), hi = _mm256_sub_epi32(_mm256_srli_epi32(v, 4), off);
      _mm256_storeu_ps(dst + 8 * h, _mm256_mul_ps(_mm256_cvtepi32_ps(lo), d));
      _mm256_storeu_ps(dst + 16 + 8 * h, _mm256_mul_ps(_mm256_cvtepi32_ps(hi), d));
    }
  }
}
/* qdecode_amd64.s:116-161 (q5_0RowAVX2): the fifth bit of element e is bit e of the 32-bit qh; offset 16. */
LO_AVX2 static void row_q5_0_avx2(const uint8_t *raw, float *dst, int K) {
  const __m256i m15 = _mm256_set1_epi32(15), one = _mm256_set1_epi32(1), off = _mm256_set1_epi32(16);
  const __m256i lanes = _mm256_setr_epi32(0, 1, 2, 3, 4, 5, 6, 7);
  for (int b = 0; b < K / 32; b++, raw += 22, dst += 32) {
    const __m256 d = _mm256_set1_ps(f16le(raw));
    uint32_t qhw;
    memcpy(&qhw, raw + 2, 4);
    const __m256i qh = _mm256_set1_epi32((int)qhw);
    for (int h = 0; h < 2; h++) {
      const __m256i v = ld8_u8(raw + 6 + 8 * h);
      const __m256i sl = _mm256_add_epi32(lanes, _mm256_set1_epi32(8 * h)), sh = _mm256_add_epi32(sl, _mm256_set1_epi32(16));
      const __m256i bl = _mm256_slli_epi32(_mm256_and_si256(_mm256_srlv_epi32(qh, sl), one), 4);
      const __m256i bh = _mm256_slli_epi32(_mm256_and_si256(_mm256_srlv_epi32(qh, sh), one), 4);
      const __m256i lo = _mm256_sub_epi32(_mm256_or_si256(_mm256_and_si256(v, m15), bl), off);
      const __m256i hi = _mm256_sub_epi32(_mm256_or_si256(_mm256_srli_epi32(v, 4), bh), off);
      _mm256_storeu_ps(dst + 8 * h, _mm256_mul_ps(_mm256_cvtepi32_ps(lo), d));
      _mm256_storeu_ps(dst + 16 + 8 * h, _mm256_mul_ps(_mm256_cvtepi32_ps(hi), d));
    }
  }
}
/* qdecode_amd64.s:163-205 (q4KBlockAVX2) + quant_matmul.go:225-236: sc[j] = d * scale_j and mn[j] = dmin * min_j
 * are formed first (scalar), then q * sc - mn as a separate multiply and subtract (VMULPS, VSUBPS). */
LO_AVX2 static void row_q4_k_avx2(const uint8_t *raw, float *dst, int K) {
  const __m256i m15 = _mm256_set1_epi32(15);
  for (int b = 0; b < K / 256; b++, raw += 144, dst += 256) {
    const float d = f16le(raw), dmin = f16le(raw + 2);
    float sc[8], mn[8];
    for (int j = 0; j < 8; j++) {
      uint8_t s, m;
      scale_min_k4(j, raw + 4, &s, &m);
      sc[j] = d * (float)s, mn[j] = dmin * (float)m;
    }
    const uint8_t *qs = raw + 16;
    for (int p = 0; p < 4; p++) {
      const __m256 s0 = _mm256_set1_ps(sc[2 * p]), m0 = _mm256_set1_ps(mn[2 * p]);
      const __m256 s1 = _mm256_set1_ps(sc[2 * p + 1]), m1 = _mm256_set1_ps(mn[2 * p + 1]);
      for (int c = 0; c < 4; c++) {
        const __m256i v = ld8_u8(qs + 32 * p + 8 * c);
        const __m256 lo = _mm256_cvtepi32_ps(_mm256_and_si256(v, m15)), hi = _mm256_cvtepi32_ps(_mm256_srli_epi32(v, 4));
        _mm256_storeu_ps(dst + 64 * p + 8 * c, _mm256_sub_ps(_mm256_mul_ps(lo, s0), m0));
        _mm256_storeu_ps(dst + 64 * p + 32 + 8 * c, _mm256_sub_ps(_mm256_mul_ps(hi, s1), m1));
      }
    }
  }
}
/* qdecode_amd64.s:207-245 (q6KBlockAVX2) + quant_matmul.go:237-247: sc[j] = d * int8 scale first, then
 * float(q - 32) * sc for the four quarters of each half. */
LO_AVX2 static void row_q6_k_avx2(const uint8_t *raw, float *dst, int K) {
  const __m256i m15 = _mm256_set1_epi32(15), m3 = _mm256_set1_epi32(3), off = _mm256_set1_epi32(32);
  for (int b = 0; b < K / 256; b++, raw += 210, dst += 256) {
    const float d = f16le(raw + 208);
    float sc[16];
    for (int j = 0; j < 16; j++) sc[j] = d * (float)(int8_t)raw[192 + j];
    for (int half = 0; half < 2; half++) {
      const uint8_t *ql = raw + 64 * half, *qh = raw + 128 + 32 * half;
      const float *s = sc + 8 * half;
      float *y = dst + 128 * half;
      for (int c = 0; c < 4; c++) {  /* l = 8c .. 8c+7; is = l / 16 */
        const int is = c >> 1;
        const __m256i a = ld8_u8(ql + 8 * c), bq = ld8_u8(ql + 32 + 8 * c), h = ld8_u8(qh + 8 * c);
        const __m256i nib[4] = {_mm256_and_si256(a, m15), _mm256_and_si256(bq, m15), _mm256_srli_epi32(a, 4), _mm256_srli_epi32(bq, 4)};
        for (int q = 0; q < 4; q++) {
          const __m256i hi = _mm256_slli_epi32(_mm256_and_si256(_mm256_srli_epi32(h, 2 * q), m3), 4);
          const __m256i code = _mm256_sub_epi32(_mm256_or_si256(nib[q], hi), off);
          _mm256_storeu_ps(y + 32 * q + 8 * c, _mm256_mul_ps(_mm256_cvtepi32_ps(code), _mm256_set1_ps(s[2 * q + is])));
        }
      }
    }
  }
}
/* qdecode_amd64.s:248-285 (int4RowAVX2): word w holds elements 8w .. 8w+7; s * (float(q) - z), the subtract in f32. */
LO_AVX2 static void row_int4_avx2(const uint32_t *words, const float *s, const float *z, float *dst, int groups, int wpg) {
  const __m256i m15 = _mm256_set1_epi32(15), sh = _mm256_setr_epi32(0, 4, 8, 12, 16, 20, 24, 28);
  for (int g = 0; g < groups; g++) {
    const __m256 sv = _mm256_set1_ps(s[g]), zv = _mm256_set1_ps(z[g]);
    for (int w = 0; w < wpg; w++, words++, dst += 8) {
      const __m256i q = _mm256_and_si256(_mm256_srlv_epi32(_mm256_set1_epi32((int)*words), sh), m15);
      _mm256_storeu_ps(dst, _mm256_mul_ps(_mm256_sub_ps(_mm256_cvtepi32_ps(q), zv), sv));
    }
  }
}

typedef void (*row_avx2)(const uint8_t *, float *, int);
/* ggufAVX2 (kernels/cpu/quant_matmul.go:172-176): the formats decodeRowAVX2 handles. */
static row_avx2 avx2_row_for(int dt) {
  switch (dt) {
    case LO_Q8_0: return row_q8_0_avx2;
    case LO_Q4_0: return row_q4_0_avx2;
    case LO_Q5_0: return row_q5_0_avx2;
    case LO_Q4_K: return row_q4_k_avx2;
    case LO_Q6_K: return row_q6_k_avx2;
  }
  return 0;
}
static int have_avx2(void);

/* One row of K elements through the AVX2 decoder of its format.  Returns -1 when the format has none or the
 * host lacks AVX2 (the caller then uses the scalar decoders, as the reference does). */
LO_API int lo_decode_row_avx2(int dt, const uint8_t *raw, float *dst, int K) {
  row_avx2 f = avx2_row_for(dt);
  if (!f || !have_avx2() || K <= 0 || K % lo_block_elems(dt)) return -1;
  f(raw, dst, K);
  return 0;
}
LO_API int lo_int4_row_avx2(const uint32_t *codes, const float *s, const float *z, float *dst, int K, int G) {
  if (!have_avx2() || G <= 0 || G % 8 || K % G) return -1;
  row_int4_avx2(codes, s, z, dst, K / G, G / 8);
  return 0;
}
/* 1 when lo_matmul_q / lo_matmul_int4 decode rows with the AVX2 decoders on this host. */
LO_API int lo_uses_avx2(void) { return have_avx2(); }

/* ------------------------------------------------ x (M,K) . W^T, W quantized */

#define TILE_ROWS 48 /* kernels/cpu/matmul_f32.go:9 */

typedef void (*row_dec)(int n, float *dst, void *ctx);
typedef struct {
  const float *x;
  float *out;
  int M, K, N;
  row_dec dec;
  void *dctx;
} rtx;

/* kernels/cpu/quant_matmul.go:118-137 (rowsTimesX): decode up to 48 weight rows, then
 * one MatTB of all M activation rows against them. */
static void rtx_range(int lo, int hi, void *p) {
  rtx *r = (rtx *)p;
  float *rows = (float *)malloc(sizeof(float) * (size_t)TILE_ROWS * (size_t)r->K);
  for (int n0 = lo; n0 < hi; n0 += TILE_ROWS) {
    int n1 = n0 + TILE_ROWS < hi ? n0 + TILE_ROWS : hi;
    for (int n = n0; n < n1; n++) r->dec(n, rows + (size_t)(n - n0) * r->K, r->dctx);
    mat_tb(r->x, r->K, rows, r->K, r->out + n0, r->N, r->M, n1 - n0, r->K);
  }
  free(rows);
}
static void rows_times_x(const float *x, float *out, int M, int K, int N, int threads, row_dec dec, void *dctx) {
  static int tuned;
  if (!tuned) { /* keep the per-worker row tiles (up to a few MB) on the heap instead of a fresh mmap per call */
    mallopt(M_MMAP_THRESHOLD, 1 << 30);
    mallopt(M_TRIM_THRESHOLD, 1 << 30);
    tuned = 1;
  }
  rtx r = {x, out, M, K, N, dec, dctx};
  int grain = 16384 / (K + 1);
  parallel_for(N, grain < 1 ? 1 : grain, threads, rtx_range, &r);
}

typedef struct {
  const uint8_t *w;
  block_dec dec;
  int be, bb, K;
  row_avx2 fast; /* non-null: kernels/cpu/quant_matmul.go:153-166, the AVX2 row decoder (K / 32 <= 2048) */
} gguf_ctx;
static void gguf_row(int n, float *dst, void *p) {
  gguf_ctx *g = (gguf_ctx *)p;
  const uint8_t *row = g->w + (size_t)n * (size_t)(g->K / g->be) * (size_t)g->bb;
  if (g->fast) {
    g->fast(row, dst, g->K);
    return;
  }
  for (int b = 0; b < g->K / g->be; b++) g->dec(row + (size_t)b * g->bb, dst + (size_t)b * g->be);
}

/* kernels/cpu/quant_matmul.go:139-170 (matmulQCPU): out (M,N) f32 = x (M,K) f32 times the
 * (N,K) block-quantized weight transposed. */
LO_API int lo_matmul_q(int dt, const float *x, const uint8_t *w, float *out, int M, int N, int K, int threads) {
  block_dec dec = decoder_for(dt);
  if (!dec || M < 0 || N < 0 || K <= 0 || K % lo_block_elems(dt)) return -1;
  gguf_ctx g = {w, dec, lo_block_elems(dt), lo_block_bytes(dt), K, 0};
  if (have_avx2() && __builtin_cpu_supports("f16c") && K / 32 <= 2048) g.fast = avx2_row_for(dt);
  rows_times_x(x, out, M, K, N, threads, gguf_row, &g);
  return 0;
}

/* ------------------------------------------------------------ int4 (GPTQ / AWQ) */

/* quant/int4.go:239-261 (Int4.Dequant) and kernels/cpu/int4.go:22-53 (int4DequantCPU):
 * W[n,k] = s[n,k/G] * (code - z[n,k/G]) in f32, rounded once when out is bf16. */
LO_API int lo_int4_dequant(const uint32_t *codes, const float *s, const float *z, void *out, int N, int K, int G,
                           int out_bf16) {
  if (G <= 0 || K % 8 || K % G) return -1;
  int ng = K / G;
  for (int n = 0; n < N; n++)
    for (int k = 0; k < K; k++) {
      int g = n * ng + k / G;
      float v = s[g] * ((float)((codes[(size_t)n * (K / 8) + k / 8] >> (4 * (k % 8))) & 0xF) - z[g]);
      if (out_bf16)
        ((uint16_t *)out)[(size_t)n * K + k] = lo_f32_to_bf16(v);
      else
        ((float *)out)[(size_t)n * K + k] = v;
    }
  return 0;
}

typedef struct {
  const uint32_t *codes;
  const float *s, *z;
  int K, G;
} int4_ctx;
static void int4_row(int n, float *dst, void *p) {
  int4_ctx *c = (int4_ctx *)p;
  int ng = c->K / c->G;
  const uint32_t *words = c->codes + (size_t)n * (c->K / 8);
  if (have_avx2() && c->G % 8 == 0) {  /* kernels/cpu/quant_matmul.go:188-191 */
    row_int4_avx2(words, c->s + (size_t)n * ng, c->z + (size_t)n * ng, dst, ng, c->G / 8);
    return;
  }
  for (int g = 0; g < ng; g++) {
    float s = c->s[(size_t)n * ng + g], z = c->z[(size_t)n * ng + g];
    for (int k = g * c->G; k < (g + 1) * c->G; k += 8) {
      uint32_t w = words[k / 8];
      for (int j = 0; j < 8; j++) dst[k + j] = s * ((float)((w >> (4 * j)) & 15) - z);
    }
  }
}

/* kernels/cpu/quant_matmul.go:175-203 (int4MatMulCPU): row decode + MatTB, any M. */
LO_API int lo_int4_matmul(const float *x, const uint32_t *codes, const float *s, const float *z, float *out, int M,
                          int N, int K, int G, int threads) {
  if (G <= 0 || K % 8 || K % G || G % 8) return -1;
  int4_ctx c = {codes, s, z, K, G};
  rows_times_x(x, out, M, K, N, threads, int4_row, &c);
  return 0;
}

static inline uint8_t nib(uint32_t w, int j) { return (uint8_t)((w >> (4 * j)) & 0xF); }

/* quant/int4.go:103-196 (FromGPTQ, ordered groups only here): qweight i32 (K/8,N) packed
 * along K, qzeros i32 (K/G,N/8) packed along N (v1 stores zero-1), scales f32 (K/G,N)
 * -> canonical codes u32 (N,K/8), scales/zeros f32 (N,K/G). */
LO_API int lo_int4_from_gptq(const uint32_t *qweight, const uint32_t *qzeros, const float *scales, int K, int N,
                             int group, int v2, uint32_t *codes, float *sc, float *zr) {
  if (group <= 0) group = K;
  if (K % 8 || N % 8 || K % group) return -1;
  int G = K / group;
  for (int g = 0; g < G; g++)
    for (int n = 0; n < N; n++) {
      sc[(size_t)n * G + g] = scales[(size_t)g * N + n];
      float z = (float)nib(qzeros[(size_t)g * (N / 8) + n / 8], n % 8);
      zr[(size_t)n * G + g] = v2 ? z : z + 1;
    }
  for (int n = 0; n < N; n++)
    for (int c = 0; c < K / 8; c++) {
      uint32_t w = 0;
      for (int j = 0; j < 8; j++) {
        int r = 8 * c + j;
        w |= (uint32_t)nib(qweight[(size_t)(r / 8) * N + n], r % 8) << (4 * j);
      }
      codes[(size_t)n * (K / 8) + c] = w;
    }
  return 0;
}

/* quant/int4.go:198-235 (FromAWQ): qweight i32 (K,N/8) and qzeros (K/G,N/8) packed along N
 * in AutoAWQ order (nibble i holds column 8c + {0,2,4,6,1,3,5,7}[i]). */
LO_API int lo_int4_from_awq(const uint32_t *qweight, const uint32_t *qzeros, const float *scales, int K, int N,
                            int group, uint32_t *codes, float *sc, float *zr) {
  static const int order[8] = {0, 2, 4, 6, 1, 3, 5, 7};
  if (group <= 0 || K % 8 || N % 8 || K % group) return -1;
  int inv[8];
  for (int i = 0; i < 8; i++) inv[order[i]] = i;
  int G = K / group;
  for (int g = 0; g < G; g++)
    for (int n = 0; n < N; n++) {
      sc[(size_t)n * G + g] = scales[(size_t)g * N + n];
      zr[(size_t)n * G + g] = (float)nib(qzeros[(size_t)g * (N / 8) + n / 8], inv[n % 8]);
    }
  for (int n = 0; n < N; n++)
    for (int c = 0; c < K / 8; c++) {
      uint32_t w = 0;
      for (int j = 0; j < 8; j++) {
        int k = 8 * c + j;
        w |= (uint32_t)nib(qweight[(size_t)k * (N / 8) + n / 8], inv[n % 8]) << (4 * j);
      }
      codes[(size_t)n * (K / 8) + c] = w;
    }
  return 0;
}

/* ---------------------------------------------------- block-scaled FP8 e4m3 */

/* kernels/cpu/fp8_dequant.go:33-69 (fp8BlockDequantCPU): out = f32(w) * scale[r/bR,c/bC],
 * rounded once when out is bf16. */
LO_API int lo_fp8_block_dequant(const uint8_t *w, const float *s, void *out, int R, int C, int bR, int bC,
                                int out_bf16) {
  if (bR <= 0 || bC <= 0 || R % bR || C % bC) return -1;
  int gc = C / bC;
  for (int r = 0; r < R; r++)
    for (int c = 0; c < C; c++) {
      float v = lo_e4m3_to_f32(w[(size_t)r * C + c]) * s[(size_t)(r / bR) * gc + c / bC];
      if (out_bf16)
        ((uint16_t *)out)[(size_t)r * C + c] = lo_f32_to_bf16(v);
      else
        ((float *)out)[(size_t)r * C + c] = v;
    }
  return 0;
}

/* --------------------------------------------------------- f32 matmul x . W^T */

typedef struct {
  const float *w;
  int K;
} f32_ctx;
static void f32_row(int n, float *dst, void *p) {
  f32_ctx *c = (f32_ctx *)p;
  memcpy(dst, c->w + (size_t)n * c->K, sizeof(float) * (size_t)c->K);
}
/* The dequantize-then-matmul fallback the reference CPU uses for fp8-block weights
 * (ops/fp8_block.go:222-233 -> kernels/cpu/matmul_f32.go:26-50): same 48-row tiles. */
LO_API int lo_matmul_f32_tb(const float *x, const float *w, float *out, int M, int N, int K, int threads) {
  if (K <= 0) return -1;
  f32_ctx c = {w, K};
  rows_times_x(x, out, M, K, N, threads, f32_row, &c);
  return 0;
}

/* ----------------------------------------------------------------- MoE */

/* ops/moe.go:62-70: pairs sorted by expert id (ascending, stable), giving SortedPairs and
 * SortedExpts; counting sort here. */
LO_API int lo_moe_sort_pairs(const int64_t *ids, int64_t M, int E, int64_t *sorted_pairs, int64_t *sorted_expts) {
  int64_t *off = (int64_t *)calloc((size_t)E + 1, sizeof(int64_t));
  for (int64_t p = 0; p < M; p++) {
    if (ids[p] < 0 || ids[p] >= E) {
      free(off);
      return -1;
    }
    off[ids[p] + 1]++;
  }
  for (int e = 0; e < E; e++) off[e + 1] += off[e];
  for (int64_t p = 0; p < M; p++) {
    int64_t i = off[ids[p]]++;
    sorted_pairs[i] = p;
    sorted_expts[i] = ids[p];
  }
  free(off);
  return 0;
}

typedef struct {
  const float *in, *w, *topkw;
  const int64_t *pairs, *expts;
  float *out;
  int64_t sizeM;
  int N, K, topk, row_per_pair;
} moe_ctx;
static void moe_range(int lo, int hi, void *p) {
  moe_ctx *c = (moe_ctx *)p;
  for (int idx = lo; idx < hi; idx++) {
    int i = idx / c->N, n = idx % c->N;
    int64_t pr = c->pairs[i];
    if (pr < 0 || pr >= c->sizeM) continue;
    int64_t r = c->row_per_pair ? pr : pr / c->topk, e = c->expts[i];
    float acc = dot(c->in + (size_t)r * c->K, c->w + ((size_t)e * c->N + n) * c->K, c->K);
    if (c->topkw) acc *= c->topkw[pr];
    c->out[(size_t)pr * c->N + n] = acc;
  }
}
/* kernels/cpu/moe.go:51-95 (moeGemmKernel, f32 branch): out[p] = w(p) * in[row(p)] . W[e]^T for
 * every sorted pair; rows of `out` for pairs not listed are left untouched. */
LO_API int lo_moe_gemm_f32(const float *in, const float *w, const int64_t *pairs, const int64_t *expts,
                           const float *topkw, float *out, int64_t n_pairs, int64_t sizeM, int N, int K, int topk,
                           int row_per_pair, int threads) {
  if (topk < 1 || K <= 0) return -1;
  moe_ctx c = {in, w, topkw, pairs, expts, out, sizeM, N, K, topk, row_per_pair};
  int grain = 16384 / (K + 1);
  parallel_for((int)(n_pairs * N), grain < 1 ? 1 : grain, threads, moe_range, &c);
  return 0;
}

/* models/deepseek_route.go:30-133 (deepseekRouter), every branch: scores in f64 -- sigmoid(logit) (V3; choice =
 * score + bias) or softmax over the experts (V2) --, then, with n_group > 1 and topk_group < n_group, only the
 * topk_group best groups stay eligible (group score: sum of its two best choices for the sigmoid router, its
 * best for the softmax router; the others' choices become -inf, resp. choice and score become 0), a stable
 * descending top-k of the choices (ties keep the lower expert id), weights = the scores, divided by
 * (their sum + 1e-20) for the sigmoid router when norm_topk. */
static int cmp_desc(const void *a, const void *b) {
  double x = *(const double *)a, y = *(const double *)b;
  return x < y ? 1 : x > y ? -1 : 0;
}
LO_API int lo_deepseek_route(const float *logits, const float *bias, int T, int E, int topk, int n_group, int topk_group,
                             int sigmoid, int norm_topk, int64_t *ids, float *weights) {
  if (n_group < 1) n_group = 1;
  if (topk < 1 || topk > E || E % n_group) return -1;
  const int per = E / n_group;
  double *scores = (double *)malloc(sizeof(double) * (size_t)E * 3);
  double *choice = scores + E, *grp = choice + E;
  int *order = (int *)malloc(sizeof(int) * (size_t)(E + n_group));
  int *gorder = order + E;
  double *gs = (double *)malloc(sizeof(double) * (size_t)n_group);
  char *keep = (char *)malloc((size_t)n_group);
  for (int t = 0; t < T; t++) {
    const float *row = logits + (size_t)t * E;
    if (sigmoid) {
      for (int e = 0; e < E; e++) {
        scores[e] = 1.0 / (1.0 + exp(-(double)row[e]));
        choice[e] = scores[e] + (bias ? (double)bias[e] : 0.0);
      }
    } else {
      double mx = -INFINITY, sum = 0;
      for (int e = 0; e < E; e++) mx = fmax(mx, (double)row[e]);
      for (int e = 0; e < E; e++) {
        scores[e] = exp((double)row[e] - mx);
        sum += scores[e];
      }
      for (int e = 0; e < E; e++) {
        scores[e] /= sum;
        choice[e] = scores[e];
      }
    }
    if (n_group > 1 && topk_group < n_group) {
      for (int g = 0; g < n_group; g++) {
        memcpy(grp, choice + (size_t)g * per, sizeof(double) * (size_t)per);
        qsort(grp, (size_t)per, sizeof(double), cmp_desc);
        gs[g] = sigmoid ? grp[0] + (per > 1 ? grp[1] : 0.0) : grp[0];
        gorder[g] = g;
      }
      /* stable descending order of the groups (insertion sort) */
      for (int i = 1; i < n_group; i++) {
        int g = gorder[i], j = i;
        while (j > 0 && gs[gorder[j - 1]] < gs[g]) gorder[j] = gorder[j - 1], j--;
        gorder[j] = g;
      }
      memset(keep, 0, (size_t)n_group);
      for (int i = 0; i < topk_group; i++) keep[gorder[i]] = 1;
      for (int e = 0; e < E; e++)
        if (!keep[e / per]) {
          if (sigmoid)
            choice[e] = -INFINITY;
          else
            choice[e] = 0, scores[e] = 0;
        }
    }
    for (int e = 0; e < E; e++) order[e] = e;
    /* stable selection of the topk largest choices (ties keep the lower expert id) */
    for (int k = 0; k < topk; k++) {
      int best = k;
      for (int j = k + 1; j < E; j++)
        if (choice[order[j]] > choice[order[best]]) best = j;
      int b = order[best];
      memmove(order + k + 1, order + k, sizeof(int) * (size_t)(best - k));
      order[k] = b;
    }
    double den = 0;
    for (int k = 0; k < topk; k++) den += scores[order[k]];
    for (int k = 0; k < topk; k++) {
      double w = scores[order[k]];
      if (sigmoid && norm_topk) w /= den + 1e-20;
      ids[(size_t)t * topk + k] = order[k];
      weights[(size_t)t * topk + k] = (float)w;
    }
  }
  free(scores);
  free(order);
  free(gs);
  free(keep);
  return 0;
}
LO_API int lo_deepseek_route_sigmoid(const float *logits, const float *bias, int T, int E, int topk, int norm_topk,
                                     int64_t *ids, float *weights) {
  return lo_deepseek_route(logits, bias, T, E, topk, 1, 1, 1, norm_topk, ids, weights);
}

/* ops/moe.go:29-71 (MoERoute) up to the sort: the k largest probabilities per token (ties keep the lower expert id),
 * their values as weights, divided by their f32 sum (added in selection order) when normalize. */
LO_API int lo_moe_route_topk(const float *probs, int T, int E, int topk, int normalize, int64_t *ids, float *weights) {
  if (topk < 1 || topk > E) return -1;
  char *taken = (char *)malloc((size_t)E);
  for (int t = 0; t < T; t++) {
    const float *row = probs + (size_t)t * E;
    memset(taken, 0, (size_t)E);
    float sum = 0;
    for (int k = 0; k < topk; k++) {
      int best = -1;
      for (int e = 0; e < E; e++)
        if (!taken[e] && (best < 0 || row[e] > row[best])) best = e;
      taken[best] = 1;
      ids[(size_t)t * topk + k] = best;
      weights[(size_t)t * topk + k] = row[best];
      sum += row[best];
    }
    if (normalize)
      for (int k = 0; k < topk; k++) weights[(size_t)t * topk + k] /= sum;
  }
  free(taken);
  return 0;
}

/* ------------------------------------------------------------------ decode-step attention */

/* ops/decode_attn.go:13-62 (KVAppend, CPU branch): k, v (B, KH, 1, D) -> row `pos` of the buffers
 * (B, KH, Cap, D).  `elt` is the element size in bytes (the copy is type-blind). */
LO_API int lo_kv_append(const void *k, const void *v, void *kbuf, void *vbuf, int64_t pos, int B, int KH, int D, int Cap,
                        int elt) {
  if (pos < 0 || pos >= Cap) return -1; /* "position %d outside capacity %d" */
  size_t row = (size_t)D * (size_t)elt;
  for (int bh = 0; bh < B * KH; bh++) {
    memcpy((char *)kbuf + ((size_t)bh * Cap + (size_t)pos) * row, (const char *)k + (size_t)bh * row, row);
    memcpy((char *)vbuf + ((size_t)bh * Cap + (size_t)pos) * row, (const char *)v + (size_t)bh * row, row);
  }
  return 0;
}

/* ops/decode_attn.go:64-170 (DecodeAttention, composed branch): per (batch, KV head), the g = NH / KH
 * query rows against keys [start, n), n = pos + 1, start = n - window when a window is set and
 * shorter than n: scores = (q k^T) * scale, softmax over the keys, times v.  f32 throughout, as the
 * reference's CPU MatMul / Affine / Softmax are; inputs and output are f32 arrays (a bf16 case is
 * decoded before and rounded after by the caller). */
LO_API int lo_decode_attn(const float *q, const float *kbuf, const float *vbuf, int64_t pos, float *out, int B, int NH,
                          int KH, int Cap, int D, float scale, int window) {
  int n = (int)pos + 1;
  if (KH <= 0 || NH % KH || n < 1 || n > Cap) return -1; /* "%d valid positions of %d" */
  int g = NH / KH, start = (window > 0 && n > window) ? n - window : 0, cnt = n - start;
  float *sc = (float *)malloc(sizeof(float) * (size_t)cnt);
  for (int b = 0; b < B; b++)
    for (int h = 0; h < NH; h++) {
      int kh = h / g;
      const float *qr = q + ((size_t)b * NH + h) * D;
      const float *K = kbuf + (((size_t)b * KH + kh) * Cap + start) * D;
      const float *V = vbuf + (((size_t)b * KH + kh) * Cap + start) * D;
      float mx = -INFINITY;
      for (int j = 0; j < cnt; j++) {
        float a = 0.f;
        for (int d = 0; d < D; d++) a += qr[d] * K[(size_t)j * D + d];
        sc[j] = a * scale;
        if (sc[j] > mx) mx = sc[j];
      }
      float sum = 0.f;
      for (int j = 0; j < cnt; j++) {
        sc[j] = expf(sc[j] - mx);
        sum += sc[j];
      }
      float *o = out + ((size_t)b * NH + h) * D;
      for (int d = 0; d < D; d++) {
        float a = 0.f;
        for (int j = 0; j < cnt; j++) a += (sc[j] / sum) * V[(size_t)j * D + d];
        o[d] = a;
      }
    }
  free(sc);
  return 0;
}

/* kernels/cpu/norm.go:27-51 (rmsnormF32): one f32 sum of squares per row, in order; the reciprocal root
 * in f64; y = x * inv * w. */
LO_API int lo_rmsnorm_f32(const float *x, const float *w, float *out, int64_t rows, int cols, double eps) {
  for (int64_t r = 0; r < rows; r++) {
    const float *rx = x + (size_t)r * cols;
    float ss = 0.f;
    for (int i = 0; i < cols; i++) ss += rx[i] * rx[i];
    float inv = (float)(1.0 / sqrt((double)(ss / (float)cols) + eps));
    for (int i = 0; i < cols; i++) out[(size_t)r * cols + i] = rx[i] * inv * w[i];
  }
  return 0;
}

/* kernels/cpu/misc_registry.go:27-62 (ropeF32CPU): rotate-half pairing, dim i with dim i + head_dim / 2
 * at angle pos * base^(-2 i / head_dim); angle, cosine and sine in f64, the rotation in f32. */
LO_API int lo_rope_f32(const float *x, const int64_t *positions, float *out, int64_t batch, int seq_len, int head_dim,
                       double base) {
  if (head_dim % 2) return -1;
  int half = head_dim / 2;
  for (int64_t b = 0; b < batch; b++)
    for (int s = 0; s < seq_len; s++) {
      double pos = (double)positions[s];
      size_t rb = ((size_t)b * seq_len + s) * head_dim;
      for (int i = 0; i < half; i++) {
        double theta = pos * pow(base, -(double)(2 * i) / (double)head_dim);
        float c = (float)cos(theta), sn = (float)sin(theta);
        float x0 = x[rb + i], x1 = x[rb + i + half];
        out[rb + i] = x0 * c - x1 * sn;
        out[rb + i + half] = x0 * sn + x1 * c;
      }
    }
  return 0;
}

/* ops/matmul_w8a8.go:65-93 (QuantizeRowsInt8): per row scale = amax / 127, q = clamp(round_to_even(x * (1 / scale))). */
LO_API int lo_quantize_rows_int8(const float *x, int8_t *q, float *scales, int64_t M, int K) {
  for (int64_t m = 0; m < M; m++) {
    const float *row = x + (size_t)m * K;
    float amax = 0.f;
    for (int k = 0; k < K; k++) {
      float a = (float)fabs((double)row[k]);
      if (a > amax) amax = a;
    }
    float scale = amax / 127, inv = 0.f;
    if (scale > 0) inv = 1 / scale;
    scales[m] = scale;
    for (int k = 0; k < K; k++) {
      float r = (float)nearbyint((double)(row[k] * inv)); /* round half to even in the default rounding mode */
      if (r > 127) r = 127;
      else if (r < -127) r = -127;
      q[(size_t)m * K + k] = (int8_t)r;
    }
  }
  return 0;
}

/* ops/matmul_w8a8.go:95-120 (matMulW8A8Reference): int32 accumulation, out = f32(acc) * xs[m] * ws[n]. */
LO_API int lo_matmul_w8a8(const float *x, const int8_t *wq, const float *ws, float *out, int32_t *acc_out, int M, int N, int K) {
  int8_t *xq = (int8_t *)malloc((size_t)M * K);
  float *xs = (float *)malloc(sizeof(float) * (size_t)M);
  lo_quantize_rows_int8(x, xq, xs, M, K);
  for (int m = 0; m < M; m++)
    for (int n = 0; n < N; n++) {
      int32_t acc = 0;
      const int8_t *xr = xq + (size_t)m * K, *wr = wq + (size_t)n * K;
      for (int k = 0; k < K; k++) acc += (int32_t)xr[k] * (int32_t)wr[k];
      if (acc_out) acc_out[(size_t)m * N + n] = acc;
      out[(size_t)m * N + n] = (float)acc * xs[m] * ws[n];
    }
  free(xq);
  free(xs);
  return 0;
}

LO_API int lo_has_avx2(void) { return have_avx2(); }
