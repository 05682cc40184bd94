// Exact per-format decoders: eight consecutive elements of one block -> f32.
//
// Every product and difference is a separately rounded f32 operation (__fmul_rn / __fsub_rn are
// never contracted into FMA), which is what the reference's CPU decoders compute
// (kernels/cpu/quant_matmul.go:28-97), so the results are bit-identical to them.
#pragma once
#include "common.cuh"

namespace lb {

__device__ __forceinline__ float f16_at(const uint8_t *p) { return f16_bits_to_f32((uint16_t)(p[0] | (p[1] << 8))); }

// 6-bit (scale, min) pair j of a Q4_K / Q5_K block (reference quant/q4_k.go:82-89).
__device__ __forceinline__ void k4_scale_min(int j, const uint8_t *q, int &sc, int &m) {
  if (j < 4) {
    sc = q[j] & 63;
    m = q[j + 4] & 63;
  } else {
    sc = (q[j + 4] & 0x0F) | ((q[j - 4] >> 6) << 4);
    m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
  }
}

// e0 is a multiple of 8 inside the block.
template <int T>
__device__ __forceinline__ void decode8(const uint8_t *blk, int e0, float out[8]);

template <>
__device__ __forceinline__ void decode8<LB200_Q8_0>(const uint8_t *b, int e0, float out[8]) {
  float d = f16_at(b);
#pragma unroll
  for (int i = 0; i < 8; i++) out[i] = __fmul_rn(d, (float)(int8_t)b[2 + e0 + i]);
}

template <>
__device__ __forceinline__ void decode8<LB200_Q4_0>(const uint8_t *b, int e0, float out[8]) {
  float d = f16_at(b);
  int hi = e0 >= 16, j0 = e0 & 15;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    int q = b[2 + j0 + i];
    out[i] = __fmul_rn(d, (float)((hi ? (q >> 4) : (q & 15)) - 8));
  }
}

template <>
__device__ __forceinline__ void decode8<LB200_Q5_0>(const uint8_t *b, int e0, float out[8]) {
  float d = f16_at(b);
  uint32_t qh = (uint32_t)b[2] | (uint32_t)b[3] << 8 | (uint32_t)b[4] << 16 | (uint32_t)b[5] << 24;
  int hi = e0 >= 16, j0 = e0 & 15;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    int q = b[6 + j0 + i];
    int v = (hi ? (q >> 4) : (q & 15)) | (int)((qh >> (e0 + i)) & 1u) << 4;
    out[i] = __fmul_rn(d, (float)(v - 16));
  }
}

template <>
__device__ __forceinline__ void decode8<LB200_Q4_K>(const uint8_t *b, int e0, float out[8]) {
  float d = f16_at(b), dmin = f16_at(b + 2);
  int p = e0 >> 6, r = e0 & 63, hi = r >> 5, l0 = r & 31, sc, m;
  k4_scale_min(2 * p + hi, b + 4, sc, m);
  float dl = __fmul_rn(d, (float)sc), ml = __fmul_rn(dmin, (float)m);
  const uint8_t *qs = b + 16 + p * 32 + l0;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    int q = hi ? (qs[i] >> 4) : (qs[i] & 15);
    out[i] = __fsub_rn(__fmul_rn(dl, (float)q), ml);
  }
}

template <>
__device__ __forceinline__ void decode8<LB200_Q5_K>(const uint8_t *b, int e0, float out[8]) {
  float d = f16_at(b), dmin = f16_at(b + 2);
  int p = e0 >> 6, r = e0 & 63, hi = r >> 5, l0 = r & 31, sc, m;
  k4_scale_min(2 * p + hi, b + 4, sc, m);
  float dl = __fmul_rn(d, (float)sc), ml = __fmul_rn(dmin, (float)m);
  const uint8_t *qh = b + 16 + l0, *qs = b + 48 + p * 32 + l0;
  int bit = 2 * p + hi;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    int q = (hi ? (qs[i] >> 4) : (qs[i] & 15)) | (((qh[i] >> bit) & 1) << 4);
    out[i] = __fsub_rn(__fmul_rn(dl, (float)q), ml);
  }
}

template <>
__device__ __forceinline__ void decode8<LB200_Q6_K>(const uint8_t *b, int e0, float out[8]) {
  float d = f16_at(b + 208);
  int half = e0 >> 7, r = e0 & 127, grp = r >> 5, l0 = r & 31;
  const uint8_t *ql = b + half * 64 + (grp & 1) * 32 + l0, *qh = b + 128 + half * 32 + l0;
  float ds = __fmul_rn(d, (float)(int8_t)b[192 + half * 8 + 2 * grp + (l0 >> 4)]);
#pragma unroll
  for (int i = 0; i < 8; i++) {
    int q = ((grp >> 1) ? (ql[i] >> 4) : (ql[i] & 15)) | (((qh[i] >> (2 * grp)) & 3) << 4);
    out[i] = __fmul_rn(ds, (float)(q - 32));
  }
}

}  // namespace lb
