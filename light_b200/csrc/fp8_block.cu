// Block-scaled FP8 weights: e4m3fn codes w (N, K) and one f32 scale per (bR x bC) block,
// W[n, k] = f32(w[n, k]) * scale[n / bR, k / bC]  (reference ops/fp8_block.go:13-60).
//
// e4m3 -> f32 goes through the hardware e4m3x2 -> f16x2 conversion, which is exact (every e4m3
// value is an f16 value), then f16 -> f32, also exact; the product is one rounded f32 multiply.
#include <cuda_fp8.h>

#include "common.cuh"

namespace lb {

__device__ __forceinline__ void e4m3x4_to_f32(uint32_t v, float out[4]) {
  __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(v & 0xFFFFu), __NV_E4M3);
  __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(v >> 16), __NV_E4M3);
  float2 a = __half22float2(__half2(lo)), b = __half22float2(__half2(hi));
  out[0] = a.x, out[1] = a.y, out[2] = b.x, out[3] = b.y;
}

// ---- dequantize: one thread per four codes (C % 4 == 0 and bC % 4 == 0 keep them in one block).
template <typename T>
__global__ void __launch_bounds__(256) fp8_block_dequant_kernel(const uint32_t *__restrict__ w,
                                                                const float *__restrict__ s, T *__restrict__ out, int R,
                                                                int C, int bR, int bC) {
  const long long n4 = (long long)R * C / 4;
  const int gc = C / bC;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    long long e = i * 4;
    int r = (int)(e / C), c = (int)(e - (long long)r * C);
    float sc = __ldg(s + (size_t)(r / bR) * gc + c / bC);
    float v[4];
    e4m3x4_to_f32(__ldg(w + i), v);
#pragma unroll
    for (int j = 0; j < 4; j++) v[j] = __fmul_rn(v[j], sc);
    if constexpr (sizeof(T) == 4) {
      *reinterpret_cast<float4 *>(out + e) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
      __nv_bfloat162 p[2] = {__floats2bfloat162_rn(v[0], v[1]), __floats2bfloat162_rn(v[2], v[3])};
      *reinterpret_cast<uint2 *>(out + e) = *reinterpret_cast<uint2 *>(p);
    }
  }
}

int fp8_block_dequant(const uint8_t *w, const float *s, void *out, int out_dtype, int R, int C, int bR, int bC,
                      cudaStream_t st) {
  long long n4 = (long long)R * C / 4;
  if (n4 == 0) return 0;
  long long blocks = (n4 + 255) / 256;
  if (blocks > 148LL * 64) blocks = 148LL * 64;
  if (out_dtype == LB200_F32)
    fp8_block_dequant_kernel<float><<<(unsigned)blocks, 256, 0, st>>>((const uint32_t *)w, s, (float *)out, R, C, bR, bC);
  else
    fp8_block_dequant_kernel<__nv_bfloat16>
        <<<(unsigned)blocks, 256, 0, st>>>((const uint32_t *)w, s, (__nv_bfloat16 *)out, R, C, bR, bC);
  return launched("fp8_block_dequant");
}

// ---- decode GEMV: one warp per weight row and MT activation rows; a lane takes 16 codes (one
// 16-byte load) per step, all under one scale because bC % 16 == 0.  The scale multiplies the
// 16-term partial sum, not each weight.
template <typename T, int MT>
__global__ void __launch_bounds__(256) fp8_block_gemv_kernel(const T *__restrict__ x, const uint4 *__restrict__ w,
                                                             const float *__restrict__ s, T *__restrict__ y, int M,
                                                             int N, int K, int bR, int bC) {
  const int lane = threadIdx.x & 31;
  const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (n >= N) return;
  const int m0 = blockIdx.y * MT;
  const int chunks = K / 16, gc = K / bC;
  const uint4 *wr = w + (size_t)n * chunks;
  const float *sr = s + (size_t)(n / bR) * gc;
  float acc[MT];
#pragma unroll
  for (int m = 0; m < MT; m++) acc[m] = 0.f;
  for (int c = lane; c < chunks; c += 32) {
    uint4 q = __ldg(wr + c);
    const int k0 = c * 16;
    const float sc = __ldg(sr + k0 / bC);
    float wv[16];
    e4m3x4_to_f32(q.x, wv);
    e4m3x4_to_f32(q.y, wv + 4);
    e4m3x4_to_f32(q.z, wv + 8);
    e4m3x4_to_f32(q.w, wv + 12);
#pragma unroll
    for (int m = 0; m < MT; m++) {
      if (m0 + m < M) {
        const T *xr = x + (size_t)(m0 + m) * K + k0;
        float a = 0.f;
#pragma unroll
        for (int j = 0; j < 16; j++) a = fmaf(wv[j], ld_act(xr, j), a);
        acc[m] = fmaf(a, sc, acc[m]);
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MT; m++) {
    float v = warp_sum(acc[m]);
    if (lane == 0 && m0 + m < M) st_act(y, (long long)(m0 + m) * N + n, v);
  }
}

int fp8_block_gemv(const void *x, const uint8_t *w, const float *s, void *y, int act_dtype, int M, int N, int K, int bR,
                   int bC, cudaStream_t st) {
  if (M == 0 || N == 0) return 0;
  constexpr int MT = 4, WARPS = 8;
  dim3 grid((N + WARPS - 1) / WARPS, (M + MT - 1) / MT);
  if (grid.y > 65535) return fail(LB200_E_TOO_LARGE, "fp8_block_gemv: M=%d exceeds the kernel's grid", M);
  if (act_dtype == LB200_F32)
    fp8_block_gemv_kernel<float, MT>
        <<<grid, WARPS * 32, 0, st>>>((const float *)x, (const uint4 *)w, s, (float *)y, M, N, K, bR, bC);
  else
    fp8_block_gemv_kernel<__nv_bfloat16, MT><<<grid, WARPS * 32, 0, st>>>((const __nv_bfloat16 *)x, (const uint4 *)w, s,
                                                                           (__nv_bfloat16 *)y, M, N, K, bR, bC);
  return launched("fp8_block_gemv");
}

}  // namespace lb
