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

}  // namespace lb
