// Group-quantized 4-bit weights (GPTQ / AWQ) in the canonical layout of the reference
// (quant/int4.go:12-31): codes u32 (N, K/8), nibble j of codes[n, c] = code of W[n, 8c+j];
// scales, zeros f32 (N, K/G);  W[n, k] = s[n, k/G] * (code - z[n, k/G]).
#include "common.cuh"

namespace lb {

// ---- dequantize: one thread per code word (eight weights of one group), product formed in
// f32 with separately rounded subtract and multiply, rounded once to the output type.
template <typename T>
__global__ void __launch_bounds__(256) int4_dequant_kernel(const uint32_t *__restrict__ codes,
                                                           const float *__restrict__ s, const float *__restrict__ z,
                                                           T *__restrict__ out, int N, int K, int G) {
  const int kw = K / 8, ng = K / G;
  const long long words = (long long)N * kw;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < words;
       i += (long long)gridDim.x * blockDim.x) {
    int n = (int)(i / kw), c = (int)(i - (long long)n * kw);
    int g = n * ng + (8 * c) / G;
    float sc = __ldg(s + g), zr = __ldg(z + g);
    uint32_t w = __ldg(codes + i);
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; j++) v[j] = __fmul_rn(sc, __fsub_rn((float)((w >> (4 * j)) & 0xFu), zr));
    long long base = (long long)n * K + 8LL * c;
    if constexpr (sizeof(T) == 4) {
      float4 *o = reinterpret_cast<float4 *>(out + base);
      o[0] = make_float4(v[0], v[1], v[2], v[3]);
      o[1] = make_float4(v[4], v[5], v[6], v[7]);
    } else {
      __nv_bfloat162 p[4];
#pragma unroll
      for (int j = 0; j < 4; j++) p[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
      *reinterpret_cast<uint4 *>(out + base) = *reinterpret_cast<uint4 *>(p);
    }
  }
}

int int4_dequant(const uint32_t *codes, const float *s, const float *z, void *out, int out_dtype, int N, int K, int G,
                 long long offset, cudaStream_t st) {
  long long words = (long long)N * (K / 8);
  if (words == 0) return 0;
  long long blocks = (words + 255) / 256;
  if (blocks > 148LL * 64) blocks = 148LL * 64;
  if (out_dtype == LB200_F32)
    int4_dequant_kernel<float><<<(unsigned)blocks, 256, 0, st>>>(codes, s, z, (float *)out + offset, N, K, G);
  else
    int4_dequant_kernel<__nv_bfloat16>
        <<<(unsigned)blocks, 256, 0, st>>>(codes, s, z, (__nv_bfloat16 *)out + offset, N, K, G);
  return launched("int4_dequant");
}

// ---- decode GEMV: one warp per weight row and MT activation rows.  A lane takes 32 codes
// (one 16-byte load) per step; the group affine is folded, sum s*(q-z)*x = s*(sum q*x - z*sum x),
// so the inner loop is one FMA per weight plus the running sum of x.
template <typename T, int MT>
__global__ void __launch_bounds__(256) int4_gemv_kernel(const T *__restrict__ x, const uint4 *__restrict__ codes,
                                                        const float *__restrict__ s, const float *__restrict__ z,
                                                        T *__restrict__ y, int M, int N, int K, int G) {
  const int lane = threadIdx.x & 31;
  const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (n >= N) return;
  const int m0 = blockIdx.y * MT;
  const int steps = K / 32, ng = K / G;
  const uint4 *row = codes + (size_t)n * steps;
  const float *sr = s + (size_t)n * ng, *zr = z + (size_t)n * ng;
  float acc[MT];
#pragma unroll
  for (int m = 0; m < MT; m++) acc[m] = 0.f;
  for (int c = lane; c < steps; c += 32) {
    uint4 q = __ldg(row + c);
    const int k0 = c * 32;
    const float sc = __ldg(sr + k0 / G), zp = __ldg(zr + k0 / G);
    const uint32_t wd[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int m = 0; m < MT; m++) {
      if (m0 + m < M) {
        const T *xr = x + (size_t)(m0 + m) * K + k0;
        float dot = 0.f, sum = 0.f;
#pragma unroll
        for (int i = 0; i < 4; i++) {
#pragma unroll
          for (int j = 0; j < 8; j++) {
            float xv = ld_act(xr, 8 * i + j);
            dot = fmaf((float)((wd[i] >> (4 * j)) & 0xFu), xv, dot);
            sum += xv;
          }
        }
        acc[m] = fmaf(sc, dot - zp * sum, acc[m]);
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MT; m++) {
    float v = warp_sum(acc[m]);
    if (lane == 0 && m0 + m < M) st_act(y, (long long)(m0 + m) * N + n, v);
  }
}

int int4_gemv(const void *x, const uint32_t *codes, const float *s, const float *z, void *y, int act_dtype, int M, int N,
              int K, int G, cudaStream_t st) {
  if (M == 0 || N == 0) return 0;
  constexpr int MT = 4, WARPS = 8;
  dim3 grid((N + WARPS - 1) / WARPS, (M + MT - 1) / MT);
  if (grid.y > 65535) return fail(LB200_E_TOO_LARGE, "int4_gemv: M=%d exceeds the kernel's grid", M);
  if (act_dtype == LB200_F32)
    int4_gemv_kernel<float, MT>
        <<<grid, WARPS * 32, 0, st>>>((const float *)x, (const uint4 *)codes, s, z, (float *)y, M, N, K, G);
  else
    int4_gemv_kernel<__nv_bfloat16, MT><<<grid, WARPS * 32, 0, st>>>((const __nv_bfloat16 *)x, (const uint4 *)codes, s,
                                                                      z, (__nv_bfloat16 *)y, M, N, K, G);
  return launched("int4_gemv");
}

}  // namespace lb
