// Shape-generic fused dequant-matmul over GGUF blocks: any format, any M, N, K % block == 0.
//
// This is the coverage kernel: odd shapes, the 32-element formats and whatever the decode and
// prefill kernels do not take land here.  One warp owns one weight row and a tile of MT
// activation rows; per iteration the 32 lanes expand 256 consecutive weights (8 each, so the
// warp reads one contiguous run of blocks), multiply them against the MT rows of x and reduce
// with shuffles.  Weights are re-read once per M tile.
#include "gguf_decode.cuh"

namespace lb {

template <int T, int MT>
__global__ void __launch_bounds__(256) gguf_matmul_generic_kernel(const float *__restrict__ x,
                                                                  const uint8_t *__restrict__ w,
                                                                  float *__restrict__ out, int M, int N, int K) {
  constexpr int BE = block_elems(T), BB = block_bytes(T);
  const int lane = threadIdx.x & 31;
  const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (n >= N) return;
  const int m0 = blockIdx.y * MT;
  const uint8_t *row = w + (size_t)n * (size_t)(K / BE) * BB;
  float acc[MT];
#pragma unroll
  for (int m = 0; m < MT; m++) acc[m] = 0.f;
  for (int e = lane * 8; e < K; e += 256) {
    int b = e / BE;
    float v[8];
    decode8<T>(row + (size_t)b * BB, e - b * BE, v);
#pragma unroll
    for (int m = 0; m < MT; m++) {
      if (m0 + m < M) {
        const float4 *xp = reinterpret_cast<const float4 *>(x + (size_t)(m0 + m) * K + e);
        float4 a = __ldg(xp), c = __ldg(xp + 1);
        acc[m] += v[0] * a.x + v[1] * a.y + v[2] * a.z + v[3] * a.w + v[4] * c.x + v[5] * c.y + v[6] * c.z + v[7] * c.w;
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MT; m++) {
    float s = warp_sum(acc[m]);
    if (lane == 0 && m0 + m < M) out[(size_t)(m0 + m) * N + n] = s;
  }
}

template <int T>
static int run(const float *x, const void *w, float *out, int M, int N, int K, cudaStream_t st) {
  constexpr int MT = 4, WARPS = 8;
  dim3 grid((N + WARPS - 1) / WARPS, (M + MT - 1) / MT);
  if (grid.y > 65535) return fail(LB200_E_TOO_LARGE, "matmul_q: M=%d exceeds the generic kernel's grid", M);
  gguf_matmul_generic_kernel<T, MT><<<grid, WARPS * 32, 0, st>>>(x, (const uint8_t *)w, out, M, N, K);
  return launched("matmul_q (generic)");
}

int gguf_matmul_generic(int type, const float *x, const void *w, float *out, int M, int N, int K, cudaStream_t st) {
  switch (type) {
    case LB200_Q4_0: return run<LB200_Q4_0>(x, w, out, M, N, K, st);
    case LB200_Q5_0: return run<LB200_Q5_0>(x, w, out, M, N, K, st);
    case LB200_Q8_0: return run<LB200_Q8_0>(x, w, out, M, N, K, st);
    case LB200_Q4_K: return run<LB200_Q4_K>(x, w, out, M, N, K, st);
    case LB200_Q5_K: return run<LB200_Q5_K>(x, w, out, M, N, K, st);
    case LB200_Q6_K: return run<LB200_Q6_K>(x, w, out, M, N, K, st);
  }
  return fail(LB200_E_DTYPE, "matmul_q: ggml type %d has no kernel", type);
}

}  // namespace lb
