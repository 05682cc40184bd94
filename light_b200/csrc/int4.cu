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

// ---- checkpoint layouts -> the canonical layout, on the device (the reference converts on the host with
// O(N K) Go loops at load time, quant/int4.go:103-261).  kind 0: AutoGPTQ "gptq" (qzeros hold zero - 1),
// 1: "gptq_v2", 2: AutoAWQ GEMM.  Ordered groups only (g_idx[k] = k / G); an act-order checkpoint keeps the
// host path, which also builds the column permutation.
__device__ __forceinline__ uint32_t nib_at(uint32_t w, int j) { return (w >> (4 * j)) & 0xFu; }
__device__ __forceinline__ int awq_slot(int col) { return (col >> 1) + 4 * (col & 1); }  // inverse of (0,2,4,6,1,3,5,7)

// codes: one thread per canonical word (n, c).  GPTQ: the word is qweight[c][n] itself (a transpose).  AWQ:
// nibble j is column n of row 8c + j.  A 32 x 32 tile goes through shared memory so that reads and writes
// are both coalesced.
__global__ void __launch_bounds__(256) int4_repack_codes_kernel(const uint32_t *__restrict__ qweight, uint32_t *__restrict__ codes,
                                                                int N, int K, int kind) {
  __shared__ uint32_t tile[32][33];
  const int KW = K / 8;
  const int c0 = blockIdx.x * 32, n0 = blockIdx.y * 32, tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int r = ty; r < 32; r += 8) {  // tile[c - c0][n - n0], read along n
    const int c = c0 + r, n = n0 + tx;
    uint32_t w = 0;
    if (c < KW && n < N) {
      if (kind == 2) {
        const int slot = awq_slot(n & 7);
#pragma unroll
        for (int j = 0; j < 8; j++) w |= nib_at(qweight[(size_t)(8 * c + j) * (N / 8) + (n >> 3)], slot) << (4 * j);
      } else {
        w = qweight[(size_t)c * N + n];
      }
    }
    tile[r][tx] = w;
  }
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {  // written along c
    const int n = n0 + r, c = c0 + tx;
    if (n < N && c < KW) codes[(size_t)n * KW + c] = tile[tx][r];
  }
}

// scales / zeros: (K/G, N) and packed (K/G, N/8) -> f32 (N, K/G)
__global__ void int4_repack_sz_kernel(const uint32_t *__restrict__ qzeros, const float *__restrict__ scales, float *__restrict__ s_out,
                                      float *__restrict__ z_out, int N, int G, int kind) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)N * G) return;
  const int g = (int)(i / N), n = (int)(i - (long long)g * N);  // read along n
  const uint32_t w = qzeros[(size_t)g * (N / 8) + (n >> 3)];
  const float z = (float)nib_at(w, kind == 2 ? awq_slot(n & 7) : (n & 7));
  s_out[(size_t)n * G + g] = scales[(size_t)g * N + n];
  z_out[(size_t)n * G + g] = kind == 0 ? z + 1.f : z;
}

int int4_repack(const uint32_t *qweight, const uint32_t *qzeros, const float *scales, uint32_t *codes, float *s_out, float *z_out,
                int N, int K, int G, int kind, cudaStream_t st) {
  if (kind < 0 || kind > 2) return fail(LB200_E_DTYPE, "light_b200: int4_repack: layout %d (0 gptq, 1 gptq_v2, 2 awq)", kind);
  if (N <= 0 || K <= 0 || G <= 0 || N % 8 || K % 8 || K % G) return fail(LB200_E_SHAPE, "light_b200: int4_repack: N %d K %d group %d", N, K, G);
  dim3 grid((K / 8 + 31) / 32, (N + 31) / 32);
  if (grid.y > 65535) return fail(LB200_E_TOO_LARGE, "light_b200: int4_repack: N=%d exceeds the kernel's grid", N);
  int4_repack_codes_kernel<<<grid, 256, 0, st>>>(qweight, codes, N, K, kind);
  const long long n = (long long)N * (K / G);
  int4_repack_sz_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(qzeros, scales, s_out, z_out, N, K / G, kind);
  return launched("int4_repack");
}


// out[m, k] = x[m, idx[k]]: the activation-column gather in front of an act-order GPTQ weight (reference
// ops/int4.go:129-147 gatherColumns: transpose, IndexSelect, transpose).  Element size 2 or 4 bytes.
template <typename T>
__global__ void __launch_bounds__(256) gather_columns_kernel(const T *__restrict__ x, const long long *__restrict__ idx, T *__restrict__ out, long long M,
                                                             int K) {
  const long long total = M * K;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long m = i / K;
    const int k = (int)(i - m * K);
    const long long src = idx[k];
    out[i] = (src >= 0 && src < K) ? x[m * K + src] : T(0);
  }
}

int gather_columns(const void *x, const int64_t *idx, void *out, int elt, long long M, int K, cudaStream_t st) {
  if (M == 0 || K == 0) return 0;
  long long blocks = (M * K + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (elt == 4)
    gather_columns_kernel<uint32_t><<<(unsigned)blocks, 256, 0, st>>>((const uint32_t *)x, (const long long *)idx, (uint32_t *)out, M, K);
  else if (elt == 2)
    gather_columns_kernel<uint16_t><<<(unsigned)blocks, 256, 0, st>>>((const uint16_t *)x, (const long long *)idx, (uint16_t *)out, M, K);
  else
    return fail(LB200_E_DTYPE, "light_b200: gather_columns: element size %d", elt);
  return launched("gather_columns");
}

}  // namespace lb
