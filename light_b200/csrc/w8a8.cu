// INT8 weights x INT8 activations: the counterpart of the reference's ops.MatMulW8A8 (ops/matmul_w8a8.go:13-120;
// its CUDA path quantises the activation rows on the device and calls cublasGemmEx with CUBLAS_COMPUTE_32I).
//   x f32 (M, K) -> per row: scale = amax / 127, q = clamp(round_to_even(x * (1 / scale)), -127, 127)
//   acc i32 (M, N) = q . wq^T                      (exact)
//   out f32 (M, N) = f32(acc) * xs[m] * ws[n]      (two f32 multiplies, in this order)
// Every step is deterministic, so the result equals the reference's Go path (matMulW8A8Reference) bit for bit.
//
// The contraction runs on the integer tensor-core path (mma.sync m16n8k32 s8 x s8 -> s32): both operands are
// K-contiguous, which is exactly the row x col fragment layout, so fragments are plain 32-bit shared-memory
// loads; tiles arrive through a three-stage cp.async ring with an 80-byte row pitch (conflict-free).
#include "common.cuh"
#include "mma_sync.cuh"

namespace lb {
namespace {

// ---- activation rows -> int8 (ops/matmul_w8a8.go:65-93, QuantizeRowsInt8)
__global__ void __launch_bounds__(256) quantize_rows_int8_kernel(const float *__restrict__ x, int8_t *__restrict__ q,
                                                                 float *__restrict__ scales, int K) {
  __shared__ float part[8];
  pdl_launch_dependents();
  pdl_wait();
  const float *row = x + (size_t)blockIdx.x * K;
  float amax = 0.f;
  for (int k = threadIdx.x; k < K; k += 256) amax = fmaxf(amax, fabsf(row[k]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = part[0];
#pragma unroll
  for (int i = 1; i < 8; i++) amax = fmaxf(amax, part[i]);
  const float scale = __fdiv_rn(amax, 127.f);
  const float inv = scale > 0.f ? __fdiv_rn(1.f, scale) : 0.f;
  if (threadIdx.x == 0) scales[blockIdx.x] = scale;
  int8_t *qr = q + (size_t)blockIdx.x * K;
  for (int k = threadIdx.x; k < K; k += 256) {
    float r = rintf(__fmul_rn(row[k], inv));  // round half to even
    r = r > 127.f ? 127.f : (r < -127.f ? -127.f : r);
    qr[k] = (int8_t)r;
  }
}

__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int W8_BM = 128, W8_BN = 128, W8_BK = 64, W8_PITCH = 80, W8_STAGES = 3;
constexpr int W8_TILE = W8_BM * W8_PITCH;                 // bytes of one operand tile of one stage
constexpr int W8_SMEM = W8_STAGES * 2 * W8_TILE;          // 61440

// out (M, N) tile of 128 x 128 per CTA; 8 warps as 2 (rows) x 4 (columns), a warp owns 64 x 32.
__global__ void __launch_bounds__(256) w8a8_gemm_kernel(const int8_t *__restrict__ xq, const int8_t *__restrict__ wq,
                                                       const float *__restrict__ xs, const float *__restrict__ ws,
                                                       float *__restrict__ out, int M, int N, int K) {
  extern __shared__ __align__(16) unsigned char dyn[];
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int wm = warp >> 2, wn = warp & 3;
  const int m0 = blockIdx.y * W8_BM, n0 = blockIdx.x * W8_BN;
  const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(dyn);
  const int ksteps = (K + W8_BK - 1) / W8_BK;  // K % 16 == 0 (launcher): granules past K are filled with zeros
  // copies: 128 rows x 4 granules of 16 bytes per operand and stage = 512 granules, two per thread
  auto issue = [&](int ks) {
    if (ks < ksteps) {
      const uint32_t st = sbase + (uint32_t)(ks % W8_STAGES) * 2 * W8_TILE;
#pragma unroll
      for (int i = 0; i < 2; i++) {
        const int c = threadIdx.x + 256 * i, r = c >> 2, p = c & 3;
        const int ra = min(m0 + r, M - 1), rb = min(n0 + r, N - 1);  // rows past the edge repeat the last row; never stored
        const int ko = ks * W8_BK + p * 16;
        if (ko < K) {
          cp_async16(st + r * W8_PITCH + p * 16, xq + (size_t)ra * K + ko);
          cp_async16(st + W8_TILE + r * W8_PITCH + p * 16, wq + (size_t)rb * K + ko);
        } else {
          cp_async16_part(st + r * W8_PITCH + p * 16, xq + (size_t)ra * K, 0);
          cp_async16_part(st + W8_TILE + r * W8_PITCH + p * 16, wq + (size_t)rb * K, 0);
        }
      }
    }
    cp_async_commit();
  };
  pdl_wait();
#pragma unroll 1
  for (int p = 0; p < W8_STAGES - 1; p++) issue(p);
  int acc[4][4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0;
  for (int ks = 0; ks < ksteps; ks++) {
    cp_async_wait<W8_STAGES - 2>();
    __syncthreads();  // stage ks has landed for everyone, and everyone is done with stage ks - 1
    issue(ks + W8_STAGES - 1);
    const uint32_t sa = sbase + (uint32_t)(ks % W8_STAGES) * 2 * W8_TILE + (wm * 64 + g) * W8_PITCH + 4 * t;
    const uint32_t sb = sbase + (uint32_t)(ks % W8_STAGES) * 2 * W8_TILE + W8_TILE + (wn * 32 + g) * W8_PITCH + 4 * t;
#pragma unroll
    for (int kk = 0; kk < 2; kk++) {  // two k32 steps per stage
      uint32_t b[4][2];
#pragma unroll
      for (int j = 0; j < 4; j++) b[j][0] = lds32(sb + j * 8 * W8_PITCH + kk * 32), b[j][1] = lds32(sb + j * 8 * W8_PITCH + kk * 32 + 16);
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const uint32_t a = sa + i * 16 * W8_PITCH + kk * 32;
        const uint32_t a0 = lds32(a), a1 = lds32(a + 8 * W8_PITCH), a2 = lds32(a + 16), a3 = lds32(a + 8 * W8_PITCH + 16);
#pragma unroll
        for (int j = 0; j < 4; j++) mma_s8(acc[i][j], a0, a1, a2, a3, b[j][0], b[j][1]);
      }
    }
  }
  cp_async_wait<0>();
  // acc[i][j]: rows m0 + wm 64 + i 16 + g (+8), columns n0 + wn 32 + j 8 + 2t (+1)
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const int m = m0 + wm * 64 + i * 16 + g + 8 * h;
      if (m >= M) continue;
      const float sx = xs[m];
#pragma unroll
      for (int j = 0; j < 4; j++)
#pragma unroll
        for (int c = 0; c < 2; c++) {
          const int n = n0 + wn * 32 + j * 8 + 2 * t + c;
          if (n < N) out[(size_t)m * N + n] = __fmul_rn(__fmul_rn((float)acc[i][j][2 * h + c], sx), ws[n]);
        }
    }
}

template <typename Kern, typename... Args>
cudaError_t launch_chain(Kern kern, dim3 grid, unsigned block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid, cfg.blockDim = dim3(block), cfg.dynamicSmemBytes = smem, cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

}  // namespace

int quantize_rows_int8(const float *x, int8_t *q, float *scales, long long M, int K, cudaStream_t st) {
  if (M == 0) return 0;
  cudaError_t e = launch_chain(quantize_rows_int8_kernel, dim3((unsigned)M), 256, 0, st, x, q, scales, K);
  if (e != cudaSuccess) return fail((int)e, "light_b200: quantize_rows_int8: %s", cudaGetErrorString(e));
  return launched("quantize_rows_int8");
}

int matmul_w8a8(const float *x, const int8_t *wq, const float *ws, float *out, int8_t *xq, float *xs, int M, int N, int K,
                cudaStream_t st) {
  if (M == 0 || N == 0) return 0;
  static DeviceOnce attr_done;
  {
    cudaError_t e = attr_done.ensure([&] { return cudaFuncSetAttribute(w8a8_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, W8_SMEM); });
    if (e != cudaSuccess) return fail((int)e, "light_b200: matmul_w8a8: %s", cudaGetErrorString(e));
  }
  if (int rc = quantize_rows_int8(x, xq, xs, M, K, st)) return rc;
  dim3 grid((N + W8_BN - 1) / W8_BN, (M + W8_BM - 1) / W8_BM);
  if (grid.y > 65535) return fail(LB200_E_TOO_LARGE, "light_b200: matmul_w8a8: M=%d exceeds the kernel's grid", M);
  cudaError_t e = launch_chain(w8a8_gemm_kernel, grid, 256, W8_SMEM, st, (const int8_t *)xq, wq, (const float *)xs, ws, out, M, N, K);
  if (e != cudaSuccess) return fail((int)e, "light_b200: matmul_w8a8: %s", cudaGetErrorString(e));
  return launched("matmul_w8a8");
}

}  // namespace lb
