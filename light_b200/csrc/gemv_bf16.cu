// Decode GEMVs over UNQUANTIZED bf16 weights: registry keys {gemv_multi, CUDA, BF16} and {gemv_gated, CUDA, BF16}
// (reference kernels/cuda/gemv.go:15-94, ops.LinearMulti / ops.GatedLinear, ops/gemv.go:21-140): one bf16
// activation row against up to four (N_i, K) bf16 matrices in one launch, and the gated pair
// act(x . Wg^T) * (x . Wu^T) with the bf16 roundings of the unfused sequence.
//
// HBM-bound: every weight byte is read once with 16-byte loads that bypass L1, four loads per lane in flight per
// row pair.  The grid is persistent (a multiple of the SM count); the rows of all matrices form one list that the
// warps of the grid walk in a strided loop, TWO rows per step so that a lane has eight independent loads in
// flight; x is converted to f32 once per CTA into shared memory.  Sums are f32 (lane partial sums in a fixed
// order, then a butterfly), rounded once on store, as the reference's kernel and its cuBLAS fallback do.
#include "common.cuh"

namespace lb {

namespace {

constexpr int GB_WARPS = 8;
constexpr int GB_MAXK = 16384;  // f32 activations in shared memory: 64 KB

struct GbSegs {
  const __nv_bfloat16 *w[4];
  void *y[4];
  int n[4];
  int end[4];  // running total of rows
  int count;
};

__device__ __forceinline__ uint4 ld_stream16(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
// eight bf16 weights against eight f32 activations (bf16 -> f32 is the bits in the high half of the word)
__device__ __forceinline__ float dot8(const uint4 u, const float *xs8, float acc) {
  const float4 x0 = *reinterpret_cast<const float4 *>(xs8), x1 = *reinterpret_cast<const float4 *>(xs8 + 4);
  acc = fmaf(__uint_as_float(u.x << 16), x0.x, acc);
  acc = fmaf(__uint_as_float(u.x & 0xffff0000u), x0.y, acc);
  acc = fmaf(__uint_as_float(u.y << 16), x0.z, acc);
  acc = fmaf(__uint_as_float(u.y & 0xffff0000u), x0.w, acc);
  acc = fmaf(__uint_as_float(u.z << 16), x1.x, acc);
  acc = fmaf(__uint_as_float(u.z & 0xffff0000u), x1.y, acc);
  acc = fmaf(__uint_as_float(u.w << 16), x1.z, acc);
  acc = fmaf(__uint_as_float(u.w & 0xffff0000u), x1.w, acc);
  return acc;
}
__device__ __forceinline__ void stage_x(const __nv_bfloat16 *x, float *xs, int K) {
  asm volatile("griddepcontrol.wait;\n" ::: "memory");  // x is the previous launch's output
  for (int i = threadIdx.x * 8; i < K; i += blockDim.x * 8) {
    const uint4 u = *reinterpret_cast<const uint4 *>(x + i);
    xs[i] = __uint_as_float(u.x << 16), xs[i + 1] = __uint_as_float(u.x & 0xffff0000u);
    xs[i + 2] = __uint_as_float(u.y << 16), xs[i + 3] = __uint_as_float(u.y & 0xffff0000u);
    xs[i + 4] = __uint_as_float(u.z << 16), xs[i + 5] = __uint_as_float(u.z & 0xffff0000u);
    xs[i + 6] = __uint_as_float(u.w << 16), xs[i + 7] = __uint_as_float(u.w & 0xffff0000u);
  }
  __syncthreads();
}
// two rows at once: a[0] . x and a[1] . x, summed over the warp
__device__ __forceinline__ void rows2(const __nv_bfloat16 *r0, const __nv_bfloat16 *r1, const float *xs, int K, int lane, float &s0, float &s1) {
  float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
  int c = lane * 8;
  for (; c + 256 < K; c += 512) {  // four loads of each row pair per trip
    const uint4 u0 = ld_stream16(r0 + c), v0 = ld_stream16(r1 + c), u1 = ld_stream16(r0 + c + 256), v1 = ld_stream16(r1 + c + 256);
    a0 = dot8(u0, xs + c, a0), b0 = dot8(v0, xs + c, b0);
    a1 = dot8(u1, xs + c + 256, a1), b1 = dot8(v1, xs + c + 256, b1);
  }
  if (c < K) {
    const uint4 u0 = ld_stream16(r0 + c), v0 = ld_stream16(r1 + c);
    a0 = dot8(u0, xs + c, a0), b0 = dot8(v0, xs + c, b0);
  }
  s0 = warp_sum(a0 + a1), s1 = warp_sum(b0 + b1);
}

__global__ void __launch_bounds__(GB_WARPS * 32) gemv_bf16_multi_kernel(const __nv_bfloat16 *__restrict__ x, const __grid_constant__ GbSegs segs,
                                                                       int K, int out_f32) {
  extern __shared__ __align__(16) float xs[];
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  stage_x(x, xs, K);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total = segs.end[segs.count - 1];
  const int stride = gridDim.x * GB_WARPS * 2;
  for (int row = (blockIdx.x * GB_WARPS + warp) * 2; row < total; row += stride) {
    // rows `row` and `row + 1` of the joint list (the second may belong to the next matrix, or not exist)
    const __nv_bfloat16 *wr[2];
    void *dst[2];
    int idx[2];
#pragma unroll
    for (int j = 0; j < 2; j++) {
      const int r = row + j < total ? row + j : row;
      int s = 0, base = 0;
#pragma unroll
      for (int i = 1; i < 4; i++)
        if (i < segs.count && r >= segs.end[i - 1]) s = i, base = segs.end[i - 1];
      wr[j] = segs.w[s] + (size_t)(r - base) * K, dst[j] = segs.y[s], idx[j] = r - base;
    }
    float s0, s1;
    rows2(wr[0], wr[1], xs, K, lane, s0, s1);
    if (lane == 0) {
      if (out_f32) {
        reinterpret_cast<float *>(dst[0])[idx[0]] = s0;
        if (row + 1 < total) reinterpret_cast<float *>(dst[1])[idx[1]] = s1;
      } else {
        reinterpret_cast<__nv_bfloat16 *>(dst[0])[idx[0]] = __float2bfloat16_rn(s0);
        if (row + 1 < total) reinterpret_cast<__nv_bfloat16 *>(dst[1])[idx[1]] = __float2bfloat16_rn(s1);
      }
    }
  }
}

// y[r] = act(x . Wg[r]) * (x . Wu[r]): both products rounded to bf16 first, the activation rounded to bf16, then the
// product rounded -- the roundings the unfused sequence (two bf16 GEMVs, activation, multiply) leaves
// (reference kernels/cuda/src/gemv.cu:85-118).
__global__ void __launch_bounds__(GB_WARPS * 32) gemv_bf16_gated_kernel(const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ wg,
                                                                       const __nv_bfloat16 *__restrict__ wu, __nv_bfloat16 *__restrict__ y, int N, int K,
                                                                       int gelu) {
  extern __shared__ __align__(16) float xs[];
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  stage_x(x, xs, K);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int row = blockIdx.x * GB_WARPS + warp; row < N; row += gridDim.x * GB_WARPS) {
    float g, u;
    rows2(wg + (size_t)row * K, wu + (size_t)row * K, xs, K, lane, g, u);
    if (lane == 0) {
      const float gb = __bfloat162float(__float2bfloat16_rn(g)), ub = __bfloat162float(__float2bfloat16_rn(u));
      float a = gelu ? 0.5f * gb * (1.f + erff(gb * 0.70710678118654752f)) : gb / (1.f + expf(-gb));
      a = __bfloat162float(__float2bfloat16_rn(a));
      y[row] = __float2bfloat16_rn(a * ub);
    }
  }
}

template <typename... Args>
cudaError_t launch_pdl(void (*kern)(Args...), unsigned grid, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid), cfg.blockDim = dim3(GB_WARPS * 32), cfg.dynamicSmemBytes = smem, cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

}  // namespace

int gemv_bf16_multi(const void *x, const void *const *w, void *const *out, const int *n, int count, int K, int out_f32, cudaStream_t st) {
  if (K > GB_MAXK) return fail(LB200_E_TOO_LARGE, "light_b200: gemv_multi: K=%d exceeds %d", K, GB_MAXK);
  static DeviceOnce attr;
  cudaError_t e = attr.ensure([&] {
    cudaError_t r = cudaFuncSetAttribute(gemv_bf16_multi_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GB_MAXK * 4);
    return r != cudaSuccess ? r : cudaFuncSetAttribute(gemv_bf16_gated_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GB_MAXK * 4);
  });
  if (e != cudaSuccess) return fail((int)e, "light_b200: gemv_multi: %s", cudaGetErrorString(e));
  GbSegs s = {};
  int total = 0;
  for (int i = 0; i < count; i++) {
    s.w[i] = (const __nv_bfloat16 *)w[i], s.y[i] = out[i], s.n[i] = n[i];
    total += n[i];
    s.end[i] = total;
  }
  s.count = count;
  const int pairs = (total + 1) / 2, want = (pairs + GB_WARPS - 1) / GB_WARPS, cap = sm_count() * 4;
  e = launch_pdl(gemv_bf16_multi_kernel, (unsigned)(want < cap ? want : cap), (size_t)K * 4, st, (const __nv_bfloat16 *)x, s, K, out_f32);
  if (e != cudaSuccess) return fail((int)e, "light_b200: gemv_multi: %s", cudaGetErrorString(e));
  return launched("gemv_multi");
}

int gemv_bf16_gated(const void *x, const void *wg, const void *wu, void *y, int N, int K, int gelu, cudaStream_t st) {
  if (K > GB_MAXK) return fail(LB200_E_TOO_LARGE, "light_b200: gemv_gated: K=%d exceeds %d", K, GB_MAXK);
  static DeviceOnce attr;
  cudaError_t e = attr.ensure([&] { return cudaFuncSetAttribute(gemv_bf16_gated_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GB_MAXK * 4); });
  if (e != cudaSuccess) return fail((int)e, "light_b200: gemv_gated: %s", cudaGetErrorString(e));
  const int want = (N + GB_WARPS - 1) / GB_WARPS, cap = sm_count() * 4;
  e = launch_pdl(gemv_bf16_gated_kernel, (unsigned)(want < cap ? want : cap), (size_t)K * 4, st, (const __nv_bfloat16 *)x, (const __nv_bfloat16 *)wg,
                 (const __nv_bfloat16 *)wu, (__nv_bfloat16 *)y, N, K, gelu);
  if (e != cudaSuccess) return fail((int)e, "light_b200: gemv_gated: %s", cudaGetErrorString(e));
  return launched("gemv_gated");
}

}  // namespace lb
