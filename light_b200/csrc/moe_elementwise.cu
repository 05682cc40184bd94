// The element-wise steps between and after the two grouped matmuls of a sparse MoE block (reference
// nn/moe.go:206-236: Narrow gate / up -> SiLU -> Mul, then ops.MoECombine, ops/moe.go:206-240), each as ONE launch with
// the roundings of the unfused sequence: the activation rounded to the tensor dtype, then the product; the slot
// rows added one after the other, slot 0 first, each sum rounded to the tensor dtype.
#include "common.cuh"

namespace lb {
namespace {

template <typename T>
__device__ __forceinline__ float rnd(float v);
template <>
__device__ __forceinline__ float rnd<float>(float v) { return v; }
template <>
__device__ __forceinline__ float rnd<__nv_bfloat16>(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
template <>
__device__ __forceinline__ float rnd<__half>(float v) { return __half2float(__float2half_rn(v)); }

template <typename T>
struct alignas(16) Vec8 {  // eight elements: one 16-byte access (bf16 / f16) or two (f32)
  T v[8];
};

// h (M, 2 I): gate = h[:, :I], up = h[:, I:] -> out (M, I) = act(gate) * up; eight elements per thread
template <typename T>
__global__ void __launch_bounds__(256) moe_gate_mul_kernel(const T *__restrict__ h, T *__restrict__ out, long long M, int I, int gelu) {
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
  const long long per_row = I / 8, total = M * per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long m = i / per_row;
    const int c = (int)(i - m * per_row) * 8;
    const Vec8<T> g = *reinterpret_cast<const Vec8<T> *>(h + m * 2 * I + c), u = *reinterpret_cast<const Vec8<T> *>(h + m * 2 * I + I + c);
    Vec8<T> o;
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const float gv = (float)g.v[j];
      const float a = gelu ? 0.5f * gv * (1.f + erff(gv * 0.70710678118654752f)) : gv / (1.f + expf(-gv));
      o.v[j] = (T)(rnd<T>(a) * (float)u.v[j]);
    }
    *reinterpret_cast<Vec8<T> *>(out + m * I + c) = o;
  }
}

// pair_out (T * topk, N) -> out (T, N): ((row 0 + row 1) + row 2) + ..., every sum rounded to T
template <typename T>
__global__ void __launch_bounds__(256) moe_combine_kernel(const T *__restrict__ pair_out, T *__restrict__ out, long long tokens, int N, int topk) {
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
  const long long per_row = N / 8, total = tokens * per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / per_row;
    const int c = (int)(i - t * per_row) * 8;
    const T *src = pair_out + t * topk * (long long)N + c;
    float acc[8];
    {
      const Vec8<T> r = *reinterpret_cast<const Vec8<T> *>(src);
#pragma unroll
      for (int j = 0; j < 8; j++) acc[j] = (float)r.v[j];
    }
    for (int s = 1; s < topk; s++) {
      const Vec8<T> r = *reinterpret_cast<const Vec8<T> *>(src + (long long)s * N);
#pragma unroll
      for (int j = 0; j < 8; j++) acc[j] = rnd<T>(acc[j] + (float)r.v[j]);
    }
    Vec8<T> o;
#pragma unroll
    for (int j = 0; j < 8; j++) o.v[j] = (T)acc[j];
    *reinterpret_cast<Vec8<T> *>(out + t * N + c) = o;
  }
}

// rows (n_rows, N) in any order, index[p] = the row of pair p (outside [0, n_rows): the pair contributes nothing),
// weights[p] its routing weight -> out f32 (tokens, N) = sum over a token's slots, slot 0 first, accumulated in f32:
// the receiving end of an expert-parallel combine, where the rows come back in expert order
template <typename T>
__global__ void __launch_bounds__(256) moe_combine_weighted_kernel(const T *__restrict__ rows, const int64_t *__restrict__ index,
                                                                   const float *__restrict__ weights, float *__restrict__ out,
                                                                   long long tokens, int N, int topk, long long n_rows) {
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
  const long long per_row = N / 8, total = tokens * per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / per_row;
    const int c = (int)(i - t * per_row) * 8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < topk; s++) {
      const long long p = t * topk + s, r = index ? index[p] : p;
      if (r < 0 || r >= n_rows) continue;
      const float w = weights ? weights[p] : 1.f;
      const Vec8<T> v = *reinterpret_cast<const Vec8<T> *>(rows + r * (long long)N + c);
#pragma unroll
      for (int j = 0; j < 8; j++) acc[j] = fmaf((float)v.v[j], w, acc[j]);
    }
    float4 *o = reinterpret_cast<float4 *>(out + t * N + c);
    o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
}

template <typename K, typename... Args>
int go(K kern, long long work, cudaStream_t st, const char *what, Args... args) {
  long long blocks = (work + 255) / 256;
  const long long cap = (long long)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)blocks), cfg.blockDim = dim3(256), cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, args...);
  if (e != cudaSuccess) return fail((int)e, "light_b200: %s: %s", what, cudaGetErrorString(e));
  return launched(what);
}

}  // namespace

int moe_gate_mul(const void *h, void *out, int dtype, long long M, int I, int gelu, cudaStream_t st) {
  const long long work = M * (I / 8);
  switch (dtype) {
    case LB200_F32: return go(moe_gate_mul_kernel<float>, work, st, "moe_gate_mul", (const float *)h, (float *)out, M, I, gelu);
    case LB200_BF16: return go(moe_gate_mul_kernel<__nv_bfloat16>, work, st, "moe_gate_mul", (const __nv_bfloat16 *)h, (__nv_bfloat16 *)out, M, I, gelu);
    case LB200_F16: return go(moe_gate_mul_kernel<__half>, work, st, "moe_gate_mul", (const __half *)h, (__half *)out, M, I, gelu);
  }
  return fail(LB200_E_DTYPE, "light_b200: moe_gate_mul: element type %d", dtype);
}

int moe_combine(const void *pair_out, void *out, int dtype, long long tokens, int N, int topk, cudaStream_t st) {
  const long long work = tokens * (N / 8);
  switch (dtype) {
    case LB200_F32: return go(moe_combine_kernel<float>, work, st, "moe_combine", (const float *)pair_out, (float *)out, tokens, N, topk);
    case LB200_BF16: return go(moe_combine_kernel<__nv_bfloat16>, work, st, "moe_combine", (const __nv_bfloat16 *)pair_out, (__nv_bfloat16 *)out, tokens, N, topk);
    case LB200_F16: return go(moe_combine_kernel<__half>, work, st, "moe_combine", (const __half *)pair_out, (__half *)out, tokens, N, topk);
  }
  return fail(LB200_E_DTYPE, "light_b200: moe_combine: element type %d", dtype);
}

int moe_combine_weighted(const void *rows, const int64_t *index, const float *weights, float *out, int dtype, long long tokens, int N,
                         int topk, long long n_rows, cudaStream_t st) {
  const long long work = tokens * (N / 8);
  switch (dtype) {
    case LB200_F32: return go(moe_combine_weighted_kernel<float>, work, st, "moe_combine_weighted", (const float *)rows, index, weights, out, tokens, N, topk, n_rows);
    case LB200_BF16: return go(moe_combine_weighted_kernel<__nv_bfloat16>, work, st, "moe_combine_weighted", (const __nv_bfloat16 *)rows, index, weights, out, tokens, N, topk, n_rows);
    case LB200_F16: return go(moe_combine_weighted_kernel<__half>, work, st, "moe_combine_weighted", (const __half *)rows, index, weights, out, tokens, N, topk, n_rows);
  }
  return fail(LB200_E_DTYPE, "light_b200: moe_combine_weighted: element type %d", dtype);
}

}  // namespace lb
