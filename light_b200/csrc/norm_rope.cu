// The small operators between the quantized matmuls of a decode step: RMSNorm (with the residual add that
// precedes it folded in) and rotary position embedding.  Counterparts of the reference's ops.RMSNorm
// (ops/norm.go:69-111; kernels rmsnorm_f32 / rmsnorm_bf16, kernels/cuda/src/elementwise.cu:275-312,
// CPU kernels/cpu/norm.go:27-95) and ops.RoPE (ops/rope.go:30-77; rope_f32,
// kernels/cuda/src/elementwise.cu:748-774, CPU kernels/cpu/misc_registry.go:27-92).
#include "common.cuh"
#include "mma_sync.cuh"

namespace lb {
namespace {

constexpr int NORM_THREADS = 256;

// One CTA per row.  With `res`: s = x + res (rounded to T, written to `sum_out`: the new residual
// stream), then out = s * rsqrt(mean(s^2) + eps) * weight; without: s = x.  The statistics are f32 sums
// (as the reference's kernels), the reciprocal root is taken in f64 as its CPU path does.
template <typename T>
__global__ void __launch_bounds__(NORM_THREADS) rmsnorm_kernel(const T *__restrict__ x, const T *__restrict__ res,
                                                               const T *__restrict__ weight, T *__restrict__ sum_out,
                                                               T *__restrict__ out, int cols, float eps) {
  __shared__ float part[NORM_THREADS / 32];
  pdl_launch_dependents();
  pdl_wait();
  const long long base = (long long)blockIdx.x * cols;
  float ss = 0.f;
  for (int j = threadIdx.x; j < cols; j += NORM_THREADS) {
    float v = ld_act(x, base + j);
    if (res) {
      v += ld_act(res, base + j);
      st_act(sum_out, base + j, v);
      v = ld_act(sum_out, base + j);  // the rounded sum is what the next operator sees
    }
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < NORM_THREADS / 32; i++) tot += part[i];
  const float inv = (float)(1.0 / sqrt((double)(tot / (float)cols) + (double)eps));
  const T *src = res ? sum_out : x;
  for (int j = threadIdx.x; j < cols; j += NORM_THREADS) st_act(out, base + j, ld_act(src, base + j) * inv * ld_act(weight, j));
}

// x (rows, head_dim), rows = batch * seq_len; rotate-half pairing: dim i with dim i + head_dim / 2 at angle
// positions[row % seq_len] * base^(-2 i / head_dim).  The angle and its sine / cosine are computed in f64
// (the reference's CPU path; its CUDA kernel uses the fast f32 intrinsics and drifts at large angles).
template <typename T>
__global__ void rope_kernel(const T *__restrict__ x, const long long *__restrict__ positions, T *__restrict__ out, long long rows,
                            int seq_len, int head_dim, double neg_log2_base_over_half) {
  pdl_launch_dependents();
  pdl_wait();
  const int half = head_dim >> 1;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (tid >= rows * half) return;
  const long long row = tid / half;
  const int i = (int)(tid - row * half);
  const double theta = (double)positions[row % seq_len] * exp2((double)i * neg_log2_base_over_half);
  double sn, c;
  sincos(theta, &sn, &c);
  const float cf = (float)c, sf = (float)sn;
  const long long o = row * head_dim + i;
  const float x0 = ld_act(x, o), x1 = ld_act(x, o + half);
  st_act(out, o, x0 * cf - x1 * sf);
  st_act(out, o + half, x0 * sf + x1 * cf);
}

// Greedy sampling: the index of the largest element of every row (ties: the lowest index), as I64.  One CTA per
// row; reference ops.Argmax on the last axis (ops/argmax.go:14-60, kernels/cuda/topk.go:56-90).
__global__ void __launch_bounds__(1024) argmax_rows_kernel(const float *__restrict__ x, long long *__restrict__ out, int cols) {
  __shared__ float bv[32];
  __shared__ int bi[32];
  pdl_launch_dependents();
  pdl_wait();
  const float *row = x + (size_t)blockIdx.x * cols;
  float v = -INFINITY;
  int idx = 0x7fffffff;
  for (int j = threadIdx.x; j < cols; j += 1024) {
    const float c = row[j];
    if (c > v || (c == v && j < idx) || idx == 0x7fffffff) v = c, idx = j;  // NaN never wins over a number; the first element seeds
  }
  auto better = [](float a, int ai, float b, int bi_) { return a > b || (a == b && ai < bi_); };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (oi != 0x7fffffff && (idx == 0x7fffffff || better(ov, oi, v, idx))) v = ov, idx = oi;
  }
  if ((threadIdx.x & 31) == 0) bv[threadIdx.x >> 5] = v, bi[threadIdx.x >> 5] = idx;
  __syncthreads();
  if (threadIdx.x < 32) {
    v = bv[threadIdx.x], idx = bi[threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      if (oi != 0x7fffffff && (idx == 0x7fffffff || better(ov, oi, v, idx))) v = ov, idx = oi;
    }
    if (threadIdx.x == 0) out[blockIdx.x] = idx;
  }
}

template <typename K, typename... Args>
cudaError_t launch_chain(K kern, unsigned grid, unsigned block, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid), cfg.blockDim = dim3(block), cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

}  // namespace

int rmsnorm(const void *x, const void *residual, const void *weight, void *sum_out, void *out, int dtype, long long rows, int cols,
            float eps, cudaStream_t st) {
  if (!x || !weight || !out || (residual && !sum_out)) return fail(LB200_E_NULL, "light_b200: rmsnorm: null pointer (a residual needs sum_out)");
  if (rows < 0 || cols <= 0 || rows > 0x7fffffffLL) return fail(LB200_E_SHAPE, "light_b200: rmsnorm: rows %lld cols %d", rows, cols);
  if (rows == 0) return 0;
  cudaError_t e;
  if (dtype == LB200_F32)
    e = launch_chain(rmsnorm_kernel<float>, (unsigned)rows, NORM_THREADS, st, (const float *)x, (const float *)residual, (const float *)weight,
                     (float *)sum_out, (float *)out, cols, eps);
  else if (dtype == LB200_BF16)
    e = launch_chain(rmsnorm_kernel<__nv_bfloat16>, (unsigned)rows, NORM_THREADS, st, (const __nv_bfloat16 *)x, (const __nv_bfloat16 *)residual,
                     (const __nv_bfloat16 *)weight, (__nv_bfloat16 *)sum_out, (__nv_bfloat16 *)out, cols, eps);
  else
    return fail(LB200_E_DTYPE, "light_b200: rmsnorm: element type %d, want F32 or BF16", dtype);
  if (e != cudaSuccess) return fail((int)e, "light_b200: rmsnorm: %s", cudaGetErrorString(e));
  return launched("rmsnorm");
}

int argmax_rows(const float *x, int64_t *out, long long rows, int cols, cudaStream_t st) {
  if (!x || !out) return fail(LB200_E_NULL, "light_b200: argmax: null pointer");
  if (rows < 0 || rows > 0x7fffffffLL || cols <= 0) return fail(LB200_E_SHAPE, "light_b200: argmax: rows %lld cols %d", rows, cols);
  if (rows == 0) return 0;
  cudaError_t e = launch_chain(argmax_rows_kernel, (unsigned)rows, 1024u, st, x, (long long *)out, cols);
  if (e != cudaSuccess) return fail((int)e, "light_b200: argmax: %s", cudaGetErrorString(e));
  return launched("argmax");
}

int rope(const void *x, const int64_t *positions, void *out, int dtype, long long rows, int seq_len, int head_dim, double base,
         cudaStream_t st) {
  if (!x || !positions || !out) return fail(LB200_E_NULL, "light_b200: rope: null pointer");
  if (rows < 0 || seq_len <= 0 || head_dim <= 0 || head_dim % 2 || rows % seq_len || !(base > 0))
    return fail(LB200_E_SHAPE, "light_b200: rope: rows %lld seq_len %d head_dim %d (must be even) base %g", rows, seq_len, head_dim, base);
  if (rows == 0) return 0;
  const long long n = rows * (head_dim / 2);
  if ((n + 255) / 256 > 0x7fffffffLL) return fail(LB200_E_TOO_LARGE, "light_b200: rope: too many rows");
  const double k = -2.0 * log2(base) / (double)head_dim;  // base^(-2 i / head_dim) = 2^(i k)
  cudaError_t e;
  if (dtype == LB200_F32)
    e = launch_chain(rope_kernel<float>, (unsigned)((n + 255) / 256), 256, st, (const float *)x, (const long long *)positions, (float *)out, rows,
                     seq_len, head_dim, k);
  else if (dtype == LB200_BF16)
    e = launch_chain(rope_kernel<__nv_bfloat16>, (unsigned)((n + 255) / 256), 256, st, (const __nv_bfloat16 *)x, (const long long *)positions,
                     (__nv_bfloat16 *)out, rows, seq_len, head_dim, k);
  else
    return fail(LB200_E_DTYPE, "light_b200: rope: element type %d, want F32 or BF16", dtype);
  if (e != cudaSuccess) return fail((int)e, "light_b200: rope: %s", cudaGetErrorString(e));
  return launched("rope");
}

}  // namespace lb
