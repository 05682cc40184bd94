// Grouped expert matmul over routed (token, slot) pairs (contract: reference
// kernels/cuda/src/moe.cu:1-24, ops/moe.go:96-107):
//
//   out[p, :] = w(p) * input[row(p), :] . weights[e, :, :]^T      for every sorted pair
//
// Pairs arrive sorted by expert, so expert e owns the index range offsets[e] .. offsets[e+1].
// The ranges come from boundary detection on the sorted expert ids (no atomics, deterministic);
// every output row is written by exactly one warp lane set, so the result is deterministic too.
#include <cuda_fp8.h>

#include <mutex>

#include "gguf_decode.cuh"

namespace lb {

// Non-zero once an expert id outside [0, E) was seen by the offsets kernel (sticky; light_b200_moe_route_status
// reports it together with the routing kernels' own word).
__device__ unsigned int g_moe_bad_ids;

// offsets[e] = first sorted index whose expert id is >= e, for e <= E (so offsets[E] = M when every id is an
// expert).  Nobody validates the ids before this kernel, so it does: both ends of a boundary are clamped
// into [-1, E] and made non-decreasing before they index anything.  A negative id therefore owns no range,
// an id >= E lies at or beyond offsets[E], outside every expert's range (the matmul kernels skip both), and
// either sets the status word.
__global__ void moe_offsets_kernel(const int64_t *__restrict__ ids, int32_t *__restrict__ offsets, long long M, int E) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (M == 0) {
    if (i <= E) offsets[i] = 0;
    return;
  }
  if (i >= M) return;
  long long cur = ids[i], prev = i == 0 ? -1 : ids[i - 1];
  if (cur < 0 || cur >= E) g_moe_bad_ids = 1u;
  cur = cur < -1 ? -1 : (cur > E ? E : cur);
  prev = prev < -1 ? -1 : (prev > E ? E : prev);
  if (cur < prev) cur = prev;  // unsorted input: no boundary here, and no store below
  for (long long e = prev + 1; e <= cur; e++) offsets[e] = (int32_t)i;
  if (i == M - 1)
    for (long long e = cur + 1; e <= E; e++) offsets[e] = (int32_t)M;
}

__global__ void moe_counts_kernel(const int32_t *__restrict__ offsets, int32_t *__restrict__ counts, int E) {
  int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e < E) counts[e] = offsets[e + 1] - offsets[e];
}

__device__ __forceinline__ void load8(const float *p, float v[8]) {
  float4 a = __ldg(reinterpret_cast<const float4 *>(p)), b = __ldg(reinterpret_cast<const float4 *>(p) + 1);
  v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16 *p, float v[8]) {
  uint4 u = __ldg(reinterpret_cast<const uint4 *>(p));
  const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&u);
#pragma unroll
  for (int i = 0; i < 4; i++) {
    float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x, v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void load8(const __half *p, float v[8]) {
  uint4 u = __ldg(reinterpret_cast<const uint4 *>(p));
  const __half2 *h = reinterpret_cast<const __half2 *>(&u);
#pragma unroll
  for (int i = 0; i < 4; i++) {
    float2 f = __half22float2(h[i]);
    v[2 * i] = f.x, v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void st_out(float *p, long long i, float v) { p[i] = v; }
__device__ __forceinline__ void st_out(__nv_bfloat16 *p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }
__device__ __forceinline__ void st_out(__half *p, long long i, float v) { p[i] = __float2half_rn(v); }

constexpr int MOE_MT = 8;     // sorted pairs per tile
constexpr int MOE_WARPS = 8;  // output columns per CTA

// What a row fetcher needs beyond the weight pointer: block-scaled FP8 (scale, bR, bC) and group-quantized 4-bit
// (scale, zeros, bC = group).
struct RowAux {
  const float *scale;
  int bR, bC;
  const float *zeros;
};

// Weight row fetchers: eight consecutive K elements of row n of expert e as f32.
template <typename T>
struct DenseRow {
  const T *row;
  __device__ DenseRow(const void *w, long long e, int n, int N, int K, const RowAux &) : row((const T *)w + ((size_t)e * N + n) * K) {}
  __device__ __forceinline__ void get(int k, float v[8]) const { load8(row + k, v); }
};
template <int QT>
struct QuantRow {
  const uint8_t *row;
  __device__ QuantRow(const void *w, long long e, int n, int N, int K, const RowAux &)
      : row((const uint8_t *)w + ((size_t)e * N + n) * (size_t)(K / block_elems(QT)) * block_bytes(QT)) {}
  __device__ __forceinline__ void get(int k, float v[8]) const {
    int b = k / block_elems(QT);
    decode8<QT>(row + (size_t)b * block_bytes(QT), k - b * block_elems(QT), v);
  }
};

// Block-scaled e4m3 codes (E, N, K) with f32 scales (E, N / bR, K / bC), bC % 8 == 0: the weight is code * scale
// rounded to the activation type TA, i.e. the value a dequantize-then-matmul at that type multiplies with
// (reference ops/fp8_block.go:13-60 followed by ops.MoEGemm).
template <typename TA>
struct F8BlockRow {
  const uint8_t *row;
  const float *srow;
  int bC;
  __device__ F8BlockRow(const void *w, long long e, int n, int N, int K, const RowAux &aux)
      : row((const uint8_t *)w + ((size_t)e * N + n) * K),
        srow(aux.scale + ((size_t)e * (N / aux.bR) + n / aux.bR) * (size_t)(K / aux.bC)),
        bC(aux.bC) {}
  __device__ __forceinline__ void get(int k, float v[8]) const {
    const uint2 q = __ldg(reinterpret_cast<const uint2 *>(row + k));
    const float sc = __ldg(srow + k / bC);
    const uint32_t u[2] = {q.x, q.y};
#pragma unroll
    for (int h = 0; h < 2; h++) {
      __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(u[h] & 0xFFFFu), __NV_E4M3);
      __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(u[h] >> 16), __NV_E4M3);
      const float2 a = __half22float2(__half2(lo)), b = __half22float2(__half2(hi));
      v[4 * h + 0] = round_to(a.x * sc), v[4 * h + 1] = round_to(a.y * sc), v[4 * h + 2] = round_to(b.x * sc), v[4 * h + 3] = round_to(b.y * sc);
    }
  }
  static __device__ __forceinline__ float round_to(float f) {
    if constexpr (sizeof(TA) == 2) return __bfloat162float(__float2bfloat16_rn(f));
    return f;
  }
};

// Group-quantized 4-bit rows in the canonical layout (codes u32 (N, K/8), nibble j of word c = W[n, 8c + j]; scales and
// zeros f32 (N, K/G), G % 8 == 0): eight weights are one code word, w = s * (q - z) with the two operations rounded
// separately, as the dequantize kernel forms them.
struct Int4Row {
  const uint32_t *row;
  const float *srow, *zrow;
  int G;
  __device__ Int4Row(const void *w, long long e, int n, int N, int K, const RowAux &aux)
      : row((const uint32_t *)w + ((size_t)e * N + n) * (size_t)(K / 8)),
        srow(aux.scale + ((size_t)e * N + n) * (size_t)(K / aux.bC)),
        zrow(aux.zeros + ((size_t)e * N + n) * (size_t)(K / aux.bC)),
        G(aux.bC) {}
  __device__ __forceinline__ void get(int k, float v[8]) const {
    const uint32_t q = __ldg(row + (k >> 3));
    const float sc = __ldg(srow + k / G), zp = __ldg(zrow + k / G);
#pragma unroll
    for (int j = 0; j < 8; j++) v[j] = __fmul_rn(sc, __fsub_rn((float)((q >> (4 * j)) & 0xFu), zp));
  }
};

// One warp: one output column n, the pairs of one tile.  A tile may straddle experts; each run
// of equal expert id inside it is handled with that expert's weight row.
template <typename TI, typename TO, typename Row>
__global__ void __launch_bounds__(MOE_WARPS * 32) moe_gemm_kernel(
    const TI *__restrict__ in, const void *__restrict__ w, const int64_t *__restrict__ pairs,
    const int64_t *__restrict__ ids, const int32_t *__restrict__ offsets, const float *__restrict__ topkw,
    TO *__restrict__ out, long long M, long long sizeM, int E, int N, int K, int topk, int rowPerPair, RowAux aux) {
  const int lane = threadIdx.x & 31;
  const int n = blockIdx.x * MOE_WARPS + (threadIdx.x >> 5);
  if (n >= N) return;
  const long long t0 = (long long)blockIdx.y * MOE_MT, t1 = t0 + MOE_MT < M ? t0 + MOE_MT : M;
  long long i = t0;
  while (i < t1) {
    const long long e = ids ? ids[i] : 0;  // no routing: one weight matrix, row m of the input gives row m of the output
    if (e < 0 || e >= E) {  // not an expert: the pair is skipped, as an out-of-range pair id is
      i++;
      continue;
    }
    long long r1 = ids ? offsets[e + 1] : t1;
    if (r1 > t1) r1 = t1;
    if (r1 <= i) r1 = i + 1;  // unsorted input: still make progress
    const int cnt = (int)(r1 - i);
    const TI *xrow[MOE_MT];
    long long pr[MOE_MT];
#pragma unroll
    for (int m = 0; m < MOE_MT; m++) {
      long long p = m < cnt ? (pairs ? pairs[i + m] : i + m) : -1;
      if (p < 0 || p >= sizeM) p = -1;
      pr[m] = p;
      xrow[m] = p < 0 ? nullptr : in + (size_t)(rowPerPair ? p : p / topk) * K;
    }
    float acc[MOE_MT];
#pragma unroll
    for (int m = 0; m < MOE_MT; m++) acc[m] = 0.f;
    Row wr(w, e, n, N, K, aux);
    for (int k = lane * 8; k < K; k += 256) {
      float wv[8];
      wr.get(k, wv);
#pragma unroll
      for (int m = 0; m < MOE_MT; m++) {
        if (xrow[m]) {
          float xv[8];
          load8(xrow[m] + k, xv);
#pragma unroll
          for (int j = 0; j < 8; j++) acc[m] = fmaf(wv[j], xv[j], acc[m]);
        }
      }
    }
#pragma unroll
    for (int m = 0; m < MOE_MT; m++) {
      float v = warp_sum(acc[m]);
      if (lane == 0 && pr[m] >= 0) st_out(out, pr[m] * N + n, topkw ? v * topkw[pr[m]] : v);
    }
    i = r1;
  }
}

static int prep(const lb200_moe_args *a, cudaStream_t st) {
  long long work = a->M > a->E + 1 ? a->M : a->E + 1;
  moe_offsets_kernel<<<(unsigned)((work + 255) / 256), 256, 0, st>>>(a->expert_ids, a->offsets, a->M, a->E);
  int rc = launched("moe expert offsets");
  if (rc) return rc;
  moe_counts_kernel<<<(a->E + 255) / 256, 256, 0, st>>>(a->offsets, a->counts, a->E);
  return launched("moe expert counts");
}

template <typename TI, typename TO, typename Row>
static int run(const lb200_moe_args *a, cudaStream_t st, RowAux aux = RowAux{nullptr, 0, 0, nullptr}) {
  if (a->M == 0 || a->N == 0) return 0;
  dim3 grid((a->N + MOE_WARPS - 1) / MOE_WARPS, (unsigned)((a->M + MOE_MT - 1) / MOE_MT));
  if ((a->M + MOE_MT - 1) / MOE_MT > 65535)
    return fail(LB200_E_TOO_LARGE, "moe_gemm: %lld pairs exceed the kernel's grid", (long long)a->M);
  moe_gemm_kernel<TI, TO, Row><<<grid, MOE_WARPS * 32, 0, st>>>(
      (const TI *)a->input, a->weights, a->sorted_pairs, a->expert_ids, a->offsets, a->topk_weights, (TO *)a->out, a->M,
      a->size_m, a->E, a->N, a->K, a->topk, a->row_per_pair, aux);
  return launched("moe_gemm");
}

// x (M, K) . W^T for one matrix through the same tile kernel (no routing): the shapes the tensor-core and one-row kernels
// of these formats do not take (K % 256 != 0, groups or blocks that are not multiples of 64).
template <typename T, typename Row>
static int run_plain(const void *x, const void *w, void *y, int M, int N, int K, const RowAux &aux, cudaStream_t st) {
  if (M == 0 || N == 0) return 0;
  dim3 grid((N + MOE_WARPS - 1) / MOE_WARPS, (unsigned)((M + MOE_MT - 1) / MOE_MT));
  if ((M + MOE_MT - 1) / MOE_MT > 65535) return fail(LB200_E_TOO_LARGE, "light_b200: matmul: %d rows exceed the kernel's grid", M);
  moe_gemm_kernel<T, T, Row><<<grid, MOE_WARPS * 32, 0, st>>>((const T *)x, w, nullptr, nullptr, nullptr, nullptr, (T *)y, M, M, 1, N, K, 1, 1, aux);
  return launched("matmul (row fetcher)");
}

int int4_rows_dot(const void *x, const uint32_t *codes, const float *s, const float *z, void *y, int act_dtype, int M, int N, int K, int G,
                  cudaStream_t st) {
  const RowAux aux{s, 0, G, z};
  if (act_dtype == LB200_F32) return run_plain<float, Int4Row>(x, codes, y, M, N, K, aux, st);
  return run_plain<__nv_bfloat16, Int4Row>(x, codes, y, M, N, K, aux, st);
}

int fp8_block_rows_dot(const void *x, const uint8_t *w, const float *s, void *y, int act_dtype, int M, int N, int K, int bR, int bC,
                       cudaStream_t st) {
  const RowAux aux{s, bR, bC, nullptr};
  if (act_dtype == LB200_F32) return run_plain<float, F8BlockRow<float>>(x, w, y, M, N, K, aux, st);
  return run_plain<__nv_bfloat16, F8BlockRow<__nv_bfloat16>>(x, w, y, M, N, K, aux, st);
}

int moe_bad_ids_status() {
  unsigned int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_moe_bad_ids, sizeof(v));
  if (e != cudaSuccess) return fail((int)e, "light_b200: moe status: %s", cudaGetErrorString(e));
  return (int)v;
}

int moe_gemm(const lb200_moe_args *a, int device, cudaStream_t st) {
  int rc = prep(a, st);
  if (rc) return rc;
  if (int took = moe_umma(a, 0, nullptr, 0, 0, device, st)) return took == 1 ? 0 : took;
  switch (a->dtype) {
    case LB200_F32: return run<float, float, DenseRow<float>>(a, st);
    case LB200_BF16: return run<__nv_bfloat16, __nv_bfloat16, DenseRow<__nv_bfloat16>>(a, st);
    case LB200_F16: return run<__half, __half, DenseRow<__half>>(a, st);
  }
  return fail(LB200_E_DTYPE, "moe_gemm: element type %d has no kernel", a->dtype);
}

// ---- grouped matmul whose expert counts / offsets live in this library's own device memory.
//
// The scratch is one file-scope device array, so the entry point needs no allocation by anyone:
// not by the caller, not by this library, not by a tensor pool.  In host code the array's name
// is only a stand-in for the device symbol, so its device address is looked up once per device
// (with that device current) and that address is what the kernels are given.
static __device__ __align__(256) int32_t g_moe_static_scratch[2 * LB200_MOE_STATIC_MAX_EXPERTS + 2];
static int32_t *g_moe_static_ptr[64];
static std::mutex g_moe_static_mu;

int moe_gemm_static_scratch(const lb200_moe_args *a, int device, cudaStream_t st) {
  if (a->E > LB200_MOE_STATIC_MAX_EXPERTS)
    return fail(LB200_E_TOO_LARGE, "light_b200: moe_gemm_static_scratch: %d experts exceed the built-in scratch (max %d)",
                a->E, LB200_MOE_STATIC_MAX_EXPERTS);
  int32_t *base;
  {
    std::lock_guard<std::mutex> lk(g_moe_static_mu);
    base = g_moe_static_ptr[device];
    if (!base) {  // first call on this device: resolve the symbol's device address
      cudaError_t e = cudaGetSymbolAddress((void **)&base, g_moe_static_scratch);
      if (e != cudaSuccess)
        return fail((int)e, "light_b200: moe_gemm_static_scratch: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
      g_moe_static_ptr[device] = base;
    }
  }
  lb200_moe_args b = *a;
  b.counts = base;                                      // E entries
  b.offsets = base + LB200_MOE_STATIC_MAX_EXPERTS + 1;  // E + 1 entries
  // Both ranges are fully overwritten by the offsets / counts kernels before the matmul reads
  // them, so what an earlier call left behind never matters and nothing needs clearing.
  return moe_gemm(&b, device, st);
}

int moe_gemm_f8block(const lb200_moe_args *a, const float *w_scale, int bR, int bC, int device, cudaStream_t st) {
  int rc = prep(a, st);
  if (rc) return rc;
  int took = moe_umma(a, 2, w_scale, bR, bC, device, st);
  if (took == 1) return 0;
  if (took) return took;
  // Few pairs (a decode step), or a shape the tensor-core path does not take: one warp per output column and
  // tile of sorted pairs, the weight row read once per tile.
  if (bR <= 0 || bC <= 0 || bC % 8 || a->K % bC || a->N % bR || a->K % 8)
    return fail(LB200_E_SHAPE, "light_b200: moe_gemm_f8block: N=%d K=%d with blocks (%d, %d): block_c must be a multiple of 8 and the blocks must tile the weight",
                a->N, a->K, bR, bC);
  const RowAux aux{w_scale, bR, bC, nullptr};
  if (a->dtype == LB200_F32) return run<float, float, F8BlockRow<float>>(a, st, aux);
  return run<__nv_bfloat16, __nv_bfloat16, F8BlockRow<__nv_bfloat16>>(a, st, aux);
}

int moe_gemm_q(const lb200_moe_args *a, int device, cudaStream_t st) {
  int rc = prep(a, st);
  if (rc) return rc;
  if (int took = moe_umma(a, 1, nullptr, 0, 0, device, st)) return took == 1 ? 0 : took;
  switch (a->dtype) {
    case LB200_Q4_0: return run<float, float, QuantRow<LB200_Q4_0>>(a, st);
    case LB200_Q5_0: return run<float, float, QuantRow<LB200_Q5_0>>(a, st);
    case LB200_Q8_0: return run<float, float, QuantRow<LB200_Q8_0>>(a, st);
    case LB200_Q4_K: return run<float, float, QuantRow<LB200_Q4_K>>(a, st);
    case LB200_Q5_K: return run<float, float, QuantRow<LB200_Q5_K>>(a, st);
    case LB200_Q6_K: return run<float, float, QuantRow<LB200_Q6_K>>(a, st);
  }
  return fail(LB200_E_DTYPE, "moe_gemm_q: ggml type %d has no kernel", a->dtype);
}

}  // namespace lb
