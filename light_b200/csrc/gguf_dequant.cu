// GGUF blocks -> f32, bit-identical to the reference's CPU decoders.
//
// One thread expands eight consecutive elements and writes them as two 16-byte stores, so a
// warp writes 1 KiB contiguously.  The kernel is bound by the 4 B/element it writes.
#include "gguf_decode.cuh"

namespace lb {

template <int T>
__global__ void __launch_bounds__(256) gguf_dequant_kernel(const uint8_t *__restrict__ src, float *__restrict__ dst,
                                                           long long n8) {
  constexpr int BE = block_elems(T), BB = block_bytes(T);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    long long e = i * 8, b = e / BE;
    float v[8];
    decode8<T>(src + b * BB, (int)(e - b * BE), v);
    float4 *o = reinterpret_cast<float4 *>(dst + e);
    o[0] = make_float4(v[0], v[1], v[2], v[3]);
    o[1] = make_float4(v[4], v[5], v[6], v[7]);
  }
}

template <int T>
static int run(const void *src, float *dst, long long n, cudaStream_t st) {
  long long n8 = n / 8;
  if (n8 == 0) return 0;
  long long blocks = (n8 + 255) / 256;
  if (blocks > 148LL * 64) blocks = 148LL * 64;
  gguf_dequant_kernel<T><<<(unsigned)blocks, 256, 0, st>>>((const uint8_t *)src, dst, n8);
  return launched("dequant");
}

int gguf_dequant(int type, const void *src, float *dst, long long n, cudaStream_t st) {
  switch (type) {
    case LB200_Q4_0: return run<LB200_Q4_0>(src, dst, n, st);
    case LB200_Q5_0: return run<LB200_Q5_0>(src, dst, n, st);
    case LB200_Q8_0: return run<LB200_Q8_0>(src, dst, n, st);
    case LB200_Q4_K: return run<LB200_Q4_K>(src, dst, n, st);
    case LB200_Q5_K: return run<LB200_Q5_K>(src, dst, n, st);
    case LB200_Q6_K: return run<LB200_Q6_K>(src, dst, n, st);
  }
  return fail(LB200_E_DTYPE, "dequant: ggml type %d has no kernel", type);
}

// Quantized embedding lookup: row ids[i] of a block-quantized table (V, K) -> f32 row i of out, the reference's
// nn.Embedding over a quantized table (IndexSelect of the byte rows, then Dequantize of the gathered rows only,
// nn/embedding.go; tested by nn/embedding_test.go:127).  An id outside [0, V) yields a row of zeros.
template <int T>
__global__ void __launch_bounds__(256) gguf_embedding_kernel(const uint8_t *__restrict__ table, const long long *__restrict__ ids,
                                                             float *__restrict__ out, long long V, int K) {
  constexpr int BE = block_elems(T), BB = block_bytes(T);
  const long long id = ids[blockIdx.x];
  const uint8_t *row = table + (size_t)id * (size_t)(K / BE) * BB;
  float *dst = out + (size_t)blockIdx.x * K;
  for (int e = threadIdx.x * 8; e < K; e += 256 * 8) {
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (id >= 0 && id < V) decode8<T>(row + (size_t)(e / BE) * BB, e % BE, v);
    float4 *o = reinterpret_cast<float4 *>(dst + e);
    o[0] = make_float4(v[0], v[1], v[2], v[3]);
    o[1] = make_float4(v[4], v[5], v[6], v[7]);
  }
}

template <int T>
static int run_embedding(const void *table, const int64_t *ids, float *out, long long n_ids, long long V, int K, cudaStream_t st) {
  gguf_embedding_kernel<T><<<(unsigned)n_ids, 256, 0, st>>>((const uint8_t *)table, (const long long *)ids, out, V, K);
  return launched("embedding_q");
}

int gguf_embedding(int type, const void *table, const int64_t *ids, float *out, long long n_ids, long long V, int K, cudaStream_t st) {
  if (n_ids == 0) return 0;
  switch (type) {
    case LB200_Q4_0: return run_embedding<LB200_Q4_0>(table, ids, out, n_ids, V, K, st);
    case LB200_Q5_0: return run_embedding<LB200_Q5_0>(table, ids, out, n_ids, V, K, st);
    case LB200_Q8_0: return run_embedding<LB200_Q8_0>(table, ids, out, n_ids, V, K, st);
    case LB200_Q4_K: return run_embedding<LB200_Q4_K>(table, ids, out, n_ids, V, K, st);
    case LB200_Q5_K: return run_embedding<LB200_Q5_K>(table, ids, out, n_ids, V, K, st);
    case LB200_Q6_K: return run_embedding<LB200_Q6_K>(table, ids, out, n_ids, V, K, st);
  }
  return fail(LB200_E_DTYPE, "embedding_q: ggml type %d has no kernel", type);
}

}  // namespace lb
