// Shared declarations of the sm_100a quantized-matmul library.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "../../include/light_b200.h"

namespace lb {

// Records the message light_b200_last_error() returns (thread local) and hands back `code`.
int fail(int code, const char *fmt, ...);
// Maps the launch status of the kernel just enqueued (no synchronisation).
int launched(const char *what);

// Set-up that belongs to ONE device -- the opt-in to more than 48 KB of dynamic shared memory of a kernel
// (cudaFuncSetAttribute), the address of a __device__ symbol -- guarded per device: one process may drive
// several GPUs through this library, from several threads.  ensure(f, want) runs f() with the calling thread's
// current device when that device has not reached level `want` yet (levels only grow: a shared-memory size).
struct DeviceOnce {
  std::mutex mu;
  size_t level[64] = {};
  template <typename F>
  cudaError_t ensure(F &&f, size_t want = 1) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lk(mu);
    if (level[dev] >= want) return cudaSuccess;
    e = f();
    if (e == cudaSuccess) level[dev] = want;
    return e;
  }
};
// SMs of the calling thread's current device (looked up once per device).
int sm_count();

// Block geometry of the GGUF formats with a fused kernel (reference dtype/dtype.go:53-60).
__host__ __device__ constexpr int block_elems(int t) {
  return (t == LB200_Q4_0 || t == LB200_Q5_0 || t == LB200_Q8_0) ? 32
         : (t == LB200_Q4_K || t == LB200_Q5_K || t == LB200_Q6_K) ? 256
                                                                    : 0;
}
__host__ __device__ constexpr int block_bytes(int t) {
  return t == LB200_Q4_0 ? 18 : t == LB200_Q5_0 ? 22 : t == LB200_Q8_0 ? 34 : t == LB200_Q4_K ? 144
         : t == LB200_Q5_K ? 176 : t == LB200_Q6_K ? 210 : 0;
}

__device__ __forceinline__ float f16_bits_to_f32(uint16_t u) {
  __half_raw r;
  r.x = u;
  return __half2float(__half(r));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// activation element access at either f32 or bf16
__device__ __forceinline__ float ld_act(const float *p, long long i) { return p[i]; }
__device__ __forceinline__ float ld_act(const __nv_bfloat16 *p, long long i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void st_act(float *p, long long i, float v) { p[i] = v; }
__device__ __forceinline__ void st_act(__nv_bfloat16 *p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }

// ---- per-file launch entry points (host side), called from abi.cu ----
int gguf_dequant(int type, const void *src, float *dst, long long n, cudaStream_t st);
int gguf_matmul_generic(int type, const float *x, const void *w, float *out, int M, int N, int K, cudaStream_t st);
// returns 1 when a fast decode kernel took the call, 0 when the shape is not covered, <0 on error
int gguf_gemv_fast(int type, const float *x, const void *w, float *out, int M, int N, int K, cudaStream_t st);
int gguf_gemv_fast_init(int device);
int gguf_decode_tile(int type, const float *x, const void *w, float *out, int M, int N, int K, cudaStream_t st);
int gguf_gemv_tp(int type, const float *x, const void *x_slots, const void *const *w, float *const *out, const int *n,
                 int count, int K, void *const *out_slots, const unsigned int *step, int world, int rank, cudaStream_t st);
int gemv_tp_status();
int gguf_gemv_tok(int type, const float *x, const void *w, float *out, int M, int N, int K, cudaStream_t st);
int gguf_gemv_tok_multi(int type, const float *x, const void *const *w, float *const *out, const int *n, int count, int M, int K,
                        cudaStream_t st);
int gguf_gemv_multi(int type, const float *x, const void *const *w, float *const *out, const int *n, int count, int act,
                    int K, cudaStream_t st, const lb200_norm *norm = nullptr);
// batched decode (2..64 rows): 1 = took the call, 0 = not covered, other = error
int gguf_gemv_batch(int type, const float *x, const void *w, float *out, int M, int N, int K, cudaStream_t st);
// tensor-core prefill: 1 = took the call, 0 = shape / workspace not covered, other = error
int gguf_prefill(int type, const float *x, const void *w, float *out, int M, int N, int K, int device, cudaStream_t st);
int int4_prefill(const void *x, const uint32_t *codes, const float *s, const float *z, void *y, int act_dtype, int M, int N,
                 int K, int G, int device, cudaStream_t st);
int fp8_prefill(const void *x, const uint8_t *w, const float *scale, void *y, int act_dtype, int M, int N, int K, int bR,
                int bC, int device, cudaStream_t st);
int set_workspace(int device, void *ptr, size_t bytes);
int comm_step_begin(unsigned int *step, cudaStream_t st);
int allgather_ll(const float *local, float *out, const lb200_peers *peers, int M, int n_local, const unsigned int *step,
                 cudaStream_t st);
int comm_status();
int prefill_status(int device);
int decode_umma_status();
int gguf_decode_umma(int type, const float *x, const void *w, float *out, int M, int N, int K, int device, cudaStream_t st);
int int4_decode_umma(const void *x, const uint32_t *codes, const float *s, const float *z, void *y, int act_dtype, int M, int N,
                     int K, int G, int device, cudaStream_t st);
int fp8_decode_umma(const void *x, const uint8_t *w, const float *scale, void *y, int act_dtype, int M, int N, int K, int bR,
                    int bC, int device, cudaStream_t st);

int int4_dequant(const uint32_t *codes, const float *s, const float *z, void *out, int out_dtype, int N, int K, int G,
                 long long offset, cudaStream_t st);
int int4_rows_dot(const void *x, const uint32_t *codes, const float *s, const float *z, void *y, int act_dtype, int M, int N, int K, int G,
                  cudaStream_t st);
int fp8_block_dequant(const uint8_t *w, const float *s, void *out, int out_dtype, int R, int C, int bR, int bC,
                      cudaStream_t st);
int fp8_block_rows_dot(const void *x, const uint8_t *w, const float *s, void *y, int act_dtype, int M, int N, int K, int bR, int bC,
                       cudaStream_t st);
int moe_gemm(const lb200_moe_args *a, int device, cudaStream_t st);
int moe_gemm_q(const lb200_moe_args *a, int device, cudaStream_t st);
int moe_gemm_f8block(const lb200_moe_args *a, const float *w_scale, int bR, int bC, int device, cudaStream_t st);
int moe_umma(const lb200_moe_args *a, int kind, const float *w_scale, int bR, int bC, int device, cudaStream_t st);
int moe_gemm_static_scratch(const lb200_moe_args *a, int device, cudaStream_t st);
int decode_attn(const lb200_decode_attn_args *a, cudaStream_t st);
int kv_append(const void *k, const void *v, void *kbuf, void *vbuf, const int64_t *pos, int dtype, int B, int KH, int D, int Cap,
              cudaStream_t st);
int inc_i64(int64_t *p, int n, cudaStream_t st);
int decode_attn_status();
int argmax_rows(const float *x, int64_t *out, long long rows, int cols, cudaStream_t st);
int moe_route_sigmoid(const float *logits, const float *bias, int64_t *ids, float *weights, int T, int E, int topk, int norm_topk,
                      cudaStream_t st);
int moe_sort_pairs(const int64_t *ids, int *counts, int *offsets, int64_t *sorted_pairs, int64_t *sorted_expts, int *scratch, long long M,
                   int E, cudaStream_t st);
int moe_route_status();
int moe_route_deepseek(const float *logits, const float *bias, int64_t *ids, float *weights, int T, int E, int topk, int n_group, int topk_group,
                       int sigmoid, int norm_topk, cudaStream_t st);
int moe_route_topk(const float *probs, int64_t *ids, float *weights, int T, int E, int topk, int normalize, cudaStream_t st);
void *workspace_ptr(int device, size_t *bytes);
size_t prefill_sk_ws_bytes();
size_t decode_nt_ws_bytes(int M, int K);
int gguf_decode_nt(int type, const float *x, const void *const *w, float *const *out, const int *n, int count, int M, int K, void *ws,
                   size_t ws_bytes, cudaStream_t st);
int decode_nt_status();
int fp8_decode_nt(const void *x, const uint8_t *w, const float *scale, void *y, int act_dtype, int M, int N, int K, int bR, int bC, void *ws,
                  size_t ws_bytes, cudaStream_t st);
int int4_decode_nt(const void *x, const uint32_t *codes, const float *s, const float *z, void *y, int act_dtype, int M, int N, int K, int G,
                   void *ws, size_t ws_bytes, cudaStream_t st);
size_t decode_ts_ws_bytes(int M, int K);
int gguf_decode_ts(int type, const float *x, const void *const *w, float *const *out, const int *n, int count, int M, int K, void *ws,
                   size_t ws_bytes, cudaStream_t st);
int decode_ts_status();
int gather_columns(const void *x, const int64_t *idx, void *out, int elt, long long M, int K, cudaStream_t st);
int moe_gate_mul(const void *h, void *out, int dtype, long long M, int I, int gelu, cudaStream_t st);
int moe_combine(const void *pair_out, void *out, int dtype, long long tokens, int N, int topk, cudaStream_t st);
int moe_combine_weighted(const void *rows, const int64_t *index, const float *weights, float *out, int dtype, long long tokens, int N,
                         int topk, long long n_rows, cudaStream_t st);
int gemv_bf16_multi(const void *x, const void *const *w, void *const *out, const int *n, int count, int K, int out_f32, cudaStream_t st);
int gemv_bf16_gated(const void *x, const void *wg, const void *wu, void *y, int N, int K, int gelu, cudaStream_t st);
size_t chain_program_bytes(int n_ops);
long long chain_arena_bytes(const lb200_chain_op *ops, int n_ops, int n_vecs, int world);
int chain_build(const lb200_chain_op *ops, int n_ops, int n_vecs, void *program, size_t program_bytes, void *const *arena, size_t arena_bytes,
                int world, int rank, cudaStream_t st);
int chain_run(const void *program, unsigned int *step, cudaStream_t st);
int chain_status();
int moe_bad_ids_status();  // 0 / 1, or a CUDA error code (> 1)
int fp8_gemv_fast(const void *x, const uint8_t *w, const float *scale, void *y, int act_dtype, int M, int N, int K, int bR, int bC,
                  cudaStream_t st);
// one-row tensor-core decode kernel for canonical int4 weights: 1 = took the call, 0 = not covered, other = error
int int4_gemv_fast(const void *x, const uint32_t *codes, const float *s, const float *z, void *y, int act_dtype, int M, int N, int K,
                   int G, cudaStream_t st);
int quantize_rows_int8(const float *x, int8_t *q, float *scales, long long M, int K, cudaStream_t st);
int matmul_w8a8(const float *x, const int8_t *wq, const float *ws, float *out, int8_t *xq, float *xs, int M, int N, int K,
                cudaStream_t st);
int gguf_embedding(int type, const void *table, const int64_t *ids, float *out, long long n_ids, long long V, int K, cudaStream_t st);
int int4_repack(const uint32_t *qweight, const uint32_t *qzeros, const float *scales, uint32_t *codes, float *s_out, float *z_out,
                int N, int K, int G, int kind, cudaStream_t st);
int rmsnorm(const void *x, const void *residual, const void *weight, void *sum_out, void *out, int dtype, long long rows, int cols,
            float eps, cudaStream_t st);
int rope(const void *x, const int64_t *positions, void *out, int dtype, long long rows, int seq_len, int head_dim, double base,
         cudaStream_t st);

}  // namespace lb
