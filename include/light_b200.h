/*
 * light_b200.h -- C ABI of the B200 (sm_100a) quantized-weight matmul library.
 *
 * Every entry point replaces one CUDA launcher of the reference (sushvibez/light), i.e. one
 * key of its kernel registry (internal/registry/registry.go:12-62) on device kind CUDA.  The
 * contract is the reference launchers' contract:
 *
 *   - all pointers are DEVICE pointers into buffers the caller owns, output included; the
 *     library never allocates, frees or copies to the host on these paths;
 *   - work is enqueued on `stream` (0 = the legacy default stream) of device `device` and the
 *     call returns without synchronising, so calls can be captured into a CUDA graph;
 *   - the return value is 0 on success, a positive cudaError_t when the CUDA runtime refused
 *     something, or a negative LB200_E_* code when the arguments are rejected; shape
 *     violations are returned, never asserted; light_b200_last_error() gives the text;
 *   - tensors are contiguous, row-major, offset 0.
 *
 * Quantized GGUF weights are passed in their on-disk block layout, (N, K) row-major, a row
 * being K / block_elems consecutive blocks (reference gguf/reader.go:237-251, quant/q4_k.go:14-24,
 * quant/q6_k.go:11-32, quant/q8_0.go:11-17).
 */
#ifndef LIGHT_B200_H
#define LIGHT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LIGHT_B200_ABI_VERSION 1

#if defined(__GNUC__)
#define LB200_API __attribute__((visibility("default")))
#else
#define LB200_API
#endif

/* ggml on-disk type codes (reference gguf/types.go:39-58) of the formats with a fused kernel
 * (reference kernels/cuda/matmul_q.go:17-24). */
enum {
  LB200_Q4_0 = 2,
  LB200_Q5_0 = 6,
  LB200_Q8_0 = 8,
  LB200_Q4_K = 12,
  LB200_Q5_K = 13,
  LB200_Q6_K = 14
};

/* Activation / output element types. */
enum { LB200_F32 = 0, LB200_BF16 = 1, LB200_F16 = 2 };

/* Argument errors (negative so they cannot collide with cudaError_t). */
enum {
  LB200_E_DTYPE = -1,     /* unknown or unsupported element / block type            */
  LB200_E_SHAPE = -2,     /* a dimension is negative, zero where it may not be, or   */
                          /* not a multiple of what the layout needs                 */
  LB200_E_NULL = -3,      /* a required pointer is null                              */
  LB200_E_ALIGN = -4,     /* a pointer is less aligned than the layout guarantees    */
  LB200_E_DEVICE = -5,    /* no such device, or not an sm_100 device                 */
  LB200_E_TOO_LARGE = -6  /* beyond a documented maximum                             */
};

/* Binds the library to `device` (makes its primary context current on the calling thread,
 * checks the compute capability, sets kernel attributes).  Every other entry point does this
 * lazily, so calling it is optional; it mirrors cudart.SetDevice + module load in the
 * reference launchers (kernels/cuda/matmul_q.go:52-58, kernels/cuda/loader.go:99-196). */
LB200_API int light_b200_init(int device);

/* Copies the calling thread's last error text into buf (NUL terminated); returns its length.
 * Reference: the `cudart: <op>: <msg> (code N)` errors of internal/cudart/runtime.go:335-363. */
LB200_API int light_b200_last_error(char *buf, size_t n);

LB200_API int light_b200_abi_version(void);

/* Number of kernels this library has launched on any stream since load (monotonic). */
LB200_API unsigned long long light_b200_launch_count(void);

/* Hands the library a per-device workspace it may use between calls on that device (device
 * memory, 1024-byte aligned, owned by the caller, valid until replaced; ptr = NULL withdraws it).
 * The reference keeps the same kind of buffer, one reusable weight scratch per device
 * (ops/fp8_block.go:105-154 weightScratch).  Here it holds the f16 copy of the activations that the
 * tensor-core prefill path streams by TMA: matmul_q with M > 64 needs M * K * 2 bytes; without a
 * large enough workspace such calls run the slower shape-generic kernel.  Batched decode (matmul_q and
 * matmul_q_multi_rows with 2 <= M <= 64 on Q4_K / Q6_K) keeps there the activations staged as f16 fragment
 * records and the split-K partial sums of its persistent grid.  Calls that use the workspace must not overlap
 * on the GPU. */
LB200_API int light_b200_set_workspace(int device, void *ptr, size_t bytes);

/* The workspace size with which light_b200_matmul_q / _multi_rows (and the int4, block-FP8 and grouped matmuls, M
 * then the number of activation rows or routed pairs) take their fastest path for M rows of K: above 64 rows the f16
 * copy of x plus about 42 MB of partial tiles for the persistent tensor-core kernel; with less, those calls run the
 * kernel that needs the copy alone. */
LB200_API unsigned long long light_b200_matmul_q_workspace_bytes(int M, int K);

/* 0 if no bounded device-side wait of the tensor-core kernels ever gave up on this device, 1 if one
 * did (the affected call's output is then incomplete).  Synchronises with the device. */
LB200_API int light_b200_prefill_status(int device);

/* Block geometry: elements / bytes per block, 0 for an unknown type
 * (reference dtype/dtype.go:53-102 blockInfo, BlockElems, BlockBytes). */
LB200_API int light_b200_block_elems(int ggml_type);
LB200_API int light_b200_block_bytes(int ggml_type);

/* Registry key {matmul_q, CUDA, <w dtype>} (reference kernels/cuda/matmul_q.go:44-91,
 * ops/matmul_q.go:27-75):  out (M,N) f32 = x (M,K) f32 . dequant(w (N,K) blocks)^T.
 * K must be a multiple of the block size.  Any M >= 0 is taken (the reference routes M >= 8 to
 * dequantize + SGEMM; here one call covers decode and prefill). */
LB200_API int light_b200_matmul_q(int ggml_type, const float *x, const void *w, float *out, int M, int N, int K, int device,
                        void *stream);

/* light_b200_matmul_q_multi for a small batch: x f32 (M, K) against up to four quantized matrices of one type
 * that share it, out[i] (M, n[i]) dense.  2 <= M <= 32 and Q4_K run as ONE launch (the token-column decode
 * kernels over the joint tile list of the matrices); other row counts and types run one launch per matrix, so
 * the call is always valid where light_b200_matmul_q is. */
LB200_API int light_b200_matmul_q_multi_rows(int ggml_type, const float *x, const void *const *w, float *const *out,
                                             const int32_t *n, int count, int M, int K, int device, void *stream);

/* Decode-time fused launches over quantized weights, the quantized twins of the reference's
 * ops.LinearMulti / registry key gemv_multi (ops/gemv.go:21-78, kernels/cuda/gemv.go:15-94) and
 * ops.GatedLinear / gemv_gated (ops/gemv.go:80-140), which the reference applies to the q/k/v trio
 * and to gate/up (models/llama.go:1085,1300; gate models/fused_linear.go:16-47) but only for BF16
 * weights.  x is ONE f32 activation row (K).
 *
 * matmul_q_multi:  out[i] (n[i]) f32 = x . dequant(w[i] (n[i],K))^T for i < count <= 4, all w of one
 *   ggml type; one launch when a fused kernel applies, else one matmul per matrix.
 * matmul_q_gated:  out (N) f32 = act(x . dequant(wg)^T) * (x . dequant(wu)^T), act 1 = SiLU,
 *   2 = GELU (erf), the two products held in f32.  Needs the fused kernel (Q4_K, K a multiple of
 *   256, N >= 16, 16-byte aligned weights); otherwise LB200_E_SHAPE / LB200_E_DTYPE and the caller
 *   keeps its unfused sequence, as the reference does when gemv_gated does not apply. */
LB200_API int light_b200_matmul_q_multi(int ggml_type, const float *x, const void *const *w, float *const *out,
                                        const int32_t *n, int count, int K, int device, void *stream);
LB200_API int light_b200_matmul_q_gated(int ggml_type, const float *x, const void *wg, const void *wu, float *out, int N,
                                        int K, int act, int device, void *stream);

/* Registry keys {gemv_multi, CUDA, BF16} and {gemv_gated, CUDA, BF16} (reference kernels/cuda/gemv.go:15-94;
 * ops.LinearMulti / ops.GatedLinear, ops/gemv.go:21-140): the same two fused launches for UNQUANTIZED bf16 weights.
 * x is one bf16 activation row (K), every w[i] (n[i], K) bf16 row-major.
 *   gemv_multi: out[i] (n[i]) = x . w[i]^T for i < count <= 4, f32 sums rounded once to bf16, or stored as f32
 *     when out_f32 != 0.
 *   gemv_gated: out (N) bf16 = act(x . wg^T) * (x . wu^T), act SiLU (gelu = 0) or GELU-erf, with both products and
 *     the activation rounded to bf16 first, as the unfused sequence leaves them.
 * K % 8 == 0 and K <= 16384 (the reference: 12288); pointers 16-byte aligned. */
LB200_API int light_b200_gemv_multi(const void *x, const void *const *w, void *const *out, const int32_t *n, int count, int K,
                                    int out_f32, int device, void *stream);
LB200_API int light_b200_gemv_gated(const void *x, const void *wg, const void *wu, void *out, int N, int K, int gelu, int device,
                                    void *stream);

/* The CUDA dequantize hook, quant.RegisterCUDADequant (reference quant/cuda_hook.go:13-46,
 * kernels/cuda/dequant.go:15-75):  dst f32 [n_elems] = dequant(src blocks).  n_elems must be a
 * whole number of blocks.  Bit-identical to the reference's CPU decoders. */
LB200_API int light_b200_dequant(int ggml_type, const void *src, float *dst, int64_t n_elems, int device, void *stream);

/* Registry key {int4_dequant, CUDA, F32|BF16} (reference kernels/cuda/int4.go:43-69):
 * canonical 4-bit layout (reference quant/int4.go:12-31) codes u32 (N,K/8), scales and zeros
 * f32 (N,K/G) -> out (N,K) at out_dtype, written `offset` ELEMENTS into `out`;
 * W = s * (code - z) formed in f32 and rounded once.  G % 8 == 0. */
LB200_API int light_b200_int4_dequant(const uint32_t *codes, const float *scales, const float *zeros, void *out, int out_dtype,
                            int N, int K, int group, int64_t offset, int device, void *stream);

/* Registry key {int4_gemv, CUDA, F32|BF16} (reference kernels/cuda/int4.go:76-101):
 * y (M,N) at act_dtype = x (M,K) at act_dtype . W^T.  K % 32 == 0, G % 32 == 0.  The reference
 * kernel stops at M = 8 (ops/int4.go:58-59); this one takes any M >= 0. */
LB200_API int light_b200_int4_gemv(const void *x, const uint32_t *codes, const float *scales, const float *zeros, void *y,
                         int act_dtype, int M, int N, int K, int group, int device, void *stream);

/* out (M, K) = x[:, idx]: the activation-column gather in front of an act-order GPTQ weight (reference ops/int4.go:129-147
 * gatherColumns, three tensor ops there).  idx (K) device I64, a permutation of 0..K-1 (an index outside yields 0);
 * dtype LB200_F32 / BF16 / F16. */
LB200_API int light_b200_gather_columns(const void *x, const int64_t *idx, void *out, int dtype, int64_t M, int K, int device,
                                        void *stream);

/* Registry key {fp8_block_dequant, CUDA, F32|BF16} (reference kernels/cuda/fp8_block.go:44-69):
 * w e4m3fn codes (R,C), scale f32 (R/bR, C/bC) -> out (R,C) = f32(w) * scale, rounded once.
 * C % 4 == 0, bC % 4 == 0, R % bR == 0, C % bC == 0. */
LB200_API int light_b200_fp8_block_dequant(const uint8_t *w, const float *scale, void *out, int out_dtype, int R, int C,
                                 int block_r, int block_c, int device, void *stream);

/* Registry key {fp8_block_gemv, CUDA, F32|BF16} (reference kernels/cuda/fp8_block.go:76-105):
 * y (M,N) = x (M,K) . (w * scale)^T.  K % 16 == 0, bC % 16 == 0.  Any M >= 0 (reference: M <= 8). */
LB200_API int light_b200_fp8_block_gemv(const void *x, const uint8_t *w, const float *scale, void *y, int act_dtype, int M, int N,
                              int K, int block_r, int block_c, int device, void *stream);

/* Arguments of the grouped expert matmuls.  Mirrors the Inputs / Attrs of the reference
 * launchers (kernels/cuda/moe.go:21-141; kernel contract kernels/cuda/src/moe.cu:1-24):
 *
 *   out[p, :] = w(p) * input[row(p), :] . weights[e, :, :]^T   for each sorted pair
 *
 * sorted_pairs[i] is the pair id p = token * topk + slot of the i-th pair in expert order and
 * expert_ids[i] its expert (non-decreasing); row(p) = p when row_per_pair, else p / topk;
 * w(p) = topk_weights[p], or 1 when topk_weights is null.  counts (E) and offsets (E+1) are
 * int32 SCRATCH the caller provides; the call fills them (offsets = exclusive prefix sum of the
 * per-expert pair counts) and they are valid outputs afterwards.  Rows of `out` whose pair id
 * does not appear (or is outside [0, size_m)) are left untouched.  An expert id outside [0, E) never
 * indexes anything: a negative id owns no range, an id >= E lies at or beyond offsets[E] (which then is the
 * index of the first such pair instead of M); their pairs are skipped, and light_b200_moe_route_status reports it. */
typedef struct lb200_moe_args {
  const void *input;          /* (rows, K) at dtype (moe_gemm) or f32 (moe_gemm_q)          */
  const void *weights;        /* (E, N, K) at dtype, or GGUF blocks of ggml_type            */
  const int64_t *sorted_pairs; /* (M)                                                        */
  const int64_t *expert_ids;  /* (M)                                                        */
  int32_t *counts;            /* (E) scratch                                                */
  int32_t *offsets;           /* (E+1) scratch                                              */
  const float *topk_weights;  /* (size_m) or null                                           */
  void *out;                  /* (size_m, N) at dtype, or f32 (moe_gemm_q)                  */
  int64_t M;                  /* number of sorted pairs                                     */
  int64_t size_m;             /* rows of out                                                */
  int32_t E, N, K;
  int32_t topk;
  int32_t row_per_pair;
  int32_t dtype;              /* LB200_F32 / BF16 / F16 (moe_gemm); ggml type (moe_gemm_q)  */
} lb200_moe_args;

/* Registry key {moe_gemm, CUDA, F32|BF16|F16} (reference kernels/cuda/moe.go:21-97). */
LB200_API int light_b200_moe_gemm(const lb200_moe_args *args, int device, void *stream);

/* Grouped matmul over block-scaled FP8 experts: weights = e4m3fn codes (E, N, K), w_scale f32
 * (E, N / block_r, K / block_c); args->dtype = activation and output type (LB200_F32 or LB200_BF16);
 * everything else as light_b200_moe_gemm.  The reference has no grouped kernel for FP8 experts: its
 * models loop over experts on the host, one ops.MatMulF8Block per expert plus gather / scatter
 * (models/moe_routed.go:34-79); this entry point is that loop as one launch.  With M >= 256 pairs, K % 128 == 0,
 * block_c % 64 == 0 and a workspace of M * K * 2 bytes (light_b200_set_workspace) the tensor-core path runs;
 * otherwise (a decode step's few pairs) one warp per output column and tile of sorted pairs, which needs only
 * block_c % 8 == 0 and blocks that tile the weight. */
LB200_API int light_b200_moe_gemm_f8block(const lb200_moe_args *args, const float *w_scale, int block_r, int block_c,
                                          int device, void *stream);

/* ---- multi-GPU: all-gather of row-split outputs over NVLink peer memory (no counterpart in the
 * reference, which is single-GPU: STATUS.md:474).  Each rank r of `world` (<= LB200_MAX_PEERS) GPUs of one
 * node owns rows [r N/P, (r+1) N/P) of a weight and so produces an (M, N/P) column block of the output.
 * slots[p] is rank p's receive buffer for THIS gathered operator: 2 * M * N slots of 8 bytes ({f32, u32 tag};
 * two sets, used on alternating steps), 8-byte aligned, in memory every rank can address (peer-mapped / symmetric memory; the caller sets that
 * up), zeroed once. */
#define LB200_MAX_PEERS 8
typedef struct lb200_peers {
  void *slots[LB200_MAX_PEERS];
  int32_t world, rank;
} lb200_peers;

/* Once per step (one pass over the model), before its first gather: bumps the step word (device memory of
 * this rank, zeroed once) that tags everything sent during the step. */
LB200_API int light_b200_comm_step_begin(uint32_t *step, int device, void *stream);

/* Writes `local` (M, n_local) f32, tagged with the step, into its slots in every peer's receive buffer and
 * into columns [rank * n_local, (rank + 1) * n_local) of `out` (M, n_local * world, this rank's own memory);
 * then fills the other columns of `out` from this rank's receive buffer as the peers' elements of the same
 * step arrive.  A slot that does not arrive within about 50 ms is given up (status: light_b200_comm_status).
 * Every rank must issue the same sequence of gathers each step, each operator with its own slots. */
LB200_API int light_b200_allgather_ll(const float *local, float *out, const lb200_peers *peers, int M, int n_local,
                                      const uint32_t *step, int device, void *stream);

/* Row-split decode matmul with the exchange INSIDE the launch (one activation row; Q4_K: up to four
 * matrices that share it, Q6_K: one).  Rank `rank` of `world` holds rows [rank n[i], (rank + 1) n[i]) of
 * output i.  For an output the next operator needs in full, out_slots[i][p] is rank p's receive buffer for it
 * (2 * world * n[i] slots of 8 bytes, two step parities, peer-addressable, zeroed once): the launch's epilogue
 * stores every value it owns there as {f32, step tag}, on every rank.  out_slots[i][*] all NULL keeps output
 * i local (out[i], n[i] f32, is written in either case).  The activations come either as plain f32 (x, K
 * values; x_slots NULL) or as this rank's receive buffer of the launch that produced them (x_slots, 2 * K
 * slots; x ignored): the kernel polls the slots until they carry the step's tag (about 50 ms at most, then
 * light_b200_comm_status reports it), so no gather launch stands between two matmuls.  `step` as for
 * light_b200_allgather_ll.  Fails with LB200_E_SHAPE when no single-launch kernel covers the shape. */
typedef struct lb200_tp {
  const void *x_slots;
  void *out_slots[4][LB200_MAX_PEERS];
  const uint32_t *step;
  int32_t world, rank;
} lb200_tp;
LB200_API int light_b200_matmul_q_tp(int ggml_type, const float *x, const void *const *w, float *const *out,
                                     const int32_t *n, int count, int K, const lb200_tp *tp, int device, void *stream);

/* 0, or 1 if a bounded wait on a peer ever gave up on this device.  Synchronises with the device. */
LB200_API int light_b200_comm_status(int device);

/* Largest expert count light_b200_moe_gemm_static_scratch accepts. */
#define LB200_MOE_STATIC_MAX_EXPERTS 1024

/* light_b200_moe_gemm for callers that cannot hand over scratch memory.  (No counterpart in the
 * reference: its launcher always receives counts / offsets tensors from the Go tensor pool.)
 *
 * Some callers of a C ABI have nothing to allocate with at the call site: a thin FFI stub that
 * only forwards the pointers it was given, a serving loop that has handed all device memory to
 * its own pool, or code that must not call cudaMalloc because it can synchronise the device and
 * can fail late.  For them this variant keeps the per-expert counts and offsets in a fixed device
 * array inside the library (8 KiB + 8 B per GPU that loads the library, held until the process
 * exits); args->counts and args->offsets are ignored and may be null.  Everything else -- inputs,
 * weights, routing, output -- is still the caller's memory, and the result is the same as
 * light_b200_moe_gemm's.  It calls no cudaMalloc / cudaFree and no allocating library routine.
 *
 *   - args->E must not exceed LB200_MOE_STATIC_MAX_EXPERTS, else LB200_E_TOO_LARGE.
 *   - The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
 *     that device current); make that first call before any stream capture begins.
 *   - Every call on a device shares the one array, which keeps the previous call's contents.
 *     Each call overwrites all E counts and E + 1 offsets before reading them, so nothing has to
 *     be cleared -- but two calls that overlap on the GPU (different streams, or graphs replayed
 *     concurrently) race on it.  Serialise them, or use light_b200_moe_gemm with own scratch. */
LB200_API int light_b200_moe_gemm_static_scratch(const lb200_moe_args *args, int device, void *stream);

/* Registry key {moe_gemm_q, CUDA, <w dtype>} (reference kernels/cuda/moe.go:99-141):
 * x f32, GGUF block-quantized experts, out f32. */
LB200_API int light_b200_moe_gemm_q(const lb200_moe_args *args, int device, void *stream);

/* ---- decode-step attention against a fixed-capacity KV cache (the step beside the quantized matmuls)
 *
 * Registry keys {kv_append, CUDA, F32|BF16}, {decode_attn, CUDA, F32|BF16}, {inc_i64, CUDA, I64}
 * (reference kernels/cuda/decode_attn.go:15-133; ops.KVAppend / ops.DecodeAttention / ops.IncrementI64,
 * ops/decode_attn.go:13-205).  `pos` is a one-element device I64: the position of the new token, so the
 * number of valid keys is pos + 1 and every launch is the same whatever the position (CUDA-graph
 * capturable, models/decode_graph.go:27-230).  With a position outside [0, Cap) nothing is appended (neither
 * by light_b200_kv_append nor by the append inside light_b200_decode_attn), the attention runs over the cached
 * rows of the clamped range, and light_b200_decode_attn_status reports it. */

/* k, v (B, KH, 1, D) contiguous -> kbuf, vbuf (B, KH, Cap, D) at position pos[0]. */
LB200_API int light_b200_kv_append(const void *k, const void *v, void *kbuf, void *vbuf, const int64_t *pos, int dtype,
                                   int B, int KH, int D, int Cap, int device, void *stream);

typedef struct lb200_decode_attn_args {
  const void *q;       /* (B, NH, 1, D) contiguous                                              */
  void *kbuf, *vbuf;   /* (B, KH, Cap, D) contiguous                                            */
  const void *k_new;   /* NULL, or k (B, KH, 1, D): appended at pos by this launch, which then   */
  const void *v_new;   /* replaces light_b200_kv_append (KVCache.decodeAttend does both)         */
  const int64_t *pos;  /* device, one element                                                    */
  void *out;           /* (B, NH, 1, D)                                                          */
  int32_t dtype;       /* LB200_F32 or LB200_BF16: q, k, v, out alike                            */
  int32_t B, NH, KH, Cap, D;
  int32_t window;      /* 0, or the sliding window: keys [n - window, n)                         */
  float scale;         /* scores = scale * q.k                                                   */
  float rope_base;     /* 0, or the rotary base (ops.RoPE, ops/rope.go:30-77): q and k_new are      */
                       /* rotated at position pos inside the launch (rotate-half pairing), the    */
                       /* key is cached rotated; without k_new only q is rotated                  */
} lb200_decode_attn_args;

/* out = softmax(scale * q K^T) V over the valid keys, one launch, no scratch.  Limits as the reference's
 * kernel (D a multiple of 32 up to 512, at most 16 query heads per KV head; else LB200_E_SHAPE and the
 * caller composes the op as it does today, ops/decode_attn.go:116-170). */
LB200_API int light_b200_decode_attn(const lb200_decode_attn_args *args, int device, void *stream);

/* Quantized embedding lookup (reference nn.Embedding over a quantized table: ops.IndexSelect of the byte
 * rows + quant.Dequantize of the gathered rows, nn/embedding.go; nn/embedding_test.go:127): out row i =
 * dequantized row ids[i] of the (V, K) table, bit-identical to light_b200_dequant of that row.  ids are
 * device I64; an id outside [0, V) yields a row of zeros. */
LB200_API int light_b200_embedding_q(int ggml_type, const void *table, const int64_t *ids, float *out, int64_t n_ids, int64_t V,
                                     int K, int device, void *stream);

/* Checkpoint tensors -> the canonical 4-bit layout, on the device (reference quant.FromGPTQ / quant.FromAWQ,
 * quant/int4.go:103-261, host loops at load time).  layout 0: AutoGPTQ "gptq" -- qweight i32 (K/8, N) packed
 * along K, qzeros i32 (K/G, N/8) packed along N holding zero - 1; 1: "gptq_v2" (qzeros hold the zero);
 * 2: AutoAWQ GEMM -- qweight (K, N/8) and qzeros packed along N in the order (0,2,4,6,1,3,5,7).  scales f32
 * (K/G, N) (cast by the caller).  Out: codes u32 (N, K/8), scales / zeros f32 (N, K/G).  Ordered groups only:
 * an act-order GPTQ checkpoint (g_idx) keeps the host path, which also builds the column permutation. */
LB200_API int light_b200_int4_repack(const void *qweight, const void *qzeros, const float *scales, void *codes, float *scales_out,
                                     float *zeros_out, int N, int K, int group, int layout, int device, void *stream);

/* Device-side routing.  The reference routes DeepSeek-style models on the host (models/deepseek_route.go:27-133)
 * and sorts pairs with TopK + Sort + count + scan launches (ops/moe.go:24-99, kernels/cuda/src/moe.cu:28-42).
 *
 * moe_route_sigmoid: router logits (T, E) and an optional per-expert bias (E) -> ids (T, topk) I64 and weights
 * (T, topk) F32: scores = sigmoid(logit) in f64, choice = score + bias, stable descending top-k of the
 * choices (ties: the lower expert id), weights = the unbiased scores, divided by (their sum + 1e-20) when
 * norm_topk.  E <= 1024, topk <= 32.
 *
 * moe_sort_pairs: ids (M) I64 -> counts i32 (E), offsets i32 (E + 1), sorted_pairs / sorted_expts I64 (M): pair
 * ids in expert order, pairs of one expert ascending (ops.MoERouteFromIDs, ops/moe.go:73-99, plus the
 * counts / offsets that light_b200_moe_gemm* otherwise compute).  scratch: M + ceil(M / 1024) * E int32.  An id
 * outside [0, E) is treated as expert 0 and reported by light_b200_moe_route_status (synchronises; the same
 * word reports ids outside [0, E) seen by the grouped matmuls' offsets kernel).  The first call on a device
 * must not be inside stream capture. */
LB200_API int light_b200_moe_route_sigmoid(const float *logits, const float *bias, int64_t *ids, float *weights, int T, int E,
                                           int topk, int norm_topk, int device, void *stream);
LB200_API int light_b200_moe_sort_pairs(const int64_t *ids, int32_t *counts, int32_t *offsets, int64_t *sorted_pairs,
                                        int64_t *sorted_expts, int32_t *scratch, int64_t M, int E, int device, void *stream);
LB200_API int light_b200_moe_route_status(int device);

/* moe_route_deepseek: every branch of the reference's host router (models/deepseek_route.go:30-133): sigmoid != 0: scores =
 * sigmoid(logit), choice = score + bias (bias may be NULL); else scores = choice = softmax(logits) (bias ignored).  With
 * n_group > 1 and topk_group < n_group only the topk_group best groups of E / n_group experts stay eligible (group score:
 * the sum of its two best choices for the sigmoid router, its best for the softmax router).  Weights are the scores of the
 * chosen experts, divided by (their sum + 1e-20) when sigmoid and norm_topk.  E <= 1024, topk <= 32, n_group <= 32,
 * E % n_group == 0.
 *
 * moe_route_topk: the selection of ops.MoERoute (ops/moe.go:29-50): probs (T, E) F32 (after the softmax) -> the topk
 * largest per token (ties: the lower expert id), their values as weights, divided by their sum when normalize.
 * light_b200_moe_sort_pairs then gives the expert-sorted pairs. */
LB200_API int light_b200_moe_route_deepseek(const float *logits, const float *bias, int64_t *ids, float *weights, int T, int E,
                                            int topk, int n_group, int topk_group, int sigmoid, int norm_topk, int device,
                                            void *stream);
LB200_API int light_b200_moe_route_topk(const float *probs, int64_t *ids, float *weights, int T, int E, int topk, int normalize,
                                        int device, void *stream);

/* The element-wise steps of a sparse MoE block around the two grouped matmuls, each as one launch with the roundings of
 * the reference's unfused sequence (nn/moe.go:206-236: Narrow gate / up -> SiLU -> Mul; ops.MoECombine, ops/moe.go:206-240).
 *   moe_gate_mul: h (M, 2 I), gate = h[:, :I], up = h[:, I:] -> out (M, I) = act(gate) * up, act SiLU (gelu = 0) or GELU-erf,
 *     the activation rounded to the element type before the product.  I % 8 == 0.
 *   moe_combine: pair_out (tokens * topk, N) -> out (tokens, N): the topk slot rows of a token added one after the other,
 *     slot 0 first, every sum rounded to the element type (routing weights were applied by the grouped matmul).  N % 8 == 0.
 * dtype LB200_F32 / BF16 / F16; pointers 16-byte aligned. */
LB200_API int light_b200_moe_gate_mul(const void *h, void *out, int dtype, int64_t M, int I, int gelu, int device, void *stream);
LB200_API int light_b200_moe_combine(const void *pair_out, void *out, int dtype, int64_t tokens, int N, int topk, int device,
                                     void *stream);
/* The combine of a block whose expert rows arrive in another order and unweighted (experts sharded over GPUs: the rows
 * come back from the experts' ranks in expert order; the reference has one GPU and no such step, the arithmetic is
 * MoEGemm's weighted epilogue followed by MoECombine, ops/moe.go:121-240, kept in f32):
 *   out f32 (tokens, N)[t] = sum over slots s, slot 0 first, of weights[t * topk + s] * rows[index[t * topk + s]]
 * rows (n_rows, N) at dtype; index int64 per pair (NULL: pair p is row p; a value outside [0, n_rows) drops the pair);
 * weights f32 per pair (NULL: 1).  N % 8 == 0; rows and out 16-byte aligned. */
LB200_API int light_b200_moe_combine_weighted(const void *rows, const int64_t *index, const float *weights, float *out, int dtype,
                                              int64_t tokens, int N, int topk, int64_t n_rows, int device, void *stream);

/* INT8 weights x INT8 activations.  Registry key {matmul_w8a8, CUDA, F32} (reference ops.MatMulW8A8,
 * ops/matmul_w8a8.go:13-120): x f32 (M, K), wq int8 (N, K), ws f32 (N) -> out f32 (M, N).  The activation
 * rows are quantised on the device exactly as QuantizeRowsInt8 does (scale = amax / 127, round half to even,
 * clamp to +-127), the contraction accumulates in int32 on the integer tensor cores, and the epilogue is
 * f32(acc) * xs[m] * ws[n]: bit-identical to the reference's Go path.  xq_scratch (M * K bytes, 16-byte
 * aligned) and xs_scratch (M floats) are the caller's, like every other scratch of this ABI.  K % 16 == 0. */
LB200_API int light_b200_quantize_rows_int8(const float *x, int8_t *q, float *scales, int64_t M, int K, int device, void *stream);
LB200_API int light_b200_matmul_w8a8(const float *x, const int8_t *wq, const float *ws, float *out, int8_t *xq_scratch,
                                     float *xs_scratch, int M, int N, int K, int device, void *stream);

/* RMSNorm (and the residual add before it) folded into the Q4_K decode launch that consumes it:
 * light_b200_rmsnorm + light_b200_matmul_q_multi (act 0: count matrices, out[i] = w[i] . y) or
 * + light_b200_matmul_q_gated (act 1 SiLU / 2 GELU: count 2, out[0] = act(w[0] . y) * (w[1] . y)) as ONE
 * launch, y = s * rsqrt(mean(s^2) + eps) * weight, s = x + residual (residual NULL: s = x).  A decoder
 * layer does exactly this twice (models/llama.go:1085-1110,1290-1326: Add, RMSNorm, then the q,k,v or
 * gate,up projections); a dependent launch costs about 5 us whatever its size, so the two small
 * operators are worth more as a prologue than as launches.  One f32 activation row, Q4_K weights,
 * K a multiple of 256 that fits the kernel's activation staging; else LB200_E_SHAPE / LB200_E_DTYPE and
 * the caller keeps its unfused sequence.  sum_out (required with a residual) receives s; it must not
 * alias x or residual, because other thread blocks of the launch still read them. */
typedef struct lb200_norm {
  const float *weight;   /* (K)                                   */
  const float *residual; /* (K) or NULL                           */
  float *sum_out;        /* (K); NULL when residual is NULL       */
  float eps;
} lb200_norm;
LB200_API int light_b200_matmul_q_fused(int ggml_type, const float *x, const lb200_norm *norm, const void *const *w,
                                        float *const *out, const int32_t *n, int count, int act, int K, int device,
                                        void *stream);

/* Registry key {rmsnorm, CUDA, F32|BF16} (reference ops.RMSNorm, ops/norm.go:69-111; kernels
 * rmsnorm_f32 / rmsnorm_bf16, kernels/cuda/src/elementwise.cu:275-312): out = s * rsqrt(mean(s^2) + eps) *
 * weight along the last axis, x (rows, cols), weight (cols).  With residual == NULL, s = x.  With a
 * residual, s = x + residual is also written to sum_out (the ops.Add that precedes the norm in every
 * decoder layer, models/llama.go, folded into the same launch); sum_out may alias x or residual. */
LB200_API int light_b200_rmsnorm(const void *x, const void *residual, const void *weight, void *sum_out, void *out, int dtype,
                                 int64_t rows, int cols, float eps, int device, void *stream);

/* Registry key {rope, CUDA, F32|BF16} (reference ops.RoPE, ops/rope.go:30-77; rope_f32,
 * kernels/cuda/src/elementwise.cu:748-774): x (rows, head_dim) with rows = batch * seq_len, positions
 * (seq_len) I64 on the device; dim i pairs with dim i + head_dim / 2 at angle pos * base^(-2 i / head_dim),
 * computed in f64 like the reference's CPU kernel (kernels/cpu/misc_registry.go:27-62). */
LB200_API int light_b200_rope(const void *x, const int64_t *positions, void *out, int dtype, int64_t rows, int seq_len,
                              int head_dim, double base, int device, void *stream);

/* Registry key {argmax, CUDA, F32}, last axis (reference ops.Argmax, ops/argmax.go:14-60; kernels/cuda/topk.go:56-90):
 * out[r] = index of the largest element of row r of x (rows, cols), the lowest index among equals.  With the
 * logits as x this is greedy sampling on the device: the token id never visits the host inside a decode graph
 * (engine/engine.go:419-565 samples on the device for the same reason). */
LB200_API int light_b200_argmax(const float *x, int64_t *out, int64_t rows, int cols, int device, void *stream);

/* p[i] += 1 for i < n (the device-side position after a step). */
LB200_API int light_b200_inc_i64(int64_t *p, int n, int device, void *stream);

/* 0, or 1 if a launch ever saw a position outside [0, Cap).  Synchronises with the device. */
LB200_API int light_b200_decode_attn_status(int device);

/* ---- a decode step's dependent matrix-vector products as ONE launch
 *
 * The reference replays a decode step as a CUDA graph with one kernel per operator (models/decode_graph.go:58-205,
 * built from models/llama.go:1070-1330: per layer RMSNorm, q/k/v, attention, o, RMSNorm, gate/up, down; then the
 * final norm and lm_head).  For one activation row every one of those launches waits for the one before it and
 * streams only a few MB, so the step is bound by launch boundaries.  A chain is a PROGRAM of such operators
 * executed by one persistent launch (one thread block per SM): an operator's outputs reach the operators that
 * consume them through "chain vectors" -- buffers of 8-byte {f32, tag} slots in an arena the caller provides --
 * with no barrier and no launch in between, while the weights of the following operators are already being
 * fetched.  One f32 activation row; Q4_K and Q6_K weights.
 *
 * lb200_chain_op: out[i] (n[i]) = dequant(w[i] (n[i], K)) . y for i < count (Q4_K: up to four matrices of one
 *   launch, Q6_K: one), or with act 1 (SiLU) / 2 (GELU-erf) and count == 2: out[0] = act(w[0] . y) * (w[1] . y).
 *   y = the activations: plain f32 `x` (K values written before the call) or chain vector x_vec (written by an
 *   earlier operator of the program).  With norm_weight: y = s * rsqrt(mean(s^2) + norm_eps) * norm_weight,
 *   s = activations + chain vector res_vec (res_vec < 0: s = activations), and s is written to chain vector
 *   sum_vec when sum_vec >= 0 (the new residual stream) -- light_b200_matmul_q_fused's arithmetic; K <= 4096.
 *   Output i goes to plain memory out[i] when that is not NULL and to chain vector out_vec[i] when that is
 *   >= 0.  A vector may be rewritten by a later operator (the layers of a model reuse their vectors), as long
 *   as at least one other operator of the chain lies between its last reader and the writer.
 *   Row-split over `world` GPUs: n[i] are the rows this rank holds, rank r's values fill positions
 *   [r n[i], (r + 1) n[i]) of the vector on EVERY rank (stores into the peers' arenas), and a consumer's K is
 *   world * n[i].  K must be a multiple of 256 (Q6_K: of 2048), n[i] >= 16, weights 16-byte aligned.
 *
 * light_b200_chain_build validates the program and writes its device form into `program`
 *   (light_b200_chain_program_bytes(n_ops) bytes of device memory, 256-byte aligned) and zeroes this rank's
 *   arena (light_b200_chain_arena_bytes bytes, 256-byte aligned; arena[p] = rank p's arena, peer-addressable
 *   when world > 1, the same layout on every rank).  Do it once, outside stream capture.
 * light_b200_chain_run enqueues one pass over the program: `step` (a device word, zeroed once) is bumped and
 *   tags everything the pass writes.  Graph-capturable; allocates nothing; two launches.  Every wait inside
 *   the kernel is bounded (about 200 ms without progress), after which light_b200_chain_status reports 1 and
 *   the pass's outputs are not valid.  Passes over programs that share an arena must not overlap on the GPU,
 *   and the GPU must be able to hold one thread block of the kernel on every SM at once (nothing else may
 *   occupy it for longer than a launch). */
typedef struct lb200_chain_op {
  int32_t wtype;            /* LB200_Q4_K or LB200_Q6_K                                   */
  int32_t K;
  int32_t count;            /* matrices that share the activations: 1..4 (Q6_K: 1)        */
  int32_t act;              /* 0, or 1 SiLU / 2 GELU gate (count == 2, result in out[0])  */
  const void *w[4];         /* (n[i], K) blocks                                           */
  int32_t n[4];
  float *out[4];            /* plain f32 (n[i]) or NULL                                   */
  int32_t out_vec[4];       /* chain vector or -1                                         */
  const float *x;           /* plain activations (K), or NULL: x_vec                      */
  int32_t x_vec;
  int32_t res_vec;          /* -1, or the vector added to the activations before the norm */
  int32_t sum_vec;          /* -1, or the vector that receives activations + residual     */
  const float *norm_weight; /* (K) or NULL: no norm                                       */
  float norm_eps;
} lb200_chain_op;
LB200_API size_t light_b200_chain_program_bytes(int n_ops);
LB200_API int64_t light_b200_chain_arena_bytes(const lb200_chain_op *ops, int n_ops, int n_vecs, int world);
LB200_API int light_b200_chain_build(const lb200_chain_op *ops, int n_ops, int n_vecs, void *program, size_t program_bytes,
                                     void *const *arena, size_t arena_bytes, int world, int rank, int device, void *stream);
LB200_API int light_b200_chain_run(const void *program, uint32_t *step, int device, void *stream);
LB200_API int light_b200_chain_status(int device);

#ifdef __cplusplus
}
#endif
#endif /* LIGHT_B200_H */
