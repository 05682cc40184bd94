// extern "C" entry points: argument checks, device binding, dispatch.  No kernel lives here.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace lb {

static thread_local char g_err[512];
static std::atomic<unsigned long long> g_launches{0};

int fail(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  int n = vsnprintf(g_err, sizeof(g_err) - 32, fmt, ap);
  va_end(ap);
  if (n < 0) n = 0;
  if ((size_t)n > sizeof(g_err) - 32) n = sizeof(g_err) - 32;
  snprintf(g_err + n, 32, " (code %d)", code);
  return code;
}

int launched(const char *what) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail((int)e, "light_b200: %s: %s", what, cudaGetErrorString(e));
  return 0;
}

static std::mutex g_mu;
static bool g_ready[64];

int sm_count() {
  static std::atomic<int> sms[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  int v = sms[dev].load(std::memory_order_relaxed);
  if (v > 0) return v;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) return 148;
  sms[dev].store(v, std::memory_order_relaxed);
  return v;
}

static int bind(int device) {
  if (device < 0 || device >= 64) return fail(LB200_E_DEVICE, "light_b200: device ordinal %d out of range", device);
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) return fail((int)e, "light_b200: cudaSetDevice(%d): %s", device, cudaGetErrorString(e));
  if (g_ready[device]) return 0;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_ready[device]) return 0;
  int major = 0;
  e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
  if (e != cudaSuccess) return fail((int)e, "light_b200: device %d: %s", device, cudaGetErrorString(e));
  if (major != 10)
    return fail(LB200_E_DEVICE, "light_b200: device %d has compute capability %d.x; this library holds sm_100a code only",
                device, major);
  int rc = gguf_gemv_fast_init(device);
  if (rc) return rc;
  g_ready[device] = true;
  return 0;
}

static bool aligned(const void *p, size_t a) { return ((uintptr_t)p & (a - 1)) == 0; }

}  // namespace lb

using namespace lb;

#define REQUIRE_PTR(p, op) \
  if (!(p)) return fail(LB200_E_NULL, "light_b200: " op ": null pointer for " #p)

extern "C" {

int light_b200_init(int device) { return bind(device); }

int light_b200_last_error(char *buf, size_t n) {
  size_t len = strlen(g_err);
  if (buf && n) {
    size_t c = len < n - 1 ? len : n - 1;
    memcpy(buf, g_err, c);
    buf[c] = 0;
  }
  return (int)len;
}

int light_b200_abi_version(void) { return LIGHT_B200_ABI_VERSION; }

int light_b200_set_workspace(int device, void *ptr, size_t bytes) {
  if (int rc = bind(device)) return rc;
  return set_workspace(device, ptr, bytes);
}

int light_b200_comm_step_begin(uint32_t *step, int device, void *stream) {
  REQUIRE_PTR(step, "comm_step_begin");
  if (int rc = bind(device)) return rc;
  return comm_step_begin(step, (cudaStream_t)stream);
}

int light_b200_allgather_ll(const float *local, float *out, const lb200_peers *peers, int M, int n_local, const uint32_t *step,
                            int device, void *stream) {
  REQUIRE_PTR(local, "allgather_ll");
  REQUIRE_PTR(out, "allgather_ll");
  REQUIRE_PTR(peers, "allgather_ll");
  REQUIRE_PTR(step, "allgather_ll");
  if (peers->world < 1 || peers->world > LB200_MAX_PEERS || peers->rank < 0 || peers->rank >= peers->world)
    return fail(LB200_E_SHAPE, "light_b200: allgather_ll: rank %d of %d (at most %d peers)", peers->rank, peers->world,
                LB200_MAX_PEERS);
  if (M < 1 || n_local < 1 || (long long)M * n_local * peers->world > 0x7fffffffLL)
    return fail(LB200_E_SHAPE, "light_b200: allgather_ll: bad shape M=%d n_local=%d", M, n_local);
  for (int i = 0; i < peers->world; i++)
    if (!peers->slots[i] || !aligned(peers->slots[i], 8))
      return fail(LB200_E_NULL, "light_b200: allgather_ll: peer %d has no (8-byte aligned) receive buffer", i);
  if (int rc = bind(device)) return rc;
  return allgather_ll(local, out, peers, M, n_local, step, (cudaStream_t)stream);
}

int light_b200_comm_status(int device) {
  if (int rc = bind(device)) return rc;
  const int a = comm_status(), b = gemv_tp_status();
  return a ? a : b;
}

int light_b200_matmul_q_tp(int t, const float *x, const void *const *w, float *const *out, const int32_t *n, int count,
                           int K, const lb200_tp *tp, int device, void *stream) {
  if (t != LB200_Q4_K && t != LB200_Q6_K) return fail(LB200_E_DTYPE, "light_b200: matmul_q_tp: ggml type %d has no row-split kernel", t);
  if (count < 1 || count > 4) return fail(LB200_E_SHAPE, "light_b200: matmul_q_tp: %d matrices, want 1..4", count);
  if (K <= 0 || K % 256) return fail(LB200_E_SHAPE, "light_b200: matmul_q_tp: K=%d not a multiple of 256", K);
  REQUIRE_PTR(w, "matmul_q_tp");
  REQUIRE_PTR(out, "matmul_q_tp");
  REQUIRE_PTR(n, "matmul_q_tp");
  REQUIRE_PTR(tp, "matmul_q_tp");
  if (!tp->x_slots) REQUIRE_PTR(x, "matmul_q_tp");
  REQUIRE_PTR(tp->step, "matmul_q_tp");
  if (tp->world < 1 || tp->world > LB200_MAX_PEERS || tp->rank < 0 || tp->rank >= tp->world)
    return fail(LB200_E_SHAPE, "light_b200: matmul_q_tp: rank %d of %d", tp->rank, tp->world);
  for (int i = 0; i < count; i++)
    if (n[i] <= 0 || !w[i] || !out[i]) return fail(LB200_E_NULL, "light_b200: matmul_q_tp: matrix %d: null pointer or no rows", i);
  if (int rc = bind(device)) return rc;
  const int took = gguf_gemv_tp(t, x, tp->x_slots, w, out, n, count, K, (void *const *)tp->out_slots, tp->step, tp->world,
                                tp->rank, (cudaStream_t)stream);
  if (took == 1) return 0;
  if (took == 0) return fail(LB200_E_SHAPE, "light_b200: matmul_q_tp: no single-launch kernel for this shape or alignment");
  return took;
}

int light_b200_prefill_status(int device) {
  if (int rc = bind(device)) return rc;
  const int a = prefill_status(device), b = decode_umma_status(), c = decode_nt_status(), d = decode_ts_status();
  return a ? a : b ? b : c ? c : d;
}
unsigned long long light_b200_matmul_q_workspace_bytes(int M, int K) {
  if (M < 1 || K <= 0) return 0;
  unsigned long long f16_copy = M > 1 ? (unsigned long long)M * K * 2 : 0;  // the tensor-core paths' f16 copy of x
  if (M > 64) f16_copy += prefill_sk_ws_bytes();  // and, behind it, the partial tiles of the persistent prefill kernel
  unsigned long long staged = M <= 64 ? decode_nt_ws_bytes(M, K) : 0;
  if (M <= 64 && decode_ts_ws_bytes(M, K) > staged) staged = decode_ts_ws_bytes(M, K);
  return f16_copy > staged ? f16_copy : staged;
}
unsigned long long light_b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }
int light_b200_block_elems(int t) { return block_elems(t); }
int light_b200_block_bytes(int t) { return block_bytes(t); }

int light_b200_matmul_q(int t, const float *x, const void *w, float *out, int M, int N, int K, int device, void *stream) {
  const int be = block_elems(t);
  if (!be) return fail(LB200_E_DTYPE, "light_b200: matmul_q: ggml type %d has no fused kernel", t);
  if (M < 0 || N < 0 || K <= 0) return fail(LB200_E_SHAPE, "light_b200: matmul_q: bad shape M=%d N=%d K=%d", M, N, K);
  if (K % be) return fail(LB200_E_SHAPE, "light_b200: matmul_q: K=%d not a multiple of the block size %d", K, be);
  if (M == 0 || N == 0) return 0;
  REQUIRE_PTR(x, "matmul_q");
  REQUIRE_PTR(w, "matmul_q");
  REQUIRE_PTR(out, "matmul_q");
  if (!aligned(x, 16) || !aligned(out, 4) || !aligned(w, 2))
    return fail(LB200_E_ALIGN, "light_b200: matmul_q: x must be 16-byte, out 4-byte, w 2-byte aligned");
  if (int rc = bind(device)) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  int took = 0;
  if (M <= 64) {  // weights expanded into tensor memory (needs the workspace)
    size_t wsb = 0;
    void *ws = workspace_ptr(device, &wsb);
    const void *wv[1] = {w};
    float *ov[1] = {out};
    const int nv[1] = {N};
    took = gguf_decode_ts(t, x, wv, ov, nv, 1, M, K, ws, wsb, st);
    if (took != 0) return took == 1 ? 0 : took;
  }
  took = gguf_gemv_fast(t, x, w, out, M, N, K, st);
  if (took < 0) return took;
  if (took) return 0;
  if (M >= 2 && M <= 64) {  // tokens as MMA columns over activations staged once (needs the workspace)
    size_t wsb = 0;
    void *ws = workspace_ptr(device, &wsb);
    const void *wv[1] = {w};
    float *ov[1] = {out};
    const int nv[1] = {N};
    took = gguf_decode_nt(t, x, wv, ov, nv, 1, M, K, ws, wsb, st);
    if (took != 0) return took == 1 ? 0 : took;
  }
  took = gguf_gemv_tok(t, x, w, out, M, N, K, st);
  if (took != 0) return took == 1 ? 0 : took;
  took = gguf_prefill(t, x, w, out, M, N, K, device, st);
  if (took != 0) return took == 1 ? 0 : took;
  took = gguf_decode_tile(t, x, w, out, M, N, K, st);
  if (took != 0) return took == 1 ? 0 : took;
  took = gguf_decode_umma(t, x, w, out, M, N, K, device, st);
  if (took != 0) return took == 1 ? 0 : took;
  took = gguf_gemv_batch(t, x, w, out, M, N, K, st);
  if (took != 0) return took == 1 ? 0 : took;
  return gguf_matmul_generic(t, x, w, out, M, N, K, st);
}

int light_b200_matmul_q_multi(int t, const float *x, const void *const *w, float *const *out, const int32_t *n, int count,
                              int K, int device, void *stream) {
  const int be = block_elems(t);
  if (!be) return fail(LB200_E_DTYPE, "light_b200: matmul_q_multi: ggml type %d has no fused kernel", t);
  if (count < 1 || count > 4) return fail(LB200_E_SHAPE, "light_b200: matmul_q_multi: %d matrices, want 1..4", count);
  if (K <= 0 || K % be) return fail(LB200_E_SHAPE, "light_b200: matmul_q_multi: K=%d not a multiple of the block size %d", K, be);
  REQUIRE_PTR(x, "matmul_q_multi");
  REQUIRE_PTR(w, "matmul_q_multi");
  REQUIRE_PTR(out, "matmul_q_multi");
  REQUIRE_PTR(n, "matmul_q_multi");
  for (int i = 0; i < count; i++) {
    if (n[i] <= 0) return fail(LB200_E_SHAPE, "light_b200: matmul_q_multi: matrix %d has %d rows", i, n[i]);
    if (!w[i] || !out[i]) return fail(LB200_E_NULL, "light_b200: matmul_q_multi: null pointer for matrix %d", i);
    if (!aligned(out[i], 4) || !aligned(w[i], 2))
      return fail(LB200_E_ALIGN, "light_b200: matmul_q_multi: out must be 4-byte, w 2-byte aligned (matrix %d)", i);
  }
  if (!aligned(x, 16)) return fail(LB200_E_ALIGN, "light_b200: matmul_q_multi: x must be 16-byte aligned");
  if (int rc = bind(device)) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  int took = gguf_gemv_multi(t, x, w, out, n, count, 0, K, st);
  if (took != 0) return took == 1 ? 0 : took;
  for (int i = 0; i < count; i++)
    if (int rc = light_b200_matmul_q(t, x, w[i], out[i], 1, n[i], K, device, stream)) return rc;
  return 0;
}

int light_b200_matmul_q_multi_rows(int t, const float *x, const void *const *w, float *const *out, const int32_t *n, int count,
                                   int M, int K, int device, void *stream) {
  if (M == 1) return light_b200_matmul_q_multi(t, x, w, out, n, count, K, device, stream);
  const int be = block_elems(t);
  if (!be) return fail(LB200_E_DTYPE, "light_b200: matmul_q_multi_rows: ggml type %d has no fused kernel", t);
  if (count < 1 || count > 4) return fail(LB200_E_SHAPE, "light_b200: matmul_q_multi_rows: %d matrices, want 1..4", count);
  if (M < 0 || K <= 0 || K % be) return fail(LB200_E_SHAPE, "light_b200: matmul_q_multi_rows: M=%d K=%d (K a multiple of %d)", M, K, be);
  if (M == 0) return 0;
  REQUIRE_PTR(x, "matmul_q_multi_rows");
  REQUIRE_PTR(w, "matmul_q_multi_rows");
  REQUIRE_PTR(out, "matmul_q_multi_rows");
  REQUIRE_PTR(n, "matmul_q_multi_rows");
  for (int i = 0; i < count; i++) {
    if (n[i] <= 0) return fail(LB200_E_SHAPE, "light_b200: matmul_q_multi_rows: matrix %d has %d rows", i, n[i]);
    if (!w[i] || !out[i]) return fail(LB200_E_NULL, "light_b200: matmul_q_multi_rows: null pointer for matrix %d", i);
  }
  if (!aligned(x, 16)) return fail(LB200_E_ALIGN, "light_b200: matmul_q_multi_rows: x must be 16-byte aligned");
  if (int rc = bind(device)) return rc;
  int took = 0;
  if (M <= 64) {
    size_t wsb = 0;
    void *ws = workspace_ptr(device, &wsb);
    took = gguf_decode_ts(t, x, w, out, n, count, M, K, ws, wsb, (cudaStream_t)stream);
    if (took != 0) return took == 1 ? 0 : took;
    took = gguf_decode_nt(t, x, w, out, n, count, M, K, ws, wsb, (cudaStream_t)stream);
    if (took != 0) return took == 1 ? 0 : took;
  }
  took = gguf_gemv_tok_multi(t, x, w, out, n, count, M, K, (cudaStream_t)stream);
  if (took != 0) return took == 1 ? 0 : took;
  for (int i = 0; i < count; i++)  // other types and row counts: one launch per matrix, each (M, n[i]) dense
    if (int rc = light_b200_matmul_q(t, x, w[i], out[i], M, n[i], K, device, stream)) return rc;
  return 0;
}

int light_b200_matmul_q_gated(int t, const float *x, const void *wg, const void *wu, float *out, int N, int K, int act,
                              int device, void *stream) {
  if (t != LB200_Q4_K) return fail(LB200_E_DTYPE, "light_b200: matmul_q_gated: ggml type %d has no gated kernel", t);
  if (act != 1 && act != 2) return fail(LB200_E_SHAPE, "light_b200: matmul_q_gated: act %d, want 1 (SiLU) or 2 (GELU)", act);
  if (N < 16 || K <= 0 || K % 256)
    return fail(LB200_E_SHAPE, "light_b200: matmul_q_gated: N=%d K=%d (N >= 16, K a multiple of 256)", N, K);
  REQUIRE_PTR(x, "matmul_q_gated");
  REQUIRE_PTR(wg, "matmul_q_gated");
  REQUIRE_PTR(wu, "matmul_q_gated");
  REQUIRE_PTR(out, "matmul_q_gated");
  if (!aligned(x, 16) || !aligned(out, 4) || !aligned(wg, 16) || !aligned(wu, 16))
    return fail(LB200_E_ALIGN, "light_b200: matmul_q_gated: x, wg, wu must be 16-byte, out 4-byte aligned");
  if (int rc = bind(device)) return rc;
  const void *w[2] = {wg, wu};
  float *o[2] = {out, out};
  const int n[2] = {N, N};
  const int took = gguf_gemv_multi(t, x, w, o, n, 2, act, K, (cudaStream_t)stream);
  if (took == 1) return 0;
  if (took == 0) return fail(LB200_E_SHAPE, "light_b200: matmul_q_gated: K=%d is too long for the fused kernel", K);
  return took;
}

int light_b200_matmul_q_fused(int t, const float *x, const lb200_norm *norm, const void *const *w, float *const *out,
                              const int32_t *n, int count, int act, int K, int device, void *stream) {
  if (t != LB200_Q4_K) return fail(LB200_E_DTYPE, "light_b200: matmul_q_fused: ggml type %d has no fused kernel", t);
  if (act < 0 || act > 2 || count < 1 || count > 4 || (act && count != 2))
    return fail(LB200_E_SHAPE, "light_b200: matmul_q_fused: act %d with %d matrices (act 0: 1..4, act 1 / 2: 2)", act, count);
  if (K <= 0 || K % 256) return fail(LB200_E_SHAPE, "light_b200: matmul_q_fused: K=%d, want a multiple of 256", K);
  REQUIRE_PTR(x, "matmul_q_fused");
  REQUIRE_PTR(norm, "matmul_q_fused");
  REQUIRE_PTR(w, "matmul_q_fused");
  REQUIRE_PTR(out, "matmul_q_fused");
  REQUIRE_PTR(n, "matmul_q_fused");
  if (!norm->weight || (norm->residual && !norm->sum_out))
    return fail(LB200_E_NULL, "light_b200: matmul_q_fused: norm weight missing, or a residual without sum_out");
  if (norm->sum_out && (norm->sum_out == x || norm->sum_out == norm->residual))
    return fail(LB200_E_SHAPE, "light_b200: matmul_q_fused: sum_out must not alias x or residual");
  if (!aligned(x, 16) || !aligned(norm->weight, 16) || !aligned(norm->residual, 16) || !aligned(norm->sum_out, 16))
    return fail(LB200_E_ALIGN, "light_b200: matmul_q_fused: x, norm weight, residual and sum_out must be 16-byte aligned");
  for (int i = 0; i < count; i++) {
    if (n[i] < 16 || (act && n[i] != n[0])) return fail(LB200_E_SHAPE, "light_b200: matmul_q_fused: matrix %d has %d rows", i, n[i]);
    if (!w[i] || !out[act ? 0 : i]) return fail(LB200_E_NULL, "light_b200: matmul_q_fused: null pointer for matrix %d", i);
    if (!aligned(w[i], 16) || !aligned(out[act ? 0 : i], 4))
      return fail(LB200_E_ALIGN, "light_b200: matmul_q_fused: w must be 16-byte, out 4-byte aligned (matrix %d)", i);
  }
  if (int rc = bind(device)) return rc;
  float *o2[2] = {out[0], out[0]};
  const int took = gguf_gemv_multi(t, x, w, act ? o2 : out, n, count, act, K, (cudaStream_t)stream, norm);
  if (took == 1) return 0;
  if (took == 0) return fail(LB200_E_SHAPE, "light_b200: matmul_q_fused: K=%d is too long for the fused kernel", K);
  return took;
}

int light_b200_dequant(int t, const void *src, float *dst, int64_t n, int device, void *stream) {
  const int be = block_elems(t);
  if (!be) return fail(LB200_E_DTYPE, "light_b200: dequant: ggml type %d has no kernel", t);
  if (n < 0 || n % be) return fail(LB200_E_SHAPE, "light_b200: dequant: %lld elements is not a whole number of %d-element blocks", (long long)n, be);
  if (n == 0) return 0;
  REQUIRE_PTR(src, "dequant");
  REQUIRE_PTR(dst, "dequant");
  if (!aligned(dst, 16)) return fail(LB200_E_ALIGN, "light_b200: dequant: dst must be 16-byte aligned");
  if (int rc = bind(device)) return rc;
  return gguf_dequant(t, src, dst, n, (cudaStream_t)stream);
}

static int act_ok(int dt) { return dt == LB200_F32 || dt == LB200_BF16; }

int light_b200_int4_dequant(const uint32_t *codes, const float *s, const float *z, void *out, int out_dtype, int N,
                            int K, int G, int64_t offset, int device, void *stream) {
  if (!act_ok(out_dtype)) return fail(LB200_E_DTYPE, "light_b200: int4_dequant: output type %d, want F32 or BF16", out_dtype);
  if (N < 0 || K < 0 || G <= 0 || K % 8 || G % 8 || K % G || offset < 0)
    return fail(LB200_E_SHAPE, "light_b200: int4_dequant: bad shape N=%d K=%d group=%d offset=%lld", N, K, G, (long long)offset);
  if (N == 0 || K == 0) return 0;
  REQUIRE_PTR(codes, "int4_dequant");
  REQUIRE_PTR(s, "int4_dequant");
  REQUIRE_PTR(z, "int4_dequant");
  REQUIRE_PTR(out, "int4_dequant");
  size_t esz = out_dtype == LB200_F32 ? 4 : 2;
  if (!aligned((const char *)out + offset * esz, 16))
    return fail(LB200_E_ALIGN, "light_b200: int4_dequant: out + offset must be 16-byte aligned");
  if (int rc = bind(device)) return rc;
  return int4_dequant(codes, s, z, out, out_dtype, N, K, G, offset, (cudaStream_t)stream);
}

int light_b200_int4_gemv(const void *x, const uint32_t *codes, const float *s, const float *z, void *y, int act_dtype,
                         int M, int N, int K, int G, int device, void *stream) {
  if (!act_ok(act_dtype)) return fail(LB200_E_DTYPE, "light_b200: int4_gemv: activation type %d, want F32 or BF16", act_dtype);
  if (M < 0 || N < 0 || K <= 0 || G <= 0 || K % 32 || G % 32 || K % G)
    return fail(LB200_E_SHAPE, "light_b200: int4_gemv: bad shape M=%d N=%d K=%d group=%d (K and group must be multiples of 32)", M, N, K, G);
  if (M == 0 || N == 0) return 0;
  REQUIRE_PTR(x, "int4_gemv");
  REQUIRE_PTR(codes, "int4_gemv");
  REQUIRE_PTR(s, "int4_gemv");
  REQUIRE_PTR(z, "int4_gemv");
  REQUIRE_PTR(y, "int4_gemv");
  if (!aligned(codes, 16) || !aligned(x, 16)) return fail(LB200_E_ALIGN, "light_b200: int4_gemv: x and codes must be 16-byte aligned");
  if (int rc = bind(device)) return rc;
  if (M >= 4 && M <= 64) {  // token tiles over activations staged once (needs the workspace)
    size_t wsb = 0;
    void *ws = workspace_ptr(device, &wsb);
    if (int took = int4_decode_nt(x, codes, s, z, y, act_dtype, M, N, K, G, ws, wsb, (cudaStream_t)stream)) return took == 1 ? 0 : took;
  }
  if (int took = int4_gemv_fast(x, codes, s, z, y, act_dtype, M, N, K, G, (cudaStream_t)stream)) return took == 1 ? 0 : took;
  if (int took = int4_prefill(x, codes, s, z, y, act_dtype, M, N, K, G, device, (cudaStream_t)stream)) return took == 1 ? 0 : took;
  if (int took = int4_decode_umma(x, codes, s, z, y, act_dtype, M, N, K, G, device, (cudaStream_t)stream)) return took == 1 ? 0 : took;
  return int4_rows_dot(x, codes, s, z, y, act_dtype, M, N, K, G, (cudaStream_t)stream);  // the tile kernel with the 4-bit row fetcher
}

int light_b200_fp8_block_dequant(const uint8_t *w, const float *s, void *out, int out_dtype, int R, int C, int bR,
                                 int bC, int device, void *stream) {
  if (!act_ok(out_dtype)) return fail(LB200_E_DTYPE, "light_b200: fp8_block_dequant: output type %d, want F32 or BF16", out_dtype);
  if (R < 0 || C < 0 || bR <= 0 || bC <= 0 || R % bR || C % bC || C % 4 || bC % 4)
    return fail(LB200_E_SHAPE, "light_b200: fp8_block_dequant: (%d, %d) not a multiple of block (%d, %d), or columns not a multiple of 4", R, C, bR, bC);
  if (R == 0 || C == 0) return 0;
  REQUIRE_PTR(w, "fp8_block_dequant");
  REQUIRE_PTR(s, "fp8_block_dequant");
  REQUIRE_PTR(out, "fp8_block_dequant");
  if (!aligned(w, 4) || !aligned(out, 16)) return fail(LB200_E_ALIGN, "light_b200: fp8_block_dequant: w must be 4-byte, out 16-byte aligned");
  if (int rc = bind(device)) return rc;
  return fp8_block_dequant(w, s, out, out_dtype, R, C, bR, bC, (cudaStream_t)stream);
}

int light_b200_fp8_block_gemv(const void *x, const uint8_t *w, const float *s, void *y, int act_dtype, int M, int N,
                              int K, int bR, int bC, int device, void *stream) {
  if (!act_ok(act_dtype)) return fail(LB200_E_DTYPE, "light_b200: fp8_block_gemv: activation type %d, want F32 or BF16", act_dtype);
  if (M < 0 || N < 0 || K <= 0 || bR <= 0 || bC <= 0 || K % 16 || bC % 16 || N % bR || K % bC)
    return fail(LB200_E_SHAPE, "light_b200: fp8_block_gemv: bad shape M=%d N=%d K=%d block (%d, %d)", M, N, K, bR, bC);
  if (M == 0 || N == 0) return 0;
  REQUIRE_PTR(x, "fp8_block_gemv");
  REQUIRE_PTR(w, "fp8_block_gemv");
  REQUIRE_PTR(s, "fp8_block_gemv");
  REQUIRE_PTR(y, "fp8_block_gemv");
  if (!aligned(w, 16) || !aligned(x, 16)) return fail(LB200_E_ALIGN, "light_b200: fp8_block_gemv: x and w must be 16-byte aligned");
  if (int rc = bind(device)) return rc;
  if (M >= 4 && M <= 64) {  // token tiles over activations staged once (needs the workspace)
    size_t wsb = 0;
    void *ws = workspace_ptr(device, &wsb);
    if (int took = fp8_decode_nt(x, w, s, y, act_dtype, M, N, K, bR, bC, ws, wsb, (cudaStream_t)stream)) return took == 1 ? 0 : took;
  }
  if (int took = fp8_gemv_fast(x, w, s, y, act_dtype, M, N, K, bR, bC, (cudaStream_t)stream)) return took == 1 ? 0 : took;
  if (int took = fp8_prefill(x, w, s, y, act_dtype, M, N, K, bR, bC, device, (cudaStream_t)stream)) return took == 1 ? 0 : took;
  if (int took = fp8_decode_umma(x, w, s, y, act_dtype, M, N, K, bR, bC, device, (cudaStream_t)stream)) return took == 1 ? 0 : took;
  return fp8_block_rows_dot(x, w, s, y, act_dtype, M, N, K, bR, bC, (cudaStream_t)stream);  // the tile kernel with the block-FP8 row fetcher
}

static int moe_check(const lb200_moe_args *a, const char *op, bool quant, bool need_scratch = true) {
  if (!a) return fail(LB200_E_NULL, "light_b200: %s: null argument block", op);
  if (a->M < 0 || a->size_m < 0 || a->E <= 0 || a->N < 0 || a->K <= 0 || a->topk < 1)
    return fail(LB200_E_SHAPE, "light_b200: %s: bad shape M=%lld size_m=%lld E=%d N=%d K=%d topk=%d", op, (long long)a->M,
                (long long)a->size_m, a->E, a->N, a->K, a->topk);
  if (quant) {
    int be = block_elems(a->dtype);
    if (!be) return fail(LB200_E_DTYPE, "light_b200: %s: ggml type %d has no fused kernel", op, a->dtype);
    if (a->K % be) return fail(LB200_E_SHAPE, "light_b200: %s: K=%d not a multiple of the block size %d", op, a->K, be);
  } else {
    if (a->dtype != LB200_F32 && a->dtype != LB200_BF16 && a->dtype != LB200_F16)
      return fail(LB200_E_DTYPE, "light_b200: %s: element type %d, want F32, BF16 or F16", op, a->dtype);
    if (a->K % 8) return fail(LB200_E_SHAPE, "light_b200: %s: K=%d must be a multiple of 8", op, a->K);
  }
  if (need_scratch && (!a->counts || !a->offsets))
    return fail(LB200_E_NULL, "light_b200: %s: counts / offsets scratch missing", op);
  if (a->M > 0 && (!a->input || !a->weights || !a->sorted_pairs || !a->expert_ids || !a->out))
    return fail(LB200_E_NULL, "light_b200: %s: null tensor pointer", op);
  if (a->M > 0 && (!aligned(a->input, 16) || !aligned(a->weights, quant ? 2 : 16)))
    return fail(LB200_E_ALIGN, "light_b200: %s: input and weights must be 16-byte aligned", op);
  return 0;
}

int light_b200_moe_gemm(const lb200_moe_args *a, int device, void *stream) {
  if (int rc = moe_check(a, "moe_gemm", false)) return rc;
  if (int rc = bind(device)) return rc;
  return moe_gemm(a, device, (cudaStream_t)stream);
}

int light_b200_moe_gemm_static_scratch(const lb200_moe_args *a, int device, void *stream) {
  if (int rc = moe_check(a, "moe_gemm_static_scratch", false, false)) return rc;
  if (int rc = bind(device)) return rc;
  return moe_gemm_static_scratch(a, device, (cudaStream_t)stream);
}

int light_b200_kv_append(const void *k, const void *v, void *kbuf, void *vbuf, const int64_t *pos, int dtype, int B, int KH,
                         int D, int Cap, int device, void *stream) {
  if (int rc = bind(device)) return rc;
  return kv_append(k, v, kbuf, vbuf, pos, dtype, B, KH, D, Cap, (cudaStream_t)stream);
}

int light_b200_decode_attn(const lb200_decode_attn_args *a, int device, void *stream) {
  if (int rc = bind(device)) return rc;
  return decode_attn(a, (cudaStream_t)stream);
}

int light_b200_embedding_q(int t, const void *table, const int64_t *ids, float *out, int64_t n_ids, int64_t V, int K, int device,
                           void *stream) {
  const int be = block_elems(t);
  if (!be) return fail(LB200_E_DTYPE, "light_b200: embedding_q: ggml type %d has no kernel", t);
  if (n_ids < 0 || n_ids > 0x7fffffffLL || V <= 0 || K <= 0 || K % be || K % 8)
    return fail(LB200_E_SHAPE, "light_b200: embedding_q: %lld ids, table (%lld, %d)", (long long)n_ids, (long long)V, K);
  if (n_ids == 0) return 0;
  REQUIRE_PTR(table, "embedding_q");
  REQUIRE_PTR(ids, "embedding_q");
  REQUIRE_PTR(out, "embedding_q");
  if (!aligned(out, 16) || !aligned(table, 2)) return fail(LB200_E_ALIGN, "light_b200: embedding_q: out must be 16-byte, table 2-byte aligned");
  if (int rc = bind(device)) return rc;
  return gguf_embedding(t, table, ids, out, n_ids, V, K, (cudaStream_t)stream);
}

int light_b200_int4_repack(const void *qweight, const void *qzeros, const float *scales, void *codes, float *scales_out, float *zeros_out,
                           int N, int K, int group, int layout, int device, void *stream) {
  REQUIRE_PTR(qweight, "int4_repack");
  REQUIRE_PTR(qzeros, "int4_repack");
  REQUIRE_PTR(scales, "int4_repack");
  REQUIRE_PTR(codes, "int4_repack");
  REQUIRE_PTR(scales_out, "int4_repack");
  REQUIRE_PTR(zeros_out, "int4_repack");
  if (int rc = bind(device)) return rc;
  return int4_repack((const uint32_t *)qweight, (const uint32_t *)qzeros, scales, (uint32_t *)codes, scales_out, zeros_out, N, K,
                     group <= 0 ? K : group, layout, (cudaStream_t)stream);
}

int light_b200_quantize_rows_int8(const float *x, int8_t *q, float *scales, int64_t M, int K, int device, void *stream) {
  if (M < 0 || M > 0x7fffffffLL || K <= 0) return fail(LB200_E_SHAPE, "light_b200: quantize_rows_int8: M=%lld K=%d", (long long)M, K);
  if (M == 0) return 0;
  REQUIRE_PTR(x, "quantize_rows_int8");
  REQUIRE_PTR(q, "quantize_rows_int8");
  REQUIRE_PTR(scales, "quantize_rows_int8");
  if (int rc = bind(device)) return rc;
  return quantize_rows_int8(x, q, scales, M, K, (cudaStream_t)stream);
}

int light_b200_matmul_w8a8(const float *x, const int8_t *wq, const float *ws, float *out, int8_t *xq_scratch, float *xs_scratch, int M,
                           int N, int K, int device, void *stream) {
  if (M < 0 || N < 0 || K <= 0) return fail(LB200_E_SHAPE, "light_b200: matmul_w8a8: bad shape M=%d N=%d K=%d", M, N, K);
  if (K % 16) return fail(LB200_E_SHAPE, "light_b200: matmul_w8a8: K=%d, want a multiple of 16", K);
  if (M == 0 || N == 0) return 0;
  REQUIRE_PTR(x, "matmul_w8a8");
  REQUIRE_PTR(wq, "matmul_w8a8");
  REQUIRE_PTR(ws, "matmul_w8a8");
  REQUIRE_PTR(out, "matmul_w8a8");
  REQUIRE_PTR(xq_scratch, "matmul_w8a8");
  REQUIRE_PTR(xs_scratch, "matmul_w8a8");
  if (!aligned(wq, 16) || !aligned(xq_scratch, 16) || !aligned(out, 4) || !aligned(x, 4))
    return fail(LB200_E_ALIGN, "light_b200: matmul_w8a8: wq and xq_scratch must be 16-byte aligned");
  if (int rc = bind(device)) return rc;
  return matmul_w8a8(x, wq, ws, out, xq_scratch, xs_scratch, M, N, K, (cudaStream_t)stream);
}

int light_b200_moe_route_sigmoid(const float *logits, const float *bias, int64_t *ids, float *weights, int T, int E, int topk,
                                 int norm_topk, int device, void *stream) {
  if (T < 0 || E < 1 || E > 1024 || topk < 1 || topk > E || topk > 32)
    return fail(LB200_E_SHAPE, "light_b200: moe_route_sigmoid: T=%d E=%d (at most 1024) topk=%d (at most 32)", T, E, topk);
  if (T == 0) return 0;
  REQUIRE_PTR(logits, "moe_route_sigmoid");
  REQUIRE_PTR(ids, "moe_route_sigmoid");
  REQUIRE_PTR(weights, "moe_route_sigmoid");
  if (int rc = bind(device)) return rc;
  return moe_route_sigmoid(logits, bias, ids, weights, T, E, topk, norm_topk, (cudaStream_t)stream);
}

int light_b200_moe_sort_pairs(const int64_t *ids, int32_t *counts, int32_t *offsets, int64_t *sorted_pairs, int64_t *sorted_expts,
                              int32_t *scratch, int64_t M, int E, int device, void *stream) {
  if (M < 0 || M > 0x7fffffffLL || E < 1 || E > 1024) return fail(LB200_E_SHAPE, "light_b200: moe_sort_pairs: M=%lld E=%d (at most 1024)", (long long)M, E);
  REQUIRE_PTR(counts, "moe_sort_pairs");
  REQUIRE_PTR(offsets, "moe_sort_pairs");
  if (M > 0) {
    REQUIRE_PTR(ids, "moe_sort_pairs");
    REQUIRE_PTR(sorted_pairs, "moe_sort_pairs");
    REQUIRE_PTR(sorted_expts, "moe_sort_pairs");
    REQUIRE_PTR(scratch, "moe_sort_pairs");
  }
  if (int rc = bind(device)) return rc;
  return moe_sort_pairs(ids, counts, offsets, sorted_pairs, sorted_expts, scratch, M, E, (cudaStream_t)stream);
}

int light_b200_moe_route_deepseek(const float *logits, const float *bias, int64_t *ids, float *weights, int T, int E, int topk, int n_group,
                                  int topk_group, int sigmoid, int norm_topk, int device, void *stream) {
  if (n_group < 1) n_group = 1;
  if (T < 0 || E < 1 || E > 1024 || topk < 1 || topk > 32 || topk > E || n_group > 32 || E % n_group || topk_group < 1)
    return fail(LB200_E_SHAPE, "light_b200: moe_route_deepseek: T=%d E=%d topk=%d n_group=%d topk_group=%d (E <= 1024, topk <= 32, n_group <= 32 divides E)",
                T, E, topk, n_group, topk_group);
  if (T == 0) return 0;
  REQUIRE_PTR(logits, "moe_route_deepseek");
  REQUIRE_PTR(ids, "moe_route_deepseek");
  REQUIRE_PTR(weights, "moe_route_deepseek");
  if (int rc = bind(device)) return rc;
  return moe_route_deepseek(logits, sigmoid ? bias : nullptr, ids, weights, T, E, topk, n_group, topk_group, sigmoid, norm_topk, (cudaStream_t)stream);
}

int light_b200_moe_route_topk(const float *probs, int64_t *ids, float *weights, int T, int E, int topk, int normalize, int device, void *stream) {
  if (T < 0 || E < 1 || E > 1024 || topk < 1 || topk > 32 || topk > E)
    return fail(LB200_E_SHAPE, "light_b200: moe_route_topk: T=%d E=%d topk=%d (E <= 1024, topk <= min(32, E))", T, E, topk);
  if (T == 0) return 0;
  REQUIRE_PTR(probs, "moe_route_topk");
  REQUIRE_PTR(ids, "moe_route_topk");
  REQUIRE_PTR(weights, "moe_route_topk");
  if (int rc = bind(device)) return rc;
  return moe_route_topk(probs, ids, weights, T, E, topk, normalize, (cudaStream_t)stream);
}

int light_b200_moe_gate_mul(const void *h, void *out, int dtype, int64_t M, int I, int gelu, int device, void *stream) {
  if (M < 0 || I <= 0 || I % 8) return fail(LB200_E_SHAPE, "light_b200: moe_gate_mul: M=%lld I=%d (I a positive multiple of 8)", (long long)M, I);
  if (M == 0) return 0;
  REQUIRE_PTR(h, "moe_gate_mul");
  REQUIRE_PTR(out, "moe_gate_mul");
  if (!aligned(h, 16) || !aligned(out, 16)) return fail(LB200_E_ALIGN, "light_b200: moe_gate_mul: pointers not 16-byte aligned");
  if (int rc = bind(device)) return rc;
  return moe_gate_mul(h, out, dtype, M, I, gelu, (cudaStream_t)stream);
}

int light_b200_moe_combine(const void *pair_out, void *out, int dtype, int64_t tokens, int N, int topk, int device, void *stream) {
  if (tokens < 0 || N <= 0 || N % 8 || topk < 1) return fail(LB200_E_SHAPE, "light_b200: moe_combine: tokens=%lld N=%d topk=%d", (long long)tokens, N, topk);
  if (tokens == 0) return 0;
  REQUIRE_PTR(pair_out, "moe_combine");
  REQUIRE_PTR(out, "moe_combine");
  if (!aligned(pair_out, 16) || !aligned(out, 16)) return fail(LB200_E_ALIGN, "light_b200: moe_combine: pointers not 16-byte aligned");
  if (int rc = bind(device)) return rc;
  return moe_combine(pair_out, out, dtype, tokens, N, topk, (cudaStream_t)stream);
}

int light_b200_moe_combine_weighted(const void *rows, const int64_t *index, const float *weights, float *out, int dtype, int64_t tokens,
                                    int N, int topk, int64_t n_rows, int device, void *stream) {
  if (tokens < 0 || N <= 0 || N % 8 || topk < 1 || n_rows < 0)
    return fail(LB200_E_SHAPE, "light_b200: moe_combine_weighted: tokens=%lld N=%d topk=%d rows=%lld", (long long)tokens, N, topk, (long long)n_rows);
  if (tokens == 0) return 0;
  REQUIRE_PTR(out, "moe_combine_weighted");
  if (n_rows) REQUIRE_PTR(rows, "moe_combine_weighted");
  if (!index && n_rows < tokens * topk) return fail(LB200_E_SHAPE, "light_b200: moe_combine_weighted: no index and fewer rows than pairs");
  if (!aligned(rows, 16) || !aligned(out, 16)) return fail(LB200_E_ALIGN, "light_b200: moe_combine_weighted: pointers not 16-byte aligned");
  if (int rc = bind(device)) return rc;
  return moe_combine_weighted(rows, index, weights, out, dtype, tokens, N, topk, n_rows, (cudaStream_t)stream);
}

int light_b200_moe_route_status(int device) {
  if (int rc = bind(device)) return rc;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return fail((int)e, "light_b200: moe_route_status: %s", cudaGetErrorString(e));
  const int a = moe_route_status(), b = moe_bad_ids_status();
  if (a > 1 || a < 0) return a;
  if (b > 1 || b < 0) return b;
  return a | b;
}

int light_b200_gather_columns(const void *x, const int64_t *idx, void *out, int dtype, int64_t M, int K, int device, void *stream) {
  if (M < 0 || K < 0) return fail(LB200_E_SHAPE, "light_b200: gather_columns: M=%lld K=%d", (long long)M, K);
  if (dtype != LB200_F32 && dtype != LB200_BF16 && dtype != LB200_F16) return fail(LB200_E_DTYPE, "light_b200: gather_columns: element type %d", dtype);
  if (M == 0 || K == 0) return 0;
  REQUIRE_PTR(x, "gather_columns");
  REQUIRE_PTR(idx, "gather_columns");
  REQUIRE_PTR(out, "gather_columns");
  if (int rc = bind(device)) return rc;
  return gather_columns(x, idx, out, dtype == LB200_F32 ? 4 : 2, M, K, (cudaStream_t)stream);
}

int light_b200_gemv_multi(const void *x, const void *const *w, void *const *out, const int32_t *n, int count, int K, int out_f32, int device,
                          void *stream) {
  if (count < 1 || count > 4) return fail(LB200_E_SHAPE, "light_b200: gemv_multi: %d weights, want 1..4", count);
  if (K <= 0 || K % 8) return fail(LB200_E_SHAPE, "light_b200: gemv_multi: K=%d not a positive multiple of 8", K);
  REQUIRE_PTR(x, "gemv_multi");
  REQUIRE_PTR(w, "gemv_multi");
  REQUIRE_PTR(out, "gemv_multi");
  REQUIRE_PTR(n, "gemv_multi");
  if (!aligned(x, 16)) return fail(LB200_E_ALIGN, "light_b200: gemv_multi: x not 16-byte aligned");
  for (int i = 0; i < count; i++) {
    if (n[i] <= 0 || !w[i] || !out[i]) return fail(LB200_E_NULL, "light_b200: gemv_multi: matrix %d: null pointer or no rows", i);
    if (!aligned(w[i], 16)) return fail(LB200_E_ALIGN, "light_b200: gemv_multi: matrix %d not 16-byte aligned", i);
  }
  if (int rc = bind(device)) return rc;
  return gemv_bf16_multi(x, w, out, n, count, K, out_f32, (cudaStream_t)stream);
}

int light_b200_gemv_gated(const void *x, const void *wg, const void *wu, void *out, int N, int K, int gelu, int device, void *stream) {
  if (N < 0 || K <= 0 || K % 8) return fail(LB200_E_SHAPE, "light_b200: gemv_gated: bad shape N=%d K=%d", N, K);
  if (N == 0) return 0;
  REQUIRE_PTR(x, "gemv_gated");
  REQUIRE_PTR(wg, "gemv_gated");
  REQUIRE_PTR(wu, "gemv_gated");
  REQUIRE_PTR(out, "gemv_gated");
  if (!aligned(x, 16) || !aligned(wg, 16) || !aligned(wu, 16)) return fail(LB200_E_ALIGN, "light_b200: gemv_gated: x / weights not 16-byte aligned");
  if (int rc = bind(device)) return rc;
  return gemv_bf16_gated(x, wg, wu, out, N, K, gelu, (cudaStream_t)stream);
}

size_t light_b200_chain_program_bytes(int n_ops) { return n_ops < 0 ? 0 : chain_program_bytes(n_ops); }

int64_t light_b200_chain_arena_bytes(const lb200_chain_op *ops, int n_ops, int n_vecs, int world) {
  if (!ops || n_ops < 1 || n_vecs < 0 || world < 1 || world > LB200_MAX_PEERS) return -1;
  return chain_arena_bytes(ops, n_ops, n_vecs, world);
}

int light_b200_chain_build(const lb200_chain_op *ops, int n_ops, int n_vecs, void *program, size_t program_bytes, void *const *arena,
                           size_t arena_bytes, int world, int rank, int device, void *stream) {
  REQUIRE_PTR(ops, "chain_build");
  REQUIRE_PTR(program, "chain_build");
  REQUIRE_PTR(arena, "chain_build");
  if (world < 1 || world > LB200_MAX_PEERS || rank < 0 || rank >= world)
    return fail(LB200_E_SHAPE, "light_b200: chain_build: rank %d of %d", rank, world);
  if (n_vecs < 0 || n_vecs > 4096) return fail(LB200_E_SHAPE, "light_b200: chain_build: %d chain vectors", n_vecs);
  for (int p = 0; p < world; p++)
    if (!arena[p] || !aligned(arena[p], 256)) return fail(LB200_E_ALIGN, "light_b200: chain_build: arena of rank %d is null or not 256-byte aligned", p);
  if (!aligned(program, 256)) return fail(LB200_E_ALIGN, "light_b200: chain_build: program buffer not 256-byte aligned");
  if (int rc = bind(device)) return rc;
  return chain_build(ops, n_ops, n_vecs, program, program_bytes, arena, arena_bytes, world, rank, (cudaStream_t)stream);
}

int light_b200_chain_run(const void *program, uint32_t *step, int device, void *stream) {
  REQUIRE_PTR(program, "chain_run");
  REQUIRE_PTR(step, "chain_run");
  if (int rc = bind(device)) return rc;
  return chain_run(program, step, (cudaStream_t)stream);
}

int light_b200_chain_status(int device) {
  if (int rc = bind(device)) return rc;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return fail((int)e, "light_b200: chain_status: %s", cudaGetErrorString(e));
  return chain_status();
}

int light_b200_argmax(const float *x, int64_t *out, int64_t rows, int cols, int device, void *stream) {
  if (int rc = bind(device)) return rc;
  return argmax_rows(x, out, rows, cols, (cudaStream_t)stream);
}

int light_b200_rmsnorm(const void *x, const void *residual, const void *weight, void *sum_out, void *out, int dtype, int64_t rows,
                       int cols, float eps, int device, void *stream) {
  if (int rc = bind(device)) return rc;
  return rmsnorm(x, residual, weight, sum_out, out, dtype, rows, cols, eps, (cudaStream_t)stream);
}

int light_b200_rope(const void *x, const int64_t *positions, void *out, int dtype, int64_t rows, int seq_len, int head_dim,
                    double base, int device, void *stream) {
  if (int rc = bind(device)) return rc;
  return rope(x, positions, out, dtype, rows, seq_len, head_dim, base, (cudaStream_t)stream);
}

int light_b200_inc_i64(int64_t *p, int n, int device, void *stream) {
  if (int rc = bind(device)) return rc;
  return inc_i64(p, n, (cudaStream_t)stream);
}

int light_b200_decode_attn_status(int device) {
  if (int rc = bind(device)) return rc;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return fail((int)e, "light_b200: decode_attn_status: %s", cudaGetErrorString(e));
  return decode_attn_status();
}

int light_b200_moe_gemm_f8block(const lb200_moe_args *a, const float *w_scale, int block_r, int block_c, int device,
                                 void *stream) {
  if (!a) return fail(LB200_E_NULL, "light_b200: moe_gemm_f8block: null argument block");
  if (a->M < 0 || a->size_m < 0 || a->E <= 0 || a->N < 0 || a->K <= 0 || a->topk < 1 || block_r <= 0 || block_c <= 0)
    return fail(LB200_E_SHAPE, "light_b200: moe_gemm_f8block: bad shape");
  if (a->dtype != LB200_F32 && a->dtype != LB200_BF16)
    return fail(LB200_E_DTYPE, "light_b200: moe_gemm_f8block: activation type %d, want F32 or BF16", a->dtype);
  if (!a->counts || !a->offsets || !w_scale) return fail(LB200_E_NULL, "light_b200: moe_gemm_f8block: counts / offsets / scale missing");
  if (a->M > 0 && (!a->input || !a->weights || !a->sorted_pairs || !a->expert_ids || !a->out))
    return fail(LB200_E_NULL, "light_b200: moe_gemm_f8block: null tensor pointer");
  if (int rc = bind(device)) return rc;
  if (a->M == 0) return 0;
  return moe_gemm_f8block(a, w_scale, block_r, block_c, device, (cudaStream_t)stream);
}

int light_b200_moe_gemm_q(const lb200_moe_args *a, int device, void *stream) {
  if (int rc = moe_check(a, "moe_gemm_q", true)) return rc;
  if (int rc = bind(device)) return rc;
  return moe_gemm_q(a, device, (cudaStream_t)stream);
}

}  // extern "C"
