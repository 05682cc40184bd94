// Prefill (many activation rows) fused dequant-matmul for Q4_K / Q6_K on the 5th-generation tensor
// cores: out (M, N) f32 = x (M, K) . dequant(W (N, K))^T.
//
//   * x is converted once to f16 (a tiny pre-pass into the workspace) and streamed by TMA as
//     128 x 64 tiles in the 128-byte swizzle layout -- the A operand;
//   * the packed weights are read straight from global memory by 256 threads, one weight row each,
//     expanded in registers (f32 arithmetic, one rounding to f16) and written into shared memory in
//     the same swizzled layout -- the B operand (256 rows x 64 k).  The expanded weight never
//     exists in HBM, and is expanded once per 256 tokens;
//   * one thread issues tcgen05.mma (M 128, N 256, K 16, f16 -> f32): two accumulators of
//     128 x 256 f32 fill the SM's tensor memory, so a CTA owns a 256 (tokens) x 256 (rows) tile;
//   * completion is tracked with mbarriers (TMA -> MMA -> free stage), the epilogue reads the
//     accumulators with tcgen05.ld and writes f32 rows.
//
// f16 (not bf16) operands: the reference multiplies f32 weights by f32 activations; rounding the
// weights to bf16 alone costs 1.7e-3 relative L2, to f16 2e-4.
#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "umma.cuh"

namespace lb {

namespace {

using namespace umma;

constexpr int BM = 256;          // tokens per CTA (two MMA tiles of 128)
constexpr int BN = 256;          // weight rows per CTA (MMA N)
constexpr int BK = 64;           // k per stage: 128 bytes of f16, one swizzle row
constexpr int SA = 3, SB = 2;    // stages of the A (x) and B (weights) rings
constexpr int A_STAGE = BM * BK * 2, B_STAGE = BN * BK * 2;
constexpr int NUM_DEQ_WARPS = 8, TMA_WARP = 8, MMA_WARP = 9, THREADS = 320;
constexpr int TMEM_COLS = 512;
constexpr int SMEM_BYTES = SA * A_STAGE + SB * B_STAGE + 1024 /*alignment*/ + 256 /*barriers*/;

__device__ int g_prefill_status;  // non-zero: a bounded wait gave up (sticky, read by the host on demand)

// Byte offset of 16-byte chunk `c` of row `r` inside a swizzled (rows x 64 f16) tile.
__device__ __forceinline__ uint32_t swz(int r, int c) { return (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4)); }

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&h);
}
// four code bytes (each 0..63) -> four f16 weights w = code * s - m, as two packed registers
__device__ __forceinline__ void expand4(uint32_t bytes, float s, float m, uint32_t &o0, uint32_t &o1) {
  const float f0 = __uint_as_float(__byte_perm(bytes, 0x4B000000u, 0x7650)) - 8388608.f;
  const float f1 = __uint_as_float(__byte_perm(bytes, 0x4B000000u, 0x7651)) - 8388608.f;
  const float f2 = __uint_as_float(__byte_perm(bytes, 0x4B000000u, 0x7652)) - 8388608.f;
  const float f3 = __uint_as_float(__byte_perm(bytes, 0x4B000000u, 0x7653)) - 8388608.f;
  o0 = pack_h2(fmaf(f0, s, -m), fmaf(f1, s, -m));
  o1 = pack_h2(fmaf(f2, s, -m), fmaf(f3, s, -m));
}

// ---- per-format row expanders: one thread, one weight row, one 256-element block at a time.
// load(): fetch the block into registers.  step(j, ...): write the 64 weights k = 64j .. 64j+63 of
// the block as 8 swizzled 16-byte chunks of row `r` of the B tile at shared address `tile`.
struct Q4KRow {
  static constexpr int BLOCK_BYTES = 144, STEPS = 4;  // one load() = one 256-element block = 4 steps
  uint4 h, q[8];
  __device__ __forceinline__ void load(const uint8_t *row, int kb) {
    const uint4 *p = reinterpret_cast<const uint4 *>(row) + (size_t)kb * 9;
    h = __ldg(p);
#pragma unroll
    for (int i = 0; i < 8; i++) q[i] = __ldg(p + 1 + i);
  }
  __device__ __forceinline__ void step(int j, uint32_t tile, int r) const {
    // sub-blocks 2j (low nibbles of qs[32j .. 32j+31]) and 2j+1 (high nibbles)
    const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(&h.x));
    uint32_t sc0, mn0, sc1, mn1;
    if (j < 2) {
      sc0 = (h.y >> (16 * j)) & 63, sc1 = (h.y >> (16 * j + 8)) & 63;
      mn0 = (h.z >> (16 * j)) & 63, mn1 = (h.z >> (16 * j + 8)) & 63;
    } else {
      const int s = 16 * (j - 2);
      sc0 = ((h.w >> s) & 0xF) | (((h.y >> (s + 6)) & 3) << 4);
      sc1 = ((h.w >> (s + 8)) & 0xF) | (((h.y >> (s + 14)) & 3) << 4);
      mn0 = ((h.w >> (s + 4)) & 0xF) | (((h.z >> (s + 6)) & 3) << 4);
      mn1 = ((h.w >> (s + 12)) & 0xF) | (((h.z >> (s + 14)) & 3) << 4);
    }
    const float s0 = dd.x * (float)sc0, m0 = dd.y * (float)mn0, s1 = dd.x * (float)sc1, m1 = dd.y * (float)mn1;
    const uint32_t w[8] = {q[2 * j].x, q[2 * j].y, q[2 * j].z, q[2 * j].w, q[2 * j + 1].x, q[2 * j + 1].y, q[2 * j + 1].z, q[2 * j + 1].w};
#pragma unroll
    for (int c = 0; c < 4; c++) {  // chunk c: k = 8c..8c+7 (low nibbles); chunk c+4: k = 32+8c.. (high nibbles)
      uint4 lo, hi;
      expand4(w[2 * c] & 0x0F0F0F0Fu, s0, m0, lo.x, lo.y);
      expand4(w[2 * c + 1] & 0x0F0F0F0Fu, s0, m0, lo.z, lo.w);
      expand4((w[2 * c] >> 4) & 0x0F0F0F0Fu, s1, m1, hi.x, hi.y);
      expand4((w[2 * c + 1] >> 4) & 0x0F0F0F0Fu, s1, m1, hi.z, hi.w);
      asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(tile + swz(r, c)), "r"(lo.x), "r"(lo.y), "r"(lo.z), "r"(lo.w));
      asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(tile + swz(r, c + 4)), "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w));
    }
  }
};

// Q6_K (210 B): [ql[128] | qh[64] | int8 sc[16] | f16 d].  One load() fetches a 128-element half h:
// ql[64h .. 64h+63], qh[32h .. 32h+31], sc[8h .. 8h+7], d.  Step j (k = 64j .. 64j+63 of the half)
// covers groups q = 2j, 2j+1: code = (ql[64h + 32(q&1) + l] >> 4j) & 15 | ((qh[32h + l] >> 2q) & 3) << 4,
// weight = d * sc[8h + 4j + k/16] * (code - 32).  Blocks are only 2-byte aligned: each word is two
// aligned 32-bit loads funnel-shifted by 0 or 16 bits (rows start 4-byte aligned, checked on the host).
struct Q6KRow {
  static constexpr int BLOCK_BYTES = 210, STEPS = 2;
  uint32_t ql[16], qh[8], sc[2];
  float d;
  __device__ __forceinline__ static uint32_t ld(const uint32_t *a, uint32_t sh) {
    const uint32_t lo = __ldg(a);
    uint32_t hi = 0;
    if (sh) hi = __ldg(a + 1);
    return __funnelshift_r(lo, hi, sh);
  }
  __device__ __forceinline__ void load(const uint8_t *row, int unit) {
    const int b = unit >> 1, h = unit & 1;
    const uint32_t sh = (b & 1) * 16u;
    const uint8_t *blk = row + (size_t)b * 210;
    const uint32_t *a = reinterpret_cast<const uint32_t *>(blk - (b & 1) * 2);  // rounded down to 4 bytes
#pragma unroll
    for (int i = 0; i < 16; i++) ql[i] = ld(a + 16 * h + i, sh);
#pragma unroll
    for (int i = 0; i < 8; i++) qh[i] = ld(a + 32 + 8 * h + i, sh);
    sc[0] = ld(a + 48 + 2 * h, sh), sc[1] = ld(a + 49 + 2 * h, sh);
    d = f16_bits_to_f32(__ldg(reinterpret_cast<const uint16_t *>(blk + 208)));
  }
  __device__ __forceinline__ void step(int j, uint32_t tile, int r) const {
#pragma unroll
    for (int c = 0; c < 8; c++) {  // chunk c: k = 8c .. 8c+7 -> group q = 2j + c/4, l = 8 (c%4) ..
      const int q = 2 * j + (c >> 2), li = 2 * (c & 3);
      const float ds = d * (float)(int8_t)((sc[j] >> (8 * (c >> 1))) & 0xff);
      const float m = 32.f * ds;
      uint4 o;
#pragma unroll
      for (int e = 0; e < 2; e++) {
        const uint32_t wq = ql[8 * (c >> 2) + li + e] >> (4 * j), wh = qh[li + e];
        const uint32_t hi2 = q == 0 ? (wh << 4) : q == 1 ? (wh << 2) : q == 2 ? wh : (wh >> 2);
        const uint32_t v = (wq & 0x0F0F0F0Fu) | (hi2 & 0x30303030u);
        if (e == 0)
          expand4(v, ds, m, o.x, o.y);
        else
          expand4(v, ds, m, o.z, o.w);
      }
      asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(tile + swz(r, c)), "r"(o.x), "r"(o.y), "r"(o.z), "r"(o.w));
    }
  }
};

// ---- the kernel.  grid = (ceil(N / 256), ceil(M / 256)); 320 threads:
//   warps 0-7  expand weights (thread r <-> weight row n0 + r), then run the epilogue
//   warp  8    TMA producer of the x tiles (one lane)
//   warp  9    owns tensor memory and issues the MMAs (one lane)
template <typename Row>
__global__ void __launch_bounds__(THREADS, 1) gguf_prefill_umma_kernel(const __grid_constant__ CUtensorMap tmap_x,
                                                                      const uint8_t *__restrict__ w,
                                                                      float *__restrict__ out, int M, int N, int K) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sA = base, sB = base + SA * A_STAGE, sBar = sB + SB * B_STAGE;
  // barriers: a_full[SA] a_empty[SA] b_full[SB] b_empty[SB] d_full, then the TMEM address word
  const uint32_t a_full = sBar, a_empty = sBar + 8 * SA, b_full = sBar + 16 * SA, b_empty = b_full + 8 * SB,
                 d_full = b_empty + 8 * SB, tmem_slot = d_full + 8;
  __shared__ int abort_flag;
  __shared__ uint32_t tmem_base_sh;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BN, m0 = blockIdx.y * BM;
  const int nkb = K / BK;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int i = 0; i < SA; i++) mbar_init(a_full + 8 * i, 1), mbar_init(a_empty + 8 * i, 1);
    for (int i = 0; i < SB; i++) mbar_init(b_full + 8 * i, NUM_DEQ_WARPS), mbar_init(b_empty + 8 * i, 1);
    mbar_init(d_full, 1);
    fence_barrier_init();
  }
  if (warp == MMA_WARP) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (threadIdx.x == 0) {
    uint32_t t;
    asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(t) : "r"(tmem_slot));
    tmem_base_sh = t;
  }
  __syncthreads();
  const uint32_t tmem_base = tmem_base_sh;
  volatile int *abort = &abort_flag;

  if (warp == TMA_WARP) {
    if (lane == 0) {
      prefetch_tmap(&tmap_x);
      int issued = 0;
      for (int kb = 0; kb < nkb; kb++) {
        const int s = kb % SA;
        if (kb >= SA && !mbar_wait(a_empty + 8 * s, ((kb / SA) - 1) & 1, abort)) break;
        mbar_arrive_expect_tx(a_full + 8 * s, A_STAGE);
        tma_load_2d(sA + s * A_STAGE, &tmap_x, a_full + 8 * s, kb * BK, m0);
        tma_load_2d(sA + s * A_STAGE + A_STAGE / 2, &tmap_x, a_full + 8 * s, kb * BK, m0 + 128);
        issued = kb + 1;
      }
      if (*abort)  // give the loads still in flight a bounded time to land before the CTA retires
        for (int kb = issued > SA ? issued - SA : 0; kb < issued; kb++)
          for (int i = 0; i < (1 << 14) && !mbar_try_wait(a_full + 8 * (kb % SA), (kb / SA) & 1); i++) {
          }
    }
  } else if (warp == MMA_WARP) {
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_f16(128, BN, false);
      for (int kb = 0; kb < nkb; kb++) {
        const int sa = kb % SA, sb = kb % SB;
        if (!mbar_wait(a_full + 8 * sa, (kb / SA) & 1, abort)) break;
        if (!mbar_wait(b_full + 8 * sb, (kb / SB) & 1, abort)) break;
        tc_fence_after();
#pragma unroll
        for (int k4 = 0; k4 < BK / 16; k4++) {
          const uint64_t bd = smem_desc_sw128(sB + sb * B_STAGE + k4 * 32);
          const uint64_t a0 = smem_desc_sw128(sA + sa * A_STAGE + k4 * 32);
          const uint64_t a1 = smem_desc_sw128(sA + sa * A_STAGE + A_STAGE / 2 + k4 * 32);
          const uint32_t acc = (kb | k4) ? 1u : 0u;
          mma_f16(tmem_base, a0, bd, idesc, acc);
          mma_f16(tmem_base + 256, a1, bd, idesc, acc);
        }
        mma_commit(a_empty + 8 * sa);
        mma_commit(b_empty + 8 * sb);
      }
      mma_commit(d_full);
    }
  } else {
    // ---- weight expansion: thread r owns row n0 + r (clamped; rows past N are never stored)
    const int r = threadIdx.x;
    const int n = min(n0 + r, N - 1);
    const uint8_t *row = w + (size_t)n * (size_t)(K / 256) * Row::BLOCK_BYTES;
    Row cur;
    cur.load(row, 0);
    bool ok = true;
    const int units = K / (BK * Row::STEPS);
    for (int u = 0; u < units && ok; u++) {
      Row nxt;
      if (u + 1 < units) nxt.load(row, u + 1);
#pragma unroll
      for (int j = 0; j < Row::STEPS; j++) {
        const int kb = u * Row::STEPS + j, s = kb % SB;
        if (kb >= SB) {  // lane 0 waits for the stage to be free, the warp follows its verdict
          int got = 1;
          if (lane == 0) got = mbar_wait(b_empty + 8 * s, ((kb / SB) - 1) & 1, abort);
          if (!__shfl_sync(0xffffffffu, got, 0)) {
            ok = false;
            break;
          }
        }
        cur.step(j, sB + s * B_STAGE, r);
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(b_full + 8 * s);
      }
      cur = nxt;
    }
    // ---- epilogue: warp w reads TMEM lanes 32 (w % 4) .. +31 (tokens) and columns 128 (w / 4) .. +127
    int done = 0;
    if (ok && lane == 0) done = mbar_wait(d_full, 0, abort);
    if (__shfl_sync(0xffffffffu, done, 0)) {
      tc_fence_after();
      const int quad = warp & 3, chalf = warp >> 2;
#pragma unroll 1
      for (int a = 0; a < 2; a++) {
        const int m = m0 + a * 128 + quad * 32 + lane;
#pragma unroll 1
        for (int c = 0; c < 4; c++) {
          uint32_t v[32];
          tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + a * 256 + chalf * 128 + c * 32, v);
          tmem_ld_wait();
          const int nc = n0 + chalf * 128 + c * 32;
          if (m < M) {
            float *o = out + (size_t)m * N + nc;
            if (nc + 32 <= N && (N & 3) == 0) {
#pragma unroll
              for (int i = 0; i < 8; i++)
                reinterpret_cast<float4 *>(o)[i] = make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                                                               __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
            } else {
#pragma unroll
              for (int i = 0; i < 32; i++)
                if (nc + i < N) o[i] = __uint_as_float(v[i]);
            }
          }
        }
      }
    }
  }
  if (abort_flag && threadIdx.x == 0) g_prefill_status = 1;
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) tmem_dealloc(tmem_base, TMEM_COLS);
}

// x f32 (M, K) -> f16, clamped to the f16 range so that an outlier cannot become an infinity
__global__ void __launch_bounds__(256) x_to_f16_kernel(const float4 *__restrict__ x, uint2 *__restrict__ y, long long n4) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 v = __ldg(x + i);
    v.x = fminf(fmaxf(v.x, -65504.f), 65504.f), v.y = fminf(fmaxf(v.y, -65504.f), 65504.f);
    v.z = fminf(fmaxf(v.z, -65504.f), 65504.f), v.w = fminf(fmaxf(v.w, -65504.f), 65504.f);
    y[i] = make_uint2(pack_h2(v.x, v.y), pack_h2(v.z, v.w));
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
std::mutex g_mu;
struct Workspace {
  void *ptr;
  size_t bytes;
} g_ws[64];

int ensure_encode() {
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_encode) return 0;
  void *fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
  if (e != cudaSuccess || !fn || q != cudaDriverEntryPointSuccess)
    return fail(e == cudaSuccess ? LB200_E_DEVICE : (int)e, "light_b200: cuTensorMapEncodeTiled is not available from the driver");
  g_encode = (EncodeTiledFn)fn;
  return 0;
}

template <typename Row>
int launch(const float *x, const void *w, float *out, int M, int N, int K, void *ws, cudaStream_t st) {
  if (int rc = ensure_encode()) return rc;
  const long long n4 = (long long)M * K / 4;
  long long blocks = (n4 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  x_to_f16_kernel<<<(unsigned)blocks, 256, 0, st>>>((const float4 *)x, (uint2 *)ws, n4);
  if (int rc = launched("matmul_q (prefill, x to f16)")) return rc;
  CUtensorMap tm;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {BK, 128};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(&tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, ws, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(LB200_E_SHAPE, "light_b200: matmul_q (prefill): cuTensorMapEncodeTiled failed (%d)", (int)r);
  auto kern = gguf_prefill_umma_kernel<Row>;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return fail((int)e, "light_b200: matmul_q (prefill): %s", cudaGetErrorString(e));
    attr_done = true;
  }
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  kern<<<grid, THREADS, SMEM_BYTES, st>>>(tm, (const uint8_t *)w, out, M, N, K);
  return launched("matmul_q (prefill)");
}

}  // namespace

int set_workspace(int device, void *ptr, size_t bytes) {
  if (device < 0 || device >= 64) return fail(LB200_E_DEVICE, "light_b200: device ordinal %d out of range", device);
  if (((uintptr_t)ptr & 1023) != 0) return fail(LB200_E_ALIGN, "light_b200: workspace must be 1024-byte aligned");
  std::lock_guard<std::mutex> lk(g_mu);
  g_ws[device] = {ptr, ptr ? bytes : 0};
  return 0;
}

// returns 1 when the tensor-core prefill kernel took the call, 0 when the shape is not covered
int gguf_prefill(int type, const float *x, const void *w, float *out, int M, int N, int K, int device, cudaStream_t st) {
  if (M < 65 || K % 256) return 0;
  if (type == LB200_Q4_K) {
    if ((uintptr_t)w & 15) return 0;
  } else if (type == LB200_Q6_K) {
    if (((uintptr_t)w & 3) || ((size_t)(K >> 8) * 210) % 4) return 0;  // rows must start 4-byte aligned
  } else {
    return 0;
  }
  Workspace ws;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    ws = g_ws[device];
  }
  if (!ws.ptr || ws.bytes < (size_t)M * K * 2) return 0;
  int rc = type == LB200_Q4_K ? launch<Q4KRow>(x, w, out, M, N, K, ws.ptr, st) : launch<Q6KRow>(x, w, out, M, N, K, ws.ptr, st);
  return rc ? rc : 1;
}

int prefill_status(int device) {
  (void)device;
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_prefill_status, sizeof(int));
  return e == cudaSuccess ? v : -(int)e;
}

}  // namespace lb
