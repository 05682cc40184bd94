// Batched decode (2 .. 64 activation rows) for every packed weight format, on the 5th-generation
// tensor cores: out (M, N) = x (M, K) . dequant(W (N, K))^T, bound by the one pass over the weights.
//
// The operands are swapped with respect to the prefill kernel: the WEIGHT rows are the M = 128 side
// of tcgen05.mma and the few tokens its N side (16, 32 or 64 columns), so the tensor-core time is
// proportional to the token count and stays below the time to expand the weights.
//
//   * grid = (ceil(N / 128), KS), launched as clusters of KS CTAs along y: the CTAs of a cluster
//     share 128 weight rows and split K into KS contiguous runs of 256-element blocks, which is
//     what gives a small matrix (N = 1024 .. 4096) enough CTAs to fill 148 SMs;
//   * 256 threads, two per weight row (each takes half of every 64-k step: the step is a chain of
//     dependent instructions, so halving it and doubling the warps both shorten it), expand the
//     packed codes into the A tile (128 rows x 64 k, 128-byte swizzle) with the row expanders the
//     prefill kernel uses, and convert the matching 64 k of the activations straight from global
//     memory into the B tile (tokens x 64 k) -- no pre-pass over x, no workspace;
//   * one thread issues tcgen05.mma (M 128, N = tokens, K 16) into a 128 x tokens f32 accumulator
//     in tensor memory; mbarriers track full / free stages (4-deep ring);
//   * each CTA parks its partial sums in its own shared memory, the cluster meets at a hardware
//     barrier, and CTA r adds up rows 128 r / KS .. of all KS partials through distributed shared
//     memory and stores them: the result is deterministic, and no partial sum touches HBM.
//
// Every mbarrier wait is bounded in time; a wait that gives up sets a sticky status word and lets
// the CTA run to its cluster barriers and retire.
#include <cuda.h>

#include <cstdlib>
#include <type_traits>

#include "common.cuh"
#include "mma_sync.cuh"
#include "row_expand.cuh"
#include "umma.cuh"

namespace lb {

namespace {

using namespace umma;

constexpr int DM = 128;  // weight rows per CTA (MMA M)
constexpr int DK = 64;   // k per stage
constexpr int SMEM_PER_CTA = 112 * 1024;  // two CTAs per SM
constexpr int D_EXP_WARPS = 8, D_MMA_WARP = 8, D_THREADS = 288;  // two expander threads per weight row
constexpr int W_TILE = DM * DK * 2;

template <typename Row, int NTOK>
struct DCfg {
  static constexpr int X_TILE = NTOK * DK * 2 < 1024 ? 1024 : NTOK * DK * 2;
  static constexpr int STAGE = W_TILE + ((X_TILE + 1023) / 1024) * 1024;
  static constexpr int RAW_SLOT = DM * Row::RAW_PITCH;           // one 256-element block of all 128 rows, packed
  static constexpr int RS = 2;                                   // blocks in flight
  static constexpr int RAW_BYTES = ((RS * RAW_SLOT + 1023) / 1024) * 1024;
  // operand stages: as many as fit beside the raw ring (4 at most, 2 at least)
  static constexpr int FIT = (SMEM_PER_CTA - 1280 - RAW_BYTES) / STAGE;
  static constexpr int DST = FIT >= 4 ? 4 : FIT >= 3 ? 3 : 2;
  static constexpr int RAW_OFF = DST * STAGE;
  static constexpr int BAR_OFF = RAW_OFF + RAW_BYTES;
  static constexpr int SMEM = BAR_OFF + 1024 /*alignment*/ + 256 /*barriers*/;
  static constexpr int TCOLS = NTOK < 32 ? 32 : NTOK;
  static_assert(DM * NTOK * 4 <= DST * STAGE, "the partial sums reuse the stage memory");
};

__device__ int g_decode_status;  // non-zero: a bounded wait gave up (sticky, read by the host on demand)

// 16-byte read-only load that stays where it is written (the compiler may not sink it to its use:
// the activations of the next k-step are requested a whole step ahead)
__device__ __forceinline__ uint4 ldg_here(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
// 8 consecutive activations k0 .. k0+7 of one token, as loaded -> one 16-byte chunk of operand values
template <typename XT>
struct XRaw;
template <>
struct XRaw<float> {
  uint4 a, b;
  __device__ __forceinline__ void zero() { a = b = make_uint4(0, 0, 0, 0); }
  __device__ __forceinline__ void load(const float *p) { a = ldg_here(p), b = ldg_here(p + 4); }
  template <bool PERM>
  __device__ __forceinline__ uint4 chunk() const {
    auto f = [](uint32_t u) { return fminf(fmaxf(__uint_as_float(u), -65504.f), 65504.f); };
    return PERM ? make_uint4(pack_h2(f(a.x), f(a.z)), pack_h2(f(a.y), f(a.w)), pack_h2(f(b.x), f(b.z)), pack_h2(f(b.y), f(b.w)))
                : make_uint4(pack_h2(f(a.x), f(a.y)), pack_h2(f(a.z), f(a.w)), pack_h2(f(b.x), f(b.y)), pack_h2(f(b.z), f(b.w)));
  }
};
template <>
struct XRaw<__nv_bfloat16> {
  uint4 a;
  __device__ __forceinline__ void zero() { a = make_uint4(0, 0, 0, 0); }
  __device__ __forceinline__ void load(const __nv_bfloat16 *p) { a = ldg_here(p); }
  template <bool PERM>
  __device__ __forceinline__ uint4 chunk() const { return a; }
};

__device__ __forceinline__ void st_out(float *o, float v) { *o = v; }
__device__ __forceinline__ void st_out(__nv_bfloat16 *o, float v) { *o = __float2bfloat16_rn(v); }

template <typename Row, int NTOK, typename XT, typename OutT>
__global__ void __launch_bounds__(D_THREADS, 2) decode_umma_kernel(const typename Row::Ctx ctx, const XT *__restrict__ x,
                                                                OutT *__restrict__ out, int M, int N, int K) {
  using Cfg = DCfg<Row, NTOK>;
  constexpr int DST = Cfg::DST;
  constexpr bool BF16 = std::is_same<XT, __nv_bfloat16>::value;
  constexpr bool PERM = Row::KPERM && !BF16;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sBar = base + Cfg::BAR_OFF, sRaw = base + Cfg::RAW_OFF;
  const uint32_t full = sBar, empty = sBar + 8 * DST, d_full = empty + 8 * DST, tmem_slot = d_full + 8;
  __shared__ int abort_flag;
  __shared__ uint32_t tmem_base_sh;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * DM;
  const int KS = gridDim.y, rank = blockIdx.y;  // cluster = all CTAs of one blockIdx.x
  // this CTA's run of 256-element blocks, as k-steps of 64
  const int nblk = K >> 8;
  const int kb0 = (nblk * rank / KS) * 4, kb1 = (nblk * (rank + 1) / KS) * 4, nk = kb1 - kb0;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int i = 0; i < DST; i++) mbar_init(full + 8 * i, D_EXP_WARPS), mbar_init(empty + 8 * i, 1);
    mbar_init(d_full, 1);
    fence_barrier_init();
  }
  if (warp == D_MMA_WARP) {
    tmem_alloc(tmem_slot, Cfg::TCOLS);
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

  if (warp == D_MMA_WARP) {
    if (lane == 0 && nk > 0) {
      constexpr uint32_t idesc = idesc_f16(DM, NTOK, BF16);
      for (int kb = 0; kb < nk; kb++) {
        const int s = kb % DST;
        if (!mbar_wait(full + 8 * s, (kb / DST) & 1, abort)) break;
        tc_fence_after();
        const uint32_t sW = base + s * Cfg::STAGE, sX = sW + W_TILE;
#pragma unroll
        for (int k4 = 0; k4 < DK / 16; k4++)
          mma_f16(tmem_base, smem_desc_sw128(sW + k4 * 32), smem_desc_sw128(sX + k4 * 32), idesc, (kb | k4) ? 1u : 0u);
        mma_commit(empty + 8 * s);
      }
      mma_commit(d_full);
    }
  } else {
    // ---- threads r and r + 128: weight row n0 + r (clamped; rows past N are never stored), chunks
    // 0-3 and 4-7 of every step, and a share of the x tile each
    const int r = threadIdx.x & (DM - 1), part = threadIdx.x >> 7;
    Row cur;
    cur.init(ctx, 0, min(n0 + r, N - 1), N, K);
    constexpr int UPB = 4 / Row::STEPS;  // load units per 256-element block
    const int b0 = kb0 / 4, b1 = kb1 / 4;
    // The packed blocks come in through a ring of shared memory, copied 16 bytes per lane with the
    // 9 .. 16 lanes of a half-warp on one row (coalesced), Cfg::RS blocks ahead of their use; a
    // thread then reads its own row's slot.  (One thread per row reading global memory directly
    // touches 32 lines per load instruction and is bound by the load unit, not by HBM.)
    const int c_row = warp * 16 + (lane >> 4) * 8, c_piece = lane & 15;  // rows c_row + i, i = 0..7
    const size_t row_stride = Row::row_stride(ctx, K);
    const bool c_clamp = n0 + DM > N;  // the last rows of the matrix: rows past N re-read row N - 1
    Row c_first;                       // row c_row of this CTA: the other seven are a fixed stride below it
    c_first.init(ctx, 0, min(n0 + c_row, N - 1), N, K);
    int i_b = b0;
    auto issue = [&]() {  // always closes a commit group, so that group counts stay uniform
      if (i_b < b1 && c_piece < Row::RAW_G) {
        const uint32_t slot = sRaw + (uint32_t)((i_b - b0) % Cfg::RS) * Cfg::RAW_SLOT;
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const int di = c_clamp ? min(i, max(N - 1 - (n0 + c_row), 0)) : i;
          // (granule-aligned like raw_src itself: the stride is added before the alignment)
          const uint8_t *src = reinterpret_cast<const uint8_t *>(
                                   (uintptr_t)(c_first.raw_src_unaligned(i_b) + (size_t)di * row_stride) & ~(uintptr_t)15) + c_piece * 16;
          const uint32_t dst = slot + (uint32_t)(c_row + i) * Row::RAW_PITCH + c_piece * 16;
          const uint8_t *lim = c_first.raw_end();
          if (lim == nullptr || src + 16 <= lim)
            cp_async16(dst, src);
          else if (src < lim)
            cp_async16_part(dst, src, (uint32_t)(lim - src));
          if constexpr (Row::RAW_G > 16) {  // a 17th granule (Q8_0: 272 bytes): the first lanes copy it too
            static_assert(Row::RAW_G <= 32, "two granules per lane at most");
            if (c_piece < Row::RAW_G - 16) cp_async16(dst + 256, src + 256);
          }
        }
      }
      i_b++;
      cp_async_commit();
    };
    auto expanders_sync = [] { asm volatile("bar.sync 1, %0;\n" ::"n"(D_EXP_WARPS * 32) : "memory"); };
#pragma unroll 1
    for (int p = 0; p < Cfg::RS; p++) issue();
    bool ok = true;
    constexpr int XT_THREADS = D_EXP_WARPS * 32;
    constexpr int XTASKS = (NTOK * 8 + XT_THREADS - 1) / XT_THREADS;  // 16-byte chunks of the x tile per thread
    XRaw<XT> xr[XTASKS];  // this thread's share of the NEXT k-step's activations, in flight
    auto x_request = [&](int kg) {
#pragma unroll
      for (int i = 0; i < XTASKS; i++) {
        const int q = (int)threadIdx.x + XT_THREADS * i, tok = q >> 3, ch = q & 7;
        xr[i].zero();
        if (q < NTOK * 8 && tok < M) xr[i].load(x + (size_t)tok * K + kg * DK + ch * 8);
      }
    };
    if (nk > 0) x_request(kb0);
    for (int b = b0; b < b1; b++) {  // (after a failed wait the loop still runs: the barriers below count every warp)
      cp_async_wait<Cfg::RS - 1>();  // this thread's granules of block b have landed ...
      expanders_sync();              // ... and so have everybody else's
      const uint32_t slot = sRaw + (uint32_t)((b - b0) % Cfg::RS) * Cfg::RAW_SLOT + (uint32_t)r * Row::RAW_PITCH;
#pragma unroll
      for (int uu = 0; uu < UPB; uu++) {
        const int u = b * UPB + uu;
        cur.load_smem(slot, u);
        if (uu == UPB - 1) {
          expanders_sync();  // every row of the slot has been read: it can take block b + RS
          issue();
        }
#pragma unroll
        for (int j = 0; j < Row::STEPS; j++) {
          const int kg = u * Row::STEPS + j, kb = kg - kb0, s = kb % DST;  // global / local k-step
          uint4 xc[XTASKS];
#pragma unroll
          for (int i = 0; i < XTASKS; i++) xc[i] = xr[i].template chunk<PERM>();
          if (kg + 1 < kb1) x_request(kg + 1);
          if (kb >= DST && ok) {  // lane 0 waits for the stage to be free, the warp follows its verdict
            int got = 1;
            if (lane == 0) got = mbar_wait(empty + 8 * s, ((kb / DST) - 1) & 1, abort);
            if (!__shfl_sync(0xffffffffu, got, 0)) ok = false;
          }
          if (ok) {
            const uint32_t sW = base + s * Cfg::STAGE, sX = sW + W_TILE;
            if (part)
              cur.template step<BF16, 1>(j, sW, r);
            else
              cur.template step<BF16, 0>(j, sW, r);
#pragma unroll
            for (int i = 0; i < XTASKS; i++) {
              const int q = (int)threadIdx.x + XT_THREADS * i;
              if (q < NTOK * 8) st_chunk(sX + swz(q >> 3, q & 7), xc[i]);
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(full + 8 * s);
          }
        }
      }
    }
    cp_async_wait<0>();
    // ---- accumulator -> partial[token][row] in this CTA's shared memory (the stages are idle now)
    int done = 0;
    if (ok && lane == 0) done = nk > 0 ? (int)mbar_wait(d_full, 0, abort) : 1;
    done = __shfl_sync(0xffffffffu, done, 0);
    if (done) tc_fence_after();
    // warps 0-3 read the first half of the token columns of their 32 rows, warps 4-7 the second
    constexpr int CPW = NTOK >= 32 ? NTOK / 2 : NTOK;  // columns per warp
    if (NTOK >= 32 || part == 0) {
#pragma unroll 1
      for (int c = (NTOK >= 32 ? part * CPW : 0); c < (NTOK >= 32 ? part * CPW : 0) + CPW; c += 16) {
        uint32_t v[16];
#pragma unroll
        for (int i = 0; i < 16; i++) v[i] = 0u;
        if (done && nk > 0) {
          tmem_ld16(tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + c, v);
          tmem_ld_wait();
        }
#pragma unroll
        for (int i = 0; i < 16; i++)
          asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(base + (uint32_t)((c + i) * DM + r) * 4u), "r"(v[i]));
      }
    }
  }
  __syncwarp();
  if (abort_flag && threadIdx.x == 0) g_decode_status = 1;
  tc_fence_before();
  // ---- add up the cluster's partials: CTA `rank` owns rows rank * 128 / KS ..
  if (KS > 1) cluster_sync(); else __syncthreads();
  {
    const int rows_per = DM / KS;
    for (int idx = threadIdx.x; idx < rows_per * NTOK; idx += D_THREADS) {
      const int tok = idx / rows_per, row = rank * rows_per + idx % rows_per;
      const uint32_t a = base + (uint32_t)(tok * DM + row) * 4u;
      float v = 0.f;
      if (KS > 1) {
        for (int p = 0; p < KS; p++) v += ld_cluster_f32(map_to_rank(a, (uint32_t)p));
      } else {
        asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(v) : "r"(a));
      }
      if (tok < M && n0 + row < N) st_out(out + (size_t)tok * N + n0 + row, v);
    }
  }
  if (KS > 1) cluster_sync(); else __syncthreads();  // nobody leaves while a peer still reads its partials
  if (warp == D_MMA_WARP) tmem_dealloc(tmem_base, Cfg::TCOLS);
}

template <typename Row, int NTOK, typename XT, typename OutT>
int launch_decode(const typename Row::Ctx &ctx, const XT *x, OutT *out, int M, int N, int K, int sms, cudaStream_t st) {
  auto kern = decode_umma_kernel<Row, NTOK, XT, OutT>;
  static DeviceOnce attr_done;
  {
    cudaError_t e = attr_done.ensure([&] { return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, DCfg<Row, NTOK>::SMEM); });
    if (e != cudaSuccess) return fail((int)e, "light_b200: decode (tcgen05): %s", cudaGetErrorString(e));
  }
  // K split: the smallest cluster that gives every SM two CTAs, at most 8 and at most one per block
  const int nx = (N + DM - 1) / DM, nblk = K >> 8;
  int ks = 1;
  while (ks < 8 && ks * 2 <= nblk && nx * ks < 2 * sms) ks *= 2;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)nx, (unsigned)ks, 1);
  cfg.blockDim = dim3(D_THREADS);
  cfg.dynamicSmemBytes = DCfg<Row, NTOK>::SMEM;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1, attr[0].val.clusterDim.y = (unsigned)ks, attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, ctx, x, out, M, N, K);
  if (e != cudaSuccess) return fail((int)e, "light_b200: decode (tcgen05): %s", cudaGetErrorString(e));
  return launched("decode (tcgen05)");
}

template <typename Row, typename XT, typename OutT>
int launch_by_tokens(const typename Row::Ctx &ctx, const XT *x, OutT *out, int M, int N, int K, int sms, cudaStream_t st) {
  if (M <= 16) return launch_decode<Row, 16, XT, OutT>(ctx, x, out, M, N, K, sms, st);
  if (M <= 32) return launch_decode<Row, 32, XT, OutT>(ctx, x, out, M, N, K, sms, st);
  return launch_decode<Row, 64, XT, OutT>(ctx, x, out, M, N, K, sms, st);
}

template <typename Row>
int launch_by_act(const typename Row::Ctx &ctx, const void *x, void *out, int act_dtype, int M, int N, int K, int sms,
                  cudaStream_t st) {
  if (act_dtype == LB200_F32) return launch_by_tokens<Row, float, float>(ctx, (const float *)x, (float *)out, M, N, K, sms, st);
  if constexpr (!Row::KPERM)
    return launch_by_tokens<Row, __nv_bfloat16, __nv_bfloat16>(ctx, (const __nv_bfloat16 *)x, (__nv_bfloat16 *)out, M, N, K, sms, st);
  return LB200_E_DTYPE;
}

int g_sm_count[64];
int sm_count(int device) {
  if (!g_sm_count[device]) {
    int v = 148;
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, device);
    g_sm_count[device] = v;
  }
  return g_sm_count[device];
}

constexpr int DECODE_MAX_M = 64;
// Token counts from which this kernel is the fastest one measured (below it the register-fed
// kernels win); LIGHT_B200_DECODE_MIN_M overrides both (tuning knob).
int g_min_m_gguf = 17, g_min_m_other = 1, g_min_m_q80 = 2;  // LIGHT_B200_DECODE_MIN_M / _MIN_M_Q80 (tuning knobs)
bool g_knobs_read = false;
void read_knobs() {
  if (g_knobs_read) return;
  if (const char *e = getenv("LIGHT_B200_DECODE_MIN_M")) g_min_m_gguf = g_min_m_other = atoi(e);
  if (const char *e = getenv("LIGHT_B200_DECODE_MIN_M_Q80")) g_min_m_q80 = atoi(e) < 1 ? 1 : atoi(e);
  g_knobs_read = true;
}

}  // namespace

int decode_umma_status() {
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_decode_status, sizeof(int));
  return e == cudaSuccess ? v : -(int)e;
}

// Each returns 1 when it launched, 0 when the shape is not covered (the caller falls through to
// its other kernels), other values are errors.
int gguf_decode_umma(int type, const float *x, const void *w, float *out, int M, int N, int K, int device, cudaStream_t st) {
  read_knobs();
  if (M > DECODE_MAX_M || K % 256 || ((uintptr_t)x & 15)) return 0;
  if (M < (type == LB200_Q8_0 ? g_min_m_q80 : (g_min_m_gguf < 2 ? 2 : g_min_m_gguf))) return 0;
  GgufCtx ctx{(const uint8_t *)w};
  int rc;
  if (type == LB200_Q8_0) {  // no register-fed decode kernel exists for this format: every token count down to g_min_m_q80
    if ((uintptr_t)w & 15) return 0;
    rc = launch_by_act<Q80Row>(ctx, x, out, LB200_F32, M, N, K, sm_count(device), st);
  } else if (type == LB200_Q4_K) {
    if ((uintptr_t)w & 15) return 0;
    rc = launch_by_act<Q4KRow>(ctx, x, out, LB200_F32, M, N, K, sm_count(device), st);
  } else if (type == LB200_Q6_K) {
    if (((uintptr_t)w & 3) || ((size_t)(K >> 8) * 210) % 4) return 0;  // rows must start 4-byte aligned
    rc = launch_by_act<Q6KRow>(ctx, x, out, LB200_F32, M, N, K, sm_count(device), st);
  } else {
    return 0;
  }
  return rc ? rc : 1;
}

int int4_decode_umma(const void *x, const uint32_t *codes, const float *s, const float *z, void *y, int act_dtype, int M, int N,
                     int K, int G, int device, cudaStream_t st) {
  // f32 activations keep the CUDA-core kernel, whose f32 weights meet the reference's 1e-4 bound for that type
  read_knobs();
  if (act_dtype != LB200_BF16 || M < g_min_m_other || M > DECODE_MAX_M || K % 256 || G % 64 || ((uintptr_t)codes & 15) || ((uintptr_t)x & 15)) return 0;
  Int4Ctx ctx{codes, s, z, G};
  const int rc = launch_by_act<Int4Row>(ctx, x, y, act_dtype, M, N, K, sm_count(device), st);
  return rc ? rc : 1;
}

int fp8_decode_umma(const void *x, const uint8_t *w, const float *scale, void *y, int act_dtype, int M, int N, int K, int bR,
                    int bC, int device, cudaStream_t st) {
  read_knobs();
  if (act_dtype != LB200_BF16 || M < g_min_m_other || M > DECODE_MAX_M || K % 256 || bC % 64 || ((uintptr_t)w & 15) || ((uintptr_t)x & 15)) return 0;
  Fp8Ctx ctx{w, scale, bR, bC};
  const int rc = launch_by_act<Fp8Row>(ctx, x, y, act_dtype, M, N, K, sm_count(device), st);
  return rc ? rc : 1;
}

}  // namespace lb
