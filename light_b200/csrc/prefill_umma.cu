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
// Two kernels share this pipeline: prefill_umma_kernel, one tile per CTA (optionally a cluster split of K), and
// prefill_sk_kernel, one persistent CTA per SM over an even split of all (tile, K block) pairs; launch() picks.
//
// f16 (not bf16) operands: the reference multiplies f32 weights by f32 activations; rounding the
// weights to bf16 alone costs 1.7e-3 relative L2, to f16 2e-4.
#include <cuda.h>
#include <cuda_fp8.h>

#include <cstdlib>
#include <mutex>
#include <type_traits>

#include <vector>

#include "common.cuh"
#include "mma_sync.cuh"
#include "row_expand.cuh"
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

// Grouped (mixture-of-experts) mode: the token rows of the A operand have been gathered into expert
// order, expert e owns rows offsets[e] .. offsets[e+1] of it; output row i goes to pair sorted_pairs[i],
// scaled by its routing weight.  offsets == nullptr selects the plain (one weight) mode.
struct Group {
  const int32_t *offsets;
  const int64_t *pairs;
  const float *topkw;
  long long size_m;
  int E;
};

template <typename OutT>
__device__ __forceinline__ void sk_store32(uint32_t (&v)[32], OutT *__restrict__ out, long long m, int N, int nc, float wgt, bool weighted) {
  if (weighted) {
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = __float_as_uint(__uint_as_float(v[i]) * wgt);
  }
  OutT *o = out + (size_t)m * N + nc;
  if (nc + 32 <= N && (N & 7) == 0) {
    if constexpr (sizeof(OutT) == 4) {
#pragma unroll
      for (int i = 0; i < 8; i++)
        reinterpret_cast<float4 *>(o)[i] =
            make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]), __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
    } else {
#pragma unroll
      for (int i = 0; i < 4; i++)
        reinterpret_cast<uint4 *>(o)[i] = make_uint4(pack2<true>(__uint_as_float(v[8 * i]), __uint_as_float(v[8 * i + 1])),
                                                     pack2<true>(__uint_as_float(v[8 * i + 2]), __uint_as_float(v[8 * i + 3])),
                                                     pack2<true>(__uint_as_float(v[8 * i + 4]), __uint_as_float(v[8 * i + 5])),
                                                     pack2<true>(__uint_as_float(v[8 * i + 6]), __uint_as_float(v[8 * i + 7])));
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; i++)
      if (nc + i < N) st_act(o, i, __uint_as_float(v[i]));
  }
}

// 32 columns of one output row per thread (row m of the thread, dead rows skipped) -> global memory.  Through shared
// memory, so that a store instruction writes whole 128-byte lines: the thread holds 32 columns of ONE token row, and rows
// are N elements apart.  `stage` is 4 KB of shared memory that only this warp uses during an epilogue: the part of weight
// stage 0 that it alone writes as an expander (its 32 rows of 128 bytes; the stage's last MMA has completed, and the warp
// expands again only after its epilogue).  16-byte chunks are XOR-swizzled by the row.  All 32 lanes must call.
template <typename OutT>
__device__ __forceinline__ void tile_store32(uint32_t (&v)[32], uint32_t stage, int lane, long long m, bool live, float wgt, bool weighted,
                                             OutT *__restrict__ out, int N, int nc) {
  if (nc + 32 <= N && (N & 7) == 0) {
    constexpr int ROWB = 32 * (int)sizeof(OutT), LPR = ROWB / 16, RPI = 32 / LPR;
    auto sw = [](int row) { return sizeof(OutT) == 4 ? (row & 7) : ((row >> 1) & 3); };
    if (weighted) {
#pragma unroll
      for (int i = 0; i < 32; i++) v[i] = __float_as_uint(__uint_as_float(v[i]) * wgt);
    }
    if constexpr (sizeof(OutT) == 4) {
#pragma unroll
      for (int i = 0; i < 8; i++) st_chunk(stage + lane * ROWB + 16 * (i ^ sw(lane)), make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]));
    } else {
#pragma unroll
      for (int i = 0; i < 4; i++)
        st_chunk(stage + lane * ROWB + 16 * (i ^ sw(lane)),
                 make_uint4(pack2<true>(__uint_as_float(v[8 * i]), __uint_as_float(v[8 * i + 1])),
                            pack2<true>(__uint_as_float(v[8 * i + 2]), __uint_as_float(v[8 * i + 3])),
                            pack2<true>(__uint_as_float(v[8 * i + 4]), __uint_as_float(v[8 * i + 5])),
                            pack2<true>(__uint_as_float(v[8 * i + 6]), __uint_as_float(v[8 * i + 7]))));
    }
    __syncwarp();
#pragma unroll
    for (int g = 0; g < 32 / RPI; g++) {
      const int row = g * RPI + lane / LPR, q = lane % LPR;
      const long long mr = __shfl_sync(0xffffffffu, m, row);
      const int lr = __shfl_sync(0xffffffffu, (int)live, row);
      const uint4 w = lds128(stage + row * ROWB + 16 * (q ^ sw(row)));
      if (lr) *reinterpret_cast<uint4 *>(reinterpret_cast<char *>(out + (size_t)mr * N + nc) + 16 * q) = w;
    }
    __syncwarp();
  } else if (live) {
    sk_store32<OutT>(v, out, m, N, nc, wgt, weighted);
  }
}

// ---- the kernel.  grid = (ceil(N / 256), ceil(M / 256)); 320 threads:
//   warps 0-7  expand weights (thread r <-> weight row n0 + r), then run the epilogue
//   warp  8    TMA producer of the x tiles (one lane)
//   warp  9    owns tensor memory and issues the MMAs (one lane)
template <typename Row, bool BF16, typename OutT>
__global__ void __launch_bounds__(THREADS, 1) prefill_umma_kernel(const __grid_constant__ CUtensorMap tmap_x,
                                                                 const typename Row::Ctx ctx, const Group grp,
                                                                 OutT *__restrict__ out, int M, int N, int K, int bm, int n256) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sA = base, sB = base + SA * A_STAGE, sBar = sB + SB * B_STAGE;
  // barriers: a_full[SA] a_empty[SA] b_full[SB] b_empty[SB] d_full, then the TMEM address word
  const uint32_t a_full = sBar, a_empty = sBar + 8 * SA, b_full = sBar + 16 * SA, b_empty = b_full + 8 * SB,
                 d_full = b_empty + 8 * SB, tmem_slot = d_full + 8;
  __shared__ int abort_flag;
  __shared__ uint32_t tmem_base_sh;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BN;
  // bm = 256, or 128 when that fills the SMs better; with n256 >= 0 the first n256 token tiles are 256 rows high and
  // the rest 128 (the tail of the last wave is cut finer)
  if (n256 >= 0) bm = (int)blockIdx.y < n256 ? 256 : 128;
  int m0 = n256 >= 0 && (int)blockIdx.y >= n256 ? n256 * 256 + ((int)blockIdx.y - n256) * 128 : blockIdx.y * bm, m_end = M, expert = 0;
  if (grp.offsets) {
    // which (expert, tile of its rows) is this CTA's?  Tiles are numbered expert by expert.
    __shared__ int tile_info[3];
    if (threadIdx.x == 0) {
      int y = blockIdx.y, e = 0;
      tile_info[0] = -1;
      for (; e < grp.E; e++) {
        const int lo = grp.offsets[e], hi = grp.offsets[e + 1], t = (hi - lo + bm - 1) / bm;
        if (y < t) {
          tile_info[0] = e, tile_info[1] = lo + y * bm, tile_info[2] = hi;
          break;
        }
        y -= t;
      }
    }
    __syncthreads();
    if (tile_info[0] < 0) return;  // beyond the last tile: the grid is sized for the worst case
    expert = tile_info[0], m0 = tile_info[1], m_end = tile_info[2];
  }
  // K split (few tokens only): gridDim.z CTAs form a cluster, each takes a contiguous run of 256-element
  // blocks; the partial tiles are added up through distributed shared memory at the end
  const int KS = gridDim.z, krank = blockIdx.z;
  const int kb0 = KS > 1 ? ((K >> 8) * krank / KS) * 4 : 0, kb1 = KS > 1 ? ((K >> 8) * (krank + 1) / KS) * 4 : K / BK;
  const int nkb = kb1 - kb0;
  const bool two = bm > 128 && m0 + 128 < m_end;  // the second 128-row tile holds real rows

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
        mbar_arrive_expect_tx(a_full + 8 * s, two ? A_STAGE : A_STAGE / 2);
        tma_load_2d(sA + s * A_STAGE, &tmap_x, a_full + 8 * s, (kb0 + kb) * BK, m0);
        if (two) tma_load_2d(sA + s * A_STAGE + A_STAGE / 2, &tmap_x, a_full + 8 * s, (kb0 + kb) * BK, m0 + 128);
        issued = kb + 1;
      }
      if (*abort)  // give the loads still in flight a bounded time to land before the CTA retires
        for (int kb = issued > SA ? issued - SA : 0; kb < issued; kb++)
          for (int i = 0; i < (1 << 14) && !mbar_try_wait(a_full + 8 * (kb % SA), (kb / SA) & 1); i++) {
          }
    }
  } else if (warp == MMA_WARP) {
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_f16(128, BN, BF16);
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
          if (two) mma_f16(tmem_base + 256, a1, bd, idesc, acc);
        }
        mma_commit(a_empty + 8 * sa);
        mma_commit(b_empty + 8 * sb);
      }
      if (nkb > 0) mma_commit(d_full);
    }
  } else {
    // ---- weight expansion: thread r owns row n0 + r (clamped; rows past N are never stored)
    const int r = threadIdx.x;
    const int n = min(n0 + r, N - 1);
    Row cur;
    cur.init(ctx, expert, n, N, K);
    const int u0 = kb0 / Row::STEPS, units = kb1 / Row::STEPS;
    if (u0 < units) cur.load(u0);
    bool ok = true;
    for (int u = u0; u < units && ok; u++) {
      Row nxt = cur;
      if (u + 1 < units) nxt.load(u + 1);
#pragma unroll
      for (int j = 0; j < Row::STEPS; j++) {
        const int kb = u * Row::STEPS + j - kb0, s = kb % SB;
        if (kb >= SB) {  // lane 0 waits for the stage to be free, the warp follows its verdict
          int got = 1;
          if (lane == 0) got = mbar_wait(b_empty + 8 * s, ((kb / SB) - 1) & 1, abort);
          if (!__shfl_sync(0xffffffffu, got, 0)) {
            ok = false;
            break;
          }
        }
        cur.template step<BF16>(j, sB + s * B_STAGE, r);
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(b_full + 8 * s);
      }
      cur = nxt;
    }
    // ---- epilogue: warp w reads TMEM lanes 32 (w % 4) .. +31 (tokens) and columns 128 (w / 4) .. +127
    int done = 0;
    if (ok && lane == 0) done = nkb > 0 ? (int)mbar_wait(d_full, 0, abort) : 1;
    done = __shfl_sync(0xffffffffu, done, 0);
    if (KS > 1) {
      // partial[token][column] (257 floats per token: a warp writes one column of 32 tokens at a time)
      // over the now idle stages; rows of the cluster's sum are shared out below
      if (done) tc_fence_after();
      const int quad = warp & 3, chalf = warp >> 2;
#pragma unroll 1
      for (int c = 0; c < 4; c++) {
        uint32_t v[32];
#pragma unroll
        for (int i = 0; i < 32; i++) v[i] = 0u;
        if (done && nkb > 0) {
          tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + chalf * 128 + c * 32, v);
          tmem_ld_wait();
        }
#pragma unroll
        for (int i = 0; i < 32; i++)
          asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(base + (uint32_t)((quad * 32 + lane) * 257 + chalf * 128 + c * 32 + i) * 4u),
                       "r"(v[i]));
      }
    } else if (done) {
      tc_fence_after();
      const int quad = warp & 3, chalf = warp >> 2;
#pragma unroll 1
      for (int a = 0; a < (two ? 2 : 1); a++) {
        const int mi = m0 + a * 128 + quad * 32 + lane;  // row of the A operand
        long long m = mi;                                 // row of the output
        float wgt = 1.f;
        bool live = mi < m_end;
        if (grp.offsets && live) {
          m = grp.pairs[mi];
          live = m >= 0 && m < grp.size_m;
          if (live && grp.topkw) wgt = grp.topkw[m];
        }
#pragma unroll 1
        for (int c = 0; c < 4; c++) {
          uint32_t v[32];
          tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + a * 256 + chalf * 128 + c * 32, v);
          tmem_ld_wait();
          tile_store32<OutT>(v, sB + (uint32_t)warp * 4096, lane, m, live, wgt, grp.topkw != nullptr, out, N, n0 + chalf * 128 + c * 32);
        }
      }
    }
  }
  __syncwarp();
  if (abort_flag && threadIdx.x == 0) g_prefill_status = 1;
  tc_fence_before();
  if (KS > 1) {
    cluster_sync();
    const int rows_per = 128 / KS;  // tokens of the tile this CTA adds up and stores
    if (threadIdx.x < BN) {
      const int col = threadIdx.x;
      for (int tt = 0; tt < rows_per; tt++) {
        const int tok = krank * rows_per + tt;
        const uint32_t a = base + (uint32_t)(tok * 257 + col) * 4u;
        float v = 0.f;
        for (int p = 0; p < KS; p++) v += ld_cluster_f32(map_to_rank(a, (uint32_t)p));
        if (m0 + tok < m_end && n0 + col < N) st_act(out, (long long)(m0 + tok) * N + n0 + col, v);
      }
    }
    cluster_sync();  // nobody leaves while a peer still reads its partials
  } else {
    __syncthreads();
  }
  if (warp == MMA_WARP) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---- the same tile as a persistent kernel over an even split of ALL k-steps (stream-K).
// A grid of equal tiles leaves the last wave of the SMs partly empty (192 tiles on 148 SMs run as two rounds), and a
// grouped launch has tiles of unequal height.  Here the work is the list of (tile, 256-element K block) pairs in tile
// order, cut into gridDim.x runs of equal length, one CTA per SM and per run.  A run is a tail of one tile, whole
// tiles, and a head of one tile; each piece ("segment") runs through the same TMA / expander / MMA pipeline, the rings
// carry on from one segment to the next, and the accumulator is handed over through one more barrier (d_empty).
//   * a segment that covers its tile stores it;
//   * a segment that does not start at k = 0 writes its 256 x 256 f32 partial tile to this CTA's slot of the
//     workspace and raises the slot's flag: it is the FIRST thing its CTA does, and it waits for nobody;
//   * the segment that starts a tile (the LAST of its CTA's run) owns it: it adds the partials of the CTAs after it, in
//     run order (a fixed order of summation), and stores.  The wait is bounded (the status word is set when it runs
//     out), and what it waits for was written at the start of the other runs, so it is there long before.
constexpr int SK_PART_FLOATS = 2 * 4 * 32 * 256;  // one partial tile: (token half, 32-column chunk, column, thread)
constexpr int SK_MAX_E = 1024;                    // experts whose tile counts fit the shared prefix table
constexpr size_t SK_FLAG_BYTES = 4096;

struct SkTile {
  int n0, m0, m_end, expert;
  bool two;
};

__device__ __forceinline__ bool sk_wait_flag(const unsigned *flag, unsigned want, volatile int *abort) {
  const unsigned long long t0 = global_ns();
  for (uint32_t i = 1;; i++) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(flag) : "memory");
    if (v == want) return true;
    if ((i & 15u) == 0) {
      if (*abort) return false;
      if (global_ns() - t0 > 200000000ull) break;
      __nanosleep(128);
    }
  }
  *abort = 1;
  return false;
}

// rows whose packed weights the persistent kernel brings in through shared memory
template <typename Row>
struct SkStaged : std::false_type {
  static constexpr int pitch = 0;
};
template <>
struct SkStaged<Fp8Row> : std::true_type {
  static constexpr int granules = 8, pitch = 144, units_per_copy = 1;  // 128 codes
};
template <>
struct SkStaged<Q6KRow> : std::true_type {
  static constexpr int granules = 14, pitch = 240, units_per_copy = 2;  // the 224 bytes that cover a 210-byte block
};
// (Q4_K rows -- 9 granules, one 144-byte block -- were measured this way too: no faster at 2048 tokens, where their main
// loop runs at the MMAs' pace, and 5-15 % slower on short runs)
template <>
struct SkStaged<Int4Row> : std::true_type {
  static constexpr int granules = 8, pitch = 144, units_per_copy = 1;  // 256 codes
};
template <typename Row>
constexpr int sk_smem_bytes() {  // staged rows: two activation stages, and one copy slot of `pitch` bytes per weight row
  return SkStaged<Row>::value ? 2 * A_STAGE + SB * B_STAGE + 1024 + 256 + 256 * SkStaged<Row>::pitch : SMEM_BYTES;
}

template <typename Row, bool BF16, typename OutT>
__global__ void __launch_bounds__(THREADS, 1) prefill_sk_kernel(const __grid_constant__ CUtensorMap tmap_x, const typename Row::Ctx ctx,
                                                               const Group grp, OutT *__restrict__ out, int M, int N, int K,
                                                               float *__restrict__ parts, unsigned *__restrict__ flags) {
  // Q6_K, 4-bit group-quantized and block-FP8 rows come in through shared memory: a thread per row reading global memory
  // touches 32 lines per load instruction (Q6_K: 27 to 54 four-byte loads per 128 weights), and that made the load unit
  // (70 % of its wavefront rate for FP8), not the MMAs, set the pace.  Each warp copies the next load unit (Q6_K: block)
  // of its 32 rows with cp.async, the lanes running along a row (a few lines per instruction), into its own slot, and
  // its threads read their rows from there into registers; the slot is then free for the next copy, which lands while
  // those registers are expanded.  The slots take the third activation stage's room.
  constexpr bool STAGED = SkStaged<Row>::value;
  constexpr int SAK = STAGED ? 2 : SA;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sA = base, sB = base + SAK * A_STAGE, sBar = sB + SB * B_STAGE, sRaw = sBar + 256;
  const uint32_t a_full = sBar, a_empty = sBar + 8 * SAK, b_full = sBar + 16 * SAK, b_empty = b_full + 8 * SB, d_full = b_empty + 8 * SB,
                 d_empty = d_full + 8, tmem_slot = d_empty + 8;
  __shared__ int abort_flag;
  __shared__ uint32_t tmem_base_sh;
  __shared__ int pre[SK_MAX_E + 1];  // grouped: token tiles before expert e
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ntx = (N + BN - 1) / BN, nb = K >> 8;
  int nty = (M + BM - 1) / BM;
  if (grp.offsets) {
    for (int e = threadIdx.x; e < grp.E; e += THREADS) pre[e + 1] = (grp.offsets[e + 1] - grp.offsets[e] + BM - 1) / BM;
    __syncthreads();
    if (threadIdx.x == 0) {
      pre[0] = 0;
      for (int e = 0; e < grp.E; e++) pre[e + 1] += pre[e];
    }
    __syncthreads();
    nty = pre[grp.E];
  }
  const long long U = (long long)ntx * nty * nb;
  const int G = gridDim.x, cta = blockIdx.x;
  auto run_start = [&](int j) { return U * j / G; };
  const long long pos0 = run_start(cta), pos1 = run_start(cta + 1);
  auto tile_of = [&](long long t) {
    SkTile T;
    const int ty = (int)(t / ntx);
    T.n0 = (int)(t - (long long)ty * ntx) * BN, T.expert = 0, T.m0 = ty * BM, T.m_end = M;
    if (grp.offsets) {
      int lo = 0, hi = grp.E - 1;  // the expert with pre[e] <= ty < pre[e + 1]
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (pre[mid + 1] <= ty) lo = mid + 1;
        else hi = mid;
      }
      T.expert = lo, T.m0 = grp.offsets[lo] + (ty - pre[lo]) * BM, T.m_end = grp.offsets[lo + 1];
    }
    T.two = T.m0 + 128 < T.m_end;
    return T;
  };

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int i = 0; i < SAK; i++) mbar_init(a_full + 8 * i, 1), mbar_init(a_empty + 8 * i, 1);
    for (int i = 0; i < SB; i++) mbar_init(b_full + 8 * i, NUM_DEQ_WARPS), mbar_init(b_empty + 8 * i, 1);
    mbar_init(d_full, 1);
    mbar_init(d_empty, NUM_DEQ_WARPS);
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
      int it = 0;  // k-steps issued over all segments
      for (long long pos = pos0; pos < pos1 && !*abort;) {
        const long long t = pos / nb;
        const int b0 = (int)(pos - t * nb), b1 = (int)min((long long)nb, b0 + (pos1 - pos));
        const SkTile T = tile_of(t);
        for (int kb = b0 * 4; kb < b1 * 4; kb++, it++) {
          const int s = it % SAK;
          if (it >= SAK && !mbar_wait(a_empty + 8 * s, ((it / SAK) - 1) & 1, abort)) break;
          mbar_arrive_expect_tx(a_full + 8 * s, T.two ? A_STAGE : A_STAGE / 2);
          tma_load_2d(sA + s * A_STAGE, &tmap_x, a_full + 8 * s, kb * BK, T.m0);
          if (T.two) tma_load_2d(sA + s * A_STAGE + A_STAGE / 2, &tmap_x, a_full + 8 * s, kb * BK, T.m0 + 128);
        }
        pos += b1 - b0;
      }
      if (*abort)  // give the loads still in flight a bounded time to land before the CTA retires
        for (int k = it > SAK ? it - SAK : 0; k < it; k++)
          for (int i = 0; i < (1 << 14) && !mbar_try_wait(a_full + 8 * (k % SAK), (k / SAK) & 1); i++) {
          }
    }
  } else if (warp == MMA_WARP) {
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_f16(128, BN, BF16);
      int it = 0, seg = 0;
      bool ok = true;
      for (long long pos = pos0; pos < pos1 && ok; seg++) {
        const long long t = pos / nb;
        const int b0 = (int)(pos - t * nb), b1 = (int)min((long long)nb, b0 + (pos1 - pos));
        const SkTile T = tile_of(t);
        // the accumulators of the segment before must have been read out
        if (seg > 0 && !mbar_wait(d_empty, (seg - 1) & 1, abort)) break;
        tc_fence_after();
        for (int kb = 0; kb < (b1 - b0) * 4; kb++, it++) {
          const int sa = it % SAK, sb = it % SB;
          if (!mbar_wait(a_full + 8 * sa, (it / SAK) & 1, abort) || !mbar_wait(b_full + 8 * sb, (it / SB) & 1, abort)) {
            ok = false;
            break;
          }
          tc_fence_after();
#pragma unroll
          for (int k4 = 0; k4 < BK / 16; k4++) {
            const uint64_t bd = smem_desc_sw128(sB + sb * B_STAGE + k4 * 32);
            const uint64_t a0 = smem_desc_sw128(sA + sa * A_STAGE + k4 * 32);
            const uint64_t a1 = smem_desc_sw128(sA + sa * A_STAGE + A_STAGE / 2 + k4 * 32);
            const uint32_t acc = (kb | k4) ? 1u : 0u;
            mma_f16(tmem_base, a0, bd, idesc, acc);
            if (T.two) mma_f16(tmem_base + 256, a1, bd, idesc, acc);
          }
          mma_commit(a_empty + 8 * sa);
          mma_commit(b_empty + 8 * sb);
        }
        if (ok) mma_commit(d_full);
        pos += b1 - b0;
      }
    }
  } else {
    // ---- weight expansion (thread r owns row n0 + r of the segment's tile), then the segment's epilogue
    const int r = threadIdx.x, quad = warp & 3, chalf = warp >> 2;
    int it = 0, seg = 0;
    bool ok = true;
    Row cur;
    for (long long pos = pos0; pos < pos1 && ok; seg++) {
      const long long t = pos / nb;
      const int b0 = (int)(pos - t * nb), b1 = (int)min((long long)nb, b0 + (pos1 - pos));
      const SkTile T = tile_of(t);
      const int kb0 = b0 * 4, u0 = kb0 / Row::STEPS, units = b1 * 4 / Row::STEPS;
      cur.init(ctx, T.expert, min(T.n0 + r, N - 1), N, K);
      auto steps_of = [&](Row &row) {  // the 64-k steps of the unit `row` holds
#pragma unroll
        for (int j = 0; j < Row::STEPS; j++, it++) {
          const int s = it % SB;
          if (it >= SB) {  // lane 0 waits for the stage to be free, the warp follows its verdict
            int got = 1;
            if (lane == 0) got = mbar_wait(b_empty + 8 * s, ((it / SB) - 1) & 1, abort);
            if (!__shfl_sync(0xffffffffu, got, 0)) {
              ok = false;
              break;
            }
          }
          row.template step<BF16>(j, sB + s * B_STAGE, r);
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) mbar_arrive(b_full + 8 * s);
        }
      };
      if constexpr (STAGED) {
        using S = SkStaged<Row>;
        constexpr int GR = S::granules, PITCH = S::pitch, CG = S::units_per_copy;
        constexpr bool HALF = std::is_same<Row, Fp8Row>::value;    // a load unit is half of a 256-code raw block
        constexpr bool SKEWED = std::is_same<Row, Q6KRow>::value;  // rows start on any even byte: the copy is of the
                                                                   // 16-byte granules that cover the block
        const int nw = min(T.n0 + warp * 32, N - 1);               // the warp's first row, and its 31 successors (clamped)
        Row c0;
        c0.init(ctx, T.expert, nw, N, K);
        const size_t rstride = Row::row_stride(ctx, K);
        const uint32_t wslot = sRaw + (uint32_t)warp * 32 * PITCH;
        const uint8_t *lim = c0.raw_end();
        int ic = u0 / CG;
        const int c_end = units / CG;
        auto issue = [&]() {  // always closes a commit group
          if (ic < c_end) {
#pragma unroll
            for (int i = 0; i < GR; i++) {  // lanes run along the granules of a row, then on to the next row
              const int q = lane + 32 * i, rr = q / GR, piece = q - rr * GR;
              const size_t down = (size_t)(min(T.n0 + warp * 32 + rr, N - 1) - nw) * rstride;
              const uint8_t *src;
              if constexpr (HALF) src = c0.raw_src(ic >> 1) + 128 * (ic & 1) + down;
              else if constexpr (SKEWED) src = reinterpret_cast<const uint8_t *>((uintptr_t)(c0.raw_src_unaligned(ic) + down) & ~(uintptr_t)15);
              else src = c0.raw_src(ic) + down;
              src += piece * 16;
              const uint32_t dst = wslot + rr * PITCH + piece * 16;
              if (lim == nullptr || src + 16 <= lim) cp_async16(dst, src);
              else if (src < lim) cp_async16_part(dst, src, (uint32_t)(lim - src));
            }
          }
          ic++;
          cp_async_commit();
        };
        issue();
        for (int c = u0 / CG; c < c_end && ok; c++) {
          cp_async_wait<0>();  // this lane's granules of copy c have landed ...
          __syncwarp();        // ... and so have the other lanes' (the rows of a warp are copied by that warp alone)
#pragma unroll
          for (int uu = 0; uu < CG; uu++) {
            const int u = c * CG + uu;
            cur.load_smem(sRaw + (uint32_t)r * PITCH - (HALF ? 128u * (u & 1) : 0u), u);
            if (uu == CG - 1) {  // the rows are in registers: the slot can take the next copy while these steps run
              __syncwarp();
              issue();
            }
            steps_of(cur);
          }
        }
        cp_async_wait<0>();
      } else {
        cur.load(u0);
        for (int u = u0; u < units && ok; u++) {
          Row nxt = cur;
          if (u + 1 < units) nxt.load(u + 1);
          steps_of(cur);
          cur = nxt;
        }
      }
      pos += b1 - b0;
      if (pos < pos1 && ok) {  // the next segment's first block of this thread's row, on its way to L2 during the epilogue
        const SkTile Tn = tile_of(pos / nb);
        Row nr;
        nr.init(ctx, Tn.expert, min(Tn.n0 + r, N - 1), N, K);
        nr.prefetch(0);
      }
      int done = 0;
      if (ok && lane == 0) done = (int)mbar_wait(d_full, seg & 1, abort);
      done = __shfl_sync(0xffffffffu, done, 0);
      if (!done) {
        ok = false;
        break;
      }
      tc_fence_after();
      const bool owner = b0 == 0, whole = owner && b1 == nb;
      const int nch = T.two ? 8 : 4;  // 32-column chunks of this warp's part of the accumulators: (token half, chunk)
      auto chunk_addr = [&](int ch) { return tmem_base + ((uint32_t)(quad * 32) << 16) + (ch >> 2) * 256 + chalf * 128 + (ch & 3) * 32; };
      uint32_t va[32], vb[32];
      if (!owner) {
        // a tail (or a middle) of a tile another CTA owns: the partial sums to this CTA's slot, then the flag
        float *mine = parts + (size_t)cta * SK_PART_FLOATS + threadIdx.x;
        auto put = [&](const uint32_t (&v)[32], int ch) {
#pragma unroll
          for (int i = 0; i < 32; i++) mine[(ch * 32 + i) * 256] = __uint_as_float(v[i]);
        };
        tmem_ld32(chunk_addr(0), va);
#pragma unroll 1
        for (int ch = 0; ch < nch; ch += 2) {  // (the next chunk leaves tensor memory while this one is stored)
          tmem_ld_wait();
          tmem_ld32(chunk_addr(ch + 1), vb);
          put(va, ch);
          tmem_ld_wait();
          if (ch + 2 < nch) tmem_ld32(chunk_addr(ch + 2), va);
          put(vb, ch + 1);
        }
        __threadfence();
        asm volatile("bar.sync 1, 256;\n" ::: "memory");
        if (threadIdx.x == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;\n" ::"l"(flags + cta), "r"(1u) : "memory");
      } else {
        // the CTAs that hold the rest of this tile's k range, in run order
        int jlast = cta;
        if (!whole) {
          const long long tile_end = (t + 1) * nb;
          while (jlast + 1 < G && run_start(jlast + 1) < tile_end) jlast++;
          for (int j = cta + 1; j <= jlast; j++)
            if (run_start(j + 1) > run_start(j) && !sk_wait_flag(flags + j, 1u, abort)) ok = false;
        }
        // this thread's token row in either half: where it goes and with what weight
        long long mrow[2];
        float wrow[2];
        bool lrow[2];
#pragma unroll
        for (int a = 0; a < 2; a++) {
          const int mi = T.m0 + a * 128 + quad * 32 + lane;  // row of the A operand
          mrow[a] = mi, wrow[a] = 1.f, lrow[a] = mi < T.m_end && (a == 0 || T.two);
          if (grp.offsets && lrow[a]) {
            mrow[a] = grp.pairs[mi];
            lrow[a] = mrow[a] >= 0 && mrow[a] < grp.size_m;
            if (lrow[a] && grp.topkw) wrow[a] = grp.topkw[mrow[a]];
          }
        }
        auto put = [&](uint32_t (&v)[32], int ch) {
          const int a = ch >> 2;
          const long long m = a ? mrow[1] : mrow[0];
          const float wgt = a ? wrow[1] : wrow[0];
          const bool live = a ? lrow[1] : lrow[0];
          if (live && ok) {
            for (int j = cta + 1; j <= jlast; j++) {
              if (run_start(j + 1) == run_start(j)) continue;  // (an empty run wrote nothing)
              const float *theirs = parts + (size_t)j * SK_PART_FLOATS + threadIdx.x + ch * 32 * 256;
#pragma unroll
              for (int i = 0; i < 32; i++) v[i] = __float_as_uint(__uint_as_float(v[i]) + __ldcg(theirs + i * 256));
            }
          }
          tile_store32<OutT>(v, sB + (uint32_t)warp * 4096, lane, m, live, wgt, grp.topkw != nullptr, out, N, T.n0 + chalf * 128 + (ch & 3) * 32);
        };
        tmem_ld32(chunk_addr(0), va);
#pragma unroll 1
        for (int ch = 0; ch < nch; ch += 2) {
          tmem_ld_wait();
          tmem_ld32(chunk_addr(ch + 1), vb);
          put(va, ch);
          tmem_ld_wait();
          if (ch + 2 < nch) tmem_ld32(chunk_addr(ch + 2), va);
          put(vb, ch + 1);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(d_empty);
    }
  }
  __syncwarp();
  if (abort_flag && threadIdx.x == 0) g_prefill_status = 1;
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) tmem_dealloc(tmem_base, TMEM_COLS);
}

// x f32 (M, K) -> f16, clamped to the f16 range so that an outlier cannot become an infinity.
// PERM: every four consecutive k are stored in the order 0, 2, 1, 3 (what a KPERM row expander pairs them with).
template <bool PERM>
__global__ void __launch_bounds__(256) x_to_f16_kernel(const float4 *__restrict__ x, uint2 *__restrict__ y, long long n4) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 v = __ldg(x + i);
    v.x = fminf(fmaxf(v.x, -65504.f), 65504.f), v.y = fminf(fmaxf(v.y, -65504.f), 65504.f);
    v.z = fminf(fmaxf(v.z, -65504.f), 65504.f), v.w = fminf(fmaxf(v.w, -65504.f), 65504.f);
    y[i] = PERM ? make_uint2(pack_h2(v.x, v.z), pack_h2(v.y, v.w)) : make_uint2(pack_h2(v.x, v.y), pack_h2(v.z, v.w));
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

// x f32 -> f16 in the workspace, or bf16 x used as it is; then the tensor map over it.
int make_x_map(CUtensorMap *tm, const void *x, int act_dtype, int M, int K, void *ws, bool perm, cudaStream_t st) {
  if (int rc = ensure_encode()) return rc;
  const void *src = x;
  CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if (act_dtype == LB200_F32) {
    const long long n4 = (long long)M * K / 4;
    long long blocks = (n4 + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (perm)
      x_to_f16_kernel<true><<<(unsigned)blocks, 256, 0, st>>>((const float4 *)x, (uint2 *)ws, n4);
    else
      x_to_f16_kernel<false><<<(unsigned)blocks, 256, 0, st>>>((const float4 *)x, (uint2 *)ws, n4);
    if (int rc = launched("prefill: activations to f16")) return rc;
    src = ws;
    dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  }
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {BK, 128};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(tm, dt, 2, const_cast<void *>(src), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(LB200_E_SHAPE, "light_b200: prefill: cuTensorMapEncodeTiled failed (%d)", (int)r);
  return 0;
}

template <typename Row, bool BF16, typename OutT>
int launch(const CUtensorMap &tm, const typename Row::Ctx &ctx, const Group &grp, OutT *out, int M, int N, int K,
           cudaStream_t st, void *sk = nullptr, size_t sk_bytes = 0) {
  // The persistent stream-K kernel when the workspace has room for its partial tiles and the split pays: each CTA needs
  // a few K blocks to spread the cost of its two extra epilogues over (measured: five), and a grid of whole 256-token tiles
  // that fills between three quarters and all of the SMs in one wave is already even (rows that only this kernel brings
  // in through shared memory take it there too: Q6_K down at 2048 tokens 300 against 325 us).  A grouped launch always takes it (its
  // tiles are uneven by nature).  LIGHT_B200_PREFILL_SK = 0: never, 2: whenever possible.
  static int use_sk = -1;
  if (use_sk < 0) use_sk = getenv("LIGHT_B200_PREFILL_SK") ? atoi(getenv("LIGHT_B200_PREFILL_SK")) : 1;
  if (use_sk && sk && K % 256 == 0 && (!grp.offsets || grp.E <= SK_MAX_E)) {
    long long G = sm_count();
    bool pays = true;
    if (!grp.offsets) {
      const long long tiles = (long long)((N + BN - 1) / BN) * ((M + BM - 1) / BM), U = tiles * (K >> 8);
      pays = U >= 5 * G && (SkStaged<Row>::value || !(M > 128 && tiles <= G && 4 * tiles >= 3 * G));
      if (U < G) G = U;
    }
    if (use_sk == 1 && !pays) G = 0;
    if (G > 0 && sk_bytes >= SK_FLAG_BYTES + (size_t)G * SK_PART_FLOATS * 4 && (size_t)G * 4 <= SK_FLAG_BYTES) {
      auto skern = prefill_sk_kernel<Row, BF16, OutT>;
      constexpr int sk_smem = sk_smem_bytes<Row>();
      static DeviceOnce sk_attr;
      cudaError_t e = sk_attr.ensure([&] { return cudaFuncSetAttribute(skern, cudaFuncAttributeMaxDynamicSharedMemorySize, sk_smem); });
      if (e == cudaSuccess) e = cudaMemsetAsync(sk, 0, (size_t)G * 4, st);
      if (e != cudaSuccess) return fail((int)e, "light_b200: prefill: %s", cudaGetErrorString(e));
      skern<<<(unsigned)G, THREADS, sk_smem, st>>>(tm, ctx, grp, out, M, N, K, (float *)((char *)sk + SK_FLAG_BYTES), (unsigned *)sk);
      return launched("prefill (tcgen05, stream-K)");
    }
  }
  auto kern = prefill_umma_kernel<Row, BF16, OutT>;
  static DeviceOnce attr_done;
  {
    cudaError_t e = attr_done.ensure([&] { return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES); });
    if (e != cudaSuccess) return fail((int)e, "light_b200: prefill: %s", cudaGetErrorString(e));
  }
  // Token-tile height: 256 amortises the weight expansion best, but when the grid of 256-row tiles leaves
  // the last wave of the 148 SMs mostly empty, 128-row tiles (twice as many CTAs) finish sooner.
  const long long nt = (N + BN - 1) / BN;
  auto waves_cost = [&](int bm_) {  // time in units of one 256-row tile
    const long long ctas = nt * ((M + bm_ - 1) / bm_);
    return (double)((ctas + 147) / 148) * (bm_ == 256 ? 1.0 : 0.75);
  };
  // (measured: a 128-row tile takes 0.75 of a 256-row tile)
  int bm = (!grp.offsets && waves_cost(128) < waves_cost(256)) ? 128 : 256;
  if (const char *e = getenv("LIGHT_B200_PREFILL_BM")) bm = (atoi(e) == 128 && !grp.offsets) ? 128 : atoi(e) == 256 ? 256 : bm;
  // Mixed heights: n256 tiles of 256 rows first, 128-row tiles for the rest.  The CTAs start in grid order on the first
  // free SM; the split with the shortest finish under that rule (a 128-row tile costs 0.75) wins over either uniform grid.
  int n256 = -1;
  static int mixed = -1;
  if (mixed < 0) mixed = getenv("LIGHT_B200_PREFILL_MIXED") ? atoi(getenv("LIGHT_B200_PREFILL_MIXED")) : 1;
  if (mixed && !grp.offsets && M > 256 && nt * ((M + 255) / 256) <= 8192) {
    static std::mutex plan_mu;
    static std::vector<std::pair<std::pair<int, long long>, int>> plans;  // (M, nt) -> n256, found once per shape
    std::lock_guard<std::mutex> lk(plan_mu);
    bool known = false;
    for (const auto &p : plans)
      if (p.first.first == M && p.first.second == nt) n256 = p.second, known = true;
    if (!known) {
      const int sms = sm_count(), big_max = M / 256;
      auto finish = [&](int nb256) {
        const int small = (M - nb256 * 256 + 127) / 128;
        std::vector<double> sm(sms, 0.0);
        double end = 0;
        auto place = [&](long long count, double cost) {
          for (long long i = 0; i < count; i++) {
            int best = 0;
            for (int j = 1; j < sms; j++)
              if (sm[j] < sm[best]) best = j;
            sm[best] += cost;
            if (sm[best] > end) end = sm[best];
          }
        };
        place((long long)nb256 * nt, 1.0);
        place((long long)small * nt, 0.75);
        return end;
      };
      double best = bm == 256 ? waves_cost(256) : waves_cost(128);
      for (int c = big_max; c >= 0 && c >= big_max - 4; c--) {
        const double f = finish(c);
        if (f < best - 1e-9) best = f, n256 = c;
      }
      if (plans.size() < 256) plans.push_back({{M, nt}, n256});
    }
  }
  // Few tokens and few weight-row tiles (fewer 128-row tiles than SMs): split K over a cluster of up to 8 CTAs so
  // that every SM has one, the smallest power of two that does
  int ks = 1;
  if (!grp.offsets && K % 256 == 0 && (M <= 128 || nt * ((M + 127) / 128) < sm_count())) {
    bm = 128, n256 = -1;
    const int nblk = K >> 8;
    const long long ctas = nt * ((M + 127) / 128);
    while (ks < 8 && ks * 2 <= nblk && ctas * ks < sm_count()) ks *= 2;
  }
  // grouped: at most ceil(M / bm) + E tiles (every expert can end with one partial tile)
  dim3 grid((unsigned)nt, (M + bm - 1) / bm + (grp.offsets ? grp.E : 0), (unsigned)ks);
  if (n256 >= 0) grid.y = (unsigned)(n256 + (M - n256 * 256 + 127) / 128);
  if (ks == 1) {
    kern<<<grid, THREADS, SMEM_BYTES, st>>>(tm, ctx, grp, out, M, N, K, bm, n256);
  } else {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = (unsigned)ks;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tm, ctx, grp, out, M, N, K, bm, n256);
    if (e != cudaSuccess) return fail((int)e, "light_b200: prefill: %s", cudaGetErrorString(e));
  }
  return launched("prefill (tcgen05)");
}

// f32 activations run with f16 operands and f32 output, bf16 activations with bf16 operands and output
template <typename Row>
int launch_by_act(const void *x, int act_dtype, const typename Row::Ctx &ctx, void *out, int M, int N, int K, void *ws,
                  size_t ws_bytes, cudaStream_t st) {
  CUtensorMap tm;
  if (Row::KPERM && act_dtype != LB200_F32)
    return fail(LB200_E_DTYPE, "light_b200: prefill: this weight format takes f32 activations only");
  if (int rc = make_x_map(&tm, x, act_dtype, M, K, ws, Row::KPERM, st)) return rc;
  const Group none{nullptr, nullptr, nullptr, 0, 0};
  // what the workspace holds beyond the f16 copy of x is the stream-K kernel's
  const size_t x_bytes = act_dtype == LB200_F32 ? (((size_t)M * K * 2 + 1023) & ~(size_t)1023) : 0;
  void *sk = ws && ws_bytes > x_bytes ? (char *)ws + x_bytes : nullptr;
  const size_t sk_bytes = sk ? ws_bytes - x_bytes : 0;
  if (act_dtype == LB200_F32) return launch<Row, false, float>(tm, ctx, none, (float *)out, M, N, K, st, sk, sk_bytes);
  if constexpr (!Row::KPERM) return launch<Row, true, __nv_bfloat16>(tm, ctx, none, (__nv_bfloat16 *)out, M, N, K, st, sk, sk_bytes);
  return LB200_E_DTYPE;
}

// workspace for an f32 activation matrix; bf16 needs none.  Returns false if there is not enough.
bool get_ws(int device, int act_dtype, int M, int K, void **ws, size_t *bytes) {
  std::lock_guard<std::mutex> lk(g_mu);
  *ws = g_ws[device].ptr, *bytes = g_ws[device].ptr ? g_ws[device].bytes : 0;
  return act_dtype != LB200_F32 || (*ws && *bytes >= (size_t)M * K * 2);
}

}  // namespace

// room the stream-K kernel wants after the f16 copy of x: the flags and one partial tile per SM (up to 160 of them)
size_t prefill_sk_ws_bytes() { return SK_FLAG_BYTES + (size_t)160 * SK_PART_FLOATS * 4 + 1024; }

void *workspace_ptr(int device, size_t *bytes) {
  std::lock_guard<std::mutex> lk(g_mu);
  *bytes = g_ws[device].bytes;
  return g_ws[device].ptr;
}

int set_workspace(int device, void *ptr, size_t bytes) {
  if (device < 0 || device >= 64) return fail(LB200_E_DEVICE, "light_b200: device ordinal %d out of range", device);
  if (((uintptr_t)ptr & 1023) != 0) return fail(LB200_E_ALIGN, "light_b200: workspace must be 1024-byte aligned");
  std::lock_guard<std::mutex> lk(g_mu);
  g_ws[device] = {ptr, ptr ? bytes : 0};
  return 0;
}

int g_prefill_min_m = 65;  // LIGHT_B200_PREFILL_MIN_M (tuning knob): fewest activation rows this kernel takes
bool g_pf_knobs = false;
void pf_knobs() {
  if (g_pf_knobs) return;
  if (const char *e = getenv("LIGHT_B200_PREFILL_MIN_M")) g_prefill_min_m = atoi(e) < 1 ? 1 : atoi(e);
  g_pf_knobs = true;
}
#define PREFILL_MIN_M (pf_knobs(), g_prefill_min_m)

// Each returns 1 when the tensor-core prefill kernel took the call, 0 when the shape (or the workspace)
// does not allow it, any other value is an error.
int gguf_prefill(int type, const float *x, const void *w, float *out, int M, int N, int K, int device, cudaStream_t st) {
  if (M < PREFILL_MIN_M || K % 256) return 0;
  if (type == LB200_Q4_K) {
    if ((uintptr_t)w & 15) return 0;
  } else if (type == LB200_Q6_K) {
    if (((uintptr_t)w & 3) || ((size_t)(K >> 8) * 210) % 4) return 0;  // rows must start 4-byte aligned
  } else if (type == LB200_Q8_0) {
    if ((uintptr_t)w & 15) return 0;  // K % 256 == 0 makes every row a whole number of 16-byte granules
  } else {
    return 0;
  }
  void *ws;
  size_t wsb;
  if (!get_ws(device, LB200_F32, M, K, &ws, &wsb)) return 0;
  GgufCtx ctx{(const uint8_t *)w};
  int rc = type == LB200_Q4_K   ? launch_by_act<Q4KRow>(x, LB200_F32, ctx, out, M, N, K, ws, wsb, st)
           : type == LB200_Q6_K ? launch_by_act<Q6KRow>(x, LB200_F32, ctx, out, M, N, K, ws, wsb, st)
                                : launch_by_act<Q80Row>(x, LB200_F32, ctx, out, M, N, K, ws, wsb, st);
  return rc ? rc : 1;
}

int int4_prefill(const void *x, const uint32_t *codes, const float *s, const float *z, void *y, int act_dtype, int M, int N,
                 int K, int G, int device, cudaStream_t st) {
  if (M < PREFILL_MIN_M || K % 256 || G % 64 || ((uintptr_t)codes & 15) || ((uintptr_t)x & 15)) return 0;
  void *ws;
  size_t wsb;
  if (!get_ws(device, act_dtype, M, K, &ws, &wsb)) return 0;
  Int4Ctx ctx{codes, s, z, G};
  int rc = launch_by_act<Int4Row>(x, act_dtype, ctx, y, M, N, K, ws, wsb, st);
  return rc ? rc : 1;
}

int fp8_prefill(const void *x, const uint8_t *w, const float *scale, void *y, int act_dtype, int M, int N, int K, int bR,
                int bC, int device, cudaStream_t st) {
  if (M < PREFILL_MIN_M || K % 128 || bC % 64 || ((uintptr_t)w & 15) || ((uintptr_t)x & 15)) return 0;
  void *ws;
  size_t wsb;
  if (!get_ws(device, act_dtype, M, K, &ws, &wsb)) return 0;
  Fp8Ctx ctx{w, scale, bR, bC};
  int rc = launch_by_act<Fp8Row>(x, act_dtype, ctx, y, M, N, K, ws, wsb, st);
  return rc ? rc : 1;
}

namespace {

// ---- grouped (mixture-of-experts) matmul on the same kernel.
// Rows of the A operand in expert order: dst[i] = in[row(sorted_pairs[i])], converted to the operand type
// (f32 -> f16 clamped, 16-bit types copied); rows of pairs outside [0, size_m) are zero.
template <typename TI, bool PERM>
__global__ void __launch_bounds__(256) gather_rows_kernel(const TI *__restrict__ in, const int64_t *__restrict__ pairs,
                                                          uint16_t *__restrict__ dst, long long Mp, int K, int topk,
                                                          int row_per_pair, long long size_m) {
  const int lane = threadIdx.x & 31;
  for (long long i = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); i < Mp; i += (long long)gridDim.x * 8) {
    const long long p = pairs[i];
    const bool ok = p >= 0 && p < size_m;
    const TI *src = in + (size_t)(row_per_pair ? p : p / topk) * K;
    for (int k = lane * 8; k < K; k += 256) {
      uint4 o = make_uint4(0, 0, 0, 0);
      if (ok) {
        if constexpr (sizeof(TI) == 4) {
          const float4 a = __ldg(reinterpret_cast<const float4 *>(src + k)), b = __ldg(reinterpret_cast<const float4 *>(src + k) + 1);
          auto cl = [](float v) { return fminf(fmaxf(v, -65504.f), 65504.f); };
          o = PERM ? make_uint4(pack_h2(cl(a.x), cl(a.z)), pack_h2(cl(a.y), cl(a.w)), pack_h2(cl(b.x), cl(b.z)), pack_h2(cl(b.y), cl(b.w)))
                   : make_uint4(pack_h2(cl(a.x), cl(a.y)), pack_h2(cl(a.z), cl(a.w)), pack_h2(cl(b.x), cl(b.y)), pack_h2(cl(b.z), cl(b.w)));
        } else {
          o = __ldg(reinterpret_cast<const uint4 *>(src + k));
        }
      }
      *reinterpret_cast<uint4 *>(dst + (size_t)i * K + k) = o;
    }
  }
}

template <typename Row, bool BF16, typename OutT, typename TI>
int moe_launch(const lb200_moe_args *a, const typename Row::Ctx &ctx, void *ws, size_t ws_bytes, cudaStream_t st) {
  if (int rc = ensure_encode()) return rc;
  long long blocks = (a->M + 7) / 8;
  if (blocks > 148 * 32) blocks = 148 * 32;
  gather_rows_kernel<TI, Row::KPERM && sizeof(TI) == 4><<<(unsigned)blocks, 256, 0, st>>>((const TI *)a->input, a->sorted_pairs, (uint16_t *)ws, a->M, a->K,
                                                          a->topk, a->row_per_pair, a->size_m);
  if (int rc = launched("moe: gather rows")) return rc;
  CUtensorMap tm;
  const cuuint64_t dims[2] = {(cuuint64_t)a->K, (cuuint64_t)a->M};
  const cuuint64_t strides[1] = {(cuuint64_t)a->K * 2};
  const cuuint32_t box[2] = {BK, 128};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(&tm, BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, ws, dims, strides, box,
                        estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(LB200_E_SHAPE, "light_b200: moe: cuTensorMapEncodeTiled failed (%d)", (int)r);
  const Group grp{a->offsets, a->sorted_pairs, a->topk_weights, a->size_m, a->E};
  const size_t x_bytes = ((size_t)a->M * a->K * 2 + 1023) & ~(size_t)1023;
  void *sk = ws_bytes > x_bytes ? (char *)ws + x_bytes : nullptr;
  return launch<Row, BF16, OutT>(tm, ctx, grp, (OutT *)a->out, (int)a->M, a->N, a->K, st, sk, sk ? ws_bytes - x_bytes : 0);
}

}  // namespace

// Grouped matmul on the tensor cores; the expert offsets must already be in a->offsets.  kind: 0 dense
// (a->dtype = BF16 only), 1 GGUF (a->dtype = Q4_K / Q6_K, x f32), 2 block-scaled FP8 (a->dtype = F32 / BF16
// activations).  Returns 1 when taken, 0 when not covered, other values are errors.
int moe_umma(const lb200_moe_args *a, int kind, const float *w_scale, int bR, int bC, int device, cudaStream_t st) {
  if (a->M < 256 || a->M > 0x7fffffffLL || ((uintptr_t)a->input & 15) || ((uintptr_t)a->weights & 15) || a->K % 64) return 0;
  void *ws;
  size_t wsb;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_ws[device].ptr || g_ws[device].bytes < (size_t)a->M * a->K * 2) return 0;
    ws = g_ws[device].ptr, wsb = g_ws[device].bytes;
  }
  int rc = 0;
  if (kind == 0) {
    if (a->dtype != LB200_BF16) return 0;
    rc = moe_launch<DenseRow, true, __nv_bfloat16, __nv_bfloat16>(a, DenseCtx{(const uint16_t *)a->weights}, ws, wsb, st);
  } else if (kind == 1) {
    if (a->K % 256) return 0;
    if (a->dtype == LB200_Q4_K)
      rc = moe_launch<Q4KRow, false, float, float>(a, GgufCtx{(const uint8_t *)a->weights}, ws, wsb, st);
    else if (a->dtype == LB200_Q6_K && ((size_t)(a->K >> 8) * 210) % 4 == 0)
      rc = moe_launch<Q6KRow, false, float, float>(a, GgufCtx{(const uint8_t *)a->weights}, ws, wsb, st);
    else if (a->dtype == LB200_Q8_0 && !((uintptr_t)a->weights & 15))
      rc = moe_launch<Q80Row, false, float, float>(a, GgufCtx{(const uint8_t *)a->weights}, ws, wsb, st);
    else
      return 0;
  } else {
    if (a->K % 128 || bC % 64 || bR <= 0 || a->N % bR || a->K % bC) return 0;
    const Fp8Ctx ctx{(const uint8_t *)a->weights, w_scale, bR, bC};
    if (a->dtype == LB200_BF16)
      rc = moe_launch<Fp8Row, true, __nv_bfloat16, __nv_bfloat16>(a, ctx, ws, wsb, st);
    else if (a->dtype == LB200_F32)
      rc = moe_launch<Fp8Row, false, float, float>(a, ctx, ws, wsb, st);
    else
      return 0;
  }
  return rc ? rc : 1;
}

int prefill_status(int device) {
  (void)device;
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_prefill_status, sizeof(int));
  return e == cudaSuccess ? v : -(int)e;
}

}  // namespace lb
