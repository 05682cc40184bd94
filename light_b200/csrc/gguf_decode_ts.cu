// Decode matmul for Q4_K weights and 1 .. 64 activation rows on the 5th-generation tensor cores, with the expanded
// weights handed to tcgen05.mma through TENSOR MEMORY (the A operand read from TMEM) instead of shared memory.
//
// A thread owns one weight ROW: it reads the row's 144-byte block from its warp's ring in shared memory, turns the
// 256 nibbles into f16 (LOP3 to 1024 + q or 64 + q, HADD2 to q - 8, HMUL2 with the sub-block's scale f16(d * sc):
// one rounding of a centred product), and stores them with tcgen05.st into its own TMEM lane, K along the columns.  Nothing
// is exchanged between lanes and no expanded weight touches shared memory; per 256 weights a thread issues about
// 450 instructions, half of what the register-fragment (mma.sync) kernels need.  The tokens are the N side of the MMA
// (16, 32 or 64 columns): their f16 image comes from a pre-pass, already in the 128-byte-swizzle layout the MMA's
// shared-memory descriptor reads, and reaches shared memory by ONE bulk copy (cp.async.bulk) per 256-element K
// block.  The sub-block constants (8 s - dmin * m_s) * sum_{k in s} x_k are two more K = 16 MMAs per block: A' = the constant as f16
// hi | lo against the sub-block sums of x as f16 hi | hi, then A' = hi | 0 against lo | 0.
//
//   warps 0-3   expanders: rows 32 w .. 32 w + 31 of the current group of 128 rows; they also read the finished
//               accumulator out of TMEM and store the output rows (or a split-K partial sum)
//   warp 4      one lane: bulk copies of the activations, and the MMAs (8 per half block + 2 for the minimum term)
//
// A sub-block pair (64 k, 32 TMEM columns) is one pipeline stage and a block's four pairs have a stage each, so the
// expanders run up to a block ahead of the tensor core.  The work list, the persistent
// grid, the equal runs and the deferred, ordered split-K fix-up are those of the token-tile kernels
// (gguf_decode_nt.cu).  Every wait is bounded: after 200 ms a waiter sets the status word and the CTA winds down,
// frees its tensor memory and exits.
#include "common.cuh"
#include "mma_sync.cuh"
#include "umma.cuh"

namespace lb {

namespace {

constexpr int EW = 4, THREADS = (EW + 1) * 32, ROWS = 16;  // four expander warps (a group of 128 rows) and the control warp
constexpr int S = 3;                       // weight tiles in flight per warp
constexpr int WTILE = 32 * 144;            // one K block of a warp's 32 rows
constexpr int MAX_GRID = 320;
constexpr int TMEM_COLS = 256, D_COL = 0, MIN_COL = 64, A_COL = 96, NSTG = 4;  // accumulator | 2 x 16 columns of minimum terms | four stages of 32 columns

struct TsArgs {  // up to four matrices that share x: their 16-row tiles form one list
  const uint8_t *w[4];
  float *out[4];
  int n[4];
  int tend[4];
  int count;
};

__device__ int g_ts_status;
__device__ unsigned int g_ts_epoch;
__device__ unsigned int g_ts_flags[MAX_GRID * 2 * EW];

__device__ __forceinline__ void resolve(const TsArgs &a, int T, int &j, int &r0) {
  j = 0;
  int base = 0;
#pragma unroll
  for (int i = 1; i < 4; i++)
    if (i < a.count && T >= a.tend[i - 1]) j = i, base = a.tend[i - 1];
  r0 = min((T - base) * ROWS, a.n[j] - ROWS);
}

__device__ __forceinline__ uint32_t h2u(__half2 v) { return *reinterpret_cast<uint32_t *>(&v); }
__device__ __forceinline__ __half2 u2h(uint32_t v) { return *reinterpret_cast<__half2 *>(&v); }

// ------------------------------------------------------------------------------------ pre-pass
// Image of one K block for NT tokens: five tiles of NT rows x 128 bytes in the 128-byte-swizzle layout (groups of 8
// rows 1024 bytes apart; 16-byte chunk j of row n at j ^ (n & 7)).  Tiles 0-3: the block's four runs of 64 values as
// f16, every four consecutive values in the order (0, 2, 1, 3) the expanded weights have.  Tile 4: chunk 0 and 1 =
// the eight sub-block sums as f16 hi, chunk 2 = their lo parts, chunk 3 = 0.  One warp per (block, token); lane l
// converts values 8 l .. 8 l + 7.
__global__ void __launch_bounds__(256) x_image_kernel(const float *__restrict__ x, uint8_t *__restrict__ img, int M, int NT, int K) {
  pdl_launch_dependents();
  const int rec = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  const int nb = K >> 8;
  pdl_wait();
  if (blockIdx.x == 0 && threadIdx.x == 0) atomicAdd(&g_ts_epoch, 1u);
  if (rec >= nb * NT) return;
  const int b = rec / NT, n = rec - b * NT;
  float4 v0 = make_float4(0.f, 0.f, 0.f, 0.f), v1 = v0;
  if (n < M) {
    const float4 *xp = reinterpret_cast<const float4 *>(x + (size_t)n * K + b * 256) + 2 * lane;
    v0 = __ldg(xp), v1 = __ldg(xp + 1);
  }
  const __half2 lim = __float2half2_rn(65504.f);
  auto cl = [&](float a, float c) { return __hmax2(__hmin2(__floats2half2_rn(a, c), lim), __hneg2(lim)); };
  const __half2 a02 = cl(v0.x, v0.z), a13 = cl(v0.y, v0.w), b02 = cl(v1.x, v1.z), b13 = cl(v1.y, v1.w);
  uint8_t *blk = img + (size_t)b * (5 * NT * 128);
  const uint32_t row = (uint32_t)(n >> 3) * 1024u + (uint32_t)(n & 7) * 128u, sw = (uint32_t)(n & 7);
  {
    const int tile = lane >> 3, j = lane & 7;
    *reinterpret_cast<uint4 *>(blk + (size_t)tile * (NT * 128) + row + ((j ^ sw) << 4)) = make_uint4(h2u(a02), h2u(a13), h2u(b02), h2u(b13));
  }
  const float2 f0 = __half22float2(a02), f1 = __half22float2(a13), f2 = __half22float2(b02), f3 = __half22float2(b13);
  float p = ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));  // of the ROUNDED values
  p += __shfl_xor_sync(0xffffffffu, p, 1), p += __shfl_xor_sync(0xffffffffu, p, 2);  // sub-block lane / 4
  float s[8];
#pragma unroll
  for (int i = 0; i < 8; i++) s[i] = __shfl_sync(0xffffffffu, p, 4 * i);
  if (lane < 8) {
    uint4 o = make_uint4(0u, 0u, 0u, 0u);
    if (lane < 3) {
      __half2 hi[4], lo[4];
#pragma unroll
      for (int i = 0; i < 4; i++) {
        hi[i] = cl(s[2 * i], s[2 * i + 1]);
        const float2 hf = __half22float2(hi[i]);
        lo[i] = cl(s[2 * i] - hf.x, s[2 * i + 1] - hf.y);
      }
      o = lane < 2 ? make_uint4(h2u(hi[0]), h2u(hi[1]), h2u(hi[2]), h2u(hi[3])) : make_uint4(h2u(lo[0]), h2u(lo[1]), h2u(lo[2]), h2u(lo[3]));
    }
    *reinterpret_cast<uint4 *>(blk + (size_t)4 * (NT * 128) + row + ((lane ^ sw) << 4)) = o;
  }
}

// ------------------------------------------------------------------------------------ PTX
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire(const unsigned int *p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release(unsigned int *p, unsigned int v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]: the A operand is read from tensor memory (lane = row, two f16 per column).
__device__ __forceinline__ void mma_ts_f16(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_ts_f16_acc(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc) {  // D += A * B
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.eq.b32 p, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc)
      : "memory");
}
// 32 registers of this thread -> 32 consecutive columns of its TMEM lane
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
      "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
      "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};\n" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
      "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

struct Run {  // the (group, block) list cut into G consecutive runs, one per CTA: q entries each (q > 0), or as even as possible
  int T, G, q, c, nb;
  __device__ __forceinline__ int begin(int cta) const { return q > 0 ? min(cta * q, T) : (int)((long long)T * cta / G); }
};

template <int NT>
struct TsCfg {
  static constexpr int XBUF = 5 * NT * 128;                        // one K block's image
  static constexpr int XS = NT <= 16 ? 3 : 2;                      // images in flight
  static constexpr int NACC = 64 / NT;                             // accumulators (64 columns in all): MMAs into one accumulator run one after
                                                                   // the other, and these MMAs are short, so the four stages of a block are spread over them
  static constexpr int SMEM = 1024 + XS * XBUF + EW * S * WTILE + 256;
};

template <int NT>
__device__ __forceinline__ float *part_of(float *parts, int cta, int slot, int warp) {
  return parts + ((size_t)(cta * 2 + slot) * EW + warp) * (NT * 32);
}

// ------------------------------------------------------------------------------------ main kernel
template <int NT>
__global__ void __launch_bounds__(THREADS, 2) q4k_ts_kernel(const uint8_t *__restrict__ img, float *__restrict__ parts, const __grid_constant__ TsArgs ma,
                                                          int tiles, int M, int K, int run_len) {
  constexpr int XS = TsCfg<NT>::XS, XBUF = TsCfg<NT>::XBUF;
  extern __shared__ unsigned char dyn_raw[];
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nb = K >> 8;
  const int groups = (tiles + 7) / 8;
  const Run run{groups * nb, (int)gridDim.x, run_len, (int)blockIdx.x, nb};
  const int it0 = run.begin(run.c), it1 = run.begin(run.c + 1), n = it1 - it0;
  const uint32_t sraw = (uint32_t)__cvta_generic_to_shared(dyn_raw);
  const uint32_t sbase = (sraw + 1023u) & ~1023u;  // the swizzled tiles want 1024-byte alignment
  unsigned char *gen = dyn_raw + (sbase - sraw);
  const uint32_t xring = sbase, wring = sbase + XS * XBUF, bars = wring + EW * S * WTILE;
  // barriers (8 bytes each): x_full[XS] x_empty[XS] a_full[4] a_empty[4] d_full d_empty, then the TMEM pointer and the flag
  const uint32_t x_full = bars, x_empty = bars + 8 * XS, a_full = bars + 16 * XS, a_empty = a_full + 8 * NSTG, d_full = a_full + 16 * NSTG, d_empty = d_full + 8;
  const uint32_t tptr = d_full + 16;
  volatile int *abort_flag = reinterpret_cast<volatile int *>(gen + XS * XBUF + EW * S * WTILE + 16 * XS + 16 * NSTG + 24);
  volatile uint32_t *tptr_gen = reinterpret_cast<volatile uint32_t *>(gen + XS * XBUF + EW * S * WTILE + 16 * XS + 16 * NSTG + 16);
  if (threadIdx.x == 0) {
#pragma unroll
    for (int i = 0; i < XS; i++) umma::mbar_init(x_full + 8 * i, 1), umma::mbar_init(x_empty + 8 * i, 1);
#pragma unroll
    for (int i = 0; i < NSTG; i++) umma::mbar_init(a_full + 8 * i, EW), umma::mbar_init(a_empty + 8 * i, 1);
    umma::mbar_init(d_full, 1), umma::mbar_init(d_empty, EW);
    *abort_flag = 0;
    umma::fence_barrier_init();
  }
  if (warp == EW) {
    umma::tmem_alloc(tptr, TMEM_COLS);
    umma::tmem_relinquish();
  }
  const uint32_t row_bytes = (uint32_t)nb * 144u;

  // ---- expander state: this warp's two 16-row tiles of the group at a list index
  struct At {
    const uint8_t *tile0[2];
    float *out[2];
    int r0[2], n[2];
    bool live[2];
  };
  auto at_group = [&](int grp) {
    At a;
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const int tile = grp * 8 + warp * 2 + h;
      int wj = 0, r0 = 0;
      a.live[h] = tile < tiles;
      if (a.live[h]) resolve(ma, tile, wj, r0);
      a.tile0[h] = ma.w[wj] + (size_t)r0 * row_bytes, a.out[h] = ma.out[wj], a.r0[h] = r0, a.n[h] = ma.n[wj];
    }
    return a;
  };
  int i_k = 0, i_blk = it0 % nb, i_grp = it0 / nb, i_slot = 0;
  At i_at;
  // a warp's tile of a K block is 288 chunks of 16 bytes: chunk c = lane + 32 i is piece c % 9 of row c / 9
  uint32_t roff[9], upper_rows = 0;
#pragma unroll
  for (int i = 0; i < 9; i++) {
    const uint32_t c = lane + 32 * i, r = c / 9u, piece = c - 9u * r;
    roff[i] = (r & 15u) * row_bytes + piece * 16u;
    upper_rows |= (r >= 16u ? 1u : 0u) << i;
  }
  auto issue = [&]() {  // always closes a commit group
    if (i_k < n) {
      const uint32_t dst = wring + (warp * S + i_slot) * WTILE + lane * 16;
      const uint32_t boff = (uint32_t)i_blk * 144u;
#pragma unroll
      for (int i = 0; i < 9; i++) {
        const bool hi = (upper_rows >> i) & 1u;
        if (hi ? i_at.live[1] : i_at.live[0]) cp_async16(dst + i * 512, (hi ? i_at.tile0[1] : i_at.tile0[0]) + (roff[i] + boff));
      }
      i_slot = i_slot + 1 == S ? 0 : i_slot + 1;
      i_k++;
      if (++i_blk == nb) {
        i_blk = 0, i_grp++;
        if (i_k < n) i_at = at_group(i_grp);
      }
    }
    cp_async_commit();
  };
  if (warp < EW) {
    i_at = at_group(i_grp);
#pragma unroll 1
    for (int p = 0; p < S; p++) issue();
  }
  umma::tc_fence_before();
  __syncthreads();  // barriers initialised, TMEM pointer written
  umma::tc_fence_after();
  const uint32_t tmem = *tptr_gen;
  pdl_wait();  // the activations' image is the pre-pass's output; the weights requested above are not
  const unsigned int epoch = *reinterpret_cast<volatile unsigned int *>(&g_ts_epoch);
  constexpr unsigned long long LIMIT = 200000000ull;

  if (warp == EW) {
    // ================================================================ control: x copies and MMAs, one lane
    if (lane == 0) {
      constexpr uint32_t idesc = umma::idesc_f16(128, NT, false);
      constexpr int NACC = TsCfg<NT>::NACC;
      int nf = 0;
      auto fetch = [&]() {
        const uint32_t h = (uint32_t)(nf % XS);
        umma::mbar_arrive_expect_tx(x_full + 8 * h, XBUF);
        bulk_g2s(xring + h * XBUF, img + (size_t)((it0 + nf) % nb) * XBUF, XBUF, x_full + 8 * h);
        nf++;
      };
      while (nf < n && nf < XS) fetch();
      int blk = it0 % nb, seg = 0;
      bool seg_first = true, ok = true;
      for (int k = 0; k < n && ok; k++) {
        while (nf < n && nf < k + XS) {  // refill: the buffer of block nf - XS is free once its MMAs have completed
          const uint32_t bar = x_empty + 8 * (uint32_t)(nf % XS), par = (uint32_t)((nf / XS - 1) & 1);
          if (umma::mbar_test_wait(bar, par)) { fetch(); continue; }
          if (nf > k) break;
          if (!umma::mbar_wait(bar, par, abort_flag, LIMIT)) { ok = false; break; }
        }
        if (!ok || !umma::mbar_wait(x_full + 8 * (uint32_t)(k % XS), (uint32_t)((k / XS) & 1), abort_flag, LIMIT)) { ok = false; break; }
        // descriptor of the block's image: every operand tile is this plus a constant number of 16-byte units
        const uint64_t xd = umma::smem_desc_sw128(xring + (uint32_t)(k % XS) * XBUF);
        const uint32_t kpar = (uint32_t)(k & 1);
#pragma unroll
        for (int p = 0; p < 4; p++) {  // sub-block pair p = stage p: values 64 p .. 64 p + 63 of the block
          if (!umma::mbar_wait(a_full + 8 * p, kpar, abort_flag, LIMIT)) { ok = false; break; }
          if (p == 0 && seg_first && !umma::mbar_wait(d_empty, (uint32_t)((seg & 1) ^ 1), abort_flag, LIMIT)) { ok = false; break; }
          umma::tc_fence_after();
          const uint32_t a0 = tmem + A_COL + 32 * p;
          const uint32_t dp = tmem + D_COL + (uint32_t)(p % NACC) * NT;  // this stage's accumulator
          if (p < NACC)
            mma_ts_f16(dp, a0, xd + (uint64_t)((p * (NT * 128)) >> 4), idesc, seg_first ? 0u : 1u);
          else
            mma_ts_f16_acc(dp, a0, xd + (uint64_t)((p * (NT * 128)) >> 4), idesc);
#pragma unroll
          for (int j = 1; j < 4; j++) mma_ts_f16_acc(dp, a0 + 8 * j, xd + (uint64_t)((p * (NT * 128) + j * 32) >> 4), idesc);
          if (p == 0) {  // the minimum term: (hi | lo) x (hi | hi), then (hi | 0) x (lo | 0)
            const uint32_t m0 = tmem + MIN_COL + 16 * kpar;
            mma_ts_f16_acc(dp, m0, xd + (uint64_t)((4 * (NT * 128)) >> 4), idesc);
            mma_ts_f16_acc(dp, m0 + 8, xd + (uint64_t)((4 * (NT * 128) + 32) >> 4), idesc);
          }
          umma::mma_commit(a_empty + 8 * p);
        }
        if (!ok) break;
        seg_first = false;
        umma::mma_commit(x_empty + 8 * (uint32_t)(k % XS));
        if (blk == nb - 1 || k == n - 1) umma::mma_commit(d_full), seg++, seg_first = true;
        blk = blk + 1 == nb ? 0 : blk + 1;
      }
      if (!ok) g_ts_status = 1;
    }
  } else {
    // ================================================================ expanders
    const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
    const uint32_t my_tile = wring + warp * S * WTILE + lane * 144;
    int slot = 0, blk = it0 % nb, grp = it0 / nb, seg_b0 = blk, seg = 0;
    At at = at_group(grp);
    int fix_grp = -1, pending = -1;  // pending: the stage whose stores have been issued but not yet handed over
    At fix_at = at;
    bool ok = true;
    const bool upper = lane >= 16;  // which of the warp's two tiles this thread's row belongs to
    auto my_out = [&](const At &a) { return upper ? a.out[1] : a.out[0]; };
    auto my_n = [&](const At &a) { return upper ? a.n[1] : a.n[0]; };
    auto my_r0 = [&](const At &a) { return upper ? a.r0[1] : a.r0[0]; };
    auto my_live = [&](const At &a) { return upper ? a.live[1] : a.live[0]; };
    for (int k = 0; k < n && ok; k++) {
      cp_async_wait<S - 1>();
      __syncwarp();
      const uint32_t src = my_tile + slot * WTILE;
      slot = slot + 1 == S ? 0 : slot + 1;
      const uint4 hd = lds128(src);
      uint4 q[8];
#pragma unroll
      for (int i = 0; i < 8; i++) q[i] = lds128(src + 16 + 16 * i);
      __syncwarp();  // the slot is free again
      issue();
      // ---- scales and minima of the eight sub-blocks
      const float2 df = __half22float2(u2h(hd.x));  // (d, dmin)
      const uint32_t scw[2] = {hd.y & 0x3F3F3F3Fu, (hd.w & 0x0F0F0F0Fu) | ((hd.y >> 2) & 0x30303030u)};
      const uint32_t mnw[2] = {hd.z & 0x3F3F3F3Fu, ((hd.w >> 4) & 0x0F0F0F0Fu) | ((hd.z >> 2) & 0x30303030u)};
      // A weight is (q - 8) * s with s = f16(d * sc): centred codes keep the products small, so their one rounding is
      // small against the result; the sub-block's constant 8 s - dmin * m goes with the minimum term (in f32, split hi | lo).
      __half2 s2[8];
      float sf[8];
      uint32_t amin[16];
#pragma unroll
      for (int s = 0; s < 8; s++) {
        const float sc = (float)((scw[s >> 2] >> (8 * (s & 3))) & 0xFFu);
        s2[s] = __float2half2_rn(df.x * sc);
        sf[s] = __low2float(s2[s]);  // the scale the tensor core multiplies with
      }
#pragma unroll
      for (int p = 0; p < 4; p++) {
        const float m0 = fmaf(8.f, sf[2 * p], -df.y * (float)((mnw[p >> 1] >> (16 * (p & 1))) & 0xFFu));
        const float m1 = fmaf(8.f, sf[2 * p + 1], -df.y * (float)((mnw[p >> 1] >> (16 * (p & 1) + 8)) & 0xFFu));
        const __half2 mh = __floats2half2_rn(m0, m1);
        const float2 mf = __half22float2(mh);
        amin[p] = h2u(mh), amin[4 + p] = h2u(__floats2half2_rn(m0 - mf.x, m1 - mf.y));
        amin[8 + p] = h2u(mh), amin[12 + p] = 0u;
      }
      const __half2 off_lo = __float2half2_rn(-1032.f), off_hi = __float2half2_rn(-72.f);  // (1024 + q) - 1032 = (64 + q) - 72 = q - 8
#pragma unroll
      for (int p = 0; p < 4; p++) {  // sub-block pair p -> stage p: low nibbles = sub-block 2p, high = 2p + 1
        const uint4 qa = q[2 * p], qb = q[2 * p + 1];
        const uint32_t wds[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
        const __half2 sl = s2[2 * p], sh = s2[2 * p + 1];
        uint32_t r[32];
#pragma unroll
        for (int w8 = 0; w8 < 8; w8++) {
          const uint32_t v = wds[w8], v8 = v >> 8;
          r[2 * w8] = h2u(__hmul2(__hadd2(u2h(and_or(v, 0x000F000Fu, 0x64006400u)), off_lo), sl));        // values 4 w, 4 w + 2 of sub-block 2p
          r[2 * w8 + 1] = h2u(__hmul2(__hadd2(u2h(and_or(v8, 0x000F000Fu, 0x64006400u)), off_lo), sl));   // 4 w + 1, 4 w + 3
          r[16 + 2 * w8] = h2u(__hmul2(__hadd2(u2h(and_or(v, 0x00F000F0u, 0x54005400u)), off_hi), sh));   // the same of sub-block 2p + 1
          r[16 + 2 * w8 + 1] = h2u(__hmul2(__hadd2(u2h(and_or(v8, 0x00F000F0u, 0x54005400u)), off_hi), sh));
        }
        // the stores of the stage before have had this expansion's time to land: hand that stage to the tensor core
        if (pending >= 0) {
          tmem_st_wait();
          umma::tc_fence_before();
          __syncwarp();
          if (lane == 0) umma::mbar_arrive(a_full + 8 * pending);
        }
        if (!umma::mbar_wait(a_empty + 8 * p, (uint32_t)((k & 1) ^ 1), abort_flag, LIMIT)) { ok = false; break; }
        umma::tc_fence_after();
        tmem_st32(lane_base + A_COL + 32 * p, r);
        if (p == 0) tmem_st16(lane_base + MIN_COL + 16 * (k & 1), amin);
        pending = p;
      }
      if (ok && (blk == nb - 1 || k == n - 1)) {  // nothing follows that would flush the last stage in time
        tmem_st_wait();
        umma::tc_fence_before();
        __syncwarp();
        if (lane == 0) umma::mbar_arrive(a_full + 8 * pending);
        pending = -1;
      }
      if (!ok) break;
      if (blk == nb - 1 || k == n - 1) {  // the run leaves this group: the accumulator is read out
        if (!umma::mbar_wait(d_full, (uint32_t)(seg & 1), abort_flag, LIMIT)) { ok = false; break; }
        umma::tc_fence_after();
        const bool whole = seg_b0 == 0 && blk == nb - 1;
        const bool first = k - (blk - seg_b0) == 0;
        float *dst = whole ? nullptr : part_of<NT>(parts, run.c, first ? 0 : 1, warp) + lane;
#pragma unroll
        for (int c0 = 0; c0 < NT; c0 += 16) {
          uint32_t v[16];
          umma::tmem_ld16(lane_base + D_COL + c0, v);
          umma::tmem_ld_wait();
#pragma unroll
          for (int a = 1; a < TsCfg<NT>::NACC; a++) {  // the other accumulators, in a fixed order
            uint32_t e[16];
            umma::tmem_ld16(lane_base + D_COL + a * NT + c0, e);
            umma::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; i++) v[i] = __float_as_uint(__uint_as_float(v[i]) + __uint_as_float(e[i]));
          }
          if (whole) {
            if (my_live(at)) {
              float *o = my_out(at) + my_r0(at) + (lane & 15);
              const size_t ld = (size_t)my_n(at);
#pragma unroll
              for (int i = 0; i < 16; i++)
                if (c0 + i < M) o[(size_t)(c0 + i) * ld] = __uint_as_float(v[i]);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 16; i++) __stcg(dst + (c0 + i) * 32, __uint_as_float(v[i]));
          }
        }
        umma::tc_fence_before();
        __syncwarp();
        if (lane == 0) umma::mbar_arrive(d_empty);
        if (!whole) {
          __threadfence();
          __syncwarp();
          if (lane == 0) st_release(&g_ts_flags[(run.c * 2 + (first ? 0 : 1)) * EW + warp], epoch);
          if (blk == nb - 1) fix_grp = grp, fix_at = at;
        }
        seg++;
        if (k + 1 < n) {
          grp++, blk = 0, seg_b0 = 0;
          at = at_group(grp);
        }
      } else {
        blk++;
      }
    }
    cp_async_wait<0>();
    if (!ok) g_ts_status = 1;
    // ---- the group whose end this CTA holds: the parts of the CTAs before it, in CTA order, then its own
    if (ok && fix_grp >= 0) {
      const int first = fix_grp * nb;
      int lo = run.q > 0 ? first / run.q : (int)((long long)first * run.G / run.T);
      while (lo > 0 && run.begin(lo) > first) lo--;
      while (run.begin(lo + 1) <= first) lo++;
      auto slot_of = [&](int cta) { return (cta == run.c || run.begin(cta) >= first) ? 0 : 1; };
      bool got = true;
      for (int base = lo; base < run.c && got; base += 32) {
        const int cta = base + lane;
        bool mine = true;
        if (cta < run.c) {
          const unsigned int *f = &g_ts_flags[(cta * 2 + slot_of(cta)) * EW + warp];
          const unsigned long long t0 = umma::global_ns();
          for (uint32_t i = 0; ld_acquire(f) != epoch; i++)
            if ((i & 63u) == 63u) {
              if (umma::global_ns() - t0 > LIMIT) { mine = false; break; }
              __nanosleep(100);
            }
        }
        got = __all_sync(0xffffffffu, mine);
      }
      if (!got) {
        g_ts_status = 2;
      } else {
        __threadfence();
        float acc[NT];
#pragma unroll
        for (int i = 0; i < NT; i++) acc[i] = 0.f;
        for (int cta = lo; cta <= run.c; cta++) {
          const float *p = part_of<NT>(parts, cta, slot_of(cta), warp) + lane;
#pragma unroll
          for (int i = 0; i < NT; i++) acc[i] += __ldcg(p + i * 32);
        }
        if (my_live(fix_at)) {
          float *o = my_out(fix_at) + my_r0(fix_at) + (lane & 15);
          const size_t ld = (size_t)my_n(fix_at);
#pragma unroll
          for (int i = 0; i < NT; i++)
            if (i < M) o[(size_t)i * ld] = acc[i];
        }
      }
    }
  }
  umma::tc_fence_before();
  __syncthreads();
  if (warp == EW) {
    umma::tc_fence_after();
    umma::tmem_dealloc(tmem, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------ launch
template <int NT>
int launch_ts(const uint8_t *img, float *parts, const TsArgs &ma, int tiles, int M, int K, int grid, int run_len, cudaStream_t st) {
  auto kern = q4k_ts_kernel<NT>;
  static DeviceOnce attr_done;
  {
    cudaError_t e = attr_done.ensure([&] { return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, TsCfg<NT>::SMEM); });
    if (e != cudaSuccess) return fail((int)e, "light_b200: matmul_q (decode, tensor memory): %s", cudaGetErrorString(e));
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = TsCfg<NT>::SMEM;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, img, parts, ma, tiles, M, K, run_len);
  if (e != cudaSuccess) return fail((int)e, "light_b200: matmul_q (decode, tensor memory): %s", cudaGetErrorString(e));
  return launched("matmul_q (decode, tensor memory)");
}

int nt_of(int M) { return M <= 16 ? 16 : M <= 32 ? 32 : 64; }
size_t image_bytes(int M, int K) { return ((size_t)(K >> 8) * 5 * nt_of(M) * 128 + 1023) & ~(size_t)1023; }
size_t parts_bytes(int M) { return (size_t)MAX_GRID * 2 * EW * nt_of(M) * 32 * sizeof(float); }

// LIGHT_B200_TS=1 switches the path on (_TS_MIN_M, _TS_MAX_M, _TS_GRID: tuning knobs).  It is off by default: alone, on
// matrices of 28672 and 128256 rows, it beats the register-fragment kernels from 17 rows up (35 against 41 us and 115
// against 152 us at 32 rows), but inside a decode step the two are level, and its weights carry two f16 roundings
// (5e-4 relative L2 against 2e-4).
int g_ts_on = -1, g_ts_min_m = 1, g_ts_max_m = 64, g_ts_grid = 0;

}  // namespace

int decode_ts_status() {
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_ts_status, sizeof(v));
  if (e != cudaSuccess) return fail((int)e, "light_b200: decode status: %s", cudaGetErrorString(e));
  return v;
}

size_t decode_ts_ws_bytes(int M, int K) { return image_bytes(M, K) + parts_bytes(M); }

// `count` (1..4) Q4_K matrices that share x (M rows, 1 .. 64).  `ws`: at least decode_ts_ws_bytes(M, K) bytes, 1024-byte
// aligned, untouched until the launches have run.  Returns 1 if launched, 0 if the shape is not covered, else an error.
int gguf_decode_ts(int type, const float *x, const void *const *w, float *const *out, const int *n, int count, int M, int K, void *ws,
                   size_t ws_bytes, cudaStream_t st) {
  if (g_ts_on < 0) {
    g_ts_on = getenv("LIGHT_B200_TS") ? atoi(getenv("LIGHT_B200_TS")) : 0;
    if (const char *e = getenv("LIGHT_B200_TS_MIN_M")) g_ts_min_m = atoi(e);
    if (const char *e = getenv("LIGHT_B200_TS_MAX_M")) g_ts_max_m = atoi(e);
    if (const char *e = getenv("LIGHT_B200_TS_GRID")) g_ts_grid = atoi(e);
  }
  if (!g_ts_on || type != LB200_Q4_K || M < g_ts_min_m || M > g_ts_max_m || M < 1 || M > 64 || K % 256 || count < 1 || count > 4 || ((uintptr_t)x & 15) ||
      !ws || ((uintptr_t)ws & 1023) || ws_bytes < decode_ts_ws_bytes(M, K))
    return 0;
  TsArgs a = {};
  int tiles = 0;
  for (int i = 0; i < count; i++) {
    if (n[i] < ROWS || ((uintptr_t)w[i] & 15)) return 0;
    tiles += (n[i] + ROWS - 1) / ROWS;
    a.w[i] = (const uint8_t *)w[i], a.out[i] = out[i], a.n[i] = n[i], a.tend[i] = tiles;
  }
  a.count = count;
  const int NT = nt_of(M), nb = K >> 8;
  const int sms = sm_count(), slots = sms * 2;
  const long long T = (long long)((tiles + 7) / 8) * nb;
  if (T >= (1ll << 30)) return 0;
  long long limit = T / 4 > sms ? T / 4 : (T < sms ? T : sms);
  if (limit > slots) limit = slots;
  if (g_ts_grid > 0) limit = g_ts_grid < T ? g_ts_grid : T;
  if (limit > MAX_GRID) limit = MAX_GRID;
  int run_len = 0;
  long long grid = limit;
  {
    const int q = (int)((T + limit - 1) / limit);
    if (limit <= sms && q <= nb && nb % q == 0) run_len = q, grid = (T + q - 1) / q;
  }
  {
    const int recs = nb * NT;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((recs + 7) / 8));
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, x_image_kernel, x, (uint8_t *)ws, M, NT, K);
    if (e != cudaSuccess) return fail((int)e, "light_b200: matmul_q (decode, activations' image): %s", cudaGetErrorString(e));
    if (int rc = launched("matmul_q (decode, activations' image)")) return rc;
  }
  float *parts = reinterpret_cast<float *>((uint8_t *)ws + image_bytes(M, K));
  const int rc = NT == 16   ? launch_ts<16>((const uint8_t *)ws, parts, a, tiles, M, K, (int)grid, run_len, st)
                 : NT == 32 ? launch_ts<32>((const uint8_t *)ws, parts, a, tiles, M, K, (int)grid, run_len, st)
                            : launch_ts<64>((const uint8_t *)ws, parts, a, tiles, M, K, (int)grid, run_len, st);
  return rc ? rc : 1;
}

}  // namespace lb
