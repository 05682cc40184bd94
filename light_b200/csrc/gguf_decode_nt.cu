// Batched decode, 2 .. 64 activation rows (tokens): fused dequant-matmul for Q4_K and Q6_K with the tokens as
// MMA columns and the activations staged ONCE per call.
//
//   pre-pass   x (M, K) f32 -> f16 in the order the B fragments are read, one 544-byte record per (K block,
//              token): 512 bytes of values and, for Q4_K, the eight sub-block sums as f16 hi | lo.  Tokens are
//              padded to a multiple of eight with zeros.  One warp per record.
//   main       the work is the list of (group of eight row tiles, K block) pairs, group-major; a persistent grid
//              (one or two CTAs per SM) cuts the list into equal consecutive runs, so every SM gets the same
//              number of blocks whatever the matrix's height.  A CTA of eight warps walks its run: warp w owns
//              row tile w of the current group.  Per block ONE bulk copy (cp.async.bulk, completion on an
//              mbarrier) brings all tokens' records into a ring shared by the eight warps, who hand a buffer back
//              through a second mbarrier (no CTA-wide barrier in the loop); the weights arrive through a per-warp
//              ring of 16-byte asynchronous copies and are expanded in registers straight into A fragments
//              (Q4_K: LOP3 to f16 (64 + q), one HFMA2 with the 6-bit scale; Q6_K: PRMT to f16 (1024 + code),
//              offset and scale by HADD2 / HMUL2), so an expanded weight never touches shared memory and serves
//              NG groups of eight tokens.  Once per block and row, acc += d * D.
//   split K    a run that starts or ends inside a group leaves a partial sum.  Partial sums go to the workspace
//              with a per-warp flag carrying the call's epoch; the CTA that holds the END of a group adds the
//              parts of the CTAs before it, in CTA order, after it has finished its own run (by then they are
//              there; the wait is bounded) and stores the rows.
//
// Every sum has a fixed order (k inside an MMA, blocks ascending inside a run, runs in CTA order), so results are
// deterministic.  x is rounded to f16 once (2^-11 relative per element, about 2e-4 relative L2 on the output).
#include <cuda_fp8.h>

#include <type_traits>

#include "common.cuh"
#include "mma_sync.cuh"
#include "umma.cuh"

namespace lb {

namespace {

constexpr int ROWS = 16, CW = 8, THREADS = CW * 32;
constexpr int TOK_PITCH = 544;  // bytes per (block, token) record: 512 of f16 + 32 (sub-block sums; bank spread)

struct NtArgs {  // up to four matrices that share x: their row tiles form one list
  const uint8_t *w[4];
  float *out[4];   // bf16 rows when out_bf16 is set
  int n[4];
  int tend[4];
  int count;
  int out_bf16;
  const float *scales[4], *zeros[4];  // group-quantized 4-bit only: (n, K / 128) each
};

struct TileAt {  // where a list index lies for one warp: its row tile
  bool live;
  int wj, r0;
  const uint8_t *tile0, *w_end;
  const float *sc, *zp;  // 4-bit only: the scale / zero rows of the tile's first row
};

__device__ int g_nt_status;  // non-zero: a bounded wait (a block of activations, a partial sum) gave up (sticky)

// Split-K bookkeeping of the persistent grid, in the library's own device memory (zero at load, never handed out):
// the epoch of the current call (bumped by the staging launch) and one flag per (CTA, first | last run, warp).
constexpr int MAX_GRID = 320;
__device__ unsigned int g_nt_epoch;
__device__ unsigned int g_nt_flags[MAX_GRID * 2 * 8];

__device__ __forceinline__ void resolve(const NtArgs &a, int T, int &j, int &r0) {
  j = 0;
  int base = 0;
#pragma unroll
  for (int i = 1; i < 4; i++)
    if (i < a.count && T >= a.tend[i - 1]) j = i, base = a.tend[i - 1];
  r0 = min((T - base) * ROWS, a.n[j] - ROWS);  // the last tile is pulled back: duplicate rows store equal values
}

__device__ __forceinline__ uint32_t h2u(__half2 v) { return *reinterpret_cast<uint32_t *>(&v); }
__device__ __forceinline__ __half2 u2h(uint32_t v) { return *reinterpret_cast<__half2 *>(&v); }

// ------------------------------------------------------------------------------------ pre-pass
// PAIR (Q4_K): the 8-byte group F (elements 4F .. 4F+3 as (x0, x2), (x1, x3)) lands at slot
// ((F / 8 & 1) * 8 + (F & 7)) * 4 + F / 16, so that lane (token g, t) finds pair t's low-nibble sub-block at
// i * 32 + t * 8 and its high-nibble sub-block 256 bytes further.  Otherwise (Q6_K) natural order.
// LAYOUT 2 (4-bit, canonical layout): a code word holds eight consecutive k, and a lane's two values of an MMA k slot
// pair are nibbles t and t + 4 of one word, so the 16 values of k step s lie as [t][j]: value 16 s + 4 j + t.
__device__ __forceinline__ float4 ld_x4(const float *p) { return __ldg(reinterpret_cast<const float4 *>(p)); }
__device__ __forceinline__ float4 ld_x4(const __nv_bfloat16 *p) {
  const uint2 u = __ldg(reinterpret_cast<const uint2 *>(p));
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&u.x)), b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&u.y));
  return make_float4(a.x, a.y, b.x, b.y);
}

template <int LAYOUT, typename XT>
__global__ void __launch_bounds__(THREADS) x_stage_kernel(const XT *__restrict__ x, uint8_t *__restrict__ xs, int M, int NT, int K) {
  constexpr bool PAIR = LAYOUT == 1;
  pdl_launch_dependents();
  const int rec = blockIdx.x * CW + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  const int nb = K >> 8;
  pdl_wait();  // x is the previous launch's output, and the launch before may still read the staging buffer
  if (blockIdx.x == 0 && threadIdx.x == 0) atomicAdd(&g_nt_epoch, 1u);  // a new call: flags of earlier calls no longer match
  if (rec >= nb * NT) return;
  const int b = rec / NT, tk = rec - b * NT;
  uint8_t *dst = xs + (size_t)rec * TOK_PITCH;
  float4 v[2];
  v[0] = v[1] = make_float4(0.f, 0.f, 0.f, 0.f);
  if (tk < M) {
    const XT *xp = x + (size_t)tk * K + b * 256;
    v[0] = ld_x4(xp + 4 * lane), v[1] = ld_x4(xp + 4 * (lane + 32));
  }
  float s[2];
#pragma unroll
  for (int j = 0; j < 2; j++) {
    const int F = lane + 32 * j;
    const __half2 lim = __float2half2_rn(65504.f);
    const __half2 h02 = __hmax2(__hmin2(__floats2half2_rn(v[j].x, v[j].z), lim), __hneg2(lim));
    const __half2 h13 = __hmax2(__hmin2(__floats2half2_rn(v[j].y, v[j].w), lim), __hneg2(lim));
    if constexpr (LAYOUT == 3) {
      // values 4 F .. 4 F + 3 = 64-byte chunk c = F / 16, granule t = (F / 4) % 4, word j = F % 4 of a weight row:
      // k step 4 c + j, lane t -> 8 bytes at (k step) * 32 + t * 8, in the order (0, 1, 2, 3)
      const int c = F >> 4, tt = (F >> 2) & 3, jj = F & 3;
      const __half2 h01 = __halves2half2(__low2half(h02), __low2half(h13)), h23 = __halves2half2(__high2half(h02), __high2half(h13));
      *reinterpret_cast<uint2 *>(dst + (4 * c + jj) * 32 + tt * 8) = make_uint2(h2u(h01), h2u(h23));
    } else if constexpr (LAYOUT == 2) {
      // values 4 F .. 4 F + 3 = k step F / 4, j = F % 4, t = 0 .. 3: four 2-byte stores, 8 bytes apart
      __half *o = reinterpret_cast<__half *>(dst) + (F >> 2) * 16 + (F & 3);
      o[0] = __low2half(h02), o[4] = __low2half(h13), o[8] = __high2half(h02), o[12] = __high2half(h13);
    } else {
      const int P = PAIR ? (((F >> 3) & 1) * 8 + (F & 7)) * 4 + (F >> 4) : F;
      *reinterpret_cast<uint2 *>(dst + P * 8) = make_uint2(h2u(h02), h2u(h13));
    }
    const float2 a = __half22float2(h02), c = __half22float2(h13);
    float p = (a.x + a.y) + (c.x + c.y);  // of the ROUNDED values, the ones the tensor core multiplies
    p += __shfl_xor_sync(0xffffffffu, p, 1), p += __shfl_xor_sync(0xffffffffu, p, 2), p += __shfl_xor_sync(0xffffffffu, p, 4);
    s[j] = p;  // sub-block lane / 8 + 4 j
  }
  const float n0 = __shfl_down_sync(0xffffffffu, s[0], 8), n1 = __shfl_down_sync(0xffffffffu, s[1], 8);
  if ((lane & 15) == 0) {  // lanes 0 / 16: sub-block pairs (0,1) (4,5) / (2,3) (6,7)
#pragma unroll
    for (int j = 0; j < 2; j++) {
      const float a0 = s[j], a1 = j ? n1 : n0;
      const __half2 lim = __float2half2_rn(65504.f);  // sums of clamped values can leave the f16 range too
      const __half2 hi = __hmax2(__hmin2(__floats2half2_rn(a0, a1), lim), __hneg2(lim));
      const float2 hf = __half22float2(hi);
      const __half2 lo = __hmax2(__hmin2(__floats2half2_rn(a0 - hf.x, a1 - hf.y), lim), __hneg2(lim));
      uint32_t *at = reinterpret_cast<uint32_t *>(dst + 512 + 4 * ((lane >> 4) + 2 * j));
      at[0] = PAIR ? h2u(hi) : 0u, at[4] = PAIR ? h2u(lo) : 0u;
    }
  }
}

// ------------------------------------------------------------------------------------ shared skeleton
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

// The ring of staged activations: XS buffers, each with a `full` mbarrier (one arrival + the copy's bytes) and an
// `empty` mbarrier (one arrival per warp).  Thread 0 is the producer; it refills a buffer as soon as all warps have
// handed it back, looking at the barrier without blocking except when its own warp needs the block.
template <int NG, int XS_CAP = 4>
struct XFeed {
  static constexpr int NT = 8 * NG, XBUF = NT * TOK_PITCH;
  static constexpr int XS_WANT = NG <= 2 ? 4 : NG == 4 ? 3 : 2;
  static constexpr int XS = XS_WANT < XS_CAP ? XS_WANT : XS_CAP;  // a format with large weight tiles caps the ring: two CTAs must fit an SM
  static constexpr int BYTES = XS * XBUF + 128;
  uint32_t buf0, full0, empty0;
  const uint8_t *xs;
  volatile int *abort_flag;
  int nf, n, nb, it0;  // next block to fetch (local index), blocks in this CTA's run
  __device__ __forceinline__ void init(uint32_t base, unsigned char *gen, const uint8_t *xs_, int it0_, int n_, int nb_) {
    buf0 = base, full0 = base + XS * XBUF, empty0 = full0 + 8 * XS, xs = xs_, nf = 0, n = n_, nb = nb_, it0 = it0_;
    abort_flag = reinterpret_cast<volatile int *>(gen + XS * XBUF + 16 * XS);
    if (threadIdx.x == 0) {
#pragma unroll
      for (int i = 0; i < XS; i++) umma::mbar_init(full0 + 8 * i, 1), umma::mbar_init(empty0 + 8 * i, CW);
      *abort_flag = 0;
      umma::fence_barrier_init();
    }
  }
  __device__ __forceinline__ uint32_t buf(int k) const { return buf0 + (uint32_t)(k % XS) * XBUF; }
  __device__ __forceinline__ void fetch() {  // thread 0: block nf of the run
    const uint32_t h = (uint32_t)(nf % XS);
    umma::mbar_arrive_expect_tx(full0 + 8 * h, XBUF);
    bulk_g2s(buf0 + h * XBUF, xs + (size_t)((it0 + nf) % nb) * XBUF, XBUF, full0 + 8 * h);
    nf++;
  }
  __device__ __forceinline__ void start() {  // thread 0, after the barriers are visible and x is staged
    while (nf < n && nf < XS) fetch();
  }
  // thread 0, before its warp waits for block k: refill what is free; block for the buffer only if block k itself
  // has not been requested yet
  __device__ __forceinline__ void pump(int k) {
    while (nf < n) {
      const uint32_t bar = empty0 + 8 * (uint32_t)(nf % XS), par = (uint32_t)((nf / XS - 1) & 1);
      if (umma::mbar_test_wait(bar, par)) { fetch(); continue; }
      if (nf > k) break;
      if (!umma::mbar_wait(bar, par, abort_flag, 200000000ull)) { g_nt_status = 1; break; }
    }
  }
  __device__ __forceinline__ bool wait_full(int k) const {
    const bool ok = umma::mbar_wait(full0 + 8 * (uint32_t)(k % XS), (uint32_t)((k / XS) & 1), abort_flag, 200000000ull);
    if (!ok) g_nt_status = 1;
    return ok;
  }
  __device__ __forceinline__ void release(int k, int lane) const {  // the warp is done reading block k
    __syncwarp();
    if (lane == 0) umma::mbar_arrive(empty0 + 8 * (uint32_t)(k % XS));
  }
};

struct Run {  // the (group, block) list cut into G consecutive runs, one per CTA: q entries each (q > 0), or as even as possible
  int T, G, q, c, nb;
  __device__ __forceinline__ int begin(int cta) const { return q > 0 ? min(cta * q, T) : (int)((long long)T * cta / G); }
};

// acc -> out rows of one tile: lane (g, t) holds rows g, g+8 x tokens 2t, 2t+1 of every group of eight
template <int NG>
__device__ __forceinline__ void store_tile(const float (&acc)[NG][4], float *out, bool bf16, int n, int r0, int M, int g, int t) {
#pragma unroll
  for (int q = 0; q < NG; q++)
#pragma unroll
    for (int c = 0; c < 4; c++) {
      const int tok = q * 8 + 2 * t + (c & 1), row = r0 + g + 8 * (c >> 1);
      if (tok < M) {
        if (bf16)
          reinterpret_cast<__nv_bfloat16 *>(out)[(size_t)tok * n + row] = __float2bfloat16_rn(acc[q][c]);
        else
          out[(size_t)tok * n + row] = acc[q][c];
      }
    }
}

template <int NG>
__device__ __forceinline__ float *part_of(float *parts, int cta, int slot, int warp) {
  return parts + ((size_t)(cta * 2 + slot) * CW + warp) * (NG * 4 * 32);
}

template <int NG>
__device__ __forceinline__ void write_part(const float (&acc)[NG][4], float *parts, int cta, int slot, int warp, int lane, unsigned int epoch) {
  float *p = part_of<NG>(parts, cta, slot, warp) + lane;
#pragma unroll
  for (int q = 0; q < NG; q++)
#pragma unroll
    for (int c = 0; c < 4; c++) __stcg(p + (q * 4 + c) * 32, acc[q][c]);
  __threadfence();
  __syncwarp();
  if (lane == 0) st_release(&g_nt_flags[(cta * 2 + slot) * CW + warp], epoch);
}

// The group whose end this CTA holds: parts of the CTAs before it (in CTA order), then its own, -> acc.  The flags
// are polled by one lane each, all at once; the parts are fetched several CTAs at a time and added in order.
template <int NG>
__device__ __forceinline__ void fix_up(const Run &run, int grp, float *parts, int warp, int lane, unsigned int epoch, float (&acc)[NG][4]) {
  const int first = grp * run.nb;  // the group's first list index
  int lo = run.q > 0 ? first / run.q : (int)((long long)first * run.G / run.T);
  while (lo > 0 && run.begin(lo) > first) lo--;
  while (run.begin(lo + 1) <= first) lo++;
  auto slot_of = [&](int cta) { return (cta == run.c || run.begin(cta) >= first) ? 0 : 1; };  // its first run, or (it began in an earlier group) its last
  for (int base = lo; base < run.c; base += 32) {
    const int cta = base + lane;
    bool ok = true;
    if (cta < run.c) {
      const unsigned int *f = &g_nt_flags[(cta * 2 + slot_of(cta)) * CW + warp];
      const unsigned long long t0 = umma::global_ns();
      for (uint32_t i = 0; ld_acquire(f) != epoch; i++)
        if ((i & 63u) == 63u) {
          if (umma::global_ns() - t0 > 200000000ull) { ok = false; break; }
          __nanosleep(100);
        }
    }
    if (!__all_sync(0xffffffffu, ok)) { g_nt_status = 2; return; }
  }
  __threadfence();
#pragma unroll
  for (int q = 0; q < NG; q++) acc[q][0] = acc[q][1] = acc[q][2] = acc[q][3] = 0.f;
  constexpr int AT = NG <= 2 ? 4 : NG == 4 ? 2 : 1;  // CTAs whose parts are in flight together
  for (int base = lo; base <= run.c; base += AT) {
    float v[AT][NG * 4];
#pragma unroll
    for (int a = 0; a < AT; a++) {
      const int cta = min(base + a, run.c);
      const float *p = part_of<NG>(parts, cta, slot_of(cta), warp) + lane;
#pragma unroll
      for (int i = 0; i < NG * 4; i++) v[a][i] = __ldcg(p + i * 32);
    }
#pragma unroll
    for (int a = 0; a < AT; a++)
      if (base + a <= run.c)
#pragma unroll
        for (int i = 0; i < NG * 4; i++) acc[i >> 2][i & 3] += v[a][i];
  }
}

// ------------------------------------------------------------------------------------ Q4_K
// Lane (g, t) holds the 32 code bytes of sub-block pair t of rows g and g+8.  Code word i gives one MMA for
// sub-block 2t (low nibbles) and one for 2t+1 (high nibbles).  The minimum term -dmin * m_s * sum_{k in s} x_k
// is a second small contraction over the eight sub-blocks: A' = -dmin * m as f16 hi + lo, B' = the sub-block
// sums of x as f16 hi (both k halves), then A' = hi against the lo half of the sums.
struct Q4Fmt {
  static constexpr int S = 3, TILE = ROWS * 144, BLOCK = 144, XS_CAP = 4;
  uint32_t soff[5], ld_off, hdr_sh;
  bool hdr_hi;
  __device__ __forceinline__ void setup(int lane, uint32_t row_bytes) {
#pragma unroll
    for (int i = 0; i < 5; i++) {
      const uint32_t c = lane + 32 * i, row = c / 9u;
      soff[i] = row * row_bytes + (c - 9u * row) * 16u;
    }
    const int g = lane >> 2, t = lane & 3;
    ld_off = g * 144u + 32u * t, hdr_hi = t >= 2, hdr_sh = (t & 1) * 16;
  }
  __device__ __forceinline__ void issue(uint32_t dst, const uint8_t *tile0, uint32_t blk, int lane, const uint8_t *) const {
    const uint8_t *base = tile0 + blk * 144u;
    dst += lane * 16;
#pragma unroll
    for (int i = 0; i < 4; i++) cp_async16(dst + i * 512, base + soff[i]);
    if (lane < 16) cp_async16(dst + 2048, base + soff[4]);
  }
  template <int NG, typename F>
  __device__ __forceinline__ void unit(uint32_t slot_addr, uint32_t xb, float (&acc)[NG][4], const TileAt &, uint32_t, int lane, F &&slot_free) const {
    const int g = lane >> 2, t = lane & 3;
    const uint32_t mask = 0x00F000F0u, magic = 0x54005400u;  // f16 (64 + nibble)
    const uint32_t sb = slot_addr + ld_off;
    const uint4 h0 = lds128(sb - 32u * t), h1 = lds128(sb - 32u * t + 8 * 144);
    const uint4 qa0 = lds128(sb + 16), qa1 = lds128(sb + 32);
    const uint4 qb0 = lds128(sb + 8 * 144 + 16), qb1 = lds128(sb + 8 * 144 + 32);
    __syncwarp();  // the slot is free again
    slot_free();
    __half2 s2[2][2], c2[2][2];
    uint32_t dmh[2], dml[2];
    float dd[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
      const uint4 &h = r ? h1 : h0;
      const float2 df = __half22float2(u2h(h.x));  // (d, dmin)
      const uint32_t scw = hdr_hi ? ((h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u)) : (h.y & 0x3F3F3F3Fu);
      const uint32_t mnw = hdr_hi ? (((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u)) : (h.z & 0x3F3F3F3Fu);
      const uint32_t sc = scw >> hdr_sh, mn = mnw >> hdr_sh;
      s2[r][0] = __half2half2(__uint2half_rn(sc & 0xFFu)), s2[r][1] = __half2half2(__uint2half_rn((sc >> 8) & 0xFFu));
      c2[r][0] = __hmul2(s2[r][0], __float2half2_rn(-64.f)), c2[r][1] = __hmul2(s2[r][1], __float2half2_rn(-64.f));
      const float m0 = -df.y * (float)(mn & 0xFFu), m1 = -df.y * (float)((mn >> 8) & 0xFFu);
      const __half2 mh = __floats2half2_rn(m0, m1);
      const float2 mf = __half22float2(mh);
      dmh[r] = h2u(mh), dml[r] = h2u(__floats2half2_rn(m0 - mf.x, m1 - mf.y));
      dd[r] = df.x;
    }
    float dq[NG][4];
#pragma unroll
    for (int q = 0; q < NG; q++) dq[q][0] = dq[q][1] = dq[q][2] = dq[q][3] = 0.f;
    const uint32_t qg[8] = {qa0.x, qa0.y, qa0.z, qa0.w, qa1.x, qa1.y, qa1.z, qa1.w};
    const uint32_t qh[8] = {qb0.x, qb0.y, qb0.z, qb0.w, qb1.x, qb1.y, qb1.z, qb1.w};
    auto scl = [](uint32_t raw, __half2 s, __half2 c) { return h2u(__hfma2(u2h(raw), s, c)); };  // (64 + q) sc - 64 sc, exact
    const uint32_t bx = xb + g * TOK_PITCH + t * 8;  // B fragments of token g of group 0
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const uint32_t vg = qg[i], vh = qh[i];
      const uint32_t e0 = scl(and_or(vg << 4, mask, magic), s2[0][0], c2[0][0]), e1 = scl(and_or(vh << 4, mask, magic), s2[1][0], c2[1][0]);
      const uint32_t e2 = scl(and_or(vg >> 4, mask, magic), s2[0][0], c2[0][0]), e3 = scl(and_or(vh >> 4, mask, magic), s2[1][0], c2[1][0]);
      const uint32_t o0 = scl(and_or(vg, mask, magic), s2[0][1], c2[0][1]), o1 = scl(and_or(vh, mask, magic), s2[1][1], c2[1][1]);
      const uint32_t o2 = scl(and_or(vg >> 8, mask, magic), s2[0][1], c2[0][1]), o3 = scl(and_or(vh >> 8, mask, magic), s2[1][1], c2[1][1]);
#pragma unroll
      for (int q = 0; q < NG; q++) {
        const uint2 be = lds64(bx + q * (8 * TOK_PITCH) + i * 32), bo = lds64(bx + q * (8 * TOK_PITCH) + (8 + i) * 32);
        mma16816(dq[q], e0, e1, e2, e3, be.x, be.y);
        mma16816(dq[q], o0, o1, o2, o3, bo.x, bo.y);
      }
    }
#pragma unroll
    for (int q = 0; q < NG; q++) {
      acc[q][0] = fmaf(dd[0], dq[q][0], acc[q][0]), acc[q][1] = fmaf(dd[0], dq[q][1], acc[q][1]);
      acc[q][2] = fmaf(dd[1], dq[q][2], acc[q][2]), acc[q][3] = fmaf(dd[1], dq[q][3], acc[q][3]);
      const uint32_t sx = xb + (q * 8 + g) * TOK_PITCH + 512 + 4 * t;
      const uint32_t sx_hi = lds32(sx), sx_lo = lds32(sx + 16);
      mma16816(acc[q], dmh[0], dmh[1], dml[0], dml[1], sx_hi, sx_hi);
      mma16816(acc[q], dmh[0], dmh[1], 0u, 0u, sx_lo, 0u);
    }
  }
};

// ------------------------------------------------------------------------------------ Q6_K
// Block (210 B): [ql[128] | qh[64] | int8 sc[16] | f16 d]; element e = 128h + 32q + l has its low nibble in
// ql[64h + 32(q&1) + l] (high nibble when q >= 2) and bits 2q..2q+1 of qh[32h + l]; its sub-block of 16 is
// 8h + 2q + l/16.  For each (h, u = l/16), lane (g, t) takes l = 16u + 4t .. +3 of rows g and g+8: one word of
// ql[64h + l], one of ql[64h + 32 + l], one of qh[32h + l].  Group q feeds ONE MMA whose 16 k slots are exactly
// sub-block m = 8h + 2q + u.  A row's block is copied as the 14 granules that cover it, to a 240-byte pitch; it
// begins `skew` = (its byte offset & 15) bytes into the row's slot: a multiple of 4 for even blocks and 2 mod 4
// for odd ones (rows hold an even number of blocks), where a word is two aligned words funnel-shifted.
__device__ __forceinline__ uint32_t lds16u(uint32_t addr) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];\n" : "=h"(v) : "r"(addr));
  return v;
}
template <bool ODD>
__device__ __forceinline__ uint32_t lds32s(uint32_t addr) {  // word at a 2-byte aligned shared address
  if constexpr (!ODD) return lds32(addr);
  return __funnelshift_r(lds32(addr - 2), lds32(addr + 2), 16);
}

struct Q6Fmt {
  static constexpr int S = 2, PITCH = 240, TILE = ROWS * PITCH, BLOCK = 210, XS_CAP = 4;
  uint32_t row_bytes, c_rsub, c_piece;
  __device__ __forceinline__ void setup(int lane, uint32_t row_bytes_) { row_bytes = row_bytes_, c_rsub = lane >> 4, c_piece = lane & 15; }
  // tile0 = first byte of the tile's first row; the copy never reads past w_end (the last rows of a matrix)
  __device__ __forceinline__ void issue(uint32_t dst, const uint8_t *tile0, uint32_t blk, int, const uint8_t *w_end) const {
    if (c_piece >= 14) return;
    const uint8_t *row = tile0 + (size_t)c_rsub * row_bytes + blk * 210u;
    dst += c_rsub * PITCH + c_piece * 16;
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const uint8_t *src = reinterpret_cast<const uint8_t *>(reinterpret_cast<uintptr_t>(row) & ~(uintptr_t)15) + c_piece * 16;
      const long long left = w_end - src;
      if (left >= 16)
        cp_async16(dst, src);
      else if (left > 0)
        cp_async16_part(dst, src, (uint32_t)left);
      row += 2 * (size_t)row_bytes, dst += 2 * PITCH;
    }
  }
  template <int NG, bool ODD, typename F>
  __device__ __forceinline__ void unit_p(uint32_t sb, uint32_t xb, float (&acc)[NG][4], uint32_t skew, int lane, F &&slot_free) const {
    const int g = lane >> 2, t = lane & 3;
    const uint32_t m0f = 0x0F0F0F0Fu;
    uint32_t wa[2][4], wc[2][4], wh[2][4], scw[2][4];
    float dd[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
      const uint32_t bk = sb + (g + 8 * r) * PITCH + skew;  // the block's first byte
#pragma unroll
      for (int hu = 0; hu < 4; hu++) {
        const int h = hu >> 1, u = hu & 1;
        wa[r][hu] = lds32s<ODD>(bk + 4 * (16 * h + 4 * u + t));
        wc[r][hu] = lds32s<ODD>(bk + 4 * (16 * h + 8 + 4 * u + t));
        wh[r][hu] = lds32s<ODD>(bk + 4 * (32 + 8 * h + 4 * u + t));
      }
#pragma unroll
      for (int i = 0; i < 4; i++) scw[r][i] = lds32s<ODD>(bk + 192 + 4 * i) ^ 0x80808080u;  // sc + 128, four per word
      dd[r] = f16_bits_to_f32((uint16_t)lds16u(bk + 208));
    }
    __syncwarp();  // the slot is free again
    slot_free();
    float dq[NG][4];
#pragma unroll
    for (int q = 0; q < NG; q++) dq[q][0] = dq[q][1] = dq[q][2] = dq[q][3] = 0.f;
    const __half2 off_c = __float2half2_rn(-1056.f), off_s = __float2half2_rn(-1152.f);
    const uint32_t bx = xb + g * TOK_PITCH + t * 8;
#pragma unroll
    for (int h = 0; h < 2; h++)
#pragma unroll
      for (int q = 0; q < 4; q++)
#pragma unroll
        for (int u = 0; u < 2; u++) {
          const int hu = 2 * h + u, m = (h * 4 + q) * 2 + u;  // MMA m = sub-block m = scale byte m
          uint32_t a[4];
#pragma unroll
          for (int r = 0; r < 2; r++) {
            const uint32_t lo4 = (q & 1) ? wc[r][hu] : wa[r][hu];
            const uint32_t nib = (q >> 1) ? (lo4 >> 4) : lo4;
            const uint32_t hi2 = q == 0 ? (wh[r][hu] << 4) : q == 1 ? (wh[r][hu] << 2) : q == 2 ? wh[r][hu] : (wh[r][hu] >> 2);
            const uint32_t v = and_or(nib, m0f, hi2 & 0x30303030u);
            // scale byte m of the row as the f16 pair (sc, sc): 1024 + (sc + 128) by PRMT, then -1152
            const uint32_t s16 = __byte_perm(scw[r][m >> 2], 0x64646464u, 0x4040 + 0x0101 * (m & 3));
            const __half2 sc = __hadd2(u2h(s16), off_s);
            a[r] = h2u(__hmul2(__hadd2(u2h(__byte_perm(v, 0x64646464u, 0x4240)), off_c), sc));
            a[2 + r] = h2u(__hmul2(__hadd2(u2h(__byte_perm(v, 0x64646464u, 0x4341)), off_c), sc));
          }
#pragma unroll
          for (int qg = 0; qg < NG; qg++) {
            const uint2 b = lds64(bx + qg * (8 * TOK_PITCH) + m * 32);
            mma16816(dq[qg], a[0], a[1], a[2], a[3], b.x, b.y);
          }
        }
#pragma unroll
    for (int qg = 0; qg < NG; qg++) {
      acc[qg][0] = fmaf(dd[0], dq[qg][0], acc[qg][0]), acc[qg][1] = fmaf(dd[0], dq[qg][1], acc[qg][1]);
      acc[qg][2] = fmaf(dd[1], dq[qg][2], acc[qg][2]), acc[qg][3] = fmaf(dd[1], dq[qg][3], acc[qg][3]);
    }
  }
  // only the low four bits of the block's byte offset from the matrix start matter (the matrix is 16-byte aligned)
  template <int NG, typename F>
  __device__ __forceinline__ void unit(uint32_t sb, uint32_t xb, float (&acc)[NG][4], const TileAt &at, uint32_t blk, int lane, F &&slot_free) const {
    const uint32_t skew = ((uint32_t)at.r0 * row_bytes + blk * 210u + (uint32_t)(lane >> 2) * row_bytes) & 15u;
    if (blk & 1)
      unit_p<NG, true>(sb, xb, acc, skew, lane, slot_free);
    else
      unit_p<NG, false>(sb, xb, acc, skew, lane, slot_free);
  }
};

// ------------------------------------------------------------------------------------ 4-bit, group 128
// Canonical layout (codes u32 (N, K/8), nibble j of word c = W[n, 8c + j]; scales, zeros f32 (N, K/128)).  A row's 256-k
// block is 128 bytes = 32 words; k step s uses words 2s and 2s + 1.  Lane (g, t) takes nibbles t and t + 4 of each (one
// shift by 4t, one LOP3 to f16 1024 + q), subtracts the group's zero point exactly (HADD2 with -(1024 + z)) and multiplies
// by the group's scale (HMUL2): w = f16((q - z) * s), one rounding.  The tile lies at a 144-byte pitch so that the eight
// rows of a load fall into distinct banks.
struct Int4Fmt {
  static constexpr int S = 3, PITCH = 144, TILE = ROWS * PITCH, BLOCK = 128, XS_CAP = 4;
  uint32_t row_bytes;
  __device__ __forceinline__ void setup(int, uint32_t row_bytes_) { row_bytes = row_bytes_; }
  __device__ __forceinline__ void issue(uint32_t dst, const uint8_t *tile0, uint32_t blk, int lane, const uint8_t *) const {
#pragma unroll
    for (int i = 0; i < 4; i++) {  // 128 chunks of 16 bytes: chunk c = lane + 32 i is piece c % 8 of row c / 8
      const uint32_t c = lane + 32 * i, r = c >> 3, piece = c & 7;
      cp_async16(dst + r * PITCH + piece * 16, tile0 + (size_t)r * row_bytes + blk * 128u + piece * 16u);
    }
  }
  template <int NG, typename F>
  __device__ __forceinline__ void unit(uint32_t sb, uint32_t xb, float (&acc)[NG][4], const TileAt &at, uint32_t blk, int lane, F &&slot_free) const {
    const int g = lane >> 2, t = lane & 3;
    __half2 sc[2][2], off[2][2];  // [row g | g + 8][group of this block]
    const int ng = (int)(row_bytes >> 6);  // groups per row: K / 128
#pragma unroll
    for (int r = 0; r < 2; r++)
#pragma unroll
      for (int gi = 0; gi < 2; gi++) {
        const size_t o = (size_t)(g + 8 * r) * ng + blk * 2 + gi;
        sc[r][gi] = __float2half2_rn(__ldg(at.sc + o));
        off[r][gi] = __float2half2_rn(-(1024.f + __ldg(at.zp + o)));
      }
    const uint32_t sh = 4u * t;
    const uint32_t bx = xb + g * TOK_PITCH + t * 8;
    auto cvt = [&](uint32_t w, __half2 o, __half2 s) { return h2u(__hmul2(__hadd2(u2h(and_or(w >> sh, 0x000F000Fu, 0x64006400u)), o), s)); };
#pragma unroll
    for (int i = 0; i < 8; i++) {  // two k steps per 16-byte load
      const int gi = i >> 2;
      const uint4 a = lds128(sb + g * PITCH + 16 * i), b = lds128(sb + (g + 8) * PITCH + 16 * i);
      const uint32_t e0 = cvt(a.x, off[0][gi], sc[0][gi]), e1 = cvt(b.x, off[1][gi], sc[1][gi]), e2 = cvt(a.y, off[0][gi], sc[0][gi]), e3 = cvt(b.y, off[1][gi], sc[1][gi]);
      const uint32_t f0 = cvt(a.z, off[0][gi], sc[0][gi]), f1 = cvt(b.z, off[1][gi], sc[1][gi]), f2 = cvt(a.w, off[0][gi], sc[0][gi]), f3 = cvt(b.w, off[1][gi], sc[1][gi]);
#pragma unroll
      for (int q = 0; q < NG; q++) {
        const uint2 be = lds64(bx + q * (8 * TOK_PITCH) + (2 * i) * 32), bo = lds64(bx + q * (8 * TOK_PITCH) + (2 * i + 1) * 32);
        mma16816(acc[q], e0, e1, e2, e3, be.x, be.y);
        mma16816(acc[q], f0, f1, f2, f3, bo.x, bo.y);
      }
    }
    __syncwarp();  // the slot is free again
    slot_free();
  }
};

// ------------------------------------------------------------------------------------ Q8_0
// Block (34 B): [f16 d | 32 int8].  A row's run of 256 k is eight blocks = 272 bytes = 17 granules (rows are whole
// granules when K % 256 == 0).  Lane (g, t) takes the word at 4t of each half block: XOR 0x80 makes the bytes unsigned,
// PRMT puts two of them into f16 1152 + q, HADD2 takes the 1152 off exactly and HMUL2 multiplies by the block's d (an
// f16 itself): one rounding per weight.  Words of even blocks lie 2 bytes off a word boundary and are funnel-shifted.
struct Q80Fmt {
  static constexpr int S = 2, PITCH = 272, TILE = ROWS * PITCH, BLOCK = 272, XS_CAP = 2;
  uint32_t row_bytes;
  __device__ __forceinline__ void setup(int, uint32_t row_bytes_) { row_bytes = row_bytes_; }
  __device__ __forceinline__ void issue(uint32_t dst, const uint8_t *tile0, uint32_t blk, int lane, const uint8_t *) const {
#pragma unroll
    for (int i = 0; i < 9; i++) {  // 272 chunks of 16 bytes: chunk c = lane + 32 i is piece c % 17 of row c / 17
      const uint32_t c = lane + 32 * i, r = (c * 241u) >> 12, piece = c - 17u * r;
      if (c < 272u) cp_async16(dst + r * PITCH + piece * 16, tile0 + (size_t)r * row_bytes + blk * 272u + piece * 16u);
    }
  }
  template <int NG, typename F>
  __device__ __forceinline__ void unit(uint32_t sb, uint32_t xb, float (&acc)[NG][4], const TileAt &, uint32_t, int lane, F &&slot_free) const {
    const int g = lane >> 2, t = lane & 3;
    const uint32_t bx = xb + g * TOK_PITCH + t * 8;
    const __half2 off = __float2half2_rn(-1152.f);
#pragma unroll
    for (int j = 0; j < 8; j++) {  // block j: k steps 2j and 2j + 1
      __half2 d2[2];
      uint32_t w[2][2];  // [row g | g + 8][half of the block]
#pragma unroll
      for (int r = 0; r < 2; r++) {
        const uint32_t bk = sb + (g + 8 * r) * PITCH + 34 * j;
        d2[r] = __half2half2(__ushort_as_half((unsigned short)lds16u(bk)));
#pragma unroll
        for (int hf = 0; hf < 2; hf++) {
          const uint32_t a = bk + 2 + 16 * hf + 4 * t;
          w[r][hf] = ((j & 1) ? lds32(a) : __funnelshift_r(lds32(a - 2), lds32(a + 2), 16)) ^ 0x80808080u;
        }
      }
#pragma unroll
      for (int hf = 0; hf < 2; hf++) {
        uint32_t a[4];
#pragma unroll
        for (int r = 0; r < 2; r++) {
          a[r] = h2u(__hmul2(__hadd2(u2h(__byte_perm(w[r][hf], 0x64646464u, 0x4240)), off), d2[r]));
          a[2 + r] = h2u(__hmul2(__hadd2(u2h(__byte_perm(w[r][hf], 0x64646464u, 0x4341)), off), d2[r]));
        }
#pragma unroll
        for (int q = 0; q < NG; q++) {
          const uint2 b = lds64(bx + q * (8 * TOK_PITCH) + (2 * j + hf) * 32);
          mma16816(acc[q], a[0], a[1], a[2], a[3], b.x, b.y);
        }
      }
    }
    __syncwarp();  // the slot is free again
    slot_free();
  }
};

// ------------------------------------------------------------------------------------ block-scaled FP8 (e4m3), 128 x 128 blocks
// A row's 256-k block is 256 bytes.  Lane (g, t) loads granule t of each 64-byte chunk (one 16-byte load per row and
// chunk); word j of it is the lane's four values of k step 4 c + j.  e4m3 -> f16 is exact (one cvt per pair), so the
// weights carry no rounding at all; the block scale (one per 128 k for the whole 16-row tile) multiplies the f32 partial
// sum of its eight k steps.
struct Fp8Fmt {
  static constexpr int S = 2, PITCH = 272, TILE = ROWS * PITCH, BLOCK = 256, XS_CAP = 2;
  uint32_t row_bytes;
  __device__ __forceinline__ void setup(int, uint32_t row_bytes_) { row_bytes = row_bytes_; }
  __device__ __forceinline__ void issue(uint32_t dst, const uint8_t *tile0, uint32_t blk, int lane, const uint8_t *) const {
#pragma unroll
    for (int i = 0; i < 8; i++) {  // 256 chunks of 16 bytes: chunk c = lane + 32 i is piece c % 16 of row c / 16
      const uint32_t c = lane + 32 * i, r = c >> 4, piece = c & 15;
      cp_async16(dst + r * PITCH + piece * 16, tile0 + (size_t)r * row_bytes + blk * 256u + piece * 16u);
    }
  }
  static __device__ __forceinline__ uint32_t cvt2(uint32_t two_codes) {
    const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)two_codes, __NV_E4M3);
    return (uint32_t)h.x | ((uint32_t)h.y << 16);
  }
  template <int NG, typename F>
  __device__ __forceinline__ void unit(uint32_t sb, uint32_t xb, float (&acc)[NG][4], const TileAt &at, uint32_t blk, int lane, F &&slot_free) const {
    const int g = lane >> 2, t = lane & 3;
    const uint32_t bx = xb + g * TOK_PITCH + t * 8;
    const float sc[2] = {__ldg(at.sc + blk * 2), __ldg(at.sc + blk * 2 + 1)};  // at.sc: the tile's row of block scales
#pragma unroll
    for (int half = 0; half < 2; half++) {  // 128 k under one scale
      float dq[NG][4];
#pragma unroll
      for (int q = 0; q < NG; q++) dq[q][0] = dq[q][1] = dq[q][2] = dq[q][3] = 0.f;
#pragma unroll
      for (int cc = 0; cc < 2; cc++) {
        const int c = 2 * half + cc;
        const uint4 a = lds128(sb + g * PITCH + 64 * c + 16 * t), b = lds128(sb + (g + 8) * PITCH + 64 * c + 16 * t);
        const uint32_t wa[4] = {a.x, a.y, a.z, a.w}, wb[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
          const uint32_t e0 = cvt2(wa[j] & 0xFFFFu), e1 = cvt2(wb[j] & 0xFFFFu), e2 = cvt2(wa[j] >> 16), e3 = cvt2(wb[j] >> 16);
#pragma unroll
          for (int q = 0; q < NG; q++) {
            const uint2 bb = lds64(bx + q * (8 * TOK_PITCH) + (4 * c + j) * 32);
            mma16816(dq[q], e0, e1, e2, e3, bb.x, bb.y);
          }
        }
      }
#pragma unroll
      for (int q = 0; q < NG; q++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[q][i] = fmaf(sc[half], dq[q][i], acc[q][i]);
    }
    __syncwarp();  // the slot is free again
    slot_free();
  }
};

template <typename Fmt, int NG>
constexpr int nt_smem() { return CW * Fmt::S * Fmt::TILE + XFeed<NG, Fmt::XS_CAP>::BYTES; }

template <typename Fmt, int NG>
__global__ void __launch_bounds__(THREADS, NG <= 4 ? 2 : 1) nt_kernel(const uint8_t *__restrict__ xs, float *__restrict__ parts,
                                                                    const __grid_constant__ NtArgs ma, int tiles, int M, int K, int run_len) {
  constexpr int S = Fmt::S;
  extern __shared__ __align__(128) unsigned char dyn[];  // [weight rings: 8 warps x S tiles][x ring][mbarriers][flag]
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int nb = K >> 8;
  const int groups = (tiles + CW - 1) / CW;
  const Run run{groups * nb, (int)gridDim.x, run_len, (int)blockIdx.x, nb};
  const int it0 = run.begin(run.c), it1 = run.begin(run.c + 1), n = it1 - it0;
  const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(dyn);
  const uint32_t ring = sbase + warp * (S * Fmt::TILE);
  XFeed<NG, Fmt::XS_CAP> xf;
  xf.init(sbase + CW * S * Fmt::TILE, dyn + CW * S * Fmt::TILE, xs, it0, n, nb);
  const uint32_t row_bytes = (uint32_t)nb * Fmt::BLOCK;
  Fmt fmt;
  fmt.setup(lane, row_bytes);

  using At = TileAt;
  auto at_group = [&](int grp) {
    At a;
    const int tile = grp * CW + warp;
    a.live = tile < tiles, a.wj = 0, a.r0 = 0;
    if (a.live) resolve(ma, tile, a.wj, a.r0);
    a.tile0 = ma.w[a.wj] + (size_t)a.r0 * row_bytes;
    a.w_end = ma.w[a.wj] + (size_t)ma.n[a.wj] * row_bytes;
    // 4-bit: one scale row per weight row; block-scaled FP8 (no zero points): one per 128 weight rows
    a.sc = ma.scales[a.wj] ? ma.scales[a.wj] + (size_t)(ma.zeros[a.wj] ? a.r0 : a.r0 >> 7) * (K >> 7) : nullptr;
    a.zp = ma.zeros[a.wj] ? ma.zeros[a.wj] + (size_t)a.r0 * (K >> 7) : nullptr;
    return a;
  };

  // ---- the weight ring runs ahead of the arithmetic, across group boundaries
  int i_k = 0, i_blk = it0 % nb, i_grp = it0 / nb, i_slot = 0;
  At i_at = at_group(i_grp);
  auto issue = [&]() {  // always closes a commit group, so that group counts stay uniform
    if (i_k < n) {
      if (i_at.live) {
        fmt.issue(ring + i_slot * Fmt::TILE, i_at.tile0, (uint32_t)i_blk, lane, i_at.w_end);
        i_slot = i_slot + 1 == S ? 0 : i_slot + 1;
      }
      i_k++;
      if (++i_blk == nb) {
        i_blk = 0, i_grp++;
        if (i_k < n) i_at = at_group(i_grp);
      }
    }
    cp_async_commit();
  };
#pragma unroll 1
  for (int p = 0; p < S; p++) issue();
  __syncthreads();  // the mbarriers are initialised
  pdl_wait();       // the staged activations are the pre-pass's output; the weights requested above are not
  const unsigned int epoch = *reinterpret_cast<volatile unsigned int *>(&g_nt_epoch);
  if (threadIdx.x == 0) xf.start();

  float acc[NG][4];
  int slot = 0, blk = it0 % nb, grp = it0 / nb, seg_b0 = blk;
  At at = at_group(grp);
  int fix_grp = -1;  // the group whose end this CTA holds after starting inside it
  At fix_at = at;
#pragma unroll
  for (int q = 0; q < NG; q++) acc[q][0] = acc[q][1] = acc[q][2] = acc[q][3] = 0.f;
  bool dead = false;
  for (int k = 0; k < n; k++) {
    if (threadIdx.x == 0) xf.pump(k);
    __syncwarp();
    if (!xf.wait_full(k)) { dead = true; break; }
    if (at.live) {
      cp_async_wait<S - 1>();
      __syncwarp();
      const uint32_t sb = ring + slot * Fmt::TILE;
      slot = slot + 1 == S ? 0 : slot + 1;
      fmt.template unit<NG>(sb, xf.buf(k), acc, at, (uint32_t)blk, lane, issue);
    } else {
      issue();  // keeps the commit-group count in step with the live warps' (and requests the next group's tiles)
    }
    xf.release(k, lane);
    if (blk == nb - 1 || k == n - 1) {  // the run leaves this group
      if (at.live) {
        if (seg_b0 == 0 && blk == nb - 1) {
          store_tile<NG>(acc, ma.out[at.wj], ma.out_bf16 != 0, ma.n[at.wj], at.r0, M, g, t);
        } else {
          const bool first = k - (blk - seg_b0) == 0;  // this CTA's first run (slot 0) or its last (slot 1)
          write_part<NG>(acc, parts, run.c, first ? 0 : 1, warp, lane, epoch);
          if (blk == nb - 1) fix_grp = grp, fix_at = at;
        }
      }
      if (k + 1 < n) {
        grp++, blk = 0, seg_b0 = 0;
        at = at_group(grp);
#pragma unroll
        for (int q = 0; q < NG; q++) acc[q][0] = acc[q][1] = acc[q][2] = acc[q][3] = 0.f;
      }
    } else {
      blk++;
    }
  }
  cp_async_wait<0>();
  if (!dead && fix_grp >= 0 && fix_at.live) {
    fix_up<NG>(run, fix_grp, parts, warp, lane, epoch, acc);
    store_tile<NG>(acc, ma.out[fix_at.wj], ma.out_bf16 != 0, ma.n[fix_at.wj], fix_at.r0, M, g, t);
  }
}

// ------------------------------------------------------------------------------------ launch
template <typename Fmt, int NG>
int launch_nt(const uint8_t *xs, float *parts, const NtArgs &ma, int tiles, int M, int K, int grid, int run_len, cudaStream_t st) {
  auto kern = nt_kernel<Fmt, NG>;
  const int smem = nt_smem<Fmt, NG>();
  static DeviceOnce attr_done;
  {
    cudaError_t e = attr_done.ensure([&] { return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); });
    if (e != cudaSuccess) return fail((int)e, "light_b200: matmul_q (decode, token tiles): %s", cudaGetErrorString(e));
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, xs, parts, ma, tiles, M, K, run_len);
  if (e != cudaSuccess) return fail((int)e, "light_b200: matmul_q (decode, token tiles): %s", cudaGetErrorString(e));
  return launched("matmul_q (decode, token tiles)");
}

template <typename Fmt>
int launch_by_ng(int ng, const uint8_t *xs, float *parts, const NtArgs &ma, int tiles, int M, int K, int grid, int run_len, cudaStream_t st) {
  switch (ng) {
    case 1: return launch_nt<Fmt, 1>(xs, parts, ma, tiles, M, K, grid, run_len, st);
    case 2: return launch_nt<Fmt, 2>(xs, parts, ma, tiles, M, K, grid, run_len, st);
    case 4: return launch_nt<Fmt, 4>(xs, parts, ma, tiles, M, K, grid, run_len, st);
    default: return launch_nt<Fmt, 8>(xs, parts, ma, tiles, M, K, grid, run_len, st);
  }
}

int g_nt_min_m = 9, g_nt_max_m = 64;  // LIGHT_B200_NT_MIN_M / _MAX_M (tuning knobs)

// the pre-pass: layout 0 (natural, Q6_K), 1 (sub-block pairs, Q4_K), 2 (4-bit code words) or 3 (FP8 granules); x f32 or bf16
int stage_x(int layout, const void *x, int x_dtype, void *ws, int M, int NT, int K, cudaStream_t st) {
  const int recs = (K >> 8) * NT;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((recs + CW - 1) / CW));
  cfg.blockDim = dim3(THREADS);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e;
  const float *xf = (const float *)x;
  const __nv_bfloat16 *xb = (const __nv_bfloat16 *)x;
  uint8_t *dst = (uint8_t *)ws;
  if (x_dtype == LB200_F32)
    e = layout == 0   ? cudaLaunchKernelEx(&cfg, x_stage_kernel<0, float>, xf, dst, M, NT, K)
        : layout == 1 ? cudaLaunchKernelEx(&cfg, x_stage_kernel<1, float>, xf, dst, M, NT, K)
        : layout == 2 ? cudaLaunchKernelEx(&cfg, x_stage_kernel<2, float>, xf, dst, M, NT, K)
                      : cudaLaunchKernelEx(&cfg, x_stage_kernel<3, float>, xf, dst, M, NT, K);
  else
    e = layout == 0   ? cudaLaunchKernelEx(&cfg, x_stage_kernel<0, __nv_bfloat16>, xb, dst, M, NT, K)
        : layout == 1 ? cudaLaunchKernelEx(&cfg, x_stage_kernel<1, __nv_bfloat16>, xb, dst, M, NT, K)
        : layout == 2 ? cudaLaunchKernelEx(&cfg, x_stage_kernel<2, __nv_bfloat16>, xb, dst, M, NT, K)
                      : cudaLaunchKernelEx(&cfg, x_stage_kernel<3, __nv_bfloat16>, xb, dst, M, NT, K);
  if (e != cudaSuccess) return fail((int)e, "light_b200: matmul (decode, staging): %s", cudaGetErrorString(e));
  return launched("matmul (decode, staging)");
}

// the persistent grid: every CTA slot of the GPU, but at least about four blocks per CTA unless SMs would idle; runs as
// even as possible, or, where one CTA per SM is all there is, of one fixed length that divides a row's blocks
void plan_grid(long long T, int nb, int ng, int env_grid, int &grid, int &run_len) {
  const int sms = sm_count(), slots = sms * (ng <= 4 ? 2 : 1);
  long long limit = T / 4 > sms ? T / 4 : (T < sms ? T : sms);
  if (limit > slots) limit = slots;
  if (env_grid > 0) limit = env_grid < T ? env_grid : T;
  if (limit > MAX_GRID) limit = MAX_GRID;
  run_len = 0;
  grid = (int)limit;
  const int q = (int)((T + limit - 1) / limit);
  if (limit <= sms && q <= nb && nb % q == 0) run_len = q, grid = (int)((T + q - 1) / q);
}

int ng_of(int M) { return M <= 8 ? 1 : M <= 16 ? 2 : M <= 32 ? 4 : 8; }
size_t stage_bytes(int M, int K) { return ((size_t)(K >> 8) * 8 * ng_of(M) * TOK_PITCH + 1023) & ~(size_t)1023; }
size_t parts_bytes(int M) { return (size_t)MAX_GRID * 2 * CW * ng_of(M) * 4 * 32 * sizeof(float); }

}  // namespace

int decode_nt_status() {
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_nt_status, sizeof(v));
  if (e != cudaSuccess) return fail((int)e, "light_b200: decode status: %s", cudaGetErrorString(e));
  return v;
}

// Workspace the path needs for M rows of K: the staged activations and the split-K partial sums.
size_t decode_nt_ws_bytes(int M, int K) { return stage_bytes(M, K) + parts_bytes(M); }

// `count` (1..4) matrices of one type (Q4_K or Q6_K) that share x (M rows, 9 .. 64 by default).  `ws` is memory of
// at least decode_nt_ws_bytes(M, K) bytes that stays untouched until the launches have run.
// Returns 1 if launched, 0 if the shape is not covered, else an error.
int gguf_decode_nt(int type, const float *x, const void *const *w, float *const *out, const int *n, int count, int M, int K, void *ws,
                   size_t ws_bytes, cudaStream_t st) {
  static bool knob = false;
  static int env_grid = 0;
  if (!knob) {
    if (const char *e = getenv("LIGHT_B200_NT_MIN_M")) g_nt_min_m = atoi(e);
    if (const char *e = getenv("LIGHT_B200_NT_MAX_M")) g_nt_max_m = atoi(e);
    if (const char *e = getenv("LIGHT_B200_NT_GRID")) env_grid = atoi(e);
    knob = true;
  }
  const bool q8 = type == LB200_Q8_0;
  if ((type != LB200_Q4_K && type != LB200_Q6_K && !q8) || M < (q8 && g_nt_min_m > 4 ? 4 : g_nt_min_m) || M > g_nt_max_m || M > 64 || M < 1 || K % 256 || count < 1 || count > 4 ||
      ((uintptr_t)x & 15) || !ws || ((uintptr_t)ws & 127) || ws_bytes < decode_nt_ws_bytes(M, K))
    return 0;
  const bool q6 = type == LB200_Q6_K;
  if (q6 && ((K >> 8) & 1)) return 0;
  NtArgs a = {};
  int tiles = 0;
  for (int i = 0; i < count; i++) {
    if (n[i] < ROWS) return 0;
    if ((uintptr_t)w[i] & 15) return 0;
    tiles += (n[i] + ROWS - 1) / ROWS;
    a.w[i] = (const uint8_t *)w[i], a.out[i] = out[i], a.n[i] = n[i], a.tend[i] = tiles;
  }
  a.count = count;
  const int ng = ng_of(M), NT = 8 * ng, nb = K >> 8;
  const long long T = (long long)((tiles + CW - 1) / CW) * nb;
  if (T >= (1ll << 30)) return 0;
  // a short list (a 4096 x 4096 matrix is 512 entries) leaves each CTA a few blocks and most of the time goes into
  // starting and the split-K fix-up: up to 32 rows the cluster kernel for Q4_K is quicker there
  if (!q6 && !q8 && M <= 32 && T < 4ll * sm_count() && !env_grid) return 0;
  int grid, run_len;
  plan_grid(T, nb, ng, env_grid, grid, run_len);
  if (int rc = stage_x(q6 || q8 ? 0 : 1, x, LB200_F32, ws, M, NT, K, st)) return rc;
  float *parts = reinterpret_cast<float *>((uint8_t *)ws + stage_bytes(M, K));
  const int rc = q6   ? launch_by_ng<Q6Fmt>(ng, (const uint8_t *)ws, parts, a, tiles, M, K, grid, run_len, st)
                 : q8 ? launch_by_ng<Q80Fmt>(ng, (const uint8_t *)ws, parts, a, tiles, M, K, grid, run_len, st)
                      : launch_by_ng<Q4Fmt>(ng, (const uint8_t *)ws, parts, a, tiles, M, K, grid, run_len, st);
  return rc ? rc : 1;
}

// Group-quantized 4-bit weights (canonical layout, group 128), x (M, K) and y (M, N) BF16, 4 .. 64 rows.  F32 activations
// stay on the kernels that keep x at f32 accuracy (the reference's bound for that type is 1e-4; f16 activations give 3e-4).
// Returns 1 if launched, 0 if the shape is not covered, else an error.
int int4_decode_nt(const void *x, const uint32_t *codes, const float *s, const float *z, void *y, int act_dtype, int M, int N, int K, int G,
                   void *ws, size_t ws_bytes, cudaStream_t st) {
  static int on = -1, min_m = 4;
  if (on < 0) {
    on = getenv("LIGHT_B200_NT_INT4") ? atoi(getenv("LIGHT_B200_NT_INT4")) : 1;
    if (const char *e = getenv("LIGHT_B200_NT_INT4_MIN_M")) min_m = atoi(e);
  }
  if (!on || act_dtype != LB200_BF16 || G != 128 || M < min_m || M > 64 || K % 256 || N < ROWS || ((uintptr_t)x & 15) || ((uintptr_t)codes & 15) || !ws || ((uintptr_t)ws & 127) ||
      ws_bytes < decode_nt_ws_bytes(M, K))
    return 0;
  NtArgs a = {};
  const int tiles = (N + ROWS - 1) / ROWS;
  a.w[0] = (const uint8_t *)codes, a.out[0] = (float *)y, a.n[0] = N, a.tend[0] = tiles, a.count = 1;
  a.out_bf16 = act_dtype == LB200_BF16, a.scales[0] = s, a.zeros[0] = z;
  const int ng = ng_of(M), NT = 8 * ng, nb = K >> 8;
  const long long T = (long long)((tiles + CW - 1) / CW) * nb;
  if (T >= (1ll << 30)) return 0;
  int grid, run_len;
  plan_grid(T, nb, ng, 0, grid, run_len);
  if (int rc = stage_x(2, x, act_dtype, ws, M, NT, K, st)) return rc;
  float *parts = reinterpret_cast<float *>((uint8_t *)ws + stage_bytes(M, K));
  const int rc = launch_by_ng<Int4Fmt>(ng, (const uint8_t *)ws, parts, a, tiles, M, K, grid, run_len, st);
  return rc ? rc : 1;
}

// Block-scaled FP8 (e4m3) weights (N, K) with f32 scales per 128 x 128 block, x and y BF16, 4 .. 64 rows.
// Returns 1 if launched, 0 if the shape is not covered, else an error.
int fp8_decode_nt(const void *x, const uint8_t *w, const float *scale, void *y, int act_dtype, int M, int N, int K, int bR, int bC, void *ws,
                  size_t ws_bytes, cudaStream_t st) {
  static int on = -1, min_m = 4;
  if (on < 0) {
    on = getenv("LIGHT_B200_NT_FP8") ? atoi(getenv("LIGHT_B200_NT_FP8")) : 1;
    if (const char *e = getenv("LIGHT_B200_NT_FP8_MIN_M")) min_m = atoi(e);
  }
  if (!on || act_dtype != LB200_BF16 || bR != 128 || bC != 128 || M < min_m || M > 64 || K % 256 || N % 128 || N < ROWS || ((uintptr_t)x & 15) ||
      ((uintptr_t)w & 15) || !ws || ((uintptr_t)ws & 127) || ws_bytes < decode_nt_ws_bytes(M, K))
    return 0;
  NtArgs a = {};
  const int tiles = N / ROWS;
  a.w[0] = w, a.out[0] = (float *)y, a.n[0] = N, a.tend[0] = tiles, a.count = 1;
  a.out_bf16 = 1, a.scales[0] = scale, a.zeros[0] = nullptr;
  const int ng = ng_of(M), NT = 8 * ng, nb = K >> 8;
  const long long T = (long long)((tiles + CW - 1) / CW) * nb;
  if (T >= (1ll << 30)) return 0;
  int grid, run_len;
  plan_grid(T, nb, ng, 0, grid, run_len);
  if (int rc = stage_x(3, x, act_dtype, ws, M, NT, K, st)) return rc;
  float *parts = reinterpret_cast<float *>((uint8_t *)ws + stage_bytes(M, K));
  const int rc = launch_by_ng<Fp8Fmt>(ng, (const uint8_t *)ws, parts, a, tiles, M, K, grid, run_len, st);
  return rc ? rc : 1;
}

}  // namespace lb
