// Batched decode, 2 .. 64 activation rows (tokens): fused dequant-matmul for Q4_K and Q6_K with the tokens as
// MMA columns and the activations staged ONCE per call.
//
//   pre-pass   x (M, K) f32 -> f16 in the order the B fragments are read, one 544-byte record per (K block,
//              token): 512 bytes of values and, for Q4_K, the eight sub-block sums as f16 hi | lo.  Tokens are
//              padded to a multiple of eight with zeros.  One warp per record.
//   main       a CTA of eight warps owns eight consecutive row tiles of 16 (one per warp, no sum across warps)
//              and walks a run of K blocks.  Per block ONE bulk copy (cp.async.bulk, completion on an mbarrier)
//              brings all tokens' records into a double buffer shared by the eight warps; the weights arrive
//              through a per-warp ring of 16-byte asynchronous copies and are expanded in registers straight
//              into A fragments (Q4_K: LOP3 to f16 (64 + q), one HFMA2 with the 6-bit scale; Q6_K: PRMT to f16
//              (1024 + code), offset and scale by HADD2 / HMUL2), so an expanded weight never touches shared
//              memory and serves NG groups of eight tokens.  Once per block and row, acc += d * D.  K is split
//              over a thread-block cluster of up to 8 CTAs whose partial sums meet in distributed shared memory.
//
// Every sum has a fixed order (k inside an MMA, blocks in a rotated but fixed sequence per CTA, cluster ranks
// ascending), so results are deterministic.  x is rounded to f16 once (2^-11 relative per element, about 2e-4
// relative L2 on the output).  Replaces, for 9 .. 64 rows, kernels that converted x inside every CTA.
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
  float *out[4];
  int n[4];
  int tend[4];
  int count;
};

__device__ int g_nt_status;  // non-zero: a bounded wait for a block of activations gave up (sticky)

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
template <bool PAIR>
__global__ void __launch_bounds__(THREADS) x_stage_kernel(const float *__restrict__ x, uint8_t *__restrict__ xs, int M, int NT, int K) {
  pdl_launch_dependents();
  const int rec = blockIdx.x * CW + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  const int nb = K >> 8;
  pdl_wait();  // x is the previous launch's output, and the launch before may still read the staging buffer
  if (rec >= nb * NT) return;
  const int b = rec / NT, tk = rec - b * NT;
  uint8_t *dst = xs + (size_t)rec * TOK_PITCH;
  float4 v[2];
  v[0] = v[1] = make_float4(0.f, 0.f, 0.f, 0.f);
  if (tk < M) {
    const float4 *xp = reinterpret_cast<const float4 *>(x + (size_t)tk * K + b * 256);
    v[0] = __ldg(xp + lane), v[1] = __ldg(xp + lane + 32);
  }
  float s[2];
#pragma unroll
  for (int j = 0; j < 2; j++) {
    const int F = lane + 32 * j;
    const __half2 lim = __float2half2_rn(65504.f);
    const __half2 h02 = __hmax2(__hmin2(__floats2half2_rn(v[j].x, v[j].z), lim), __hneg2(lim));
    const __half2 h13 = __hmax2(__hmin2(__floats2half2_rn(v[j].y, v[j].w), lim), __hneg2(lim));
    const int P = PAIR ? (((F >> 3) & 1) * 8 + (F & 7)) * 4 + (F >> 4) : F;
    *reinterpret_cast<uint2 *>(dst + P * 8) = make_uint2(h2u(h02), h2u(h13));
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

template <int NG>
struct XFeed {  // a ring of XS buffers of staged activations, one mbarrier each
  static constexpr int NT = 8 * NG, XBUF = NT * TOK_PITCH;
  static constexpr int XS = NG <= 2 ? 4 : NG == 4 ? 3 : 2;  // blocks of x in flight: the copy's latency spans several short blocks
  static constexpr int BYTES = XS * XBUF + 64;
  uint32_t buf0, bar0;
  const uint8_t *xs;
  volatile int *abort_flag;
  __device__ __forceinline__ void init(uint32_t base, unsigned char *gen, const uint8_t *xs_) {
    buf0 = base, bar0 = base + XS * XBUF, xs = xs_;
    abort_flag = reinterpret_cast<volatile int *>(gen + XS * XBUF + 8 * XS);
    if (threadIdx.x == 0) {
#pragma unroll
      for (int i = 0; i < XS; i++) umma::mbar_init(bar0 + 8 * i, 1);
      *abort_flag = 0;
      umma::fence_barrier_init();
    }
  }
  __device__ __forceinline__ uint32_t buf(int i) const { return buf0 + (uint32_t)(i % XS) * XBUF; }
  __device__ __forceinline__ void fetch(int i, int block) const {  // one thread
    const uint32_t h = (uint32_t)(i % XS);
    umma::mbar_arrive_expect_tx(bar0 + 8 * h, XBUF);
    bulk_g2s(buf0 + h * XBUF, xs + (size_t)block * XBUF, XBUF, bar0 + 8 * h);
  }
  __device__ __forceinline__ bool wait(int i) const {
    const bool ok = umma::mbar_wait(bar0 + 8 * (i % XS), (uint32_t)((i / XS) & 1), abort_flag, 200000000ull);
    if (!ok) g_nt_status = 1;
    return ok;
  }
};

// The CTA's partial sums partial[token][128 rows] (over its drained weight ring) -> out, summed over the cluster.
template <int NT>
__device__ __forceinline__ void reduce_out(const NtArgs &ma, uint32_t sbase, int KS, int rank, int tiles, int M) {
  if (KS > 1) umma::cluster_sync(); else __syncthreads();
  const int per = NT / KS;  // KS divides 8
  for (int idx = threadIdx.x; idx < per * 128; idx += THREADS) {
    const int tok = rank * per + (idx >> 7), rr = idx & 127, tile = blockIdx.x * CW + (rr >> 4);
    const uint32_t a = sbase + (uint32_t)(tok * 128 + rr) * 4u;
    float v = 0.f;
    if (KS > 1) {
      for (int p = 0; p < KS; p++) v += umma::ld_cluster_f32(umma::map_to_rank(a, (uint32_t)p));
    } else {
      asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(v) : "r"(a));
    }
    if (tok < M && tile < tiles) {
      int oj, orow;
      resolve(ma, tile, oj, orow);
      ma.out[oj][(size_t)tok * ma.n[oj] + orow + (rr & 15)] = v;
    }
  }
  if (KS > 1) umma::cluster_sync();  // nobody leaves while a peer still reads its partials
}

template <int NG>
__device__ __forceinline__ void park_acc(const float (&acc)[NG][4], uint32_t sbase, int warp, int g, int t) {
#pragma unroll
  for (int q = 0; q < NG; q++)
#pragma unroll
    for (int c = 0; c < 4; c++) {
      const int tok = q * 8 + 2 * t + (c & 1), row = warp * ROWS + g + 8 * (c >> 1);
      asm volatile("st.shared.f32 [%0], %1;\n" ::"r"(sbase + (uint32_t)(tok * 128 + row) * 4u), "f"(acc[q][c]));
    }
}

// ------------------------------------------------------------------------------------ Q4_K
// Lane (g, t) holds the 32 code bytes of sub-block pair t of rows g and g+8.  Code word i gives one MMA for
// sub-block 2t (low nibbles) and one for 2t+1 (high nibbles).  The minimum term -dmin * m_s * sum_{k in s} x_k
// is a second small contraction over the eight sub-blocks: A' = -dmin * m as f16 hi + lo, B' = the sub-block
// sums of x as f16 hi (both k halves), then A' = hi against the lo half of the sums.
constexpr int Q4_STAGES = 3, Q4_TILE = ROWS * 144, Q4_RING = CW * Q4_STAGES * Q4_TILE;

template <int NG>
constexpr int q4_smem() { return Q4_RING + XFeed<NG>::BYTES; }

template <int NG>
__global__ void __launch_bounds__(THREADS, NG <= 4 ? 2 : 1) q4k_nt_kernel(const uint8_t *__restrict__ xs, const __grid_constant__ NtArgs ma,
                                                                        int tiles, int M, int K) {
  constexpr int S = Q4_STAGES;
  static_assert(8 * NG * 128 * 4 <= Q4_RING, "the partial sums reuse the ring");
  extern __shared__ __align__(128) unsigned char dyn[];  // [ring: 8 warps x S tiles][x buffer 0][x buffer 1][2 mbarriers][flag]
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int nb = K >> 8;
  const int KS = gridDim.y, rank = blockIdx.y;
  const int b0 = nb * rank / KS, b1 = nb * (rank + 1) / KS, nloc = b1 - b0;
  // CTAs of one K run start at different blocks of it: otherwise all of them ask L2 for the same lines at once
  const int rot = (int)(blockIdx.x * 5u) % nloc;
  auto blk = [&](int i) { const int j = i + rot; return b0 + (j >= nloc ? j - nloc : j); };
  const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(dyn);
  XFeed<NG> xf;
  xf.init(sbase + Q4_RING, dyn + Q4_RING, xs);

  const int tile = blockIdx.x * CW + warp;
  const bool live = tile < tiles;
  int wj = 0, r0 = 0;
  if (live) resolve(ma, tile, wj, r0);
  const uint8_t *w = ma.w[wj];
  const uint32_t row_bytes = (uint32_t)nb * 144u;
  const uint32_t ring = sbase + warp * (S * Q4_TILE);
  const bool hdr_hi = t >= 2;
  const int hdr_sh = (t & 1) * 16;
  const uint32_t mask = 0x00F000F0u, magic = 0x54005400u;  // f16 (64 + nibble)
  uint32_t soff[5];
#pragma unroll
  for (int i = 0; i < 5; i++) {
    const uint32_t c = lane + 32 * i, row = c / 9u;
    soff[i] = row * row_bytes + (c - 9u * row) * 16u;
  }
  const uint32_t ld_off = g * 144u + 32u * t;
  int i_b = 0, i_slot = 0;
  auto issue = [&]() {  // always closes a commit group, so that group counts stay uniform
    if (live && i_b < nloc) {
      const uint8_t *base = w + ((size_t)r0 * row_bytes + (uint32_t)blk(i_b) * 144u);
      const uint32_t dst = ring + i_slot * Q4_TILE + lane * 16;
#pragma unroll
      for (int i = 0; i < 4; i++) cp_async16(dst + i * 512, base + soff[i]);
      if (lane < 16) cp_async16(dst + 2048, base + soff[4]);
      i_slot = i_slot + 1 == S ? 0 : i_slot + 1;
      i_b++;
    }
    cp_async_commit();
  };
#pragma unroll 1
  for (int p = 0; p < S; p++) issue();
  __syncthreads();  // the mbarriers are initialised
  pdl_wait();       // the staged activations are the pre-pass's output; the weights requested above are not
  if (threadIdx.x == 0)
    for (int i = 0; i < XFeed<NG>::XS && i < nloc; i++) xf.fetch(i, blk(i));

  float acc[NG][4];
#pragma unroll
  for (int q = 0; q < NG; q++) acc[q][0] = acc[q][1] = acc[q][2] = acc[q][3] = 0.f;
  int slot = 0;
  for (int bi = 0; bi < nloc; bi++) {
    const uint32_t xb = xf.buf(bi);
    if (!xf.wait(bi)) break;
    if (live) {
      cp_async_wait<S - 1>();
      __syncwarp();
      const uint32_t sb = ring + slot * Q4_TILE + ld_off;
      slot = slot + 1 == S ? 0 : slot + 1;
      const uint4 h0 = lds128(sb - 32u * t), h1 = lds128(sb - 32u * t + 8 * 144);
      const uint4 qa0 = lds128(sb + 16), qa1 = lds128(sb + 32);
      const uint4 qb0 = lds128(sb + 8 * 144 + 16), qb1 = lds128(sb + 8 * 144 + 32);
      __syncwarp();  // the slot is free again
      issue();
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
    __syncthreads();  // every warp is done with this block's half of the x buffer
    if (threadIdx.x == 0 && bi + XFeed<NG>::XS < nloc) xf.fetch(bi + XFeed<NG>::XS, blk(bi + XFeed<NG>::XS));
  }
  cp_async_wait<0>();
  __syncthreads();  // every warp is done with its ring slots
  if (live) park_acc<NG>(acc, sbase, warp, g, t);
  reduce_out<8 * NG>(ma, sbase, KS, rank, tiles, M);
}

// ------------------------------------------------------------------------------------ Q6_K
// Block (210 B): [ql[128] | qh[64] | int8 sc[16] | f16 d]; element e = 128h + 32q + l has its low nibble in
// ql[64h + 32(q&1) + l] (high nibble when q >= 2) and bits 2q..2q+1 of qh[32h + l]; its sub-block of 16 is
// 8h + 2q + l/16.  For each (h, u = l/16), lane (g, t) takes l = 16u + 4t .. +3 of rows g and g+8: one word of
// ql[64h + l], one of ql[64h + 32 + l], one of qh[32h + l].  Group q feeds ONE MMA whose 16 k slots are exactly
// sub-block m = 8h + 2q + u.  A row's block is copied as the 14 granules that cover it, to a 240-byte pitch; it
// begins `skew` = (its byte offset & 15) bytes into the row's slot: a multiple of 4 for even blocks and 2 mod 4
// for odd ones (rows hold an even number of blocks), where a word is two aligned words funnel-shifted.
constexpr int Q6_PITCH = 240, Q6_TILE = ROWS * Q6_PITCH, Q6_STAGES = 2, Q6_RING = CW * Q6_STAGES * Q6_TILE;

template <int NG>
constexpr int q6_smem() { return Q6_RING + XFeed<NG>::BYTES; }

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

template <int NG>
__global__ void __launch_bounds__(THREADS, NG <= 4 ? 2 : 1) q6k_nt_kernel(const uint8_t *__restrict__ xs, const __grid_constant__ NtArgs ma,
                                                                        int tiles, int M, int K) {
  constexpr int S = Q6_STAGES;
  static_assert(8 * NG * 128 * 4 <= Q6_RING, "the partial sums reuse the ring");
  extern __shared__ __align__(128) unsigned char dyn[];
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int nb = K >> 8;
  const int KS = gridDim.y, rank = blockIdx.y;
  const int b0 = nb * rank / KS, b1 = nb * (rank + 1) / KS, nloc = b1 - b0;
  const int rot = (int)(blockIdx.x * 5u) % nloc;
  auto blk = [&](int i) { const int j = i + rot; return b0 + (j >= nloc ? j - nloc : j); };
  const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(dyn);
  XFeed<NG> xf;
  xf.init(sbase + Q6_RING, dyn + Q6_RING, xs);

  const int tile = blockIdx.x * CW + warp;
  const bool live = tile < tiles;
  int wj = 0, r0 = 0;
  if (live) resolve(ma, tile, wj, r0);
  const uint8_t *w = ma.w[wj];
  const uint32_t row_bytes = (uint32_t)nb * 210u;  // a multiple of 4: nb is even (checked by the launcher)
  const uint8_t *w_end = w + (size_t)ma.n[wj] * row_bytes;
  const uint32_t ring = sbase + warp * (S * Q6_TILE);
  const uint32_t m0f = 0x0F0F0F0Fu;
  const uint32_t c_rsub = lane >> 4, c_piece = lane & 15;
  int i_b = 0, i_slot = 0;
  auto issue = [&]() {
    if (live && i_b < nloc) {
      uint32_t ro = (uint32_t)r0 * row_bytes + (uint32_t)blk(i_b) * 210u + c_rsub * row_bytes;
      uint32_t dst = ring + i_slot * Q6_TILE + c_rsub * Q6_PITCH + c_piece * 16;
      if (c_piece < 14) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const uint8_t *src = w + ((ro & ~15u) + c_piece * 16);
          const long long left = w_end - src;  // the last rows of the matrix: never read past its end
          if (left >= 16)
            cp_async16(dst, src);
          else if (left > 0)
            cp_async16_part(dst, src, (uint32_t)left);
          ro += 2 * row_bytes, dst += 2 * Q6_PITCH;
        }
      }
      i_slot = i_slot + 1 == S ? 0 : i_slot + 1;
      i_b++;
    }
    cp_async_commit();
  };
#pragma unroll 1
  for (int p = 0; p < S; p++) issue();
  __syncthreads();
  pdl_wait();
  if (threadIdx.x == 0)
    for (int i = 0; i < XFeed<NG>::XS && i < nloc; i++) xf.fetch(i, blk(i));

  float acc[NG][4];
#pragma unroll
  for (int q = 0; q < NG; q++) acc[q][0] = acc[q][1] = acc[q][2] = acc[q][3] = 0.f;

  // one unit: rows g, g+8 of this warp's tile x one K block out of ring slot `sb`, all token groups of buffer `xb`
  auto unit = [&](auto odd_tag, uint32_t sb, uint32_t skew, uint32_t xb) {
    constexpr bool ODD = decltype(odd_tag)::value;
    uint32_t wa[2][4], wc[2][4], wh[2][4], scw[2][4];
    float dd[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
      const uint32_t bk = sb + (g + 8 * r) * Q6_PITCH + skew;  // the block's first byte
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
    issue();
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
  };

  int slot = 0;
  for (int bi = 0; bi < nloc; bi++) {
    const uint32_t xb = xf.buf(bi);
    if (!xf.wait(bi)) break;
    if (live) {
      cp_async_wait<S - 1>();
      __syncwarp();
      const uint32_t sb = ring + slot * Q6_TILE;
      slot = slot + 1 == S ? 0 : slot + 1;
      const int b = blk(bi);
      const uint32_t skew = ((uint32_t)r0 * row_bytes + (uint32_t)b * 210u + (uint32_t)g * row_bytes) & 15u;
      if (b & 1)
        unit(std::true_type{}, sb, skew, xb);
      else
        unit(std::false_type{}, sb, skew, xb);
    }
    __syncthreads();
    if (threadIdx.x == 0 && bi + XFeed<NG>::XS < nloc) xf.fetch(bi + XFeed<NG>::XS, blk(bi + XFeed<NG>::XS));
  }
  cp_async_wait<0>();
  __syncthreads();
  if (live) park_acc<NG>(acc, sbase, warp, g, t);
  reduce_out<8 * NG>(ma, sbase, KS, rank, tiles, M);
}

// ------------------------------------------------------------------------------------ launch
template <int NG, bool Q6>
int launch_nt(const uint8_t *xs, const NtArgs &ma, int tiles, int M, int K, cudaStream_t st) {
  auto kern = Q6 ? q6k_nt_kernel<NG> : q4k_nt_kernel<NG>;
  const int smem = Q6 ? q6_smem<NG>() : q4_smem<NG>();
  static DeviceOnce attr_done;
  {
    cudaError_t e = attr_done.ensure([&] { return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); });
    if (e != cudaSuccess) return fail((int)e, "light_b200: matmul_q (decode, token tiles): %s", cudaGetErrorString(e));
  }
  const int nx = (tiles + CW - 1) / CW, nb = K >> 8, sms = sm_count();
  const int per_sm = NG <= 4 ? 2 : 1;
  // short K runs win (a CTA's start-up and its first block of x are not overlapped with anything) until the SMs'
  // CTA slots are taken and more CTAs wait behind them
  // first until every SM has a CTA, then, while a K run keeps at least four blocks, until the CTA slots are taken
  int ks = 1;
  while (ks < 8 && ks * 2 <= nb && (nx * ks * 2 <= sms || (nx * ks * 2 <= sms * per_sm && nb / (ks * 2) >= 4))) ks *= 2;
  static int env_ks = -1;
  if (env_ks < 0) env_ks = getenv("LIGHT_B200_NT_KS") ? atoi(getenv("LIGHT_B200_NT_KS")) : 0;
  if (env_ks >= 1 && env_ks <= 8 && (env_ks & (env_ks - 1)) == 0 && env_ks <= nb) ks = env_ks;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)nx, (unsigned)ks, 1);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = 1, attr[1].val.clusterDim.y = (unsigned)ks, attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, xs, ma, tiles, M, K);
  if (e != cudaSuccess) return fail((int)e, "light_b200: matmul_q (decode, token tiles): %s", cudaGetErrorString(e));
  return launched("matmul_q (decode, token tiles)");
}

template <bool Q6>
int launch_by_ng(int ng, const uint8_t *xs, const NtArgs &ma, int tiles, int M, int K, cudaStream_t st) {
  switch (ng) {
    case 1: return launch_nt<1, Q6>(xs, ma, tiles, M, K, st);
    case 2: return launch_nt<2, Q6>(xs, ma, tiles, M, K, st);
    case 4: return launch_nt<4, Q6>(xs, ma, tiles, M, K, st);
    default: return launch_nt<8, Q6>(xs, ma, tiles, M, K, st);
  }
}

int g_nt_min_m = 9, g_nt_max_m = 64;  // LIGHT_B200_NT_MIN_M / _MAX_M (tuning knobs)

}  // namespace

int decode_nt_status() {
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_nt_status, sizeof(v));
  if (e != cudaSuccess) return fail((int)e, "light_b200: decode status: %s", cudaGetErrorString(e));
  return v;
}

// `count` (1..4) matrices of one type (Q4_K or Q6_K) that share x (M rows, 9 .. 64 by default).  `ws` is staging
// memory of at least decode_nt_ws_bytes(M, K) bytes that stays untouched until the launches have run.
// Returns 1 if launched, 0 if the shape is not covered, else an error.
size_t decode_nt_ws_bytes(int M, int K) {
  const int ng = M <= 8 ? 1 : M <= 16 ? 2 : M <= 32 ? 4 : 8;
  return (size_t)(K >> 8) * 8 * ng * TOK_PITCH;
}

int gguf_decode_nt(int type, const float *x, const void *const *w, float *const *out, const int *n, int count, int M, int K, void *ws,
                   size_t ws_bytes, cudaStream_t st) {
  static bool knob = false;
  if (!knob) {
    if (const char *e = getenv("LIGHT_B200_NT_MIN_M")) g_nt_min_m = atoi(e);
    if (const char *e = getenv("LIGHT_B200_NT_MAX_M")) g_nt_max_m = atoi(e);
    knob = true;
  }
  if ((type != LB200_Q4_K && type != LB200_Q6_K) || M < g_nt_min_m || M > g_nt_max_m || M > 64 || M < 1 || K % 256 || count < 1 || count > 4 ||
      ((uintptr_t)x & 15) || !ws || ((uintptr_t)ws & 15) || ws_bytes < decode_nt_ws_bytes(M, K))
    return 0;
  const bool q6 = type == LB200_Q6_K;
  if (q6 && ((K >> 8) & 1)) return 0;
  NtArgs a = {};
  int tiles = 0;
  for (int i = 0; i < count; i++) {
    if (n[i] < ROWS) return 0;
    if (q6 ? (((uintptr_t)w[i] & 3) || (unsigned long long)n[i] * (K >> 8) * 210ull >= (1ull << 32)) : ((uintptr_t)w[i] & 15)) return 0;
    tiles += (n[i] + ROWS - 1) / ROWS;
    a.w[i] = (const uint8_t *)w[i], a.out[i] = out[i], a.n[i] = n[i], a.tend[i] = tiles;
  }
  a.count = count;
  const int ng = M <= 8 ? 1 : M <= 16 ? 2 : M <= 32 ? 4 : 8, NT = 8 * ng;
  {
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
    cudaError_t e = q6 ? cudaLaunchKernelEx(&cfg, x_stage_kernel<false>, x, (uint8_t *)ws, M, NT, K)
                       : cudaLaunchKernelEx(&cfg, x_stage_kernel<true>, x, (uint8_t *)ws, M, NT, K);
    if (e != cudaSuccess) return fail((int)e, "light_b200: matmul_q (decode, staging): %s", cudaGetErrorString(e));
    if (int rc = launched("matmul_q (decode, staging)")) return rc;
  }
  const int rc = q6 ? launch_by_ng<true>(ng, (const uint8_t *)ws, a, tiles, M, K, st) : launch_by_ng<false>(ng, (const uint8_t *)ws, a, tiles, M, K, st);
  return rc ? rc : 1;
}

}  // namespace lb
