// Decode (few activation rows) fused dequant-matmul for Q4_K and Q6_K: HBM-bound GEMV.
//
// The weights are read exactly once, with 16-byte (Q4_K) or 4-byte aligned (Q6_K, whose 210-byte
// blocks allow no more) coalesced loads, and never expanded to f32.  The arithmetic runs on the
// tensor cores although this is a matrix-vector product:
//
//   * a warp owns 16 weight rows (the M of mma.m16n8k16) and a contiguous range of K;
//   * the packed integer codes become exact f16 values with one LOP3 / PRMT per pair of weights
//     ((code bits) | magic exponent = offset + code), and form the A fragment directly in
//     registers -- there is no int -> float conversion, no per-weight scale multiply and no FMA
//     on the CUDA cores;
//   * the eight columns of the MMA are not eight tokens but EIGHT SUB-BLOCKS: the B fragment
//     holds the activations block-diagonally, B[k][c] = x[k] if element k lies in sub-block c,
//     else 0.  D[row][c] is then sum_{k in sub-block c} (offset + code) * x[k], the per-sub-block
//     integer dot product that a scale applies to -- accumulated over the whole 256-element
//     block by the tensor core, so the CUDA cores touch each (row, sub-block) once:
//         acc += (d*sc) * (D - offset * Sx) - (dmin*m) * Sx,     Sx = sum of x over the sub-block;
//   * lane (g, t) of the warp ends up holding exactly the D columns whose scales it decoded
//     (sub-blocks 2t and 2t+1 of rows g and g+8), so there is no cross-lane traffic until the
//     final reduction;
//   * activations stay f32-accurate: x is split as f16 hi + f16 lo (two MMAs into the same
//     accumulator) after an exact power-of-two prescale that keeps it inside f16 range.
//
// Per 256 weights of a row a lane issues ~2 instructions per weight-byte instead of ~8, which is
// what lets one SM keep up with its share of 6.5 TB/s.
#include "common.cuh"

namespace lb {

namespace {

constexpr int WARPS = 4;        // warps per CTA, splitting K
constexpr int ROWS = 16;        // weight rows per CTA (one m16 tile)
constexpr int ZERO_BYTES = 512; // zero page read by lanes whose B fragment is structurally zero

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}

// Shared memory layout, per activation row m (stride tok_stride bytes):
//   xh: K halves, hi part of the prescaled x, in natural element order except that inside each
//       group of four the order is (0, 2, 1, 3), so that one 8-byte load yields both B registers
//       of an MMA whose A fragment was cut from four consecutive code bytes;
//   xl: K halves, lo part, same order;
//   sx: K/SUB floats, sum of the prescaled x over each sub-block of SUB elements.
// Then ZERO_BYTES of zeros, then the cross-warp reduction buffer.
template <int SUB>
__host__ __device__ constexpr int tok_bytes(int K) {
  return 4 * K + 4 * (K / SUB);
}

// Each warp converts the K range it will consume: [e0, e1), multiples of 256.
// Returns the power of two by which the warp's partial sums must be multiplied back.
template <int SUB>
__device__ __forceinline__ float stage_x(const float *__restrict__ x, unsigned char *tok, int K, int e0, int e1,
                                         int lane) {
  float amax = 0.f;
  for (int e = e0 + lane * 4; e < e1; e += 128) {
    float4 v = __ldg(reinterpret_cast<const float4 *>(x + e));
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  // exact power-of-two prescale: only when |x| would leave f16 range
  int ex = ((__float_as_int(amax) >> 23) & 0xff) - 127;
  int sh = ex > 14 ? ex - 14 : 0;
  if (sh > 100) sh = 100;
  const float down = __int_as_float((127 - sh) << 23), up = __int_as_float((127 + sh) << 23);
  __half *xh = reinterpret_cast<__half *>(tok);
  __half *xl = xh + K;
  float *sx = reinterpret_cast<float *>(tok + 4 * K);
  constexpr int LANES_PER_SUB = SUB / 4;
  for (int e = e0 + lane * 4; e < e1; e += 128) {
    float4 v = __ldg(reinterpret_cast<const float4 *>(x + e));
    v.x *= down, v.y *= down, v.z *= down, v.w *= down;
    __half2 h02 = __floats2half2_rn(v.x, v.z), h13 = __floats2half2_rn(v.y, v.w);
    float2 f02 = __half22float2(h02), f13 = __half22float2(h13);
    __half2 l02 = __floats2half2_rn(v.x - f02.x, v.z - f02.y), l13 = __floats2half2_rn(v.y - f13.x, v.w - f13.y);
    uint2 hv, lv;
    hv.x = *reinterpret_cast<uint32_t *>(&h02), hv.y = *reinterpret_cast<uint32_t *>(&h13);
    lv.x = *reinterpret_cast<uint32_t *>(&l02), lv.y = *reinterpret_cast<uint32_t *>(&l13);
    *reinterpret_cast<uint2 *>(xh + e) = hv;
    *reinterpret_cast<uint2 *>(xl + e) = lv;
    float s = (v.x + v.y) + (v.z + v.w);
#pragma unroll
    for (int o = 1; o < LANES_PER_SUB; o <<= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((lane & (LANES_PER_SUB - 1)) == 0) sx[e / SUB] = s;
  }
  return up;
}

// ------------------------------------------------------------------------------------ Q4_K
//
// Block (144 B): [f16 d | f16 dmin | scales[12] | qs[128]]; byte qs[32p + l] holds element
// 64p + l (low nibble, sub-block 2p) and 64p + 32 + l (high nibble, sub-block 2p+1).
// Lane (g, t) loads the 32 qs bytes of pair p = t of rows g and g+8 (two 16-byte loads each)
// and the 16-byte header of both rows.  Code word i (bytes 4i..4i+3) feeds two MMAs:
//   even sub-block 2t: a0 = codes(b0.lo, b2.lo)  a2 = codes(b1.lo, b3.lo)   (k slots 2t,2t+1 | 2t+8,2t+9)
//   odd  sub-block 2t+1: the same with the high nibbles.
// All four come out as f16 (64 + code): (word >> {-4,0,4,8}) & 0x00F000F0 | 0x54005400.
// The B lane (col c, tid) is non-zero only when c == 2*tid (even MMA) or c == 2*tid+1 (odd MMA).

struct Q4KBlk {
  uint4 hdr[2];   // rows g, g+8
  uint4 q[2][2];  // [row][half of the 32 bytes]
};

__device__ __forceinline__ Q4KBlk q4k_load(const uint4 *rg, const uint4 *rg8, int b, int t) {
  Q4KBlk k;
  const uint4 *pg = rg + b * 9, *pg8 = rg8 + b * 9;
  k.hdr[0] = __ldg(pg);
  k.hdr[1] = __ldg(pg8);
  k.q[0][0] = __ldg(pg + 1 + 2 * t);
  k.q[0][1] = __ldg(pg + 2 + 2 * t);
  k.q[1][0] = __ldg(pg8 + 1 + 2 * t);
  k.q[1][1] = __ldg(pg8 + 2 + 2 * t);
  return k;
}

// (d*sc, dmin*m) of sub-blocks 2t and 2t+1 from one header.
__device__ __forceinline__ void q4k_scales(const uint4 &h, int t, float (&dsc)[2], float (&dmn)[2]) {
  const float d = f16_bits_to_f32((uint16_t)(h.x & 0xffffu)), dmin = f16_bits_to_f32((uint16_t)(h.x >> 16));
  // packed 6-bit fields as one byte each: sub-blocks 0..3 and 4..7
  const uint32_t sc_lo = h.y & 0x3F3F3F3Fu, mn_lo = h.z & 0x3F3F3F3Fu;
  const uint32_t sc_hi = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);
  const uint32_t mn_hi = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
  const uint32_t scw = t < 2 ? sc_lo : sc_hi, mnw = t < 2 ? mn_lo : mn_hi;
  const int sh = (t & 1) * 16;
  dsc[0] = d * (float)((scw >> sh) & 0xFFu);
  dsc[1] = d * (float)((scw >> (sh + 8)) & 0xFFu);
  dmn[0] = dmin * (float)((mnw >> sh) & 0xFFu);
  dmn[1] = dmin * (float)((mnw >> (sh + 8)) & 0xFFu);
}

template <int MT, bool LO>
__global__ void __launch_bounds__(WARPS * 32) q4k_gemv_mma_kernel(const float *__restrict__ x,
                                                                  const uint8_t *__restrict__ w,
                                                                  float *__restrict__ out, int M, int N, int K) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int nb = K >> 8;
  const int b0 = warp * nb / WARPS, b1 = (warp + 1) * nb / WARPS;
  const int tokb = tok_bytes<32>(K);
  unsigned char *zero = smem + MT * tokb;
  float *red = reinterpret_cast<float *>(zero + ZERO_BYTES);

  for (int i = threadIdx.x; i < ZERO_BYTES / 4; i += WARPS * 32) reinterpret_cast<uint32_t *>(zero)[i] = 0u;
  float up[MT];
#pragma unroll
  for (int m = 0; m < MT; m++)
    up[m] = m < M ? stage_x<32>(x + (size_t)m * K, smem + m * tokb, K, b0 * 256, b1 * 256, lane) : 0.f;
  __syncthreads();  // zero page; each warp reads back only what it staged itself

  const int n0 = blockIdx.x * ROWS;
  const int rg = min(n0 + g, N - 1), rg8 = min(n0 + g + 8, N - 1);
  const size_t row_u4 = (size_t)nb * 9;
  const uint4 *wg = reinterpret_cast<const uint4 *>(w) + (size_t)rg * row_u4;
  const uint4 *wg8 = reinterpret_cast<const uint4 *>(w) + (size_t)rg8 * row_u4;

  const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(smem), szero = (uint32_t)__cvta_generic_to_shared(zero);
  // B addresses: even MMA live iff g == 2t, odd MMA live iff g == 2t+1; sub-block index == g.
  const bool live_e = g == 2 * t, live_o = g == 2 * t + 1;
  uint32_t pe = live_e ? sbase + b0 * 512 + g * 64 : szero;
  uint32_t po = live_o ? sbase + b0 * 512 + g * 64 : szero;
  const uint32_t adv_e = live_e ? 512u : 0u, adv_o = live_o ? 512u : 0u;
  const uint32_t lo_e = live_e ? (uint32_t)(2 * K) : 0u, lo_o = live_o ? (uint32_t)(2 * K) : 0u;
  const uint32_t tok_e = live_e ? (uint32_t)tokb : 0u, tok_o = live_o ? (uint32_t)tokb : 0u;

  float acc[MT][2];
#pragma unroll
  for (int m = 0; m < MT; m++) acc[m][0] = acc[m][1] = 0.f;

  constexpr uint32_t MASK = 0x00F000F0u, MAGIC = 0x54005400u;  // f16 (64 + nibble)
  if (b0 < b1) {
    Q4KBlk cur = q4k_load(wg, wg8, b0, t);
    for (int b = b0; b < b1; b++) {
      Q4KBlk nxt;
      if (b + 1 < b1) nxt = q4k_load(wg, wg8, b + 1, t);
      float dsc[2][2], dmn[2][2];
      q4k_scales(cur.hdr[0], t, dsc[0], dmn[0]);
      q4k_scales(cur.hdr[1], t, dsc[1], dmn[1]);
      float d[MT][4];
#pragma unroll
      for (int m = 0; m < MT; m++) d[m][0] = d[m][1] = d[m][2] = d[m][3] = 0.f;
      const uint32_t qg[8] = {cur.q[0][0].x, cur.q[0][0].y, cur.q[0][0].z, cur.q[0][0].w,
                              cur.q[0][1].x, cur.q[0][1].y, cur.q[0][1].z, cur.q[0][1].w};
      const uint32_t qh[8] = {cur.q[1][0].x, cur.q[1][0].y, cur.q[1][0].z, cur.q[1][0].w,
                              cur.q[1][1].x, cur.q[1][1].y, cur.q[1][1].z, cur.q[1][1].w};
#pragma unroll
      for (int i = 0; i < 8; i++) {
        const uint32_t vg = qg[i], vh = qh[i];
        const uint32_t e0 = ((vg << 4) & MASK) | MAGIC, e1 = ((vh << 4) & MASK) | MAGIC;
        const uint32_t e2 = ((vg >> 4) & MASK) | MAGIC, e3 = ((vh >> 4) & MASK) | MAGIC;
        const uint32_t o0 = (vg & MASK) | MAGIC, o1 = (vh & MASK) | MAGIC;
        const uint32_t o2 = ((vg >> 8) & MASK) | MAGIC, o3 = ((vh >> 8) & MASK) | MAGIC;
#pragma unroll
        for (int m = 0; m < MT; m++) {
          uint2 be = lds64(pe + m * tok_e + i * 8);
          mma16816(d[m], e0, e1, e2, e3, be.x, be.y);
          uint2 bo = lds64(po + m * tok_o + i * 8);
          mma16816(d[m], o0, o1, o2, o3, bo.x, bo.y);
          if (LO) {
            uint2 bel = lds64(pe + m * tok_e + lo_e + i * 8);
            mma16816(d[m], e0, e1, e2, e3, bel.x, bel.y);
            uint2 bol = lds64(po + m * tok_o + lo_o + i * 8);
            mma16816(d[m], o0, o1, o2, o3, bol.x, bol.y);
          }
        }
      }
      // lane (g, t): d[.][0], d[.][1] = row g, sub-blocks 2t, 2t+1;  d[.][2], d[.][3] = row g+8.
#pragma unroll
      for (int m = 0; m < MT; m++) {
        const float2 sx = *reinterpret_cast<const float2 *>(smem + m * tokb + 4 * K + (b * 8 + 2 * t) * 4);
#pragma unroll
        for (int r = 0; r < 2; r++) {
          float v = dsc[r][0] * d[m][2 * r] - (64.f * dsc[r][0] + dmn[r][0]) * sx.x;
          v += dsc[r][1] * d[m][2 * r + 1] - (64.f * dsc[r][1] + dmn[r][1]) * sx.y;
          acc[m][r] += v;
        }
      }
      pe += adv_e;
      po += adv_o;
      cur = nxt;
    }
  }
  // sum the four t-lanes of each row, undo the prescale, then the warps of the CTA
#pragma unroll
  for (int m = 0; m < MT; m++)
#pragma unroll
    for (int r = 0; r < 2; r++) {
      float v = acc[m][r];
      v += __shfl_xor_sync(0xffffffffu, v, 1);
      v += __shfl_xor_sync(0xffffffffu, v, 2);
      if (t == 0) red[(warp * MT + m) * ROWS + g + 8 * r] = v * up[m];
    }
  __syncthreads();
  for (int i = threadIdx.x; i < MT * ROWS; i += WARPS * 32) {
    const int m = i / ROWS, r = i % ROWS;
    if (m < M && n0 + r < N) {
      float v = 0.f;
#pragma unroll
      for (int wq = 0; wq < WARPS; wq++) v += red[(wq * MT + m) * ROWS + r];
      out[(size_t)m * N + n0 + r] = v;
    }
  }
}

// ------------------------------------------------------------------------------------ Q6_K
//
// Block (210 B): [ql[128] | qh[64] | int8 sc[16] | f16 d]; element e = 128h + 32q + l
// (half h, group q, l < 32) has low nibble in ql[64h + 32(q&1) + l] (high nibble when q >= 2) and
// bits 2q..2q+1 of qh[32h + l]; its sub-block of 16 is s = e / 16 = 8h + 2q + l/16.
// Lane (g, t) takes group q = t of rows g and g+8.  For each (h, u = l/16) it needs the 16 ql
// bytes at 64h + 32(t&1) + 16u and the 16 qh bytes at 128 + 32h + 16u.  Blocks are only 2-byte
// aligned, so each run is fetched as five aligned 32-bit words and funnel-shifted by 0 or 16.
// Code word i (l = 16u + 4i .. +3) becomes four 6-bit bytes, then two f16x2 (1024 + code)
// with PRMT, and feeds ONE MMA (all 16 k slots of it belong to sub-block 8h + 2t + u):
//   column = sub-block mod 8 = 2t + u -> B lane (col c, tid) live iff c == 2*tid + u, as for Q4_K.
// One accumulator fragment per half h.

__device__ __forceinline__ void ld_run16(const uint8_t *p, uint32_t (&v)[4]) {
  const uint32_t sh = ((uint32_t)(uintptr_t)p & 2u) * 8u;  // 0 or 16
  const uint32_t *a = reinterpret_cast<const uint32_t *>((uintptr_t)p & ~(uintptr_t)3);
  uint32_t r[5];
#pragma unroll
  for (int i = 0; i < 5; i++) r[i] = __ldg(a + i);
#pragma unroll
  for (int i = 0; i < 4; i++) v[i] = __funnelshift_r(r[i], r[i + 1], sh);
}

template <int MT, bool LO>
__global__ void __launch_bounds__(WARPS * 32) q6k_gemv_mma_kernel(const float *__restrict__ x,
                                                                  const uint8_t *__restrict__ w,
                                                                  float *__restrict__ out, int M, int N, int K) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int nb = K >> 8;
  const int b0 = warp * nb / WARPS, b1 = (warp + 1) * nb / WARPS;
  const int tokb = tok_bytes<16>(K);
  unsigned char *zero = smem + MT * tokb;
  float *red = reinterpret_cast<float *>(zero + ZERO_BYTES);

  for (int i = threadIdx.x; i < ZERO_BYTES / 4; i += WARPS * 32) reinterpret_cast<uint32_t *>(zero)[i] = 0u;
  float up[MT];
#pragma unroll
  for (int m = 0; m < MT; m++)
    up[m] = m < M ? stage_x<16>(x + (size_t)m * K, smem + m * tokb, K, b0 * 256, b1 * 256, lane) : 0.f;
  __syncthreads();

  const int n0 = blockIdx.x * ROWS;
  const size_t row_bytes = (size_t)nb * 210;
  const uint8_t *wr[2] = {w + (size_t)min(n0 + g, N - 1) * row_bytes, w + (size_t)min(n0 + g + 8, N - 1) * row_bytes};

  const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(smem), szero = (uint32_t)__cvta_generic_to_shared(zero);
  const bool live0 = g == 2 * t, live1 = g == 2 * t + 1;  // u = 0 / u = 1 MMAs
  uint32_t p0 = live0 ? sbase + b0 * 512 + g * 32 : szero;
  uint32_t p1 = live1 ? sbase + b0 * 512 + g * 32 : szero;
  const uint32_t adv0 = live0 ? 512u : 0u, adv1 = live1 ? 512u : 0u;
  const uint32_t lo0 = live0 ? (uint32_t)(2 * K) : 0u, lo1 = live1 ? (uint32_t)(2 * K) : 0u;
  const uint32_t tok0 = live0 ? (uint32_t)tokb : 0u, tok1 = live1 ? (uint32_t)tokb : 0u;
  const uint32_t half0 = live0 ? 256u : 0u, half1 = live1 ? 256u : 0u;  // +128 elements for h = 1

  const int sA = (t >> 1) * 4, sH = 2 * t;
  float acc[MT][2];
#pragma unroll
  for (int m = 0; m < MT; m++) acc[m][0] = acc[m][1] = 0.f;

  for (int b = b0; b < b1; b++) {
    // scales of sub-blocks 8h + 2t + u and the block scale d, for both rows
    float ds[2][2][2];  // [row][h][u]
#pragma unroll
    for (int r = 0; r < 2; r++) {
      const uint8_t *blk = wr[r] + (size_t)b * 210;
      const uint16_t s0 = __ldg(reinterpret_cast<const uint16_t *>(blk + 192 + 2 * t));
      const uint16_t s1 = __ldg(reinterpret_cast<const uint16_t *>(blk + 200 + 2 * t));
      const float d = f16_bits_to_f32(__ldg(reinterpret_cast<const uint16_t *>(blk + 208)));
      ds[r][0][0] = d * (float)(int8_t)(s0 & 0xff);
      ds[r][0][1] = d * (float)(int8_t)(s0 >> 8);
      ds[r][1][0] = d * (float)(int8_t)(s1 & 0xff);
      ds[r][1][1] = d * (float)(int8_t)(s1 >> 8);
    }
#pragma unroll
    for (int h = 0; h < 2; h++) {
      float d[MT][4];
#pragma unroll
      for (int m = 0; m < MT; m++) d[m][0] = d[m][1] = d[m][2] = d[m][3] = 0.f;
#pragma unroll
      for (int u = 0; u < 2; u++) {
        uint32_t ql[2][4], qh[2][4];
#pragma unroll
        for (int r = 0; r < 2; r++) {
          const uint8_t *blk = wr[r] + (size_t)b * 210;
          ld_run16(blk + 64 * h + 32 * (t & 1) + 16 * u, ql[r]);
          ld_run16(blk + 128 + 32 * h + 16 * u, qh[r]);
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
          uint32_t a[4];
#pragma unroll
          for (int r = 0; r < 2; r++) {
            const uint32_t v = ((ql[r][i] >> sA) & 0x0F0F0F0Fu) | (((qh[r][i] >> sH) << 4) & 0x30303030u);
            a[r] = __byte_perm(v, 0x64646464u, 0x4240);      // (1024 + b0, 1024 + b2)
            a[2 + r] = __byte_perm(v, 0x64646464u, 0x4341);  // (1024 + b1, 1024 + b3)
          }
          const uint32_t pu = u ? p1 : p0, toku = u ? tok1 : tok0, lou = u ? lo1 : lo0, hu = u ? half1 : half0;
#pragma unroll
          for (int m = 0; m < MT; m++) {
            uint2 bb = lds64(pu + m * toku + h * hu + i * 8);
            mma16816(d[m], a[0], a[1], a[2], a[3], bb.x, bb.y);
            if (LO) {
              uint2 bl = lds64(pu + m * toku + lou + h * hu + i * 8);
              mma16816(d[m], a[0], a[1], a[2], a[3], bl.x, bl.y);
            }
          }
        }
      }
      // lane (g, t): d[.][0], d[.][1] = row g, sub-blocks 8h+2t, 8h+2t+1;  d[.][2], d[.][3] = row g+8
#pragma unroll
      for (int m = 0; m < MT; m++) {
        const float2 sx = *reinterpret_cast<const float2 *>(smem + m * tokb + 4 * K + (b * 16 + 8 * h + 2 * t) * 4);
#pragma unroll
        for (int r = 0; r < 2; r++)
          acc[m][r] += ds[r][h][0] * (d[m][2 * r] - 1056.f * sx.x) + ds[r][h][1] * (d[m][2 * r + 1] - 1056.f * sx.y);
      }
    }
    p0 += adv0;
    p1 += adv1;
  }
#pragma unroll
  for (int m = 0; m < MT; m++)
#pragma unroll
    for (int r = 0; r < 2; r++) {
      float v = acc[m][r];
      v += __shfl_xor_sync(0xffffffffu, v, 1);
      v += __shfl_xor_sync(0xffffffffu, v, 2);
      if (t == 0) red[(warp * MT + m) * ROWS + g + 8 * r] = v * up[m];
    }
  __syncthreads();
  for (int i = threadIdx.x; i < MT * ROWS; i += WARPS * 32) {
    const int m = i / ROWS, r = i % ROWS;
    if (m < M && n0 + r < N) {
      float v = 0.f;
#pragma unroll
      for (int wq = 0; wq < WARPS; wq++) v += red[(wq * MT + m) * ROWS + r];
      out[(size_t)m * N + n0 + r] = v;
    }
  }
}

constexpr int MAX_SMEM = 200 * 1024;

template <int SUB>
size_t smem_bytes(int MT, int K) {
  return (size_t)MT * tok_bytes<SUB>(K) + ZERO_BYTES + (size_t)WARPS * MT * ROWS * 4;
}

template <typename Kern>
int set_smem(Kern k) {
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, MAX_SMEM);
  return e == cudaSuccess ? 0 : fail((int)e, "light_b200: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
}

}  // namespace

int gguf_gemv_fast_init(int) {
  int rc = 0;
  if ((rc = set_smem(q4k_gemv_mma_kernel<1, true>))) return rc;
  if ((rc = set_smem(q4k_gemv_mma_kernel<2, true>))) return rc;
  if ((rc = set_smem(q4k_gemv_mma_kernel<4, true>))) return rc;
  if ((rc = set_smem(q6k_gemv_mma_kernel<1, true>))) return rc;
  if ((rc = set_smem(q6k_gemv_mma_kernel<2, true>))) return rc;
  if ((rc = set_smem(q6k_gemv_mma_kernel<4, true>))) return rc;
  return 0;
}

int gguf_gemv_fast(int type, const float *x, const void *w, float *out, int M, int N, int K, cudaStream_t st) {
  if (M < 1 || M > 4 || K % 256) return 0;
  const int MT = M == 1 ? 1 : M == 2 ? 2 : 4;
  const unsigned grid = (unsigned)((N + ROWS - 1) / ROWS);
  if (type == LB200_Q4_K) {
    if ((uintptr_t)w & 15) return 0;
    size_t sm = smem_bytes<32>(MT, K);
    if (sm > (size_t)MAX_SMEM) return 0;
    const uint8_t *wb = (const uint8_t *)w;
    if (MT == 1) q4k_gemv_mma_kernel<1, true><<<grid, WARPS * 32, sm, st>>>(x, wb, out, M, N, K);
    else if (MT == 2) q4k_gemv_mma_kernel<2, true><<<grid, WARPS * 32, sm, st>>>(x, wb, out, M, N, K);
    else q4k_gemv_mma_kernel<4, true><<<grid, WARPS * 32, sm, st>>>(x, wb, out, M, N, K);
    int rc = launched("matmul_q (Q4_K decode)");
    return rc ? rc : 1;
  }
  if (type == LB200_Q6_K) {
    // rows must start 4-byte aligned for the aligned-word loads: (K/256)*210 % 4 == 0
    if (((uintptr_t)w & 3) || ((size_t)(K >> 8) * 210) % 4) return 0;
    size_t sm = smem_bytes<16>(MT, K);
    if (sm > (size_t)MAX_SMEM) return 0;
    const uint8_t *wb = (const uint8_t *)w;
    if (MT == 1) q6k_gemv_mma_kernel<1, true><<<grid, WARPS * 32, sm, st>>>(x, wb, out, M, N, K);
    else if (MT == 2) q6k_gemv_mma_kernel<2, true><<<grid, WARPS * 32, sm, st>>>(x, wb, out, M, N, K);
    else q6k_gemv_mma_kernel<4, true><<<grid, WARPS * 32, sm, st>>>(x, wb, out, M, N, K);
    int rc = launched("matmul_q (Q6_K decode)");
    return rc ? rc : 1;
  }
  return 0;
}

}  // namespace lb
