// Decode (few activation rows) fused dequant-matmul for Q4_K and Q6_K: HBM-bound GEMV.
//
// The weights are read exactly once, coalesced, and never expanded to f32.  The arithmetic runs
// on the tensor cores although this is a matrix-vector product:
//
//   * a warp owns one 256-element K block and walks down RT tiles of 16 weight rows (the M of
//     mma.m16n8k16), so the activations of its block are converted once and reused;
//   * the packed integer codes become exact f16 values with one LOP3 / PRMT per pair of weights
//     ((code bits) | magic exponent = offset + code) and form the A fragment directly in
//     registers -- no int -> float conversion, no per-weight scale multiply, no CUDA-core FMA;
//   * the eight columns of the MMA are not eight tokens but EIGHT SUB-BLOCKS: the B fragment
//     holds the activations block-diagonally, B[k][c] = x[k] if element k lies in sub-block c,
//     else 0.  D[row][c] is then sum_{k in sub-block c} (offset + code) * x[k], the per-sub-block
//     integer dot product that a scale applies to, accumulated over the whole 256-element block
//     by the tensor core.  The CUDA cores touch each (row, sub-block) once:
//         acc += (d*sc) * (D - offset * Sx) - (dmin*m) * Sx,     Sx = sum of x over the sub-block;
//   * lane (g, t) of the warp ends up holding exactly the D columns whose scales it decoded
//     (sub-blocks 2t and 2t+1 of rows g and g+8), so there is no cross-lane traffic until the
//     final reduction;
//   * activations stay f32-accurate: x is split as f16 hi + f16 lo (two MMAs into the same
//     accumulator) after an exact power-of-two prescale that keeps it inside f16 range.
//
// A CTA covers 16*RT rows and all of K (its warps take K blocks round-robin and reduce through
// shared memory), so every output element is written once, deterministically, without atomics.
// The kernels are launched with programmatic dependent launch: the first weight tile is
// requested before griddepcontrol.wait, so the head of each launch overlaps the tail of the one
// before it in the stream -- a decode step is a chain of a few hundred such launches.
#include <cstdlib>
#include <type_traits>

#include "common.cuh"
#include "mma_sync.cuh"
#include "decode_units.cuh"
#include "umma.cuh"

namespace lb {

namespace {

constexpr int WARPS = 8;  // warps per CTA, taking K blocks round-robin
constexpr int ROWS = 16;  // weight rows per tile (one m16 MMA tile)

// Per-warp activation slab for one 256-element K block, SUB elements per sub-block:
//   hi[256/SUB sub-blocks][SUB halves + pad]  lo[...same...]  sx[256/SUB floats]
// Inside each group of four elements the order is (0, 2, 1, 3), so that one 8-byte load yields
// both B registers of an MMA whose A fragment was cut from four consecutive code bytes.  The pad
// (8 bytes per sub-block) spreads the live lanes of a B-fragment load over distinct banks.
template <int SUB>
struct Slab {
  static constexpr int NSUB = 256 / SUB;
  static constexpr int SUB_BYTES = SUB * 2 + 8;
  static constexpr int LO_OFF = NSUB * SUB_BYTES;
  static constexpr int SX_OFF = 2 * LO_OFF;
  static constexpr int BYTES = SX_OFF + NSUB * 4;
  static constexpr int ZERO_BYTES = LO_OFF + SUB_BYTES * NSUB;  // a zero page as large as hi + lo
};

// Converts one block's activations (two float4 per lane, already loaded) into the warp's slab.
// Returns the power of two the block's partial sums must be multiplied by (exact prescale that
// keeps |x| inside f16 range; 1 unless some |x| >= 2^15).
template <int SUB>
__device__ __forceinline__ float stage_block(const float4 (&xv)[2], uint32_t slab, int lane) {
  using S = Slab<SUB>;
  uint32_t m = 0;
#pragma unroll
  for (int i = 0; i < 2; i++) {
    m = max(m, __float_as_uint(xv[i].x) & 0x7fffffffu);
    m = max(m, __float_as_uint(xv[i].y) & 0x7fffffffu);
    m = max(m, __float_as_uint(xv[i].z) & 0x7fffffffu);
    m = max(m, __float_as_uint(xv[i].w) & 0x7fffffffu);
  }
  m = __reduce_max_sync(0xffffffffu, m);
  int sh = (int)(m >> 23) - 127 - 14;
  sh = sh < 0 ? 0 : (sh > 100 ? 100 : sh);
  const float down = __uint_as_float((uint32_t)(127 - sh) << 23), up = __uint_as_float((uint32_t)(127 + sh) << 23);
  constexpr int LPS = SUB / 4;  // lanes per sub-block
#pragma unroll
  for (int i = 0; i < 2; i++) {
    float4 v = xv[i];
    if (sh) v.x *= down, v.y *= down, v.z *= down, v.w *= down;
    __half2 h02 = __floats2half2_rn(v.x, v.z), h13 = __floats2half2_rn(v.y, v.w);
    float2 f02 = __half22float2(h02), f13 = __half22float2(h13);
    __half2 l02 = __floats2half2_rn(v.x - f02.x, v.z - f02.y), l13 = __floats2half2_rn(v.y - f13.x, v.w - f13.y);
    const int e = i * 128 + lane * 4;  // element index inside the block
    const uint32_t a = slab + (e / SUB) * S::SUB_BYTES + (e % SUB) * 2;
    sts64(a, *reinterpret_cast<uint32_t *>(&h02), *reinterpret_cast<uint32_t *>(&h13));
    sts64(a + S::LO_OFF, *reinterpret_cast<uint32_t *>(&l02), *reinterpret_cast<uint32_t *>(&l13));
    float s = (v.x + v.y) + (v.z + v.w);
#pragma unroll
    for (int o = 1; o < LPS; o <<= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((lane & (LPS - 1)) == 0)
      asm volatile("st.shared.f32 [%0], %1;\n" ::"r"(slab + S::SX_OFF + (e / SUB) * 4), "f"(s));
  }
  return up;
}

// ------------------------------------------------------------------------------------ Q4_K
//
// Block (144 B): [f16 d | f16 dmin | scales[12] | qs[128]]; byte qs[32p + l] holds element
// 64p + l (low nibble, sub-block 2p) and 64p + 32 + l (high nibble, sub-block 2p+1).
// Lane (g, t) loads the 32 qs bytes of pair p = t of rows g and g+8 (two 16-byte loads each)
// and the 16-byte header of both rows.  Code word i (bytes 4i..4i+3) feeds two MMAs:
//   even sub-block 2t:   a0 = codes(b0.lo, b2.lo)  a2 = codes(b1.lo, b3.lo)  (k slots 2t,2t+1 | 2t+8,2t+9)
//   odd  sub-block 2t+1: the same with the high nibbles.
// All four come out as f16 (64 + code): (word >> {-4, 4, 0, 8}) & 0x00F000F0 | 0x54005400.
// The B lane (col c, tid) is non-zero only when c == 2*tid (even MMA) or c == 2*tid+1 (odd MMA);
// all other lanes read a page of zeros.

struct Q4KTile {
  uint4 h0, h1, qa0, qa1, qb0, qb1;  // headers of rows g, g+8; the 32 code bytes of pair t of each
};


// ---- row-split execution over several GPUs, with the exchange inside the matmul launches.
// A rank computes rows [rank n, (rank + 1) n) of an output of `world` n rows.  Instead of a gather
// launch between two matmuls, the PRODUCER's epilogue stores every value it owns, as an 8-byte
// {value, step tag} slot, into the receive buffer of every rank (plain NVLink peer stores; its own
// rank included), and the CONSUMER's activation load polls its own receive buffer until the slots
// carry the current step's tag: the data is its own arrival flag, there is no fence and no extra
// launch.  Receive buffers hold two sets of slots, used on alternating steps.
struct TpArgs {
  const uint2 *x_slots;                // this launch's activations as 2 K slots (two step parities); nullptr: plain f32 x
  uint2 *peer[4][LB200_MAX_PEERS];     // per matrix: every rank's receive buffer for its output; peer[j][0] == nullptr: not exchanged
  const unsigned int *step;            // device step word: the tag
  int world, rank;
};

__device__ int g_tp_status;  // non-zero: a bounded wait for a peer's activations gave up (sticky)

// four consecutive slots -> four activations, once all four carry `tag` (bounded: about 50 ms)
__device__ __forceinline__ float4 ld_slots4(const uint2 *s, unsigned int tag, unsigned long long t0, bool &gave_up) {
  uint4 a, b;
  for (unsigned int it = 0;; it++) {
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w) : "l"(s) : "memory");
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(s + 2) : "memory");
    if ((a.y == tag && a.w == tag && b.y == tag && b.w == tag) || gave_up) break;
    if ((it & 255u) == 255u) {
      unsigned long long t1;
      asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(t1));
      if (t1 - t0 > 50000000ull) {  // a peer is gone or a step behind for good
        g_tp_status = 1;
        gave_up = true;
      }
    }
  }
  return make_float4(__uint_as_float(a.x), __uint_as_float(a.z), __uint_as_float(b.x), __uint_as_float(b.z));
}
// one output value of row `e` of the full-height output to every rank
__device__ __forceinline__ void st_slots(uint2 *const (&peer)[LB200_MAX_PEERS], int world, size_t e, float v, unsigned int tag) {
  for (int p = 0; p < world; p++)
    asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};\n" ::"l"(peer[p] + e), "r"(__float_as_uint(v)), "r"(tag) : "memory");
}

// Up to four weight matrices that share one activation row and one K, served by ONE launch: the
// row tiles of all of them form one list, which the CTAs split evenly.  With act != 0 there are
// two matrices of equal height (gate, up), their tiles alternate in the list, and the launch
// stores act(gate . x) * (up . x) into out[0].
struct MultiArgs {
  const uint8_t *w[4];
  float *out[4];
  int n[4];     // rows of each matrix (>= 16)
  int tend[4];  // running total of row tiles (not used when act != 0)
  int count;
  int act;      // 0: plain outputs, 1: SiLU gate, 2: GELU (erf) gate
};

// Which matrix and which first row tile T of the list stands for.  A tile that would run past the
// last row is pulled back to n - 16: it recomputes rows of the tile before it, and the duplicate
// stores write identical values.
__device__ __forceinline__ void resolve_tile(const MultiArgs &a, int T, int &j, int &r0) {
  if (a.act) {
    j = T & 1;
    r0 = min((T >> 1) * ROWS, a.n[0] - ROWS);
    return;
  }
  j = 0;
  int base = 0;
#pragma unroll
  for (int i = 1; i < 4; i++)
    if (i < a.count && T >= a.tend[i - 1]) j = i, base = a.tend[i - 1];
  r0 = min((T - base) * ROWS, a.n[j] - ROWS);
}

__device__ __forceinline__ float gate_act(float v, int act) {
  return act == 1 ? v / (1.f + expf(-v)) : 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
}

constexpr int Q4K_TILE_BYTES = ROWS * 144;  // one K block of 16 rows, dense in shared memory
constexpr int GROUP = 4;                    // row tiles whose partial sums a CTA holds at a time
constexpr int Q4K_SLAB = Slab<32>::BYTES + 16;  // a block's activations + its prescale factor

// One CTA per SM slot walks a contiguous range of row tiles (a balanced share of N/16), GROUP tiles
// at a time; its warps take the K blocks round-robin and meet once per group to add up their parts.
//
// The packed tiles travel global -> shared with 16-byte asynchronous copies into a ring of S tiles
// per warp, requested S tiles ahead of their use: the bytes in flight per SM (what hides the DRAM
// latency) are set by the ring, not by registers, and the ring keeps filling across group
// boundaries.  Each of the 144 chunks of a tile is fetched once (lane l takes chunks l, l+32, ...).
// Row r of a tile sits at r*144 in its slot: 16-byte reads of lanes (g, t) at g*144 + 16 + 32t fall
// into distinct banks.
//
// The grid never exceeds the SM count and a CTA takes less than half of an SM, so under
// programmatic dependent launch the NEXT launch of the stream is resident beside this one: its
// rings fill with its own weights (requested before griddepcontrol.wait) while this launch
// computes, and HBM stays busy through the dependency bubble between two launches.
//
// All activations are converted once per CTA (warp w converts the blocks it will use), so the
// tile loop holds no activation traffic at all.
// RMSNorm (and the residual add before it) folded into the launch: the activations are s = x + residual
// (residual may be null), every CTA stages s * weight and accumulates sum(s^2) on the way, and the outputs
// are multiplied by rsqrt(mean(s^2) + eps) at the end -- W (s w) r = r W (s w).  CTA 0 writes s to sum_out
// (the new residual stream), which therefore must not alias x or residual: the other CTAs still read them.
struct NormArgs {
  const float *weight, *residual;
  float *sum_out;
  float eps;
};

template <int S, int MINB, bool TP, bool NORM = false>
__global__ void __launch_bounds__(WARPS * 32, MINB) q4k_gemv_mma_kernel(const float *__restrict__ x,
                                                                       const __grid_constant__ MultiArgs a,
                                                                       const __grid_constant__ TpArgs tp,
                                                                       const __grid_constant__ NormArgs nrm, int tiles, int K) {
  __shared__ float nrm_part[WARPS];
  using SL = Slab<32>;
  extern __shared__ __align__(16) unsigned char dyn[];  // [ring: WARPS x S tiles][slabs: K/256]
  __shared__ __align__(16) unsigned char zero[SL::ZERO_BYTES];
  __shared__ __align__(16) float2 red[2][WARPS * GROUP * 32];  // by group parity
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int nb = K >> 8;
  const uint32_t row_bytes = (uint32_t)nb * 144u;
  for (int i = threadIdx.x; i < SL::ZERO_BYTES / 4; i += WARPS * 32) reinterpret_cast<uint32_t *>(zero)[i] = 0u;

  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(dyn) + warp * (S * Q4K_TILE_BYTES);
  const uint32_t slabs = (uint32_t)__cvta_generic_to_shared(dyn) + WARPS * S * Q4K_TILE_BYTES;
  const uint32_t szero = (uint32_t)__cvta_generic_to_shared(zero);
  const uint32_t red_lane = (uint32_t)__cvta_generic_to_shared(&red[0][warp * GROUP * 32 + lane]);
  constexpr uint32_t RED_PARITY = WARPS * GROUP * 32 * 8;
  // B addresses inside a slab.  The even MMA works on sub-block 2t of A-lane t: its column 2t
  // carries the hi half of x and the otherwise unused column 2t+1 the lo half, so one MMA does
  // both.  The odd MMA (sub-block 2t+1) has hi in column 2t+1 and lo in column 2t.  Every other
  // column reads zeros.
  const bool mine = (g >> 1) == t;
  const uint32_t pe_off = (2 * t) * SL::SUB_BYTES + ((g & 1) ? SL::LO_OFF : 0);
  const uint32_t po_off = (2 * t + 1) * SL::SUB_BYTES + ((g & 1) ? 0 : SL::LO_OFF);
  const bool hdr_hi = t >= 2;
  const int hdr_sh = (t & 1) * 16;
  const uint32_t mask = 0x00F000F0u, magic = 0x54005400u;  // f16 (64 + nibble)

  // this CTA's share [t0, t1) of the tile list (whole gate/up pairs when act != 0)
  const int unit = a.act ? 2 : 1, lt = tiles / unit;
  const int t0 = (int)((uint32_t)lt * blockIdx.x / gridDim.x) * unit,  // lt * gridDim.x < 2^32 (launcher)
            t1 = (int)((uint32_t)lt * (blockIdx.x + 1) / gridDim.x) * unit;

  // source offsets of this lane's chunks, relative to the tile's first byte (row 0, this block)
  uint32_t soff[5];
#pragma unroll
  for (int i = 0; i < 5; i++) {
    const uint32_t c = lane + 32 * i, row = c / 9u;
    soff[i] = row * row_bytes + (c - 9u * row) * 16u;
  }
  const uint32_t ld_off = g * 144u + 32u * t;
  // The requests run S units ahead of the arithmetic; both walk (group, block, tile) in this order.
  int i_gt = t0, i_gs = min(GROUP, t1 - t0), i_b = warp, i_rt = 0, i_slot = 0;
  auto issue = [&]() {  // always closes a commit group, so that group counts stay uniform
    if (i_gt < t1 && warp < nb) {
      int j, r0;
      resolve_tile(a, i_gt + i_rt, j, r0);
      const uint8_t *base = a.w[j] + ((size_t)r0 * row_bytes + (uint32_t)i_b * 144u);
      const uint32_t dst = ring + i_slot * Q4K_TILE_BYTES + lane * 16;
#pragma unroll
      for (int i = 0; i < 4; i++) cp_async16(dst + i * 512, base + soff[i]);
      if (lane < 16) cp_async16(dst + 2048, base + soff[4]);
      i_slot = (i_slot + 1) & (S - 1);
      if (++i_rt == i_gs) {
        i_rt = 0, i_b += WARPS;
        if (i_b >= nb) i_b = warp, i_gt += i_gs, i_gs = min(GROUP, t1 - i_gt);
      }
    }
    cp_async_commit();
  };
#pragma unroll 1
  for (int p = 0; p < S; p++) issue();
  pdl_wait();  // x is the previous launch's output; the weights requested above are not
  unsigned int tag = 0;
  unsigned long long tp_t0 = 0;
  bool tp_gave_up = false;
  if constexpr (TP) {
    tag = *reinterpret_cast<const volatile unsigned int *>(tp.step);
    if (tp.x_slots) asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(tp_t0));
  }
  float nrm_ss = 0.f;
  for (int b = warp; b < nb; b += WARPS) {
    float4 xv[2];
    if (TP && tp.x_slots) {  // the peers' parts of x arrive as tagged slots
      const uint2 *xs = tp.x_slots + (size_t)(tag & 1u) * K + b * 256 + lane * 4;
      xv[0] = ld_slots4(xs, tag, tp_t0, tp_gave_up);
      xv[1] = ld_slots4(xs + 128, tag, tp_t0, tp_gave_up);
    } else {
      xv[0] = __ldg(reinterpret_cast<const float4 *>(x + b * 256) + lane);
      xv[1] = __ldg(reinterpret_cast<const float4 *>(x + b * 256 + 128) + lane);
    }
    if constexpr (NORM) {
#pragma unroll
      for (int i = 0; i < 2; i++) {
        const int e4 = b * 64 + i * 32 + lane;  // float4 index into the row
        if (nrm.residual) {
          const float4 r = __ldg(reinterpret_cast<const float4 *>(nrm.residual) + e4);
          xv[i].x += r.x, xv[i].y += r.y, xv[i].z += r.z, xv[i].w += r.w;
          if (blockIdx.x == 0) reinterpret_cast<float4 *>(nrm.sum_out)[e4] = xv[i];
        }
        nrm_ss = fmaf(xv[i].x, xv[i].x, fmaf(xv[i].y, xv[i].y, fmaf(xv[i].z, xv[i].z, fmaf(xv[i].w, xv[i].w, nrm_ss))));
        const float4 wn = __ldg(reinterpret_cast<const float4 *>(nrm.weight) + e4);
        xv[i].x *= wn.x, xv[i].y *= wn.y, xv[i].z *= wn.z, xv[i].w *= wn.w;
      }
    }
    const uint32_t slab = slabs + b * Q4K_SLAB;
    const float up = stage_block<32>(xv, slab, lane);
    if (lane == 0) asm volatile("st.shared.f32 [%0], %1;\n" ::"r"(slab + SL::BYTES), "f"(up));
  }
  if constexpr (NORM) {
    nrm_ss = warp_sum(nrm_ss);
    if (lane == 0) nrm_part[warp] = nrm_ss;
  }
  __syncthreads();
  float nrm_inv = 1.f;
  if constexpr (NORM) {
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < WARPS; i++) tot += nrm_part[i];
    nrm_inv = (float)(1.0 / sqrt((double)(tot / (float)K) + (double)nrm.eps));
  }
  int slot = 0, parity = 0;
  for (int gt = t0; gt < t1; gt += GROUP, parity ^= 1) {
    const int gs = min(GROUP, t1 - gt);
    const uint32_t red_g = red_lane + parity * RED_PARITY;
    for (int b = warp; b < nb; b += WARPS) {
      const uint32_t slab = slabs + b * Q4K_SLAB;
      const uint32_t pe = mine ? slab + pe_off : szero, po = mine ? slab + po_off : szero;
      float2 sx;
      float up;
      asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];\n" : "=f"(sx.x), "=f"(sx.y) : "r"(slab + SL::SX_OFF + 8 * t));
      asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(up) : "r"(slab + SL::BYTES));
      for (int rt = 0; rt < gs; rt++) {
        cp_async_wait<S - 1>();  // this lane's chunks of the tile have landed ...
        __syncwarp();            // ... and so have the other lanes'
        const uint32_t sb = ring + slot * Q4K_TILE_BYTES + ld_off;
        slot = (slot + 1) & (S - 1);
        const uint4 h0 = lds128(sb - 32u * t), h1 = lds128(sb - 32u * t + 8 * 144);
        const uint4 qa0 = lds128(sb + 16), qa1 = lds128(sb + 32);
        const uint4 qb0 = lds128(sb + 8 * 144 + 16), qb1 = lds128(sb + 8 * 144 + 32);
        __syncwarp();  // the slot is free again
        issue();
        float dsc[2][2], dmn[2][2];
        q4k_scales(h0, hdr_hi, hdr_sh, dsc[0], dmn[0]);
        q4k_scales(h1, hdr_hi, hdr_sh, dsc[1], dmn[1]);
        float de[4] = {0.f, 0.f, 0.f, 0.f}, dq[4] = {0.f, 0.f, 0.f, 0.f};  // even / odd sub-block chains
        const uint32_t qg[8] = {qa0.x, qa0.y, qa0.z, qa0.w, qa1.x, qa1.y, qa1.z, qa1.w};
        const uint32_t qh[8] = {qb0.x, qb0.y, qb0.z, qb0.w, qb1.x, qb1.y, qb1.z, qb1.w};
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const uint32_t vg = qg[i], vh = qh[i];
          const uint32_t e0 = and_or(vg << 4, mask, magic), e1 = and_or(vh << 4, mask, magic);
          const uint32_t e2 = and_or(vg >> 4, mask, magic), e3 = and_or(vh >> 4, mask, magic);
          const uint32_t o0 = and_or(vg, mask, magic), o1 = and_or(vh, mask, magic);
          const uint32_t o2 = and_or(vg >> 8, mask, magic), o3 = and_or(vh >> 8, mask, magic);
          const uint2 be = lds64(pe + i * 8), bo = lds64(po + i * 8);
          mma16816(de, e0, e1, e2, e3, be.x, be.y);
          mma16816(dq, o0, o1, o2, o3, bo.x, bo.y);
        }
        // lane (g, t): de[0] + de[1] = row g, sub-block 2t (hi + lo parts of x); dq[0] + dq[1] =
        // row g, sub-block 2t+1; [2], [3] the same for row g+8.
        float vr[2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
          float v = dsc[r][0] * (de[2 * r] + de[2 * r + 1]) - (64.f * dsc[r][0] + dmn[r][0]) * sx.x;
          v += dsc[r][1] * (dq[2 * r] + dq[2 * r + 1]) - (64.f * dsc[r][1] + dmn[r][1]) * sx.y;
          vr[r] = v * up;
        }
        // the warp's first block of a group overwrites what an earlier group left behind
        const uint32_t ra = red_g + rt * (32 * 8);
        float2 o = make_float2(0.f, 0.f);
        if (b != warp) asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];\n" : "=f"(o.x), "=f"(o.y) : "r"(ra));
        asm volatile("st.shared.v2.f32 [%0], {%1,%2};\n" ::"r"(ra), "f"(o.x + vr[0]), "f"(o.y + vr[1]));
      }
    }
    // red[parity][warp][rt][lane] (float2: rows g, g+8): sum the four t-lanes of a row and the
    // warps in a fixed order.
    __syncthreads();  // also orders this group's reads of red[parity] before its reuse two groups on
    auto row_sum = [&](int rt, int row) {
      const int gg = row & 7, hi = row >> 3;
      float v = 0.f;
#pragma unroll
      for (int wq = 0; wq < WARPS; wq++) {
        if (wq >= nb) break;  // a warp without a K block never wrote its part
        const float2 *p = &red[parity][(wq * GROUP + rt) * 32 + gg * 4];
#pragma unroll
        for (int tt = 0; tt < 4; tt++) v += hi ? p[tt].y : p[tt].x;
      }
      return v;
    };
    if (a.act) {
      for (int i = threadIdx.x; i < (gs >> 1) * ROWS; i += WARPS * 32) {
        const int pr = i >> 4, row = i & 15;
        int j, r0;
        resolve_tile(a, gt + 2 * pr, j, r0);
        const float v = gate_act(row_sum(2 * pr, row) * nrm_inv, a.act) * (row_sum(2 * pr + 1, row) * nrm_inv);
        a.out[0][r0 + row] = v;
        if (TP && tp.peer[0][0]) st_slots(tp.peer[0], tp.world, (size_t)(tag & 1u) * a.n[0] * tp.world + (size_t)tp.rank * a.n[0] + r0 + row, v, tag);
      }
    } else {
      for (int i = threadIdx.x; i < gs * ROWS; i += WARPS * 32) {
        const int rt = i >> 4, row = i & 15;
        int j, r0;
        resolve_tile(a, gt + rt, j, r0);
        const float v = row_sum(rt, row) * nrm_inv;
        a.out[j][r0 + row] = v;
        if (TP && tp.peer[j][0]) st_slots(tp.peer[j], tp.world, (size_t)(tag & 1u) * a.n[j] * tp.world + (size_t)tp.rank * a.n[j] + r0 + row, v, tag);
      }
    }
  }
  cp_async_wait<0>();
}

// ------------------------------------------------------------------------------------ Q4_K, 2 .. 8 rows of x
//
// The same persistent, ring-fed decomposition as q4k_gemv_mma_kernel, with the eight MMA columns
// given to eight TOKENS.  A lane then needs weights that carry their sub-block scale, because one
// accumulator sums over the whole 256-element block:
//   * codes -> f16 (64 + q) by LOP3 as before, then ONE HFMA2 with the 6-bit scale: (64 + q) * sc
//     - 64 * sc = q * sc, exact (an integer below 2048).  D = sum_k (q * sc)_k x_k over the block,
//     accumulated by the tensor core; once per block and row, acc += d * D.
//   * the minimum term -dmin * m_s * sum_{k in s} x_k is a second tiny contraction over the eight
//     sub-blocks: A' = -dmin * m split into f16 hi + lo (k slots 0-7 and 8-15), B' = the
//     per-sub-block sums of x as f16 hi (both k halves), then A' = hi only against the lo half of
//     the sums: two MMAs per block, straight into the running accumulator.
// x is rounded to f16 (no hi/lo split of the activations themselves): 2^-11 relative per element,
// about 2e-4 relative L2 on the output, inside the 1e-3 bound for M >= 2.
// A warp converts its K block's x for all tokens into a private slab (token stride 544 B: the
// 8-byte B-fragment loads of lanes (token g, t) fall into distinct banks), once per group of four
// row tiles.
constexpr int TOK = 8;                       // tokens per launch (MMA N)
constexpr int TOK_PITCH = 544;               // bytes per token in a warp's slab
constexpr int TOK_SX = TOK * TOK_PITCH;      // then per token: 8 sub-block sums as f16 hi | 8 as f16 lo
constexpr int TOK_SLAB = TOK_SX + TOK * 32;
constexpr int Q4K_TOK_STAGES = 3;
constexpr int Q4K_TOK_SMEM = WARPS * Q4K_TOK_STAGES * Q4K_TILE_BYTES + WARPS * TOK_SLAB + WARPS * GROUP * 32 * 16;

__device__ __forceinline__ uint32_t h2_as_u32(__half2 v) { return *reinterpret_cast<uint32_t *>(&v); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t v) { return *reinterpret_cast<__half2 *>(&v); }

template <int S>
__global__ void __launch_bounds__(WARPS * 32, 2) q4k_gemv_tok_kernel(const float *__restrict__ x, const __grid_constant__ MultiArgs ma,
                                                                    int tiles, int M, int K) {
  extern __shared__ __align__(16) unsigned char dyn[];  // [ring: WARPS x S tiles][slabs: WARPS][red: WARPS x GROUP x 32 float4]
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int nb = K >> 8;
  const uint32_t row_bytes = (uint32_t)nb * 144u;
  const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(dyn);
  const uint32_t ring = sbase + warp * (S * Q4K_TILE_BYTES);
  const uint32_t slab = sbase + WARPS * S * Q4K_TILE_BYTES + warp * TOK_SLAB;
  const uint32_t red = sbase + WARPS * S * Q4K_TILE_BYTES + WARPS * TOK_SLAB;
  const uint32_t red_lane = red + (uint32_t)((warp * GROUP) * 32 + lane) * 16u;
  const bool hdr_hi = t >= 2;
  const int hdr_sh = (t & 1) * 16;
  const uint32_t mask = 0x00F000F0u, magic = 0x54005400u;  // f16 (64 + nibble)

  const int t0 = (int)((uint32_t)tiles * blockIdx.x / gridDim.x), t1 = (int)((uint32_t)tiles * (blockIdx.x + 1) / gridDim.x);
  uint32_t soff[5];
#pragma unroll
  for (int i = 0; i < 5; i++) {
    const uint32_t c = lane + 32 * i, row = c / 9u;
    soff[i] = row * row_bytes + (c - 9u * row) * 16u;
  }
  const uint32_t ld_off = g * 144u + 32u * t;

  int i_gt = t0, i_gs = min(GROUP, t1 - t0), i_b = warp, i_rt = 0, i_slot = 0;
  auto issue = [&]() {  // always closes a commit group, so that group counts stay uniform
    if (i_gt < t1 && warp < nb) {
      int j, r0;
      resolve_tile(ma, i_gt + i_rt, j, r0);  // up to four matrices that share x form one tile list
      const uint8_t *base = ma.w[j] + ((size_t)r0 * row_bytes + (uint32_t)i_b * 144u);
      const uint32_t dst = ring + i_slot * Q4K_TILE_BYTES + lane * 16;
#pragma unroll
      for (int i = 0; i < 4; i++) cp_async16(dst + i * 512, base + soff[i]);
      if (lane < 16) cp_async16(dst + 2048, base + soff[4]);
      i_slot = i_slot + 1 == S ? 0 : i_slot + 1;
      if (++i_rt == i_gs) {
        i_rt = 0, i_b += WARPS;
        if (i_b >= nb) i_b = warp, i_gt += i_gs, i_gs = min(GROUP, t1 - i_gt);
      }
    }
    cp_async_commit();
  };
#pragma unroll 1
  for (int p = 0; p < S; p++) issue();
  pdl_wait();  // x is the previous launch's output; the weights requested above are not

  int slot = 0;
  for (int gt = t0; gt < t1; gt += GROUP) {
    const int gs = min(GROUP, t1 - gt);
    float acc[GROUP][4];
#pragma unroll
    for (int r = 0; r < GROUP; r++) acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.f;
    for (int b = warp; b < nb; b += WARPS) {
      // ---- this block's activations, all tokens, into the warp's slab.  A token's 256 values are 64
      // float4: lane l takes float4 l and l + 32 (coalesced), i.e. four values of sub-block l / 8 (+ 4).
      __syncwarp();  // every lane is done reading the previous block's slab
#pragma unroll 4
      for (int tk = 0; tk < TOK; tk++) {
        const float4 *xp = reinterpret_cast<const float4 *>(x + (size_t)tk * K + b * 256);
        float4 v[2];
        v[0] = v[1] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (tk < M) v[0] = __ldg(xp + lane), v[1] = __ldg(xp + lane + 32);
        float s[2];
#pragma unroll
        for (int j = 0; j < 2; j++) {
          const int F = lane + 32 * j;  // elements 4F .. 4F+3 = 64 (F / 16) + 32 ((F / 8) & 1) + 4 (F & 7) + 0..3
          const __half2 lim = __float2half2_rn(65504.f);
          const __half2 h02 = __hmax2(__hmin2(__floats2half2_rn(v[j].x, v[j].z), lim), __hneg2(lim));
          const __half2 h13 = __hmax2(__hmin2(__floats2half2_rn(v[j].y, v[j].w), lim), __hneg2(lim));
          sts64(slab + tk * TOK_PITCH + (uint32_t)((((F >> 3) & 1) * 8 + (F & 7)) * 4 + (F >> 4)) * 8u, h2_as_u32(h02), h2_as_u32(h13));
          // the sums are those of the ROUNDED values, the ones the tensor core multiplies
          const float2 a = __half22float2(h02), c = __half22float2(h13);
          float p = (a.x + a.y) + (c.x + c.y);
          p += __shfl_xor_sync(0xffffffffu, p, 1), p += __shfl_xor_sync(0xffffffffu, p, 2), p += __shfl_xor_sync(0xffffffffu, p, 4);
          s[j] = p;  // sub-block (lane / 8) + 4 j
        }
        // lanes 0 and 16 (j = 0: sub-blocks 0,1 / 2,3; j = 1: 4,5 / 6,7) write the hi | lo pairs
        const float n0 = __shfl_down_sync(0xffffffffu, s[0], 8), n1 = __shfl_down_sync(0xffffffffu, s[1], 8);
        if ((lane & 15) == 0) {
#pragma unroll
          for (int j = 0; j < 2; j++) {
            const float a0 = s[j], a1 = j ? n1 : n0;
            const __half2 slim = __float2half2_rn(65504.f);  // sums of clamped values can leave the f16 range too
            const __half2 hi = __hmax2(__hmin2(__floats2half2_rn(a0, a1), slim), __hneg2(slim));
            const float2 hf = __half22float2(hi);
            const __half2 lo = __hmax2(__hmin2(__floats2half2_rn(a0 - hf.x, a1 - hf.y), slim), __hneg2(slim));
            const uint32_t at = slab + TOK_SX + tk * 32 + 4 * ((lane >> 4) + 2 * j);
            asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(at), "r"(h2_as_u32(hi)));
            asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(at + 16), "r"(h2_as_u32(lo)));
          }
        }
      }
      __syncwarp();
      const uint32_t bx = slab + g * TOK_PITCH + t * 8;  // B fragments of token g
      const uint32_t sx_hi = lds32(slab + TOK_SX + g * 32 + 4 * t), sx_lo = lds32(slab + TOK_SX + g * 32 + 16 + 4 * t);
#pragma unroll
      for (int rt = 0; rt < GROUP; rt++) {
        if (rt < gs) {
          cp_async_wait<S - 1>();  // this lane's chunks of the tile have landed ...
          __syncwarp();            // ... and so have the other lanes'
          const uint32_t sb = ring + slot * Q4K_TILE_BYTES + ld_off;
          slot = slot + 1 == S ? 0 : slot + 1;
          const uint4 h0 = lds128(sb - 32u * t), h1 = lds128(sb - 32u * t + 8 * 144);
          const uint4 qa0 = lds128(sb + 16), qa1 = lds128(sb + 32);
          const uint4 qb0 = lds128(sb + 8 * 144 + 16), qb1 = lds128(sb + 8 * 144 + 32);
          __syncwarp();  // the slot is free again
          issue();
          // 6-bit scales and minima of sub-blocks 2t, 2t+1 of rows g (h0) and g+8 (h1)
          __half2 s2[2][2], c2[2][2];
          uint32_t dmh[2], dml[2];
          float dd[2];
#pragma unroll
          for (int r = 0; r < 2; r++) {
            const uint4 &h = r ? h1 : h0;
            const float2 df = __half22float2(u32_as_h2(h.x));  // (d, dmin)
            const uint32_t scw = hdr_hi ? ((h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u)) : (h.y & 0x3F3F3F3Fu);
            const uint32_t mnw = hdr_hi ? (((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u)) : (h.z & 0x3F3F3F3Fu);
            const uint32_t sc = scw >> hdr_sh, mn = mnw >> hdr_sh;
            s2[r][0] = __half2half2(__uint2half_rn(sc & 0xFFu)), s2[r][1] = __half2half2(__uint2half_rn((sc >> 8) & 0xFFu));
            c2[r][0] = __hmul2(s2[r][0], __float2half2_rn(-64.f)), c2[r][1] = __hmul2(s2[r][1], __float2half2_rn(-64.f));
            const float m0 = -df.y * (float)(mn & 0xFFu), m1 = -df.y * (float)((mn >> 8) & 0xFFu);
            const __half2 mh = __floats2half2_rn(m0, m1);
            const float2 mf = __half22float2(mh);
            dmh[r] = h2_as_u32(mh), dml[r] = h2_as_u32(__floats2half2_rn(m0 - mf.x, m1 - mf.y));
            dd[r] = df.x;
          }
          float dq[4] = {0.f, 0.f, 0.f, 0.f};
          const uint32_t qg[8] = {qa0.x, qa0.y, qa0.z, qa0.w, qa1.x, qa1.y, qa1.z, qa1.w};
          const uint32_t qh[8] = {qb0.x, qb0.y, qb0.z, qb0.w, qb1.x, qb1.y, qb1.z, qb1.w};
          auto scl = [](uint32_t raw, __half2 s, __half2 c) { return h2_as_u32(__hfma2(u32_as_h2(raw), s, c)); };
#pragma unroll
          for (int i = 0; i < 8; i++) {
            const uint32_t vg = qg[i], vh = qh[i];
            const uint32_t e0 = scl(and_or(vg << 4, mask, magic), s2[0][0], c2[0][0]), e1 = scl(and_or(vh << 4, mask, magic), s2[1][0], c2[1][0]);
            const uint32_t e2 = scl(and_or(vg >> 4, mask, magic), s2[0][0], c2[0][0]), e3 = scl(and_or(vh >> 4, mask, magic), s2[1][0], c2[1][0]);
            const uint32_t o0 = scl(and_or(vg, mask, magic), s2[0][1], c2[0][1]), o1 = scl(and_or(vh, mask, magic), s2[1][1], c2[1][1]);
            const uint32_t o2 = scl(and_or(vg >> 8, mask, magic), s2[0][1], c2[0][1]), o3 = scl(and_or(vh >> 8, mask, magic), s2[1][1], c2[1][1]);
            const uint2 be = lds64(bx + i * 32), bo = lds64(bx + (8 + i) * 32);
            mma16816(dq, e0, e1, e2, e3, be.x, be.y);
            mma16816(dq, o0, o1, o2, o3, bo.x, bo.y);
          }
          acc[rt][0] = fmaf(dd[0], dq[0], acc[rt][0]), acc[rt][1] = fmaf(dd[0], dq[1], acc[rt][1]);
          acc[rt][2] = fmaf(dd[1], dq[2], acc[rt][2]), acc[rt][3] = fmaf(dd[1], dq[3], acc[rt][3]);
          mma16816(acc[rt], dmh[0], dmh[1], dml[0], dml[1], sx_hi, sx_hi);
          mma16816(acc[rt], dmh[0], dmh[1], 0u, 0u, sx_lo, 0u);
        }
      }
    }
    // ---- add up the warps' parts: lane (g, t) of tile rt holds rows g, g+8 x tokens 2t, 2t+1
    __syncthreads();  // the previous group's sums have been read
#pragma unroll
    for (int rt = 0; rt < GROUP; rt++)
      asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};\n" ::"r"(red_lane + rt * 512), "f"(acc[rt][0]), "f"(acc[rt][1]),
                   "f"(acc[rt][2]), "f"(acc[rt][3]));
    __syncthreads();
    for (int i = threadIdx.x; i < gs * ROWS * TOK; i += WARPS * 32) {
      const int row = i & 15, tok = (i >> 4) & 7, rt = i >> 7;
      const uint32_t a = red + (uint32_t)(rt * 32 + (row & 7) * 4 + (tok >> 1)) * 16u + (uint32_t)((row >> 3) * 2 + (tok & 1)) * 4u;
      float v = 0.f;
#pragma unroll
      for (int wq = 0; wq < WARPS; wq++) {
        if (wq >= nb) break;  // a warp without a K block holds zeros it never stored
        float p;
        asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(p) : "r"(a + wq * (GROUP * 512)));
        v += p;
      }
      if (tok < M) {
        int j, r0;
        resolve_tile(ma, gt + rt, j, r0);
        ma.out[j][(size_t)tok * ma.n[j] + r0 + row] = v;
      }
    }
  }
  cp_async_wait<0>();
}

// ------------------------------------------------------------------------------------ Q4_K, 9 .. 64 rows of x
//
// More tokens than one MMA has columns: the token-column arithmetic of q4k_gemv_tok_kernel with NG groups
// of eight tokens per code word, and a decomposition that lets all warps of a CTA share ONE copy of the
// converted activations.  A CTA owns eight consecutive row tiles (one per warp, no sum across warps) and
// walks a run of K blocks; every thread requests its share of block b + 1 of x (all tokens) before the
// warp works on block b and converts it into the other half of a double buffer afterwards, one CTA
// barrier per block.  K is split over a
// thread-block cluster of KS CTAs, whose partial sums meet in distributed shared memory at the end, as in
// decode_umma_kernel.  The expanded weights never leave registers: per 4096 weights this kernel issues
// about a third of the instructions of the shared-memory-operand kernel.
constexpr int DT_CW = 8, DT_THREADS = DT_CW * 32;
constexpr int DT_STAGES = 3;
constexpr int DT_RING = DT_CW * DT_STAGES * Q4K_TILE_BYTES;
template <int NG>
struct DtCfg {
  static constexpr int NT = 8 * NG;                        // token columns
  static constexpr int SX = NT * TOK_PITCH;                // then per token 8 hi | 8 lo sub-block sums
  static constexpr int XBUF = SX + NT * 32;
  static constexpr int SMEM = DT_RING + 2 * XBUF;
  static_assert(NT * 128 * 4 <= DT_RING, "the partial sums reuse the ring");
};

template <int NG>
__global__ void __launch_bounds__(DT_THREADS, 2) q4k_decode_tile_kernel(const float *__restrict__ x,
                                                                                     const __grid_constant__ MultiArgs ma, int tiles,
                                                                                     int M, int K) {
  using Cfg = DtCfg<NG>;
  constexpr int S = DT_STAGES;
  extern __shared__ __align__(16) unsigned char dyn[];  // [ring: 8 warps x S tiles][x buffer 0][x buffer 1]
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int nb = K >> 8;
  const int KS = gridDim.y, rank = blockIdx.y;
  const int b0 = nb * rank / KS, b1 = nb * (rank + 1) / KS, nloc = b1 - b0;
  // CTAs of one K run start at different blocks of it: otherwise all of them ask L2 for the same lines of x
  // at the same moment
  const int rot = (int)(blockIdx.x * 5u) % nloc;
  auto blk = [&](int i) { const int j = i + rot; return b0 + (j >= nloc ? j - nloc : j); };
  const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(dyn);
  const uint32_t xs0 = sbase + DT_RING;

  // this thread's share of a block of x: float4 F = tid & 63 of tokens (tid >> 6) + 4 j
  constexpr int XJ = Cfg::NT / 4;
  const int xF = threadIdx.x & 63, xT = threadIdx.x >> 6;
  auto x_load = [&](int b, float4 (&v)[XJ]) {
#pragma unroll
    for (int j = 0; j < XJ; j++) {
      const int tk = xT + 4 * j;
      v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (tk < M) v[j] = __ldg(reinterpret_cast<const float4 *>(x + (size_t)tk * K + b * 256) + xF);
    }
  };
  auto x_store = [&](uint32_t xb, const float4 (&v)[XJ]) {
#pragma unroll
    for (int j = 0; j < XJ; j++) {
      const int tk = xT + 4 * j;
      const __half2 lim = __float2half2_rn(65504.f);
      const __half2 h02 = __hmax2(__hmin2(__floats2half2_rn(v[j].x, v[j].z), lim), __hneg2(lim));
      const __half2 h13 = __hmax2(__hmin2(__floats2half2_rn(v[j].y, v[j].w), lim), __hneg2(lim));
      sts64(xb + tk * TOK_PITCH + (uint32_t)((((xF >> 3) & 1) * 8 + (xF & 7)) * 4 + (xF >> 4)) * 8u, h2_as_u32(h02), h2_as_u32(h13));
      const float2 a = __half22float2(h02), c = __half22float2(h13);
      float s = (a.x + a.y) + (c.x + c.y);  // of the ROUNDED values, the ones the tensor core multiplies
      s += __shfl_xor_sync(0xffffffffu, s, 1), s += __shfl_xor_sync(0xffffffffu, s, 2), s += __shfl_xor_sync(0xffffffffu, s, 4);
      const float s1 = __shfl_down_sync(0xffffffffu, s, 8);
      if ((lane & 15) == 0) {  // sub-blocks (F / 8, F / 8 + 1) = pair F / 16
        const __half2 hi = __hmax2(__hmin2(__floats2half2_rn(s, s1), lim), __hneg2(lim));  // sums of clamped values can leave the f16 range too
        const float2 hf = __half22float2(hi);
        const __half2 lo = __hmax2(__hmin2(__floats2half2_rn(s - hf.x, s1 - hf.y), lim), __hneg2(lim));
        asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(xb + Cfg::SX + tk * 32 + 4 * (xF >> 4)), "r"(h2_as_u32(hi)));
        asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(xb + Cfg::SX + tk * 32 + 16 + 4 * (xF >> 4)), "r"(h2_as_u32(lo)));
      }
    }
  };
  {
    // ---- consumers: warp w owns row tile 8 blockIdx.x + w over blocks b0 .. b1
    const int tile = blockIdx.x * DT_CW + warp;
    const bool live = tile < tiles;
    int wj = 0, r0 = 0;
    if (live) resolve_tile(ma, tile, wj, r0);  // up to four matrices that share x form one tile list
    const uint8_t *w = ma.w[wj];
    const uint32_t row_bytes = (uint32_t)nb * 144u;
    const uint32_t ring = sbase + warp * (S * Q4K_TILE_BYTES);
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
        const uint32_t dst = ring + i_slot * Q4K_TILE_BYTES + lane * 16;
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
    pdl_wait();  // x is the previous launch's output; the weights requested above are not
    {
      float4 v0[XJ];
      x_load(blk(0), v0);
      x_store(xs0, v0);
    }
    __syncthreads();

    float acc[NG][4];
#pragma unroll
    for (int q = 0; q < NG; q++) acc[q][0] = acc[q][1] = acc[q][2] = acc[q][3] = 0.f;
    int slot = 0;
    for (int bi = 0; bi < nloc; bi++) {
      const int half = bi & 1;
      const uint32_t xb = xs0 + half * Cfg::XBUF;
      float4 xn[XJ];
      if (bi + 1 < nloc) x_load(blk(bi + 1), xn);
      if (live) {
        cp_async_wait<S - 1>();
        __syncwarp();
        const uint32_t sb = ring + slot * Q4K_TILE_BYTES + ld_off;
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
          const float2 df = __half22float2(u32_as_h2(h.x));  // (d, dmin)
          const uint32_t scw = hdr_hi ? ((h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u)) : (h.y & 0x3F3F3F3Fu);
          const uint32_t mnw = hdr_hi ? (((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u)) : (h.z & 0x3F3F3F3Fu);
          const uint32_t sc = scw >> hdr_sh, mn = mnw >> hdr_sh;
          s2[r][0] = __half2half2(__uint2half_rn(sc & 0xFFu)), s2[r][1] = __half2half2(__uint2half_rn((sc >> 8) & 0xFFu));
          c2[r][0] = __hmul2(s2[r][0], __float2half2_rn(-64.f)), c2[r][1] = __hmul2(s2[r][1], __float2half2_rn(-64.f));
          const float m0 = -df.y * (float)(mn & 0xFFu), m1 = -df.y * (float)((mn >> 8) & 0xFFu);
          const __half2 mh = __floats2half2_rn(m0, m1);
          const float2 mf = __half22float2(mh);
          dmh[r] = h2_as_u32(mh), dml[r] = h2_as_u32(__floats2half2_rn(m0 - mf.x, m1 - mf.y));
          dd[r] = df.x;
        }
        float dq[NG][4];
#pragma unroll
        for (int q = 0; q < NG; q++) dq[q][0] = dq[q][1] = dq[q][2] = dq[q][3] = 0.f;
        const uint32_t qg[8] = {qa0.x, qa0.y, qa0.z, qa0.w, qa1.x, qa1.y, qa1.z, qa1.w};
        const uint32_t qh[8] = {qb0.x, qb0.y, qb0.z, qb0.w, qb1.x, qb1.y, qb1.z, qb1.w};
        auto scl = [](uint32_t raw, __half2 s, __half2 c) { return h2_as_u32(__hfma2(u32_as_h2(raw), s, c)); };
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
          const uint32_t sx_hi = lds32(xb + Cfg::SX + (q * 8 + g) * 32 + 4 * t), sx_lo = lds32(xb + Cfg::SX + (q * 8 + g) * 32 + 16 + 4 * t);
          mma16816(acc[q], dmh[0], dmh[1], dml[0], dml[1], sx_hi, sx_hi);
          mma16816(acc[q], dmh[0], dmh[1], 0u, 0u, sx_lo, 0u);
        }
      }
      if (bi + 1 < nloc) x_store(xs0 + (half ^ 1) * Cfg::XBUF, xn);
      __syncthreads();  // block b + 1 of x is in place, block b's half is free
    }
    cp_async_wait<0>();
    __syncthreads();  // every warp is done with its ring slots
    // ---- partial[token][128 rows of this CTA] over the (drained) ring
#pragma unroll
    for (int q = 0; q < NG; q++)
#pragma unroll
      for (int c = 0; c < 4; c++) {
        const int tok = q * 8 + 2 * t + (c & 1), row = warp * ROWS + g + 8 * (c >> 1);
        asm volatile("st.shared.f32 [%0], %1;\n" ::"r"(sbase + (uint32_t)(tok * 128 + row) * 4u), "f"(acc[q][c]));
      }
  }
  // ---- add up the cluster's partials: CTA `rank` stores tokens rank NT / KS ..
  if (KS > 1) umma::cluster_sync(); else __syncthreads();
  {
    const int per = Cfg::NT / KS;
    for (int idx = threadIdx.x; idx < per * 128; idx += DT_THREADS) {
      const int tok = rank * per + (idx >> 7), rr = idx & 127, tile = blockIdx.x * DT_CW + (rr >> 4);
      const uint32_t a = sbase + (uint32_t)(tok * 128 + rr) * 4u;
      float v = 0.f;
      if (KS > 1) {
        for (int p = 0; p < KS; p++) v += umma::ld_cluster_f32(umma::map_to_rank(a, (uint32_t)p));
      } else {
        asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(v) : "r"(a));
      }
      if (tok < M && tile < tiles) {
        int oj, orow;
        resolve_tile(ma, tile, oj, orow);
        ma.out[oj][(size_t)tok * ma.n[oj] + orow + (rr & 15)] = v;
      }
    }
  }
  if (KS > 1) umma::cluster_sync();  // nobody leaves while a peer still reads its partials
}

// ------------------------------------------------------------------------------------ Q6_K
//
// Block (210 B): [ql[128] | qh[64] | int8 sc[16] | f16 d]; element e = 128h + 32q + l
// (half h, group q, l < 32) has its low nibble in ql[64h + 32(q&1) + l] (high nibble when q >= 2)
// and bits 2q..2q+1 of qh[32h + l]; its sub-block of 16 is s = e / 16 = 8h + 2q + l/16.
// For each (h, u = l/16), lane (g, t) takes l = 16u + 4t .. +3 of rows g and g+8: one word of
// ql[64h + l], one of ql[64h + 32 + l] and one of qh[32h + l] -- every byte of the block is
// read by exactly one lane.  From the three words come the four
// groups' 6-bit codes as bytes, then f16x2 (1024 + code) with PRMT, and group q feeds ONE MMA
// whose 16 k slots are exactly sub-block 8h + 2q + u, live column 2q + u.

// The tiles travel through a per-warp ring of shared memory like the Q4_K ones.  A 16-byte
// asynchronous copy keeps the byte offset inside its 16-byte granule, and a 210-byte block starts
// anywhere on a 2-byte grid: each row's block is copied as the 14 granules that cover it (224 B,
// to a 240-byte pitch that spreads the rows over the banks), and the block begins `skew` = (its
// byte offset & 15) bytes into the row's slot.  With an even number of blocks per row the skew is
// the same for rows g and g+8, and it is a multiple of 4 for even blocks and 2 mod 4 for odd
// ones, where a word is two aligned words funnel-shifted by 16 bits.
constexpr int Q6K_PITCH = 240;
constexpr int Q6K_TILE_BYTES = ROWS * Q6K_PITCH;
constexpr int Q6K_STAGES = 2;

__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];\n" : "=h"(v) : "r"(addr));
  return v;
}
// word at a 2-byte aligned shared address: odd == false -> 4-byte aligned
template <bool ODD>
__device__ __forceinline__ uint32_t lds32_skew(uint32_t addr) {
  if constexpr (!ODD) return lds32(addr);
  return __funnelshift_r(lds32(addr - 2), lds32(addr + 2), 16);
}

template <int S, bool TP>
__global__ void __launch_bounds__(WARPS * 32, 2) q6k_gemv_mma_kernel(const float *__restrict__ x,
                                                                    const uint8_t *__restrict__ w,
                                                                    float *__restrict__ out, const __grid_constant__ TpArgs tp,
                                                                    int N, int K) {
  using SL = Slab<16>;
  extern __shared__ __align__(16) unsigned char dyn[];  // ring: WARPS x S tiles
  __shared__ __align__(16) unsigned char slabs[WARPS][SL::BYTES];
  __shared__ __align__(16) unsigned char zero[SL::ZERO_BYTES];
  __shared__ __align__(16) float2 red[2][WARPS * GROUP * 32];  // by group parity
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int nb = K >> 8;
  const uint32_t row_bytes = (uint32_t)nb * 210u;  // a multiple of 4 (nb is even: checked by the launcher)
  const uint8_t *w_end = w + (size_t)N * row_bytes;
  for (int i = threadIdx.x; i < SL::ZERO_BYTES / 4; i += WARPS * 32) reinterpret_cast<uint32_t *>(zero)[i] = 0u;

  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(dyn) + warp * (S * Q6K_TILE_BYTES);
  const uint32_t slab = (uint32_t)__cvta_generic_to_shared(slabs[warp]);
  const uint32_t szero = (uint32_t)__cvta_generic_to_shared(zero);
  const uint32_t red_lane = (uint32_t)__cvta_generic_to_shared(&red[0][warp * GROUP * 32 + lane]);
  constexpr uint32_t RED_PARITY = WARPS * GROUP * 32 * 8;
  // B address of the MMA of (group q, u), which works on sub-block 8h + 2q + u: column 2q + u
  // carries the hi half of x, the neighbouring column 2q + 1 - u (unused in this accumulator) the
  // lo half; a lane of those columns reads elements 4t..4t+3 (h adds an immediate).  All other
  // columns read zeros.
  uint32_t pb[4][2];
#pragma unroll
  for (int q = 0; q < 4; q++)
#pragma unroll
    for (int u = 0; u < 2; u++)
      pb[q][u] = (g >> 1) == q ? slab + (2 * q + u) * SL::SUB_BYTES + 8 * t + ((g & 1) == u ? 0 : SL::LO_OFF) : szero;
  const uint32_t m0f = 0x0F0F0F0Fu;

  const int tiles = (N + ROWS - 1) / ROWS;
  const int t0 = (int)((uint32_t)tiles * blockIdx.x / gridDim.x), t1 = (int)((uint32_t)tiles * (blockIdx.x + 1) / gridDim.x);

  // requests: lanes 0..13 / 16..29 copy the 14 granules of rows 2i / 2i+1, i = 0..7
  const uint32_t c_rsub = lane >> 4, c_piece = lane & 15;
  int i_gt = t0, i_gs = min(GROUP, t1 - t0), i_b = warp, i_rt = 0, i_slot = 0;
  auto issue = [&]() {  // always closes a commit group, so that group counts stay uniform
    if (i_gt < t1 && warp < nb) {
      const int r0 = min((i_gt + i_rt) * ROWS, N - ROWS);
      uint32_t ro = (uint32_t)r0 * row_bytes + (uint32_t)i_b * 210u + c_rsub * row_bytes;
      uint32_t dst = ring + i_slot * Q6K_TILE_BYTES + c_rsub * Q6K_PITCH + c_piece * 16;
      if (c_piece < 14) {
        if (r0 + ROWS < N) {
#pragma unroll
          for (int i = 0; i < 8; i++) {
            cp_async16(dst, w + ((ro & ~15u) + c_piece * 16));
            ro += 2 * row_bytes, dst += 2 * Q6K_PITCH;
          }
        } else {  // the last rows of the matrix: never read past its end
#pragma unroll
          for (int i = 0; i < 8; i++) {
            const uint8_t *src = w + ((ro & ~15u) + c_piece * 16);
            const long long left = w_end - src;
            if (left >= 16)
              cp_async16(dst, src);
            else if (left > 0)
              cp_async16_part(dst, src, (uint32_t)left);
            ro += 2 * row_bytes, dst += 2 * Q6K_PITCH;
          }
        }
      }
      i_slot = (i_slot + 1) & (S - 1);
      if (++i_rt == i_gs) {
        i_rt = 0, i_b += WARPS;
        if (i_b >= nb) i_b = warp, i_gt += i_gs, i_gs = min(GROUP, t1 - i_gt);
      }
    }
    cp_async_commit();
  };
#pragma unroll 1
  for (int p = 0; p < S; p++) issue();

  pdl_wait();  // x is the previous launch's output; the weights requested above are not
  __syncthreads();
  float4 xn[2];  // the activations of the block this warp stages next, requested one block ahead
  unsigned int tag = 0;
  unsigned long long tp_t0 = 0;
  bool tp_gave_up = false;
  if constexpr (TP) {
    tag = *reinterpret_cast<const volatile unsigned int *>(tp.step);
    if (tp.x_slots) asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(tp_t0));
  }
  auto load_x = [&](int b) {
    if (TP && tp.x_slots) {  // the peers' parts of x arrive as tagged slots
      const uint2 *xs = tp.x_slots + (size_t)(tag & 1u) * K + b * 256 + lane * 4;
      xn[0] = ld_slots4(xs, tag, tp_t0, tp_gave_up);
      xn[1] = ld_slots4(xs + 128, tag, tp_t0, tp_gave_up);
    } else {
      xn[0] = __ldg(reinterpret_cast<const float4 *>(x + b * 256) + lane);
      xn[1] = __ldg(reinterpret_cast<const float4 *>(x + b * 256 + 128) + lane);
    }
  };
  if (warp < nb) load_x(warp);

  // one unit: rows g, g+8 of one tile x one K block, out of ring slot `sb`
  auto unit = [&](auto odd_tag, uint32_t sb, uint32_t skew, const float2 (&sx)[2], float up, float (&vr)[2]) {
    constexpr bool ODD = decltype(odd_tag)::value;
    uint32_t wa[2][4], wc[2][4], wh[2][4], scw[2];
    float dd[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
      const uint32_t blk = sb + (g + 8 * r) * Q6K_PITCH + skew;  // the block's first byte
#pragma unroll
      for (int hu = 0; hu < 4; hu++) {
        const int h = hu >> 1, u = hu & 1;
        wa[r][hu] = lds32_skew<ODD>(blk + 4 * (16 * h + 4 * u + t));
        wc[r][hu] = lds32_skew<ODD>(blk + 4 * (16 * h + 8 + 4 * u + t));
        wh[r][hu] = lds32_skew<ODD>(blk + 4 * (32 + 8 * h + 4 * u + t));
      }
      scw[r] = lds16(blk + 192 + 2 * t) | (lds16(blk + 200 + 2 * t) << 16);  // scales 2t, 2t+1 | 8+2t, 8+2t+1
      dd[r] = f16_bits_to_f32((uint16_t)lds16(blk + 208));
    }
    __syncwarp();  // the slot is free again
    issue();
    vr[0] = vr[1] = 0.f;
#pragma unroll
    for (int h = 0; h < 2; h++) {
      float d0[4] = {0.f, 0.f, 0.f, 0.f}, d1[4] = {0.f, 0.f, 0.f, 0.f};  // u = 0 / u = 1 chains
#pragma unroll
      for (int u = 0; u < 2; u++) {
        const int hu = 2 * h + u;
#pragma unroll
        for (int q = 0; q < 4; q++) {
          uint32_t a[4];
#pragma unroll
          for (int r = 0; r < 2; r++) {
            const uint32_t lo4 = (q & 1) ? wc[r][hu] : wa[r][hu];
            const uint32_t nib = (q >> 1) ? (lo4 >> 4) : lo4;
            const uint32_t hi2 = q == 0 ? (wh[r][hu] << 4) : q == 1 ? (wh[r][hu] << 2) : q == 2 ? wh[r][hu] : (wh[r][hu] >> 2);
            const uint32_t v = and_or(nib, m0f, hi2 & 0x30303030u);
            a[r] = __byte_perm(v, 0x64646464u, 0x4240);      // f16x2 (1024 + b0, 1024 + b2)
            a[2 + r] = __byte_perm(v, 0x64646464u, 0x4341);  // f16x2 (1024 + b1, 1024 + b3)
          }
          const uint2 bh = lds64(pb[q][u] + h * (8 * SL::SUB_BYTES));
          if (u == 0)
            mma16816(d0, a[0], a[1], a[2], a[3], bh.x, bh.y);
          else
            mma16816(d1, a[0], a[1], a[2], a[3], bh.x, bh.y);
        }
      }
      // lane (g, t): d0[0] + d0[1] = row g, sub-block 8h+2t; d1[0] + d1[1] = row g, sub-block 8h+2t+1;
      // [2], [3] the same for row g+8
#pragma unroll
      for (int r = 0; r < 2; r++) {
        const float s0 = dd[r] * (float)(int8_t)((scw[r] >> (16 * h)) & 0xff);
        const float s1 = dd[r] * (float)(int8_t)((scw[r] >> (16 * h + 8)) & 0xff);
        vr[r] += s0 * (d0[2 * r] + d0[2 * r + 1] - 1056.f * sx[h].x) + s1 * (d1[2 * r] + d1[2 * r + 1] - 1056.f * sx[h].y);
      }
    }
    vr[0] *= up, vr[1] *= up;
  };

  int slot = 0, parity = 0;
  for (int gt = t0; gt < t1; gt += GROUP, parity ^= 1) {
    const int gs = min(GROUP, t1 - gt);
    const uint32_t red_g = red_lane + parity * RED_PARITY;
    for (int b = warp; b < nb; b += WARPS) {
      // this block's activations into the warp's slab; the next block's are requested meanwhile
      const float4 xv[2] = {xn[0], xn[1]};
      {
        const int bn = b + WARPS < nb ? b + WARPS : warp;
        if (b + WARPS < nb || gt + GROUP < t1) load_x(bn);
      }
      __syncwarp();  // every lane is done reading the previous block's slab
      const float up = stage_block<16>(xv, slab, lane);
      __syncwarp();
      float2 sx[2];
      asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];\n" : "=f"(sx[0].x), "=f"(sx[0].y) : "r"(slab + SL::SX_OFF + 8 * t));
      asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];\n" : "=f"(sx[1].x), "=f"(sx[1].y) : "r"(slab + SL::SX_OFF + 32 + 8 * t));
      for (int rt = 0; rt < gs; rt++) {
        cp_async_wait<S - 1>();  // this lane's granules of the tile have landed ...
        __syncwarp();            // ... and so have the other lanes'
        const uint32_t sb = ring + slot * Q6K_TILE_BYTES;
        slot = (slot + 1) & (S - 1);
        const int r0 = min((gt + rt) * ROWS, N - ROWS);
        const uint32_t skew = ((uint32_t)r0 * row_bytes + (uint32_t)b * 210u + (uint32_t)g * row_bytes) & 15u;
        float vr[2];
        if (b & 1)
          unit(std::true_type{}, sb, skew, sx, up, vr);
        else
          unit(std::false_type{}, sb, skew, sx, up, vr);
        // the warp's first block of a group overwrites what an earlier group left behind
        const uint32_t ra = red_g + rt * (32 * 8);
        float2 o = make_float2(0.f, 0.f);
        if (b != warp) asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];\n" : "=f"(o.x), "=f"(o.y) : "r"(ra));
        asm volatile("st.shared.v2.f32 [%0], {%1,%2};\n" ::"r"(ra), "f"(o.x + vr[0]), "f"(o.y + vr[1]));
      }
    }
    __syncthreads();  // also orders this group's reads of red[parity] before its reuse two groups on
    for (int i = threadIdx.x; i < gs * ROWS; i += WARPS * 32) {
      const int rt = i >> 4, row = i & 15, gg = row & 7, hi = row >> 3;
      float v = 0.f;
#pragma unroll
      for (int wq = 0; wq < WARPS; wq++) {
        if (wq >= nb) break;  // a warp without a K block never wrote its part
        const float2 *p = &red[parity][(wq * GROUP + rt) * 32 + gg * 4];
#pragma unroll
        for (int tt = 0; tt < 4; tt++) v += hi ? p[tt].y : p[tt].x;
      }
      const int orow = min((gt + rt) * ROWS, N - ROWS) + row;
      out[orow] = v;
      if (TP && tp.peer[0][0]) st_slots(tp.peer[0], tp.world, (size_t)(tag & 1u) * N * tp.world + (size_t)tp.rank * N + orow, v, tag);
    }
  }
  cp_async_wait<0>();
}

// ------------------------------------------------------------------------------------ Q8_0
//
// The Q6_K kernel's structure (per-warp ring of 16-row tiles, activations staged per run of 256 k with the
// next run requested ahead, one MMA per 16-element sub-block with the hi and lo halves of x in
// neighbouring columns) on 34-byte blocks: a run of 256 k is eight blocks = 272 bytes = 17 granules per
// row, rows are whole granules (K % 256 == 0), and a 272-byte pitch puts rows g and lanes t on 32
// different banks.  reference: matmul_q8_0_f32_mv, kernels/cuda/src/matmul_q.cu:58-431.
constexpr int Q80_PITCH = 272;
constexpr int Q80_TILE_BYTES = ROWS * Q80_PITCH;
constexpr int Q80_STAGES = 2;

template <int S>
__global__ void __launch_bounds__(WARPS * 32, 2) q80_gemv_mma_kernel(const float *__restrict__ x, const uint8_t *__restrict__ w,
                                                                    float *__restrict__ out, int N, int K) {
  using SL = Slab<16>;
  extern __shared__ __align__(16) unsigned char dyn[];  // ring: WARPS x S tiles
  __shared__ __align__(16) unsigned char slabs[WARPS][SL::BYTES];
  __shared__ __align__(16) unsigned char zero[SL::ZERO_BYTES];
  __shared__ __align__(16) float2 red[2][WARPS * GROUP * 32];  // by group parity
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int nb = K >> 8;
  const uint32_t row_bytes = (uint32_t)nb * 272u;  // eight 34-byte blocks per 256 elements: rows are whole granules
  for (int i = threadIdx.x; i < SL::ZERO_BYTES / 4; i += WARPS * 32) reinterpret_cast<uint32_t *>(zero)[i] = 0u;

  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(dyn) + warp * (S * Q80_TILE_BYTES);
  const uint32_t slab = (uint32_t)__cvta_generic_to_shared(slabs[warp]);
  const uint32_t szero = (uint32_t)__cvta_generic_to_shared(zero);
  const uint32_t red_lane = (uint32_t)__cvta_generic_to_shared(&red[0][warp * GROUP * 32 + lane]);
  constexpr uint32_t RED_PARITY = WARPS * GROUP * 32 * 8;
  // B address of the MMA of (group q, u), which works on sub-block 8h + 2q + u: column 2q + u
  // carries the hi half of x, the neighbouring column 2q + 1 - u (unused in this accumulator) the
  // lo half; a lane of those columns reads elements 4t..4t+3 (h adds an immediate).  All other
  // columns read zeros.
  uint32_t pb[4][2];
#pragma unroll
  for (int q = 0; q < 4; q++)
#pragma unroll
    for (int u = 0; u < 2; u++)
      pb[q][u] = (g >> 1) == q ? slab + (2 * q + u) * SL::SUB_BYTES + 8 * t + ((g & 1) == u ? 0 : SL::LO_OFF) : szero;

  const int tiles = (N + ROWS - 1) / ROWS;
  const int t0 = (int)((uint32_t)tiles * blockIdx.x / gridDim.x), t1 = (int)((uint32_t)tiles * (blockIdx.x + 1) / gridDim.x);

  // requests: lanes 0..15 / 16..31 copy granules 0..15 of rows 2i / 2i+1, i = 0..7; lanes 0 / 16 also the 17th
  const uint32_t c_rsub = lane >> 4, c_piece = lane & 15;
  int i_gt = t0, i_gs = min(GROUP, t1 - t0), i_b = warp, i_rt = 0, i_slot = 0;
  auto issue = [&]() {  // always closes a commit group, so that group counts stay uniform
    if (i_gt < t1 && warp < nb) {
      const int r0 = min((i_gt + i_rt) * ROWS, N - ROWS);
      const uint8_t *src = w + ((size_t)(r0 + c_rsub) * row_bytes + (uint32_t)i_b * 272u + c_piece * 16);
      uint32_t dst = ring + i_slot * Q80_TILE_BYTES + c_rsub * Q80_PITCH + c_piece * 16;
#pragma unroll
      for (int i = 0; i < 8; i++) {
        cp_async16(dst, src);
        if (c_piece == 0) cp_async16(dst + 256, src + 256);
        src += 2 * row_bytes, dst += 2 * Q80_PITCH;
      }
      i_slot = (i_slot + 1) & (S - 1);
      if (++i_rt == i_gs) {
        i_rt = 0, i_b += WARPS;
        if (i_b >= nb) i_b = warp, i_gt += i_gs, i_gs = min(GROUP, t1 - i_gt);
      }
    }
    cp_async_commit();
  };
#pragma unroll 1
  for (int p = 0; p < S; p++) issue();

  pdl_wait();  // x is the previous launch's output; the weights requested above are not
  __syncthreads();
  float4 xn[2];  // the activations of the block this warp stages next, requested one block ahead
  auto load_x = [&](int b) {
    xn[0] = __ldg(reinterpret_cast<const float4 *>(x + b * 256) + lane);
    xn[1] = __ldg(reinterpret_cast<const float4 *>(x + b * 256 + 128) + lane);
  };
  if (warp < nb) load_x(warp);

  // One unit: rows g, g+8 of one tile x one run of 256 k (eight 34-byte blocks), out of ring slot `sb`.
  // Sub-block s = 8h + 2q + u (16 codes) is half s & 1 of block s >> 1; lane t takes its word t.  Even
  // blocks start 2 bytes into a word (34 j + 2), odd ones on a word boundary.  XOR 0x80 makes the codes
  // unsigned and PRMT gives f16 (1024 + 128 + q): the MMA sums (1152 + q) x, and 1152 sum(x) comes off.
  auto unit = [&](uint32_t sb, const float2 (&sx)[2], float up, float (&vr)[2]) {
    uint32_t wq[2][16];
    float dd[2][2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
      const uint32_t blk = sb + (g + 8 * r) * Q80_PITCH;
#pragma unroll
      for (int s = 0; s < 16; s++) {
        const uint32_t a = blk + 34 * (s >> 1) + 2 + 16 * (s & 1) + 4 * t;
        wq[r][s] = (((s >> 1) & 1) ? lds32(a) : __funnelshift_r(lds32(a - 2), lds32(a + 2), 16)) ^ 0x80808080u;
      }
      dd[r][0] = f16_bits_to_f32((uint16_t)lds16(blk + 34 * t)), dd[r][1] = f16_bits_to_f32((uint16_t)lds16(blk + 34 * (4 + t)));
    }
    __syncwarp();  // the slot is free again
    issue();
    vr[0] = vr[1] = 0.f;
#pragma unroll
    for (int h = 0; h < 2; h++) {
      float d0[4] = {0.f, 0.f, 0.f, 0.f}, d1[4] = {0.f, 0.f, 0.f, 0.f};  // u = 0 / u = 1 chains
#pragma unroll
      for (int u = 0; u < 2; u++) {
#pragma unroll
        for (int q = 0; q < 4; q++) {
          const int s = 8 * h + 2 * q + u;
          uint32_t a[4];
#pragma unroll
          for (int r = 0; r < 2; r++) {
            a[r] = __byte_perm(wq[r][s], 0x64646464u, 0x4240);      // f16x2 (1024 + b0, 1024 + b2)
            a[2 + r] = __byte_perm(wq[r][s], 0x64646464u, 0x4341);  // f16x2 (1024 + b1, 1024 + b3)
          }
          const uint2 bh = lds64(pb[q][u] + h * (8 * SL::SUB_BYTES));
          if (u == 0)
            mma16816(d0, a[0], a[1], a[2], a[3], bh.x, bh.y);
          else
            mma16816(d1, a[0], a[1], a[2], a[3], bh.x, bh.y);
        }
      }
      // lane (g, t): d0[0] + d0[1] = row g, sub-block 8h+2t; d1[0] + d1[1] = row g, sub-block 8h+2t+1: the
      // two halves of block 4h + t; [2], [3] the same for row g+8
#pragma unroll
      for (int r = 0; r < 2; r++)
        vr[r] += dd[r][h] * ((d0[2 * r] + d0[2 * r + 1]) + (d1[2 * r] + d1[2 * r + 1]) - 1152.f * (sx[h].x + sx[h].y));
    }
    vr[0] *= up, vr[1] *= up;
  };

  int slot = 0, parity = 0;
  for (int gt = t0; gt < t1; gt += GROUP, parity ^= 1) {
    const int gs = min(GROUP, t1 - gt);
    const uint32_t red_g = red_lane + parity * RED_PARITY;
    for (int b = warp; b < nb; b += WARPS) {
      // this block's activations into the warp's slab; the next block's are requested meanwhile
      const float4 xv[2] = {xn[0], xn[1]};
      {
        const int bn = b + WARPS < nb ? b + WARPS : warp;
        if (b + WARPS < nb || gt + GROUP < t1) load_x(bn);
      }
      __syncwarp();  // every lane is done reading the previous block's slab
      const float up = stage_block<16>(xv, slab, lane);
      __syncwarp();
      float2 sx[2];
      asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];\n" : "=f"(sx[0].x), "=f"(sx[0].y) : "r"(slab + SL::SX_OFF + 8 * t));
      asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];\n" : "=f"(sx[1].x), "=f"(sx[1].y) : "r"(slab + SL::SX_OFF + 32 + 8 * t));
      for (int rt = 0; rt < gs; rt++) {
        cp_async_wait<S - 1>();  // this lane's granules of the tile have landed ...
        __syncwarp();            // ... and so have the other lanes'
        const uint32_t sb = ring + slot * Q80_TILE_BYTES;
        slot = (slot + 1) & (S - 1);
        float vr[2];
        unit(sb, sx, up, vr);
        // the warp's first block of a group overwrites what an earlier group left behind
        const uint32_t ra = red_g + rt * (32 * 8);
        float2 o = make_float2(0.f, 0.f);
        if (b != warp) asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];\n" : "=f"(o.x), "=f"(o.y) : "r"(ra));
        asm volatile("st.shared.v2.f32 [%0], {%1,%2};\n" ::"r"(ra), "f"(o.x + vr[0]), "f"(o.y + vr[1]));
      }
    }
    __syncthreads();  // also orders this group's reads of red[parity] before its reuse two groups on
    for (int i = threadIdx.x; i < gs * ROWS; i += WARPS * 32) {
      const int rt = i >> 4, row = i & 15, gg = row & 7, hi = row >> 3;
      float v = 0.f;
#pragma unroll
      for (int wq = 0; wq < WARPS; wq++) {
        if (wq >= nb) break;  // a warp without a K block never wrote its part
        const float2 *p = &red[parity][(wq * GROUP + rt) * 32 + gg * 4];
#pragma unroll
        for (int tt = 0; tt < 4; tt++) v += hi ? p[tt].y : p[tt].x;
      }
      const int orow = min((gt + rt) * ROWS, N - ROWS) + row;
      out[orow] = v;
    }
  }
  cp_async_wait<0>();
}

// ------------------------------------------------------------------------------------ block-scaled FP8 (e4m3), one row of x
//
// The Q8_0 kernel's structure on one-byte codes: a run of 256 k is 256 bytes = 16 granules per row, a
// 272-byte pitch keeps the 32 lanes on 32 banks.  The codes need no offset and no table: two shifts and a
// LOP3 turn a pair of e4m3 bytes into their exact f16 values / 256.  One f32 scale per 128 x 128 block, applied
// once per run and lane.  Needs K % 256 == 0, bC % 32 == 0, bR % 16 == 0.  reference: fp8_block_gemv_f32 /
// _bf16, kernels/cuda/src/fp8_block.cu:60-130.
constexpr int F8_PITCH = 272;
constexpr int F8_TILE_BYTES = ROWS * F8_PITCH;
constexpr int F8_STAGES = 2;

template <int S, typename XT>
__global__ void __launch_bounds__(WARPS * 32, 2) fp8_gemv_mma_kernel(const XT *__restrict__ x, const uint8_t *__restrict__ w,
                                                                    const float *__restrict__ scale, XT *__restrict__ out, int N, int K,
                                                                    int bR, int bC) {
  using SL = Slab<16>;
  extern __shared__ __align__(16) unsigned char dyn[];  // ring: WARPS x S tiles
  __shared__ __align__(16) unsigned char slabs[WARPS][SL::BYTES];
  __shared__ __align__(16) unsigned char zero[SL::ZERO_BYTES];
  __shared__ __align__(16) float2 red[2][WARPS * GROUP * 32];  // by group parity
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int nb = K >> 8;
  const uint32_t row_bytes = (uint32_t)K;  // one byte per weight
  const int scols = K / bC;
  for (int i = threadIdx.x; i < SL::ZERO_BYTES / 4; i += WARPS * 32) reinterpret_cast<uint32_t *>(zero)[i] = 0u;

  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(dyn) + warp * (S * F8_TILE_BYTES);
  const uint32_t slab = (uint32_t)__cvta_generic_to_shared(slabs[warp]);
  const uint32_t szero = (uint32_t)__cvta_generic_to_shared(zero);
  const uint32_t red_lane = (uint32_t)__cvta_generic_to_shared(&red[0][warp * GROUP * 32 + lane]);
  constexpr uint32_t RED_PARITY = WARPS * GROUP * 32 * 8;
  // B address of the MMA of (group q, u), which works on sub-block 8h + 2q + u: column 2q + u
  // carries the hi half of x, the neighbouring column 2q + 1 - u (unused in this accumulator) the
  // lo half; a lane of those columns reads elements 4t..4t+3 (h adds an immediate).  All other
  // columns read zeros.
  uint32_t pb[4][2];
#pragma unroll
  for (int q = 0; q < 4; q++)
#pragma unroll
    for (int u = 0; u < 2; u++)
      pb[q][u] = (g >> 1) == q ? slab + (2 * q + u) * SL::SUB_BYTES + 8 * t + ((g & 1) == u ? 0 : SL::LO_OFF) : szero;

  const int tiles = (N + ROWS - 1) / ROWS;
  const int t0 = (int)((uint32_t)tiles * blockIdx.x / gridDim.x), t1 = (int)((uint32_t)tiles * (blockIdx.x + 1) / gridDim.x);

  // requests: lanes 0..15 / 16..31 copy the 16 granules of rows 2i / 2i+1, i = 0..7
  const uint32_t c_rsub = lane >> 4, c_piece = lane & 15;
  int i_gt = t0, i_gs = min(GROUP, t1 - t0), i_b = warp, i_rt = 0, i_slot = 0;
  auto issue = [&]() {  // always closes a commit group, so that group counts stay uniform
    if (i_gt < t1 && warp < nb) {
      const int r0 = min((i_gt + i_rt) * ROWS, N - ROWS);
      const uint8_t *src = w + ((size_t)(r0 + c_rsub) * row_bytes + (uint32_t)i_b * 256u + c_piece * 16);
      uint32_t dst = ring + i_slot * F8_TILE_BYTES + c_rsub * F8_PITCH + c_piece * 16;
#pragma unroll
      for (int i = 0; i < 8; i++) {
        cp_async16(dst, src);
        src += 2 * row_bytes, dst += 2 * F8_PITCH;
      }
      i_slot = (i_slot + 1) & (S - 1);
      if (++i_rt == i_gs) {
        i_rt = 0, i_b += WARPS;
        if (i_b >= nb) i_b = warp, i_gt += i_gs, i_gs = min(GROUP, t1 - i_gt);
      }
    }
    cp_async_commit();
  };
#pragma unroll 1
  for (int p = 0; p < S; p++) issue();

  pdl_wait();  // x is the previous launch's output; the weights requested above are not
  __syncthreads();
  float4 xn[2];  // the activations of the block this warp stages next, requested one block ahead
  auto load_x = [&](int b) {
    if constexpr (std::is_same<XT, float>::value) {
      xn[0] = __ldg(reinterpret_cast<const float4 *>(x + b * 256) + lane);
      xn[1] = __ldg(reinterpret_cast<const float4 *>(x + b * 256 + 128) + lane);
    } else {
#pragma unroll
      for (int i = 0; i < 2; i++) {
        const uint2 v = __ldg(reinterpret_cast<const uint2 *>(x + b * 256 + 128 * i) + lane);
        xn[i] = make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xFFFF0000u), __uint_as_float(v.y << 16), __uint_as_float(v.y & 0xFFFF0000u));
      }
    }
  };
  if (warp < nb) load_x(warp);

  // One unit: rows g, g+8 of one tile x one run of 256 k, out of ring slot `sb`.  Sub-block s = 8h + 2q + u is
  // bytes 16 s .. 16 s + 15 of the row's 256; lane t takes its word t.  An e4m3 code c becomes the f16 with the
  // bits sign(c) << 15 | (c & 0x7F) << 7, which is the code's value / 256 for normal and subnormal codes alike
  // (exact); the 256 goes into the block scale.
  auto unit = [&](uint32_t sb, int r0, int b, float up, float (&vr)[2]) {
    uint32_t wq[2][16];
#pragma unroll
    for (int r = 0; r < 2; r++) {
      const uint32_t blk = sb + (g + 8 * r) * F8_PITCH + 4 * t;
#pragma unroll
      for (int s = 0; s < 16; s++) wq[r][s] = lds32(blk + 16 * s);
    }
    __syncwarp();  // the slot is free again
    issue();
    // both rows of the tile lie in one row block (the launcher checks bR % 16 == 0)
    const float *srow = scale + (size_t)(r0 / bR) * scols;
    vr[0] = vr[1] = 0.f;
#pragma unroll
    for (int h = 0; h < 2; h++) {
      float d0[4] = {0.f, 0.f, 0.f, 0.f}, d1[4] = {0.f, 0.f, 0.f, 0.f};  // u = 0 / u = 1 chains
#pragma unroll
      for (int u = 0; u < 2; u++) {
#pragma unroll
        for (int q = 0; q < 4; q++) {
          const int s = 8 * h + 2 * q + u;
          uint32_t a[4];
#pragma unroll
          for (int r = 0; r < 2; r++) {
            const uint32_t p02 = __byte_perm(wq[r][s], 0u, 0x2404), p13 = __byte_perm(wq[r][s], 0u, 0x3414);  // codes in the high bytes
            a[r] = and_or(p02, 0x80008000u, (p02 >> 1) & 0x3F803F80u);
            a[2 + r] = and_or(p13, 0x80008000u, (p13 >> 1) & 0x3F803F80u);
          }
          const uint2 bh = lds64(pb[q][u] + h * (8 * SL::SUB_BYTES));
          if (u == 0)
            mma16816(d0, a[0], a[1], a[2], a[3], bh.x, bh.y);
          else
            mma16816(d1, a[0], a[1], a[2], a[3], bh.x, bh.y);
        }
      }
      // lane (g, t): d0[0] + d0[1] = row g, sub-block 8h+2t; d1[0] + d1[1] = row g, sub-block 8h+2t+1; [2], [3]
      // the same for row g+8.  Both sub-blocks lie in elements 256 b + 128 h + 32 t .. + 31: one column block
      const float sc = __ldg(srow + (b * 256 + 128 * h + 32 * t) / bC) * 256.f;
#pragma unroll
      for (int r = 0; r < 2; r++) vr[r] += sc * ((d0[2 * r] + d0[2 * r + 1]) + (d1[2 * r] + d1[2 * r + 1]));
    }
    vr[0] *= up, vr[1] *= up;
  };

  int slot = 0, parity = 0;
  for (int gt = t0; gt < t1; gt += GROUP, parity ^= 1) {
    const int gs = min(GROUP, t1 - gt);
    const uint32_t red_g = red_lane + parity * RED_PARITY;
    for (int b = warp; b < nb; b += WARPS) {
      // this block's activations into the warp's slab; the next block's are requested meanwhile
      const float4 xv[2] = {xn[0], xn[1]};
      {
        const int bn = b + WARPS < nb ? b + WARPS : warp;
        if (b + WARPS < nb || gt + GROUP < t1) load_x(bn);
      }
      __syncwarp();  // every lane is done reading the previous block's slab
      const float up = stage_block<16>(xv, slab, lane);
      __syncwarp();
      for (int rt = 0; rt < gs; rt++) {
        cp_async_wait<S - 1>();  // this lane's granules of the tile have landed ...
        __syncwarp();            // ... and so have the other lanes'
        const uint32_t sb = ring + slot * F8_TILE_BYTES;
        slot = (slot + 1) & (S - 1);
        float vr[2];
        unit(sb, min((gt + rt) * ROWS, N - ROWS), b, up, vr);
        // the warp's first block of a group overwrites what an earlier group left behind
        const uint32_t ra = red_g + rt * (32 * 8);
        float2 o = make_float2(0.f, 0.f);
        if (b != warp) asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];\n" : "=f"(o.x), "=f"(o.y) : "r"(ra));
        asm volatile("st.shared.v2.f32 [%0], {%1,%2};\n" ::"r"(ra), "f"(o.x + vr[0]), "f"(o.y + vr[1]));
      }
    }
    __syncthreads();  // also orders this group's reads of red[parity] before its reuse two groups on
    for (int i = threadIdx.x; i < gs * ROWS; i += WARPS * 32) {
      const int rt = i >> 4, row = i & 15, gg = row & 7, hi = row >> 3;
      float v = 0.f;
#pragma unroll
      for (int wq = 0; wq < WARPS; wq++) {
        if (wq >= nb) break;  // a warp without a K block never wrote its part
        const float2 *p = &red[parity][(wq * GROUP + rt) * 32 + gg * 4];
#pragma unroll
        for (int tt = 0; tt < 4; tt++) v += hi ? p[tt].y : p[tt].x;
      }
      const int orow = min((gt + rt) * ROWS, N - ROWS) + row;
      st_act(out, orow, v);
    }
  }
  cp_async_wait<0>();
}

// ------------------------------------------------------------------------------------ int4 (GPTQ / AWQ), one row of x
//
// The canonical 4-bit layout (codes u32 (N, K/8), nibble j of word c = element 8c + j; scales / zeros f32
// (N, K/G)) through the Q4_K arithmetic: LOP3 turns nibble pairs into f16 (64 + code), the MMA columns are
// sets of 32 elements that share a scale (here the even- and the odd-numbered elements of a lane's 64), and
// acc += s (D - (64 + z) Sx).  Structure as the Q8_0 kernel (per-warp ring, activations staged per run of
// 256 k, so any K fits); a tile row sits 16 bytes into a 144-byte slot, which keeps the Q4_K kernel's
// conflict-free 16-byte loads.  Needs G % 64 == 0 and K % 256 == 0.  reference: int4_gemv_f32 / _bf16,
// kernels/cuda/src/int4.cu:43-106.
constexpr int I4_PITCH = 144;
constexpr int I4_TILE_BYTES = ROWS * I4_PITCH;
constexpr int I4_STAGES = 4;

// stage_block<32> for the int4 element order: lanes l, l^1 hold the eight elements of one code word; the even
// lane assembles (x0, x4, x2, x6) for the even set, the odd lane (x1, x5, x3, x7) for the odd set.
__device__ __forceinline__ float stage_block_int4(const float4 (&xv)[2], uint32_t slab, int lane) {
  using S = Slab<32>;
  uint32_t m = 0;
#pragma unroll
  for (int i = 0; i < 2; i++) {
    m = max(m, __float_as_uint(xv[i].x) & 0x7fffffffu);
    m = max(m, __float_as_uint(xv[i].y) & 0x7fffffffu);
    m = max(m, __float_as_uint(xv[i].z) & 0x7fffffffu);
    m = max(m, __float_as_uint(xv[i].w) & 0x7fffffffu);
  }
  m = __reduce_max_sync(0xffffffffu, m);
  int sh = (int)(m >> 23) - 127 - 14;
  sh = sh < 0 ? 0 : (sh > 100 ? 100 : sh);
  const float down = __uint_as_float((uint32_t)(127 - sh) << 23), up = __uint_as_float((uint32_t)(127 + sh) << 23);
  const bool odd = lane & 1;
#pragma unroll
  for (int i = 0; i < 2; i++) {
    float4 v = xv[i];
    if (sh) v.x *= down, v.y *= down, v.z *= down, v.w *= down;
    // the even lane needs the partner's x and z, the odd lane the partner's y and w
    const float ra = __shfl_xor_sync(0xffffffffu, odd ? v.x : v.y, 1), rb = __shfl_xor_sync(0xffffffffu, odd ? v.z : v.w, 1);
    const float s0 = odd ? ra : v.x, s1 = odd ? v.y : ra, s2 = odd ? rb : v.z, s3 = odd ? v.w : rb;  // slots 0..3 of this word
    __half2 h01 = __floats2half2_rn(s0, s1), h23 = __floats2half2_rn(s2, s3);
    float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
    __half2 l01 = __floats2half2_rn(s0 - f01.x, s1 - f01.y), l23 = __floats2half2_rn(s2 - f23.x, s3 - f23.y);
    const int t = 2 * i + (lane >> 4), w = (lane >> 1) & 7, vs = 2 * t + (lane & 1);  // lane quarter, word, set
    const uint32_t a = slab + vs * S::SUB_BYTES + w * 8;
    sts64(a, *reinterpret_cast<uint32_t *>(&h01), *reinterpret_cast<uint32_t *>(&h23));
    sts64(a + S::LO_OFF, *reinterpret_cast<uint32_t *>(&l01), *reinterpret_cast<uint32_t *>(&l23));
    float s = (s0 + s1) + (s2 + s3);
    s += __shfl_xor_sync(0xffffffffu, s, 2), s += __shfl_xor_sync(0xffffffffu, s, 4), s += __shfl_xor_sync(0xffffffffu, s, 8);
    if (w == 0) asm volatile("st.shared.f32 [%0], %1;\n" ::"r"(slab + S::SX_OFF + vs * 4), "f"(s));
  }
  return up;
}

template <int S, typename XT>
__global__ void __launch_bounds__(WARPS * 32, 2) int4_gemv_mma_kernel(const XT *__restrict__ x, const uint8_t *__restrict__ w,
                                                                     const float *__restrict__ scales, const float *__restrict__ zeros,
                                                                     XT *__restrict__ out, int N, int K, int G) {
  using SL = Slab<32>;
  extern __shared__ __align__(16) unsigned char dyn[];  // ring: WARPS x S tiles
  __shared__ __align__(16) unsigned char slabs[WARPS][SL::BYTES];
  __shared__ __align__(16) unsigned char zero[SL::ZERO_BYTES];
  __shared__ __align__(16) float2 red[2][WARPS * GROUP * 32];  // by group parity
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int nb = K >> 8;
  const uint32_t row_bytes = (uint32_t)K >> 1;  // 128 bytes of codes per 256 elements
  const int ngrp = K / G;
  for (int i = threadIdx.x; i < SL::ZERO_BYTES / 4; i += WARPS * 32) reinterpret_cast<uint32_t *>(zero)[i] = 0u;

  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(dyn) + warp * (S * I4_TILE_BYTES);
  const uint32_t slab = (uint32_t)__cvta_generic_to_shared(slabs[warp]);
  const uint32_t szero = (uint32_t)__cvta_generic_to_shared(zero);
  const uint32_t red_lane = (uint32_t)__cvta_generic_to_shared(&red[0][warp * GROUP * 32 + lane]);
  constexpr uint32_t RED_PARITY = WARPS * GROUP * 32 * 8;
  // B addresses inside the slab, as in the Q4_K kernel: the even MMA's column 2t carries the hi half of the
  // even-numbered elements of lane t's 64, column 2t+1 their lo half; the odd MMA the other way round
  const bool mine = (g >> 1) == t;
  const uint32_t pe = mine ? slab + (2 * t) * SL::SUB_BYTES + ((g & 1) ? SL::LO_OFF : 0) : szero;
  const uint32_t po = mine ? slab + (2 * t + 1) * SL::SUB_BYTES + ((g & 1) ? 0 : SL::LO_OFF) : szero;
  const uint32_t mask = 0x00F000F0u, magic = 0x54005400u;  // f16 (64 + nibble)

  const int tiles = (N + ROWS - 1) / ROWS;
  const int t0 = (int)((uint32_t)tiles * blockIdx.x / gridDim.x), t1 = (int)((uint32_t)tiles * (blockIdx.x + 1) / gridDim.x);

  // requests: a tile is 16 rows x 8 granules; lane l copies granule l & 7 of rows (l >> 3) + 4 i, i = 0..3
  const uint32_t c_row = lane >> 3, c_piece = lane & 7;
  int i_gt = t0, i_gs = min(GROUP, t1 - t0), i_b = warp, i_rt = 0, i_slot = 0;
  auto issue = [&]() {  // always closes a commit group, so that group counts stay uniform
    if (i_gt < t1 && warp < nb) {
      const int r0 = min((i_gt + i_rt) * ROWS, N - ROWS);
      const uint8_t *src = w + ((size_t)(r0 + c_row) * row_bytes + (uint32_t)i_b * 128u + c_piece * 16);
      uint32_t dst = ring + i_slot * I4_TILE_BYTES + c_row * I4_PITCH + 16 + c_piece * 16;
#pragma unroll
      for (int i = 0; i < 4; i++) {
        cp_async16(dst, src);
        src += 4 * row_bytes, dst += 4 * I4_PITCH;
      }
      i_slot = (i_slot + 1) & (S - 1);
      if (++i_rt == i_gs) {
        i_rt = 0, i_b += WARPS;
        if (i_b >= nb) i_b = warp, i_gt += i_gs, i_gs = min(GROUP, t1 - i_gt);
      }
    }
    cp_async_commit();
  };
#pragma unroll 1
  for (int p = 0; p < S; p++) issue();

  pdl_wait();  // x is the previous launch's output; the weights requested above are not
  __syncthreads();
  float4 xn[2];  // the activations of the block this warp stages next, requested one block ahead
  auto load_x = [&](int b) {
    if constexpr (std::is_same<XT, float>::value) {
      xn[0] = __ldg(reinterpret_cast<const float4 *>(x + b * 256) + lane);
      xn[1] = __ldg(reinterpret_cast<const float4 *>(x + b * 256 + 128) + lane);
    } else {
#pragma unroll
      for (int i = 0; i < 2; i++) {
        const uint2 v = __ldg(reinterpret_cast<const uint2 *>(x + b * 256 + 128 * i) + lane);
        xn[i] = make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xFFFF0000u), __uint_as_float(v.y << 16), __uint_as_float(v.y & 0xFFFF0000u));
      }
    }
  };
  if (warp < nb) load_x(warp);

  // One unit: rows g, g+8 of one tile x one run of 256 k, out of ring slot `sb`.  Lane t owns words 8t .. 8t+7
  // of both rows (elements 64t .. 64t+63, one quantization group).  Word i gives the even MMA the f16 pairs
  // (64 + n0, 64 + n4), (64 + n2, 64 + n6) and the odd MMA (n1, n5), (n3, n7); the slab holds x in that order.
  // acc += s ((D_even + D_odd) - (64 + z) (Sx_even + Sx_odd)).
  auto unit = [&](uint32_t sb, const float (&sc)[2], const float (&zp)[2], const float2 sx, float up, float (&vr)[2]) {
    const uint32_t la = sb + g * I4_PITCH + 32u * t;
    const uint4 qa0 = lds128(la + 16), qa1 = lds128(la + 32);
    const uint4 qb0 = lds128(la + 8 * I4_PITCH + 16), qb1 = lds128(la + 8 * I4_PITCH + 32);
    __syncwarp();  // the slot is free again
    issue();
    float de[4] = {0.f, 0.f, 0.f, 0.f}, dq[4] = {0.f, 0.f, 0.f, 0.f};  // even / odd element chains
    const uint32_t qg[8] = {qa0.x, qa0.y, qa0.z, qa0.w, qa1.x, qa1.y, qa1.z, qa1.w};
    const uint32_t qh[8] = {qb0.x, qb0.y, qb0.z, qb0.w, qb1.x, qb1.y, qb1.z, qb1.w};
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const uint32_t vg = qg[i], vh = qh[i];
      const uint32_t e0 = and_or(vg << 4, mask, magic), e1 = and_or(vh << 4, mask, magic);
      const uint32_t e2 = and_or(vg >> 4, mask, magic), e3 = and_or(vh >> 4, mask, magic);
      const uint32_t o0 = and_or(vg, mask, magic), o1 = and_or(vh, mask, magic);
      const uint32_t o2 = and_or(vg >> 8, mask, magic), o3 = and_or(vh >> 8, mask, magic);
      const uint2 be = lds64(pe + i * 8), bo = lds64(po + i * 8);
      mma16816(de, e0, e1, e2, e3, be.x, be.y);
      mma16816(dq, o0, o1, o2, o3, bo.x, bo.y);
    }
    const float ssum = sx.x + sx.y;
#pragma unroll
    for (int r = 0; r < 2; r++)
      vr[r] = sc[r] * (((de[2 * r] + de[2 * r + 1]) + (dq[2 * r] + dq[2 * r + 1])) - (64.f + zp[r]) * ssum) * up;
  };

  int slot = 0, parity = 0;
  for (int gt = t0; gt < t1; gt += GROUP, parity ^= 1) {
    const int gs = min(GROUP, t1 - gt);
    const uint32_t red_g = red_lane + parity * RED_PARITY;
    for (int b = warp; b < nb; b += WARPS) {
      // this block's activations into the warp's slab; the next block's are requested meanwhile
      const float4 xv[2] = {xn[0], xn[1]};
      {
        const int bn = b + WARPS < nb ? b + WARPS : warp;
        if (b + WARPS < nb || gt + GROUP < t1) load_x(bn);
      }
      // scales and zeros of this block's row tiles: requested here, used after the staging and the first MMAs
      float scg[GROUP][2], zpg[GROUP][2];
      {
        const int grp = (b * 256 + 64 * t) / G;
#pragma unroll
        for (int rt = 0; rt < GROUP; rt++)
#pragma unroll
          for (int r = 0; r < 2; r++) {
            const size_t o = (size_t)(min((gt + min(rt, gs - 1)) * ROWS, N - ROWS) + g + 8 * r) * ngrp + grp;
            scg[rt][r] = __ldg(scales + o), zpg[rt][r] = __ldg(zeros + o);
          }
      }
      __syncwarp();  // every lane is done reading the previous block's slab
      const float up = stage_block_int4(xv, slab, lane);
      __syncwarp();
      float2 sx;
      asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];\n" : "=f"(sx.x), "=f"(sx.y) : "r"(slab + SL::SX_OFF + 8 * t));
#pragma unroll
      for (int rt = 0; rt < GROUP; rt++) {
        if (rt >= gs) break;
        cp_async_wait<S - 1>();  // this lane's granules of the tile have landed ...
        __syncwarp();            // ... and so have the other lanes'
        const uint32_t sb = ring + slot * I4_TILE_BYTES;
        slot = (slot + 1) & (S - 1);
        float vr[2];
        unit(sb, scg[rt], zpg[rt], sx, up, vr);
        // the warp's first block of a group overwrites what an earlier group left behind
        const uint32_t ra = red_g + rt * (32 * 8);
        float2 o = make_float2(0.f, 0.f);
        if (b != warp) asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];\n" : "=f"(o.x), "=f"(o.y) : "r"(ra));
        asm volatile("st.shared.v2.f32 [%0], {%1,%2};\n" ::"r"(ra), "f"(o.x + vr[0]), "f"(o.y + vr[1]));
      }
    }
    __syncthreads();  // also orders this group's reads of red[parity] before its reuse two groups on
    for (int i = threadIdx.x; i < gs * ROWS; i += WARPS * 32) {
      const int rt = i >> 4, row = i & 15, gg = row & 7, hi = row >> 3;
      float v = 0.f;
#pragma unroll
      for (int wq = 0; wq < WARPS; wq++) {
        if (wq >= nb) break;  // a warp without a K block never wrote its part
        const float2 *p = &red[parity][(wq * GROUP + rt) * 32 + gg * 4];
#pragma unroll
        for (int tt = 0; tt < 4; tt++) v += hi ? p[tt].y : p[tt].x;
      }
      const int orow = min((gt + rt) * ROWS, N - ROWS) + row;
      st_act(out, orow, v);
    }
  }
  cp_async_wait<0>();
}

// ------------------------------------------------------------------------------------ Q6_K, 2 .. 8 rows of x
//
// Tokens as MMA columns, as in q4k_gemv_tok_kernel.  The 16 k slots of an MMA are one 16-element
// sub-block here, so every MMA has ONE int8 scale per row: the codes become (code - 32) exactly (PRMT to
// 1024 + code, HADD2 -1056), one HMUL2 applies the scale ((code - 32) * sc is an integer of at most
// 4096: exact up to 2048, rounded to even above, 2.4e-4 relative at worst), and one accumulator sums the
// whole block; once per block and row, acc += d * D.  There is no minimum term.  Float4 F of a token's
// 256 activations is exactly what lane F & 3 feeds to MMA F >> 2, so the slab is x in its own order with
// the (0, 2, 1, 3) pairing inside each four.
constexpr int Q6K_TOK_STAGES = 2;
constexpr int Q6K_TOK_SLAB = TOK * TOK_PITCH;
constexpr int Q6K_TOK_SMEM = WARPS * Q6K_TOK_STAGES * Q6K_TILE_BYTES + WARPS * Q6K_TOK_SLAB + WARPS * GROUP * 32 * 16;

template <int S>
__global__ void __launch_bounds__(WARPS * 32, 2) q6k_gemv_tok_kernel(const float *__restrict__ x, const uint8_t *__restrict__ w,
                                                                    float *__restrict__ out, int M, int N, int K) {
  extern __shared__ __align__(16) unsigned char dyn[];  // [ring: WARPS x S tiles][slabs: WARPS][red: WARPS x GROUP x 32 float4]
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int nb = K >> 8;
  const uint32_t row_bytes = (uint32_t)nb * 210u;  // a multiple of 4 (nb is even: checked by the launcher)
  const uint8_t *w_end = w + (size_t)N * row_bytes;
  const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(dyn);
  const uint32_t ring = sbase + warp * (S * Q6K_TILE_BYTES);
  const uint32_t slab = sbase + WARPS * S * Q6K_TILE_BYTES + warp * Q6K_TOK_SLAB;
  const uint32_t red = sbase + WARPS * S * Q6K_TILE_BYTES + WARPS * Q6K_TOK_SLAB;
  const uint32_t red_lane = red + (uint32_t)((warp * GROUP) * 32 + lane) * 16u;
  const uint32_t m0f = 0x0F0F0F0Fu;

  const int tiles = (N + ROWS - 1) / ROWS;
  const int t0 = (int)((uint32_t)tiles * blockIdx.x / gridDim.x), t1 = (int)((uint32_t)tiles * (blockIdx.x + 1) / gridDim.x);
  const uint32_t c_rsub = lane >> 4, c_piece = lane & 15;
  int i_gt = t0, i_gs = min(GROUP, t1 - t0), i_b = warp, i_rt = 0, i_slot = 0;
  auto issue = [&]() {  // always closes a commit group, so that group counts stay uniform
    if (i_gt < t1 && warp < nb) {
      const int r0 = min((i_gt + i_rt) * ROWS, N - ROWS);
      uint32_t ro = (uint32_t)r0 * row_bytes + (uint32_t)i_b * 210u + c_rsub * row_bytes;
      uint32_t dst = ring + i_slot * Q6K_TILE_BYTES + c_rsub * Q6K_PITCH + c_piece * 16;
      if (c_piece < 14) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const uint8_t *src = w + ((ro & ~15u) + c_piece * 16);
          const long long left = w_end - src;  // the last rows of the matrix: never read past its end
          if (left >= 16)
            cp_async16(dst, src);
          else if (left > 0)
            cp_async16_part(dst, src, (uint32_t)left);
          ro += 2 * row_bytes, dst += 2 * Q6K_PITCH;
        }
      }
      i_slot = i_slot + 1 == S ? 0 : i_slot + 1;
      if (++i_rt == i_gs) {
        i_rt = 0, i_b += WARPS;
        if (i_b >= nb) i_b = warp, i_gt += i_gs, i_gs = min(GROUP, t1 - i_gt);
      }
    }
    cp_async_commit();
  };
#pragma unroll 1
  for (int p = 0; p < S; p++) issue();
  pdl_wait();  // x is the previous launch's output; the weights requested above are not

  // one unit: rows g, g+8 of one tile x one K block out of ring slot `sb`, all tokens of the slab
  auto unit = [&](auto odd_tag, uint32_t sb, uint32_t skew, float (&accr)[4]) {
    constexpr bool ODD = decltype(odd_tag)::value;
    uint32_t wa[2][4], wc[2][4], wh[2][4], scw[2][4];
    float dd[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
      const uint32_t blk = sb + (g + 8 * r) * Q6K_PITCH + skew;  // the block's first byte
#pragma unroll
      for (int hu = 0; hu < 4; hu++) {
        const int h = hu >> 1, u = hu & 1;
        wa[r][hu] = lds32_skew<ODD>(blk + 4 * (16 * h + 4 * u + t));
        wc[r][hu] = lds32_skew<ODD>(blk + 4 * (16 * h + 8 + 4 * u + t));
        wh[r][hu] = lds32_skew<ODD>(blk + 4 * (32 + 8 * h + 4 * u + t));
      }
#pragma unroll
      for (int i = 0; i < 4; i++) scw[r][i] = lds32_skew<ODD>(blk + 192 + 4 * i) ^ 0x80808080u;  // sc + 128, four per word
      dd[r] = f16_bits_to_f32((uint16_t)lds16(blk + 208));
    }
    __syncwarp();  // the slot is free again
    issue();
    float dq[4] = {0.f, 0.f, 0.f, 0.f};
    const __half2 off_c = __float2half2_rn(-1056.f), off_s = __float2half2_rn(-1152.f);
    const uint32_t bx = slab + g * TOK_PITCH + t * 8;  // B fragments of token g
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
            // scale byte m of the row, as the f16 pair (sc, sc): 1024 + (sc + 128) by PRMT, then -1152
            const uint32_t s16 = __byte_perm(scw[r][m >> 2], 0x64646464u, 0x4040 + 0x0101 * (m & 3));
            const __half2 sc = __hadd2(u32_as_h2(s16), off_s);
            a[r] = h2_as_u32(__hmul2(__hadd2(u32_as_h2(__byte_perm(v, 0x64646464u, 0x4240)), off_c), sc));
            a[2 + r] = h2_as_u32(__hmul2(__hadd2(u32_as_h2(__byte_perm(v, 0x64646464u, 0x4341)), off_c), sc));
          }
          const uint2 b = lds64(bx + m * 32);
          mma16816(dq, a[0], a[1], a[2], a[3], b.x, b.y);
        }
    accr[0] = fmaf(dd[0], dq[0], accr[0]), accr[1] = fmaf(dd[0], dq[1], accr[1]);
    accr[2] = fmaf(dd[1], dq[2], accr[2]), accr[3] = fmaf(dd[1], dq[3], accr[3]);
  };

  int slot = 0;
  for (int gt = t0; gt < t1; gt += GROUP) {
    const int gs = min(GROUP, t1 - gt);
    float acc[GROUP][4];
#pragma unroll
    for (int r = 0; r < GROUP; r++) acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.f;
    for (int b = warp; b < nb; b += WARPS) {
      // ---- this block's activations, all tokens, into the warp's slab: lane l takes float4 l and l + 32
      __syncwarp();  // every lane is done reading the previous block's slab
#pragma unroll 4
      for (int tk = 0; tk < TOK; tk++) {
        const float4 *xp = reinterpret_cast<const float4 *>(x + (size_t)tk * K + b * 256);
        float4 v[2];
        v[0] = v[1] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (tk < M) v[0] = __ldg(xp + lane), v[1] = __ldg(xp + lane + 32);
#pragma unroll
        for (int j = 0; j < 2; j++) {
          const __half2 lim = __float2half2_rn(65504.f);
          const __half2 h02 = __hmax2(__hmin2(__floats2half2_rn(v[j].x, v[j].z), lim), __hneg2(lim));
          const __half2 h13 = __hmax2(__hmin2(__floats2half2_rn(v[j].y, v[j].w), lim), __hneg2(lim));
          sts64(slab + tk * TOK_PITCH + (uint32_t)(lane + 32 * j) * 8u, h2_as_u32(h02), h2_as_u32(h13));
        }
      }
      __syncwarp();
#pragma unroll
      for (int rt = 0; rt < GROUP; rt++) {
        if (rt < gs) {
          cp_async_wait<S - 1>();  // this lane's granules of the tile have landed ...
          __syncwarp();            // ... and so have the other lanes'
          const uint32_t sb = ring + slot * Q6K_TILE_BYTES;
          slot = slot + 1 == S ? 0 : slot + 1;
          const int r0 = min((gt + rt) * ROWS, N - ROWS);
          const uint32_t skew = ((uint32_t)r0 * row_bytes + (uint32_t)b * 210u + (uint32_t)g * row_bytes) & 15u;
          if (b & 1)
            unit(std::true_type{}, sb, skew, acc[rt]);
          else
            unit(std::false_type{}, sb, skew, acc[rt]);
        }
      }
    }
    // ---- add up the warps' parts: lane (g, t) of tile rt holds rows g, g+8 x tokens 2t, 2t+1
    __syncthreads();  // the previous group's sums have been read
#pragma unroll
    for (int rt = 0; rt < GROUP; rt++)
      asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};\n" ::"r"(red_lane + rt * 512), "f"(acc[rt][0]), "f"(acc[rt][1]),
                   "f"(acc[rt][2]), "f"(acc[rt][3]));
    __syncthreads();
    for (int i = threadIdx.x; i < gs * ROWS * TOK; i += WARPS * 32) {
      const int row = i & 15, tok = (i >> 4) & 7, rt = i >> 7;
      const uint32_t a = red + (uint32_t)(rt * 32 + (row & 7) * 4 + (tok >> 1)) * 16u + (uint32_t)((row >> 3) * 2 + (tok & 1)) * 4u;
      float v = 0.f;
#pragma unroll
      for (int wq = 0; wq < WARPS; wq++) {
        if (wq >= nb) break;
        float p;
        asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(p) : "r"(a + wq * (GROUP * 512)));
        v += p;
      }
      if (tok < M) out[(size_t)tok * N + min((gt + rt) * ROWS, N - ROWS) + row] = v;
    }
  }
  cp_async_wait<0>();
}

template <typename... Args>
int launch_pdl(void (*kern)(Args...), unsigned grid, size_t dyn_smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(WARPS * 32);
  cfg.dynamicSmemBytes = dyn_smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, args...);
  if (e != cudaSuccess) return fail((int)e, "light_b200: matmul_q (decode): %s", cudaGetErrorString(e));
  return 0;
}

#define g_sms (sm_count())  // SMs of the calling thread's current device (every entry point binds it first)
int g_waves = 2;       // LIGHT_B200_GEMV_WAVES: CTAs per SM of the persistent kernels' grids (1 or 2)
int g_q4k_stages = 4;  // LIGHT_B200_Q4K_STAGES: ring depth (2 or 4)
constexpr size_t MAX_DYN_SMEM = 96 * 1024;  // keeps two launches resident per SM

}  // namespace

int gguf_gemv_fast_init(int device) {
  if (const char *e = getenv("LIGHT_B200_GEMV_WAVES")) g_waves = atoi(e) == 1 ? 1 : 2;
  if (const char *e = getenv("LIGHT_B200_Q4K_STAGES")) g_q4k_stages = atoi(e) == 2 ? 2 : 4;
  cudaError_t err = cudaFuncSetAttribute(q4k_gemv_mma_kernel<4, 2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MAX_DYN_SMEM);
  if (err == cudaSuccess)
    err = cudaFuncSetAttribute(q4k_gemv_mma_kernel<2, 3, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MAX_DYN_SMEM);
  if (err == cudaSuccess)
    err = cudaFuncSetAttribute(q6k_gemv_mma_kernel<Q6K_STAGES, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               WARPS * Q6K_STAGES * Q6K_TILE_BYTES);
  if (err == cudaSuccess)
    err = cudaFuncSetAttribute(q80_gemv_mma_kernel<Q80_STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, WARPS * Q80_STAGES * Q80_TILE_BYTES);
  if (err == cudaSuccess)
    err = cudaFuncSetAttribute(q4k_gemv_mma_kernel<4, 2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MAX_DYN_SMEM);
  if (err == cudaSuccess)
    err = cudaFuncSetAttribute(q4k_gemv_mma_kernel<4, 2, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MAX_DYN_SMEM);
  if (err == cudaSuccess)
    err = cudaFuncSetAttribute(q6k_gemv_mma_kernel<Q6K_STAGES, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               WARPS * Q6K_STAGES * Q6K_TILE_BYTES);
  if (err == cudaSuccess)
    err = cudaFuncSetAttribute(q4k_gemv_tok_kernel<Q4K_TOK_STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, Q4K_TOK_SMEM);
  if (err == cudaSuccess)
    err = cudaFuncSetAttribute(q6k_gemv_tok_kernel<Q6K_TOK_STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, Q6K_TOK_SMEM);
  if (err != cudaSuccess) return fail((int)err, "light_b200: init (decode): %s", cudaGetErrorString(err));
  return 0;
}

// One launch over up to four Q4_K matrices that share x (M = 1).  Returns 1 if launched, 0 if this
// path does not apply, < 0 or a CUDA code on error.
static const NormArgs NO_NORM = {};
static int q4k_launch(const float *x, const MultiArgs &a, const TpArgs &tp, int tiles, int K, cudaStream_t st, const NormArgs &nrm = NO_NORM) {
  const size_t dyn = (size_t)WARPS * (tp.step || nrm.weight ? 4 : g_q4k_stages) * Q4K_TILE_BYTES + (size_t)(K >> 8) * Q4K_SLAB;
  if (dyn > MAX_DYN_SMEM) return 0;  // very long rows: the activations do not fit beside the rings
  const int lt = a.act ? tiles / 2 : tiles;
  const int per_sm = (g_q4k_stages == 2 && !tp.step && !nrm.weight) ? 3 : g_waves;  // the 2-deep ring leaves room for three CTAs per SM
  const unsigned grid = (unsigned)(lt < g_sms * per_sm ? lt : g_sms * per_sm);
  int rc = nrm.weight         ? launch_pdl(q4k_gemv_mma_kernel<4, 2, false, true>, grid, dyn, st, x, a, tp, nrm, tiles, K)
           : tp.step           ? launch_pdl(q4k_gemv_mma_kernel<4, 2, true>, grid, dyn, st, x, a, tp, nrm, tiles, K)
           : g_q4k_stages == 2 ? launch_pdl(q4k_gemv_mma_kernel<2, 3, false>, grid, dyn, st, x, a, tp, nrm, tiles, K)
                               : launch_pdl(q4k_gemv_mma_kernel<4, 2, false>, grid, dyn, st, x, a, tp, nrm, tiles, K);
  if (rc) return rc;
  rc = launched("matmul_q (decode)");
  return rc ? rc : 1;
}

static const TpArgs NO_TP = {};

int gguf_gemv_fast(int type, const float *x, const void *w, float *out, int M, int N, int K, cudaStream_t st) {
  if (type == LB200_Q8_0 && M >= 2 && M <= 3) {  // no token-column kernel for this format: a pass per row beats the tensor-core kernel up to three rows
    for (int m = 0; m < M; m++) {
      const int rc = gguf_gemv_fast(type, x + (size_t)m * K, w, out + (size_t)m * N, 1, N, K, st);
      if (rc != 1) return m == 0 ? rc : fail(rc < 0 ? rc : LB200_E_SHAPE, "light_b200: matmul_q (decode): row %d refused after row 0 was launched", m);
    }
    return 1;
  }
  if (M != 1 || K % 256 || N < ROWS) return 0;
  if (type != LB200_Q4_K && type != LB200_Q6_K && type != LB200_Q8_0) return 0;
  if ((uintptr_t)w & 15) return 0;
  // Q6_K: an even number of blocks per row keeps every row's skew equal for rows 8 apart and
  // word-aligned for even blocks; byte offsets are 32-bit
  if (type == LB200_Q6_K && (((K >> 8) & 1) || (unsigned long long)N * (K >> 8) * 210ull >= (1ull << 32))) return 0;
  const uint8_t *wb = (const uint8_t *)w;
  const int tiles = (N + ROWS - 1) / ROWS;
  if (type == LB200_Q4_K) {
    MultiArgs a = {};
    a.w[0] = wb, a.out[0] = out, a.n[0] = N, a.tend[0] = tiles, a.count = 1;
    return q4k_launch(x, a, NO_TP, tiles, K, st);
  }
  const unsigned grid = (unsigned)(tiles < g_sms * g_waves ? tiles : g_sms * g_waves);
  if (type == LB200_Q8_0) {
    int rc = launch_pdl(q80_gemv_mma_kernel<Q80_STAGES>, grid, (size_t)WARPS * Q80_STAGES * Q80_TILE_BYTES, st, x, wb, out, N, K);
    if (rc) return rc;
    rc = launched("matmul_q (decode)");
    return rc ? rc : 1;
  }
  int rc = launch_pdl(q6k_gemv_mma_kernel<Q6K_STAGES, false>, grid, (size_t)WARPS * Q6K_STAGES * Q6K_TILE_BYTES, st, x, wb, out, NO_TP, N, K);
  if (rc) return rc;
  rc = launched("matmul_q (decode)");
  return rc ? rc : 1;
}

// One to a few activation rows against group-quantized 4-bit weights in the canonical layout: a pass of the
// one-row kernel per row: bf16 activations up to three rows (then the tensor-core decode kernel wins), f32
// activations up to 64 (their only other kernel below the prefill range is the CUDA-core one, which a pass per
// row beats at every count: 10.5 us against 236 us per row at 18944 x 3584).  Returns 1 if launched, 0 if
// the shape is not covered.
int g_int4_fast_max_f32 = 64, g_int4_fast_max_bf16 = 3;  // LIGHT_B200_INT4_FAST_MAX_M (tuning knob, both)
int int4_gemv_fast(const void *x, const uint32_t *codes, const float *s, const float *z, void *y, int act_dtype, int M, int N, int K,
                   int G, cudaStream_t st) {
  static bool knob = false;
  if (!knob) {
    if (const char *e = getenv("LIGHT_B200_INT4_FAST_MAX_M")) g_int4_fast_max_f32 = g_int4_fast_max_bf16 = atoi(e);
    knob = true;
  }
  if (M < 1 || M > (act_dtype == LB200_F32 ? g_int4_fast_max_f32 : g_int4_fast_max_bf16)) return 0;
  if (K % 256 || G % 64 || N < ROWS || ((uintptr_t)codes & 15) || ((uintptr_t)x & 15) || (act_dtype == LB200_BF16 && (K % 8))) return 0;
  if (act_dtype != LB200_F32 && act_dtype != LB200_BF16) return 0;
  static DeviceOnce attr_done;
  {
    cudaError_t e = attr_done.ensure([&] {
      cudaError_t r = cudaFuncSetAttribute(int4_gemv_mma_kernel<I4_STAGES, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, WARPS * I4_STAGES * I4_TILE_BYTES);
      return r != cudaSuccess ? r : cudaFuncSetAttribute(int4_gemv_mma_kernel<I4_STAGES, __nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, WARPS * I4_STAGES * I4_TILE_BYTES);
    });
    if (e != cudaSuccess) return fail((int)e, "light_b200: int4_gemv (decode): %s", cudaGetErrorString(e));
  }
  const int tiles = (N + ROWS - 1) / ROWS;
  const unsigned grid = (unsigned)(tiles < g_sms * g_waves ? tiles : g_sms * g_waves);
  const size_t dyn = (size_t)WARPS * I4_STAGES * I4_TILE_BYTES;
  for (int m = 0; m < M; m++) {
    int rc;
    if (act_dtype == LB200_F32)
      rc = launch_pdl(int4_gemv_mma_kernel<I4_STAGES, float>, grid, dyn, st, (const float *)x + (size_t)m * K, (const uint8_t *)codes, s, z,
                      (float *)y + (size_t)m * N, N, K, G);
    else
      rc = launch_pdl(int4_gemv_mma_kernel<I4_STAGES, __nv_bfloat16>, grid, dyn, st, (const __nv_bfloat16 *)x + (size_t)m * K, (const uint8_t *)codes,
                      s, z, (__nv_bfloat16 *)y + (size_t)m * N, N, K, G);
    if (rc) return rc;
    if (int l = launched("int4_gemv (decode)")) return l;
  }
  return 1;
}

// One to a few activation rows against block-scaled e4m3 weights: a pass of the one-row kernel per row (bf16
// up to two rows, f32 up to 64: as for int4).  Returns 1 if launched, 0 if the shape is not covered.
int g_fp8_fast_max_f32 = 64, g_fp8_fast_max_bf16 = 2;  // LIGHT_B200_FP8_FAST_MAX_M (tuning knob, both)
int fp8_gemv_fast(const void *x, const uint8_t *w, const float *scale, void *y, int act_dtype, int M, int N, int K, int bR, int bC,
                  cudaStream_t st) {
  static bool knob = false;
  if (!knob) {
    if (const char *e = getenv("LIGHT_B200_FP8_FAST_MAX_M")) g_fp8_fast_max_f32 = g_fp8_fast_max_bf16 = atoi(e);
    knob = true;
  }
  if (act_dtype != LB200_F32 && act_dtype != LB200_BF16) return 0;
  if (M < 1 || M > (act_dtype == LB200_F32 ? g_fp8_fast_max_f32 : g_fp8_fast_max_bf16)) return 0;
  if (K % 256 || bC % 32 || bR % 16 || N < ROWS || N % bR || K % bC || ((uintptr_t)w & 15) || ((uintptr_t)x & 15)) return 0;
  static DeviceOnce attr_done;
  {
    cudaError_t e = attr_done.ensure([&] {
      cudaError_t r = cudaFuncSetAttribute(fp8_gemv_mma_kernel<F8_STAGES, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, WARPS * F8_STAGES * F8_TILE_BYTES);
      return r != cudaSuccess ? r : cudaFuncSetAttribute(fp8_gemv_mma_kernel<F8_STAGES, __nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, WARPS * F8_STAGES * F8_TILE_BYTES);
    });
    if (e != cudaSuccess) return fail((int)e, "light_b200: fp8_block_gemv (decode): %s", cudaGetErrorString(e));
  }
  const int tiles = (N + ROWS - 1) / ROWS;
  const unsigned grid = (unsigned)(tiles < g_sms * g_waves ? tiles : g_sms * g_waves);
  const size_t dyn = (size_t)WARPS * F8_STAGES * F8_TILE_BYTES;
  for (int m = 0; m < M; m++) {
    int rc;
    if (act_dtype == LB200_F32)
      rc = launch_pdl(fp8_gemv_mma_kernel<F8_STAGES, float>, grid, dyn, st, (const float *)x + (size_t)m * K, w, scale, (float *)y + (size_t)m * N, N, K,
                      bR, bC);
    else
      rc = launch_pdl(fp8_gemv_mma_kernel<F8_STAGES, __nv_bfloat16>, grid, dyn, st, (const __nv_bfloat16 *)x + (size_t)m * K, w, scale,
                      (__nv_bfloat16 *)y + (size_t)m * N, N, K, bR, bC);
    if (rc) return rc;
    if (int l = launched("fp8_block_gemv (decode)")) return l;
  }
  return 1;
}

// 2 .. 8 activation rows against one Q4_K or Q6_K matrix, tokens as MMA columns.  Returns 1 if launched, 0 if
// the shape is not covered.
int g_tok_max_m = 8;  // LIGHT_B200_TOK_MAX_M (tuning knob): most activation rows served by passes of eight (beyond 8 the other kernels win)
int gguf_gemv_tok(int type, const float *x, const void *w, float *out, int M, int N, int K, cudaStream_t st) {
  static bool knob = false;
  if (!knob) {
    if (const char *e = getenv("LIGHT_B200_TOK_MAX_M")) g_tok_max_m = atoi(e);
    knob = true;
  }
  if ((type != LB200_Q4_K && type != LB200_Q6_K) || M < 2 || M > g_tok_max_m || K % 256 || N < ROWS || ((uintptr_t)w & 15) || ((uintptr_t)x & 15)) return 0;
  if (type == LB200_Q6_K && (((K >> 8) & 1) || (unsigned long long)N * (K >> 8) * 210ull >= (1ull << 32))) return 0;
  const int tiles = (N + ROWS - 1) / ROWS;
  const unsigned grid = (unsigned)(tiles < g_sms * 2 ? tiles : g_sms * 2);
  // eight tokens per pass; a second pass finds a decode-sized matrix in the 126 MB L2
  for (int m0 = 0; m0 < M; m0 += TOK) {
    const int mm = M - m0 < TOK ? M - m0 : TOK;
    const float *xm = x + (size_t)m0 * K;
    float *om = out + (size_t)m0 * N;
    MultiArgs a = {};
    a.w[0] = (const uint8_t *)w, a.out[0] = om, a.n[0] = N, a.tend[0] = tiles, a.count = 1;
    int rc = type == LB200_Q4_K
                 ? launch_pdl(q4k_gemv_tok_kernel<Q4K_TOK_STAGES>, grid, (size_t)Q4K_TOK_SMEM, st, xm, a, tiles, mm, K)
                 : launch_pdl(q6k_gemv_tok_kernel<Q6K_TOK_STAGES>, grid, (size_t)Q6K_TOK_SMEM, st, xm, (const uint8_t *)w, om, mm, N, K);
    if (rc) return rc;
    rc = launched("matmul_q (decode, 2-8 rows)");
    if (rc) return rc;
  }
  return 1;
}

// 9 .. 32 activation rows per pass (more rows: passes of 32) against one Q4_K matrix: eight row tiles per CTA,
// K split over a cluster.  Returns 1 if launched, 0 if the shape is not covered.
template <int NG>
static int launch_tile(const float *x, const MultiArgs &ma, int tiles, int M, int K, cudaStream_t st) {
  auto kern = q4k_decode_tile_kernel<NG>;
  static DeviceOnce attr_done;
  {
    cudaError_t e = attr_done.ensure([&] { return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, DtCfg<NG>::SMEM); });
    if (e != cudaSuccess) return fail((int)e, "light_b200: matmul_q (decode, tiles): %s", cudaGetErrorString(e));
  }
  const int nx = (tiles + DT_CW - 1) / DT_CW, nb = K >> 8;
  // measured on 4096 x 4096, 1024 x 4096 and 14336 x 4096: short K runs win (a CTA's start-up and its first
  // block of x are not overlapped with anything) until two CTAs per SM are resident and more wait behind them
  int ks = nx * 2 >= g_sms ? 2 : 8;
  while (ks > nb) ks >>= 1;
  if (const char *e = getenv("LIGHT_B200_TILE_KS")) { const int v = atoi(e); if (v >= 1 && v <= 8 && v <= nb) ks = v; }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)nx, (unsigned)ks, 1);
  cfg.blockDim = dim3(DT_THREADS);
  cfg.dynamicSmemBytes = DtCfg<NG>::SMEM;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = 1, attr[1].val.clusterDim.y = (unsigned)ks, attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, x, ma, tiles, M, K);
  if (e != cudaSuccess) return fail((int)e, "light_b200: matmul_q (decode, tiles): %s", cudaGetErrorString(e));
  return launched("matmul_q (decode, tiles)");
}

int g_tile_min_m = 9, g_tile_max_m = 32;  // LIGHT_B200_TILE_MIN_M / _MAX_M (tuning knobs)
int gguf_decode_tile(int type, const float *x, const void *w, float *out, int M, int N, int K, cudaStream_t st) {
  static bool knob = false;
  if (!knob) {
    if (const char *e = getenv("LIGHT_B200_TILE_MIN_M")) g_tile_min_m = atoi(e);
    if (const char *e = getenv("LIGHT_B200_TILE_MAX_M")) g_tile_max_m = atoi(e);
    knob = true;
  }
  if (type != LB200_Q4_K || M < g_tile_min_m || M > g_tile_max_m || K % 256 || N < ROWS || ((uintptr_t)w & 15) || ((uintptr_t)x & 15)) return 0;
  for (int m0 = 0; m0 < M; m0 += 32) {
    const int mm = M - m0 < 32 ? M - m0 : 32;
    const float *xm = x + (size_t)m0 * K;
    float *om = out + (size_t)m0 * N;
    MultiArgs ma = {};
    const int tiles = (N + ROWS - 1) / ROWS;
    ma.w[0] = (const uint8_t *)w, ma.out[0] = om, ma.n[0] = N, ma.tend[0] = tiles, ma.count = 1;
    const int rc = mm <= 16 ? launch_tile<2>(xm, ma, tiles, mm, K, st) : launch_tile<4>(xm, ma, tiles, mm, K, st);
    if (rc) return rc;
  }
  return 1;
}

// 2 .. 32 activation rows against up to four Q4_K matrices that share them (q, k, v; gate, up), one launch:
// ops.LinearMulti for a small batch (the token-column kernel up to 8 rows, the eight-tiles-per-CTA kernel above:
// q,k,v of configs[1] at 32 rows 23.4 us merged against 32.9 us as three launches; gate,up the same either way).  Returns 1 if launched, 0 if the shape is not covered.
int gguf_gemv_tok_multi(int type, const float *x, const void *const *w, float *const *out, const int *n, int count, int M, int K,
                        cudaStream_t st) {
  static int tile_multi = -1;  // LIGHT_B200_TILE_MULTI=0 (tuning knob): merge only up to 8 rows
  if (tile_multi < 0) tile_multi = getenv("LIGHT_B200_TILE_MULTI") ? atoi(getenv("LIGHT_B200_TILE_MULTI")) : 1;
  if (type != LB200_Q4_K || M < 2 || M > (tile_multi ? g_tile_max_m : TOK) || count < 1 || count > 4 || K % 256 || ((uintptr_t)x & 15)) return 0;
  MultiArgs a = {};
  int tiles = 0;
  for (int i = 0; i < count; i++) {
    if (n[i] < ROWS || ((uintptr_t)w[i] & 15)) return 0;
    tiles += (n[i] + ROWS - 1) / ROWS;
    a.w[i] = (const uint8_t *)w[i], a.out[i] = out[i], a.n[i] = n[i], a.tend[i] = tiles;
  }
  a.count = count;
  if (M > TOK) {  // 9 .. 32 rows: the kernel with eight row tiles per CTA
    const int rc = M <= 16 ? launch_tile<2>(x, a, tiles, M, K, st) : launch_tile<4>(x, a, tiles, M, K, st);
    return rc ? rc : 1;
  }
  const unsigned grid = (unsigned)(tiles < g_sms * 2 ? tiles : g_sms * 2);
  int rc = launch_pdl(q4k_gemv_tok_kernel<Q4K_TOK_STAGES>, grid, (size_t)Q4K_TOK_SMEM, st, x, a, tiles, M, K);
  if (rc) return rc;
  rc = launched("matmul_q_multi (2-8 rows)");
  return rc ? rc : 1;
}

// Several matrices of one type against one activation row in one launch (act == 0), or the gated
// pair act(w[0] x) * (w[1] x) -> out[0] (act 1 = SiLU, 2 = GELU).  Returns 1 if launched, 0 if no
// single-launch kernel applies (the caller then issues one matmul per matrix), else an error.
int gguf_gemv_multi(int type, const float *x, const void *const *w, float *const *out, const int *n, int count, int act,
                    int K, cudaStream_t st, const lb200_norm *norm) {
  if (type != LB200_Q4_K || K % 256 || count < 1 || count > 4) return 0;
  NormArgs nrm = {};
  if (norm) {
    if (((uintptr_t)norm->weight | (uintptr_t)norm->residual | (uintptr_t)norm->sum_out) & 15) return 0;
    nrm.weight = norm->weight, nrm.residual = norm->residual, nrm.sum_out = norm->sum_out, nrm.eps = norm->eps;
  }
  if (act && (count != 2 || n[0] != n[1])) return 0;
  MultiArgs a = {};
  int tiles = 0;
  for (int i = 0; i < count; i++) {
    if (n[i] < ROWS || ((uintptr_t)w[i] & 15)) return 0;
    tiles += (n[i] + ROWS - 1) / ROWS;
    a.w[i] = (const uint8_t *)w[i], a.out[i] = out[i], a.n[i] = n[i], a.tend[i] = tiles;
  }
  a.count = count, a.act = act;
  return q4k_launch(x, a, NO_TP, tiles, K, st, nrm);
}

// Row-split matmul with the exchange inside the launch (see TpArgs): `count` matrices of one type that
// share x; x comes as plain f32 (x) or as this rank's receive buffer of the producing launch (x_slots);
// out_slots[i * LB200_MAX_PEERS + p] is rank p's receive buffer for output i, or all null for an output that
// stays local.  Returns 1 if launched, 0 if no kernel covers the shape, else an error.
int gguf_gemv_tp(int type, const float *x, const void *x_slots, const void *const *w, float *const *out, const int *n,
                 int count, int K, void *const *out_slots, const unsigned int *step, int world, int rank, cudaStream_t st) {
  if (K % 256 || count < 1 || count > 4 || world < 1 || world > LB200_MAX_PEERS || rank < 0 || rank >= world) return 0;
  if (((uintptr_t)x_slots & 31) || (x && ((uintptr_t)x & 15))) return 0;
  TpArgs tp = {};
  tp.x_slots = (const uint2 *)x_slots, tp.step = step, tp.world = world, tp.rank = rank;
  for (int i = 0; i < count; i++)
    for (int p = 0; p < world; p++) {
      tp.peer[i][p] = (uint2 *)out_slots[i * LB200_MAX_PEERS + p];
      if ((tp.peer[i][p] == nullptr) != (tp.peer[i][0] == nullptr) || ((uintptr_t)tp.peer[i][p] & 7)) return 0;
    }
  if (type == LB200_Q4_K) {
    MultiArgs a = {};
    int tiles = 0;
    for (int i = 0; i < count; i++) {
      if (n[i] < ROWS || ((uintptr_t)w[i] & 15)) return 0;
      tiles += (n[i] + ROWS - 1) / ROWS;
      a.w[i] = (const uint8_t *)w[i], a.out[i] = out[i], a.n[i] = n[i], a.tend[i] = tiles;
    }
    a.count = count;
    return q4k_launch(x, a, tp, tiles, K, st);
  }
  if (type != LB200_Q6_K || count != 1 || n[0] < ROWS || ((uintptr_t)w[0] & 15)) return 0;
  if (((K >> 8) & 1) || (unsigned long long)n[0] * (K >> 8) * 210ull >= (1ull << 32)) return 0;
  const int tiles = (n[0] + ROWS - 1) / ROWS;
  const unsigned grid = (unsigned)(tiles < g_sms * g_waves ? tiles : g_sms * g_waves);
  int rc = launch_pdl(q6k_gemv_mma_kernel<Q6K_STAGES, true>, grid, (size_t)WARPS * Q6K_STAGES * Q6K_TILE_BYTES, st, x,
                      (const uint8_t *)w[0], out[0], tp, n[0], K);
  if (rc) return rc;
  rc = launched("matmul_q (decode, row-split)");
  return rc ? rc : 1;
}

int gemv_tp_status() {
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_tp_status, sizeof(int));
  return e == cudaSuccess ? v : -(int)e;
}

}  // namespace lb
