// A decode step's DEPENDENT matrix-vector products as ONE persistent launch.
//
// The reference replays a decode step as a CUDA graph of one kernel per operator (models/decode_graph.go:58-205,
// models/llama.go:1070-1330): every quantized linear is a launch whose input is the previous launch's output.
// For one activation row a launch streams a few MB, so the step is bound by what stands between two launches
// (grid completion, launch, first-tile latency), not by HBM.  This kernel runs a whole PROGRAM of such
// operators -- q,k,v -> o -> gate,up -> down -> next layer ... -> lm_head -- in one launch of one CTA per SM:
//
//   * no barrier between operators.  Every vector that one operator hands to the next is a buffer of 8-byte
//     slots {f32 value, u32 tag}, tag = (step, producing operator).  The thread that holds a finished output
//     value stores the slot with one 8-byte store; a consumer's activation load polls the slots it needs until
//     they carry the expected tag (bounded, then a sticky status word).  The data is its own arrival flag: no
//     fence, no counter, no grid-wide barrier, and the dependency is as fine as a 256-element block of x;
//   * the weight stream never stops.  Each warp owns a ring of shared-memory slots filled by bulk asynchronous
//     copies (cp.async.bulk, completion on an mbarrier per slot; one 144-byte Q4_K / 224-byte Q6_K row piece
//     per lane) that run STAGES tiles ahead of the arithmetic -- across operator boundaries: while the CTA
//     waits for the activations of operator i+1, the tiles of operator i+1 (which do not depend on them) are
//     already landing;
//   * the arithmetic is integer: a warp owns one 256-element K block of x and walks down row tiles of 16
//     weight rows.  The packed codes become the A fragment of mma.sync.m16n8k32 (u8 x s8 -> s32) with ONE
//     logic instruction per four weights (Q4_K: code & 0x0F0F0F0F, or & 0xF0F0F0F0 = 16 * code; Q6_K: the 6-bit
//     codes as bytes); the activations are split once per block into three signed 8-bit terms
//     x ~ s0 hi + s1 mid + s2 lo (s1 = s0 / 254, s2 = s1 / 254; error below 2^-23 of the block's largest
//     value), and the eight columns of the MMA hold these terms block-diagonally per sub-block, so that
//     D[row][col] are the per-sub-block integer dot products a scale applies to.  The CUDA cores touch each
//     (row, sub-block) once.
//
// Row-split over several GPUs is the same program with the slot stores going to every rank's buffer.
#include <cstdlib>
#include <cstring>
#include <type_traits>
#include <vector>

#include "common.cuh"
#include "decode_units.cuh"
#include "mma_sync.cuh"
#include "umma.cuh"

namespace lb {

namespace {

constexpr int CW = 16;           // warps per CTA
constexpr int CT = CW * 32;      // threads per CTA
constexpr int ROWS = 16;         // weight rows per tile
constexpr int GROUP = 4;         // row tiles whose partial sums a warp holds at a time
constexpr int STAGES = 3;        // ring slots per warp
constexpr int Q4_PITCH = 144;    // a Q4_K block per row, dense
constexpr int Q6_PITCH = 240;    // the 14 granules that cover a Q6_K block, padded
constexpr int Q6_COPY = 224;
constexpr int SLOT = ROWS * Q6_PITCH;  // 3840 bytes: either tile kind
constexpr int RING = CW * STAGES * SLOT;

// Per-warp activation slab: three planes of signed bytes (hi, mid, lo), the sub-block sums of x, the scales.
//   Q4_K layout: plane p at p * 320, 32-element sub-block s at 40 * s (the 8-byte pad spreads the B-fragment
//                loads of the four sub-block pairs and the two planes of one MMA over distinct banks);
//   Q6_K layout: plane p at p * 272, element e at e.
constexpr int X4_SUB = 40, X4_PLANE = 320, X6_PLANE = 272;
constexpr int SLAB_SX = 960;     // 16 floats: sums of x over 16-element (Q6_K) or 32-element (Q4_K) sub-blocks
constexpr int SLAB_SC = 1024;    // s0, s1, s2, up
constexpr int SLAB = 1040;

constexpr int RED_FLOATS = 2 * CW * GROUP * ROWS;  // two parities
constexpr int SMEM_RED = RING + CW * SLAB;
constexpr int SMEM_NRM = SMEM_RED + RED_FLOATS * 4;  // [2][CW] floats
constexpr int SMEM_BAR = SMEM_NRM + 2 * CW * 4;
constexpr int SMEM_ZERO = SMEM_BAR + CW * STAGES * 8;  // what the B-fragment loads of lanes outside an MMA's live columns read
constexpr int ZERO_BYTES = 160;
constexpr int SMEM_ABORT = SMEM_ZERO + ZERO_BYTES;  // one int: a bounded wait of this CTA gave up
constexpr int SMEM_BYTES = SMEM_ABORT + 16;

constexpr uint32_t NONE = 0xFFFFFFFFu;

// One operator of the program, as the kernel reads it (device memory, read-only during a launch).
struct alignas(16) OpDev {
  const uint8_t *w[4];
  float *out[4];
  int n[4];       // rows this rank holds of each matrix
  int tend[4];    // running total of row tiles (act == 0)
  uint32_t out_off[4];  // byte offset of output i's slots inside the arena, or NONE
  const float *x_plain;
  const float *norm_w;
  uint32_t x_off, res_off, sum_off;  // slot vectors: activations, residual, where x + residual goes (or NONE)
  uint32_t x_tag, res_tag;           // 1 + index of the operator that produced them
  float eps;
  int kind;   // 0: Q4_K, 1: Q6_K
  int K, count, act, tiles;
  int pad[3];
};
static_assert(sizeof(OpDev) % 16 == 0, "OpDev is copied and read in 16-byte pieces");

struct alignas(16) Header {
  uint8_t *arena[LB200_MAX_PEERS];
  int n_ops, world, rank, pad;
};
constexpr size_t HEADER_BYTES = 256;

__device__ unsigned int g_chain_status;  // non-zero: a bounded wait gave up (sticky)

__device__ __forceinline__ void imma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// the first MMA of a chain: the accumulator starts from zero (no registers to clear)
__device__ __forceinline__ void imma_u8s8_first(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
               : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void sts32(uint32_t addr, uint32_t v) { asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(addr), "r"(v)); }
__device__ __forceinline__ uint32_t lds16u(uint32_t addr) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];\n" : "=h"(v) : "r"(addr));
  return v;
}
template <bool ODD>
__device__ __forceinline__ uint32_t lds32_at2(uint32_t addr) {  // word at a 2-byte aligned address; ODD: not 4-byte aligned
  if constexpr (!ODD) return lds32(addr);
  return __funnelshift_r(lds32(addr - 2), lds32(addr + 2), 16);
}
// one row piece global -> shared, completion counted in bytes on the slot's mbarrier
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(bar) : "memory");
}

// Bounded waits: every poll loop calls this now and then.  It gives up 200 ms after the loop's own start, or as
// soon as any thread of the CTA has given up (the flag in shared memory), sets the sticky status word, and from
// then on every wait of the CTA falls through: the launch ends quickly, with outputs that are not valid.
__device__ __forceinline__ bool wait_expired(volatile int *abort_flag, unsigned long long &t0) {
  if (*abort_flag) return true;
  const unsigned long long t = umma::global_ns();
  if (t0 == 0) t0 = t;
  if (t - t0 > 200000000ull) {
    g_chain_status = 1u;
    *abort_flag = 1;
    return true;
  }
  return false;
}

// one value, tagged, into the same slot of every rank's arena (one rank: this GPU's own)
__device__ __forceinline__ void st_slot(const Header *hd, uint8_t *arena_me, int world, uint32_t off, size_t e, float v, unsigned int tag) {
  if (world == 1) {
    asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};\n" ::"l"(reinterpret_cast<uint2 *>(arena_me + off) + e), "r"(__float_as_uint(v)), "r"(tag)
                 : "memory");
    return;
  }
  for (int p = 0; p < world; p++) {
    uint8_t *a = (uint8_t *)__ldg(reinterpret_cast<const unsigned long long *>(&hd->arena[p]));
    asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};\n" ::"l"(reinterpret_cast<uint2 *>(a + off) + e), "r"(__float_as_uint(v)), "r"(tag) : "memory");
  }
}

__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d) {
  return __byte_perm(__byte_perm((uint32_t)a, (uint32_t)b, 0x0040), __byte_perm((uint32_t)c, (uint32_t)d, 0x0040), 0x5410);
}

// One block's activations (two float4 per lane: elements 4 lane .. +3 and 128 + 4 lane .. +3) -> the warp's
// slab: x * 2^-e = s0 hi + s1 mid + s2 lo with |hi|, |mid|, |lo| <= 127, s0 = max / 127, s1 = s0 / 254, s2 = s1 / 254.
template <bool Q6>
__device__ __forceinline__ void stage3(const float4 (&xv)[2], uint32_t slab, int lane) {
  uint32_t m = 0;
#pragma unroll
  for (int i = 0; i < 2; i++) {
    m = max(m, __float_as_uint(xv[i].x) & 0x7fffffffu);
    m = max(m, __float_as_uint(xv[i].y) & 0x7fffffffu);
    m = max(m, __float_as_uint(xv[i].z) & 0x7fffffffu);
    m = max(m, __float_as_uint(xv[i].w) & 0x7fffffffu);
  }
  m = __reduce_max_sync(0xffffffffu, m);
  uint32_t eb = m >> 23;
  eb = eb < 1u ? 1u : (eb > 253u ? 253u : eb);
  const float down = __uint_as_float((254u - eb) << 23), up = __uint_as_float(eb << 23);  // exact powers of two
  const float mx = __uint_as_float(m) * down;                                            // in [1, 2) unless clamped
  const bool any = mx > 0.f;
  const float s0 = mx * (1.f / 127.f), s1 = s0 * (1.f / 254.f), s2 = s1 * (1.f / 254.f);
  const float i0 = any ? 1.f / s0 : 0.f, i1 = any ? 1.f / s1 : 0.f, i2 = any ? 1.f / s2 : 0.f;
  constexpr int PLANE = Q6 ? X6_PLANE : X4_PLANE;
  constexpr int LPS = Q6 ? 4 : 8;  // lanes per sub-block
#pragma unroll
  for (int i = 0; i < 2; i++) {
    const float v[4] = {xv[i].x * down, xv[i].y * down, xv[i].z * down, xv[i].w * down};
    int h[4], md[4], lo[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const float fh = rintf(v[j] * i0);
      const float r1 = fmaf(-fh, s0, v[j]);
      const float fm = fminf(fmaxf(rintf(r1 * i1), -127.f), 127.f);
      const float r2 = fmaf(-fm, s1, r1);
      const float fl = fminf(fmaxf(rintf(r2 * i2), -127.f), 127.f);
      h[j] = (int)fh, md[j] = (int)fm, lo[j] = (int)fl;
    }
    const int e = i * 128 + lane * 4;
    const uint32_t a = slab + (Q6 ? e : (e >> 5) * X4_SUB + (e & 31));
    sts32(a, pack4(h[0], h[1], h[2], h[3]));
    sts32(a + PLANE, pack4(md[0], md[1], md[2], md[3]));
    sts32(a + 2 * PLANE, pack4(lo[0], lo[1], lo[2], lo[3]));
    float s = (v[0] + v[1]) + (v[2] + v[3]);
#pragma unroll
    for (int o = 1; o < LPS; o <<= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((lane & (LPS - 1)) == 0) asm volatile("st.shared.f32 [%0], %1;\n" ::"r"(slab + SLAB_SX + (Q6 ? (e >> 4) : (e >> 5)) * 4), "f"(s));
  }
  if (lane == 0) asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};\n" ::"r"(slab + SLAB_SC), "f"(s0), "f"(s1), "f"(s2), "f"(up));
}

// Which matrix and which first row a tile of the joint list stands for.  A tile that would run past the
// last row is pulled back to n - 16: it recomputes rows of the tile before it, and the duplicate stores
// write identical values.
__device__ __forceinline__ void resolve_tile(const OpDev *op, int T, int &j, int &r0) {
  if (__ldg(&op->act)) {
    j = T & 1;
    r0 = min((T >> 1) * ROWS, __ldg(&op->n[0]) - ROWS);
    return;
  }
  j = 0;
  int base = 0;
  const int count = __ldg(&op->count);
#pragma unroll
  for (int i = 1; i < 4; i++) {
    const int te = __ldg(&op->tend[i - 1]);
    if (i < count && T >= te) j = i, base = te;
  }
  r0 = min((T - base) * ROWS, __ldg(&op->n[j]) - ROWS);
}

__device__ __forceinline__ float gate_act(float v, int act) {
  return act == 1 ? v / (1.f + expf(-v)) : 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
}

// This CTA's share [t0, t1) of an operator's tile list (whole gate/up pairs when act != 0).
__device__ __forceinline__ void cta_share(int tiles, int act, int &t0, int &t1) {
  const int unit = act ? 2 : 1, lt = tiles / unit;
  t0 = (int)((uint32_t)lt * blockIdx.x / gridDim.x) * unit;
  t1 = (int)((uint32_t)lt * (blockIdx.x + 1) / gridDim.x) * unit;
}

// A block of x into the warp's slab (once per operator when K <= 4096: the warp's block never changes).  All the
// slots a lane needs -- eight of the activations, eight of the residual -- are requested together and checked
// together: one trip to L2 when they are there.  With a norm: the activations are s = x + residual, the writer
// CTA stores s into the sum vector, the slab receives s * weight and the function returns this lane's share of
// sum(s^2) (0 without a norm).
__device__ __forceinline__ float stage_block(const OpDev *op, const Header *hd, uint8_t *arena_me, int b, uint32_t slab, int lane, int world,
                                          unsigned int tag0, unsigned int tag_me, bool writer, int kind, volatile int *abort_flag) {
  const int e0 = b * 256 + lane * 4;
  const float *x_plain = (const float *)__ldg(reinterpret_cast<const unsigned long long *>(&op->x_plain));
  const float *norm_w = (const float *)__ldg(reinterpret_cast<const unsigned long long *>(&op->norm_w));
  const uint32_t x_off = __ldg(&op->x_off), res_off = __ldg(&op->res_off), sum_off = __ldg(&op->sum_off);
  const unsigned int tag_x = tag0 + __ldg(&op->x_tag), tag_r = tag0 + __ldg(&op->res_tag);
  float nrm_ss = 0.f;
  float4 wn[2];
  if (norm_w) wn[0] = __ldg(reinterpret_cast<const float4 *>(norm_w + e0)), wn[1] = __ldg(reinterpret_cast<const float4 *>(norm_w + e0 + 128));
  float4 xv[2];
  const bool has_res = norm_w && res_off != NONE;
  if (x_plain) {
    xv[0] = __ldcg(reinterpret_cast<const float4 *>(x_plain + e0));
    xv[1] = __ldcg(reinterpret_cast<const float4 *>(x_plain + e0 + 128));
  }
  if (!x_plain || has_res) {
    const uint2 *xs = x_plain ? nullptr : reinterpret_cast<const uint2 *>(arena_me + x_off) + e0;
    const uint2 *rs = has_res ? reinterpret_cast<const uint2 *>(arena_me + res_off) + e0 : nullptr;
    uint4 a[4], r[4];
    auto ld16 = [](const uint2 *p) {
      uint4 v;
      asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
      return v;
    };
    unsigned long long ts = 0;
    for (unsigned int it = 1;; it++) {
      bool ok = true;
      if (xs) {
        a[0] = ld16(xs), a[1] = ld16(xs + 2), a[2] = ld16(xs + 128), a[3] = ld16(xs + 130);
#pragma unroll
        for (int i = 0; i < 4; i++) ok = ok && a[i].y == tag_x && a[i].w == tag_x;
      }
      if (rs) {
        r[0] = ld16(rs), r[1] = ld16(rs + 2), r[2] = ld16(rs + 128), r[3] = ld16(rs + 130);
#pragma unroll
        for (int i = 0; i < 4; i++) ok = ok && r[i].y == tag_r && r[i].w == tag_r;
      }
      if (ok) break;
      if ((it & 31u) == 0u && wait_expired(abort_flag, ts)) break;
      __nanosleep(100);  // the polls of 148 x 16 warps share L2 with the weight stream
    }
    if (xs) {
      xv[0] = make_float4(__uint_as_float(a[0].x), __uint_as_float(a[0].z), __uint_as_float(a[1].x), __uint_as_float(a[1].z));
      xv[1] = make_float4(__uint_as_float(a[2].x), __uint_as_float(a[2].z), __uint_as_float(a[3].x), __uint_as_float(a[3].z));
    }
    if (rs) {
      xv[0].x += __uint_as_float(r[0].x), xv[0].y += __uint_as_float(r[0].z), xv[0].z += __uint_as_float(r[1].x), xv[0].w += __uint_as_float(r[1].z);
      xv[1].x += __uint_as_float(r[2].x), xv[1].y += __uint_as_float(r[2].z), xv[1].z += __uint_as_float(r[3].x), xv[1].w += __uint_as_float(r[3].z);
    }
  }
  if (norm_w) {
#pragma unroll
    for (int i = 0; i < 2; i++) {
      const int e = e0 + i * 128;
      if (sum_off != NONE && writer) {
        st_slot(hd, arena_me, world, sum_off, e, xv[i].x, tag_me), st_slot(hd, arena_me, world, sum_off, e + 1, xv[i].y, tag_me);
        st_slot(hd, arena_me, world, sum_off, e + 2, xv[i].z, tag_me), st_slot(hd, arena_me, world, sum_off, e + 3, xv[i].w, tag_me);
      }
      nrm_ss = fmaf(xv[i].x, xv[i].x, fmaf(xv[i].y, xv[i].y, fmaf(xv[i].z, xv[i].z, fmaf(xv[i].w, xv[i].w, nrm_ss))));
      xv[i].x *= wn[i].x, xv[i].y *= wn[i].y, xv[i].z *= wn[i].z, xv[i].w *= wn[i].w;
    }
  }
  __syncwarp();  // every lane is done reading the slab of the block before
  if (kind)
    stage3<true>(xv, slab, lane);
  else
    stage3<false>(xv, slab, lane);
  __syncwarp();
  return nrm_ss;
}

template <bool BULK>
__global__ void __launch_bounds__(CT, 1) chain_kernel(const uint8_t *__restrict__ program, const unsigned int *__restrict__ step) {
  extern __shared__ __align__(128) unsigned char dyn[];
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(dyn);
  const uint32_t ring = sbase + warp * (STAGES * SLOT);
  const uint32_t slab = sbase + RING + warp * SLAB;
  float *red = reinterpret_cast<float *>(dyn + SMEM_RED);
  float *nrm = reinterpret_cast<float *>(dyn + SMEM_NRM);
  const uint32_t bar0 = sbase + SMEM_BAR + warp * (STAGES * 8);
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; s++) umma::mbar_init(bar0 + 8 * s, BULK ? 1u : 32u);
    umma::fence_barrier_init();
  }
  if (threadIdx.x < (ZERO_BYTES + 16) / 4) reinterpret_cast<uint32_t *>(dyn + SMEM_ZERO)[threadIdx.x] = 0u;
  volatile int *abort_flag = reinterpret_cast<volatile int *>(dyn + SMEM_ABORT);
  const uint32_t zpage = sbase + SMEM_ZERO;
  __syncthreads();

  const Header *hd = reinterpret_cast<const Header *>(program);
  const OpDev *ops = reinterpret_cast<const OpDev *>(program + HEADER_BYTES);
  const int n_ops = __ldg(&hd->n_ops), world = __ldg(&hd->world), rank = __ldg(&hd->rank);
  uint8_t *const arena_me = (uint8_t *)__ldg(reinterpret_cast<const unsigned long long *>(&hd->arena[rank]));

  // ---- the weight requests: a cursor over (operator, group of row tiles, K block of this warp, tile), which
  // is exactly the order in which the arithmetic below consumes them, STAGES tiles ahead of it
  int i_op = -1, i_gt = 0, i_t1 = 0, i_gs = 0, i_b = 0, i_rt = 0, i_nb = 0, i_kind = 0, i_slot = 0;
  uint32_t i_rb = 0, i_blk = 144u;
  // this lane's first copy inside a tile, fixed per operator.  Q4_K: lanes 0..26 copy granule lane % 9 of rows
  // 3i + lane / 9, i = 0..4 (consecutive lanes, consecutive bytes), lanes 0..8 also row 15; Q6_K: lanes 0..13 /
  // 16..29 copy one of the 14 granules of rows 2i / 2i+1, i = 0..7
  uint32_t i_so = 0u;
  unsigned long long i_tb = 0;  // lane rt < i_gs: first byte of row tile i_gt + rt of the current group
  auto load_group = [&]() {
    i_tb = 0;
    if (lane < i_gs) {
      const OpDev *op = ops + i_op;
      int j, r0;
      resolve_tile(op, i_gt + lane, j, r0);
      i_tb = __ldg(reinterpret_cast<const unsigned long long *>(&op->w[j])) + (unsigned long long)r0 * i_rb;
    }
  };
  auto next_op = [&]() {  // first operator after i_op in which this warp has tiles
    for (i_op++; i_op < n_ops; i_op++) {
      const OpDev *op = ops + i_op;
      int t0, t1;
      cta_share(__ldg(&op->tiles), __ldg(&op->act), t0, t1);
      i_nb = __ldg(&op->K) >> 8;
      if (t0 < t1 && warp < i_nb) {
        i_kind = __ldg(&op->kind);
        i_blk = i_kind ? 210u : 144u;
        i_rb = (uint32_t)i_nb * i_blk;
        i_so = i_kind ? (uint32_t)(lane >> 4) * i_rb + (uint32_t)(lane & 15) * 16u : (uint32_t)(lane / 9) * i_rb + (uint32_t)(lane % 9) * 16u;
        i_gt = t0, i_t1 = t1, i_gs = min(GROUP, t1 - t0), i_b = warp, i_rt = 0;
        load_group();
        return;
      }
    }
  };
  auto issue = [&]() {
    if (i_op < n_ops) {
    const uint32_t tlo = __shfl_sync(0xffffffffu, (uint32_t)i_tb, i_rt), thi = __shfl_sync(0xffffffffu, (uint32_t)(i_tb >> 32), i_rt);
    const uint8_t *base = reinterpret_cast<const uint8_t *>(((unsigned long long)thi << 32) | tlo) + (uint32_t)i_b * i_blk;
    const uint32_t dst = ring + i_slot * SLOT, bar = bar0 + 8 * i_slot;
    if constexpr (BULK) {
      if (lane == 0) umma::mbar_arrive_expect_tx(bar, (uint32_t)ROWS * (i_kind ? (uint32_t)Q6_COPY : (uint32_t)Q4_PITCH));
      __syncwarp();
      if (lane < ROWS) {
        const uint8_t *src = base + (size_t)lane * i_rb;
        if (i_kind)
          bulk_g2s(dst + lane * Q6_PITCH, (const void *)((uintptr_t)src & ~(uintptr_t)15), Q6_COPY, bar);
        else
          bulk_g2s(dst + lane * Q4_PITCH, src, Q4_PITCH, bar);
      }
    } else {
      if (i_kind) {
        if ((lane & 15) < 14) {
          const uint8_t *src = reinterpret_cast<const uint8_t *>((uintptr_t)base & ~(uintptr_t)15) + i_so;
          uint32_t d = dst + (lane >> 4) * Q6_PITCH + (lane & 15) * 16;
#pragma unroll
          for (int i = 0; i < 8; i++) {
            cp_async16(d, src);
            src += 2u * i_rb, d += 2 * Q6_PITCH;
          }
        }
      } else {
        if (lane < 27) {
          const uint8_t *src = base + i_so;
          const uint32_t d = dst + lane * 16;  // row r' of a triple starts 9 granules after row r' - 1: the tile is dense
#pragma unroll
          for (int i = 0; i < 5; i++) cp_async16(d + i * (3 * Q4_PITCH), src + (size_t)i * (3u * i_rb));
          if (lane < 9) cp_async16(d + 15 * Q4_PITCH, src + (size_t)15u * i_rb);
        }
      }
      cp_async_arrive_noinc(bar);
    }
    if (++i_rt == i_gs) {
      i_rt = 0, i_b += CW;
      if (i_b >= i_nb) {
        i_b = warp, i_gt += i_gs, i_gs = min(GROUP, i_t1 - i_gt);
        if (i_gt >= i_t1)
          next_op();
        else
          load_group();
      }
    }
      }
    i_slot = i_slot + 1 == STAGES ? 0 : i_slot + 1;  // also past the end of the program: the arithmetic's slot index follows this one
  };
  next_op();
#pragma unroll 1
  for (int p = 0; p < STAGES; p++) issue();

  pdl_wait();  // activations and the step word are earlier launches' outputs; the weights requested above are not
  const unsigned int tag0 = (*reinterpret_cast<const volatile unsigned int *>(step)) << 10;
  uint32_t c_phase = 0;  // (the slot consumed next is the slot requested next: i_slot)
  int parity = 0;
  auto slot_wait = [&]() -> uint32_t {  // the next tile of this warp has landed; returns its shared address
    const uint32_t bar = bar0 + 8 * i_slot;
    if (!umma::mbar_test_wait(bar, c_phase)) {
      unsigned long long ts = 0;
      for (unsigned int it = 1; !umma::mbar_test_wait(bar, c_phase); it++)
        if ((it & 255u) == 0u && wait_expired(abort_flag, ts)) break;
    }
    const uint32_t sb = ring + i_slot * SLOT;
    if (i_slot + 1 == STAGES) c_phase ^= 1u;
    return sb;
  };

  const bool hdr_hi = t >= 2;
  const int hdr_sh = (t & 1) * 16;
  // B-fragment addresses inside the slab (see the unit bodies)
  // (lanes whose column is not live in an MMA read the zero page instead)
  const bool own4 = (g >> 1) == t;  // Q4_K: this lane's column belongs to the sub-block pair of A-lane t
  const uint32_t pe1 = own4 ? slab + ((g & 1) ? X4_PLANE : 0) + (2 * t) * X4_SUB : zpage;            // even MMA, (hi | mid) of sub-block 2t
  const uint32_t pe2 = own4 && !(g & 1) ? slab + 2 * X4_PLANE + (2 * t) * X4_SUB : zpage;            // even MMA, lo (column 2t only)
  const uint32_t po1 = own4 ? slab + ((g & 1) ? 0 : X4_PLANE) + (2 * t + 1) * X4_SUB : zpage;        // odd MMA, (mid | hi) of sub-block 2t+1
  const uint32_t po2 = own4 && (g & 1) ? slab + 2 * X4_PLANE + (2 * t + 1) * X4_SUB : zpage;         // odd MMA, lo (column 2t+1 only)
  const uint32_t q6sel = g >> 1;  // Q6_K: the group (0..3) whose sub-blocks this column serves
  const uint32_t p6a = slab + ((g & 1) ? X6_PLANE : 0) + 32 * q6sel + 4 * t;                         // (hi | mid), + 128 h + 16 u
  const uint32_t p6b = (g & 1) ? zpage : slab + 2 * X6_PLANE + 32 * q6sel + 4 * t;                   // lo (even columns only)

  for (int oi = 0; oi < n_ops; oi++) {
    const OpDev *op = ops + oi;
    if (oi + 1 < n_ops && lane == 0) {  // the next operator's record into L1 while this one computes
      asm volatile("prefetch.global.L1 [%0];\n" ::"l"(reinterpret_cast<const uint8_t *>(op + 1)));
      asm volatile("prefetch.global.L1 [%0];\n" ::"l"(reinterpret_cast<const uint8_t *>(op + 1) + 128));
    }
    const int kind = __ldg(&op->kind), K = __ldg(&op->K), act = __ldg(&op->act), nb = K >> 8;
    int t0, t1;
    cta_share(__ldg(&op->tiles), act, t0, t1);
    const bool has_norm = __ldg(reinterpret_cast<const unsigned long long *>(&op->norm_w)) != 0ull;
    const unsigned int tag_me = tag0 + (unsigned)oi + 1u;
    const uint32_t row_bytes = (uint32_t)nb * (kind ? 210u : 144u);
    const bool writer = blockIdx.x == gridDim.x - 1;  // the CTA that always has tiles writes x + residual
    float nrm_ss = 0.f, nrm_inv = 1.f;
    int staged = -1;

    auto stage = [&](int b) {
      nrm_ss += stage_block(op, hd, arena_me, b, slab, lane, world, tag0, tag_me, writer, kind, abort_flag);
      staged = b;
    };
    for (int gt = t0; gt < t1; gt += GROUP, parity ^= 1) {
      const int gs = min(GROUP, t1 - gt);
      // partial sums of this warp: red[parity][warp][tile of the group][row], written by the lanes t == 0 after
      // the four t-lanes of a row have been added up
      float *const my_red = red + ((parity * CW + warp) * GROUP) * ROWS;
      for (int b = warp; b < nb; b += CW) {
        if (b != staged) stage(b);
        const bool first = b == warp;  // the warp's first block of a group overwrites what an earlier group left behind
        auto park = [&](int rt, float v0, float v1) {
          v0 += __shfl_xor_sync(0xffffffffu, v0, 1), v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
          v0 += __shfl_xor_sync(0xffffffffu, v0, 2), v1 += __shfl_xor_sync(0xffffffffu, v1, 2);
          if (t == 0) {
            float *p = my_red + rt * ROWS;
            if (!first) v0 += p[g], v1 += p[g + 8];
            p[g] = v0, p[g + 8] = v1;
          }
        };
        if (kind == 0) {
#pragma unroll 1
          for (int rt = 0; rt < gs; rt++) {
            const uint32_t sb = slot_wait() + g * Q4_PITCH;
            const uint4 h0 = lds128(sb), h1 = lds128(sb + 8 * Q4_PITCH);
            const uint4 qa0 = lds128(sb + 16 + 32 * t), qa1 = lds128(sb + 32 + 32 * t);
            const uint4 qb0 = lds128(sb + 8 * Q4_PITCH + 16 + 32 * t), qb1 = lds128(sb + 8 * Q4_PITCH + 32 + 32 * t);
            __syncwarp();  // the slot is free again
            issue();
            const uint32_t qg[8] = {qa0.x, qa0.y, qa0.z, qa0.w, qa1.x, qa1.y, qa1.z, qa1.w};
            const uint32_t qh[8] = {qb0.x, qb0.y, qb0.z, qb0.w, qb1.x, qb1.y, qb1.z, qb1.w};
            float4 sc;  // s0, s1, s2, up
            asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];\n" : "=f"(sc.x), "=f"(sc.y), "=f"(sc.z), "=f"(sc.w) : "r"(slab + SLAB_SC));
            float de[2], dq[2];
            {  // even sub-block 2t: the low nibbles; elements 8 i .. 8 i + 7 per MMA
              int E[4], E2[4];
#pragma unroll
              for (int i = 0; i < 4; i++) {
                const uint32_t lo = 0x0F0F0F0Fu;
                const uint2 be1 = lds64(pe1 + 8 * i), be2 = lds64(pe2 + 8 * i);
                const uint32_t a0 = qg[2 * i] & lo, a1 = qh[2 * i] & lo, a2 = qg[2 * i + 1] & lo, a3 = qh[2 * i + 1] & lo;
                if (i == 0) {
                  imma_u8s8_first(E, a0, a1, a2, a3, be1.x, be1.y);
                  imma_u8s8_first(E2, a0, a1, a2, a3, be2.x, be2.y);
                } else {
                  imma_u8s8(E, a0, a1, a2, a3, be1.x, be1.y);
                  imma_u8s8(E2, a0, a1, a2, a3, be2.x, be2.y);
                }
              }
              // lane (g, t): E[0], E[1] = row g against (hi, mid); E2[0] against lo; [2], [3] the same for row g+8
              de[0] = fmaf(sc.x, (float)E[0], fmaf(sc.y, (float)E[1], sc.z * (float)E2[0]));
              de[1] = fmaf(sc.x, (float)E[2], fmaf(sc.y, (float)E[3], sc.z * (float)E2[2]));
            }
            {  // odd sub-block 2t+1: the high nibbles, taken as 16 * code
              int O[4], O2[4];
#pragma unroll
              for (int i = 0; i < 4; i++) {
                const uint32_t hi = 0xF0F0F0F0u;
                const uint2 bo1 = lds64(po1 + 8 * i), bo2 = lds64(po2 + 8 * i);
                const uint32_t o0 = qg[2 * i] & hi, o1 = qh[2 * i] & hi, o2 = qg[2 * i + 1] & hi, o3 = qh[2 * i + 1] & hi;
                if (i == 0) {
                  imma_u8s8_first(O, o0, o1, o2, o3, bo1.x, bo1.y);
                  imma_u8s8_first(O2, o0, o1, o2, o3, bo2.x, bo2.y);
                } else {
                  imma_u8s8(O, o0, o1, o2, o3, bo1.x, bo1.y);
                  imma_u8s8(O2, o0, o1, o2, o3, bo2.x, bo2.y);
                }
              }
              // O[1], O[0] = row g against (hi, mid); O2[1] against lo
              dq[0] = fmaf(sc.x, (float)O[1], fmaf(sc.y, (float)O[0], sc.z * (float)O2[1])) * 0.0625f;
              dq[1] = fmaf(sc.x, (float)O[3], fmaf(sc.y, (float)O[2], sc.z * (float)O2[3])) * 0.0625f;
            }
            float dsc[2][2], dmn[2][2];
            q4k_scales(h0, t >= 2, (t & 1) * 16, dsc[0], dmn[0]);
            q4k_scales(h1, t >= 2, (t & 1) * 16, dsc[1], dmn[1]);
            float2 sx;
            asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];\n" : "=f"(sx.x), "=f"(sx.y) : "r"(slab + SLAB_SX + 8 * t));
            const float v0 = fmaf(dsc[0][0], de[0], -dmn[0][0] * sx.x) + fmaf(dsc[0][1], dq[0], -dmn[0][1] * sx.y);
            const float v1 = fmaf(dsc[1][0], de[1], -dmn[1][0] * sx.x) + fmaf(dsc[1][1], dq[1], -dmn[1][1] * sx.y);
            park(rt, v0 * sc.w, v1 * sc.w);
          }
        } else {
          const int n0 = __ldg(&op->n[0]);
          const uintptr_t w0 = (uintptr_t)__ldg(reinterpret_cast<const unsigned long long *>(&op->w[0]));
          // one unit: rows g, g+8 of one tile x one K block; `ODD`: the block starts 2 bytes off a word.  The two
          // 128-element halves of the block are loaded and multiplied one after the other; the slot is released
          // (and requested again) once the second half's words are in registers.
          auto unit6 = [&](auto odd_tag, uint32_t sb, uint32_t skew, float (&vr)[2]) {
            constexpr bool ODD = decltype(odd_tag)::value;
            const uint32_t m0f = 0x0F0F0F0Fu, m30 = 0x30303030u;
            float4 sc;  // s0, s1, s2, up
            asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];\n" : "=f"(sc.x), "=f"(sc.y), "=f"(sc.z), "=f"(sc.w) : "r"(slab + SLAB_SC));
            uint32_t scw[2];
            float dd[2], half0_u1[2];
            vr[0] = vr[1] = 0.f;
#pragma unroll
            for (int h = 0; h < 2; h++) {
              uint32_t wa[2][2], wc[2][2], wh[2][2];  // [row][u]
#pragma unroll
              for (int r = 0; r < 2; r++) {
                const uint32_t blk = sb + (g + 8 * r) * Q6_PITCH + skew;  // the block's first byte
#pragma unroll
                for (int u = 0; u < 2; u++) {
                  wa[r][u] = lds32_at2<ODD>(blk + 4 * (16 * h + 4 * u + t));
                  wc[r][u] = lds32_at2<ODD>(blk + 4 * (16 * h + 8 + 4 * u + t));
                  wh[r][u] = lds32_at2<ODD>(blk + 4 * (32 + 8 * h + 4 * u + t));
                }
                if (h == 1) {
                  scw[r] = lds16u(blk + 192 + 2 * t) | (lds16u(blk + 200 + 2 * t) << 16);  // scales 2t, 2t+1 | 8+2t, 8+2t+1
                  dd[r] = f16_bits_to_f32((uint16_t)lds16u(blk + 208));
                }
              }
              if (h == 1) {
                __syncwarp();  // the slot is free again
                issue();
              }
              int A1[2][4], A2[2][4];
#pragma unroll
              for (int u = 0; u < 2; u++) {
                uint32_t v[4][2];  // [group q][row]: four 6-bit codes as bytes
#pragma unroll
                for (int r = 0; r < 2; r++) {
                  v[0][r] = and_or(wa[r][u], m0f, (wh[r][u] << 4) & m30);
                  v[1][r] = and_or(wc[r][u], m0f, (wh[r][u] << 2) & m30);
                  v[2][r] = and_or(wa[r][u] >> 4, m0f, wh[r][u] & m30);
                  v[3][r] = and_or(wc[r][u] >> 4, m0f, (wh[r][u] >> 2) & m30);
                }
                // the columns of group q = q6sel: (hi | mid) in both sets' first MMA, lo in the second
                const uint32_t x1 = lds32(p6a + 128 * h + 16 * u), x2 = lds32(p6b + 128 * h + 16 * u);
                const uint32_t b0_01 = q6sel == 0 ? x1 : 0u, b1_01 = q6sel == 1 ? x1 : 0u, b0_23 = q6sel == 2 ? x1 : 0u, b1_23 = q6sel == 3 ? x1 : 0u;
                const uint32_t c0_01 = q6sel == 0 ? x2 : 0u, c1_01 = q6sel == 1 ? x2 : 0u, c0_23 = q6sel == 2 ? x2 : 0u, c1_23 = q6sel == 3 ? x2 : 0u;
                imma_u8s8_first(A1[u], v[0][0], v[0][1], v[1][0], v[1][1], b0_01, b1_01);
                imma_u8s8(A1[u], v[2][0], v[2][1], v[3][0], v[3][1], b0_23, b1_23);
                imma_u8s8_first(A2[u], v[0][0], v[0][1], v[1][0], v[1][1], c0_01, c1_01);
                imma_u8s8(A2[u], v[2][0], v[2][1], v[3][0], v[3][1], c0_23, c1_23);
              }
              // lane (g, t): A1[u][0], A1[u][1] = row g, sub-block 8h + 2t + u against (hi, mid); A2[u][0] against lo;
              // [2], [3] the same for row g+8.  Half 0's sums wait for the scales, which arrive with half 1.
              float2 sx;
              asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];\n" : "=f"(sx.x), "=f"(sx.y) : "r"(slab + SLAB_SX + 32 * h + 8 * t));
              float d_[2][2];  // [row][u]
#pragma unroll
              for (int r = 0; r < 2; r++) {
                d_[r][0] = fmaf(-32.f, sx.x, fmaf(sc.x, (float)A1[0][2 * r], fmaf(sc.y, (float)A1[0][2 * r + 1], sc.z * (float)A2[0][2 * r])));
                d_[r][1] = fmaf(-32.f, sx.y, fmaf(sc.x, (float)A1[1][2 * r], fmaf(sc.y, (float)A1[1][2 * r + 1], sc.z * (float)A2[1][2 * r])));
              }
              if (h == 0) {  // kept unscaled until the scales are read
                vr[0] = d_[0][0], vr[1] = d_[1][0], half0_u1[0] = d_[0][1], half0_u1[1] = d_[1][1];
              } else {
#pragma unroll
                for (int r = 0; r < 2; r++) {
                  const float s00 = dd[r] * (float)(int8_t)(scw[r] & 0xff), s01 = dd[r] * (float)(int8_t)((scw[r] >> 8) & 0xff);
                  const float s10 = dd[r] * (float)(int8_t)((scw[r] >> 16) & 0xff), s11 = dd[r] * (float)(int8_t)((scw[r] >> 24) & 0xff);
                  vr[r] = (s00 * vr[r] + s01 * half0_u1[r] + s10 * d_[r][0] + s11 * d_[r][1]) * sc.w;
                }
              }
            }
          };
#pragma unroll 1
          for (int rt = 0; rt < gs; rt++) {
            const uint32_t sb = slot_wait();
            const int r0 = min((gt + rt) * ROWS, n0 - ROWS);
            const uint32_t skew = (uint32_t)((w0 + (size_t)(r0 + g) * row_bytes + (uint32_t)b * 210u) & 15u);
            float vr[2];
            if (skew & 2u)
              unit6(std::true_type{}, sb, skew, vr);
            else
              unit6(std::false_type{}, sb, skew, vr);
            park(rt, vr[0], vr[1]);
          }
        }
      }
      if (has_norm && gt == t0) {
        nrm_ss = warp_sum(nrm_ss);
        if (lane == 0) nrm[(oi & 1) * CW + warp] = warp < nb ? nrm_ss : 0.f;
      }
      __syncthreads();  // also orders this group's reads of red[parity] before its reuse two groups on
      if (has_norm && gt == t0) {
        float tot = 0.f;
#pragma unroll
        for (int i = 0; i < CW; i++) tot += nrm[(oi & 1) * CW + i];
        nrm_inv = (float)(1.0 / sqrt((double)(tot / (float)K) + (double)__ldg(&op->eps)));
      }
      const int nw = nb < CW ? nb : CW;  // warps that hold a partial sum
      auto row_sum = [&](int rt, int row) {
        float v = 0.f;
        for (int wq = 0; wq < nw; wq++) v += red[((parity * CW + wq) * GROUP + rt) * ROWS + row];
        return v * nrm_inv;
      };
      if (act) {
        for (int i = threadIdx.x; i < (gs >> 1) * ROWS; i += CT) {
          const int pr = i >> 4, row = i & 15;
          int j, r0;
          resolve_tile(op, gt + 2 * pr, j, r0);
          const float v = gate_act(row_sum(2 * pr, row), act) * row_sum(2 * pr + 1, row);
          float *o = (float *)__ldg(reinterpret_cast<const unsigned long long *>(&op->out[0]));
          if (o) o[r0 + row] = v;
          const uint32_t off = __ldg(&op->out_off[0]);
          if (off != NONE) st_slot(hd, arena_me, world, off, (size_t)rank * __ldg(&op->n[0]) + r0 + row, v, tag_me);
        }
      } else {
        for (int i = threadIdx.x; i < gs * ROWS; i += CT) {
          const int rt = i >> 4, row = i & 15;
          int j, r0;
          resolve_tile(op, gt + rt, j, r0);
          const float v = row_sum(rt, row);
          float *o = (float *)__ldg(reinterpret_cast<const unsigned long long *>(&op->out[j]));
          if (o) o[r0 + row] = v;
          const uint32_t off = __ldg(&op->out_off[j]);
          if (off != NONE) st_slot(hd, arena_me, world, off, (size_t)rank * __ldg(&op->n[j]) + r0 + row, v, tag_me);
        }
      }
    }
  }
  // Nothing is in flight here (the requests end with the program and every requested tile was waited for) unless
  // a wait gave up: then let the outstanding copies land before the CTA's shared memory goes away.
  if (*abort_flag) {
    const unsigned long long ts = umma::global_ns();
    while (umma::global_ns() - ts < 2000000ull) __nanosleep(1000);
  }
}

__global__ void chain_step_kernel(unsigned int *step) { *step += 1; }

bool g_chain_bulk = false;  // LIGHT_B200_CHAIN_BULK=1: bulk copies (one row piece per lane) instead of 16-byte cp.async copies: measured slower (2.2 against 2.9 TB/s on one large Q4_K matrix)

}  // namespace

// ---- host side: build the device program, launch it

size_t chain_program_bytes(int n_ops) { return HEADER_BYTES + (size_t)n_ops * sizeof(OpDev); }

static uint32_t vec_bytes(long long len) { return (uint32_t)((len * 8 + 255) / 256 * 256); }

// Lengths and offsets of the chain vectors, from the operators that write them.  Returns total arena bytes or -1.
static long long layout_vectors(const lb200_chain_op *ops, int n_ops, int n_vecs, int world, std::vector<long long> &len, std::vector<int> &producer,
                                std::vector<uint32_t> &off) {
  len.assign(n_vecs, 0), producer.assign(n_vecs, -1), off.assign(n_vecs, 0);
  for (int i = 0; i < n_ops; i++) {
    const lb200_chain_op &o = ops[i];
    const int outs = o.act ? 1 : o.count;
    for (int j = 0; j < outs; j++) {
      const int v = o.out_vec[j];
      if (v < 0) continue;
      if (v >= n_vecs) return -1;
      const long long l = (long long)world * o.n[j];
      if (len[v] && len[v] != l) return -1;
      len[v] = l;
    }
    if (o.sum_vec >= 0) {
      if (o.sum_vec >= n_vecs) return -1;
      if (len[o.sum_vec] && len[o.sum_vec] != o.K) return -1;
      len[o.sum_vec] = o.K;
    }
  }
  long long total = 0;
  for (int v = 0; v < n_vecs; v++) {
    if (total > 0xF0000000ll) return -1;
    off[v] = (uint32_t)total;
    total += vec_bytes(len[v]);
  }
  return total;
}

long long chain_arena_bytes(const lb200_chain_op *ops, int n_ops, int n_vecs, int world) {
  std::vector<long long> len;
  std::vector<int> prod;
  std::vector<uint32_t> off;
  const long long t = layout_vectors(ops, n_ops, n_vecs, world, len, prod, off);
  return t < 0 ? -1 : (t < 256 ? 256 : t);
}

int chain_build(const lb200_chain_op *ops, int n_ops, int n_vecs, void *program, size_t program_bytes, void *const *arena, size_t arena_bytes,
                int world, int rank, cudaStream_t st) {
  if (n_ops < 1 || n_ops > 1000) return fail(LB200_E_SHAPE, "light_b200: chain_build: %d operators, want 1..1000", n_ops);
  if (program_bytes < chain_program_bytes(n_ops))
    return fail(LB200_E_SHAPE, "light_b200: chain_build: program buffer of %zu bytes, need %zu", program_bytes, chain_program_bytes(n_ops));
  std::vector<long long> len;
  std::vector<int> prod_unused;
  std::vector<uint32_t> off;
  const long long total = layout_vectors(ops, n_ops, n_vecs, world, len, prod_unused, off);
  if (total < 0) return fail(LB200_E_SHAPE, "light_b200: chain_build: a chain vector index is out of range or written with two lengths");
  if ((long long)arena_bytes < total) return fail(LB200_E_SHAPE, "light_b200: chain_build: arena of %zu bytes, need %lld", arena_bytes, total);
  std::vector<int> tag_of(n_vecs, 0);  // 1 + index of the operator that last wrote the vector, while walking the program
  std::vector<uint8_t> host(chain_program_bytes(n_ops), 0);
  Header *hd = reinterpret_cast<Header *>(host.data());
  for (int p = 0; p < world; p++) hd->arena[p] = (uint8_t *)arena[p];
  hd->n_ops = n_ops, hd->world = world, hd->rank = rank;
  OpDev *dv = reinterpret_cast<OpDev *>(host.data() + HEADER_BYTES);
  for (int i = 0; i < n_ops; i++) {
    const lb200_chain_op &o = ops[i];
    OpDev &d = dv[i];
    if (o.wtype != LB200_Q4_K && o.wtype != LB200_Q6_K) return fail(LB200_E_DTYPE, "light_b200: chain_build: operator %d: ggml type %d (Q4_K and Q6_K only)", i, o.wtype);
    d.kind = o.wtype == LB200_Q6_K;
    if (o.K <= 0 || o.K % 256 || (d.kind && o.K % 2048))
      return fail(LB200_E_SHAPE, "light_b200: chain_build: operator %d: K=%d (Q4_K: a multiple of 256; Q6_K: of 2048)", i, o.K);
    if (o.count < 1 || o.count > 4 || (o.act && o.count != 2) || o.act < 0 || o.act > 2 || (d.kind && o.count != 1))
      return fail(LB200_E_SHAPE, "light_b200: chain_build: operator %d: count=%d act=%d (Q6_K: one matrix; a gate: two)", i, o.count, o.act);
    int tiles = 0;
    for (int j = 0; j < 4; j++) {
      d.out_off[j] = NONE;
      if (j >= o.count) continue;
      if (!o.w[j] || o.n[j] < ROWS) return fail(LB200_E_SHAPE, "light_b200: chain_build: operator %d, matrix %d: null or fewer than 16 rows", i, j);
      if ((uintptr_t)o.w[j] & 15) return fail(LB200_E_ALIGN, "light_b200: chain_build: operator %d, matrix %d: weights misaligned", i, j);
      if (o.act && o.n[j] != o.n[0]) return fail(LB200_E_SHAPE, "light_b200: chain_build: operator %d: gate and up differ in height", i);
      d.w[j] = (const uint8_t *)o.w[j], d.n[j] = o.n[j];
      tiles += (o.n[j] + ROWS - 1) / ROWS;
      d.tend[j] = tiles;
      if (!o.act || j == 0) {
        d.out[j] = o.out[j];
        if (o.out_vec[j] >= 0) d.out_off[j] = off[o.out_vec[j]];
      }
    }
    d.tiles = tiles, d.K = o.K, d.count = o.count, d.act = o.act;
    d.x_plain = o.x, d.x_off = NONE, d.res_off = NONE, d.sum_off = NONE;
    if (!o.x) {
      if (o.x_vec < 0 || o.x_vec >= n_vecs || !tag_of[o.x_vec] || len[o.x_vec] != o.K)
        return fail(LB200_E_SHAPE, "light_b200: chain_build: operator %d: its activations must be a chain vector of %d values written by an earlier operator", i, o.K);
      d.x_off = off[o.x_vec], d.x_tag = (uint32_t)tag_of[o.x_vec];
    }
    d.norm_w = o.norm_weight, d.eps = o.norm_eps;
    if (o.norm_weight) {
      if (o.K > CW * 256) return fail(LB200_E_SHAPE, "light_b200: chain_build: operator %d: a norm needs K <= %d", i, CW * 256);
      if (o.res_vec >= 0) {
        if (o.res_vec >= n_vecs || !tag_of[o.res_vec] || len[o.res_vec] != o.K)
          return fail(LB200_E_SHAPE, "light_b200: chain_build: operator %d: the residual must be a chain vector of %d values written earlier", i, o.K);
        d.res_off = off[o.res_vec], d.res_tag = (uint32_t)tag_of[o.res_vec];
      }
      if (o.sum_vec >= 0) d.sum_off = off[o.sum_vec];
    } else if (o.res_vec >= 0 || o.sum_vec >= 0) {
      return fail(LB200_E_SHAPE, "light_b200: chain_build: operator %d: residual / sum vectors need a norm weight", i);
    }
    // an operator never writes a vector it reads: other CTAs may still be polling the old tag
    for (int j = 0; j < 4; j++) {
      const int ov = j < (o.act ? 1 : o.count) ? o.out_vec[j] : -1;
      if (ov >= 0 && ((!o.x && ov == o.x_vec) || ov == o.res_vec || ov == o.sum_vec))
        return fail(LB200_E_SHAPE, "light_b200: chain_build: operator %d: output %d goes to a vector the operator itself reads or writes", i, j);
    }
    if (o.sum_vec >= 0 && ((!o.x && o.sum_vec == o.x_vec) || o.sum_vec == o.res_vec))
      return fail(LB200_E_SHAPE, "light_b200: chain_build: operator %d: sum_vec is the vector its activations or residual come from", i);
    // what this operator writes carries its tag from here on
    if (o.sum_vec >= 0) tag_of[o.sum_vec] = i + 1;
    for (int j = 0; j < (o.act ? 1 : o.count); j++)
      if (o.out_vec[j] >= 0) tag_of[o.out_vec[j]] = i + 1;
  }
  cudaError_t e = cudaMemcpyAsync(program, host.data(), host.size(), cudaMemcpyHostToDevice, st);
  if (e == cudaSuccess) e = cudaMemsetAsync(arena[rank], 0, arena_bytes, st);
  if (e != cudaSuccess) return fail((int)e, "light_b200: chain_build: %s", cudaGetErrorString(e));
  return 0;
}

int chain_run(const void *program, unsigned int *step, cudaStream_t st) {
  static DeviceOnce attr;
  static bool knob = false;
  if (!knob) {
    if (const char *e = getenv("LIGHT_B200_CHAIN_BULK")) g_chain_bulk = atoi(e) != 0;
    knob = true;
  }
  cudaError_t e = attr.ensure([&] {
    cudaError_t r = cudaFuncSetAttribute(chain_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    return r != cudaSuccess ? r : cudaFuncSetAttribute(chain_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  });
  if (e != cudaSuccess) return fail((int)e, "light_b200: chain_run: %s", cudaGetErrorString(e));
  chain_step_kernel<<<1, 1, 0, st>>>(step);
  int rc = launched("chain step");
  if (rc) return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)sm_count());  // one CTA per SM: all of them must be resident at once
  cfg.blockDim = dim3(CT);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  const uint8_t *prog = (const uint8_t *)program;
  const unsigned int *stp = step;
  e = g_chain_bulk ? cudaLaunchKernelEx(&cfg, chain_kernel<true>, prog, stp) : cudaLaunchKernelEx(&cfg, chain_kernel<false>, prog, stp);
  if (e != cudaSuccess) return fail((int)e, "light_b200: chain_run: %s", cudaGetErrorString(e));
  return launched("decode chain");
}

int chain_status() {
  unsigned int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_chain_status, sizeof(v));
  if (e != cudaSuccess) return fail((int)e, "light_b200: chain_status: %s", cudaGetErrorString(e));
  return (int)v;
}

}  // namespace lb
