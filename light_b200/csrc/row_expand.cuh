// Row expanders shared by the tensor-core kernels: one thread owns one weight row and turns its packed
// codes into the 16-bit operand values of a (rows x 64 k) shared-memory tile in the 128-byte swizzle
// layout that tcgen05.mma reads (rows of 128 bytes, 16-byte chunk c of row r stored at c ^ (r & 7)).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>

#include "common.cuh"
#include "mma_sync.cuh"

namespace lb {
namespace {

// Byte offset of 16-byte chunk `c` of row `r` inside a swizzled (rows x 64 f16) tile.
__device__ __forceinline__ uint32_t swz(int r, int c) { return (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4)); }

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&h);
}
// two f32 -> one register of two f16 (BF16 = false) or two bf16 (BF16 = true), round to nearest even
template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  if (BF16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
  }
  return pack_h2(a, b);
}
// byte i of `bytes` as f32 (0 .. 255), exact, without the conversion pipe
__device__ __forceinline__ float byte_f32(uint32_t bytes, int i) {
  return __uint_as_float(__byte_perm(bytes, 0x4B000000u, 0x7650 + i)) - 8388608.f;
}
// four code bytes -> four weights code * s - m (one f32 FMA, one rounding), as two packed registers
template <bool BF16>
__device__ __forceinline__ void expand4(uint32_t bytes, float s, float m, uint32_t &o0, uint32_t &o1) {
  o0 = pack2<BF16>(fmaf(byte_f32(bytes, 0), s, -m), fmaf(byte_f32(bytes, 1), s, -m));
  o1 = pack2<BF16>(fmaf(byte_f32(bytes, 2), s, -m), fmaf(byte_f32(bytes, 3), s, -m));
}
// asks for the 128-byte lines [p, p + bytes) to be brought into L2 (no register, no wait)
__device__ __forceinline__ void prefetch_l2(const void *p, int bytes) {
  const uintptr_t a = (uintptr_t)p & ~(uintptr_t)127, e = (uintptr_t)p + bytes;
  for (uintptr_t q = a; q < e; q += 128) asm volatile("prefetch.global.L2 [%0];\n" ::"l"(q));
}
__device__ __forceinline__ void st_chunk(uint32_t addr, const uint4 &v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w));
}

// ---- per-format row expanders: one thread, one weight row, one 256-element block at a time.
// load(): fetch the block into registers.  step(j, ...): write the 64 weights k = 64j .. 64j+63 of
// the block as 8 swizzled 16-byte chunks of row `r` of the B tile at shared address `tile`
// (PART 0 / 1: only chunks 0-3 / 4-7, for two threads that share a row; 2: all eight).
struct GgufCtx {
  const uint8_t *w;
};
// The expansion runs on packed f16 pairs.  One LOP3 turns two nibbles of a code word into the f16
// pair (1024 + q, 1024 + q') (low nibbles of bytes 0 and 2) or (64 + q, 64 + q') (high nibbles); one
// HFMA2 with the sub-block's 6-bit scale gives q * sc exactly (an integer below 2048), and a second
// one d * (q * sc) - dmin * m with a single rounding of the weight (dmin * m itself is rounded to
// f16 once per sub-block).  A code word yields the pairs (0, 2) and (1, 3) of its four bytes, so
// the activations are stored with every four consecutive k in the order 0, 2, 1, 3 (KPERM) and no
// instruction is spent on putting the weights back in order.
struct Q4KRow {
  using Ctx = GgufCtx;
  static constexpr int STEPS = 4;  // one load() = one 256-element block = 4 steps of 64
  static constexpr bool KPERM = true;
  const uint8_t *row;
  uint4 h, q[8];
  __device__ __forceinline__ void init(const Ctx &c, int e, int n, int N, int K) {
    row = c.w + ((size_t)e * N + n) * (size_t)(K / 256) * 144;
  }
  __device__ __forceinline__ void load(int kb) {
    const uint4 *p = reinterpret_cast<const uint4 *>(row) + (size_t)kb * 9;
    h = __ldg(p);
#pragma unroll
    for (int i = 0; i < 8; i++) q[i] = __ldg(p + 1 + i);
  }
  __device__ __forceinline__ void prefetch(int kb) const { prefetch_l2(row + (size_t)kb * 144, 144); }
  // Staged path: the 256-element block `b` of this row is the RAW_G 16-byte granules at raw_src(b);
  // a kernel copies them (coalesced, asynchronously) to RAW_PITCH-byte row slots in shared memory,
  // and load_smem() fetches a load unit from the row's slot instead of from global memory.
  static constexpr int RAW_G = 9, RAW_PITCH = 144;
  __device__ __forceinline__ const uint8_t *raw_end() const { return nullptr; }  // granules never pass the end
  __device__ __forceinline__ const uint8_t *raw_src(int b) const { return row + (size_t)b * 144; }
  __device__ __forceinline__ const uint8_t *raw_src_unaligned(int b) const { return raw_src(b); }
  __device__ __forceinline__ static size_t row_stride(const Ctx &, int K) { return (size_t)(K / 256) * 144; }
  __device__ __forceinline__ void load_smem(uint32_t slot, int) {
    h = lds128(slot);
#pragma unroll
    for (int i = 0; i < 8; i++) q[i] = lds128(slot + 16 + 16 * i);
  }
  __device__ __forceinline__ static uint32_t h2u(__half2 v) { return *reinterpret_cast<uint32_t *>(&v); }
  __device__ __forceinline__ static __half2 u2h(uint32_t v) { return *reinterpret_cast<__half2 *>(&v); }
  template <bool BF16, int PART = 2>
  __device__ __forceinline__ void step(int j, uint32_t tile, int r) const {
    // sub-blocks 2j (low nibbles of qs[32j .. 32j+31]) and 2j+1 (high nibbles)
    const __half2 dd = u2h(h.x);  // (d, dmin)
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
    const __half2 d2 = __low2half2(dd);
    const float dmin = __high2float(dd);
    const __half2 s0 = __half2half2(__uint2half_rn(sc0)), s1 = __half2half2(__uint2half_rn(sc1));
    const __half2 c0 = __hmul2(s0, __float2half2_rn(-1024.f)), c1 = __hmul2(s1, __float2half2_rn(-64.f));  // exact
    const __half2 nm0 = __float2half2_rn(-dmin * (float)mn0), nm1 = __float2half2_rn(-dmin * (float)mn1);
    const uint32_t mlo = 0x000F000Fu, glo = 0x64006400u, mhi = 0x00F000F0u, ghi = 0x54005400u;
    const uint32_t w[8] = {q[2 * j].x, q[2 * j].y, q[2 * j].z, q[2 * j].w, q[2 * j + 1].x, q[2 * j + 1].y, q[2 * j + 1].z, q[2 * j + 1].w};
    auto lo2 = [&](uint32_t v) { return h2u(__hfma2(__hfma2(u2h(and_or(v, mlo, glo)), s0, c0), d2, nm0)); };
    auto hi2 = [&](uint32_t v) { return h2u(__hfma2(__hfma2(u2h(and_or(v, mhi, ghi)), s1, c1), d2, nm1)); };
#pragma unroll
    for (int c = 0; c < 4; c++) {  // chunk c: k = 8c..8c+7 (low nibbles); chunk c+4: k = 32+8c.. (high nibbles)
      const uint32_t a = w[2 * c], b = w[2 * c + 1], a8 = a >> 8, b8 = b >> 8;
      if (PART != 1) st_chunk(tile + swz(r, c), make_uint4(lo2(a), lo2(a8), lo2(b), lo2(b8)));
      if (PART != 0) st_chunk(tile + swz(r, c + 4), make_uint4(hi2(a), hi2(a8), hi2(b), hi2(b8)));
    }
  }
};

// Q6_K (210 B): [ql[128] | qh[64] | int8 sc[16] | f16 d].  One load() fetches a 128-element half h:
// ql[64h .. 64h+63], qh[32h .. 32h+31], sc[8h .. 8h+7], d.  Step j (k = 64j .. 64j+63 of the half)
// covers groups q = 2j, 2j+1: code = (ql[64h + 32(q&1) + l] >> 4j) & 15 | ((qh[32h + l] >> 2q) & 3) << 4,
// weight = d * sc[8h + 4j + k/16] * (code - 32).  Blocks are only 2-byte aligned: each word is two
// aligned 32-bit loads funnel-shifted by 0 or 16 bits (rows start 4-byte aligned, checked on the host).
struct Q6KRow {
  using Ctx = GgufCtx;
  static constexpr bool KPERM = true;
  static constexpr int STEPS = 2;
  const uint8_t *row;
  uint32_t ql[16], qh[8], sc[2];
  float d;
  const uint8_t *end;  // one past the last byte of the matrix: the granule copies stop there
  __device__ __forceinline__ void init(const Ctx &c, int e, int n, int N, int K) {
    row = c.w + ((size_t)e * N + n) * (size_t)(K / 256) * 210;
    end = c.w + ((size_t)e + 1) * N * (size_t)(K / 256) * 210;
  }
  __device__ __forceinline__ const uint8_t *raw_end() const { return end; }
  __device__ __forceinline__ static uint32_t ld(const uint32_t *a, uint32_t sh) {
    const uint32_t lo = __ldg(a);
    uint32_t hi = 0;
    if (sh) hi = __ldg(a + 1);
    return __funnelshift_r(lo, hi, sh);
  }
  __device__ __forceinline__ void prefetch(int unit) const {
    if (!(unit & 1)) prefetch_l2(row + (size_t)(unit >> 1) * 210, 210);
  }
  // staged path: the block's 210 bytes lie `skew` bytes into the 14 granules that cover them
  static constexpr int RAW_G = 14, RAW_PITCH = 240;
  __device__ __forceinline__ const uint8_t *raw_src(int b) const {
    return reinterpret_cast<const uint8_t *>((uintptr_t)(row + (size_t)b * 210) & ~(uintptr_t)15);
  }
  __device__ __forceinline__ const uint8_t *raw_src_unaligned(int b) const { return row + (size_t)b * 210; }
  __device__ __forceinline__ static size_t row_stride(const Ctx &, int K) { return (size_t)(K / 256) * 210; }
  __device__ __forceinline__ static uint32_t lds_sh(uint32_t a, uint32_t sh) {
    uint32_t lo, hi = 0;
    asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(lo) : "r"(a));
    if (sh) asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(hi) : "r"(a + 4));
    return __funnelshift_r(lo, hi, sh);
  }
  __device__ __forceinline__ void load_smem(uint32_t slot, int unit) {
    const int b = unit >> 1, h = unit & 1;
    const uint32_t skew = (uint32_t)((uintptr_t)(row + (size_t)b * 210) & 15);
    const uint32_t a = slot + (skew & ~3u), sh = (skew & 2u) * 8u;
#pragma unroll
    for (int i = 0; i < 16; i++) ql[i] = lds_sh(a + 4 * (16 * h + i), sh);
#pragma unroll
    for (int i = 0; i < 8; i++) qh[i] = lds_sh(a + 4 * (32 + 8 * h + i), sh);
    sc[0] = lds_sh(a + 4 * (48 + 2 * h), sh), sc[1] = lds_sh(a + 4 * (49 + 2 * h), sh);
    uint16_t dh;
    asm volatile("ld.shared.u16 %0, [%1];\n" : "=h"(dh) : "r"(slot + skew + 208));
    d = f16_bits_to_f32(dh);
  }
  __device__ __forceinline__ void load(int unit) {
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
  // Packed f16 arithmetic as in the Q4_K expander: PRMT builds (1024 + code) pairs of bytes (0, 2)
  // and (1, 3), one HADD2 takes 1056 off (code - 32, exact), one HMUL2 applies d * sc rounded to f16.
  template <bool BF16, int PART = 2>
  __device__ __forceinline__ void step(int j, uint32_t tile, int r) const {
    const __half2 off = __float2half2_rn(-1056.f);
#pragma unroll
    for (int c = (PART == 1 ? 4 : 0); c < (PART == 0 ? 4 : 8); c++) {  // chunk c: k = 8c .. 8c+7 -> group q = 2j + c/4, l = 8 (c%4) ..
      const int q = 2 * j + (c >> 2), li = 2 * (c & 3);
      const __half2 ds = __float2half2_rn(d * (float)(int8_t)((sc[j] >> (8 * (c >> 1))) & 0xff));
      uint32_t o[4];
#pragma unroll
      for (int e = 0; e < 2; e++) {
        const uint32_t wq = ql[8 * (c >> 2) + li + e] >> (4 * j), wh = qh[li + e];
        const uint32_t hi2 = q == 0 ? (wh << 4) : q == 1 ? (wh << 2) : q == 2 ? wh : (wh >> 2);
        const uint32_t v = and_or(wq, 0x0F0F0F0Fu, hi2 & 0x30303030u);
        const uint32_t p02 = __byte_perm(v, 0x64646464u, 0x4240), p13 = __byte_perm(v, 0x64646464u, 0x4341);
        const __half2 w02 = __hmul2(__hadd2(*reinterpret_cast<const __half2 *>(&p02), off), ds);
        const __half2 w13 = __hmul2(__hadd2(*reinterpret_cast<const __half2 *>(&p13), off), ds);
        o[2 * e] = *reinterpret_cast<const uint32_t *>(&w02), o[2 * e + 1] = *reinterpret_cast<const uint32_t *>(&w13);
      }
      st_chunk(tile + swz(r, c), make_uint4(o[0], o[1], o[2], o[3]));
    }
  }
};

// Q8_0 (34 B per 32 elements): [f16 d | int8 q[32]], blocks only 2-byte aligned.  One load() fetches 128
// elements = 4 blocks = 136 bytes as 34 aligned words (rows start 4-byte aligned, checked on the host, and
// 136 is a multiple of 8); block i of the unit starts 34 i bytes in, so its codes sit on word boundaries
// for odd i and 16 bits into a word for even i: a funnel shift known at compile time.  Packed f16
// arithmetic: XOR 0x80 makes the codes unsigned, PRMT builds (1024 + 128 + q) pairs in natural order, one
// HADD2 takes 1152 off (q, exact), one HMUL2 applies d: the weight fl16(d q), one rounding.
struct Q80Row {
  using Ctx = GgufCtx;
  static constexpr bool KPERM = false;
  static constexpr int STEPS = 2;
  const uint8_t *row;
  uint32_t w[34];
  __device__ __forceinline__ void init(const Ctx &c, int e, int n, int N, int K) {
    row = c.w + ((size_t)e * N + n) * (size_t)(K / 32) * 34;
  }
  __device__ __forceinline__ void load(int unit) {
    const uint32_t *p = reinterpret_cast<const uint32_t *>(row + (size_t)unit * 136);
#pragma unroll
    for (int i = 0; i < 34; i++) w[i] = __ldg(p + i);
  }
  __device__ __forceinline__ void prefetch(int unit) const {
    if (!(unit & 1)) prefetch_l2(row + (size_t)(unit >> 1) * 272, 272);
  }
  // staged path: a 256-element run is 272 bytes = 17 granules (rows are 16-byte aligned when K % 256 == 0)
  static constexpr int RAW_G = 17, RAW_PITCH = 304;
  __device__ __forceinline__ const uint8_t *raw_end() const { return nullptr; }
  __device__ __forceinline__ const uint8_t *raw_src(int b) const { return row + (size_t)b * 272; }
  __device__ __forceinline__ const uint8_t *raw_src_unaligned(int b) const { return raw_src(b); }
  __device__ __forceinline__ static size_t row_stride(const Ctx &, int K) { return (size_t)(K / 32) * 34; }
  __device__ __forceinline__ void load_smem(uint32_t slot, int unit) {
    const uint32_t a = slot + (uint32_t)(unit & 1) * 136u;
#pragma unroll
    for (int i = 0; i < 34; i++) w[i] = lds32(a + 4 * i);
  }
  template <bool BF16, int PART = 2>
  __device__ __forceinline__ void step(int j, uint32_t tile, int r) const {
    const __half2 off = __float2half2_rn(-1152.f);
#pragma unroll
    for (int c = (PART == 1 ? 4 : 0); c < (PART == 0 ? 4 : 8); c++) {  // chunk c: k = 8c .. 8c+7 of block 2j + c/4
      const int bi = 2 * j + (c >> 2), byte0 = 34 * bi, qw = (byte0 + 2) / 4 + 2 * (c & 3);
      const uint32_t dw = w[byte0 / 4];
      const __half dh = (byte0 & 2) ? __ushort_as_half((unsigned short)(dw >> 16)) : __ushort_as_half((unsigned short)(dw & 0xFFFFu));
      const __half2 d2 = __half2half2(dh);
      uint32_t o[4];
#pragma unroll
      for (int e = 0; e < 2; e++) {
        const uint32_t raw = (bi & 1) ? w[qw + e] : __funnelshift_r(w[qw + e], w[qw + e + 1], 16);
        const uint32_t u = raw ^ 0x80808080u;
        const uint32_t p01 = __byte_perm(u, 0x64646464u, 0x5140), p23 = __byte_perm(u, 0x64646464u, 0x7362);
        const __half2 w01 = __hmul2(__hadd2(*reinterpret_cast<const __half2 *>(&p01), off), d2);
        const __half2 w23 = __hmul2(__hadd2(*reinterpret_cast<const __half2 *>(&p23), off), d2);
        o[2 * e] = *reinterpret_cast<const uint32_t *>(&w01), o[2 * e + 1] = *reinterpret_cast<const uint32_t *>(&w23);
      }
      st_chunk(tile + swz(r, c), make_uint4(o[0], o[1], o[2], o[3]));
    }
  }
};

// Group-quantized int4 in the reference's canonical layout (quant/int4.go:12-31): codes u32 (N, K/8),
// nibble i of word c = element 8c + i; scales / zeros f32 (N, K/G).  W = fl(s * fl(code - z)): the two
// f32 roundings of the reference's dequantize kernel (kernels/cuda/src/int4.cu:16-41), then one
// rounding to the operand type, so a bf16 operand equals the reference's bf16 weight bit for bit.
// One load() = 256 elements (32 code words); requires G % 64 == 0.
struct Int4Ctx {
  const uint32_t *codes;
  const float *s, *z;
  int G;
};
struct Int4Row {
  using Ctx = Int4Ctx;
  static constexpr bool KPERM = false;
  static constexpr int STEPS = 4;
  const uint4 *row;
  const float *sr, *zr;
  int G, unit;
  uint4 q[8];
  __device__ __forceinline__ void init(const Ctx &c, int e, int n, int N, int K) {
    const size_t r = (size_t)e * N + n;
    row = reinterpret_cast<const uint4 *>(c.codes + r * (K / 8));
    sr = c.s + r * (K / c.G), zr = c.z + r * (K / c.G), G = c.G;
  }
  __device__ __forceinline__ void prefetch(int u) const { prefetch_l2(row + (size_t)u * 8, 128); }
  static constexpr int RAW_G = 8, RAW_PITCH = 144;  // 128 bytes of codes; the odd pitch spreads the rows over the banks
  __device__ __forceinline__ const uint8_t *raw_end() const { return nullptr; }
  __device__ __forceinline__ const uint8_t *raw_src(int b) const { return reinterpret_cast<const uint8_t *>(row + (size_t)b * 8); }
  __device__ __forceinline__ const uint8_t *raw_src_unaligned(int b) const { return raw_src(b); }
  __device__ __forceinline__ static size_t row_stride(const Ctx &, int K) { return (size_t)(K / 8) * 4; }
  __device__ __forceinline__ void load_smem(uint32_t slot, int u) {
    unit = u;
#pragma unroll
    for (int i = 0; i < 8; i++) q[i] = lds128(slot + 16 * i);
  }
  __device__ __forceinline__ void load(int u) {
    unit = u;
#pragma unroll
    for (int i = 0; i < 8; i++) q[i] = __ldg(row + (size_t)u * 8 + i);
  }
  template <bool BF16, int PART = 2>
  __device__ __forceinline__ void step(int j, uint32_t tile, int r) const {
    const int grp = (unit * 256 + j * 64) / G;
    const float sc = __ldg(sr + grp), z = __ldg(zr + grp);
    const uint32_t w[8] = {q[2 * j].x, q[2 * j].y, q[2 * j].z, q[2 * j].w, q[2 * j + 1].x, q[2 * j + 1].y, q[2 * j + 1].z, q[2 * j + 1].w};
#pragma unroll
    for (int c = (PART == 1 ? 4 : 0); c < (PART == 0 ? 4 : 8); c++) {  // chunk c = code word c: nibbles 0..7 in element order
      const uint32_t lo = w[c] & 0x0F0F0F0Fu, hi = (w[c] >> 4) & 0x0F0F0F0Fu;  // even / odd nibbles
      uint4 o;
      o.x = pack2<BF16>(__fmul_rn(sc, __fsub_rn(byte_f32(lo, 0), z)), __fmul_rn(sc, __fsub_rn(byte_f32(hi, 0), z)));
      o.y = pack2<BF16>(__fmul_rn(sc, __fsub_rn(byte_f32(lo, 1), z)), __fmul_rn(sc, __fsub_rn(byte_f32(hi, 1), z)));
      o.z = pack2<BF16>(__fmul_rn(sc, __fsub_rn(byte_f32(lo, 2), z)), __fmul_rn(sc, __fsub_rn(byte_f32(hi, 2), z)));
      o.w = pack2<BF16>(__fmul_rn(sc, __fsub_rn(byte_f32(lo, 3), z)), __fmul_rn(sc, __fsub_rn(byte_f32(hi, 3), z)));
      st_chunk(tile + swz(r, c), o);
    }
  }
};

// Block-scaled FP8: e4m3fn codes (N, K), one f32 scale per (bR x bC) block; W = fl(f32(code) * scale)
// (kernels/cuda/src/fp8_block.cu:34-62), then one rounding to the operand type.  One load() = 128
// elements; requires bC % 64 == 0.
struct Fp8Ctx {
  const uint8_t *w;
  const float *scale;
  int bR, bC;
};
struct Fp8Row {
  using Ctx = Fp8Ctx;
  static constexpr bool KPERM = false;
  static constexpr int STEPS = 2;
  const uint4 *row;
  const float *sr;
  int bC, unit;
  uint4 q[8];
  __device__ __forceinline__ void init(const Ctx &c, int e, int n, int N, int K) {
    row = reinterpret_cast<const uint4 *>(c.w + ((size_t)e * N + n) * K);
    sr = c.scale + ((size_t)e * (N / c.bR) + n / c.bR) * (K / c.bC), bC = c.bC;
  }
  __device__ __forceinline__ void prefetch(int u) const { prefetch_l2(row + (size_t)u * 8, 128); }
  static constexpr int RAW_G = 16, RAW_PITCH = 272;  // 256 codes = two load units of 128
  __device__ __forceinline__ const uint8_t *raw_end() const { return nullptr; }
  __device__ __forceinline__ const uint8_t *raw_src(int b) const { return reinterpret_cast<const uint8_t *>(row + (size_t)b * 16); }
  __device__ __forceinline__ const uint8_t *raw_src_unaligned(int b) const { return raw_src(b); }
  __device__ __forceinline__ static size_t row_stride(const Ctx &, int K) { return (size_t)K; }
  __device__ __forceinline__ void load_smem(uint32_t slot, int u) {
    unit = u;
#pragma unroll
    for (int i = 0; i < 8; i++) q[i] = lds128(slot + 128 * (u & 1) + 16 * i);
  }
  __device__ __forceinline__ void load(int u) {
    unit = u;
#pragma unroll
    for (int i = 0; i < 8; i++) q[i] = __ldg(row + (size_t)u * 8 + i);
  }
  template <bool BF16>
  __device__ __forceinline__ static uint2 four(uint32_t v, float sc) {
    __half2_raw a = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(v & 0xFFFFu), __NV_E4M3);
    __half2_raw b = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(v >> 16), __NV_E4M3);
    const float2 fa = __half22float2(__half2(a)), fb = __half22float2(__half2(b));
    return make_uint2(pack2<BF16>(__fmul_rn(fa.x, sc), __fmul_rn(fa.y, sc)), pack2<BF16>(__fmul_rn(fb.x, sc), __fmul_rn(fb.y, sc)));
  }
  template <bool BF16, int PART = 2>
  __device__ __forceinline__ void step(int j, uint32_t tile, int r) const {
    const float sc = __ldg(sr + (unit * 128 + j * 64) / bC);
#pragma unroll
    for (int c = (PART == 1 ? 2 : 0); c < (PART == 0 ? 2 : 4); c++) {  // 16 bytes = two chunks of 8 codes
      const uint4 v = q[4 * j + c];
      const uint2 a = four<BF16>(v.x, sc), b = four<BF16>(v.y, sc), e = four<BF16>(v.z, sc), f = four<BF16>(v.w, sc);
      st_chunk(tile + swz(r, 2 * c), make_uint4(a.x, a.y, b.x, b.y));
      st_chunk(tile + swz(r, 2 * c + 1), make_uint4(e.x, e.y, f.x, f.y));
    }
  }
};

// Dense 16-bit weights (bf16 with bf16 operands, f16 with f16 operands): the row is copied as it is.
struct DenseCtx {
  const uint16_t *w;
};
struct DenseRow {
  using Ctx = DenseCtx;
  static constexpr bool KPERM = false;
  static constexpr int STEPS = 1;
  const uint4 *row;
  uint4 q[8];
  __device__ __forceinline__ void init(const Ctx &c, int e, int n, int N, int K) {
    row = reinterpret_cast<const uint4 *>(c.w + ((size_t)e * N + n) * K);
  }
  __device__ __forceinline__ void prefetch(int u) const { prefetch_l2(row + (size_t)u * 8, 128); }
  __device__ __forceinline__ void load(int u) {
#pragma unroll
    for (int i = 0; i < 8; i++) q[i] = __ldg(row + (size_t)u * 8 + i);
  }
  template <bool BF16, int PART = 2>
  __device__ __forceinline__ void step(int, uint32_t tile, int r) const {
#pragma unroll
    for (int c = (PART == 1 ? 4 : 0); c < (PART == 0 ? 4 : 8); c++) st_chunk(tile + swz(r, c), q[c]);
  }
};

}  // namespace
}  // namespace lb
