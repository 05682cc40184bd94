// Batched decode: fused dequant-matmul for 2 .. 16 activation rows (tokens) per launch, Q4_K and Q6_K.
//
// Same decomposition as the single-row kernels (a warp owns a 256-element K block and walks down row
// tiles of 16; a CTA covers all of K and reduces through shared memory), but the eight MMA columns
// are now eight TOKENS, so the weights are expanded completely before the MMA: every code becomes
// w = code * (d*sc) - dmin*m in f32, is rounded once to f16 and lands directly in the A fragment
// registers.  The activations are rounded to f16 once per K block into a per-warp shared slab.
// One pass over the weights serves up to 16 tokens; the instruction count per weight is that of
// the expansion (about 1.4x the single-row kernel) plus one MMA per 8 tokens.
#include "common.cuh"
#include "mma_sync.cuh"

namespace lb {

namespace {

constexpr int WARPS = 8, ROWS = 16, MAX_RT = 2, MAX_NT = 2;
constexpr int TOK_STRIDE = 544;               // bytes per token in the slab: 512 of f16 + 32 pad (8 banks)
constexpr int SLAB_BYTES = 8 * MAX_NT * TOK_STRIDE;
constexpr int SMEM_BYTES = WARPS * SLAB_BYTES + WARPS * MAX_RT * MAX_NT * 32 * 16;

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&h);
}
// four code bytes -> four f16 weights code * s - m, as (e0, e1), (e2, e3)
__device__ __forceinline__ void expand4(uint32_t bytes, float s, float m, uint32_t &o0, uint32_t &o1) {
  const float f0 = __uint_as_float(__byte_perm(bytes, 0x4B000000u, 0x7650)) - 8388608.f;
  const float f1 = __uint_as_float(__byte_perm(bytes, 0x4B000000u, 0x7651)) - 8388608.f;
  const float f2 = __uint_as_float(__byte_perm(bytes, 0x4B000000u, 0x7652)) - 8388608.f;
  const float f3 = __uint_as_float(__byte_perm(bytes, 0x4B000000u, 0x7653)) - 8388608.f;
  o0 = pack_h2(fmaf(f0, s, -m), fmaf(f1, s, -m));
  o1 = pack_h2(fmaf(f2, s, -m), fmaf(f3, s, -m));
}

// Rounds block b of x (tokens m < M, 256 elements each) to f16 into the warp's slab.  PAIR: Q4_K
// layout, the 64 elements of sub-block pair p at p * 136 bytes (banks: 2 words per pair); otherwise
// natural order.  Tokens beyond M are zero.
template <bool PAIR>
__device__ __forceinline__ void stage_tokens(const float *__restrict__ x, int M, int K, int b, int ntok, uint32_t slab,
                                             int lane) {
  for (int i = lane; i < ntok * 64; i += 32) {
    const int tok = i >> 6, e = (i & 63) * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (tok < M) v = __ldg(reinterpret_cast<const float4 *>(x + (size_t)tok * K + b * 256 + e));
    const uint32_t off = PAIR ? (e >> 6) * 136 + (e & 63) * 2 : e * 2;
    sts64(slab + tok * TOK_STRIDE + off, pack_h2(v.x, v.y), pack_h2(v.z, v.w));
  }
}

// red[warp][rt][nt][lane] float4 = D fragment (row g: tokens 2t, 2t+1; row g+8: tokens 2t, 2t+1)
__device__ __forceinline__ void flush(const float (&d)[4], uint32_t addr) {
  float4 o;
  asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];\n" : "=f"(o.x), "=f"(o.y), "=f"(o.z), "=f"(o.w) : "r"(addr));
  o.x += d[0], o.y += d[1], o.z += d[2], o.w += d[3];
  asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};\n" ::"r"(addr), "f"(o.x), "f"(o.y), "f"(o.z), "f"(o.w));
}

__device__ __forceinline__ void reduce_store(const float4 *red, float *__restrict__ out, int n0, int M, int N, int RT,
                                             int NT) {
  __syncthreads();
  // one thread per (token, row): sum the warps in a fixed order
  for (int i = threadIdx.x; i < NT * 8 * RT * ROWS; i += WARPS * 32) {
    const int tok = i / (RT * ROWS), rr = i % (RT * ROWS), rt = rr >> 4, row = rr & 15;
    if (tok < M && n0 + rr < N) {
      const int nt = tok >> 3, tt = (tok & 7) >> 1, odd = tok & 1, g = row & 7, hi = row >> 3;
      float v = 0.f;
#pragma unroll
      for (int wq = 0; wq < WARPS; wq++) {
        const float4 f = red[((wq * MAX_RT + rt) * MAX_NT + nt) * 32 + g * 4 + tt];
        v += hi ? (odd ? f.w : f.z) : (odd ? f.y : f.x);
      }
      out[(size_t)tok * N + n0 + rr] = v;
    }
  }
}

// ------------------------------------------------------------------------------------ Q4_K
// Lane (g, t) holds the 32 code bytes of pair t of rows g and g+8.  Code word i (bytes 4i..4i+3) gives
// one MMA for sub-block 2t (low nibbles) and one for 2t+1 (high nibbles): k slots (2t, 2t+1 | 2t+8,
// 2t+9) <-> elements 4i .. 4i+3 of that sub-block, so the B lane (token, t) reads 8 bytes of x at
// pair t, element 4i (+32 for the high-nibble sub-block).
__device__ __forceinline__ void q4k_scale4(const uint4 &h, bool hi, int sh, float (&dsc)[2], float (&dmn)[2]) {
  const float2 df = __half22float2(*reinterpret_cast<const __half2 *>(&h.x));
  const uint32_t scw = hi ? ((h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u)) : (h.y & 0x3F3F3F3Fu);
  const uint32_t mnw = hi ? (((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u)) : (h.z & 0x3F3F3F3Fu);
  const uint32_t s2 = scw >> sh, m2 = mnw >> sh;
  dsc[0] = df.x * (float)(s2 & 0xFFu), dsc[1] = df.x * (float)((s2 >> 8) & 0xFFu);
  dmn[0] = df.y * (float)(m2 & 0xFFu), dmn[1] = df.y * (float)((m2 >> 8) & 0xFFu);
}

__global__ void __launch_bounds__(WARPS * 32, 2) q4k_gemv_batch_kernel(const float *__restrict__ x,
                                                                      const uint8_t *__restrict__ w,
                                                                      float *__restrict__ out, int M, int N, int K, int RT) {
  extern __shared__ __align__(16) unsigned char dsm[];
  unsigned char *slabs = dsm;
  float4 *red = reinterpret_cast<float4 *>(dsm + WARPS * SLAB_BYTES);
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int nb = K >> 8, NT = (M + 7) >> 3;
  const int n0 = blockIdx.x * (ROWS * RT), last = N - 1;
  const uint32_t row_u4 = (uint32_t)nb * 9;
  const uint4 *w4 = reinterpret_cast<const uint4 *>(w);
  for (int i = lane; i < MAX_RT * MAX_NT * 32; i += 32) red[warp * MAX_RT * MAX_NT * 32 + i] = make_float4(0.f, 0.f, 0.f, 0.f);
  const uint32_t slab = (uint32_t)__cvta_generic_to_shared(slabs + warp * SLAB_BYTES);
  const uint32_t red_lane = (uint32_t)__cvta_generic_to_shared(red + warp * MAX_RT * MAX_NT * 32 + lane);
  const uint32_t pb = slab + g * TOK_STRIDE + t * 136;  // token g of a tile, pair t
  const bool hdr_hi = t >= 2;
  const int hdr_sh = (t & 1) * 16;
  pdl_wait();
  __syncthreads();
  for (int b = warp; b < nb; b += WARPS) {
    __syncwarp();
    stage_tokens<true>(x, M, K, b, NT * 8, slab, lane);
    __syncwarp();
    for (int rt = 0; rt < RT; rt++) {
      const int rg = min(n0 + rt * ROWS + g, last), rg8 = min(n0 + rt * ROWS + g + 8, last);
      const uint4 *pg = w4 + (size_t)((uint32_t)rg * row_u4 + (uint32_t)b * 9u);
      const uint4 *pg8 = w4 + (size_t)((uint32_t)rg8 * row_u4 + (uint32_t)b * 9u);
      const uint4 h0 = __ldg(pg), h1 = __ldg(pg8);
      const uint4 qa0 = __ldg(pg + 1 + 2 * t), qa1 = __ldg(pg + 2 + 2 * t);
      const uint4 qb0 = __ldg(pg8 + 1 + 2 * t), qb1 = __ldg(pg8 + 2 + 2 * t);
      float s0[2], m0[2], s1[2], m1[2];
      q4k_scale4(h0, hdr_hi, hdr_sh, s0, m0);
      q4k_scale4(h1, hdr_hi, hdr_sh, s1, m1);
      float d[MAX_NT][4];
#pragma unroll
      for (int nt = 0; nt < MAX_NT; nt++) d[nt][0] = d[nt][1] = d[nt][2] = d[nt][3] = 0.f;
      const uint32_t qg[8] = {qa0.x, qa0.y, qa0.z, qa0.w, qa1.x, qa1.y, qa1.z, qa1.w};
      const uint32_t qh[8] = {qb0.x, qb0.y, qb0.z, qb0.w, qb1.x, qb1.y, qb1.z, qb1.w};
#pragma unroll
      for (int i = 0; i < 8; i++) {
        uint32_t a[4], c[4];
        expand4(qg[i] & 0x0F0F0F0Fu, s0[0], m0[0], a[0], a[2]);          // row g, sub-block 2t
        expand4(qh[i] & 0x0F0F0F0Fu, s1[0], m1[0], a[1], a[3]);          // row g+8
        expand4((qg[i] >> 4) & 0x0F0F0F0Fu, s0[1], m0[1], c[0], c[2]);   // row g, sub-block 2t+1
        expand4((qh[i] >> 4) & 0x0F0F0F0Fu, s1[1], m1[1], c[1], c[3]);
#pragma unroll
        for (int nt = 0; nt < MAX_NT; nt++) {
          if (nt < NT) {
            const uint2 be = lds64(pb + nt * 8 * TOK_STRIDE + i * 8), bo = lds64(pb + nt * 8 * TOK_STRIDE + 64 + i * 8);
            mma16816(d[nt], a[0], a[1], a[2], a[3], be.x, be.y);
            mma16816(d[nt], c[0], c[1], c[2], c[3], bo.x, bo.y);
          }
        }
      }
#pragma unroll
      for (int nt = 0; nt < MAX_NT; nt++)
        if (nt < NT) flush(d[nt], red_lane + ((rt * MAX_NT + nt) * 32) * 16);
    }
  }
  reduce_store(red, out, n0, M, N, RT, NT);
}

// ------------------------------------------------------------------------------------ Q6_K
// For each (h, u = l / 16), lane (g, t) takes l = 16u + 4t .. +3 of rows g and g+8 (one word of
// ql[64h + l], one of ql[64h + 32 + l], one of qh[32h + l]); group q gives ONE MMA whose 16 k slots
// are sub-block s = 8h + 2q + u, elements 4t .. 4t+3 from lane t.
__device__ __forceinline__ uint32_t ld_u32_sh(const uint32_t *a, uint32_t sh) {
  const uint32_t lo = __ldg(a);
  uint32_t hi = 0;
  if (sh) hi = __ldg(a + 1);
  return __funnelshift_r(lo, hi, sh);
}

__global__ void __launch_bounds__(WARPS * 32, 2) q6k_gemv_batch_kernel(const float *__restrict__ x,
                                                                      const uint8_t *__restrict__ w,
                                                                      float *__restrict__ out, int M, int N, int K, int RT) {
  extern __shared__ __align__(16) unsigned char dsm[];
  unsigned char *slabs = dsm;
  float4 *red = reinterpret_cast<float4 *>(dsm + WARPS * SLAB_BYTES);
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int nb = K >> 8, NT = (M + 7) >> 3;
  const int n0 = blockIdx.x * (ROWS * RT), last = N - 1;
  const uint32_t row_bytes = (uint32_t)nb * 210u;
  for (int i = lane; i < MAX_RT * MAX_NT * 32; i += 32) red[warp * MAX_RT * MAX_NT * 32 + i] = make_float4(0.f, 0.f, 0.f, 0.f);
  const uint32_t slab = (uint32_t)__cvta_generic_to_shared(slabs + warp * SLAB_BYTES);
  const uint32_t red_lane = (uint32_t)__cvta_generic_to_shared(red + warp * MAX_RT * MAX_NT * 32 + lane);
  const uint32_t pb = slab + g * TOK_STRIDE + 8 * t;  // token g of a tile, elements 4t.. of a sub-block
  pdl_wait();
  __syncthreads();
  for (int b = warp; b < nb; b += WARPS) {
    __syncwarp();
    stage_tokens<false>(x, M, K, b, NT * 8, slab, lane);
    __syncwarp();
    const uint32_t sh = (b & 1) * 16u;
    const uint32_t boff = (uint32_t)b * 210u - (b & 1) * 2u;
    for (int rt = 0; rt < RT; rt++) {
      const int rg[2] = {min(n0 + rt * ROWS + g, last), min(n0 + rt * ROWS + g + 8, last)};
      uint32_t wa[2][4], wc[2][4], wh[2][4], scw[2][4];
      float dd[2];
#pragma unroll
      for (int r = 0; r < 2; r++) {
        const uint8_t *base = w + (size_t)rg[r] * row_bytes + boff;
        const uint32_t *blk = reinterpret_cast<const uint32_t *>(base);
        const uint8_t *bb = base + (sh >> 3);
#pragma unroll
        for (int hu = 0; hu < 4; hu++) {
          const int h = hu >> 1, u = hu & 1;
          wa[r][hu] = ld_u32_sh(blk + 16 * h + 4 * u + t, sh);
          wc[r][hu] = ld_u32_sh(blk + 16 * h + 8 + 4 * u + t, sh);
          wh[r][hu] = ld_u32_sh(blk + 32 + 8 * h + 4 * u + t, sh);
        }
#pragma unroll
        for (int i = 0; i < 4; i++) scw[r][i] = ld_u32_sh(blk + 48 + i, sh);  // the 16 int8 scales
        dd[r] = f16_bits_to_f32(__ldg(reinterpret_cast<const uint16_t *>(bb + 208)));
      }
      float d[MAX_NT][4];
#pragma unroll
      for (int nt = 0; nt < MAX_NT; nt++) d[nt][0] = d[nt][1] = d[nt][2] = d[nt][3] = 0.f;
#pragma unroll
      for (int hu = 0; hu < 4; hu++) {
        const int h = hu >> 1, u = hu & 1;
#pragma unroll
        for (int q = 0; q < 4; q++) {
          const int s = 8 * h + 2 * q + u;  // sub-block of this MMA
          uint32_t a[4];
#pragma unroll
          for (int r = 0; r < 2; r++) {
            const float ds = dd[r] * (float)(int8_t)((scw[r][s >> 2] >> (8 * (s & 3))) & 0xff);
            const uint32_t lo4 = (q & 1) ? wc[r][hu] : wa[r][hu];
            const uint32_t nib = (q >> 1) ? (lo4 >> 4) : lo4;
            const uint32_t hi2 = q == 0 ? (wh[r][hu] << 4) : q == 1 ? (wh[r][hu] << 2) : q == 2 ? wh[r][hu] : (wh[r][hu] >> 2);
            expand4((nib & 0x0F0F0F0Fu) | (hi2 & 0x30303030u), ds, 32.f * ds, a[r], a[2 + r]);
          }
#pragma unroll
          for (int nt = 0; nt < MAX_NT; nt++) {
            if (nt < NT) {
              const uint2 bx = lds64(pb + nt * 8 * TOK_STRIDE + s * 32);
              mma16816(d[nt], a[0], a[1], a[2], a[3], bx.x, bx.y);
            }
          }
        }
      }
#pragma unroll
      for (int nt = 0; nt < MAX_NT; nt++)
        if (nt < NT) flush(d[nt], red_lane + ((rt * MAX_NT + nt) * 32) * 16);
    }
  }
  reduce_store(red, out, n0, M, N, RT, NT);
}

template <typename... Args>
int launch_pdl(void (*kern)(Args...), unsigned grid, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(WARPS * 32);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, args...);
  if (e != cudaSuccess) return fail((int)e, "light_b200: matmul_q (batched decode): %s", cudaGetErrorString(e));
  return 0;
}

}  // namespace

// returns 1 when taken, 0 when the shape is not covered, other values are errors
int gguf_gemv_batch(int type, const float *x, const void *w, float *out, int M, int N, int K, cudaStream_t st) {
  if (M < 2 || M > 64 || K % 256) return 0;
  if (type != LB200_Q4_K && type != LB200_Q6_K) return 0;
  if (type == LB200_Q4_K && ((uintptr_t)w & 15)) return 0;
  if (type == LB200_Q6_K && (((uintptr_t)w & 3) || ((size_t)(K >> 8) * 210) % 4)) return 0;
  static DeviceOnce attr_done;
  {
    cudaError_t e = attr_done.ensure([&] {
      cudaError_t r = cudaFuncSetAttribute(q4k_gemv_batch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
      return r != cudaSuccess ? r : cudaFuncSetAttribute(q6k_gemv_batch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    });
    if (e != cudaSuccess) return fail((int)e, "light_b200: matmul_q (batched decode): %s", cudaGetErrorString(e));
  }
  const int tiles = (N + ROWS - 1) / ROWS;
  const int rt = tiles >= 148 * 6 ? 2 : 1;
  const unsigned grid = (unsigned)((N + ROWS * rt - 1) / (ROWS * rt));
  for (int m0 = 0; m0 < M; m0 += 8 * MAX_NT) {  // 16 tokens per pass over the weights
    const int mc = M - m0 < 8 * MAX_NT ? M - m0 : 8 * MAX_NT;
    const float *xm = x + (size_t)m0 * K;
    float *om = out + (size_t)m0 * N;
    int rc = type == LB200_Q4_K ? launch_pdl(q4k_gemv_batch_kernel, grid, st, xm, (const uint8_t *)w, om, mc, N, K, rt)
                                : launch_pdl(q6k_gemv_batch_kernel, grid, st, xm, (const uint8_t *)w, om, mc, N, K, rt);
    if (rc) return rc;
    if ((rc = launched("matmul_q (batched decode)"))) return rc;
  }
  return 1;
}

}  // namespace lb
