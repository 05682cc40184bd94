// Decode-step attention against a fixed-capacity KV cache whose length lives on the device: the
// counterparts of the reference's ops.KVAppend, ops.DecodeAttention and ops.IncrementI64
// (ops/decode_attn.go:13-205, kernels/cuda/decode_attn.go:44-133, kernels/cuda/src/decode_attn.cu:1-161).
//
// The reference runs three launches per layer (append; split-K partials into a scratch tensor, one block
// per 32 keys of the CAPACITY; combine).  Here one launch does all of it: a thread-block cluster of up to
// eight CTAs serves one (batch, KV head); the cluster divides the VALID keys [start, n) evenly (n is read
// on the device), every warp walks its keys with an online softmax for all query heads of the group (one
// lane owns D / 32 consecutive dims, so a key or value row is one coalesced warp load), the warps' and
// then the CTAs' partial (max, sum, sum p v) meet in shared and distributed shared memory, and CTA r
// writes slice r of the output.  No scratch tensor, no atomics, the same launch at every position.  With
// k_new / v_new given, the new row is read from there by the warp that owns position `pos` and copied
// into the cache by rank 0, so the append needs no launch of its own.
#include "common.cuh"
#include "mma_sync.cuh"
#include "umma.cuh"

namespace lb {
namespace {

constexpr int DA_WARPS = 16, DA_THREADS = DA_WARPS * 32;
constexpr int DA_MAX_G = 16;  // query heads per KV head, the reference's limit (decode_attn.cu:11)

__device__ unsigned int g_attn_status = 0;  // bit 0: a position outside [0, Cap) was seen (and clamped)

struct AttnArgs {
  const void *q, *k_new, *v_new;
  void *kbuf, *vbuf, *out;
  const long long *pos;
  int B, NH, KH, Cap, window;
  float scale;
  double rope_k;  // 0: no rotation; else -2 log2(base) / D, so that base^(-2 i / D) = 2^(i rope_k)
};

// cos and sin of pos * base^(-2 i / D): the angle in f64 (an f32 angle of a few hundred radians is already
// off by 1e-5), reduced to [-pi, pi] there, then the f32 functions.  Out of line: its registers are not the
// attention loop's.
__device__ __noinline__ float2 rope_cos_sin(long long pos, int i, double rope_k) {
  const double theta = (double)pos * exp2((double)i * rope_k);
  const double r = theta - 6.283185307179586476925 * rint(theta * 0.15915494309189533577);
  float sn, c;
  sincosf((float)r, &sn, &c);
  return make_float2(c, sn);
}

// PER consecutive elements of a row, as floats; 2 to 64 bytes per lane, naturally aligned
template <int PER>
__device__ __forceinline__ void load_row(const float *p, float (&f)[PER]) {
  if constexpr (PER >= 4) {
#pragma unroll
    for (int i = 0; i < PER / 4; i++) {
      const float4 v = __ldg(reinterpret_cast<const float4 *>(p) + i);
      f[4 * i] = v.x, f[4 * i + 1] = v.y, f[4 * i + 2] = v.z, f[4 * i + 3] = v.w;
    }
  } else if constexpr (PER == 2) {
    const float2 v = __ldg(reinterpret_cast<const float2 *>(p));
    f[0] = v.x, f[1] = v.y;
  } else {
    f[0] = __ldg(p);
  }
}
template <int PER>
__device__ __forceinline__ void load_row(const __nv_bfloat16 *p, float (&f)[PER]) {
  if constexpr (PER >= 8) {
#pragma unroll
    for (int i = 0; i < PER / 8; i++) {
      const uint4 v = __ldg(reinterpret_cast<const uint4 *>(p) + i);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int c = 0; c < 4; c++) f[8 * i + 2 * c] = __uint_as_float(w[c] << 16), f[8 * i + 2 * c + 1] = __uint_as_float(w[c] & 0xFFFF0000u);
    }
  } else if constexpr (PER == 4) {
    const uint2 v = __ldg(reinterpret_cast<const uint2 *>(p));
    f[0] = __uint_as_float(v.x << 16), f[1] = __uint_as_float(v.x & 0xFFFF0000u);
    f[2] = __uint_as_float(v.y << 16), f[3] = __uint_as_float(v.y & 0xFFFF0000u);
  } else if constexpr (PER == 2) {
    const uint32_t v = __ldg(reinterpret_cast<const uint32_t *>(p));
    f[0] = __uint_as_float(v << 16), f[1] = __uint_as_float(v & 0xFFFF0000u);
  } else {
    f[0] = __bfloat162float(*p);
  }
}

template <int PER, int GH_>
struct AttnCfg {
  static constexpr int D = PER * 32;
  static constexpr int GH = GH_;                                        // query heads per pass over the keys
  static constexpr int U = PER >= 16 ? 1 : PER == 8 ? 2 : 4;           // keys per batch of a warp (two batches in flight)
  static constexpr int ROW = D + 2;                                     // max, sum, D dims
  static constexpr int WPART = DA_WARPS * GH * ROW;                     // floats: per-warp partials of a pass
  static size_t smem(int g) { return (size_t)(WPART + g * ROW) * sizeof(float); }
};

template <typename T, int PER, int GH_>
__global__ void __launch_bounds__(DA_THREADS, 1) decode_attn_kernel(AttnArgs a) {
  using Cfg = AttnCfg<PER, GH_>;
  constexpr int D = Cfg::D, GH = Cfg::GH, U = Cfg::U, ROW = Cfg::ROW;
  constexpr int NV = GH * U;  // dot products per batch of keys
  constexpr int SH = NV >= 32 ? 0 : NV == 16 ? 1 : NV == 8 ? 2 : NV == 4 ? 3 : NV == 2 ? 4 : 5;
  extern __shared__ __align__(16) float sm[];  // [warp][head of the pass][ROW] then [head][ROW] of this CTA
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KS = gridDim.y, rank = blockIdx.y, bkh = blockIdx.x;
  const int g = a.NH / a.KH, b = bkh / a.KH, kh = bkh - b * a.KH;
  float *wpart = sm, *cpart = sm + Cfg::WPART;
  pdl_wait();  // q, k_new, v_new are the previous launch's output; pos is older
  long long pos = a.pos[0];
  // A position outside the cache: reported, nothing is appended (as kv_append_kernel), and the launch attends
  // over the cached rows of the clamped range, so that append-inside stays equal to append-then-attend.
  const bool in_range = pos >= 0 && pos < a.Cap;
  if (!in_range) {
    if (threadIdx.x == 0) atomicOr(&g_attn_status, 1u);
    pos = pos < 0 ? 0 : a.Cap - 1;
  }
  const int n = (int)pos + 1;
  const int start = a.window > 0 ? max(0, n - a.window) : 0;
  const int chunk = (n - start + KS - 1) / KS;
  const int j0 = start + rank * chunk, j1 = min(n, j0 + chunk);
  const T *Kb = static_cast<const T *>(a.kbuf) + (size_t)bkh * a.Cap * D + lane * PER;
  const T *Vb = static_cast<const T *>(a.vbuf) + (size_t)bkh * a.Cap * D + lane * PER;
  const T *kn = a.k_new && in_range ? static_cast<const T *>(a.k_new) + (size_t)bkh * D + lane * PER : nullptr;
  const T *vn = a.k_new && in_range ? static_cast<const T *>(a.v_new) + (size_t)bkh * D + lane * PER : nullptr;
  // rotary embedding of q and of the new key at position pos (rotate-half pairing: dim i with i + D / 2,
  // which is lane ^ 16 here); cached keys were rotated when they were appended
  const bool roped = a.rope_k != 0.0;
  float rc[PER], rs[PER];
  if (roped) {
#pragma unroll
    for (int p = 0; p < PER; p++) {
      const float2 cs = rope_cos_sin(pos, (lane * PER + p) & (D / 2 - 1), a.rope_k);
      rc[p] = cs.x, rs[p] = cs.y;
    }
  }
  auto rotate = [&](float (&v)[PER]) {
#pragma unroll
    for (int p = 0; p < PER; p++) {
      const float o = __shfl_xor_sync(0xffffffffu, v[p], 16);
      v[p] = lane < 16 ? v[p] * rc[p] - o * rs[p] : o * rs[p] + v[p] * rc[p];
    }
  };
  if (kn && rank == 0 && threadIdx.x < D) {  // the append: readers of position pos take the row from k_new
    const T *ks = static_cast<const T *>(a.k_new) + (size_t)bkh * D;
    const size_t dst = ((size_t)bkh * a.Cap + (size_t)pos) * D + threadIdx.x;
    if (roped) {
      const int i = threadIdx.x & (D / 2 - 1);
      const float2 cs = rope_cos_sin(pos, i, a.rope_k);
      const float x0 = ld_act(ks, i), x1 = ld_act(ks, i + D / 2);
      st_act(static_cast<T *>(a.kbuf), (long long)dst, (int)threadIdx.x < D / 2 ? x0 * cs.x - x1 * cs.y : x0 * cs.y + x1 * cs.x);
    } else {
      static_cast<T *>(a.kbuf)[dst] = ks[threadIdx.x];
    }
    static_cast<T *>(a.vbuf)[dst] = static_cast<const T *>(a.v_new)[(size_t)bkh * D + threadIdx.x];
  }

  for (int h0 = 0; h0 < g; h0 += GH) {
    const int gh = min(GH, g - h0);
    float qf[GH][PER], acc[GH][PER], m[GH], l[GH];
    float m_own = -INFINITY;  // m[head of the value this lane owns in the reduce-scatter]
#pragma unroll
    for (int h = 0; h < GH; h++) {
      m[h] = -INFINITY, l[h] = 0.f;
#pragma unroll
      for (int p = 0; p < PER; p++) acc[h][p] = 0.f, qf[h][p] = 0.f;
      if (h < gh) load_row<PER>(static_cast<const T *>(a.q) + ((size_t)b * a.NH + (size_t)kh * g + h0 + h) * D + lane * PER, qf[h]);
      if (roped) rotate(qf[h]);
    }
    float kf[U][PER], vf[U][PER];
    auto fetch = [&](int j, float (&kk)[U][PER], float (&vv)[U][PER]) {
#pragma unroll
      for (int u = 0; u < U; u++) {
        if (j + u < j1) {
          const bool fresh = kn && j + u == (int)pos;
          load_row<PER>(fresh ? kn : Kb + (size_t)(j + u) * D, kk[u]);
          load_row<PER>(fresh ? vn : Vb + (size_t)(j + u) * D, vv[u]);
          if (fresh && roped) rotate(kk[u]);
        } else {
#pragma unroll
          for (int p = 0; p < PER; p++) kk[u][p] = 0.f, vv[u][p] = 0.f;
        }
      }
    };
    if (j0 + warp * U < j1) fetch(j0 + warp * U, kf, vf);
    for (int j = j0 + warp * U; j < j1; j += DA_WARPS * U) {
      float kx[U][PER], vx[U][PER];  // the next batch is requested before this one is used
      if (j + DA_WARPS * U < j1) fetch(j + DA_WARPS * U, kx, vx);
      if constexpr (NV <= 32) {
        // The GH x U dot products of this batch are summed over the lanes by a reduce-scatter: at every
        // step a lane hands half of its partial sums to its partner and keeps the other half, so that
        // value i (head i / U, key i % U) ends up, complete, in lanes [i << SH, (i + 1) << SH) -- NV + 1
        // shuffles instead of 5 NV -- and the exponentials are computed once, by the owners.
        float v[NV];
#pragma unroll
        for (int h = 0; h < GH; h++)
#pragma unroll
          for (int u = 0; u < U; u++) {
            float d = 0.f;
#pragma unroll
            for (int p = 0; p < PER; p++) d = fmaf(qf[h][p], kf[u][p], d);
            v[h * U + u] = d;
          }
        int cnt = NV;
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
          if (cnt > 1) {
            const int half = cnt / 2;
            const bool up = lane & off;
#pragma unroll
            for (int i = 0; i < half; i++) {
              const float send = up ? v[i] : v[i + half], keep = up ? v[i + half] : v[i];
              v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
            }
            cnt = half;
          } else {
            v[0] += __shfl_xor_sync(0xffffffffu, v[0], off);
          }
        }
        const int own = lane >> SH;  // this lane's value: head own / U, key own % U
        const float s_own = j + (own % U) < j1 ? v[0] * a.scale : -INFINITY;
        float bm = s_own;            // maximum over the batch's keys of the own head
#pragma unroll
        for (int off = 1 << SH; off < (U << SH); off <<= 1) bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, off));
        m_own = fmaxf(m_own, bm);
        const float e_own = __expf(s_own - m_own);  // -inf for a missing key: 0
#pragma unroll
        for (int h = 0; h < GH; h++) {
          const float mx = fmaxf(m[h], __shfl_sync(0xffffffffu, bm, (h * U) << SH));
          const float corr = __expf(m[h] - mx);  // m = -inf on the first batch: 0
          m[h] = mx;
          l[h] *= corr;
#pragma unroll
          for (int p = 0; p < PER; p++) acc[h][p] *= corr;
#pragma unroll
          for (int u = 0; u < U; u++) {
            const float e = __shfl_sync(0xffffffffu, e_own, (h * U + u) << SH);
            l[h] += e;
#pragma unroll
            for (int p = 0; p < PER; p++) acc[h][p] = fmaf(e, vf[u][p], acc[h][p]);
          }
        }
      } else {
#pragma unroll
        for (int h = 0; h < GH; h++) {
          if (h < gh) {
            float s[U], mx = m[h];
  #pragma unroll
            for (int u = 0; u < U; u++) {
              float d = 0.f;
  #pragma unroll
              for (int p = 0; p < PER; p++) d = fmaf(qf[h][p], kf[u][p], d);
              s[u] = j + u < j1 ? warp_sum(d) * a.scale : -INFINITY;
              mx = fmaxf(mx, s[u]);
            }
            const float corr = __expf(m[h] - mx);  // m = -inf on the first batch: 0
            m[h] = mx;
            l[h] *= corr;
  #pragma unroll
            for (int p = 0; p < PER; p++) acc[h][p] *= corr;
  #pragma unroll
            for (int u = 0; u < U; u++) {
              const float e = __expf(s[u] - mx);  // -inf for a missing key: 0
              l[h] += e;
  #pragma unroll
              for (int p = 0; p < PER; p++) acc[h][p] = fmaf(e, vf[u][p], acc[h][p]);
            }
          }
        }
      }
      if (j + DA_WARPS * U < j1) {
#pragma unroll
        for (int u = 0; u < U; u++)
#pragma unroll
          for (int p = 0; p < PER; p++) kf[u][p] = kx[u][p], vf[u][p] = vx[u][p];
      }
    }
    // ---- the warps of this CTA
#pragma unroll
    for (int h = 0; h < GH; h++) {
      if (h < gh) {
        float *row = wpart + (warp * GH + h) * ROW;
        if (lane == 0) row[0] = m[h], row[1] = l[h];
#pragma unroll
        for (int p = 0; p < PER; p++) row[2 + lane * PER + p] = acc[h][p];
      }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < gh * D; idx += DA_THREADS) {
      const int h = idx / D, d = idx - h * D;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < DA_WARPS; w++) M = fmaxf(M, wpart[(w * GH + h) * ROW]);
      float L = 0.f, A = 0.f;
      if (M > -INFINITY) {
#pragma unroll
        for (int w = 0; w < DA_WARPS; w++) {
          const float *row = wpart + (w * GH + h) * ROW;
          const float e = __expf(row[0] - M);
          L = fmaf(e, row[1], L), A = fmaf(e, row[2 + d], A);
        }
      }
      float *dst = cpart + (h0 + h) * ROW;
      dst[2 + d] = A;
      if (d == 0) dst[0] = M, dst[1] = L;
    }
    __syncthreads();
  }
  // ---- the CTAs of this cluster: rank r writes elements r (g D) / KS .. of the group's output
  if (KS > 1) umma::cluster_sync();
  {
    const int tot = g * D, e0 = tot * rank / KS, e1 = tot * (rank + 1) / KS;
    const uint32_t cbase = (uint32_t)__cvta_generic_to_shared(cpart);
    for (int idx = e0 + threadIdx.x; idx < e1; idx += DA_THREADS) {
      const int h = idx / D, d = idx - h * D;
      const uint32_t ra = cbase + (uint32_t)(h * ROW) * 4u;
      float M = -INFINITY, L = 0.f, A = 0.f;
      if (KS > 1) {
        float mr[8];
#pragma unroll
        for (int r = 0; r < 8; r++) {
          mr[r] = r < KS ? umma::ld_cluster_f32(umma::map_to_rank(ra, (uint32_t)r)) : -INFINITY;
          M = fmaxf(M, mr[r]);
        }
#pragma unroll
        for (int r = 0; r < 8; r++) {
          if (r < KS && mr[r] > -INFINITY) {  // a rank without keys holds (-inf, 0, 0)
            const float e = __expf(mr[r] - M);
            L = fmaf(e, umma::ld_cluster_f32(umma::map_to_rank(ra + 4u, (uint32_t)r)), L);
            A = fmaf(e, umma::ld_cluster_f32(umma::map_to_rank(ra + 8u + (uint32_t)d * 4u, (uint32_t)r)), A);
          }
        }
      } else {
        L = cpart[h * ROW + 1], A = cpart[h * ROW + 2 + d];
      }
      st_act(static_cast<T *>(a.out), ((long long)b * a.NH + (long long)kh * g + h) * D + d, A / L);
    }
  }
  if (KS > 1) umma::cluster_sync();  // nobody leaves while a peer still reads its partials
}

template <typename T>
__global__ void kv_append_kernel(const T *__restrict__ k, const T *__restrict__ v, T *__restrict__ kbuf, T *__restrict__ vbuf,
                                 const long long *__restrict__ pos, long long n, int D, int Cap) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const long long p = pos[0];
  if (p < 0 || p >= Cap) {
    if (i == 0) atomicOr(&g_attn_status, 1u);
    return;
  }
  const long long bh = i / D;
  const long long dst = (bh * Cap + p) * D + (i - bh * D);
  kbuf[dst] = k[i];
  vbuf[dst] = v[i];
}

__global__ void inc_i64_kernel(long long *p, int n) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] += 1;
}

template <typename K, typename... Args>
cudaError_t launch_chain(K kern, dim3 grid, dim3 block, size_t smem, unsigned cluster_y, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = 1, attr[1].val.clusterDim.y = cluster_y, attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = cluster_y > 1 ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

template <typename T, int PER, int GH>
int launch_attn(const AttnArgs &a, int ks, cudaStream_t st) {
  auto kern = decode_attn_kernel<T, PER, GH>;
  const size_t smem = AttnCfg<PER, GH>::smem(a.NH / a.KH);
  static DeviceOnce smem_set;  // per instantiation and device: the largest size opted in so far
  {
    cudaError_t e = smem_set.ensure([&] { return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); }, smem);
    if (e != cudaSuccess) return fail((int)e, "light_b200: decode_attn: %s", cudaGetErrorString(e));
  }
  cudaError_t e = launch_chain(kern, dim3((unsigned)(a.B * a.KH), (unsigned)ks), dim3(DA_THREADS), smem, (unsigned)ks, st, a);
  if (e != cudaSuccess) return fail((int)e, "light_b200: decode_attn: %s", cudaGetErrorString(e));
  return launched("decode_attn");
}

// heads per pass: the smallest of 1, 2, 4, ... that covers the group, while heads x dims-per-lane stays
// within 32 accumulators per lane (larger groups walk the keys again; they hit in L2)
template <typename T, int PER>
int launch_attn_g(const AttnArgs &a, int ks, cudaStream_t st) {
  constexpr int GMAX = 32 / PER < DA_MAX_G ? 32 / PER : DA_MAX_G;
  const int g = a.NH / a.KH;
  if constexpr (GMAX >= 2) {
    if (g <= GMAX / 2) {
      if constexpr (GMAX >= 4) {
        if (g <= GMAX / 4) return launch_attn<T, PER, GMAX / 4>(a, ks, st);
      }
      return launch_attn<T, PER, GMAX / 2>(a, ks, st);
    }
  }
  return launch_attn<T, PER, GMAX>(a, ks, st);
}

template <typename T>
int launch_attn_d(const AttnArgs &a, int D, int ks, cudaStream_t st) {
  switch (D / 32) {
    case 1: return launch_attn_g<T, 1>(a, ks, st);
    case 2: return launch_attn_g<T, 2>(a, ks, st);
    case 4: return launch_attn_g<T, 4>(a, ks, st);
    case 8: return launch_attn_g<T, 8>(a, ks, st);
    case 16: return launch_attn_g<T, 16>(a, ks, st);
  }
  return fail(LB200_E_SHAPE, "light_b200: decode_attn: head dim %d (want 32, 64, 128, 256 or 512)", D);
}

}  // namespace

int decode_attn(const lb200_decode_attn_args *p, cudaStream_t st) {
  if (!p) return fail(LB200_E_NULL, "light_b200: decode_attn: null argument block");
  if (!p->q || !p->kbuf || !p->vbuf || !p->pos || !p->out || (!p->k_new) != (!p->v_new))
    return fail(LB200_E_NULL, "light_b200: decode_attn: null pointer (k_new and v_new come together)");
  if (p->dtype != LB200_F32 && p->dtype != LB200_BF16) return fail(LB200_E_DTYPE, "light_b200: decode_attn: element type %d", p->dtype);
  if (p->B <= 0 || p->NH <= 0 || p->KH <= 0 || p->Cap <= 0 || p->D <= 0 || p->NH % p->KH || p->window < 0)
    return fail(LB200_E_SHAPE, "light_b200: decode_attn: B %d NH %d KH %d Cap %d D %d window %d", p->B, p->NH, p->KH, p->Cap, p->D, p->window);
  const int g = p->NH / p->KH;
  // the reference's own limits (kernels/cuda/decode_attn.go:36-38): other shapes take its composed path
  if (p->D % 32 || p->D > 512 || g > DA_MAX_G) return fail(LB200_E_SHAPE, "light_b200: decode_attn: head dim %d / group %d unsupported", p->D, g);
  if ((long long)p->B * p->KH > 65535ll * 1024) return fail(LB200_E_TOO_LARGE, "light_b200: decode_attn: B x KH too large");
  const uintptr_t al = (uintptr_t)p->q | (uintptr_t)p->kbuf | (uintptr_t)p->vbuf | (uintptr_t)p->k_new | (uintptr_t)p->v_new;
  if (al & 15) return fail(LB200_E_ALIGN, "light_b200: decode_attn: q / k / v must be 16-byte aligned");
  if (p->rope_base < 0.f) return fail(LB200_E_SHAPE, "light_b200: decode_attn: rope_base %g", (double)p->rope_base);
  const double rope_k = p->rope_base > 0.f ? -2.0 * log2((double)p->rope_base) / (double)p->D : 0.0;
  AttnArgs a{p->q, p->k_new, p->v_new, p->kbuf, p->vbuf, p->out, (const long long *)p->pos, p->B, p->NH, p->KH, p->Cap, p->window, p->scale, rope_k};
  // enough CTAs to fill the GPU, at least 32 keys of the capacity each, a portable cluster
  int ks = 1;
  while (ks < 8 && p->B * p->KH * ks < 148 && p->Cap >= 64 * ks) ks *= 2;
  return p->dtype == LB200_F32 ? launch_attn_d<float>(a, p->D, ks, st) : launch_attn_d<__nv_bfloat16>(a, p->D, ks, st);
}

int kv_append(const void *k, const void *v, void *kbuf, void *vbuf, const int64_t *pos, int dtype, int B, int KH, int D, int Cap,
              cudaStream_t st) {
  if (!k || !v || !kbuf || !vbuf || !pos) return fail(LB200_E_NULL, "light_b200: kv_append: null pointer");
  if (B <= 0 || KH <= 0 || D <= 0 || Cap <= 0) return fail(LB200_E_SHAPE, "light_b200: kv_append: B %d KH %d D %d Cap %d", B, KH, D, Cap);
  const long long n = (long long)B * KH * D;
  const unsigned grid = (unsigned)((n + 255) / 256);
  cudaError_t e;
  if (dtype == LB200_F32)
    e = launch_chain(kv_append_kernel<float>, dim3(grid), dim3(256), 0, 1, st, (const float *)k, (const float *)v, (float *)kbuf, (float *)vbuf,
                     (const long long *)pos, n, D, Cap);
  else if (dtype == LB200_BF16)
    e = launch_chain(kv_append_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, 1, st, (const __nv_bfloat16 *)k, (const __nv_bfloat16 *)v,
                     (__nv_bfloat16 *)kbuf, (__nv_bfloat16 *)vbuf, (const long long *)pos, n, D, Cap);
  else
    return fail(LB200_E_DTYPE, "light_b200: kv_append: element type %d", dtype);
  if (e != cudaSuccess) return fail((int)e, "light_b200: kv_append: %s", cudaGetErrorString(e));
  return launched("kv_append");
}

int inc_i64(int64_t *p, int n, cudaStream_t st) {
  if (!p) return fail(LB200_E_NULL, "light_b200: inc_i64: null pointer");
  if (n <= 0) return fail(LB200_E_SHAPE, "light_b200: inc_i64: n %d", n);
  cudaError_t e = launch_chain(inc_i64_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, 1, st, (long long *)p, n);
  if (e != cudaSuccess) return fail((int)e, "light_b200: inc_i64: %s", cudaGetErrorString(e));
  return launched("inc_i64");
}

int decode_attn_status() {
  unsigned int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_attn_status, sizeof(v));
  if (e != cudaSuccess) return fail((int)e, "light_b200: decode_attn_status: %s", cudaGetErrorString(e));
  return (int)v;
}

}  // namespace lb
