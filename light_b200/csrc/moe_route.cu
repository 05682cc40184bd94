// Device-side MoE routing: the reference routes DeepSeek-style models on the HOST (models/deepseek_route.go:27-133
// says so itself) and builds the expert-sorted pair list with TopK + Sort + count + scan launches
// (ops/moe.go:24-99, kernels/cuda/src/moe.cu:28-42).  Here:
//   moe_route_sigmoid   logits (T, E) [+ bias (E)] -> top-k ids (T, k) and weights (T, k): the V3 "sigmoid" branch
//                       with one group (scores = sigmoid(logit) in f64, choice = score + bias, stable descending
//                       top-k of the choices, weights = unbiased scores, renormalised by sum + 1e-20)
//   moe_sort_pairs      ids (M) -> counts (E), offsets (E + 1), sorted_pairs (M), sorted_expts (M): a stable
//                       counting sort (pairs of one expert stay in ascending order), three small launches, no
//                       host round trip and no library sort
#include "common.cuh"
#include "mma_sync.cuh"

namespace lb {
namespace {

constexpr int RT_MAX_PER_LANE = 32;  // experts per lane: E <= 1024

// one warp per token
__global__ void __launch_bounds__(256) moe_route_sigmoid_kernel(const float *__restrict__ logits, const float *__restrict__ bias,
                                                                long long *__restrict__ ids, float *__restrict__ weights, int T, int E,
                                                                int topk, int norm_topk) {
  pdl_launch_dependents();
  pdl_wait();
  const int tok = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (tok >= T) return;
  const int per = (E + 31) / 32;
  double score[RT_MAX_PER_LANE], choice[RT_MAX_PER_LANE];
#pragma unroll 1
  for (int i = 0; i < per; i++) {
    const int e = i * 32 + lane;  // expert e sits in slot e / 32 of lane e % 32
    if (e < E) {
      score[i] = 1.0 / (1.0 + exp(-(double)logits[(size_t)tok * E + e]));
      choice[i] = score[i] + (bias ? (double)bias[e] : 0.0);
    } else {
      score[i] = 0.0, choice[i] = -INFINITY;
    }
  }
  unsigned taken = 0;  // bit i: slot i of this lane was selected
  double den = 0.0, mine_w = 0.0;
  long long mine_id = 0;
  for (int k = 0; k < topk; k++) {
    // this lane's best free slot (the lowest expert id among equals: slots ascend with the id)
    double bv = -INFINITY;
    int be = 0x7fffffff;
#pragma unroll 1
    for (int i = 0; i < per; i++)
      if (!(taken >> i & 1u) && i * 32 + lane < E && choice[i] > bv) bv = choice[i], be = i * 32 + lane;
    // the warp's best: larger choice, then lower expert id
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const double ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ov > bv || (ov == bv && oe < be)) bv = ov, be = oe;
    }
    double sc = 0.0;
    if ((be & 31) == lane && be < E) {
      taken |= 1u << (be >> 5);
      sc = score[be >> 5];
    }
    sc = __shfl_sync(0xffffffffu, sc, be & 31);
    den += sc;
    if (lane == k % 32) mine_w = sc, mine_id = be;  // lane k keeps selection k (topk <= 32)
  }
  if (lane < topk) {
    const double w = norm_topk ? mine_w / (den + 1e-20) : mine_w;
    ids[(size_t)tok * topk + lane] = mine_id;
    weights[(size_t)tok * topk + lane] = (float)w;
  }
}

// The general DeepSeek router (models/deepseek_route.go:30-133, every branch), one warp per token, f64 like the
// host code it replaces: sigmoid scores with a selection bias (V3) or a softmax over the experts (V2); with
// n_group > 1 and topk_group < n_group only the topk_group best groups stay eligible (group score: the sum of its
// two best choices for the sigmoid router, its best for the softmax router); then the stable descending top-k.
// Expert e sits in slot e / 32 of lane e % 32; group g's score sits in lane g (n_group <= 32).
__global__ void __launch_bounds__(256) moe_route_deepseek_kernel(const float *__restrict__ logits, const float *__restrict__ bias,
                                                                 long long *__restrict__ ids, float *__restrict__ weights, int T, int E, int topk,
                                                                 int n_group, int topk_group, int sigmoid, int norm_topk) {
  pdl_launch_dependents();
  pdl_wait();
  const int tok = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (tok >= T) return;
  const int per = (E + 31) / 32, gsize = E / n_group;
  double score[RT_MAX_PER_LANE], choice[RT_MAX_PER_LANE];
  if (sigmoid) {
#pragma unroll 1
    for (int i = 0; i < per; i++) {
      const int e = i * 32 + lane;
      if (e < E) {
        score[i] = 1.0 / (1.0 + exp(-(double)logits[(size_t)tok * E + e]));
        choice[i] = score[i] + (bias ? (double)bias[e] : 0.0);
      } else {
        score[i] = 0.0, choice[i] = -INFINITY;
      }
    }
  } else {
    double mx = -INFINITY;
#pragma unroll 1
    for (int i = 0; i < per; i++) {
      const int e = i * 32 + lane;
      score[i] = e < E ? (double)logits[(size_t)tok * E + e] : -INFINITY;
      mx = fmax(mx, score[i]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmax(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    double sum = 0.0;  // added in expert order, as the host loop does
#pragma unroll 1
    for (int i = 0; i < per; i++) {
      const int e = i * 32 + lane;
      score[i] = e < E ? exp(score[i] - mx) : 0.0;
      for (int l = 0; l < 32; l++) {
        const double v = __shfl_sync(0xffffffffu, score[i], l);
        if (i * 32 + l < E) sum += v;
      }
    }
#pragma unroll 1
    for (int i = 0; i < per; i++) {
      const int e = i * 32 + lane;
      score[i] = e < E ? score[i] / sum : 0.0;
      choice[i] = e < E ? score[i] : -INFINITY;
    }
  }
  if (n_group > 1 && topk_group < n_group) {
    double gsv = -INFINITY;  // lane g: score of group g
    for (int g = 0; g < n_group; g++) {
      double b1 = -INFINITY, b2 = -INFINITY;  // this lane's two best choices inside group g
#pragma unroll 1
      for (int i = 0; i < per; i++) {
        const int e = i * 32 + lane;
        if (e < E && e / gsize == g) {
          if (choice[i] > b1)
            b2 = b1, b1 = choice[i];
          else if (choice[i] > b2)
            b2 = choice[i];
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {  // merge two sorted pairs
        const double o1 = __shfl_xor_sync(0xffffffffu, b1, o), o2 = __shfl_xor_sync(0xffffffffu, b2, o);
        const double n1 = fmax(b1, o1), n2 = fmax(fmin(b1, o1), fmax(b2, o2));
        b1 = n1, b2 = n2;
      }
      const double sc = sigmoid ? b1 + (gsize > 1 ? b2 : 0.0) : b1;
      if (lane == g) gsv = sc;
    }
    // stable descending rank of each group: groups ahead of it are the larger ones and the equal ones before it
    int rank = 0;
    for (int h = 0; h < n_group; h++) {
      const double ov = __shfl_sync(0xffffffffu, gsv, h);
      if (ov > gsv || (ov == gsv && h < lane)) rank++;
    }
    const int keep = lane < n_group && rank < topk_group;
#pragma unroll 1
    for (int i = 0; i < per; i++) {
      const int e = i * 32 + lane;
      const int kept = __shfl_sync(0xffffffffu, keep, e < E ? e / gsize : 0);
      if (e < E && !kept) {
        if (sigmoid)
          choice[i] = -INFINITY;
        else
          choice[i] = 0.0, score[i] = 0.0;
      }
    }
  }
  unsigned taken = 0;
  double den = 0.0, mine_w = 0.0;
  long long mine_id = 0;
  for (int k = 0; k < topk; k++) {
    double bv = -INFINITY;
    int be = 0x7fffffff;
    bool have = false;
#pragma unroll 1
    for (int i = 0; i < per; i++)
      if (!(taken >> i & 1u) && i * 32 + lane < E && (!have || choice[i] > bv)) bv = choice[i], be = i * 32 + lane, have = true;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const double ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (oe != 0x7fffffff && (be == 0x7fffffff || ov > bv || (ov == bv && oe < be))) bv = ov, be = oe;
    }
    double sc = 0.0;
    if ((be & 31) == lane && be < E) {
      taken |= 1u << (be >> 5);
      sc = score[be >> 5];
    }
    sc = __shfl_sync(0xffffffffu, sc, be & 31);
    den += sc;
    if (lane == k % 32) mine_w = sc, mine_id = be;
  }
  if (lane < topk) {
    const double w = (sigmoid && norm_topk) ? mine_w / (den + 1e-20) : mine_w;
    ids[(size_t)tok * topk + lane] = mine_id;
    weights[(size_t)tok * topk + lane] = (float)w;
  }
}

// ops.MoERoute's selection (ops/moe.go:29-50): the k largest router probabilities of a token (ties keep the lower
// expert id), their values as weights, divided by their f32 sum (added in selection order) when normalize.
__global__ void __launch_bounds__(256) moe_route_topk_kernel(const float *__restrict__ probs, long long *__restrict__ ids, float *__restrict__ weights,
                                                             int T, int E, int topk, int normalize) {
  pdl_launch_dependents();
  pdl_wait();
  const int tok = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (tok >= T) return;
  const int per = (E + 31) / 32;
  float v[RT_MAX_PER_LANE];
#pragma unroll 1
  for (int i = 0; i < per; i++) v[i] = i * 32 + lane < E ? probs[(size_t)tok * E + i * 32 + lane] : 0.f;
  unsigned taken = 0;
  float sum = 0.f, mine_w = 0.f;
  long long mine_id = 0;
  for (int k = 0; k < topk; k++) {
    float bv = 0.f;
    int be = 0x7fffffff;
#pragma unroll 1
    for (int i = 0; i < per; i++)
      if (!(taken >> i & 1u) && i * 32 + lane < E && (be == 0x7fffffff || v[i] > bv)) bv = v[i], be = i * 32 + lane;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (oe != 0x7fffffff && (be == 0x7fffffff || ov > bv || (ov == bv && oe < be))) bv = ov, be = oe;
    }
    if ((be & 31) == lane && be < E) taken |= 1u << (be >> 5);
    sum += bv;
    if (lane == k % 32) mine_w = bv, mine_id = be;
  }
  if (lane < topk) {
    ids[(size_t)tok * topk + lane] = mine_id;
    weights[(size_t)tok * topk + lane] = normalize ? mine_w / sum : mine_w;
  }
}

// ---- stable counting sort of M pair ids by expert, in blocks of 1024 pairs
constexpr int SORT_BLOCK = 1024;

// local rank of every pair among the pairs of its expert inside its block, and the block's histogram
__global__ void __launch_bounds__(SORT_BLOCK) moe_sort_local_kernel(const long long *__restrict__ ids, int *__restrict__ local_rank,
                                                                    int *__restrict__ block_hist, long long M, int E,
                                                                    unsigned int *__restrict__ status) {
  extern __shared__ int warp_hist[];  // [32 warps][E]
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 32 * E; i += SORT_BLOCK) warp_hist[i] = 0;
  __syncthreads();
  const long long p = (long long)blockIdx.x * SORT_BLOCK + threadIdx.x;
  long long e = p < M ? ids[p] : -1;
  if (p < M && (e < 0 || e >= E)) {  // reported, and parked with expert 0 so that nothing is written out of range
    atomicOr(status, 1u);
    e = 0;
  }
  const unsigned same = __match_any_sync(0xffffffffu, e);
  const int r = __popc(same & ((1u << lane) - 1u));
  if (e >= 0 && r == 0) warp_hist[warp * E + (int)e] = __popc(same);
  __syncthreads();
  // exclusive scan over the warps, per expert; the total is the block's count
  for (int x = threadIdx.x; x < E; x += SORT_BLOCK) {
    int run = 0;
#pragma unroll 1
    for (int w = 0; w < 32; w++) {
      const int c = warp_hist[w * E + x];
      warp_hist[w * E + x] = run;
      run += c;
    }
    block_hist[(size_t)blockIdx.x * E + x] = run;
  }
  __syncthreads();
  if (p < M) local_rank[p] = warp_hist[warp * E + (int)e] + r;
}

// counts, offsets, and the base of every (block, expert) run: one CTA
__global__ void __launch_bounds__(1024) moe_sort_scan_kernel(int *__restrict__ block_hist, int *__restrict__ counts, int *__restrict__ offsets,
                                                             int nblocks, int E) {
  __shared__ int tot[1024];
  pdl_launch_dependents();
  pdl_wait();
  for (int x = threadIdx.x; x < E; x += 1024) {
    int run = 0;
#pragma unroll 1
    for (int b = 0; b < nblocks; b++) {
      const int c = block_hist[(size_t)b * E + x];
      block_hist[(size_t)b * E + x] = run;  // pairs of expert x in earlier blocks
      run += c;
    }
    tot[x] = run;
    counts[x] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int x = 0; x < E; x++) offsets[x] = run, run += tot[x];
    offsets[E] = run;
  }
}

__global__ void __launch_bounds__(SORT_BLOCK) moe_sort_scatter_kernel(const long long *__restrict__ ids, const int *__restrict__ local_rank,
                                                                      const int *__restrict__ block_hist, const int *__restrict__ offsets,
                                                                      long long *__restrict__ sorted_pairs, long long *__restrict__ sorted_expts,
                                                                      long long M, int E) {
  pdl_launch_dependents();
  pdl_wait();
  const long long p = (long long)blockIdx.x * SORT_BLOCK + threadIdx.x;
  if (p >= M) return;
  long long e = ids[p];
  if (e < 0 || e >= E) e = 0;
  const long long pos = (long long)offsets[e] + block_hist[(size_t)blockIdx.x * E + e] + local_rank[p];
  sorted_pairs[pos] = p;
  sorted_expts[pos] = e;
}

__device__ unsigned int g_route_status = 0;  // bit 0: an expert id outside [0, E) was seen

template <typename Kern, typename... Args>
cudaError_t launch_chain(Kern kern, unsigned grid, unsigned block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid), cfg.blockDim = dim3(block), cfg.dynamicSmemBytes = smem, cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

}  // namespace

int moe_route_sigmoid(const float *logits, const float *bias, int64_t *ids, float *weights, int T, int E, int topk, int norm_topk,
                      cudaStream_t st) {
  if (T == 0) return 0;
  cudaError_t e = launch_chain(moe_route_sigmoid_kernel, (unsigned)((T + 7) / 8), 256, 0, st, logits, bias, (long long *)ids, weights, T, E, topk,
                               norm_topk);
  if (e != cudaSuccess) return fail((int)e, "light_b200: moe_route_sigmoid: %s", cudaGetErrorString(e));
  return launched("moe_route_sigmoid");
}

int moe_route_deepseek(const float *logits, const float *bias, int64_t *ids, float *weights, int T, int E, int topk, int n_group, int topk_group,
                       int sigmoid, int norm_topk, cudaStream_t st) {
  if (T == 0) return 0;
  cudaError_t e = launch_chain(moe_route_deepseek_kernel, (unsigned)((T + 7) / 8), 256, 0, st, logits, bias, (long long *)ids, weights, T, E, topk,
                               n_group, topk_group, sigmoid, norm_topk);
  if (e != cudaSuccess) return fail((int)e, "light_b200: moe_route_deepseek: %s", cudaGetErrorString(e));
  return launched("moe_route_deepseek");
}

int moe_route_topk(const float *probs, int64_t *ids, float *weights, int T, int E, int topk, int normalize, cudaStream_t st) {
  if (T == 0) return 0;
  cudaError_t e = launch_chain(moe_route_topk_kernel, (unsigned)((T + 7) / 8), 256, 0, st, probs, (long long *)ids, weights, T, E, topk, normalize);
  if (e != cudaSuccess) return fail((int)e, "light_b200: moe_route_topk: %s", cudaGetErrorString(e));
  return launched("moe_route_topk");
}

// scratch: M + nblocks * E ints (local ranks, then the per-block histograms)
int moe_sort_pairs(const int64_t *ids, int *counts, int *offsets, int64_t *sorted_pairs, int64_t *sorted_expts, int *scratch, long long M,
                   int E, cudaStream_t st) {
  const int nblocks = (int)((M + SORT_BLOCK - 1) / SORT_BLOCK);
  int *local_rank = scratch, *block_hist = scratch + M;
  // per device: the sort kernel's shared-memory opt-in, and the address of this device's copy of the status word
  static DeviceOnce attr_done;
  static unsigned int *status_of[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess && (dev < 0 || dev >= 64)) e = cudaErrorInvalidDevice;
  if (e == cudaSuccess)
    e = attr_done.ensure([&] {  // the first call on a device: make it outside stream capture
      cudaError_t r = cudaFuncSetAttribute(moe_sort_local_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 32 * 1024 * 4);
      return r != cudaSuccess ? r : cudaGetSymbolAddress((void **)&status_of[dev], g_route_status);
    });
  if (e != cudaSuccess) return fail((int)e, "light_b200: moe_sort_pairs: %s", cudaGetErrorString(e));
  unsigned int *status = status_of[dev];
  if (e == cudaSuccess && nblocks > 0)
    e = launch_chain(moe_sort_local_kernel, (unsigned)nblocks, SORT_BLOCK, (size_t)32 * E * 4, st, (const long long *)ids, local_rank, block_hist, M, E,
                     status);
  if (e == cudaSuccess) e = launch_chain(moe_sort_scan_kernel, 1u, 1024u, 0, st, block_hist, counts, offsets, nblocks, E);
  if (e == cudaSuccess && nblocks > 0)
    e = launch_chain(moe_sort_scatter_kernel, (unsigned)nblocks, SORT_BLOCK, 0, st, (const long long *)ids, (const int *)local_rank,
                     (const int *)block_hist, (const int *)offsets, (long long *)sorted_pairs, (long long *)sorted_expts, M, E);
  if (e != cudaSuccess) return fail((int)e, "light_b200: moe_sort_pairs: %s", cudaGetErrorString(e));
  return launched("moe_sort_pairs");
}

int moe_route_status() {
  unsigned int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_route_status, sizeof(v));
  if (e != cudaSuccess) return fail((int)e, "light_b200: moe_route_status: %s", cudaGetErrorString(e));
  return (int)v;
}

}  // namespace lb
