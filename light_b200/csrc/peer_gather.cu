// All-gather of row-split matmul outputs over NVLink peer memory, without NCCL and without fences.
//
// Every rank holds, in symmetric (peer-mapped) memory, one receive buffer per gathered operator: one
// 8-byte slot per output element, {f32 value, u32 step tag}.  After a rank's matmul has produced its
// (M, N/P) column block, ONE kernel
//   1. writes each of its elements, tagged with the current step, into the slot of that element in every
//      peer's receive buffer (one aligned 8-byte store per element and peer: value and tag can never be seen
//      torn, so no fence and no separate flag is needed), and into its own full-width output directly;
//   2. reads the slots of the other ranks' elements from its own receive buffer, polling each until its
//      tag equals the current step (bounded), and writes the values into its full-width output.
// The cost is one NVLink one-way latency.  Tags only grow (the step word is bumped once per step on the
// device, so CUDA-graph replays need no parameter update).  Each operator has two sets of slots used on
// alternating steps: a slot is rewritten two steps later, and a rank can only get there after it has
// received every peer's data of the step in between, which a peer sends only after it has consumed the
// earlier step.  Plain stores and loads to peer pointers only: no TMA, no multicast, no multimem.
#include "common.cuh"

namespace lb {

namespace {

__device__ int g_comm_status;  // non-zero: a bounded wait on a peer gave up (sticky)

__global__ void step_begin_kernel(unsigned int *step) { *step += 1; }

struct Slots {
  uint2 *ll[LB200_MAX_PEERS];
};

__global__ void __launch_bounds__(256) allgather_ll_kernel(const float *__restrict__ local, float *__restrict__ out,
                                                           Slots slots, int world, int rank, int M, int n_local,
                                                           const unsigned int *__restrict__ step) {
  // programmatic dependent launch on both sides: the matmul after this gather may start (and request
  // its weights) at once, and this kernel's own launch overlapped the tail of the matmul before it
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  asm volatile("griddepcontrol.wait;\n" ::: "memory");  // `local` and the step word are the predecessors' outputs
  const unsigned int tag = *step;
  const int N = n_local * world, mine = M * n_local, total = M * N;
  const int tid = blockIdx.x * blockDim.x + threadIdx.x, nthr = gridDim.x * blockDim.x;
  const size_t half = (size_t)(tag & 1u) * total;  // two sets of slots, alternating by step
  // 1. my block: to every peer's slots, and into my own output
  for (int i = tid; i < mine; i += nthr) {
    const int m = i / n_local, c = i - m * n_local;
    const size_t e = (size_t)m * N + (size_t)rank * n_local + c;
    const float v = local[i];
    out[e] = v;
    const uint2 pkt = make_uint2(__float_as_uint(v), tag);
    for (int p = 0; p < world; p++)
      if (p != rank) asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};\n" ::"l"(slots.ll[p] + half + e), "r"(pkt.x), "r"(pkt.y) : "memory");
  }
  // 2. everybody else's blocks, from my own slots
  unsigned long long t0;
  asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(t0));
  const uint2 *rx = slots.ll[rank] + half;
  bool gave_up = false;
  for (int i = tid; i < total - mine; i += nthr) {
    // i-th element that is not mine, row-major
    const int per_row = N - n_local, m = i / per_row;
    int c = i - m * per_row;
    if (c >= rank * n_local) c += n_local;
    const size_t e = (size_t)m * N + c;
    uint2 pkt;
    for (unsigned int it = 0;; it++) {
      asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];\n" : "=r"(pkt.x), "=r"(pkt.y) : "l"(rx + e) : "memory");
      if (pkt.y == tag || gave_up) break;
      if ((it & 255u) == 255u) {
        unsigned long long t1;
        asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(t1));
        if (t1 - t0 > 50000000ull) {  // 50 ms: a peer is gone or a step behind for good
          g_comm_status = 1;
          gave_up = true;
        }
      }
    }
    out[e] = __uint_as_float(pkt.x);
  }
}

}  // namespace

int comm_step_begin(unsigned int *step, cudaStream_t st) {
  step_begin_kernel<<<1, 1, 0, st>>>(step);
  return launched("step_begin");
}

int allgather_ll(const float *local, float *out, const lb200_peers *peers, int M, int n_local, const unsigned int *step,
                 cudaStream_t st) {
  Slots s;
  for (int i = 0; i < LB200_MAX_PEERS; i++) s.ll[i] = i < peers->world ? (uint2 *)peers->slots[i] : nullptr;
  const int total = M * n_local * peers->world;
  int grid = (total + 1023) / 1024;  // about four elements per thread
  if (grid < 1) grid = 1;
  if (grid > 148) grid = 148;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(256);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, allgather_ll_kernel, local, out, s, peers->world, peers->rank, M, n_local, step);
  if (e != cudaSuccess) return fail((int)e, "light_b200: allgather_ll: %s", cudaGetErrorString(e));
  return launched("allgather_ll");
}

int comm_status() {
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_comm_status, sizeof(int));
  return e == cudaSuccess ? v : -(int)e;
}

}  // namespace lb
