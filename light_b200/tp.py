"""Row-split (tensor-parallel) placement of quantized weights over the GPUs of one node.

The reference is single-GPU (STATUS.md:474), so the contract here is "same numbers as one GPU".
Every weight layout on this path is row-major with whole blocks per row (GGUF: K/256 blocks of 144
or 210 bytes; int4: codes / scales / zeros all (N, .); fp8-block: split on multiples of the block
height), so giving rank r the rows [r*N/P, (r+1)*N/P) is a plain slice with no repacking -- the same
property the reference's loader uses when it permutes and concatenates rows at byte level
(models/llama_gguf.go:344-382).  Each rank computes its (M, N/P) slice of the output; where the
next operator needs the whole row, the slices are all-gathered.

Only host-side logic lives here (it is exercised on CPU with the gloo backend); the matmuls themselves
are the single-GPU kernels.
"""
from __future__ import annotations

import torch


def row_range(N: int, rank: int, world: int) -> tuple[int, int]:
    """Rows of an (N, K) weight owned by `rank`; N must divide evenly so that every rank runs the
    same launch shape."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"row_range: rank {rank} outside world of {world}")
    if N % world:
        raise ValueError(f"row_range: {N} rows do not split evenly over {world} ranks")
    per = N // world
    return rank * per, (rank + 1) * per


def shard_rows(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """The rank's rows of a weight held as a 2-D tensor whose first dimension is N (block bytes, codes,
    scales or zeros alike).  A view, not a copy."""
    lo, hi = row_range(w.shape[0], rank, world)
    return w[lo:hi]


def shard_fp8_block(w: torch.Tensor, scale: torch.Tensor, block_r: int, rank: int, world: int):
    """Block-scaled FP8: rows split on multiples of the block height so that scale rows split with them."""
    lo, hi = row_range(w.shape[0], rank, world)
    if lo % block_r or hi % block_r:
        raise ValueError(f"shard_fp8_block: {w.shape[0]} rows over {world} ranks does not fall on {block_r}-row blocks")
    return w[lo:hi], scale[lo // block_r:hi // block_r]


def all_gather_columns(local: torch.Tensor, out: torch.Tensor | None = None, group=None) -> torch.Tensor:
    """(M, N/P) slices -> (M, N): rank r's slice becomes columns [r*N/P, (r+1)*N/P).  One collective."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    M, n = local.shape
    if out is None:
        out = torch.empty(M, n * world, dtype=local.dtype, device=local.device)
    if M == 1:
        dist.all_gather_into_tensor(out.view(-1), local.contiguous().view(-1), group=group)
        return out
    tmp = torch.empty(world, M, n, dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(tmp.view(-1), local.contiguous().view(-1), group=group)
    out.view(M, world, n).copy_(tmp.permute(1, 0, 2))
    return out


def expert_range(E: int, rank: int, world: int) -> tuple[int, int]:
    """Experts owned by `rank` under expert parallelism (contiguous blocks of E / P)."""
    return row_range(E, rank, world)


def split_pairs_by_rank(sorted_expts: torch.Tensor, E: int, world: int) -> torch.Tensor:
    """Number of routed pairs each rank receives: because pairs are already sorted by expert
    (ops.MoERoute), rank r's pairs are one contiguous run of the sorted list.  Returns (world + 1)
    offsets into it."""
    per = E // world
    bounds = torch.arange(0, world + 1, device=sorted_expts.device, dtype=sorted_expts.dtype) * per
    return torch.searchsorted(sorted_expts.contiguous(), bounds)


class PeerGather:
    """All-gather of row-split f32 outputs through NVLink peer stores (light_b200_allgather_ll).

    One symmetric-memory arena per rank holds a receive buffer (8 bytes per output element) for every
    gathered operator; `plan(shapes)` lays them out identically on all ranks.  Symmetric memory comes from
    torch.distributed._symmetric_memory (plumbing only); the data path is this library's kernel.  Raises if
    the ranks cannot map each other's memory -- callers then fall back to NCCL.
    """

    def __init__(self, device: torch.device, group=None):
        import torch.distributed as dist

        self.device, self.group = device, group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)

    def plan(self, shapes: list[tuple[int, int]]) -> list[torch.Tensor]:
        """shapes: (M, N) of each gathered output, in the order they are gathered every step.  Returns the
        full-width output tensors (ordinary local memory)."""
        import ctypes as C

        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        from . import _lib

        offs, total = [], 0
        for M, N in shapes:
            offs.append(total)
            total += (2 * M * N * 8 + 255) // 256 * 256  # two sets of slots, alternating by step
        arena = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
        arena.zero_()
        try:
            hdl = symm_mem.rendezvous(arena, self.group)
        except TypeError:
            hdl = symm_mem.rendezvous(arena, self.group.group_name)
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)
        self.arena, self.handle = arena, hdl
        ptrs = [int(p) for p in hdl.buffer_ptrs]
        self.peers = []
        for off in offs:
            p = _lib.Peers(world=self.world, rank=self.rank)
            for r in range(self.world):
                p.slots[r] = ptrs[r] + off
            self.peers.append(p)
        self.step = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.outs = [torch.empty(M, N, dtype=torch.float32, device=self.device) for M, N in shapes]
        self._C = C
        return self.outs

    def step_begin(self) -> None:
        from . import _lib

        dev = self.device.index or 0
        _lib.check(_lib.lib().light_b200_comm_step_begin(self._C.c_void_p(self.step.data_ptr()), dev,
                                                         self._C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)))

    def gather(self, index: int, local: torch.Tensor) -> torch.Tensor:
        """Sends this rank's (M, N/P) block of gathered output `index` and receives the others; the returned
        full-width tensor is complete for whatever runs next on the stream."""
        from . import _lib

        C = self._C
        dev = self.device.index or 0
        M, n = local.shape
        _lib.check(_lib.lib().light_b200_allgather_ll(C.c_void_p(local.data_ptr()), C.c_void_p(self.outs[index].data_ptr()),
                                                      C.byref(self.peers[index]), M, n, C.c_void_p(self.step.data_ptr()), dev,
                                                      C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)))
        return self.outs[index]

    def status(self) -> int:
        from . import _lib

        return _lib.lib().light_b200_comm_status(self.device.index or 0)


class FusedExchange:
    """Row-split decode with the exchange inside the matmul launches (light_b200_matmul_q_tp): the
    producing launch stores every value it owns, tagged with the step, into every rank's receive buffer
    for that output, and the consuming launch polls its own receive buffer while it loads its activations.
    No gather launch, no collective, no fence.

    plan(widths) lays out one receive buffer (2 * N slots of 8 bytes) per exchanged output identically on
    all ranks in symmetric memory (torch.distributed._symmetric_memory: plumbing only).
    """

    def __init__(self, device: torch.device, group=None):
        import torch.distributed as dist

        self.device, self.group = device, group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)

    def plan(self, widths: list[int]) -> None:
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        offs, total = [], 0
        for N in widths:
            offs.append(total)
            total += (2 * N * 8 + 255) // 256 * 256
        arena = symm_mem.empty(max(total, 256), dtype=torch.uint8, device=self.device)
        arena.zero_()
        try:
            hdl = symm_mem.rendezvous(arena, self.group)
        except TypeError:
            hdl = symm_mem.rendezvous(arena, self.group.group_name)
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)
        self.arena, self.handle = arena, hdl
        ptrs = [int(p) for p in hdl.buffer_ptrs]
        self.slots = [[ptrs[r] + off for r in range(self.world)] for off in offs]  # [output][rank] -> address
        self.step = torch.zeros(1, dtype=torch.int32, device=self.device)

    def step_begin(self) -> None:
        import ctypes as C

        from . import _lib

        dev = self.device.index or 0
        _lib.check(_lib.lib().light_b200_comm_step_begin(C.c_void_p(self.step.data_ptr()), dev,
                                                         C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)))

    def args(self, x_from: int | None, outs_to: list[int | None]):
        """lb200_tp for one launch: activations from exchanged output `x_from` (None: plain x), output i to
        exchanged output outs_to[i] (None: stays local)."""
        from . import _lib

        a = _lib.TpArgs()
        a.x_slots = self.slots[x_from][self.rank] if x_from is not None else None
        for i, o in enumerate(outs_to):
            if o is not None:
                for r in range(self.world):
                    a.out_slots[i][r] = self.slots[o][r]
        a.step = self.step.data_ptr()
        a.world, a.rank = self.world, self.rank
        return a

    def matmul(self, ggml_type: int, x: torch.Tensor | None, ws: list[torch.Tensor], outs: list[torch.Tensor], K: int, args) -> None:
        """One row-split launch: ws are this rank's row slices (block bytes), outs its local (n_i,) f32 outputs."""
        import ctypes as C

        from . import _lib

        n = len(ws)
        wp = (C.c_void_p * n)(*[w.data_ptr() for w in ws])
        op = (C.c_void_p * n)(*[o.data_ptr() for o in outs])
        nn = (C.c_int32 * n)(*[o.numel() for o in outs])
        dev = self.device.index or 0
        _lib.check(_lib.lib().light_b200_matmul_q_tp(ggml_type, C.c_void_p(x.data_ptr() if x is not None else 0), wp, op, nn, n, K,
                                                     C.byref(args), dev, C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)))

    def read(self, index: int, N: int, timeout_s: float = 2.0) -> torch.Tensor:
        """The exchanged output `index` of the step last begun, as (N,) f32 (test helper: synchronises).

        A local synchronise only proves that THIS rank's launches are done: a slower peer may still be storing
        its part of an output that no local launch has consumed yet.  So the slots' tags are compared with the
        step word, and re-read until they all match; after timeout_s a RuntimeError names the stale slots."""
        import time

        torch.cuda.synchronize(self.device)
        step = int(self.step.item()) & 0xFFFFFFFF
        par = step & 1
        off = self.slots[index][self.rank] - int(self.handle.buffer_ptrs[self.rank])
        t0 = time.time()
        while True:
            sl = self.arena[off + par * N * 8: off + (par + 1) * N * 8].view(torch.int32).view(N, 2).clone()
            stale = int((sl[:, 1].to(torch.int64) & 0xFFFFFFFF != step).sum().item())
            if stale == 0:
                return sl[:, 0].contiguous().view(torch.float32).clone()
            if time.time() - t0 > timeout_s:
                raise RuntimeError(f"FusedExchange.read: {stale} of {N} slots of output {index} do not carry step {step}")
            time.sleep(0.001)

    def status(self) -> int:
        from . import _lib

        return _lib.lib().light_b200_comm_status(self.device.index or 0)


def build_chain_symmetric(chain, group=None) -> None:
    """Builds a row-split chain.DecodeChain whose chain vectors live in symmetric memory: every rank allocates an
    arena of the same size, the ranks exchange the addresses (torch.distributed._symmetric_memory: plumbing only),
    and each rank's program stores its output slots into all of them.  Call on every rank with the same program."""
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm_mem

    group = group if group is not None else dist.group.WORLD
    nbytes = chain.arena_bytes()
    arena = symm_mem.empty(nbytes + 256, dtype=torch.uint8, device=chain.device)
    arena.zero_()
    try:
        hdl = symm_mem.rendezvous(arena, group)
    except TypeError:
        hdl = symm_mem.rendezvous(arena, group.group_name)
    torch.cuda.synchronize(chain.device)
    dist.barrier(group)
    ptrs = [int(p) for p in hdl.buffer_ptrs]
    chain._symm = (arena, hdl)
    chain.build(arenas=[p + (-p) % 256 for p in ptrs], arena=arena)
    torch.cuda.synchronize(chain.device)
    dist.barrier(group)   # nobody stores into an arena that its owner is still zeroing


class ExpertParallel:
    """Mixture-of-experts layer with the experts sharded over the ranks (E / P contiguous experts each)
    and a token all-to-all on either side of the local grouped matmuls -- the multi-GPU form of the
    reference's single-GPU sparse block (nn/moe.go:121-237: route, grouped GEMMs in expert order,
    combine).  Every rank brings its own tokens.

        dispatch : pairs (token, slot) sorted by expert are one contiguous run per destination rank
                   (split_pairs_by_rank); their hidden rows and expert ids go out in one all-to-all each
        local    : the receiver regroups the rows it got (from all ranks) by local expert and runs
                   `ffn(rows, routing_local)` -- on a GPU the grouped tensor-core matmuls of this
                   library (ops.MoEGemm / MoEGemmQ / MoEGemmF8Block with row_per_pair), on CPU whatever
                   the test injects
        combine  : results travel back with the split sizes reversed, and each token sums its top-k
                   rows with the routing weights (ops.MoECombine's arithmetic)

    The exchange is torch.distributed.all_to_all_single (NCCL over NVLink on GPUs, gloo in the CPU
    tests): a real exchange step, the one place on this path where a collective is the right tool.
    """

    def __init__(self, num_experts: int, group=None):
        import torch.distributed as dist

        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.E = num_experts
        self.lo, self.hi = expert_range(num_experts, self.rank, self.world)

    def plan(self, topk_ids: torch.Tensor, routing=None):
        """Routing of this rank's tokens: (sorted_pairs, sorted_expts, send_counts, recv_counts).  `routing`
        (ops.MoERouting of the same ids, from the router) brings the expert order the router already made; the
        counts of all ranks and the range check of all ids take one exchange and one read on the host, and a bad
        id on any rank raises on every rank (nobody is left waiting in the next exchange)."""
        import torch.distributed as dist

        T, topk = topk_ids.shape
        if routing is not None and routing.sorted_pairs is not None and routing.sorted_expts is not None:
            sorted_expts, sorted_pairs = routing.sorted_expts, routing.sorted_pairs
            if sorted_pairs.numel() != T * topk:
                raise ValueError(f"ExpertParallel: routing holds {sorted_pairs.numel()} pairs, the ids {T * topk}")
        else:
            sorted_expts, sorted_pairs = torch.sort(topk_ids.reshape(T * topk).to(torch.int64), stable=True)
        offs = split_pairs_by_rank(sorted_expts, self.E, self.world)
        ends = torch.stack([sorted_expts[0], sorted_expts[-1]]) if T * topk else torch.zeros(2, dtype=torch.int64, device=topk_ids.device)
        mine = torch.cat([(offs[1:] - offs[:-1]).to(torch.int64), ends.to(torch.int64)])
        table = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(table, mine, group=self.group)
        table = torch.stack(table).tolist()
        for r, row in enumerate(table):
            if row[self.world] < 0 or row[self.world + 1] >= self.E:
                raise ValueError(f"ExpertParallel: expert id outside [0, {self.E}) on rank {r}")
        return sorted_pairs, sorted_expts, table[self.rank][:self.world], [table[r][self.rank] for r in range(self.world)]

    def forward(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor, ffn, routing=None) -> torch.Tensor:
        """x (T, H) this rank's tokens, topk_ids / topk_weights (T, topk); ffn(rows (R, H), order (R,) int64,
        local_expert_of_order (R,) int64 non-decreasing) -> (R, H_out) rows in the order it was given them.
        `routing`: the router's ops.MoERouting for these ids, when there is one (its expert order is reused).
        Returns (T, H_out) f32."""
        import torch.distributed as dist

        T, topk = topk_ids.shape
        sorted_pairs, sorted_expts, send, recv = self.plan(topk_ids, routing)
        rows = x.index_select(0, sorted_pairs // topk).contiguous()
        R = sum(recv)
        got_rows = torch.empty(R, x.shape[1], dtype=x.dtype, device=x.device)
        got_expts = torch.empty(R, dtype=torch.int64, device=x.device)
        dist.all_to_all_single(got_rows, rows, output_split_sizes=recv, input_split_sizes=send, group=self.group)
        dist.all_to_all_single(got_expts, sorted_expts.contiguous(), output_split_sizes=recv, input_split_sizes=send, group=self.group)
        # what arrived is sorted by expert inside each source rank's run: regroup over all runs
        local_sorted, order = torch.sort(got_expts - self.lo, stable=True)
        done = ffn(got_rows, order, local_sorted)
        back = torch.empty(rows.shape[0], done.shape[1], dtype=done.dtype, device=x.device)
        dist.all_to_all_single(back, done.contiguous(), output_split_sizes=send, input_split_sizes=recv, group=self.group)
        w = topk_weights.reshape(T * topk).float()
        if back.is_cuda and back.shape[1] % 8 == 0 and back.dtype in (torch.float32, torch.bfloat16, torch.float16):
            from . import ops

            # row of every pair in `back`, then one launch: weight, sum over the slots in slot order, f32
            where = torch.empty(T * topk, dtype=torch.int64, device=x.device)
            where[sorted_pairs] = torch.arange(T * topk, dtype=torch.int64, device=x.device)
            return ops.MoECombineWeighted(back, where, w, T, topk)
        out = torch.zeros(T, done.shape[1], dtype=torch.float32, device=x.device)
        out.index_add_(0, sorted_pairs // topk, back.float() * w.index_select(0, sorted_pairs)[:, None])
        return out
