"""Host logic of the multi-GPU placement, run as two gloo ranks on CPU (no GPU needed): each rank
computes its row slice with the oracle, the slices are all-gathered, and the result equals the
single-rank result bit for bit."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from light_b200 import synth, tp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import binding as ob

        N, K, dt = 64, 512, ob.Q4_K
        w = torch.from_numpy(synth.random_blocks(5, dt, N, K))
        for M in (1, 3):
            x = torch.randn(M, K, generator=torch.Generator().manual_seed(6))
            mine = tp.shard_rows(w, rank, world)
            local = torch.from_numpy(ob.matmul_q(dt, x.numpy(), mine.contiguous().numpy(), N // world))
            full = tp.all_gather_columns(local)
            want = torch.from_numpy(ob.matmul_q(dt, x.numpy(), w.numpy(), N))
            assert torch.equal(full, want), f"rank {rank} M={M}"
        # expert parallelism: the sorted pair list splits into one contiguous run per rank
        se = torch.tensor([0, 0, 1, 3, 3, 3, 4, 6, 7, 7])
        offs = tp.split_pairs_by_rank(se, 8, world)
        assert offs.tolist() == [0, 6, 10]
        assert tp.expert_range(8, rank, world) == (4 * rank, 4 * rank + 4)
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        q.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


def test_row_split_all_gather_two_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(60)
    assert res == {0: "ok", 1: "ok"}, res


def test_row_range_errors():
    assert tp.row_range(128, 3, 4) == (96, 128)
    with pytest.raises(ValueError, match="do not split evenly"):
        tp.row_range(10, 0, 4)
    with pytest.raises(ValueError, match="outside world"):
        tp.row_range(8, 4, 4)
    w = torch.zeros(256, 4, dtype=torch.uint8)
    s = torch.zeros(2, 1)
    a, b = tp.shard_fp8_block(w, s, 128, 1, 2)
    assert a.shape[0] == 128 and b.shape[0] == 1
    with pytest.raises(ValueError, match="does not fall on"):
        tp.shard_fp8_block(w, s, 128, 0, 4)
