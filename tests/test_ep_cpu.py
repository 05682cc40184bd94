"""Expert parallelism, host logic and exchange, as two and four gloo ranks on CPU: each rank routes its own
tokens, the pairs travel to the rank that owns their expert, a stand-in expert function (a dense matmul
per expert in torch, the arithmetic of kernels/cpu/moe.go:51-123) runs there, and the combined output
equals the single-rank sparse block (nn/moe.go:121-237) on the same tokens."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from light_b200 import tp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _reference(x, ids, w, W):
    """Every token: sum over its slots of weight * (x . W[e]^T)."""
    out = torch.zeros(x.shape[0], W.shape[1], dtype=torch.float64)
    for t in range(x.shape[0]):
        for s in range(ids.shape[1]):
            out[t] += w[t, s].double() * (W[ids[t, s]].double() @ x[t].double())
    return out


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        E, H, O, topk = 8, 16, 12, 3
        g = torch.Generator().manual_seed(77)
        W = torch.randn(E, O, H, generator=g)              # every rank draws all experts, keeps its own
        ep = tp.ExpertParallel(E)
        Wl = W[ep.lo:ep.hi]
        for T in (5, 1, 0, 9):                             # ragged, and a rank with no tokens at all
            gt = torch.Generator().manual_seed(100 * T + rank)
            x = torch.randn(T, H, generator=gt)
            logits = torch.randn(T, E, generator=gt) + (torch.arange(E) < 2) * 2.0   # skew towards rank 0's experts
            w, ids = torch.topk(torch.softmax(logits, 1), topk, dim=1) if T else (torch.zeros(0, topk), torch.zeros(0, topk, dtype=torch.int64))

            def ffn(rows, order, local_e):
                out = torch.empty(rows.shape[0], O)
                for i in range(rows.shape[0]):
                    out[order[i]] = Wl[local_e[i]] @ rows[order[i]]
                assert bool((local_e[1:] >= local_e[:-1]).all()) and (rows.shape[0] == 0 or 0 <= int(local_e.min()) and int(local_e.max()) < E // world)
                return out

            got = ep.forward(x, ids, w, ffn)
            want = _reference(x, ids, w, W)
            assert got.shape == (T, O)
            assert torch.allclose(got.double(), want, rtol=1e-5, atol=1e-5), f"rank {rank} T={T}"
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        q.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_ranks(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(30)
    assert res == {r: "ok" for r in range(world)}, res
