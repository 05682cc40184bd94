"""The NVLink peer-store all-gather (light_b200_allgather_ll) on two or more GPUs, one process per GPU:
several steps with fresh data each, two gathered operators per step, against NCCL's all-gather.
Skipped on a single-GPU box."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from light_b200 import tp

        pg = tp.PeerGather(dev)
        shapes = [(1, 512 * world), (3, 64 * world)]
        outs = pg.plan(shapes)
        for step in range(5):
            pg.step_begin()
            for i, (M, N) in enumerate(shapes):
                g = torch.Generator(device=dev)
                g.manual_seed(1000 * step + 10 * i + rank)
                local = torch.randn(M, N // world, generator=g, device=dev)
                got = pg.gather(i, local)
                want = tp.all_gather_columns(local)
                torch.cuda.synchronize(dev)
                assert torch.equal(got, want), f"rank {rank} step {step} op {i}"
        assert pg.status() == 0
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        q.put((rank, repr(e)))
    finally:
        dist.barrier()
        torch.cuda.synchronize(dev)
        os._exit(0)


def test_allgather_ll_matches_nccl():
    world = torch.cuda.device_count()
    if world < 2:
        pytest.skip("needs at least two GPUs")
    world = min(world, 8)
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=240) for _ in procs)
    for p in procs:
        p.join(60)
    assert res == {r: "ok" for r in range(world)}, res
