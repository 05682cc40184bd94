"""Expert parallelism on two or more GPUs, one process per GPU: tokens of every rank are dispatched by
all-to-all to the rank that owns their experts, run through this library's grouped matmuls there
(SwiGLU expert: gate_up, SiLU * up, down), and come back; the result must equal the same sparse block
computed on one GPU with all experts.  Skipped on a single-GPU box."""
import datetime
import os
import socket
import time

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
    # (a short collective timeout: a rank that fails leaves at once, and the others then report their aborted
    # collective instead of waiting for it)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=120))
    failed = False
    try:
        from light_b200 import ops, tp

        E, H, I, topk = 4 * world, 256, 128, 2
        g = torch.Generator().manual_seed(5)
        W1 = (torch.randn(E, 2 * I, H, generator=g) * 0.05).to(torch.bfloat16).to(dev)
        W2 = (torch.randn(E, H, I, generator=g) * 0.05).to(torch.bfloat16).to(dev)
        ep = tp.ExpertParallel(E)

        def expert_block(rows, order, expts, w1, w2):
            r = ops.MoERouting(None, None, order.contiguous(), expts.contiguous())
            h = ops.MoEGemm(rows, w1, r, None, 1)
            act = (torch.nn.functional.silu(h[:, :I].float()) * h[:, I:].float()).to(torch.bfloat16)
            return ops.MoEGemm(act, w2, r, None, 1)

        for T in (48, 300):
            gt = torch.Generator().manual_seed(10 * T + rank)
            x = torch.randn(T, H, generator=gt).to(torch.bfloat16).to(dev)
            logits = torch.randn(T, E, generator=gt)
            w, ids = torch.topk(torch.softmax(logits, 1), topk, dim=1)
            w, ids = w.to(dev), ids.to(dev)
            got = ep.forward(x, ids, w, lambda rows, order, le: expert_block(rows, order, le, W1[ep.lo:ep.hi], W2[ep.lo:ep.hi]))
            # one GPU, all experts, same tokens
            flat = ids.reshape(-1)
            se, sp = torch.sort(flat, stable=True)
            rows = x.index_select(0, sp // topk)
            order = torch.arange(rows.shape[0], device=dev)
            y = expert_block(rows, order, se, W1, W2)
            want = torch.zeros(T, H, device=dev)
            want.index_add_(0, sp // topk, y.float() * w.reshape(-1).index_select(0, sp)[:, None])
            torch.cuda.synchronize(dev)
            err = ((got - want).norm() / want.norm()).item()
            assert err <= 1e-3, f"rank {rank} T={T} rel err {err}"
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        failed = True
        q.put((rank, repr(e)))
    finally:
        if not failed:
            dist.barrier()
            torch.cuda.synchronize(dev)
        time.sleep(0.5)  # (let the queue's feeder thread send)
        os._exit(1 if failed else 0)


def test_expert_parallel_matches_single_gpu():
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
    res, deadline = {}, time.time() + 600
    while len(res) < world and time.time() < deadline:
        try:
            r, msg = q.get(timeout=5)
            res[r] = msg
        except Exception:  # noqa: BLE001  (queue.Empty: keep waiting while any worker lives)
            if not any(p.is_alive() for p in procs):
                break
    for p in procs:
        p.join(30)
        if p.is_alive():
            p.terminate()
    assert res == {r: "ok" for r in range(world)}, res
