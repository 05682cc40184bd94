"""Row-split decode with the exchange inside the matmul launches (light_b200_matmul_q_tp) on two or more
GPUs, one process per GPU: a chain qkv (Q4_K, three matrices, q exchanged) -> o (Q4_K) -> down-like (Q6_K),
each fed by the previous exchanged output, several steps; every rank must end up with exactly what one GPU
computes with the full matrices.  Skipped on a single-GPU box."""
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
        from light_b200 import ops, synth, tp

        H, KV, F = 1024, 256, 2048      # q / o width, k / v width, "down" input width
        assert H % (16 * world) == 0 and KV % (16 * world) == 0 and F % (16 * world) == 0
        full = {"q": synth.gaussian_weight(1, ops.Q4_K, H, H), "k": synth.gaussian_weight(2, ops.Q4_K, KV, H),
                "v": synth.gaussian_weight(3, ops.Q4_K, KV, H), "o": synth.gaussian_weight(4, ops.Q4_K, F, H),
                "d": synth.gaussian_weight(5, ops.Q6_K, H, F)}
        mine = {k: tp.shard_rows(w, rank, world).contiguous().to(dev) for k, w in full.items()}
        fx = tp.FusedExchange(dev)
        fx.plan([H, F, H])              # exchanged: q, o, d
        a_qkv = fx.args(None, [0, None, None])
        a_o = fx.args(0, [1])
        a_d = fx.args(1, [2])
        loc = {k: torch.empty(w.shape[0], device=dev) for k, w in mine.items()}

        def qt(k, dt, K):  # one GPU, full matrices
            return ops.QTensor(full[k].reshape(-1).to(dev), dt, (full[k].shape[0], K))

        for step in range(4):
            x = torch.randn(1, H, generator=torch.Generator().manual_seed(50 + step)).to(dev)
            fx.step_begin()
            fx.matmul(ops.Q4_K, x, [mine["q"], mine["k"], mine["v"]], [loc["q"], loc["k"], loc["v"]], H, a_qkv)
            fx.matmul(ops.Q4_K, None, [mine["o"]], [loc["o"]], H, a_o)
            fx.matmul(ops.Q6_K, None, [mine["d"]], [loc["d"]], F, a_d)
            # q and o were consumed by a later local launch, which polled their tags; nothing local waited for the
            # peers' stores of d: read() polls the tags itself
            got_q, got_o, got_d = fx.read(0, H), fx.read(1, F), fx.read(2, H)
            want_q = ops.MatMulQ(x, qt("q", ops.Q4_K, H))
            want_o = ops.MatMulQ(want_q, qt("o", ops.Q4_K, H))
            want_d = ops.MatMulQ(want_o, qt("d", ops.Q6_K, F))
            want_k = ops.MatMulQ(x, qt("k", ops.Q4_K, H))
            torch.cuda.synchronize(dev)
            assert torch.equal(got_q, want_q.reshape(-1)), f"rank {rank} step {step}: q"
            assert torch.equal(got_o, want_o.reshape(-1)), f"rank {rank} step {step}: o"
            assert torch.equal(got_d, want_d.reshape(-1)), f"rank {rank} step {step}: d"
            lo, hi = tp.row_range(KV, rank, world)
            assert torch.equal(loc["k"], want_k.reshape(-1)[lo:hi]), f"rank {rank} step {step}: k (local)"
        # several steps enqueued back to back with no host synchronisation between them, so that the ranks run
        # skewed across steps (the case the two slot sets per output exist for); only the last step is checked
        xs = [torch.randn(1, H, generator=torch.Generator().manual_seed(90 + i)).to(dev) for i in range(6)]
        torch.cuda.synchronize(dev)
        for x in xs:
            fx.step_begin()
            fx.matmul(ops.Q4_K, x, [mine["q"], mine["k"], mine["v"]], [loc["q"], loc["k"], loc["v"]], H, a_qkv)
            fx.matmul(ops.Q4_K, None, [mine["o"]], [loc["o"]], H, a_o)
            fx.matmul(ops.Q6_K, None, [mine["d"]], [loc["d"]], F, a_d)
        torch.cuda.synchronize(dev)
        dist.barrier()
        got_d = fx.read(2, H)
        want_q = ops.MatMulQ(xs[-1], qt("q", ops.Q4_K, H))
        want_d = ops.MatMulQ(ops.MatMulQ(want_q, qt("o", ops.Q4_K, H)), qt("d", ops.Q6_K, F))
        assert torch.equal(got_d, want_d.reshape(-1)), f"rank {rank}: d after six unsynchronised steps"
        assert fx.status() == 0
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        import traceback

        q.put((rank, repr(e) + traceback.format_exc()[-600:]))
    finally:
        dist.barrier()
        torch.cuda.synchronize(dev)
        os._exit(0)


def test_fused_exchange_chain():
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
    res = dict(q.get(timeout=300) for _ in procs)
    for p in procs:
        p.join(60)
    assert res == {r: "ok" for r in range(world)}, res
