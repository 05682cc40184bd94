"""The sticky device-side status words, each exercised in a process of its own (a word, once set, stays set
for the life of the process, and every other test asserts that it is zero).

None of these cases faults or hangs the GPU: a bounded wait runs out after about 50 ms and the kernel
returns, a bad expert id or position is clamped or skipped.  What is checked is that the library notices,
reports, and leaves neighbouring memory alone.
"""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PRELUDE = """
import ctypes as C, sys, time
import torch
sys.path.insert(0, %r)
from light_b200 import _lib, ops, synth
L = _lib.lib()
_lib.check(L.light_b200_init(0))
dev = torch.device("cuda:0")
P = lambda t: C.c_void_p(t.data_ptr())
""" % ROOT


def run_case(body: str, timeout=300):
    r = subprocess.run([sys.executable, "-c", PRELUDE + textwrap.dedent(body)], capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, f"child failed:\nSTDOUT:\n{r.stdout}\nSTDERR:\n{r.stderr[-4000:]}"
    assert "CASE OK" in r.stdout, r.stdout


def test_moe_bad_expert_ids_are_contained(cuda):
    """Expert ids -1 and E (and far outside) in the sorted id list: counts / offsets keep their guard bands,
    pairs with such ids are skipped, the rest is computed, and the status word reports it."""
    run_case("""
    E, N, K, G = 5, 16, 32, 64
    for ids_l in ([-1, 0, 0, 2, 4, E], [-(1 << 40), -3, 1, 3, 3, 1 << 40], [-1] * 6, [E] * 6):
        ids = torch.tensor(ids_l, dtype=torch.int64, device=dev)
        M = ids.numel()
        pairs = torch.arange(M, dtype=torch.int64, device=dev)
        guard = torch.full((G + E + G + E + 1 + G,), -7, dtype=torch.int32, device=dev)
        counts, offsets = guard[G:G + E], guard[G + E + G:G + E + G + E + 1]
        x = torch.randn(M, K, device=dev)
        w = torch.randn(E, N, K, device=dev)
        out = torch.full((M, N), 123.0, device=dev)
        a = _lib.MoeArgs(input=x.data_ptr(), weights=w.data_ptr(), sorted_pairs=pairs.data_ptr(), expert_ids=ids.data_ptr(),
                         counts=counts.data_ptr(), offsets=offsets.data_ptr(), topk_weights=None, out=out.data_ptr(), M=M, size_m=M,
                         E=E, N=N, K=K, topk=1, row_per_pair=1, dtype=_lib.F32)
        _lib.check(L.light_b200_moe_gemm(C.byref(a), 0, None))
        torch.cuda.synchronize()
        g = guard.cpu()
        assert (g[:G] == -7).all() and (g[G + E:G + E + G] == -7).all() and (g[-G:] == -7).all(), ("guard bands", ids_l, g.tolist())
        off = offsets.cpu().tolist()
        assert all(0 <= o <= M for o in off) and off == sorted(off), off
        assert off[-1] == sum(1 for e in ids_l if e < E), off      # offsets[E]: the first pair whose id is not an expert
        for i, e in enumerate(ids_l):
            row = out[i].cpu()
            if 0 <= e < E:
                want = (x[i] @ w[e].T).cpu()
                assert torch.allclose(row, want, rtol=1e-4, atol=1e-4), (ids_l, i)
            else:
                assert (row == 123.0).all(), (ids_l, i)
        # the same through the entry point that keeps counts / offsets in the library's own array
        out.fill_(123.0)
        _lib.check(L.light_b200_moe_gemm_static_scratch(C.byref(a), 0, None))
        torch.cuda.synchronize()
        for i, e in enumerate(ids_l):
            if not 0 <= e < E:
                assert (out[i].cpu() == 123.0).all(), (ids_l, i)
    assert L.light_b200_moe_route_status(0) == 1
    print("CASE OK")
    """)


def test_decode_attn_position_outside_cache_appends_nothing(cuda):
    """The append inside the attention launch and light_b200_kv_append agree in the error case too: a
    position outside [0, Cap) leaves the cache as it was and sets the status word."""
    run_case("""
    import math
    B, NH, KH, Cap, D = 1, 8, 2, 64, 128
    g = torch.Generator(device=dev); g.manual_seed(3)
    kb = torch.randn(B, KH, Cap, D, generator=g, device=dev); vb = torch.randn(B, KH, Cap, D, generator=g, device=dev)
    q = torch.randn(B, NH, 1, D, generator=g, device=dev)
    kn = torch.randn(B, KH, 1, D, generator=g, device=dev); vn = torch.randn(B, KH, 1, D, generator=g, device=dev)
    outs = []
    for pos_v in (Cap, -1, Cap + 1000):
        pos = torch.tensor([pos_v], dtype=torch.int64, device=dev)
        k0, v0 = kb.clone(), vb.clone()
        out = torch.zeros(B, NH, 1, D, device=dev)
        a = _lib.DecodeAttnArgs(q.data_ptr(), k0.data_ptr(), v0.data_ptr(), kn.data_ptr(), vn.data_ptr(), pos.data_ptr(), out.data_ptr(),
                                _lib.F32, B, NH, KH, Cap, D, 0, 1.0 / math.sqrt(D), 0.0)
        _lib.check(L.light_b200_decode_attn(C.byref(a), 0, None))
        # append-then-attend
        k1, v1 = kb.clone(), vb.clone()
        out1 = torch.zeros(B, NH, 1, D, device=dev)
        _lib.check(L.light_b200_kv_append(P(kn), P(vn), P(k1), P(v1), P(pos), _lib.F32, B, KH, D, Cap, 0, None))
        a1 = _lib.DecodeAttnArgs(q.data_ptr(), k1.data_ptr(), v1.data_ptr(), None, None, pos.data_ptr(), out1.data_ptr(),
                                 _lib.F32, B, NH, KH, Cap, D, 0, 1.0 / math.sqrt(D), 0.0)
        _lib.check(L.light_b200_decode_attn(C.byref(a1), 0, None))
        torch.cuda.synchronize()
        assert torch.equal(k0, kb) and torch.equal(v0, vb), pos_v
        assert torch.equal(k1, kb) and torch.equal(v1, vb), pos_v
        assert torch.equal(out, out1), pos_v
        assert torch.isfinite(out).all()
    assert L.light_b200_decode_attn_status(0) == 1
    print("CASE OK")
    """)


def test_allgather_wait_runs_out(cuda):
    """A gather whose peer never sends: the bounded wait gives up after about 50 ms, the call returns, the
    status word is set, and the context stays usable.  (One GPU stands in for rank 0 of 2; rank 1's receive
    buffer is local memory that nobody reads.)"""
    run_case("""
    M, n = 1, 256
    slots0 = torch.zeros(2 * M * 2 * n * 2, dtype=torch.int32, device=dev)   # 2 sets x M x (2 n) slots x 8 bytes
    slots1 = torch.zeros_like(slots0)
    step = torch.zeros(1, dtype=torch.int32, device=dev)
    peers = _lib.Peers(world=2, rank=0)
    peers.slots[0], peers.slots[1] = slots0.data_ptr(), slots1.data_ptr()
    local = torch.randn(M, n, device=dev)
    out = torch.zeros(M, 2 * n, device=dev)
    assert L.light_b200_comm_status(0) == 0
    _lib.check(L.light_b200_comm_step_begin(P(step), 0, None))
    t0 = time.time()
    _lib.check(L.light_b200_allgather_ll(P(local), P(out), C.byref(peers), M, n, P(step), 0, None))
    torch.cuda.synchronize()
    dt = time.time() - t0
    assert dt < 5.0, dt
    assert L.light_b200_comm_status(0) == 1
    assert torch.equal(out[:, :n], local)          # this rank's own columns are there
    y = torch.ones(8, device=dev) * 2              # the context is alive
    assert float(y.sum().item()) == 16.0
    print("CASE OK")
    """)


def test_matmul_q_tp_wait_runs_out(cuda):
    """The in-launch exchange with activations that never arrive (slots never tagged): the poll gives up after
    about 50 ms, the launch ends, light_b200_comm_status reports it."""
    run_case("""
    N, K = 64, 1024
    raw = synth.gaussian_weight(5, ops.Q4_K, N, K, device=dev)
    x_slots = torch.zeros(2 * K * 2, dtype=torch.int32, device=dev)     # two parities x K slots x 8 bytes, never tagged
    step = torch.zeros(1, dtype=torch.int32, device=dev)
    out = torch.zeros(N, device=dev)
    a = _lib.TpArgs()
    a.x_slots = x_slots.data_ptr()
    a.step = step.data_ptr()
    a.world, a.rank = 2, 0
    wp = (C.c_void_p * 1)(raw.data_ptr()); op = (C.c_void_p * 1)(out.data_ptr()); nn = (C.c_int32 * 1)(N)
    assert L.light_b200_comm_status(0) == 0
    _lib.check(L.light_b200_comm_step_begin(P(step), 0, None))
    t0 = time.time()
    _lib.check(L.light_b200_matmul_q_tp(ops.Q4_K, None, wp, op, nn, 1, K, C.byref(a), 0, None))
    torch.cuda.synchronize()
    dt = time.time() - t0
    assert dt < 5.0, dt
    assert L.light_b200_comm_status(0) == 1
    y = torch.ones(8, device=dev) * 2
    assert float(y.sum().item()) == 16.0
    print("CASE OK")
    """)
