"""Batched decode with the tokens as MMA columns over activations staged once per call (Q4_K and Q6_K, 2 to 64
activation rows; reference cutover ops/matmul_q.go:52-60, kernel contract kernels/cuda/matmul_q.go:44-91).  The
oracle is the f64 product with the CPU-dequantized weights, as in ops/matmul_q_test.go:105-146."""
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest
import torch

from helpers import rel_l2
from light_b200 import ops, synth

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _weight(seed, dt, N, K, cuda, oracle):
    raw = synth.gaussian_weight(seed, dt, N, K).numpy()
    deq = oracle.dequant(dt, raw.reshape(-1), N * K).reshape(N, K).astype(np.float64)
    return ops.QTensor(torch.from_numpy(raw.reshape(-1)).to(cuda), dt, (N, K)), deq


@pytest.mark.parametrize("dt,N,K", [(ops.Q4_K, 4096, 4096), (ops.Q4_K, 16, 256), (ops.Q4_K, 300, 1280), (ops.Q4_K, 2064, 768),
                                     (ops.Q6_K, 4096, 2048), (ops.Q6_K, 16, 512), (ops.Q6_K, 300, 3584), (ops.Q6_K, 1030, 14336)])
def test_token_tiles(cuda, oracle, dt, N, K):
    """One to 56 blocks per row (clusters of 1 to 8, K runs of uneven length), a single row tile, ragged heights
    (a last tile that overlaps the one before, CTAs with fewer than eight live tiles), token counts that fill two,
    four and eight groups of eight partly and fully; the same bits twice."""
    w, deq = _weight(500 + N, dt, N, K, cuda, oracle)
    g = torch.Generator().manual_seed(501)
    for M in (9, 16, 17, 31, 32, 33, 57, 64):
        x = torch.randn(M, K, generator=g)
        got = ops.MatMulQ(x.to(cuda), w)
        assert torch.equal(got, ops.MatMulQ(x.to(cuda), w)), "the cluster reduction must be deterministic"
        err = rel_l2(got.cpu().numpy(), x.numpy().astype(np.float64) @ deq.T)
        assert err <= 1e-3, (dt, N, K, M, err)
    assert ops.prefill_status(cuda.index or 0) == 0


@pytest.mark.parametrize("dt", [ops.Q4_K, ops.Q6_K])
def test_token_tiles_shared_activations(cuda, oracle, dt):
    """Several matrices that share x in one launch (q, k, v heights; gate and up): every output equals the
    single-matrix call bit for bit."""
    K = 2048
    hs = (512, 128, 144)
    ws = [_weight(510 + i, dt, n, K, cuda, oracle) for i, n in enumerate(hs)]
    g = torch.Generator().manual_seed(511)
    for M in (12, 32, 64):
        x = torch.randn(M, K, generator=g).to(cuda)
        outs = ops.MatMulQMulti(x, [w for w, _ in ws])
        for (w, deq), o in zip(ws, outs):
            assert o.shape == (M, w.shape[0])
            assert torch.equal(o, ops.MatMulQ(x, w))
            assert rel_l2(o.cpu().numpy(), x.cpu().numpy().astype(np.float64) @ deq.T) <= 1e-3
    assert ops.prefill_status(cuda.index or 0) == 0


def test_token_tiles_extreme_values(cuda, oracle):
    """Activations beyond the f16 range are clamped, as in the other tensor-core paths; zeros and a constant row
    (the minimum term alone) come out exactly as the oracle's."""
    N, K, M = 64, 1024, 16
    w, deq = _weight(520, ops.Q4_K, N, K, cuda, oracle)
    x = torch.zeros(M, K)
    x[1] = 1.0
    x[2, ::7] = -3.5
    x[3] = torch.randn(K, generator=torch.Generator().manual_seed(521)) * 1e-3
    got = ops.MatMulQ(x.to(cuda), w).cpu().numpy()
    want = x.numpy().astype(np.float64) @ deq.T
    assert np.all(got[0] == 0) and np.all(got[4:] == 0)
    assert rel_l2(got[1:4], want[1:4]) <= 1e-3
    big = torch.full((M, K), 1e6)
    assert bool(torch.isfinite(ops.MatMulQ(big.to(cuda), w)).all())


CHILD = """
import sys, numpy as np, torch
sys.path.insert(0, %r)
from light_b200 import ops, synth
from oracle import binding as oracle
oracle.build()
dev = torch.device("cuda:0")
for dt, N, K in ((ops.Q4_K, 300, 1280), (ops.Q6_K, 272, 2048), (ops.Q4_K, 4096, 4096)):
    raw = synth.gaussian_weight(530, dt, N, K).numpy()
    deq = oracle.dequant(dt, raw.reshape(-1), N * K).reshape(N, K).astype(np.float64)
    w = ops.QTensor(torch.from_numpy(raw.reshape(-1)).to(dev), dt, (N, K))
    g = torch.Generator().manual_seed(531)
    for M in %s:
        x = torch.randn(M, K, generator=g)
        got = ops.MatMulQ(x.to(dev), w).cpu().numpy()
        want = x.numpy().astype(np.float64) @ deq.T
        err = float(np.linalg.norm(got - want) / np.linalg.norm(want))
        assert err <= 1e-3, (dt, N, K, M, err)
assert ops.prefill_status(0) == 0
print("CASE OK")
""" % (ROOT, "%s")


@pytest.mark.parametrize("env,ms", [({"LIGHT_B200_NT_MIN_M": "2"}, "(2, 3, 8)"), ({"LIGHT_B200_NT_MAX_M": "0"}, "(9, 32, 64)"),
                                    ({"LIGHT_B200_TS": "1"}, "(1, 5, 16, 17, 32, 33, 64)"), ({"LIGHT_B200_TS": "1", "LIGHT_B200_TS_GRID": "7"}, "(1, 32, 64)")])
def test_token_tiles_row_count_knobs(cuda, env, ms):
    """The same kernels serve 2 to 8 rows when asked to (one group of eight); with the path switched off the
    earlier kernels still serve 9 to 64 rows; and the kernel that hands the expanded weights to tcgen05.mma through
    tensor memory (opt-in) serves 1 to 64 rows of Q4_K, also when a grid of 7 CTAs cuts every group's K range into
    partial sums."""
    r = subprocess.run([sys.executable, "-c", textwrap.dedent(CHILD % ms)], capture_output=True, text=True, timeout=600, env={**os.environ, **env})
    assert r.returncode == 0 and "CASE OK" in r.stdout, r.stdout + r.stderr[-3000:]
