"""GPU parity of the fused decode launches over quantized weights (matmul_q_multi, matmul_q_gated),
the quantized twins of the reference's ops.LinearMulti / ops.GatedLinear (ops/gemv.go:21-140).
The reference tests those against separate Linear calls (ops/gemv_test.go); here the bar is the same
plus the f64 oracle: a fused launch must return what one MatMulQ per weight returns."""
import ctypes as C
import math

import numpy as np
import pytest
import torch

from helpers import rel_l2
from light_b200 import _lib, ops, synth

pytestmark = pytest.mark.gpu


def _qt(raw, dt, shape, dev):
    t = raw if isinstance(raw, torch.Tensor) else torch.from_numpy(raw)
    return ops.QTensor(t.reshape(-1).to(dev), dt, shape)


def _deq(oracle, dt, raw, N, K):
    r = raw.numpy() if isinstance(raw, torch.Tensor) else raw
    return oracle.dequant(dt, r.reshape(-1), N * K).reshape(N, K).astype(np.float64)


@pytest.mark.parametrize("Ns,K", [((4096, 1024, 1024), 4096), ((16, 17, 4097, 33), 1024), ((48,), 256), ((1000, 24), 2048)])
def test_multi_matches_single_and_oracle(cuda, oracle, Ns, K):
    """q/k/v-shaped trio and ragged heights (tiles that are pulled back to the last 16 rows, one K
    block only, four weights): bit-identical to one MatMulQ per weight, <= 1e-5 rel-L2 vs f64."""
    dt = ops.Q4_K
    raws = [synth.random_blocks(500 + i, dt, N, K) for i, N in enumerate(Ns)]
    ws = [_qt(r, dt, (N, K), cuda) for r, N in zip(raws, Ns)]
    x = torch.randn(1, K, generator=torch.Generator().manual_seed(9))
    outs = ops.MatMulQMulti(x.to(cuda), ws)
    for o, w, r, N in zip(outs, ws, raws, Ns):
        single = ops.MatMulQ(x.to(cuda), w)
        assert o.shape == (1, N)
        assert torch.equal(o, single)
        want = x.numpy().astype(np.float64) @ _deq(oracle, dt, r, N, K).T
        assert rel_l2(o.cpu().numpy(), want) <= 1e-5


def test_multi_falls_back_for_other_types(cuda, oracle):
    """Types without a fused multi kernel are served by one matmul per weight, same results."""
    K = 1024
    for dt in (ops.Q8_0, ops.Q6_K):
        raws = [synth.random_blocks(520 + i, dt, N, K) for i, N in enumerate((40, 24))]
        ws = [_qt(r, dt, (N, K), cuda) for r, N in zip(raws, (40, 24))]
        x = torch.randn(K, generator=torch.Generator().manual_seed(10))
        outs = ops.MatMulQMulti(x.to(cuda), ws)
        for o, w in zip(outs, ws):
            assert o.shape == (w.shape[0],)
            assert torch.equal(o.reshape(1, -1), ops.MatMulQ(x.reshape(1, K).to(cuda), w))


@pytest.mark.parametrize("N,K,gelu", [(14336, 4096, False), (40, 512, False), (1000, 1024, True)])
def test_gated_matches_unfused_and_oracle(cuda, oracle, N, K, gelu):
    """act(gate . x) * (up . x) with Gaussian Q4_K weights (the gate/up shape of the decoder) and
    ragged heights; vs the unfused sequence on the GPU and vs f64."""
    dt = ops.Q4_K
    rg, ru = synth.gaussian_weight(61, dt, N, K), synth.gaussian_weight(62, dt, N, K)
    wg, wu = _qt(rg, dt, (N, K), cuda), _qt(ru, dt, (N, K), cuda)
    x = torch.randn(1, K, generator=torch.Generator().manual_seed(11))
    got = ops.MatMulQGated(x.to(cuda), wg, wu, gelu=gelu)
    g, u = ops.MatMulQ(x.to(cuda), wg), ops.MatMulQ(x.to(cuda), wu)
    act = torch.nn.functional.gelu(g) if gelu else torch.nn.functional.silu(g)
    assert rel_l2(got.cpu().numpy(), (act * u).cpu().numpy()) <= 1e-6
    g64 = x.numpy().astype(np.float64) @ _deq(oracle, dt, rg, N, K).T
    u64 = x.numpy().astype(np.float64) @ _deq(oracle, dt, ru, N, K).T
    a64 = 0.5 * g64 * (1 + np.vectorize(math.erf)(g64 / math.sqrt(2))) if gelu else g64 / (1 + np.exp(-g64))
    assert rel_l2(got.cpu().numpy(), a64 * u64) <= 1e-5


def test_multi_and_gated_errors(cuda):
    L = _lib.lib()
    K = 512
    raw = synth.random_blocks(70, ops.Q4_K, 32, K)
    w = _qt(raw, ops.Q4_K, (32, K), cuda)
    x = torch.randn(1, K, device=cuda)
    with pytest.raises(ValueError):
        ops.MatMulQMulti(x, [w] * 5)
    with pytest.raises(ValueError):
        ops.MatMulQMulti(x.to(torch.bfloat16), [w])
    with pytest.raises(ValueError):
        ops.MatMulQMulti(torch.randn(2, K + 256, device=cuda), [w])
    w6 = _qt(synth.random_blocks(71, ops.Q6_K, 32, K), ops.Q6_K, (32, K), cuda)
    with pytest.raises(ops.Light200Error):
        ops.MatMulQGated(x, w6, w6)
    out = torch.empty(32, device=cuda)
    rc = L.light_b200_matmul_q_gated(ops.Q4_K, C.c_void_p(x.data_ptr()), C.c_void_p(w.data.data_ptr()),
                                     C.c_void_p(w.data.data_ptr()), C.c_void_p(out.data_ptr()), 32, K, 3, 0, None)
    assert rc != 0


@pytest.mark.parametrize("K", [4096, 2048, 256])
def test_norm_folded_into_the_launch(cuda, oracle, K):
    """RMSNorm(x [+ residual]) then LinearMulti / GatedLinear as one launch (light_b200_matmul_q_fused) against
    the oracle's RMSNorm followed by the f64 products; the residual sum comes back bit for bit."""
    g = torch.Generator().manual_seed(500 + K)
    ns = (256, 64, 80)
    raws = [synth.gaussian_weight(510 + i, ops.Q4_K, n, K).numpy() for i, n in enumerate(ns)]
    deqs = [oracle.dequant(ops.Q4_K, r.reshape(-1), n * K).reshape(n, K).astype(np.float64) for r, n in zip(raws, ns)]
    ws = [ops.QTensor(torch.from_numpy(r.reshape(-1)).to(cuda), ops.Q4_K, (n, K)) for r, n in zip(raws, ns)]
    x, r, nw = torch.randn(1, K, generator=g) * 3, torch.randn(1, K, generator=g), torch.randn(K, generator=g)
    for res in (None, r):
        s = x if res is None else x + res
        y = oracle.rmsnorm(s.numpy(), nw.numpy(), 1e-5).astype(np.float64)
        got = ops.NormMatMulQ(x.to(cuda), nw.to(cuda), 1e-5, ws, residual=None if res is None else res.to(cuda))
        if res is not None:
            got, total = got
            assert torch.equal(total.cpu(), s)
        for o, d in zip(got, deqs):
            assert rel_l2(o.cpu().numpy(), y @ d.T) <= 1e-4
    # gated pair: two matrices of equal height
    pair = [ws[1], ops.QTensor(torch.from_numpy(synth.gaussian_weight(520, ops.Q4_K, 64, K).numpy().reshape(-1)).to(cuda), ops.Q4_K, (64, K))]
    du = oracle.dequant(ops.Q4_K, synth.gaussian_weight(520, ops.Q4_K, 64, K).numpy().reshape(-1), 64 * K).reshape(64, K).astype(np.float64)
    y = oracle.rmsnorm((x + r).numpy(), nw.numpy(), 1e-5).astype(np.float64)
    got, total = ops.NormMatMulQ(x.to(cuda), nw.to(cuda), 1e-5, pair, residual=r.to(cuda), gate="silu")
    gl, up = y @ deqs[1].T, y @ du.T
    assert rel_l2(got.cpu().numpy(), gl / (1 + np.exp(-gl)) * up) <= 1e-4
    assert torch.equal(total.cpu(), x + r)


@pytest.mark.parametrize("M", [2, 5, 8, 9, 16, 27, 32, 40])
def test_multi_for_a_small_batch(cuda, oracle, M):
    """LinearMulti for 2..8 rows of x as one launch of the token-column kernel (q, k, v heights of configs[1] scaled
    down, a ragged one among them), of the eight-tiles-per-CTA kernel for 9..32 rows; 40 rows fall back to one
    launch per matrix: same results either way."""
    K = 2048
    ns = (256, 64, 72)
    raws = [synth.gaussian_weight(530 + i, ops.Q4_K, n, K).numpy() for i, n in enumerate(ns)]
    ws = [ops.QTensor(torch.from_numpy(r.reshape(-1)).to(cuda), ops.Q4_K, (n, K)) for r, n in zip(raws, ns)]
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(540 + M))
    outs = ops.MatMulQMulti(x.to(cuda), ws)
    for o, w, r, n in zip(outs, ws, raws, ns):
        assert o.shape == (M, n)
        assert torch.equal(o, ops.MatMulQ(x.to(cuda), w))  # the same kernel arithmetic, tile by tile
        deq = oracle.dequant(ops.Q4_K, r.reshape(-1), n * K).reshape(n, K).astype(np.float64)
        assert rel_l2(o.cpu().numpy(), x.numpy().astype(np.float64) @ deq.T) <= 1e-3
