"""The persistent decode chain (light_b200_chain_*) through the C ABI: single operators against the f64 dot of the
bit-exact dequantized weights (the arbiter of ops/matmul_q_cpu_test.go:66-78), then programs of dependent
operators -- the shape of a decoder layer's linears, models/llama.go:1070-1330 -- against the same chain computed
operator by operator in f64."""
import numpy as np
import pytest
import torch

from helpers import rel_l2
from light_b200 import chain, ops, synth

pytestmark = pytest.mark.gpu


def _w(seed, dt, N, K, dev, oracle):
    raw = synth.gaussian_weight(seed, dt, N, K)
    deq = oracle.dequant(dt, raw.numpy().reshape(-1), N * K).reshape(N, K).astype(np.float64)
    return ops.QTensor(raw.reshape(-1).to(dev), dt, (N, K)), deq


@pytest.mark.parametrize("dt,N,K", [(ops.Q4_K, 304, 4096), (ops.Q4_K, 300, 1024), (ops.Q4_K, 16, 256), (ops.Q4_K, 5000, 4096),
                                    (ops.Q6_K, 200, 2048), (ops.Q6_K, 64, 14336), (ops.Q6_K, 4100, 4096)])
def test_single_operator(cuda, oracle, dt, N, K):
    w, deq = _w(11, dt, N, K, cuda, oracle)
    c = chain.DecodeChain(cuda)
    x = torch.randn(K, generator=torch.Generator().manual_seed(12)).to(cuda)
    out = torch.full((N + 64,), 7.0, device=cuda)  # guard band behind the output
    c.matmul([w], x=x, outs=[out[:N]])
    c.build()
    for rep in range(3):  # the step tag moves on; the result must not
        out[:N].zero_()
        c.run()
        torch.cuda.synchronize()
        want = deq @ x.cpu().numpy().astype(np.float64)
        assert rel_l2(out[:N].cpu().numpy(), want) <= 1e-5, (dt, N, K, rep)
        assert (out[N:] == 7.0).all()
    assert c.status() == 0


def test_random_bytes_and_wide_range_activations(cuda, oracle):
    """Every code value and scale pattern (random bytes, f16 scales pinned to [2^-6, 2^-5), ops/matmul_q_test.go:19-56)
    and activations whose blocks differ by orders of magnitude (the three-term split is per block)."""
    for dt, N, K in ((ops.Q4_K, 128, 2048), (ops.Q6_K, 128, 2048)):
        raw = torch.from_numpy(synth.random_blocks(31, dt, N, K))
        deq = oracle.dequant(dt, raw.numpy().reshape(-1), N * K).reshape(N, K).astype(np.float64)
        g = torch.Generator().manual_seed(32)
        x = torch.randn(K, generator=g) * (10.0 ** torch.randint(-6, 7, (K // 256,), generator=g).float()).repeat_interleave(256)
        x[5] = 0.0
        x[256:512] = 0.0  # an all-zero block
        c = chain.DecodeChain(cuda)
        out = torch.empty(N, device=cuda)
        c.matmul([ops.QTensor(raw.reshape(-1).to(cuda), dt, (N, K))], x=x.to(cuda), outs=[out])
        c.build()
        c.run()
        torch.cuda.synchronize()
        want = deq @ x.numpy().astype(np.float64)
        scale = 1.0 + np.abs(deq) @ np.abs(x.numpy().astype(np.float64))
        assert np.max(np.abs(out.cpu().numpy() - want) / scale) <= 2e-4   # the reference's CPU <-> CUDA bound
        assert rel_l2(out.cpu().numpy(), want) <= 1e-5
        assert c.status() == 0


def test_shared_activations_and_gate(cuda, oracle):
    """Up to four matrices in one operator (LinearMulti, ops/gemv.go:21-78) and the gated pair (GatedLinear, :80-140)."""
    K = 2048
    ws = [_w(40 + i, ops.Q4_K, n, K, cuda, oracle) for i, n in enumerate((512, 128, 144, 48))]
    x = torch.randn(K, generator=torch.Generator().manual_seed(41)).to(cuda)
    outs = [torch.empty(w.shape[0], device=cuda) for w, _ in ws]
    wg, dg = _w(50, ops.Q4_K, 1000, K, cuda, oracle)
    wu, du = _w(51, ops.Q4_K, 1000, K, cuda, oracle)
    act_s, act_g = torch.empty(1000, device=cuda), torch.empty(1000, device=cuda)
    c = chain.DecodeChain(cuda)
    c.matmul([w for w, _ in ws], x=x, outs=outs)
    c.matmul([wg, wu], x=x, outs=[act_s], act=1)
    c.matmul([wg, wu], x=x, outs=[act_g], act=2)
    c.build()
    c.run()
    torch.cuda.synchronize()
    x64 = x.cpu().numpy().astype(np.float64)
    for o, (_, d) in zip(outs, ws):
        assert rel_l2(o.cpu().numpy(), d @ x64) <= 1e-5
    gl, ul = dg @ x64, du @ x64
    assert rel_l2(act_s.cpu().numpy(), gl / (1 + np.exp(-gl)) * ul) <= 1e-5
    from math import erf
    ge = 0.5 * gl * (1 + np.vectorize(erf)(gl / np.sqrt(2)))
    assert rel_l2(act_g.cpu().numpy(), ge * ul) <= 1e-5
    assert c.status() == 0


def _layers(cuda, oracle, H, KV, F, V, L):
    """L decoder layers' linears + final norm + lm_head as one program; returns (chain, tensors, f64 reference fn)."""
    nw = [(1 + 0.1 * torch.randn(H, generator=torch.Generator().manual_seed(70 + i))).to(cuda) for i in range(2 * L + 1)]
    W = []
    for l in range(L):
        W.append({"q": _w(100 + 10 * l, ops.Q4_K, H, H, cuda, oracle), "k": _w(101 + 10 * l, ops.Q4_K, KV, H, cuda, oracle),
                  "v": _w(102 + 10 * l, ops.Q4_K, KV, H, cuda, oracle), "o": _w(103 + 10 * l, ops.Q4_K, H, H, cuda, oracle),
                  "g": _w(104 + 10 * l, ops.Q4_K, F, H, cuda, oracle), "u": _w(105 + 10 * l, ops.Q4_K, F, H, cuda, oracle),
                  "d": _w(106 + 10 * l, ops.Q6_K, H, F, cuda, oracle)})
    head = _w(99, ops.Q6_K, V, H, cuda, oracle)
    h0 = torch.randn(H, generator=torch.Generator().manual_seed(60)).to(cuda)
    k_out = [torch.empty(KV, device=cuda) for _ in range(L)]
    v_out = [torch.empty(KV, device=cuda) for _ in range(L)]
    logits = torch.empty(V, device=cuda)
    c = chain.DecodeChain(cuda)
    # chain vectors, reused by every layer: q (stands in for the attention output), o, act, down and the two
    # alternating residual streams
    vq, vo, va, vd, vh = c.vec(), c.vec(), c.vec(), c.vec(), [c.vec(), c.vec()]
    cur = None  # the vector holding the residual stream (None: plain h0)
    for l in range(L):
        other = None if cur is None else (vh[0] if cur == vh[1] else vh[1])   # the new sum never overwrites the vector it is read from
        kw = dict(x=h0) if cur is None else dict(x_vec=cur, res_vec=vd, sum_vec=other)
        c.matmul([W[l]["q"][0], W[l]["k"][0], W[l]["v"][0]], outs=[None, k_out[l], v_out[l]], out_vecs=[vq, None, None],
                 norm_weight=nw[2 * l], eps=1e-5, **kw)
        stream1 = other
        c.matmul([W[l]["o"][0]], x_vec=vq, out_vecs=[vo])
        if stream1 is None:   # layer 0: the stream is still the plain h0
            c.matmul([W[l]["g"][0], W[l]["u"][0]], x=h0, res_vec=vo, sum_vec=vh[1], act=1, out_vecs=[va], norm_weight=nw[2 * l + 1], eps=1e-5)
            cur = vh[1]
        else:
            nxt = vh[0] if stream1 == vh[1] else vh[1]
            c.matmul([W[l]["g"][0], W[l]["u"][0]], x_vec=stream1, res_vec=vo, sum_vec=nxt, act=1, out_vecs=[va], norm_weight=nw[2 * l + 1], eps=1e-5)
            cur = nxt
        c.matmul([W[l]["d"][0]], x_vec=va, out_vecs=[vd])
    last = vh[0] if cur == vh[1] else vh[1]
    c.matmul([head[0]], x_vec=cur, res_vec=vd, sum_vec=last, outs=[logits], norm_weight=nw[2 * L], eps=1e-5)
    c.build()

    def reference():
        def norm(s, w):
            return s / np.sqrt(np.mean(s * s) + 1e-5) * w.cpu().numpy().astype(np.float64)

        h = h0.cpu().numpy().astype(np.float64)
        down, ks = None, []
        for l in range(L):
            s = h if down is None else h + down
            y = norm(s, nw[2 * l])
            q = W[l]["q"][1] @ y
            ks.append((W[l]["k"][1] @ y, W[l]["v"][1] @ y))
            o = W[l]["o"][1] @ q
            s2 = s + o
            y2 = norm(s2, nw[2 * l + 1])
            gl, ul = W[l]["g"][1] @ y2, W[l]["u"][1] @ y2
            down = W[l]["d"][1] @ (gl / (1 + np.exp(-gl)) * ul)
            h = s2
        return head[1] @ norm(h + down, nw[2 * L]), ks

    return c, (h0, k_out, v_out, logits), reference


@pytest.mark.parametrize("H,KV,F,V,L", [(2048, 256, 4096, 3000, 3), (4096, 1024, 14336, 5008, 2)])
def test_decoder_layers_as_one_launch(cuda, oracle, H, KV, F, V, L):
    c, (h0, k_out, v_out, logits), reference = _layers(cuda, oracle, H, KV, F, V, L)
    want, ks = reference()
    for rep in range(2):
        logits.zero_()
        c.run()
        torch.cuda.synchronize()
        assert rel_l2(logits.cpu().numpy(), want) <= 1e-4, rep     # errors of the layers' f32 arithmetic compound
        for l in range(L):
            assert rel_l2(k_out[l].cpu().numpy(), ks[l][0]) <= 1e-4 and rel_l2(v_out[l].cpu().numpy(), ks[l][1]) <= 1e-4
    assert c.status() == 0
    # replayed from a CUDA graph with new activations: the tags advance on the device, nothing is re-recorded
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        c.run()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    with torch.cuda.graph(g):
        c.run()
    h0.copy_(torch.randn(H, generator=torch.Generator().manual_seed(61)).to(cuda))
    want2, _ = reference()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    assert rel_l2(logits.cpu().numpy(), want2) <= 1e-4
    assert c.status() == 0


def test_build_rejects_bad_programs(cuda, oracle):
    w, _ = _w(1, ops.Q4_K, 64, 512, cuda, oracle)
    w6, _ = _w(2, ops.Q6_K, 64, 512, cuda, oracle)
    x = torch.zeros(512, device=cuda)
    from light_b200 import _lib

    c = chain.DecodeChain(cuda)
    c.matmul([w6], x=x, outs=[torch.empty(64, device=cuda)])       # Q6_K needs K % 2048 == 0
    with pytest.raises(_lib.Light200Error):
        c.build()
    c = chain.DecodeChain(cuda)
    v = c.vec()
    c.matmul([w], x_vec=v, outs=[torch.empty(64, device=cuda)])    # reads a vector nobody wrote
    with pytest.raises(_lib.Light200Error):
        c.build()
    c = chain.DecodeChain(cuda)
    v, v2 = c.vec(), c.vec()
    nwt = torch.ones(512, device=cuda)
    w5, _ = _w(3, ops.Q4_K, 512, 512, cuda, oracle)
    c.matmul([w5], x=x, out_vecs=[v])
    c.matmul([w5], x_vec=v, out_vecs=[v2])
    c.matmul([w5], x_vec=v2, res_vec=v, sum_vec=v2, norm_weight=nwt, eps=1e-5, outs=[torch.empty(512, device=cuda)])   # sum over its own input
    with pytest.raises(_lib.Light200Error):
        c.build()
    c = chain.DecodeChain(cuda)
    v = c.vec()
    c.matmul([w], x=x, out_vecs=[v])                               # 64 values ...
    c.matmul([w], x_vec=v, outs=[torch.empty(64, device=cuda)])    # ... read as 512
    with pytest.raises(_lib.Light200Error):
        c.build()
