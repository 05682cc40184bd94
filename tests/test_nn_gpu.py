"""The layer types that choose among the quantized matmuls (light_b200.nn, mirroring nn/linear.go:193-354, 476-516 and
nn/moe.go:121-245), the 4-bit sparse block (ops.MoEInt4, ops/int4.go:157-268), the activation-column gather in front
of an act-order weight (ops/int4.go:129-147) and the checkpoint-side helpers takeInt4 / concatInt4
(models/int4_load.go:169-244), each against the CPU oracle on the same seeded inputs."""
import numpy as np
import pytest
import torch

from light_b200 import nn, ops, safetensors, synth
from helpers import rel_l2

pytestmark = pytest.mark.gpu


def _int4(seed, N, K, G, dev):
    codes, s, z = synth.random_int4(seed, N, K, G)
    return (codes, s, z), ops.Int4(torch.from_numpy(codes.view(np.int32)).to(dev), torch.from_numpy(s).to(dev), torch.from_numpy(z).to(dev), G)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,K", [(1, 256), (7, 4096), (300, 1000)])
def test_gather_columns(cuda, dtype, M, K):
    g = torch.Generator().manual_seed(K + M)
    x = torch.randn(M, K, generator=g).to(dtype)
    idx = torch.randperm(K, generator=g)
    got = ops.GatherColumns(x.to(cuda), idx.to(cuda))
    assert torch.equal(got.cpu(), x[:, idx])
    with pytest.raises(ValueError, match="gather_columns"):
        ops.GatherColumns(x.to(cuda), idx[:-1].to(cuda))
    bad = idx.clone()
    bad[3], bad[5] = -1, K                     # an index outside the row reads as zero, nothing else moves
    got = ops.GatherColumns(x.to(cuda), bad.to(cuda)).cpu()
    want = x[:, idx].clone()
    want[:, 3] = 0
    want[:, 5] = 0
    assert torch.equal(got, want)


def test_linear_dispatch(cuda, oracle):
    """One Linear per weight kind; every result equals the op the reference's Forward would have chosen."""
    N, K, M = 96, 512, 5
    g = torch.Generator().manual_seed(11)
    x = torch.randn(M, 2, K, generator=g)                 # rank 3: flattened to (M * 2, K) and restored
    xd = x.to(cuda)
    # GGUF block-quantized
    for dt in (ops.Q4_K, ops.Q6_K, ops.Q8_0):
        raw = synth.random_blocks(12 + dt, dt, N, K)
        lin = nn.Linear(K, N)
        lin.set_weight(ops.QTensor(torch.from_numpy(raw.reshape(-1)).to(cuda), dt, (N, K)))
        y = lin.forward(xd)
        assert y.shape == (M, 2, N) and y.dtype == torch.float32
        want = oracle.matmul_q(dt, x.reshape(-1, K).numpy(), raw.reshape(-1), N)
        assert rel_l2(y.reshape(-1, N).cpu().numpy(), want) <= 2e-3
        with pytest.raises(ValueError, match="needs F32 activations"):
            lin.forward(xd.to(torch.bfloat16))
    # 4-bit, with a bias: BF16 activations are widened, the bias is added in F32, one rounding at the end
    (codes, s, z), w4 = _int4(21, N, K, 128, cuda)
    b = torch.randn(N, generator=g)
    lin = nn.Linear(K, N, B=b.to(cuda))
    lin.set_int4(w4)
    xb = x.to(torch.bfloat16)
    y = lin.forward(xb.to(cuda))
    assert y.dtype == torch.bfloat16 and y.shape == (M, 2, N)
    deq = oracle.int4_dequant(codes, s, z, 128).astype(np.float64)
    want = xb.float().reshape(-1, K).numpy().astype(np.float64) @ deq.T + b.numpy()
    assert rel_l2(y.float().reshape(-1, N).cpu().numpy(), want) <= 6e-3
    y32 = nn.Linear(K, N, W4=w4).forward(xd)
    assert y32.dtype == torch.float32 and rel_l2(y32.reshape(-1, N).cpu().numpy(), x.reshape(-1, K).numpy().astype(np.float64) @ deq.T) <= 1e-3
    # block-scaled FP8
    w8, s8 = synth.random_fp8_block(22, 128, K, 128, 128)
    lin = nn.Linear(K, 128, W=w8.to(cuda).view(torch.float8_e4m3fn), WBlockScale=s8.to(cuda), WBlock=(128, 128))
    y = lin.forward(xd)
    want = x.reshape(-1, K).numpy().astype(np.float64) @ oracle.fp8_block_dequant(w8.numpy(), s8.numpy(), 128, 128).astype(np.float64).T
    assert rel_l2(y.reshape(-1, 128).cpu().numpy(), want) <= 1e-3
    with pytest.raises(ValueError, match="F32 or BF16 activations, got F16"):
        lin.forward(xd.half())
    # dense F32 and BF16 + bias (one rounding)
    w = torch.randn(N, K, generator=g) * 0.05
    y = nn.Linear(K, N, W=w.to(cuda), B=b.to(cuda)).forward(xd)
    assert rel_l2(y.cpu().numpy().reshape(-1, N), (x.reshape(-1, K).double() @ w.double().t() + b.double()).numpy()) <= 1e-4
    wb = w.to(torch.bfloat16)
    y = nn.Linear(K, N, W=wb.to(cuda), B=(b * 40).to(torch.bfloat16).to(cuda)).forward(xb.to(cuda))
    exact = xb.reshape(-1, K).double() @ wb.double().t() + (b * 40).to(torch.bfloat16).double()
    assert y.dtype == torch.bfloat16
    # a single rounding: at most half a BF16 step (2^-9 relative) away from the exact sum, plus the F32 product's error
    assert float(((y.reshape(-1, N).cpu().double() - exact).abs() / exact.abs().clamp_min(1e-3)).max()) <= 2 ** -8 + 1e-4
    with pytest.raises(ValueError, match="cast at the boundary"):
        nn.Linear(K, N, W=wb.to(cuda)).forward(xd.half())
    with pytest.raises(ValueError, match="weight not loaded"):
        nn.Linear(K, N).forward(xd)
    with pytest.raises(ValueError, match="in_features"):
        nn.Linear(K, N, W=w.to(cuda)).forward(xd[..., :-1])


def _moe_oracle(x, gu_deq, dn_deq, ids, wts, gelu=False):
    """Token by token in float64: sum over slots of weight * down(act(gate) * up)."""
    T, H = x.shape
    I = dn_deq.shape[2]
    out = np.zeros((T, H))
    for t in range(T):
        for slot in range(ids.shape[1]):
            e = int(ids[t, slot])
            h = gu_deq[e].astype(np.float64) @ x[t].astype(np.float64)
            gte = h[:I]
            if gelu:
                from math import erf
                a = np.array([0.5 * v * (1 + erf(v / np.sqrt(2))) for v in gte])
            else:
                a = gte / (1 + np.exp(-gte))
            out[t] += float(wts[t, slot]) * (dn_deq[e].astype(np.float64) @ (a * h[I:]))
    return out


@pytest.mark.parametrize("kind", ["dense", "q4_k", "int4", "fp8"])
def test_sparse_moe_block(cuda, oracle, kind):
    E, H, I, T, topk = 8, 512, 256, 37, 2
    g = torch.Generator().manual_seed(100)
    x = torch.randn(T, H, generator=g) * 0.5
    router = torch.randn(E, H, generator=g) * 0.1
    gate = nn.Linear(H, E, W=router.to(cuda))
    m = nn.SparseMoE(gate, TopK=topk, NormTopK=True)
    if kind == "dense":
        gu, dn = torch.randn(E, 2 * I, H, generator=g) * 0.05, torch.randn(E, H, I, generator=g) * 0.05
        m.GateUp, m.Down = gu.to(cuda), dn.to(cuda)
        gu_d, dn_d = gu.numpy(), dn.numpy()
        tol = 1e-3                                 # TF32-free F32 grouped GEMM against float64
    elif kind == "q4_k":
        gr, dr = synth.random_blocks(101, ops.Q4_K, E * 2 * I, H), synth.random_blocks(102, ops.Q4_K, E * H, I)
        m.GateUp = ops.QTensor(torch.from_numpy(gr.reshape(-1)).to(cuda), ops.Q4_K, (E, 2 * I, H))
        m.Down = ops.QTensor(torch.from_numpy(dr.reshape(-1)).to(cuda), ops.Q4_K, (E, H, I))
        gu_d = oracle.dequant(ops.Q4_K, gr.reshape(-1), E * 2 * I * H).reshape(E, 2 * I, H)
        dn_d = oracle.dequant(ops.Q4_K, dr.reshape(-1), E * H * I).reshape(E, H, I)
        tol = 4e-3
    elif kind == "int4":
        gq, dq, gu_l, dn_l = [], [], [], []
        for e in range(E):
            (cg, sg, zg), wg = _int4(200 + e, I, H, 128, cuda)
            (cu, su, zu), wu = _int4(300 + e, I, H, 128, cuda)
            (cd, sd, zd), wd = _int4(400 + e, H, I, 128, cuda)
            gq.append(ops.ConcatInt4(wg, wu))
            dq.append(wd)
            gu_l.append(np.concatenate([oracle.int4_dequant(cg, sg, zg, 128), oracle.int4_dequant(cu, su, zu, 128)], 0))
            dn_l.append(oracle.int4_dequant(cd, sd, zd, 128))
        m.GateUpQ4, m.DownQ4 = gq, dq
        gu_d, dn_d = np.stack(gu_l), np.stack(dn_l)
        tol = 1e-3
    else:
        w1, s1 = synth.random_fp8_block(103, E * 2 * I, H, 128, 128)
        w2, s2 = synth.random_fp8_block(104, E * H, I, 128, 128)
        m.GateUp, m.GateUpScale = w1.reshape(E, 2 * I, H).to(cuda).view(torch.float8_e4m3fn), s1.reshape(E, 2 * I // 128, H // 128).to(cuda)
        m.Down, m.DownScale = w2.reshape(E, H, I).to(cuda).view(torch.float8_e4m3fn), s2.reshape(E, H // 128, I // 128).to(cuda)
        m.Block = (128, 128)
        gu_d = oracle.fp8_block_dequant(w1.numpy(), s1.numpy(), 128, 128).reshape(E, 2 * I, H)
        dn_d = oracle.fp8_block_dequant(w2.numpy(), s2.numpy(), 128, 128).reshape(E, H, I)
        x = x * 0.02                                # the FP8 synthetic weights are O(0.1): keep SiLU in its curved range
        tol = 1e-3
    y = m.forward(x.to(cuda).reshape(T, 1, H))
    assert y.shape == (T, 1, H) and y.dtype == torch.float32
    assert ops.moe_route_status(0) == 0
    route = m.route(x.to(cuda))
    ids, wts = route.topk_ids.cpu().numpy(), route.weights.reshape(T, topk).cpu().numpy()
    # the routing itself against the oracle, from the same probabilities
    probs = torch.softmax((x.to(cuda) @ router.to(cuda).t()).float(), -1).cpu().numpy()
    oids, owts = oracle.moe_route_topk(probs, topk, True)[:2]
    assert np.array_equal(ids, np.asarray(oids).reshape(T, topk)) and np.array_equal(wts, np.asarray(owts, np.float32).reshape(T, topk))
    want = _moe_oracle(x.numpy(), gu_d, dn_d, ids, wts)
    assert rel_l2(y.reshape(T, H).cpu().numpy(), want) <= tol, kind


def test_moe_int4_expands_only_routed_experts(cuda, oracle):
    """A routing that uses 2 of 6 experts, GELU gate, BF16 activations: MoEInt4 equals the per-token oracle, and
    unused experts may even be absent (None) since they are never touched."""
    E, H, I, T, topk = 6, 256, 128, 9, 2
    g = torch.Generator().manual_seed(7)
    x = (torch.randn(T, H, generator=g) * 0.5).to(torch.bfloat16)
    ids = torch.tensor([[4, 1]] * T)
    wts = torch.rand(T, topk, generator=g)
    gq, dq, gu_d, dn_d = [None] * E, [None] * E, np.zeros((E, 2 * I, H), np.float32), np.zeros((E, H, I), np.float32)
    for e in (1, 4):
        (cg, sg, zg), wg = _int4(50 + e, 2 * I, H, 64, cuda)
        (cd, sd, zd), wd = _int4(60 + e, H, I, 64, cuda)
        gq[e], dq[e] = wg, wd
        gu_d[e], dn_d[e] = oracle.int4_dequant(cg, sg, zg, 64), oracle.int4_dequant(cd, sd, zd, 64)
    gq[0], dq[0] = gq[1], dq[1]                    # shapes are read from expert 0
    r = ops.MoERouteFromIDs(ids.to(cuda), wts.to(cuda), T, topk)
    y = ops.MoEInt4(x.to(cuda), gq, dq, r, topk, gelu=True)
    assert y.dtype == torch.bfloat16 and y.shape == (T, H)
    want = _moe_oracle(x.float().numpy(), gu_d, dn_d, ids.numpy(), wts.numpy(), gelu=True)
    assert rel_l2(y.float().cpu().numpy(), want) <= 2e-2     # BF16 roundings of h, the activation, the pair rows and the sums
    with pytest.raises(ValueError, match="expert out of range"):
        ops.MoEInt4(x.to(cuda), gq, dq, ops.MoERouteFromIDs(torch.full((T, topk), E).to(cuda), wts.to(cuda), T, topk), topk)


@pytest.mark.parametrize("method,v2", [("gptq", False), ("gptq", True), ("awq", False)])
def test_take_int4_from_checkpoint_tensors(cuda, oracle, method, v2):
    """safetensors bytes -> takeInt4 -> MatMulInt4, the ordered grouping."""
    import io
    N, K, G = 64, 512, 128
    codes, s, z = synth.random_int4(70, N, K, G)
    if method == "gptq" and not v2:
        z[z == 0] = 1.0            # the v1 format stores zero - 1 in four bits
    qw, qz, sc = synth.to_awq(codes, s, z) if method == "awq" else synth.to_gptq(codes, s, z, v2)
    ck = {"m.qweight": torch.from_numpy(np.ascontiguousarray(qw)), "m.qzeros": torch.from_numpy(np.ascontiguousarray(qz)),
          "m.scales": torch.from_numpy(np.ascontiguousarray(sc)).to(torch.float16), "other": torch.ones(3)}
    if method == "gptq":
        ck["m.g_idx"] = (torch.arange(K) // G).to(torch.int32)
    buf = io.BytesIO()
    safetensors.write(buf, ck)
    hf, _ = safetensors.load(io.BytesIO(buf.getvalue()))
    w = safetensors.take_int4(hf, "m", method, G, cuda, v2=v2)
    assert set(hf) == {"other"} and w.perm is None
    assert np.array_equal(w.codes.cpu().numpy().view(np.uint32), codes) and np.array_equal(w.zeros.cpu().numpy(), z)
    assert np.array_equal(w.scales.cpu().numpy(), s)          # scales were f16-representable to begin with
    with pytest.raises(safetensors.SafetensorsError, match="missing tensor"):
        safetensors.take_int4(hf, "m", method, G, cuda)


def test_take_int4_act_order(cuda, oracle):
    """A GPTQ checkpoint whose g_idx assigns input rows to groups out of order (quant/int4.go:122-151): the weight is
    stored sorted by group with the order kept as `perm`; x @ W^T is unchanged."""
    N, K, G = 32, 512, 128
    rng = np.random.default_rng(3)
    q = rng.integers(0, 16, (K, N), dtype=np.uint32)                 # nibble of input row k, output n
    g_idx = rng.permutation(np.arange(K) // G).astype(np.int32)       # every group still has G members
    sc = (rng.uniform(0.005, 0.02, (K // G, N)).astype(np.float16)).astype(np.float32)
    zr = rng.integers(1, 16, (K // G, N)).astype(np.uint32)     # v1 stores zero - 1 in four bits
    qweight = np.zeros((K // 8, N), np.uint32)
    for j in range(8):
        qweight |= q[j::8] << np.uint32(4 * j)
    qzeros = np.zeros((K // G, N // 8), np.uint32)
    for j in range(8):
        qzeros |= ((zr[:, j::8] - 1) & 0xF) << np.uint32(4 * j)      # "gptq" stores zero - 1
    hf = {"m.qweight": torch.from_numpy(qweight.view(np.int32)), "m.qzeros": torch.from_numpy(qzeros.view(np.int32)),
          "m.scales": torch.from_numpy(sc).to(torch.float16), "m.g_idx": torch.from_numpy(g_idx)}
    w = safetensors.take_int4(hf, "m", "gptq", G, cuda)
    assert w.perm is not None and hf == {}
    perm = w.perm.cpu().numpy()
    assert np.array_equal(g_idx[perm], np.arange(K) // G)
    assert all(perm[i] < perm[i + 1] for i in range(K - 1) if g_idx[perm[i]] == g_idx[perm[i + 1]])      # stable
    # the dense weight the checkpoint means: W[n, k] = s[g(k), n] * (q[k, n] - z[g(k), n])
    W = (sc[g_idx] * (q.astype(np.float32) - zr[g_idx].astype(np.float32))).T.astype(np.float64)
    x = torch.randn(5, K, generator=torch.Generator().manual_seed(4))
    y = ops.MatMulInt4(x.to(cuda), w)
    assert rel_l2(y.cpu().numpy(), x.numpy().astype(np.float64) @ W.T) <= 1e-3
    y1 = ops.MatMulInt4(x[:1].to(cuda), w)                           # the one-row path gathers too
    assert rel_l2(y1.cpu().numpy(), x[:1].numpy().astype(np.float64) @ W.T) <= 1e-3
    hf2 = {"m.qweight": torch.from_numpy(qweight.view(np.int32)), "m.qzeros": torch.from_numpy(qzeros.view(np.int32)),
           "m.scales": torch.from_numpy(sc).to(torch.float16), "m.g_idx": torch.from_numpy(np.where(np.arange(K) < 3, 1, g_idx).astype(np.int32))}
    with pytest.raises(safetensors.SafetensorsError, match="not all of size"):
        safetensors.take_int4(hf2, "m", "gptq", G, cuda)
