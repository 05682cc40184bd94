"""Parity at the full shapes of the benchmark configurations.  The CPU oracle cannot multiply these sizes in
seconds, so each case checks a seeded SAMPLE of output columns (weight rows) -- every activation row against the
f64 dot of the bit-exact dequantized weight rows, the arbiter the reference's own tests use
(ops/matmul_q_cpu_test.go:66-78, ops/int4_test.go:97-106) -- which exercises the kernel branches that only these
shapes select (tile height, wave quantisation, K split), plus whole-output sanity (finite, status word)."""
import numpy as np
import pytest
import torch

from helpers import max_rel, rel_l2
from light_b200 import ops, synth

pytestmark = pytest.mark.gpu


def _sample_rows(seed, N, n=96):
    rng = np.random.Generator(np.random.Philox(seed))
    rows = np.unique(np.concatenate([[0, 1, N - 1, N // 2], rng.integers(0, N, n)]))
    return rows


# configs[2]: prefill matmuls of the Llama-3-8B layer at M = 2048, bf16-valued activations
@pytest.mark.parametrize("name,dt,N,K", [("qkv", ops.Q4_K, 6144, 4096), ("o", ops.Q4_K, 4096, 4096),
                                         ("gate_up", ops.Q4_K, 28672, 4096), ("down", ops.Q6_K, 4096, 14336)])
def test_prefill_llama8b_shapes(cuda, oracle, name, dt, N, K):
    M = 2048
    raw = synth.gaussian_weight(300 + N % 97, dt, N, K, device=cuda)           # (N, row_bytes) uint8 on the device
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(301)).to(torch.bfloat16).float()
    got = ops.MatMulQ(x.to(cuda), ops.QTensor(raw.reshape(-1), dt, (N, K)))
    torch.cuda.synchronize()
    assert ops.prefill_status(0) == 0 and bool(torch.isfinite(got).all())
    rows = _sample_rows(302, N)
    sub = raw[torch.from_numpy(rows).to(cuda)].cpu().numpy()
    deq = oracle.dequant(dt, sub.reshape(-1), len(rows) * K).reshape(len(rows), K).astype(np.float64)
    want = x.numpy().astype(np.float64) @ deq.T
    assert rel_l2(got[:, torch.from_numpy(rows).to(cuda)].cpu().numpy(), want) <= 1e-3, name


# configs[1]: batched decode at M = 8, 32, 64 on the layer shapes (the kernels are chosen by M and shape)
@pytest.mark.parametrize("M", [8, 32, 64])
@pytest.mark.parametrize("dt,N,K", [(ops.Q4_K, 14336, 4096), (ops.Q6_K, 4096, 14336)])
def test_batched_decode_llama8b_shapes(cuda, oracle, M, dt, N, K):
    raw = synth.gaussian_weight(310, dt, N, K, device=cuda)
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(311 + M))
    got = ops.MatMulQ(x.to(cuda), ops.QTensor(raw.reshape(-1), dt, (N, K)))
    torch.cuda.synchronize()
    rows = _sample_rows(312, N)
    sub = raw[torch.from_numpy(rows).to(cuda)].cpu().numpy()
    deq = oracle.dequant(dt, sub.reshape(-1), len(rows) * K).reshape(len(rows), K).astype(np.float64)
    want = x.numpy().astype(np.float64) @ deq.T
    assert rel_l2(got[:, torch.from_numpy(rows).to(cuda)].cpu().numpy(), want) <= 1e-3, (M, dt)
    assert ops.prefill_status(0) == 0 and bool(torch.isfinite(got).all())


# configs[3]: GPTQ / AWQ-style W4A16 at Qwen2.5-7B shapes, group 128, bf16 activations (ops.MatMulInt4 takes F32 / BF16)
@pytest.mark.parametrize("M,N,K", [(1, 4608, 3584), (16, 4608, 3584), (256, 4608, 3584), (4096, 18944, 3584), (256, 3584, 18944)])
def test_int4_qwen7b_shapes(cuda, oracle, M, N, K):
    G = 128
    codes, s, z = synth.random_int4(320 + M, N, K, G)
    w = ops.Int4(torch.from_numpy(codes.view(np.int32)).to(cuda), torch.from_numpy(s).to(cuda), torch.from_numpy(z).to(cuda), G)
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(321)).to(torch.bfloat16)
    got = ops.MatMulInt4(x.to(cuda), w)
    torch.cuda.synchronize()
    assert got.dtype == torch.bfloat16 and bool(torch.isfinite(got.float()).all()) and ops.prefill_status(0) == 0
    rows = _sample_rows(322, N)
    # the reference rounds the dequantized weight once to bf16 (kernels/cuda/src/int4.cu:29) and multiplies in bf16 x bf16 -> f32
    deq = oracle.int4_dequant(np.ascontiguousarray(codes[rows]), np.ascontiguousarray(s[rows]), np.ascontiguousarray(z[rows]), G, bf16=True)
    if deq.dtype == np.uint16:  # bf16 bit patterns
        deq = (deq.astype(np.uint32) << 16).view(np.float32)
    deq = deq.astype(np.float64)
    want = x.float().numpy().astype(np.float64) @ deq.T
    assert max_rel(got[:, torch.from_numpy(rows).to(cuda)].float().cpu().numpy(), want) <= 3e-2    # ops/int4_test.go's bf16 bound
    assert rel_l2(got[:, torch.from_numpy(rows).to(cuda)].float().cpu().numpy(), want) <= 4e-3      # one bf16 rounding of the output


# configs[4]: one DeepSeek-V3-shaped MoE layer, 256 block-scaled FP8 experts, 4096 tokens routed top-8 by the biased
# sigmoid router.  Sampled tokens are checked end to end against the per-expert loop the reference runs
# (models/moe_routed.go:34-79) in f64.
def test_moe_deepseek_v3_layer(cuda, oracle):
    E, H, I, T, topk, b = 256, 7168, 2048, 4096, 8, 128
    free, _ = torch.cuda.mem_get_info()
    if free < 20 * (1 << 30):
        pytest.skip("needs about 20 GB of free device memory")
    w1, s1 = synth.random_fp8_block(401, E * 2 * I, H, b, b, device=cuda)      # gate_up: (E, 2I, H)
    w2, s2 = synth.random_fp8_block(402, E * H, I, b, b, device=cuda)          # down:    (E, H, I)
    w1, s1 = w1.reshape(E, 2 * I, H), s1.reshape(E, 2 * I // b, H // b)
    w2, s2 = w2.reshape(E, H, I), s2.reshape(E, H // b, I // b)
    g = torch.Generator(device=cuda)
    g.manual_seed(403)
    x = torch.randn(T, H, generator=g, device=cuda).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g, device=cuda)
    bias = torch.randn(E, generator=g, device=cuda) * 0.5
    r = ops.MoERouteSigmoid(logits, bias, topk, True)
    assert ops.moe_route_status(0) == 0
    counts = torch.bincount(r.sorted_expts, minlength=E)
    assert int(counts.sum()) == T * topk and int(counts.max()) > 2 * T * topk // E      # the bias skews the load
    h = ops.MoEGemmF8Block(x, w1, s1, b, b, r, None, topk)                              # (T * topk, 2I), one row per pair
    act = ops.SwiGLU(h) if hasattr(ops, "SwiGLU") else (torch.nn.functional.silu(h[:, :I].float()) * h[:, I:].float()).to(torch.bfloat16)
    y = ops.MoEGemmF8Block(act, w2, s2, b, b, r, r.weights, topk)                       # (T * topk, H), routing weight applied
    out = ops.MoECombine(y, topk)
    torch.cuda.synchronize()
    assert ops.prefill_status(0) == 0 and bool(torch.isfinite(out.float()).all())
    ids, wts = r.topk_ids.cpu().numpy(), r.weights.reshape(T, topk).cpu().numpy()
    bf = lambda a: torch.from_numpy(np.asarray(a, np.float32)).to(torch.bfloat16).float().numpy().astype(np.float64)  # noqa: E731
    for tok in (0, 1777, T - 1):
        xt = x[tok].float().cpu().numpy().astype(np.float64)
        want = np.zeros(H)
        for slot in range(topk):
            e = int(ids[tok, slot])
            d1 = bf(oracle.fp8_block_dequant(w1[e].cpu().numpy(), s1[e].cpu().numpy(), b, b))
            d2 = bf(oracle.fp8_block_dequant(w2[e].cpu().numpy(), s2[e].cpu().numpy(), b, b))
            hh = bf(d1 @ xt)
            a = bf(hh[:I] / (1 + np.exp(-hh[:I])) * hh[I:])
            want += bf(float(wts[tok, slot]) * (d2 @ a))
        got = out[tok].float().cpu().numpy()
        assert rel_l2(got, want) <= 2e-2, tok        # bf16 roundings of h, act and y on both sides; sums of 8 bf16 rows
