"""Pins the oracle's decoders with the reference's own known-answer tests, re-expressed as data:
quant/q4_k_test.go:48-127, quant/q6_k_test.go:61-147, quant/others_test.go:30-51,
quant/quantize_test.go:13-45, ops/fp8_block_test.go:16-71, and an element-by-element restatement
of every layout formula (independent of the C code path)."""
import numpy as np
import pytest
import torch

from helpers import build_q4_k_block, build_q6_k_block, build_q8_0_block, rel_l2
from light_b200 import synth


def test_q4_k_kat(oracle):
    # TestDequantQ4_K: sub-block j has scale j+1, min j, all quants (j+1)&15; d = dmin = 1
    sc = [j + 1 for j in range(8)]
    mn = [j for j in range(8)]
    q = [((j + 1) & 0xF) for j in range(8) for _ in range(32)]
    out = oracle.dequant(oracle.Q4_K, build_q4_k_block(1.0, 1.0, sc, mn, q), 256)
    for j in range(8):
        assert np.all(out[j * 32:(j + 1) * 32] == sc[j] * (sc[j] & 0xF) - mn[j])


def test_q4_k_multiblock_kat(oracle):
    # TestDequantQ4_KMultiBlock
    sc = [2 * j for j in range(8)]
    mn = [j for j in range(8)]
    q = [i % 16 for i in range(256)]
    raw = np.concatenate([build_q4_k_block(0.5, 0.25, sc, mn, q), build_q4_k_block(2.0, 1.0, sc, mn, q)])
    out = oracle.dequant(oracle.Q4_K, raw, 512)
    assert out[7 * 32] == -1.75
    assert out[256 + 7 * 32] == -7.0
    # every element, closed form
    for b, (d, dmin) in enumerate([(0.5, 0.25), (2.0, 1.0)]):
        for i in range(256):
            j = i // 32
            assert out[b * 256 + i] == np.float32(d * sc[j]) * np.float32(q[i]) - np.float32(dmin * mn[j])


def test_q6_k_kats(oracle):
    # TestDequantQ6_K: raw 32 -> q = 0
    out = oracle.dequant(oracle.Q6_K, build_q6_k_block(0.5, [i + 1 for i in range(16)], [32] * 256), 256)
    assert np.all(out == 0)
    # TestDequantQ6_KKnownValues: scale 1, d 1, sub-block s encodes q = s
    raw = [s + 32 for s in range(16) for _ in range(16)]
    out = oracle.dequant(oracle.Q6_K, build_q6_k_block(1.0, [1] * 16, raw), 256)
    for s in range(16):
        assert np.all(out[s * 16:(s + 1) * 16] == s)
    # TestDequantQ6_KNegativeScale: 0.25 * -3 * 8 = -6
    out = oracle.dequant(oracle.Q6_K, build_q6_k_block(0.25, [-3] * 16, [40] * 256), 256)
    assert np.all(out == -6.0)


def test_q8_0_kat(oracle):
    # TestDequantQ8_0
    vals = [i - 16 for i in range(32)]
    out = oracle.dequant(oracle.Q8_0, build_q8_0_block(0.25, vals), 32)
    assert np.array_equal(out, 0.25 * np.array(vals, np.float32))


def test_wrong_sizes_rejected(oracle):
    with pytest.raises(ValueError):
        oracle.dequant(oracle.Q4_K, np.zeros(144, np.uint8), 100)
    with pytest.raises(ValueError):
        oracle.dequant(99, np.zeros(144, np.uint8), 256)


def _ref_decode(dt, raw, oracle):
    """Element-at-a-time restatement of the layout comments (quant/q4_k.go:14-24, q6_k.go:11-32,
    q8_0.go:11-17, kernels/cuda/src/matmul_q.cu:58-115,200-228), in numpy float32 arithmetic."""
    f32 = np.float32
    be, bb = oracle.block_elems(dt), oracle.block_bytes(dt)
    nb = raw.size // bb
    out = np.zeros(nb * be, np.float32)
    h = lambda b, o: f32(np.frombuffer(b[o:o + 2].tobytes(), np.float16)[0])
    for bi in range(nb):
        b = raw[bi * bb:(bi + 1) * bb]
        for i in range(be):
            if dt == oracle.Q8_0:
                v = h(b, 0) * f32(np.int8(b[2 + i]))
            elif dt == oracle.Q4_0:
                q = (b[2 + i % 16] >> (4 * (i // 16))) & 15
                v = h(b, 0) * f32(int(q) - 8)
            elif dt == oracle.Q5_0:
                qh = int.from_bytes(b[2:6].tobytes(), "little")
                q = ((b[6 + i % 16] >> (4 * (i // 16))) & 15) | (((qh >> i) & 1) << 4)
                v = h(b, 0) * f32(int(q) - 16)
            elif dt in (oracle.Q4_K, oracle.Q5_K):
                s = b[4:16]
                j = i // 32
                if j < 4:
                    sc, m = s[j] & 63, s[j + 4] & 63
                else:
                    sc, m = (s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4), (s[j + 4] >> 4) | ((s[j] >> 6) << 4)
                p, l, hi = i // 64, i % 32, (i % 64) // 32
                qs = b[16:] if dt == oracle.Q4_K else b[48:]
                q = (qs[p * 32 + l] >> (4 * hi)) & 15
                if dt == oracle.Q5_K:
                    q |= ((b[16 + l] >> j) & 1) << 4
                v = f32(h(b, 0) * f32(sc)) * f32(q) - f32(h(b, 2) * f32(m))
            else:  # Q6_K
                half, r = i // 128, i % 128
                g, l = r // 32, r % 32
                lo = (b[half * 64 + (g & 1) * 32 + l] >> (4 * (g >> 1))) & 15
                hi2 = (b[128 + half * 32 + l] >> (2 * g)) & 3
                sc = np.int8(b[192 + i // 16])
                v = f32(h(b, 208) * f32(sc)) * f32(int(lo | (hi2 << 4)) - 32)
            out[bi * be + i] = v
    return out


@pytest.mark.parametrize("name", ["q4_0", "q5_0", "q8_0", "q4_k", "q5_k", "q6_k"])
def test_decoders_match_layout_restatement(oracle, name):
    dt = oracle.GGUF_TYPES[name]
    K = 512
    raw = synth.random_blocks(11, dt, 3, K).reshape(-1)
    got = oracle.dequant(dt, raw, 3 * K)
    want = _ref_decode(dt, raw, oracle)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_q8_0_encoder_roundtrip(oracle):
    """quant/quantize_test.go:13-45: Q8_0 round trip rel-L2 <= 0.01; encoder matches the torch one
    used to make synthetic weights."""
    g = torch.Generator().manual_seed(1)
    w = torch.randn(8, 256, generator=g)
    enc = oracle.quantize_q8_0(w.numpy())
    back = oracle.dequant(oracle.Q8_0, enc, w.numel())
    assert rel_l2(back, w.numpy().ravel()) <= 0.01
    assert np.array_equal(enc, synth.quantize_q8_0(w).numpy().ravel())


@pytest.mark.parametrize("name,tol", [("q4_k", 0.12), ("q6_k", 0.03), ("q8_0", 0.01)])
def test_synthetic_quantizers_are_layout_valid(oracle, name, tol):
    """The builder-designed encoders decode (through the pinned oracle) back to the weight."""
    dt = oracle.GGUF_TYPES[name]
    g = torch.Generator().manual_seed(2)
    w = torch.randn(16, 1024, generator=g) * 0.02
    enc = synth.QUANTIZERS[dt](w).numpy()
    assert enc.shape == (16, synth.row_bytes(dt, 1024))
    back = oracle.dequant(dt, enc.reshape(-1), w.numel())
    assert rel_l2(back, w.numpy().ravel()) <= tol


def test_matmul_q_cpu_vs_f64(oracle):
    """ops/matmul_q_cpu_test.go:19-81: CPU matmul_q vs f64 dot of the dequantized weight,
    tol 1e-5 * (1 + sum|p|), M in {1, 9}, N = 37, K = 512; 1 and 3 threads agree."""
    N, K = 37, 512
    rng = np.random.Generator(np.random.Philox(9))
    for name, dt in oracle.GGUF_TYPES.items():
        w = synth.random_blocks(12, dt, N, K)
        deq = oracle.dequant(dt, w.reshape(-1), N * K).reshape(N, K).astype(np.float64)
        for M in (1, 9):
            x = rng.standard_normal((M, K)).astype(np.float32)
            got = oracle.matmul_q(dt, x, w, N, threads=1)
            want = x.astype(np.float64) @ deq.T
            bound = 1e-5 * (1 + np.abs(x.astype(np.float64))[:, None, :] * np.abs(deq)[None, :, :]).sum(-1)
            assert np.all(np.abs(got - want) <= bound), name
            assert np.array_equal(got, oracle.matmul_q(dt, x, w, N, threads=3))


def test_fp8_block_dequant_kat(oracle):
    """ops/fp8_block_test.go:16-71: 12 x 32 weight, 4 x 8 blocks, exact in f32 and bf16."""
    R, C_, br, bc = 12, 32, 4, 8
    g = torch.Generator().manual_seed(1)
    codes = (torch.randn(R, C_, generator=g) * 50).clamp(-448, 448).to(torch.float8_e4m3fn)
    scales = (torch.rand(R // br, C_ // bc, generator=g) * 0.01 + 1e-4).float()
    want = codes.float() * scales.repeat_interleave(br, 0).repeat_interleave(bc, 1)
    got = oracle.fp8_block_dequant(codes.view(torch.uint8).numpy(), scales.numpy(), br, bc)
    assert np.array_equal(got, want.numpy())
    got16 = oracle.fp8_block_dequant(codes.view(torch.uint8).numpy(), scales.numpy(), br, bc, bf16=True)
    assert np.array_equal(got16, want.to(torch.bfloat16).view(torch.int16).numpy().astype(np.uint16))
    with pytest.raises(ValueError):
        oracle.fp8_block_dequant(codes.view(torch.uint8).numpy(), scales.numpy(), 5, bc)


def test_int4_dequant_and_converters(oracle):
    """quant/int4.go:239-261 (Dequant) and the GPTQ v1/v2 and AWQ converters (quant/int4.go:103-235):
    packing a canonical weight into each checkpoint layout and converting back is the identity."""
    N, K, G = 16, 256, 128
    codes, s, z = synth.random_int4(4, N, K, G)
    deq = oracle.int4_dequant(codes, s, z, G)
    nib = synth._nibbles(codes).astype(np.float32)
    want = np.repeat(s, G, axis=1) * (nib - np.repeat(z, G, axis=1))
    assert np.array_equal(deq, want.astype(np.float32))
    deq16 = oracle.int4_dequant(codes, s, z, G, bf16=True)
    assert np.array_equal(deq16, torch.from_numpy(want).to(torch.bfloat16).view(torch.int16).numpy().astype(np.uint16))
    z1 = np.clip(z, 1, 15)  # GPTQ v1 stores zero - 1 in 4 bits
    for v2, zz in ((False, z1), (True, z)):
        c2, s2, z2 = oracle.int4_from_gptq(*synth.to_gptq(codes, s, zz, v2=v2), group=G, v2=v2)
        assert np.array_equal(c2, codes) and np.array_equal(s2, s) and np.array_equal(z2, zz)
    c3, s3, z3 = oracle.int4_from_awq(*synth.to_awq(codes, s, z), group=G)
    assert np.array_equal(c3, codes) and np.array_equal(s3, s) and np.array_equal(z3, z)


def test_int4_matmul_vs_f64(oracle):
    """ops/int4_test.go:80-145: matmul vs f64 reference, tol 1e-4 relative, M in {1, 3, 8, 9}."""
    N, K, G = 24, 256, 128
    codes, s, z = synth.random_int4(5, N, K, G)
    deq = oracle.int4_dequant(codes, s, z, G).astype(np.float64)
    rng = np.random.Generator(np.random.Philox(6))
    for M in (1, 3, 8, 9):
        x = rng.standard_normal((M, K)).astype(np.float32)
        got = oracle.int4_matmul(x, codes, s, z, G)
        want = x.astype(np.float64) @ deq.T
        assert np.max(np.abs(got - want) / (1 + np.abs(want))) <= 1e-4


def test_moe_gemm_matches_per_expert_loop(oracle):
    """ops/moe_test.go:52-120: grouped GEMM equals a per-expert loop; fixed ids of
    ops/int4_test.go TestMoEInt4MatchesDense {0,2,2,1,3,0,2,3,1,2}."""
    ids = np.array([0, 2, 2, 1, 3, 0, 2, 3, 1, 2], np.int64)
    T, topk, E, N, K = 5, 2, 4, 6, 16
    rng = np.random.Generator(np.random.Philox(8))
    x = rng.standard_normal((T, K)).astype(np.float32)
    w = rng.standard_normal((E, N, K)).astype(np.float32)
    tw = rng.random(T * topk).astype(np.float32)
    sp, se = oracle.moe_sort_pairs(ids, E)
    assert np.all(np.diff(se) >= 0) and sorted(sp.tolist()) == list(range(T * topk))
    out = oracle.moe_gemm_f32(x, w, sp, se, tw, T * topk, topk, row_per_pair=False)
    for p in range(T * topk):
        want = (x[p // topk].astype(np.float64) @ w[ids[p]].astype(np.float64).T) * tw[p]
        assert np.allclose(out[p], want, rtol=1e-5, atol=1e-5)
    # second GEMM of an MoE layer: one input row per pair, no weights
    h = rng.standard_normal((T * topk, K)).astype(np.float32)
    out2 = oracle.moe_gemm_f32(h, w, sp, se, None, T * topk, topk, row_per_pair=True)
    for p in range(T * topk):
        assert np.allclose(out2[p], h[p].astype(np.float64) @ w[ids[p]].astype(np.float64).T, rtol=1e-5, atol=1e-5)


def test_deepseek_router(oracle):
    """models/deepseek_route.go:30-133, V3 branch: sigmoid scores + bias pick the experts, the
    unbiased scores weight them, renormalised."""
    rng = np.random.Generator(np.random.Philox(10))
    T, E, topk = 7, 16, 4
    logits = rng.standard_normal((T, E)).astype(np.float32)
    bias = (rng.standard_normal(E) * 0.5).astype(np.float32)
    ids, ws = oracle.deepseek_route_sigmoid(logits, bias, topk, True)
    sc = 1 / (1 + np.exp(-logits.astype(np.float64)))
    for t in range(T):
        order = np.argsort(-(sc[t] + bias), kind="stable")[:topk]
        assert np.array_equal(ids[t], order)
        assert np.allclose(ws[t], sc[t][order] / sc[t][order].sum(), rtol=1e-6)
