"""The oracle's decode-step attention (ops/decode_attn.go:13-170 restated) against an independent f64
softmax attention in numpy, on the shapes of the reference's own test (ops/decode_attn_cuda_test.go:30-38)."""
import numpy as np
import pytest

# name, B, NH, KH, HD, capacity, n, window  (the f32 and bf16 cases alike: the oracle computes on f32 arrays)
CASES = [("short", 2, 8, 2, 64, 256, 7, 0), ("llama-ish", 1, 32, 8, 64, 512, 300, 0), ("qwen-ish", 1, 16, 2, 128, 512, 129, 0),
         ("hd256 g1", 1, 4, 4, 256, 256, 200, 0), ("window mid-block", 1, 4, 1, 256, 1024, 700, 512),
         ("window short", 2, 8, 2, 64, 256, 100, 33), ("window wider than n", 1, 8, 2, 64, 256, 20, 512),
         ("hd512", 1, 8, 2, 512, 1024, 650, 0)]


def attention_f64(q, kbuf, vbuf, n, scale, window):
    B, NH, _, D = q.shape
    KH = kbuf.shape[1]
    g = NH // KH
    start = n - window if 0 < window < n else 0
    out = np.zeros((B, NH, 1, D))
    for b in range(B):
        for h in range(NH):
            K = kbuf[b, h // g, start:n].astype(np.float64)
            V = vbuf[b, h // g, start:n].astype(np.float64)
            s = K @ q[b, h, 0].astype(np.float64) * scale
            p = np.exp(s - s.max())
            out[b, h, 0] = (p / p.sum()) @ V
    return out


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_oracle_attention(oracle, case):
    _, B, NH, KH, D, cap, n, window = case
    rng = np.random.Generator(np.random.Philox(70))
    kbuf = rng.standard_normal((B, KH, cap, D)).astype(np.float32)
    vbuf = rng.standard_normal((B, KH, cap, D)).astype(np.float32)
    q = rng.standard_normal((B, NH, 1, D)).astype(np.float32)
    k, v = rng.standard_normal((B, KH, 1, D)).astype(np.float32), rng.standard_normal((B, KH, 1, D)).astype(np.float32)
    oracle.kv_append(kbuf, vbuf, k, v, n - 1)
    assert np.array_equal(kbuf[:, :, n - 1], k[:, :, 0]) and np.array_equal(vbuf[:, :, n - 1], v[:, :, 0])
    got = oracle.decode_attn(q, kbuf, vbuf, n - 1, 1 / np.sqrt(D), window)
    want = attention_f64(q, kbuf, vbuf, n, 1 / np.sqrt(D), window)
    assert np.max(np.abs(got - want) / np.maximum(1, np.abs(want))) <= 1e-5


def test_oracle_rejects_positions_outside_the_cache(oracle):
    kbuf = np.zeros((1, 1, 8, 32), np.float32)
    k = np.zeros((1, 1, 1, 32), np.float32)
    with pytest.raises(Exception):
        oracle.kv_append(kbuf, kbuf.copy(), k, k, 8)
    with pytest.raises(Exception):
        oracle.decode_attn(np.zeros((1, 1, 1, 32), np.float32), kbuf, kbuf, 8, 1.0)
