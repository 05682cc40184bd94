"""The oracle's AVX2 row decoders produce exactly the scalar decoders' floats -- the reference's own check of
its assembly decoders (kernels/cpu/qdecode_test.go:38-89: K = 1024, 20 rows per format, random bytes with
small f16 scale fields; int4 at G = 32 and 128) -- and the timed matmul, which uses them, still matches the
f64 dot of the dequantized weights (ops/matmul_q_cpu_test.go:19-81)."""
import numpy as np
import pytest

from light_b200 import synth


def _need_avx2(oracle):
    if not oracle.has_avx2():
        pytest.skip("host has no AVX2 + FMA")


@pytest.mark.parametrize("name", ["q8_0", "q4_0", "q5_0", "q4_k", "q6_k"])
def test_avx2_row_decoders_exact(oracle, name):
    _need_avx2(oracle)
    dt = oracle.GGUF_TYPES[name]
    K = 1024
    for i in range(20):
        raw = synth.random_blocks(1100 + i, dt, 1, K).reshape(-1)
        want = oracle.dequant(dt, raw, K)
        got = oracle.decode_row_avx2(dt, raw, K)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (name, i)


@pytest.mark.parametrize("G", [32, 128])
def test_avx2_int4_row_exact(oracle, G):
    _need_avx2(oracle)
    K = 1024
    rng = np.random.Generator(np.random.Philox(12))
    for _ in range(5):
        codes = rng.integers(0, 1 << 32, K // 8, dtype=np.uint64).astype(np.uint32)
        s = (0.01 * rng.random(K // G)).astype(np.float32)
        z = (8 * rng.random(K // G)).astype(np.float32)
        got = oracle.int4_row_avx2(codes, s, z, G)
        want = oracle.int4_dequant(codes.reshape(1, -1), s.reshape(1, -1), z.reshape(1, -1), G).reshape(-1)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("name", ["q8_0", "q4_k", "q6_k"])
@pytest.mark.parametrize("M", [1, 9])
def test_matmul_q_with_avx2_rows_matches_f64(oracle, name, M):
    dt = oracle.GGUF_TYPES[name]
    N, K = 37, 512
    raw = synth.random_blocks(77, dt, N, K).reshape(-1)
    x = np.random.Generator(np.random.Philox(78)).standard_normal((M, K)).astype(np.float32)
    got = oracle.matmul_q(dt, x, raw, N, threads=3)
    w = oracle.dequant(dt, raw, N * K).reshape(N, K).astype(np.float64)
    want = x.astype(np.float64) @ w.T
    tol = 1e-5 * (1 + np.abs(x.astype(np.float64))[:, None, :] * np.abs(w)[None, :, :]).sum(-1)
    assert (np.abs(got - want) <= tol).all()
