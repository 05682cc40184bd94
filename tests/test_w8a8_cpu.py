"""The oracle's W8A8 path (ops/matmul_w8a8.go:65-120 restated) against an independent numpy statement of the same
arithmetic: int8 rows by amax / 127 with round-half-to-even, exact int32 accumulation, f32 epilogue in the
reference's order."""
import numpy as np
import pytest

CASES = [(1, 256, 512), (7, 1024, 1000), (64, 2048, 2048), (130, 512, 4)]  # ops/matmul_w8a8_test.go:25


def reference(x, wq, ws):
    amax = np.abs(x).max(axis=1)
    scale = (amax / np.float32(127)).astype(np.float32)
    inv = np.where(scale > 0, np.float32(1) / np.where(scale > 0, scale, 1).astype(np.float32), 0).astype(np.float32)
    q = np.clip(np.rint((x * inv[:, None]).astype(np.float32)), -127, 127).astype(np.int8)
    acc = q.astype(np.int32) @ wq.astype(np.int32).T
    out = (acc.astype(np.float32) * scale[:, None]).astype(np.float32) * ws[None, :]
    return q, scale, acc, out.astype(np.float32)


def make(M, K, N, seed=130):
    rng = np.random.Generator(np.random.Philox(seed))
    return (rng.standard_normal((M, K)).astype(np.float32), rng.integers(-127, 128, size=(N, K)).astype(np.int8),
            (0.005 + 0.02 * rng.random(N)).astype(np.float32))


@pytest.mark.parametrize("M,K,N", CASES)
def test_oracle_w8a8(oracle, M, K, N):
    x, wq, ws = make(M, K, N)
    x[0, :3] = [0.5, 1.5, 2.5]  # ties
    q, scale, acc, out = reference(x, wq, ws)
    gq, gs = oracle.quantize_rows_int8(x)
    assert np.array_equal(gq, q) and np.array_equal(gs, scale)
    gout, gacc = oracle.matmul_w8a8(x, wq, ws)
    assert np.array_equal(gacc, acc)
    assert np.array_equal(gout.view(np.uint32), out.view(np.uint32))


def test_zero_row(oracle):
    x = np.zeros((2, 64), np.float32)
    x[1, 5] = -3.0
    q, s = oracle.quantize_rows_int8(x)
    assert s[0] == 0 and not q[0].any() and q[1, 5] == -127
