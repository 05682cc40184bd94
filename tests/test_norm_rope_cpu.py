"""The oracle's RMSNorm and RoPE (kernels/cpu/norm.go:27-51, kernels/cpu/misc_registry.go:27-62 restated)
against the reference's own known-answer tests (ops/norm_test.go:11-46) and independent f64 formulas."""
import numpy as np


def test_rmsnorm_kat(oracle):
    # TestRMSNorm: x = [1, 2, 3], w = 1, eps = 1e-6 -> x / sqrt(14 / 3 + 1e-6)
    x = np.array([[1.0, 2.0, 3.0]], np.float32)
    got = oracle.rmsnorm(x, np.ones(3, np.float32), 1e-6)
    rms = np.float32(np.sqrt(14.0 / 3.0 + 1e-6))
    assert np.max(np.abs(got[0] - x[0] / rms)) <= 1e-5
    # TestRMSNormWeight: w = [1, 1, 2] -> y[2] / y[0] = 6
    got = oracle.rmsnorm(x, np.array([1, 1, 2], np.float32), 1e-6)
    assert abs(got[0, 2] / got[0, 0] - 6.0) <= 1e-4


def test_rmsnorm_f64(oracle):
    rng = np.random.Generator(np.random.Philox(90))
    x = rng.standard_normal((5, 4096)).astype(np.float32) * 3
    w = rng.standard_normal(4096).astype(np.float32)
    want = x.astype(np.float64) / np.sqrt((x.astype(np.float64) ** 2).mean(-1, keepdims=True) + 1e-5) * w
    assert np.max(np.abs(oracle.rmsnorm(x, w, 1e-5) - want) / (1 + np.abs(want))) <= 1e-5


def rope_f64(x, positions, base):
    hd = x.shape[-1]
    half = hd // 2
    inv = base ** (-2.0 * np.arange(half) / hd)
    th = positions.astype(np.float64)[:, None] * inv[None, :]
    x0, x1 = x[..., :half].astype(np.float64), x[..., half:].astype(np.float64)
    return np.concatenate([x0 * np.cos(th) - x1 * np.sin(th), x0 * np.sin(th) + x1 * np.cos(th)], -1)


def test_rope_f64(oracle):
    rng = np.random.Generator(np.random.Philox(91))
    x = rng.standard_normal((2, 8, 6, 128)).astype(np.float32)
    pos = np.array([0, 1, 17, 1023, 4095, 100000], np.int64)
    got = oracle.rope(x, pos, 500000.0)
    assert np.max(np.abs(got - rope_f64(x, pos, 500000.0))) <= 1e-6
    assert np.array_equal(got[:, :, 0], x[:, :, 0])  # position 0 is the identity
