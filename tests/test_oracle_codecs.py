"""Pins the oracle's scalar codecs (dtype/half.go, dtype/f8.go of the reference) against
independent implementations: numpy float16, torch bfloat16 and torch float8_e4m3fn."""
import numpy as np
import torch


def test_f16_decode_all_codes(oracle):
    bits = np.arange(65536, dtype=np.uint16)
    want = bits.view(np.float16).astype(np.float32)
    got = np.array([oracle.f16_to_f32(int(b)) for b in bits], np.float32)
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(got[~nan].view(np.uint32), want[~nan].view(np.uint32))


def test_f16_encode_rne(oracle):
    rng = np.random.Generator(np.random.Philox(3))
    vals = np.concatenate([
        rng.standard_normal(4000).astype(np.float32) * 10.0 ** rng.integers(-9, 6, 4000),
        np.array([0.0, -0.0, 65504.0, 65520.0, 65519.99, 1e-8, 5.96e-8, 2.98e-8, 6.1e-5, np.inf, -np.inf], np.float32),
        # exact ties between neighbouring f16 values
        (np.arange(1024, 1100, dtype=np.float32) + 0.5) * np.float32(2.0 ** -10),
    ]).astype(np.float32)
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).view(np.uint16)
    got = np.array([oracle.f32_to_f16(float(v)) for v in vals], np.uint16)
    # One deliberate deviation from IEEE: the reference flushes everything below 2^-24 to zero
    # (dtype/half.go:45-48, `realExp < -24`), although (2^-25, 2^-24) rounds up to the smallest
    # subnormal under round-to-nearest-even.  The oracle restates the reference, quirk included.
    quirk = (np.abs(vals) > 2.0 ** -25) & (np.abs(vals) < 2.0 ** -24)
    assert quirk.any()
    assert np.array_equal(got[~quirk], want[~quirk])
    assert np.all((got[quirk] & 0x7FFF) == 0) and np.all((want[quirk] & 0x7FFF) == 1)


def test_bf16_rne_matches_torch(oracle):
    g = torch.Generator().manual_seed(5)
    vals = torch.randn(5000, generator=g) * 10.0 ** torch.randint(-6, 6, (5000,), generator=g)
    want = vals.to(torch.bfloat16).view(torch.int16).numpy().astype(np.uint16)
    got = np.array([oracle.f32_to_bf16(float(v)) for v in vals.numpy()], np.uint16)
    assert np.array_equal(got, want)
    back = np.array([oracle.bf16_to_f32(int(b)) for b in got], np.float32)
    assert np.array_equal(back, vals.to(torch.bfloat16).float().numpy())


def test_e4m3_decode_matches_torch(oracle):
    codes = torch.arange(256, dtype=torch.uint8)
    want = codes.view(torch.float8_e4m3fn).float().numpy()
    got = oracle.e4m3_table()
    nan = np.isnan(want)
    assert list(np.nonzero(nan)[0]) == [0x7F, 0xFF]
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(got[~nan], want[~nan])


def test_e4m3_half_trick_table(oracle):
    """ops/fp8_block_test.go:74-104 (TestFP8HalfTrickMatchesDecoder): the word-level bit trick of
    the reference CUDA kernels reproduces the decoder for all non-NaN codes in all 4 byte lanes."""
    for c in range(256):
        if c & 0x7F == 0x7F:
            continue
        want = oracle.e4m3_to_f32(c)
        for pos in range(4):
            v = (c << (8 * pos)) & 0xFFFFFFFF
            lo = (((v & 0x007F007F) << 7) | ((v & 0x00800080) << 8)) & 0xFFFFFFFF
            hi = ((v & 0x7F007F00) >> 1) | (v & 0x80008000)
            bits = [lo & 0xFFFF, hi & 0xFFFF, lo >> 16, hi >> 16][pos]
            assert oracle.f16_to_f32(bits) * 256 == want, (c, pos)


def test_e4m3_encode_matches_torch_and_saturates(oracle):
    g = torch.Generator().manual_seed(7)
    vals = torch.cat([torch.randn(4000, generator=g) * 60, torch.randn(2000, generator=g) * 0.01,
                      torch.tensor([0.0, 448.0, 464.0, 1e9, -1e9, 2.0 ** -9, 2.0 ** -10, 0.0175])])
    got = np.array([oracle.f32_to_e4m3(float(v)) for v in vals.numpy()], np.uint8)
    inr = vals.abs() <= 448
    want = vals[inr].to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(got[inr.numpy()], want)
    # saturating: beyond +-448 clamps to 0x7E / 0xFE (dtype/f8.go:33-35)
    assert oracle.f32_to_e4m3(1e9) == 0x7E and oracle.f32_to_e4m3(-1e9) == 0xFE
    assert oracle.f32_to_e4m3(float("nan")) == 0x7F


def test_block_geometry(oracle):
    """dtype/dtype.go:53-60."""
    want = {oracle.Q4_0: (32, 18), oracle.Q5_0: (32, 22), oracle.Q8_0: (32, 34), oracle.Q4_K: (256, 144),
            oracle.Q5_K: (256, 176), oracle.Q6_K: (256, 210)}
    for dt, (be, bb) in want.items():
        assert oracle.block_elems(dt) == be and oracle.block_bytes(dt) == bb
    assert oracle.block_elems(99) == 0
