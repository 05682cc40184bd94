"""Seeded synthetic weights in the on-disk block layouts of the hot path.

Real checkpoints are not available offline, so tests, the smoke run and the benchmark
use weights made here.  Two kinds:

* ``random_blocks``: uniformly random block bytes with the f16 scale fields forced into
  [2^-6, 2^-5) -- the construction the reference's own CUDA parity tests use
  (ops/matmul_q_test.go:19-56).  Every code value occurs, so this is the parity workload.
* ``quantize_q4_k`` / ``quantize_q6_k`` / ``quantize_q8_0``: layout-valid encoders for
  N(0, sigma) weights.  The reference has no K-quant encoder (quant/quantize.go:14-20), and
  these are NOT ggml's search-based quantizers either: they are a plain min/max affine fit
  per sub-block, good enough to give decode-realistic value distributions.  Only the
  byte layout is normative (quant/q4_k.go:14-24, quant/q6_k.go:11-32, quant/q8_0.go:11-17).

Everything is torch, so the same code makes small CPU fixtures and multi-GB weights
directly in device memory.
"""
from __future__ import annotations

import numpy as np
import torch

Q4_0, Q5_0, Q8_0, Q4_K, Q5_K, Q6_K = 2, 6, 8, 12, 13, 14
BLOCK = {Q4_0: (32, 18), Q5_0: (32, 22), Q8_0: (32, 34), Q4_K: (256, 144), Q5_K: (256, 176), Q6_K: (256, 210)}
# byte offsets of the f16 scale fields inside one block
_F16_FIELDS = {Q4_0: (0,), Q5_0: (0,), Q8_0: (0,), Q4_K: (0, 2), Q5_K: (0, 2), Q6_K: (208,)}


def row_bytes(dt: int, K: int) -> int:
    be, bb = BLOCK[dt]
    assert K % be == 0
    return K // be * bb


def random_blocks(seed: int, dt: int, N: int, K: int) -> np.ndarray:
    """(N, K) weight as uint8 [N, row_bytes]: random bytes, f16 scales in [2^-6, 2^-5)."""
    be, bb = BLOCK[dt]
    rng = np.random.Generator(np.random.Philox(seed))
    nb = N * K // be
    buf = rng.integers(0, 256, size=(nb, bb), dtype=np.uint8)
    for off in _F16_FIELDS[dt]:
        h = (0x2400 | rng.integers(0, 0x400, size=nb)).astype(np.uint16)
        buf[:, off] = (h & 0xFF).astype(np.uint8)
        buf[:, off + 1] = (h >> 8).astype(np.uint8)
    return buf.reshape(N, K // be * bb)


def _f16_bytes(v: torch.Tensor) -> torch.Tensor:
    """f32 [n] -> uint8 [n, 2] little-endian f16 (round to nearest even)."""
    return v.to(torch.float16).view(torch.uint8).reshape(-1, 2)


def pack_q4_k(d: torch.Tensor, dmin: torch.Tensor, sc: torch.Tensor, mn: torch.Tensor, q: torch.Tensor) -> torch.Tensor:
    """Pack Q4_K super-blocks.  d, dmin f32 [nb]; sc, mn int [nb, 8] in 0..63; q int [nb, 256]
    in 0..15 -> uint8 [nb, 144] (quant/q4_k.go:14-24; scale packing of getScaleMinK4)."""
    nb = d.shape[0]
    sc = sc.to(torch.int32)
    mn = mn.to(torch.int32)
    q = q.to(torch.int32)
    out = torch.empty(nb, 144, dtype=torch.uint8, device=d.device)
    out[:, 0:2] = _f16_bytes(d)
    out[:, 2:4] = _f16_bytes(dmin)
    s12 = torch.empty(nb, 12, dtype=torch.int32, device=d.device)
    s12[:, 0:4] = (sc[:, 0:4] & 0x3F) | ((sc[:, 4:8] & 0x30) << 2)
    s12[:, 4:8] = (mn[:, 0:4] & 0x3F) | ((mn[:, 4:8] & 0x30) << 2)
    s12[:, 8:12] = (sc[:, 4:8] & 0x0F) | ((mn[:, 4:8] & 0x0F) << 4)
    out[:, 4:16] = s12.to(torch.uint8)
    q4 = q.reshape(nb, 4, 2, 32)  # pair p, (low | high) half, l
    out[:, 16:144] = ((q4[:, :, 0, :] & 0xF) | ((q4[:, :, 1, :] & 0xF) << 4)).reshape(nb, 128).to(torch.uint8)
    return out


def pack_q6_k(d: torch.Tensor, sc: torch.Tensor, raw: torch.Tensor) -> torch.Tensor:
    """Pack Q6_K super-blocks.  d f32 [nb]; sc int [nb, 16] in -128..127; raw int [nb, 256] in
    0..63 (= q + 32) -> uint8 [nb, 210] (quant/q6_k.go:11-32)."""
    nb = d.shape[0]
    r = raw.to(torch.int32).reshape(nb, 2, 4, 32)  # half, group (l, l+32, l+64, l+96), l
    ql = torch.empty(nb, 2, 64, dtype=torch.int32, device=d.device)
    ql[:, :, 0:32] = (r[:, :, 0] & 0xF) | ((r[:, :, 2] & 0xF) << 4)
    ql[:, :, 32:64] = (r[:, :, 1] & 0xF) | ((r[:, :, 3] & 0xF) << 4)
    qh = ((r[:, :, 0] >> 4) & 3) | (((r[:, :, 1] >> 4) & 3) << 2) | (((r[:, :, 2] >> 4) & 3) << 4) | (
        ((r[:, :, 3] >> 4) & 3) << 6)
    out = torch.empty(nb, 210, dtype=torch.uint8, device=d.device)
    out[:, 0:128] = ql.reshape(nb, 128).to(torch.uint8)
    out[:, 128:192] = qh.reshape(nb, 64).to(torch.uint8)
    out[:, 192:208] = sc.to(torch.int8).view(torch.uint8)
    out[:, 208:210] = _f16_bytes(d)
    return out


def pack_q8_0(d: torch.Tensor, q: torch.Tensor) -> torch.Tensor:
    """d f32 [nb]; q int [nb, 32] in -128..127 -> uint8 [nb, 34] (quant/q8_0.go:11-17)."""
    nb = d.shape[0]
    out = torch.empty(nb, 34, dtype=torch.uint8, device=d.device)
    out[:, 0:2] = _f16_bytes(d)
    out[:, 2:34] = q.to(torch.int8).view(torch.uint8)
    return out


def quantize_q4_k(w: torch.Tensor) -> torch.Tensor:
    """f32 [N, K] -> uint8 [N, K/256*144].  Min/max affine fit per 32-element sub-block, 6-bit
    sub-block scales/mins against per-super-block f16 d/dmin.  Not ggml's quantizer."""
    N, K = w.shape
    x = w.reshape(-1, 8, 32).float()
    lo = x.amin(dim=2).clamp(max=0.0)
    hi = x.amax(dim=2)
    scale = (hi - lo) / 15.0  # [nb, 8]
    mins = -lo
    d = (scale.amax(dim=1) / 63.0).to(torch.float16).float()
    dmin = (mins.amax(dim=1) / 63.0).to(torch.float16).float()
    sc = torch.where(d[:, None] > 0, torch.round(scale / d[:, None].clamp(min=1e-30)), torch.zeros_like(scale)).clamp(0, 63)
    mn = torch.where(dmin[:, None] > 0, torch.round(mins / dmin[:, None].clamp(min=1e-30)), torch.zeros_like(mins)).clamp(0, 63)
    eff = (d[:, None] * sc)[:, :, None]
    off = (dmin[:, None] * mn)[:, :, None]
    q = torch.where(eff > 0, torch.round((x + off) / eff.clamp(min=1e-30)), torch.zeros_like(x)).clamp(0, 15)
    return pack_q4_k(d, dmin, sc, mn, q.reshape(-1, 256)).reshape(N, K // 256 * 144)


def quantize_q6_k(w: torch.Tensor) -> torch.Tensor:
    """f32 [N, K] -> uint8 [N, K/256*210].  Symmetric fit per 16-element sub-block, int8
    sub-block scales against a per-super-block f16 d.  Not ggml's quantizer."""
    N, K = w.shape
    x = w.reshape(-1, 16, 16).float()
    amax = x.abs().amax(dim=2)
    scale = amax / 31.0  # [nb, 16]
    d = (scale.amax(dim=1) / 127.0).to(torch.float16).float()
    sc = torch.where(d[:, None] > 0, torch.round(scale / d[:, None].clamp(min=1e-30)), torch.zeros_like(scale)).clamp(0, 127)
    eff = (d[:, None] * sc)[:, :, None]
    q = torch.where(eff > 0, torch.round(x / eff.clamp(min=1e-30)), torch.zeros_like(x)).clamp(-32, 31)
    return pack_q6_k(d, sc, (q + 32).reshape(-1, 256)).reshape(N, K // 256 * 210)


def quantize_q8_0(w: torch.Tensor) -> torch.Tensor:
    """f32 [N, K] -> uint8 [N, K/32*34]; d = amax/127, q = round-half-even(v * (1/d)), the
    reference's own Q8_0 encoder (quant/quantize.go:70-86)."""
    N, K = w.shape
    x = w.reshape(-1, 32).float()
    d = x.abs().amax(dim=1) / 127.0
    inv = torch.where(d != 0, 1.0 / d, torch.zeros_like(d))
    q = torch.round(x * inv[:, None]).clamp(-128, 127)
    return pack_q8_0(d, q).reshape(N, K // 32 * 34)


QUANTIZERS = {Q4_K: quantize_q4_k, Q6_K: quantize_q6_k, Q8_0: quantize_q8_0}


def gaussian_weight(seed: int, dt: int, N: int, K: int, sigma: float = 0.02, device="cpu",
                    rows_per_chunk: int = 8192) -> torch.Tensor:
    """N(0, sigma) weight drawn from `seed`, quantized to `dt`: uint8 [N, row_bytes] on `device`."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    out = torch.empty(N, row_bytes(dt, K), dtype=torch.uint8, device=device)
    for r0 in range(0, N, rows_per_chunk):
        r1 = min(N, r0 + rows_per_chunk)
        w = torch.randn(r1 - r0, K, generator=g, device=device, dtype=torch.float32) * sigma
        out[r0:r1] = QUANTIZERS[dt](w)
    return out


# ---------------------------------------------------------------- int4 (GPTQ / AWQ)

def random_int4(seed: int, N: int, K: int, G: int = 128):
    """Canonical 4-bit layout (quant/int4.go:12-31): codes u32 (N, K/8) uniform, scales f32
    (N, K/G) ~ U(0.005, 0.02) rounded through f16, zeros f32 (N, K/G) ~ U{0..15}."""
    rng = np.random.Generator(np.random.Philox(seed))
    codes = rng.integers(0, 2**32, size=(N, K // 8), dtype=np.uint64).astype(np.uint32)
    s = rng.uniform(0.005, 0.02, size=(N, K // G)).astype(np.float16).astype(np.float32)
    z = rng.integers(0, 16, size=(N, K // G)).astype(np.float32)
    return codes, s, z


def _nibbles(codes: np.ndarray) -> np.ndarray:
    """codes u32 (N, K/8) -> uint8 (N, K)."""
    sh = (np.arange(8, dtype=np.uint32) * 4)[None, None, :]
    return ((codes[:, :, None] >> sh) & 0xF).astype(np.uint8).reshape(codes.shape[0], -1)


def to_gptq(codes: np.ndarray, s: np.ndarray, z: np.ndarray, v2: bool = False):
    """Canonical -> AutoGPTQ checkpoint tensors (quant/int4.go:103-110): qweight i32 (K/8, N)
    packed along K, qzeros i32 (K/G, N/8) packed along N (v1 stores zero - 1), scales (K/G, N)."""
    q = _nibbles(codes)  # (N, K)
    N, K = q.shape
    qt = q.T.reshape(K // 8, 8, N).astype(np.uint32)
    qweight = np.zeros((K // 8, N), np.uint32)
    for j in range(8):
        qweight |= qt[:, j, :] << (4 * j)
    zz = (z.T.astype(np.int64) - (0 if v2 else 1)) & 0xF  # (K/G, N)
    zz = zz.reshape(zz.shape[0], N // 8, 8).astype(np.uint32)
    qzeros = np.zeros(zz.shape[:2], np.uint32)
    for j in range(8):
        qzeros |= zz[:, :, j] << (4 * j)
    return qweight, qzeros, np.ascontiguousarray(s.T)


_AWQ_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)


def to_awq(codes: np.ndarray, s: np.ndarray, z: np.ndarray):
    """Canonical -> AutoAWQ GEMM tensors (quant/int4.go:198-204): qweight i32 (K, N/8) and
    qzeros (K/G, N/8) packed along N, nibble i holding column 8c + (0,2,4,6,1,3,5,7)[i]."""
    q = _nibbles(codes)
    N, K = q.shape
    qt = q.T.reshape(K, N // 8, 8).astype(np.uint32)
    qweight = np.zeros((K, N // 8), np.uint32)
    zz = z.T.astype(np.uint32).reshape(-1, N // 8, 8)
    qzeros = np.zeros(zz.shape[:2], np.uint32)
    for i, col in enumerate(_AWQ_ORDER):
        qweight |= qt[:, :, col] << (4 * i)
        qzeros |= zz[:, :, col] << (4 * i)
    return qweight, qzeros, np.ascontiguousarray(s.T)


# ---------------------------------------------------------------- block-scaled FP8

def random_fp8_block(seed: int, N: int, K: int, bR: int = 128, bC: int = 128, sigma: float = 60.0,
                     device="cpu"):
    """e4m3 codes uint8 (N, K) = e4m3(N(0, sigma)) and f32 scales (N/bR, K/bC) ~ U(1e-4, 2.1e-3)
    (value ranges of ops/fp8_block_test.go:110-120).  NaN codes never occur."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    v = torch.randn(N, K, generator=g, device=device) * sigma
    codes = v.clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
    s = torch.rand(N // bR, K // bC, generator=g, device=device) * 2e-3 + 1e-4
    return codes, s.float()
