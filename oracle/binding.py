"""ctypes binding of the CPU oracle (oracle/light_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by ``__graft_entry__.smoke()`` and by the
``cpu_baseline`` / ``--impl reference`` legs of bench.py -- never by the ``light_b200``
package.  Arrays are numpy, contiguous, little-endian.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "liblight_oracle.so")

# ggml on-disk type codes (gguf/types.go:39-58 of the reference)
Q4_0, Q5_0, Q8_0, Q4_K, Q5_K, Q6_K = 2, 6, 8, 12, 13, 14
GGUF_TYPES = {"q4_0": Q4_0, "q5_0": Q5_0, "q8_0": Q8_0, "q4_k": Q4_K, "q5_k": Q5_K, "q6_k": Q6_K}


def build(force: bool = False) -> None:
    """Compile liblight_oracle.so (and, when the reference checkout is present, its CUDA
    kernels into oracle/_ref/)."""
    if force and os.path.exists(LIB_PATH):
        os.remove(LIB_PATH)
    ref = os.environ.get("LIGHT_REFERENCE_DIR", "")
    if not ref:  # the checkout sits beside this repository where the build is developed; absent elsewhere
        cand = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
        ref = cand if os.path.isdir(os.path.join(cand, "kernels", "cuda", "src")) else ""
    subprocess.run(["make", "-s", "-C", HERE] + ([f"REF={ref}"] if ref else []), check=True)


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        src = os.path.join(HERE, "light_oracle.c")
        if not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src):
            build()
        _lib = C.CDLL(LIB_PATH)
        _lib.lo_f16_to_f32.restype = C.c_float
        _lib.lo_f16_to_f32.argtypes = [C.c_uint16]
        _lib.lo_f32_to_f16.restype = C.c_uint16
        _lib.lo_f32_to_f16.argtypes = [C.c_float]
        _lib.lo_f32_to_bf16.restype = C.c_uint16
        _lib.lo_f32_to_bf16.argtypes = [C.c_float]
        _lib.lo_bf16_to_f32.restype = C.c_float
        _lib.lo_bf16_to_f32.argtypes = [C.c_uint16]
        _lib.lo_e4m3_to_f32.restype = C.c_float
        _lib.lo_e4m3_to_f32.argtypes = [C.c_uint8]
        _lib.lo_f32_to_e4m3.restype = C.c_uint8
        _lib.lo_f32_to_e4m3.argtypes = [C.c_float]
    return _lib


def _p(a: np.ndarray | None):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.c_void_p)


def _chk(rc: int, what: str) -> None:
    if rc != 0:
        raise ValueError(f"oracle {what}: rejected arguments (rc={rc})")


def block_elems(dt: int) -> int:
    return lib().lo_block_elems(dt)


def block_bytes(dt: int) -> int:
    return lib().lo_block_bytes(dt)


def f16_to_f32(h: int) -> float:
    return lib().lo_f16_to_f32(h)


def f32_to_f16(f: float) -> int:
    return lib().lo_f32_to_f16(f)


def f32_to_bf16(f: float) -> int:
    return lib().lo_f32_to_bf16(f)


def bf16_to_f32(b: int) -> float:
    return lib().lo_bf16_to_f32(b)


def e4m3_to_f32(c: int) -> float:
    return lib().lo_e4m3_to_f32(c)


def f32_to_e4m3(f: float) -> int:
    return lib().lo_f32_to_e4m3(f)


def e4m3_table() -> np.ndarray:
    return np.array([e4m3_to_f32(i) for i in range(256)], dtype=np.float32)


def dequant(dt: int, raw: np.ndarray, n_elems: int) -> np.ndarray:
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    out = np.empty(n_elems, dtype=np.float32)
    _chk(lib().lo_dequant(dt, _p(raw), _p(out), C.c_int64(n_elems)), "dequant")
    return out


def quantize_q8_0(src: np.ndarray) -> np.ndarray:
    src = np.ascontiguousarray(src, dtype=np.float32).ravel()
    out = np.empty(src.size // 32 * 34, dtype=np.uint8)
    _chk(lib().lo_quantize_q8_0(_p(src), _p(out), C.c_int64(src.size)), "quantize_q8_0")
    return out


def matmul_q(dt: int, x: np.ndarray, w: np.ndarray, N: int, threads: int = 1) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.uint8)
    M, K = x.shape
    out = np.empty((M, N), dtype=np.float32)
    _chk(lib().lo_matmul_q(dt, _p(x), _p(w), _p(out), M, N, K, threads), "matmul_q")
    return out


def int4_dequant(codes, s, z, G: int, bf16: bool = False) -> np.ndarray:
    codes = np.ascontiguousarray(codes, dtype=np.uint32)
    s = np.ascontiguousarray(s, dtype=np.float32)
    z = np.ascontiguousarray(z, dtype=np.float32)
    N, K = codes.shape[0], codes.shape[1] * 8
    out = np.empty((N, K), dtype=np.uint16 if bf16 else np.float32)
    _chk(lib().lo_int4_dequant(_p(codes), _p(s), _p(z), _p(out), N, K, G, int(bf16)), "int4_dequant")
    return out


def int4_matmul(x, codes, s, z, G: int, threads: int = 1) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    codes = np.ascontiguousarray(codes, dtype=np.uint32)
    s = np.ascontiguousarray(s, dtype=np.float32)
    z = np.ascontiguousarray(z, dtype=np.float32)
    M, K = x.shape
    N = codes.shape[0]
    out = np.empty((M, N), dtype=np.float32)
    _chk(lib().lo_int4_matmul(_p(x), _p(codes), _p(s), _p(z), _p(out), M, N, K, G, threads), "int4_matmul")
    return out


def int4_from_gptq(qweight, qzeros, scales, group: int, v2: bool = False):
    qweight = np.ascontiguousarray(qweight).view(np.uint32)
    qzeros = np.ascontiguousarray(qzeros).view(np.uint32)
    scales = np.ascontiguousarray(scales, dtype=np.float32)
    K, N = qweight.shape[0] * 8, qweight.shape[1]
    G = K // group
    codes = np.empty((N, K // 8), np.uint32)
    sc = np.empty((N, G), np.float32)
    zr = np.empty((N, G), np.float32)
    _chk(lib().lo_int4_from_gptq(_p(qweight), _p(qzeros), _p(scales), K, N, group, int(v2), _p(codes), _p(sc), _p(zr)),
         "int4_from_gptq")
    return codes, sc, zr


def int4_from_awq(qweight, qzeros, scales, group: int):
    qweight = np.ascontiguousarray(qweight).view(np.uint32)
    qzeros = np.ascontiguousarray(qzeros).view(np.uint32)
    scales = np.ascontiguousarray(scales, dtype=np.float32)
    K, N = qweight.shape[0], qweight.shape[1] * 8
    G = K // group
    codes = np.empty((N, K // 8), np.uint32)
    sc = np.empty((N, G), np.float32)
    zr = np.empty((N, G), np.float32)
    _chk(lib().lo_int4_from_awq(_p(qweight), _p(qzeros), _p(scales), K, N, group, _p(codes), _p(sc), _p(zr)),
         "int4_from_awq")
    return codes, sc, zr


def fp8_block_dequant(w, s, bR: int, bC: int, bf16: bool = False) -> np.ndarray:
    w = np.ascontiguousarray(w, dtype=np.uint8)
    s = np.ascontiguousarray(s, dtype=np.float32)
    R, Cc = w.shape
    out = np.empty((R, Cc), dtype=np.uint16 if bf16 else np.float32)
    _chk(lib().lo_fp8_block_dequant(_p(w), _p(s), _p(out), R, Cc, bR, bC, int(bf16)), "fp8_block_dequant")
    return out


def matmul_f32_tb(x, w, threads: int = 1) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    M, K = x.shape
    N = w.shape[0]
    out = np.empty((M, N), dtype=np.float32)
    _chk(lib().lo_matmul_f32_tb(_p(x), _p(w), _p(out), M, N, K, threads), "matmul_f32_tb")
    return out


def moe_sort_pairs(ids, E: int):
    ids = np.ascontiguousarray(ids, dtype=np.int64).ravel()
    sp = np.empty_like(ids)
    se = np.empty_like(ids)
    _chk(lib().lo_moe_sort_pairs(_p(ids), C.c_int64(ids.size), E, _p(sp), _p(se)), "moe_sort_pairs")
    return sp, se


def moe_gemm_f32(inp, w, pairs, expts, topkw, sizeM: int, topk: int, row_per_pair: bool, threads: int = 1,
                 out: np.ndarray | None = None) -> np.ndarray:
    inp = np.ascontiguousarray(inp, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    pairs = np.ascontiguousarray(pairs, dtype=np.int64)
    expts = np.ascontiguousarray(expts, dtype=np.int64)
    if topkw is not None:
        topkw = np.ascontiguousarray(topkw, dtype=np.float32)
    E, N, K = w.shape
    if out is None:
        out = np.zeros((sizeM, N), dtype=np.float32)
    _chk(lib().lo_moe_gemm_f32(_p(inp), _p(w), _p(pairs), _p(expts), _p(topkw), _p(out), C.c_int64(pairs.size),
                               C.c_int64(sizeM), N, K, topk, int(row_per_pair), threads), "moe_gemm_f32")
    return out


def deepseek_route_sigmoid(logits, bias, topk: int, norm_topk: bool = True):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    if bias is not None:
        bias = np.ascontiguousarray(bias, dtype=np.float32)
    T, E = logits.shape
    ids = np.empty((T, topk), np.int64)
    ws = np.empty((T, topk), np.float32)
    _chk(lib().lo_deepseek_route_sigmoid(_p(logits), _p(bias), T, E, topk, int(norm_topk), _p(ids), _p(ws)),
         "deepseek_route")
    return ids, ws


def deepseek_route(logits, bias, topk: int, n_group: int = 1, topk_group: int = 1, sigmoid: bool = True, norm_topk: bool = True):
    """models/deepseek_route.go:30-133, every branch -> (ids (T, topk) i64, weights (T, topk) f32)."""
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    if bias is not None:
        bias = np.ascontiguousarray(bias, dtype=np.float32)
    T, E = logits.shape
    ids = np.empty((T, topk), np.int64)
    ws = np.empty((T, topk), np.float32)
    _chk(lib().lo_deepseek_route(_p(logits), _p(bias), T, E, topk, n_group, topk_group, int(sigmoid), int(norm_topk), _p(ids), _p(ws)), "deepseek_route")
    return ids, ws


def moe_route_topk(probs, topk: int, normalize: bool):
    """ops.MoERoute's selection (ops/moe.go:29-50) -> (ids (T, topk) i64, weights (T, topk) f32)."""
    probs = np.ascontiguousarray(probs, dtype=np.float32)
    T, E = probs.shape
    ids = np.empty((T, topk), np.int64)
    ws = np.empty((T, topk), np.float32)
    _chk(lib().lo_moe_route_topk(_p(probs), T, E, topk, int(normalize), _p(ids), _p(ws)), "moe_route_topk")
    return ids, ws


def kv_append(kbuf: np.ndarray, vbuf: np.ndarray, k: np.ndarray, v: np.ndarray, pos: int) -> None:
    """In place; arrays of any one element size, kbuf / vbuf (B, KH, Cap, D), k / v (B, KH, 1, D)."""
    B, KH, Cap, D = kbuf.shape
    assert kbuf.flags.c_contiguous and vbuf.flags.c_contiguous and k.dtype == kbuf.dtype
    k, v = np.ascontiguousarray(k), np.ascontiguousarray(v)
    _chk(lib().lo_kv_append(_p(k), _p(v), _p(kbuf), _p(vbuf), C.c_int64(pos), B, KH, D, Cap, kbuf.dtype.itemsize), "kv_append")


def decode_attn(q, kbuf, vbuf, pos: int, scale: float, window: int = 0) -> np.ndarray:
    """q (B, NH, 1, D), buffers (B, KH, Cap, D), all f32 -> (B, NH, 1, D) f32."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    kbuf = np.ascontiguousarray(kbuf, dtype=np.float32)
    vbuf = np.ascontiguousarray(vbuf, dtype=np.float32)
    B, NH, _, D = q.shape
    KH, Cap = kbuf.shape[1], kbuf.shape[2]
    out = np.empty_like(q)
    _chk(lib().lo_decode_attn(_p(q), _p(kbuf), _p(vbuf), C.c_int64(pos), _p(out), B, NH, KH, Cap, D, C.c_float(scale), window),
         "decode_attn")
    return out


def rmsnorm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    out = np.empty_like(x)
    _chk(lib().lo_rmsnorm_f32(_p(x), _p(w), _p(out), C.c_int64(x.size // x.shape[-1]), x.shape[-1], C.c_double(eps)), "rmsnorm")
    return out


def rope(x: np.ndarray, positions: np.ndarray, base: float) -> np.ndarray:
    """x (..., seq_len, head_dim) f32, positions (seq_len,) i64."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    positions = np.ascontiguousarray(positions, dtype=np.int64)
    out = np.empty_like(x)
    seq_len, hd = x.shape[-2], x.shape[-1]
    _chk(lib().lo_rope_f32(_p(x), _p(positions), _p(out), C.c_int64(x.size // (seq_len * hd)), seq_len, hd, C.c_double(base)), "rope")
    return out


def quantize_rows_int8(x: np.ndarray):
    x = np.ascontiguousarray(x, dtype=np.float32)
    M, K = x.shape
    q, s = np.empty((M, K), np.int8), np.empty(M, np.float32)
    _chk(lib().lo_quantize_rows_int8(_p(x), _p(q), _p(s), C.c_int64(M), K), "quantize_rows_int8")
    return q, s


def matmul_w8a8(x: np.ndarray, wq: np.ndarray, ws: np.ndarray):
    """-> (out f32 (M, N), the int32 accumulators)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    wq = np.ascontiguousarray(wq, dtype=np.int8)
    ws = np.ascontiguousarray(ws, dtype=np.float32)
    M, K = x.shape
    N = wq.shape[0]
    out, acc = np.empty((M, N), np.float32), np.empty((M, N), np.int32)
    _chk(lib().lo_matmul_w8a8(_p(x), _p(wq), _p(ws), _p(out), _p(acc), M, N, K), "matmul_w8a8")
    return out, acc


def has_avx2() -> bool:
    return bool(lib().lo_has_avx2())


def decode_row_avx2(dt: int, raw: np.ndarray, K: int) -> np.ndarray:
    """One weight row through the AVX2 row decoder of its format (kernels/cpu/quant_matmul.go:208-250)."""
    raw = np.ascontiguousarray(raw, np.uint8)
    out = np.empty(K, np.float32)
    _chk(lib().lo_decode_row_avx2(dt, _p(raw), _p(out), K), "decode_row_avx2")
    return out


def int4_row_avx2(codes: np.ndarray, s: np.ndarray, z: np.ndarray, G: int) -> np.ndarray:
    """One canonical int4 row (K / 8 words, K / G scales and zeros) through int4RowAVX2's restatement."""
    codes = np.ascontiguousarray(codes, np.uint32)
    K = codes.size * 8
    out = np.empty(K, np.float32)
    _chk(lib().lo_int4_row_avx2(_p(codes), _p(np.ascontiguousarray(s, np.float32)), _p(np.ascontiguousarray(z, np.float32)), _p(out), K, G),
         "int4_row_avx2")
    return out
