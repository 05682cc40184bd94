"""No-GPU checks of the C ABI: the library loads, exports every symbol the header declares, and
rejects bad arguments with the documented codes before touching a device."""
import ctypes as C
import os
import re

import pytest
import torch

from light_b200 import _lib, ops

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "light_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(light_b200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = _declared()
    assert len(names) >= 14
    raw = C.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(raw, n), f"{n} declared in include/light_b200.h but not exported"
    assert set(names) == set(_lib.SYMBOLS), "ctypes table and header disagree"


def test_version_and_geometry():
    l = _lib.lib()
    assert l.light_b200_abi_version() == 1
    want = {2: (32, 18), 6: (32, 22), 8: (32, 34), 12: (256, 144), 13: (256, 176), 14: (256, 210), 3: (0, 0)}
    for t, (be, bb) in want.items():
        assert l.light_b200_block_elems(t) == be and l.light_b200_block_bytes(t) == bb


def test_argument_errors_need_no_device():
    l = _lib.lib()
    one = C.c_void_p(16)  # never dereferenced: the checks fail first
    assert l.light_b200_matmul_q(99, one, one, one, 1, 8, 256, 0, None) == -1
    assert "ggml type 99" in _lib.last_error()
    assert l.light_b200_matmul_q(12, one, one, one, 1, 8, 100, 0, None) == -2
    assert "not a multiple of the block size 256" in _lib.last_error()
    assert l.light_b200_matmul_q(12, one, one, one, -1, 8, 256, 0, None) == -2
    assert l.light_b200_matmul_q(12, None, one, one, 1, 8, 256, 0, None) == -3
    assert l.light_b200_matmul_q(12, C.c_void_p(4), one, one, 1, 8, 256, 0, None) == -4
    assert l.light_b200_matmul_q(12, one, one, one, 0, 8, 256, 0, None) == 0  # empty: nothing to do
    assert l.light_b200_dequant(12, one, one, 100, 0, None) == -2
    assert l.light_b200_dequant(7, one, one, 256, 0, None) == -1
    assert l.light_b200_int4_gemv(one, one, one, one, one, 0, 1, 8, 48, 32, 0, None) == -2  # K % 32
    assert l.light_b200_int4_gemv(one, one, one, one, one, 2, 1, 8, 64, 32, 0, None) == -1  # F16 activations
    assert l.light_b200_int4_dequant(one, one, one, one, 0, 4, 64, 12, 0, 0, None) == -2    # G % 8
    assert l.light_b200_fp8_block_dequant(one, one, one, 0, 12, 32, 5, 8, 0, None) == -2    # 12 % 5
    assert l.light_b200_fp8_block_gemv(one, one, one, one, 0, 1, 128, 24, 128, 8, 0, None) == -2
    a = _lib.MoeArgs(E=0, N=4, K=8, topk=1, M=0, size_m=0, dtype=0)
    assert l.light_b200_moe_gemm(C.byref(a), 0, None) == -2
    a = _lib.MoeArgs(E=2, N=4, K=8, topk=1, M=0, size_m=0, dtype=0)
    assert l.light_b200_moe_gemm(C.byref(a), 0, None) == -3  # scratch missing
    assert l.light_b200_moe_gemm(None, 0, None) == -3


def test_host_ops_reject_cpu_tensors_and_bad_shapes():
    w = ops.QTensor(torch.zeros(4 * 144, dtype=torch.uint8), ops.Q4_K, (4, 256))
    with pytest.raises(ValueError, match="CUDA kernels only"):
        ops.MatMulQ(torch.zeros(1, 256), w)
    with pytest.raises(ValueError, match="x must be F32"):
        ops.MatMulQ(torch.zeros(1, 256, dtype=torch.bfloat16), w)
    with pytest.raises(ValueError, match="inner dim mismatch"):
        ops.MatMulQ(torch.zeros(1, 512), w)
    with pytest.raises(ValueError, match="not a multiple"):
        ops.QTensor(torch.zeros(144, dtype=torch.uint8), ops.Q4_K, (1, 100))
    with pytest.raises(ValueError, match="expected"):
        ops.QTensor(torch.zeros(100, dtype=torch.uint8), ops.Q4_K, (1, 256))
    i4 = ops.Int4(torch.zeros(4, 8, dtype=torch.int32), torch.zeros(4, 1), torch.zeros(4, 1), 64)
    with pytest.raises(ValueError, match="want F32 or BF16"):
        ops.MatMulInt4(torch.zeros(1, 64, dtype=torch.float16), i4)
    with pytest.raises(ValueError, match="weight"):
        ops.MatMulInt4(torch.zeros(1, 32), i4)
    r = ops.MoERouteFromIDs(torch.tensor([[0, 1], [1, 0]]), torch.ones(2, 2), 2, 2)
    assert r.sorted_expts.tolist() == [0, 0, 1, 1] and r.sorted_pairs.tolist() == [0, 3, 1, 2]
    with pytest.raises(ValueError, match="input rows"):
        ops.MoEGemm(torch.zeros(3, 8), torch.zeros(2, 4, 8), r, None, 2)
    with pytest.raises(ValueError, match="topk 5 out of range"):
        ops.MoERoute(torch.zeros(2, 4), 5, False)
    with pytest.raises(ValueError, match="multiple of 8"):
        ops.MoECombine(torch.arange(8.0).reshape(4, 2), 2)
    with pytest.raises(ValueError, match="CUDA kernels only"):
        ops.MoECombine(torch.zeros(4, 8), 2)
    with pytest.raises(ValueError, match="CUDA kernels only"):
        ops.GatherColumns(torch.zeros(4, 8), torch.arange(8))
    with pytest.raises(ValueError, match="concatInt4"):
        ops.ConcatInt4(i4, ops.Int4(i4.codes, i4.scales, i4.zeros, i4.group * 2))


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/liblight_b200.so")
    with pytest.raises(_lib.Light200Error, match="no CPU or PyTorch fallback"):
        _lib.lib()
