"""GPU parity of ops.MatMulW8A8 through the C ABI: the reference's own cases (ops/matmul_w8a8_test.go:22-88) plus
ragged edges; the int8 rows, their scales and the f32 outputs equal the oracle's bit for bit (the contraction is
exact in int32 and every f32 step is one correctly rounded operation)."""
import ctypes as C

import numpy as np
import pytest
import torch

from light_b200 import _lib, ops
from test_w8a8_cpu import CASES, make

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,K,N", CASES + [(129, 80, 131), (300, 4096, 260), (5, 16, 16)])
def test_w8a8_bit_exact(cuda, oracle, M, K, N):
    x, wq, ws = make(M, K, N, seed=140)
    x[0, :3] = [0.5, 1.5, 2.5]
    want, _ = oracle.matmul_w8a8(x, wq, ws)
    xd = torch.from_numpy(x).to(cuda)
    got = ops.MatMulW8A8(xd, torch.from_numpy(wq).to(cuda), torch.from_numpy(ws).to(cuda)).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    q = torch.empty(M, K, dtype=torch.int8, device=cuda)
    s = torch.empty(M, device=cuda)
    _lib.check(_lib.lib().light_b200_quantize_rows_int8(C.c_void_p(xd.data_ptr()), C.c_void_p(q.data_ptr()), C.c_void_p(s.data_ptr()), M, K, 0, None))
    wq8, ws8 = oracle.quantize_rows_int8(x)
    assert np.array_equal(q.cpu().numpy(), wq8) and np.array_equal(s.cpu().numpy(), ws8)


def test_w8a8_arguments(cuda):
    x = torch.zeros(2, 24, device=cuda)
    with pytest.raises(_lib.Light200Error):  # K must be a multiple of 16
        ops.MatMulW8A8(x, torch.zeros(8, 24, dtype=torch.int8, device=cuda), torch.ones(8, device=cuda))
    with pytest.raises(ValueError):
        ops.MatMulW8A8(x, torch.zeros(8, 32, dtype=torch.int8, device=cuda), torch.ones(8, device=cuda))
