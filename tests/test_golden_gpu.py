"""The CUDA path against the frozen vectors of tests/golden/vectors.npz, through the C ABI and without the
oracle at run time: dequantized weights bit for bit, f32 products within 1e-3 relative L2 of the stored f64
products."""
import os

import numpy as np
import pytest
import torch

from helpers import rel_l2
from light_b200 import ops

pytestmark = pytest.mark.gpu

G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "vectors.npz"))
GGUF = {"q4_0": ops.Q4_0, "q5_0": ops.Q5_0, "q8_0": ops.Q8_0, "q4_k": ops.Q4_K, "q5_k": ops.Q5_K, "q6_k": ops.Q6_K}
TOL = 1e-3


@pytest.mark.parametrize("name", list(GGUF))
def test_gguf(cuda, name):
    raw, want = G[f"{name}.raw"], G[f"{name}.dequant_bits"]
    w = ops.QTensor(torch.from_numpy(raw.reshape(-1).copy()).to(cuda), GGUF[name], want.shape)
    got = ops.Dequantize(w).cpu().numpy().view(np.uint32)
    assert np.array_equal(got, want)
    x = torch.from_numpy(G["x"].copy()).to(cuda)
    for m in (1, 3):
        y = ops.MatMulQ(x[:m].contiguous(), w).cpu().numpy()
        assert rel_l2(y, G[f"{name}.y64"][:m]) <= TOL


def test_int4(cuda):
    w = ops.Int4(torch.from_numpy(G["int4.codes"].view(np.int32).copy()).to(cuda), torch.from_numpy(G["int4.scales"].copy()).to(cuda),
                 torch.from_numpy(G["int4.zeros"].copy()).to(cuda), 128)
    assert np.array_equal(ops.DequantizeInt4(w, torch.float32).cpu().numpy().view(np.uint32), G["int4.dequant_bits"])
    assert np.array_equal(ops.DequantizeInt4(w, torch.bfloat16).view(torch.int16).cpu().numpy().view(np.uint16), G["int4.dequant_bf16"])
    x = torch.from_numpy(G["int4.x"].copy()).to(cuda)
    assert rel_l2(ops.MatMulInt4(x, w).cpu().numpy(), G["int4.y64"]) <= TOL


def test_fp8(cuda):
    codes, s = torch.from_numpy(G["fp8.codes"].copy()).to(cuda), torch.from_numpy(G["fp8.scale"].copy()).to(cuda)
    assert np.array_equal(ops.DequantizeF8Block(codes, s, 128, 128, torch.float32).cpu().numpy().view(np.uint32), G["fp8.dequant_bits"])
    got = ops.DequantizeF8Block(codes, s, 128, 128, torch.bfloat16).view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got, G["fp8.dequant_bf16"])
