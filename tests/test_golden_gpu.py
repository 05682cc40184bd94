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


@pytest.mark.parametrize("layout", ["gptq", "awq"])
def test_int4_checkpoint_layouts_on_the_device(cuda, layout):
    """quant.FromGPTQ / quant.FromAWQ (quant/int4.go:103-261) as device kernels land on the stored canonical layout."""
    t = lambda k: torch.from_numpy(G[k].view(np.int32).copy() if G[k].dtype == np.uint32 else G[k].copy()).to(cuda)
    w = ops.Int4FromCheckpoint(t(f"int4.{layout}_qweight"), t(f"int4.{layout}_qzeros"), t(f"int4.{layout}_scales"), 128, layout)
    assert np.array_equal(w.codes.cpu().numpy().view(np.uint32), G["int4.codes"])
    assert np.array_equal(w.scales.cpu().numpy(), G["int4.scales"]) and np.array_equal(w.zeros.cpu().numpy(), G["int4.zeros"])
    assert np.array_equal(ops.DequantizeInt4(w, torch.float32).cpu().numpy().view(np.uint32), G["int4.dequant_bits"])


@pytest.mark.parametrize("name", list(GGUF))
def test_quantized_embedding_rows(cuda, name):
    """nn/embedding_test.go:127: the gathered rows equal the dequantized table's rows, bit for bit; ids repeat,
    come in any shape, and one outside the table gives zeros."""
    raw, want = G[f"{name}.raw"], G[f"{name}.dequant_bits"]
    table = ops.QTensor(torch.from_numpy(raw.reshape(-1).copy()).to(cuda), GGUF[name], want.shape)
    ids = torch.tensor([[4, 0, 2], [2, 4, 1]], dtype=torch.int64, device=cuda)
    got = ops.EmbeddingQ(table, ids).cpu().numpy().view(np.uint32)
    assert got.shape == (2, 3, want.shape[1])
    assert np.array_equal(got, want[ids.cpu().numpy()])
    out = ops.EmbeddingQ(table, torch.tensor([want.shape[0], -1, 3], dtype=torch.int64, device=cuda)).cpu().numpy()
    assert not out[:2].any() and np.array_equal(out[2].view(np.uint32), want[3])
