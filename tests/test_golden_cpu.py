"""The CPU oracle against the frozen vectors of tests/golden/vectors.npz (made by tests/golden/make_golden.py):
same bits for every dequantized weight, the checkpoint-layout converters land on the canonical int4 layout
(quant/int4.go:103-235), the expert sort matches (ops/moe.go:37-70)."""
import os

import numpy as np
import pytest

from light_b200 import ops

G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "vectors.npz"))
GGUF = {"q4_0": ops.Q4_0, "q5_0": ops.Q5_0, "q8_0": ops.Q8_0, "q4_k": ops.Q4_K, "q5_k": ops.Q5_K, "q6_k": ops.Q6_K}


@pytest.mark.parametrize("name", list(GGUF))
def test_gguf_dequant_bits(oracle, name):
    raw = G[f"{name}.raw"]
    want = G[f"{name}.dequant_bits"]
    got = oracle.dequant(GGUF[name], raw.reshape(-1), want.size).view(np.uint32).reshape(want.shape)
    assert np.array_equal(got, want)
    y = oracle.matmul_q(GGUF[name], G["x"], raw.reshape(-1), want.shape[0])
    assert np.linalg.norm(y - G[f"{name}.y64"]) <= 1e-5 * np.linalg.norm(G[f"{name}.y64"])


def test_int4_bits_and_converters(oracle):
    codes, s, z = G["int4.codes"], G["int4.scales"], G["int4.zeros"]
    assert np.array_equal(oracle.int4_dequant(codes, s, z, 128).view(np.uint32), G["int4.dequant_bits"])
    assert np.array_equal(oracle.int4_dequant(codes, s, z, 128, bf16=True), G["int4.dequant_bf16"])
    for conv, key in ((lambda a, b, c: oracle.int4_from_gptq(a, b, c, 128), "gptq"), (lambda a, b, c: oracle.int4_from_awq(a, b, c, 128), "awq")):
        c2, s2, z2 = conv(G[f"int4.{key}_qweight"], G[f"int4.{key}_qzeros"], G[f"int4.{key}_scales"])
        assert np.array_equal(c2, codes) and np.array_equal(s2, s) and np.array_equal(z2, z), key


def test_fp8_bits(oracle):
    codes, s = G["fp8.codes"], G["fp8.scale"]
    assert np.array_equal(oracle.fp8_block_dequant(codes, s, 128, 128).view(np.uint32), G["fp8.dequant_bits"])
    assert np.array_equal(oracle.fp8_block_dequant(codes, s, 128, 128, bf16=True), G["fp8.dequant_bf16"])
    assert np.array_equal(oracle.e4m3_table().view(np.uint32), G["fp8.e4m3_table_bits"])


def test_moe_sort(oracle):
    pairs, expts = oracle.moe_sort_pairs(G["moe.ids"], 4)
    assert np.array_equal(pairs, G["moe.sorted_pairs"]) and np.array_equal(expts, G["moe.sorted_expts"])
    assert list(expts) == sorted(G["moe.ids"].tolist())
