"""Writes tests/golden/vectors.npz: small seeded inputs of every weight format of the quantized-matmul path with
the outputs of the CPU oracle (oracle/light_oracle.c), which tests/test_oracle_kat.py pins to the reference's own
known-answer tests.  The reference is Go and cannot run where this was made, so the vectors come from the
pinned oracle, not from the reference binary; what they add is a frozen copy: the oracle cannot drift
unnoticed (tests/test_golden_cpu.py), and the CUDA path is compared with bytes on disk
(tests/test_golden_gpu.py).

    python tests/golden/make_golden.py        # rewrites vectors.npz; the result must be byte-stable

Inputs follow the reference's test construction (ops/matmul_q_test.go:19-56: random bytes, f16 scale
fields forced into [2^-6, 2^-5); ops/int4_test.go:20-60; ops/fp8_block_test.go:106-120)."""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from light_b200 import ops, synth  # noqa: E402
from oracle import binding as oracle  # noqa: E402

GGUF = {"q4_0": ops.Q4_0, "q5_0": ops.Q5_0, "q8_0": ops.Q8_0, "q4_k": ops.Q4_K, "q5_k": ops.Q5_K, "q6_k": ops.Q6_K}
N, K, M = 5, 512, 3


def build() -> dict:
    out = {}
    rng = np.random.Generator(np.random.Philox(1001))
    x = rng.standard_normal((M, K)).astype(np.float32)
    out["x"] = x
    for i, (name, dt) in enumerate(GGUF.items()):
        raw = synth.random_blocks(1100 + i, dt, N, K)
        deq = oracle.dequant(dt, raw.reshape(-1), N * K).reshape(N, K)
        out[f"{name}.raw"] = raw
        out[f"{name}.dequant_bits"] = deq.view(np.uint32)
        out[f"{name}.y64"] = x.astype(np.float64) @ deq.astype(np.float64).T
    # int4, canonical layout + the two checkpoint layouts it is converted from
    Ni, Ki, G = 16, 256, 128
    codes, s, z = synth.random_int4(1200, Ni, Ki, G)
    z[z == 0] = 1.0  # GPTQ v1 stores zero - 1 in four bits
    out["int4.codes"], out["int4.scales"], out["int4.zeros"] = codes, s, z
    out["int4.dequant_bits"] = oracle.int4_dequant(codes, s, z, G).view(np.uint32)
    out["int4.dequant_bf16"] = oracle.int4_dequant(codes, s, z, G, bf16=True)
    qw, qz, sc = synth.to_gptq(codes, s, z)
    out["int4.gptq_qweight"], out["int4.gptq_qzeros"], out["int4.gptq_scales"] = qw, qz, sc
    qw, qz, sc = synth.to_awq(codes, s, z)
    out["int4.awq_qweight"], out["int4.awq_qzeros"], out["int4.awq_scales"] = qw, qz, sc
    xi = rng.standard_normal((M, Ki)).astype(np.float32)
    out["int4.x"] = xi
    out["int4.y64"] = xi.astype(np.float64) @ oracle.int4_dequant(codes, s, z, G).astype(np.float64).T
    # block-scaled FP8: every code that is not NaN, 128 x 128 blocks
    Nf, Kf, b = 128, 256, 128
    fcodes = rng.permutation(np.tile(np.array([c for c in range(256) if (c & 0x7F) != 0x7F], np.uint8), Nf * Kf // 254 + 1))[:Nf * Kf].reshape(Nf, Kf)
    fs = rng.uniform(1e-4, 2.1e-3, size=(Nf // b, Kf // b)).astype(np.float32)
    out["fp8.codes"], out["fp8.scale"] = fcodes, fs
    out["fp8.dequant_bits"] = oracle.fp8_block_dequant(fcodes, fs, b, b).view(np.uint32)
    out["fp8.dequant_bf16"] = oracle.fp8_block_dequant(fcodes, fs, b, b, bf16=True)
    out["fp8.e4m3_table_bits"] = oracle.e4m3_table().view(np.uint32)
    # grouped matmul: the fixed expert ids of ops/int4_test.go's MoE case, sorted into expert order
    ids = np.array([0, 2, 2, 1, 3, 0, 2, 3, 1, 2], np.int64)
    pairs, expts = oracle.moe_sort_pairs(ids, 4)
    out["moe.ids"], out["moe.sorted_pairs"], out["moe.sorted_expts"] = ids, np.asarray(pairs), np.asarray(expts)
    return out


if __name__ == "__main__":
    path = os.path.join(HERE, "vectors.npz")
    np.savez_compressed(path, **build())
    print(path, os.path.getsize(path), "bytes")
