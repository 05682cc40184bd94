"""One quantized matmul shape, run a few times: the small case behind a kernel measurement or an `ncu` capture.

    python -m light_b200.cases --type q4_k --rows 14336 --k 4096 --tokens 32 --rotate 6 --passes 2

(--type f8: block-scaled FP8 e4m3 weights, 128 x 128 blocks, bf16 activations, through ops.MatMulF8Block)
runs light_b200_matmul_q on `rotate` copies of one weight (more than L2 holds when rows * k is large enough, so DRAM
figures mean something) `passes` times, prints the mean time per call from CUDA events and the status words.  The
library's environment knobs select the kernel under test (LIGHT_B200_TS=1: weights through tensor memory;
LIGHT_B200_NT_MAX_M=0: the kernels before the token-tile path).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json

import torch

from . import _lib, ops, synth

TYPES = {"q4_k": ops.Q4_K, "q6_k": ops.Q6_K, "q8_0": ops.Q8_0}


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--type", choices=sorted(TYPES) + ["f8"], default="q4_k")
    ap.add_argument("--rows", type=int, default=14336)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--tokens", type=int, default=1)
    ap.add_argument("--rotate", type=int, default=6)
    ap.add_argument("--passes", type=int, default=2)
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    lib = _lib.lib()
    _lib.check(lib.light_b200_init(0))
    if a.type == "f8":
        return f8_case(a, dev)
    dt, N, K, M = TYPES[a.type], a.rows, a.k, a.tokens
    ops.ensure_workspace(0, max(int(lib.light_b200_matmul_q_workspace_bytes(M, K)), 1 << 20))
    base = synth.gaussian_weight(1, dt, N, K, device=dev)
    ws = [base] + [base.clone() for _ in range(a.rotate - 1)]
    x = torch.randn(M, K, device=dev)
    out = torch.empty(M, N, device=dev)

    def once():
        for w in ws:
            _lib.check(lib.light_b200_matmul_q(dt, C.c_void_p(x.data_ptr()), C.c_void_p(w.data_ptr()), C.c_void_p(out.data_ptr()), M, N, K, 0, None))

    once()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.passes):
        once()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (a.passes * len(ws))
    nbytes = N * synth.row_bytes(dt, K)
    print(json.dumps({"type": a.type, "rows": N, "k": K, "tokens": M, "us_per_call": us, "weight_gbs": nbytes / us / 1e3,
                      "launches": int(lib.light_b200_launch_count()), "status": ops.prefill_status(0),
                      "mean_abs_out": float(out.abs().mean())}))


def f8_case(a, dev) -> None:
    N, K, M = a.rows, a.k, a.tokens
    ws = [synth.random_fp8_block(11 + i, N, K, device=dev) for i in range(a.rotate)]
    x = (torch.randn(M, K, device=dev) * 0.05).to(torch.bfloat16)
    out = None

    def once():
        nonlocal out
        for codes, scale in ws:
            out = ops.MatMulF8Block(x, codes, scale, 128, 128)

    once()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.passes):
        once()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (a.passes * len(ws))
    print(json.dumps({"type": "f8", "rows": N, "k": K, "tokens": M, "us_per_call": us, "tflops": 2.0 * M * N * K / us / 1e6,
                      "launches": int(_lib.lib().light_b200_launch_count()), "status": ops.prefill_status(0),
                      "mean_abs_out": float(out.float().abs().mean())}))


if __name__ == "__main__":
    main()
