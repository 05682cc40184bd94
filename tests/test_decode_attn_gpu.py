"""GPU parity of the decode-step attention trio (KVAppend, DecodeAttention, IncrementI64) through the C ABI:
the cases and tolerances of the reference's own test (ops/decode_attn_cuda_test.go:20-91: 1e-4 of
max(1, |x|) at f32, 3e-2 at bf16), against the CPU oracle and against the reference's kernels
(kernels/cuda/src/decode_attn.cu compiled for sm_100a under oracle/_ref)."""
import ctypes as C
import math

import numpy as np
import pytest
import torch

from helpers import RefCuda
from light_b200 import ops
from test_decode_attn_cpu import CASES

pytestmark = pytest.mark.gpu

DTYPES = {"short": torch.float32, "llama-ish": torch.bfloat16, "qwen-ish": torch.bfloat16, "hd256 g1": torch.float32,
          "window mid-block": torch.bfloat16, "window short": torch.float32, "window wider than n": torch.float32,
          "hd512": torch.bfloat16}


def _inputs(case, dt, dev, seed=80):
    _, B, NH, KH, D, cap, n, window = case
    g = torch.Generator().manual_seed(seed)
    mk = lambda *s: torch.randn(*s, generator=g).to(dt)
    return mk(B, KH, cap, D).to(dev), mk(B, KH, cap, D).to(dev), mk(B, NH, 1, D).to(dev), mk(B, KH, 1, D).to(dev), mk(B, KH, 1, D).to(dev)


def _close(got, want, tol):
    got, want = got.float().cpu().numpy().astype(np.float64), np.asarray(want, np.float64)
    return float(np.max(np.abs(got - want) / np.maximum(1, np.abs(want)))) <= tol


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_append_attend_increment(cuda, oracle, case, dt):
    name, B, NH, KH, D, cap, n, window = case
    tol = 1e-4 if dt == torch.float32 else 3e-2
    kbuf, vbuf, q, k, v = _inputs(case, dt, cuda)
    pos = torch.tensor([n - 1], dtype=torch.int64, device=cuda)
    scale = 1 / math.sqrt(D)
    kb2, vb2 = kbuf.clone(), vbuf.clone()
    ops.KVAppend(kbuf, vbuf, k, v, pos)
    assert torch.equal(kbuf[:, :, n - 1], k[:, :, 0]) and torch.equal(vbuf[:, :, n - 1], v[:, :, 0])
    out = ops.DecodeAttention(q, kbuf, vbuf, pos, scale, window)
    want = oracle.decode_attn(q.float().cpu().numpy(), kbuf.float().cpu().numpy(), vbuf.float().cpu().numpy(), n - 1, scale, window)
    assert _close(out, want, tol), name
    # append inside the attention launch: same cache, same bits out
    fused = ops.DecodeAttention(q, kb2, vb2, pos, scale, window, k_new=k, v_new=v)
    assert torch.equal(kb2, kbuf) and torch.equal(vb2, vbuf)
    assert torch.equal(fused, out)
    ops.IncrementI64(pos)
    assert int(pos.item()) == n
    assert ops.decode_attn_status(0) == 0


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_against_reference_kernels(cuda, case):
    """decode_attn_partial_* + decode_attn_combine_* launched as kernels/cuda/decode_attn.go:76-121 does."""
    if not RefCuda.available("decode_attn"):
        pytest.skip("oracle/_ref/decode_attn.cubin not built")
    name, B, NH, KH, D, cap, n, window = case
    dt = DTYPES[name]
    tol = 1e-4 if dt == torch.float32 else 3e-2
    kbuf, vbuf, q, k, v = _inputs(case, dt, cuda, seed=81)
    pos = torch.tensor([n - 1], dtype=torch.int64, device=cuda)
    scale = 1 / math.sqrt(D)
    ref = RefCuda()
    sfx = "f32" if dt == torch.float32 else "bf16"
    P = lambda t: C.c_void_p(t.data_ptr())
    nel = B * KH * D
    ref.launch("decode_attn", "kv_append_" + sfx, [(nel + 255) // 256], [256],
               [P(k), P(v), P(kbuf), P(vbuf), P(pos), C.c_int(B), C.c_int(KH), C.c_int(D), C.c_int(cap)])
    g, splits = NH // KH, (cap + 31) // 32
    part = torch.zeros(B * NH * splits * (D + 2), device=cuda)
    want = torch.empty(B, NH, 1, D, dtype=dt, device=cuda)
    ref.launch("decode_attn", "decode_attn_partial_" + sfx, [B * KH, splits], [128],
               [P(q), P(kbuf), P(vbuf), P(part), P(pos), C.c_int(NH), C.c_int(KH), C.c_int(cap), C.c_int(D), C.c_float(scale), C.c_int(window)],
               shmem=(g * (D + 1) + g * 32) * 4)
    ref.launch("decode_attn", "decode_attn_combine_" + sfx, [B * NH], [min(max(D, 32), 1024)],
               [P(part), P(want), P(pos), C.c_int(splits), C.c_int(D), C.c_int(window)])
    torch.cuda.synchronize()
    got = ops.DecodeAttention(q, kbuf, vbuf, pos, scale, window)
    assert _close(got, want.float().cpu().numpy(), tol), name


def test_one_graph_serves_every_position(cuda, oracle):
    """models/decode_graph.go:27-230: the step is captured once and replayed while the device-side position
    advances; here append + attend + increment, Llama-3-8B head shapes."""
    B, NH, KH, D, cap = 2, 32, 8, 128, 96
    g = torch.Generator().manual_seed(82)
    kbuf, vbuf = torch.zeros(B, KH, cap, D, device=cuda), torch.zeros(B, KH, cap, D, device=cuda)
    ks, vs, qs = torch.randn(5, B, KH, 1, D, generator=g), torch.randn(5, B, KH, 1, D, generator=g), torch.randn(5, B, NH, 1, D, generator=g)
    k, v, q = ks[0].to(cuda), vs[0].to(cuda), qs[0].to(cuda)
    pos = torch.zeros(1, dtype=torch.int64, device=cuda)
    scale = 1 / math.sqrt(D)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        out = ops.DecodeAttention(q, kbuf, vbuf, pos, scale, 0, k_new=k, v_new=v)  # warm-up outside capture
        pos.zero_()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            out = ops.DecodeAttention(q, kbuf, vbuf, pos, scale, 0, k_new=k, v_new=v)
            ops.IncrementI64(pos)
    kb, vb = np.zeros((B, KH, cap, D), np.float32), np.zeros((B, KH, cap, D), np.float32)
    for t in range(5):
        k.copy_(ks[t]), v.copy_(vs[t]), q.copy_(qs[t])
        graph.replay()
        torch.cuda.synchronize()
        oracle.kv_append(kb, vb, ks[t].numpy(), vs[t].numpy(), t)
        want = oracle.decode_attn(qs[t].numpy(), kb, vb, t, scale, 0)
        assert _close(out, want, 1e-4), t
        assert int(pos.item()) == t + 1
    assert np.array_equal(kbuf.cpu().numpy(), kb)


def test_limits_are_reported_not_asserted(cuda):
    """kernels/cuda/decode_attn.go:36-38,85-87: head dims that are no multiple of 32 and groups above 16 are
    refused (the caller composes the op); a position outside the cache is clamped and recorded."""
    from light_b200 import _lib

    q = torch.zeros(1, 34, 1, 48, device=cuda)
    kbuf = torch.zeros(1, 2, 16, 48, device=cuda)
    pos = torch.zeros(1, dtype=torch.int64, device=cuda)
    with pytest.raises(_lib.Light200Error):
        ops.DecodeAttention(q, kbuf, kbuf.clone(), pos, 1.0)
    q = torch.zeros(1, 34, 1, 64, device=cuda)
    kbuf = torch.zeros(1, 2, 16, 64, device=cuda)
    with pytest.raises(_lib.Light200Error):
        ops.DecodeAttention(q, kbuf, kbuf.clone(), pos, 1.0)
    with pytest.raises(ValueError):
        ops.DecodeAttention(q, kbuf, kbuf.clone(), pos.to(torch.int32), 1.0)
