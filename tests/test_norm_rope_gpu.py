"""GPU parity of RMSNorm (with the residual add folded in), RoPE, and the rotation inside the decode
attention launch, through the C ABI: against the CPU oracle, and against the reference's own kernels
(rmsnorm_f32, rope_f32 of kernels/cuda/src/elementwise.cu compiled for sm_100a under oracle/_ref)."""
import ctypes as C
import math

import numpy as np
import pytest
import torch

from helpers import RefCuda
from light_b200 import ops

pytestmark = pytest.mark.gpu


def _err(got, want):
    got, want = got.float().cpu().numpy().astype(np.float64), np.asarray(want, np.float64)
    return float(np.max(np.abs(got - want) / np.maximum(1, np.abs(want))))


@pytest.mark.parametrize("rows,cols", [(1, 4096), (8, 4096), (3, 14336), (5, 100), (64, 3584)])
def test_rmsnorm(cuda, oracle, rows, cols):
    g = torch.Generator().manual_seed(100 + rows)
    x, r, w = torch.randn(rows, cols, generator=g) * 2, torch.randn(rows, cols, generator=g), torch.randn(cols, generator=g)
    got = ops.RMSNorm(x.to(cuda), w.to(cuda), 1e-5)
    assert _err(got, oracle.rmsnorm(x.numpy(), w.numpy(), 1e-5)) <= 1e-5  # ops/norm_test.go's bound
    y, s = ops.RMSNorm(x.to(cuda), w.to(cuda), 1e-5, residual=r.to(cuda))
    assert torch.equal(s.cpu(), x + r)
    assert _err(y, oracle.rmsnorm((x + r).numpy(), w.numpy(), 1e-5)) <= 1e-5
    # bf16: statistics and product in f32, one rounding (kernels/cpu/norm.go:53-95)
    xb, wb = x.to(torch.bfloat16), w.to(torch.bfloat16)
    gotb = ops.RMSNorm(xb.to(cuda), wb.to(cuda), 1e-5)
    assert gotb.dtype == torch.bfloat16
    assert _err(gotb, oracle.rmsnorm(xb.float().numpy(), wb.float().numpy(), 1e-5)) <= 1e-2
    if RefCuda.available("elementwise"):
        ref = RefCuda()
        xd, wd = x.to(cuda), w.to(cuda)
        want = torch.empty_like(xd)
        ref.launch("elementwise", "rmsnorm_f32", [rows], [256],
                   [C.c_void_p(xd.data_ptr()), C.c_void_p(wd.data_ptr()), C.c_void_p(want.data_ptr()), C.c_ulong(rows), C.c_ulong(cols), C.c_float(1e-5)],
                   shmem=256 * 4)
        torch.cuda.synchronize()
        assert _err(got, want.cpu().numpy()) <= 1e-5


@pytest.mark.parametrize("shape,base", [((1, 32, 1, 128), 500000.0), ((2, 8, 5, 64), 10000.0), ((3, 7, 256), 10000.0)])
def test_rope(cuda, oracle, shape, base):
    g = torch.Generator().manual_seed(110)
    x = torch.randn(*shape, generator=g)
    pos = torch.randint(0, 8192, (shape[-2],), generator=g, dtype=torch.int64)
    got = ops.RoPE(x.to(cuda), pos.to(cuda), base)
    want = oracle.rope(x.numpy(), pos.numpy(), base)
    assert _err(got, want) <= 1e-5  # ops/rope_test.go:62 (CUDA against CPU)
    gotb = ops.RoPE(x.to(torch.bfloat16).to(cuda), pos.to(cuda), base)
    assert _err(gotb, oracle.rope(x.to(torch.bfloat16).float().numpy(), pos.numpy(), base)) <= 3e-2
    if RefCuda.available("elementwise"):  # the reference's kernel takes f32 angles and fast-math sine / cosine: small positions only
        small = torch.randint(0, 16, (shape[-2],), generator=g, dtype=torch.int64).to(cuda)
        xd = x.to(cuda)
        want2 = torch.empty_like(xd)
        rows, hd = x.numel() // shape[-1], shape[-1]
        RefCuda().launch("elementwise", "rope_f32", [(rows * hd // 2 + 255) // 256], [256],
                         [C.c_void_p(xd.data_ptr()), C.c_void_p(small.data_ptr()), C.c_void_p(want2.data_ptr()), C.c_ulong(rows), C.c_ulong(shape[-2]),
                          C.c_ulong(hd), C.c_float(base)])
        torch.cuda.synchronize()
        assert _err(ops.RoPE(xd, small, base), want2.cpu().numpy()) <= 1e-4


@pytest.mark.parametrize("dt,tol", [(torch.float32, 1e-4), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("B,NH,KH,D,cap,n", [(1, 32, 8, 128, 1100, 1024), (2, 8, 2, 64, 64, 9), (1, 4, 4, 256, 300, 300)])
def test_rotation_inside_the_attention_launch(cuda, oracle, dt, tol, B, NH, KH, D, cap, n):
    """RoPE(q), RoPE(k), append, attend as one launch against the four operators of the oracle."""
    g = torch.Generator().manual_seed(120)
    mk = lambda *s: torch.randn(*s, generator=g).to(dt)
    kbuf, vbuf, q, k, v = mk(B, KH, cap, D), mk(B, KH, cap, D), mk(B, NH, 1, D), mk(B, KH, 1, D), mk(B, KH, 1, D)
    base, scale = 500000.0, 1 / math.sqrt(D)
    pos = torch.tensor([n - 1], dtype=torch.int64)
    kd, vd = kbuf.to(cuda), vbuf.to(cuda)
    out = ops.DecodeAttention(q.to(cuda), kd, vd, pos.to(cuda), scale, 0, k_new=k.to(cuda), v_new=v.to(cuda), rope_base=base)
    qr = oracle.rope(q.float().numpy(), pos.numpy(), base)
    kr = oracle.rope(k.float().numpy(), pos.numpy(), base)
    kb, vb = kbuf.float().numpy().copy(), vbuf.float().numpy().copy()
    oracle.kv_append(kb, vb, kr, v.float().numpy(), n - 1)
    want = oracle.decode_attn(qr, kb, vb, n - 1, scale, 0)
    assert _err(out, want) <= tol
    assert _err(kd[:, :, n - 1], kr[:, :, 0]) <= (1e-6 if dt == torch.float32 else 1e-2)  # the key is cached rotated
    assert torch.equal(vd[:, :, n - 1].cpu(), v[:, :, 0])
    assert ops.decode_attn_status(0) == 0


@pytest.mark.parametrize("rows,cols", [(1, 128256), (5, 1000), (64, 33), (2, 1)])
def test_argmax(cuda, rows, cols):
    """ops.Argmax over the last axis: the lowest index among equal maxima."""
    g = torch.Generator().manual_seed(130)
    x = torch.randn(rows, cols, generator=g)
    if cols > 40:
        x[0, 37] = x[0, 5] = 9.0  # a tie: index 5
    got = ops.Argmax(x.to(cuda)).cpu()
    want = torch.tensor([int(np.flatnonzero(r == r.max())[0]) for r in x.numpy()])
    assert torch.equal(got, want)
