"""The bf16 decode GEMVs (registry keys gemv_multi / gemv_gated) against an f64 reference with the reference's
roundings, with the bound of its own CUDA test (ops/gemv_cuda_test.go:37-79: |got - want| <= 3e-2 * max(0.05, |want|))."""
import numpy as np
import pytest
import torch

from light_b200 import ops

pytestmark = pytest.mark.gpu


def _check(got, want, tol=3e-2):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert np.all(np.abs(got - want) <= tol * np.maximum(0.05, np.abs(want)))


@pytest.mark.parametrize("K", [64, 896, 4096, 12288])
def test_linear_multi(cuda, K):
    g = torch.Generator().manual_seed(K)
    x = torch.randn(K, generator=g).to(torch.bfloat16)
    ws = [(torch.randn(n, K, generator=g) * 0.05).to(torch.bfloat16) for n in (33, 7, 128, 1)]
    for out_dtype in (torch.bfloat16, torch.float32):
        outs = ops.LinearMulti(x.to(cuda), [w.to(cuda) for w in ws], out_dtype)
        for o, w in zip(outs, ws):
            want = w.double() @ x.double()
            assert o.dtype == out_dtype and o.shape == (w.shape[0],)
            _check(o.float().cpu().numpy(), want.numpy(), 3e-2 if out_dtype == torch.bfloat16 else 1e-4)
    one = ops.LinearMulti(x.to(cuda), [ws[0].to(cuda)])
    _check(one[0].float().cpu().numpy(), (ws[0].double() @ x.double()).numpy())


@pytest.mark.parametrize("gelu", [False, True])
def test_gated_linear(cuda, gelu):
    K, N = 1024, 300
    g = torch.Generator().manual_seed(5)
    x = torch.randn(K, generator=g).to(torch.bfloat16)
    wg = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
    wu = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
    got = ops.GatedLinear(x.to(cuda), wg.to(cuda), wu.to(cuda), gelu)
    gb = (wg.double() @ x.double()).to(torch.bfloat16).double()
    ub = (wu.double() @ x.double()).to(torch.bfloat16).double()
    a = (0.5 * gb * (1 + torch.erf(gb / 2 ** 0.5))) if gelu else gb / (1 + torch.exp(-gb))
    want = (a.to(torch.bfloat16).double() * ub)
    _check(got.float().cpu().numpy(), want.numpy())


def test_rejects(cuda):
    x = torch.zeros(12, dtype=torch.bfloat16, device=cuda)
    w = torch.zeros(4, 12, dtype=torch.bfloat16, device=cuda)
    with pytest.raises(ValueError):
        ops.LinearMulti(x, [w])          # K % 8 != 0
    with pytest.raises(ValueError):
        ops.LinearMulti(x.float(), [w])
