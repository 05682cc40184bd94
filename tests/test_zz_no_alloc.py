"""The grouped expert matmul that brings its own scratch (light_b200_moe_gemm_static_scratch).

Collected last on purpose: a run that stops at the first failure has then already run every other
test.  It must pass alone in a fresh process and after the rest of the suite, so it builds
everything it needs itself and assumes nothing about the state the library's scratch is in.
"""
import ctypes as C

import pytest
import torch

from light_b200 import _lib

pytestmark = pytest.mark.gpu


def _case(seed, T, E, topk, N, K, dev):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, E, (T * topk,), generator=g)
    expts, pairs = torch.sort(ids, stable=True)
    x = torch.randn(T, K, generator=g)
    w = torch.randn(E, N, K, generator=g) * 0.1
    tw = torch.rand(T * topk, generator=g)
    return [t.to(dev) for t in (x, w, pairs, expts, tw)]


def _run(fn, x, w, pairs, expts, tw, topk, own_scratch):
    E, N, K = w.shape
    M = pairs.numel()
    out = torch.zeros(M, N, device=x.device)
    counts = torch.zeros(E, dtype=torch.int32, device=x.device) if own_scratch else None
    offsets = torch.zeros(E + 1, dtype=torch.int32, device=x.device) if own_scratch else None
    a = _lib.MoeArgs(input=x.data_ptr(), weights=w.data_ptr(), sorted_pairs=pairs.data_ptr(),
                     expert_ids=expts.data_ptr(), counts=counts.data_ptr() if own_scratch else 0,
                     offsets=offsets.data_ptr() if own_scratch else 0, topk_weights=tw.data_ptr(), out=out.data_ptr(),
                     M=M, size_m=M, E=E, N=N, K=K, topk=topk, row_per_pair=0, dtype=_lib.F32)
    _lib.check(fn(C.byref(a), 0, C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    return out


def test_static_scratch_matches_caller_scratch_twice_in_a_row():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    dev = torch.device("cuda:0")
    l = _lib.lib()
    _lib.check(l.light_b200_init(0))
    # Two different routings back to back: the second has fewer experts and fewer pairs, so any
    # count or offset left over from the first call would show up as wrong rows.
    for seed, T, E, topk, N, K in ((201, 40, 24, 2, 48, 64), (202, 9, 5, 3, 16, 32)):
        case = _case(seed, T, E, topk, N, K, dev)
        want = _run(l.light_b200_moe_gemm, *case, topk, own_scratch=True)
        got = _run(l.light_b200_moe_gemm_static_scratch, *case, topk, own_scratch=False)
        # same kernels, same order of operations: the tolerance of the other f32 MoE tests (1e-4)
        err = ((got - want).abs() / (1 + want.abs())).max().item()
        assert err <= 1e-4, (seed, err)
        ref = torch.stack([(case[1][case[3][i]] @ case[0][case[2][i] // topk]) * case[4][case[2][i]]
                           for i in range(case[2].numel())])
        assert torch.allclose(got[case[2]], ref, atol=1e-3)


def test_static_scratch_rejects_too_many_experts():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    l = _lib.lib()
    one = 256  # never dereferenced: the size check comes first
    a = _lib.MoeArgs(input=one, weights=one, sorted_pairs=one, expert_ids=one, counts=0, offsets=0, topk_weights=0,
                     out=one, M=1, size_m=1, E=1025, N=8, K=8, topk=1, row_per_pair=1, dtype=_lib.F32)
    assert l.light_b200_moe_gemm_static_scratch(C.byref(a), 0, None) == -6
    assert "exceed the built-in scratch (max 1024)" in _lib.last_error()
