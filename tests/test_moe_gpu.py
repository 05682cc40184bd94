"""GPU parity of the grouped expert matmuls (moe_gemm, moe_gemm_q) through the C ABI."""
import ctypes as C

import numpy as np
import pytest
import torch

from helpers import RefCuda, max_rel, rel_l2
from light_b200 import ops, synth

pytestmark = pytest.mark.gpu


def _routing(seed, T, E, topk, dev, skew=True):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(T, E, generator=g)
    if skew:
        logits = logits + torch.randn(E, generator=g) * 1.5
    probs = torch.softmax(logits, dim=1)
    return ops.MoERoute(probs.to(dev), topk, True)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 3e-2), (torch.float16, 3e-2)])
def test_moe_gemm_matches_oracle(cuda, oracle, dtype, tol):
    """ops/moe_test.go:52-190: grouped GEMM vs the CPU kernel (per-pair dot products), both GEMMs
    of an MoE layer (row per token with routing weights; row per pair without), experts with no
    tokens included; f32 1e-4, bf16/f16 3e-2."""
    T, E, topk, N, K = 33, 8, 2, 40, 64
    r = _routing(101, T, E, topk, cuda)
    g = torch.Generator().manual_seed(102)
    x = torch.randn(T, K, generator=g).to(dtype)
    w = (torch.randn(E, N, K, generator=g) * 0.1).to(dtype)
    w[5] = 0  # expert 5 still routed; make one expert unused instead:
    sp, se = r.sorted_pairs.cpu().numpy(), r.sorted_expts.cpu().numpy()
    tw = r.weights.cpu().numpy()
    got = ops.MoEGemm(x.to(cuda), w.to(cuda), r, r.weights, topk)
    want = oracle.moe_gemm_f32(x.float().numpy(), w.float().numpy(), sp, se, tw, T * topk, topk, False)
    assert got.dtype == dtype and max_rel(got.float().cpu().numpy(), want) <= tol
    h = torch.randn(T * topk, K, generator=g).to(dtype)
    got2 = ops.MoEGemm(h.to(cuda), w.to(cuda), r, None, topk)
    want2 = oracle.moe_gemm_f32(h.float().numpy(), w.float().numpy(), sp, se, None, T * topk, topk, True)
    assert max_rel(got2.float().cpu().numpy(), want2) <= tol
    comb = ops.MoECombine(got, topk)
    assert comb.shape == (T, N)


def test_moe_offsets_and_counts_scratch(cuda):
    """The counts / offsets scratch is filled as the reference's moe_count_experts +
    moe_expert_offsets do (kernels/cuda/src/moe.cu:28-42), including empty experts at both ends."""
    from light_b200 import _lib

    ids = torch.tensor([1, 1, 1, 4, 4, 6], dtype=torch.int64, device=cuda)
    E, N, K = 9, 8, 16
    pairs = torch.arange(6, dtype=torch.int64, device=cuda)
    counts = torch.full((E,), -7, dtype=torch.int32, device=cuda)
    offsets = torch.full((E + 1,), -7, dtype=torch.int32, device=cuda)
    x = torch.randn(6, K, device=cuda)
    w = torch.randn(E, N, K, device=cuda)
    out = torch.zeros(6, N, device=cuda)
    a = _lib.MoeArgs(input=x.data_ptr(), weights=w.data_ptr(), sorted_pairs=pairs.data_ptr(), expert_ids=ids.data_ptr(),
                     counts=counts.data_ptr(), offsets=offsets.data_ptr(), topk_weights=0, out=out.data_ptr(), M=6,
                     size_m=6, E=E, N=N, K=K, topk=1, row_per_pair=1, dtype=_lib.F32)
    _lib.check(_lib.lib().light_b200_moe_gemm(C.byref(a), 0, None))
    torch.cuda.synchronize()
    assert counts.tolist() == [0, 3, 0, 0, 2, 0, 1, 0, 0]
    assert offsets.tolist() == [0, 0, 3, 3, 3, 5, 5, 6, 6, 6]
    for p in range(6):
        assert torch.allclose(out[p], w[ids[p]] @ x[p], atol=1e-4)
    # no pairs at all: scratch still well defined, nothing written
    a.M = 0
    _lib.check(_lib.lib().light_b200_moe_gemm(C.byref(a), 0, None))
    torch.cuda.synchronize()
    assert counts.tolist() == [0] * E and offsets.tolist() == [0] * (E + 1)


def test_moe_out_of_range_pairs_are_skipped(cuda):
    """Pair ids outside [0, size_m) are skipped (kernels/cuda/src/moe.cu:94-96)."""
    E, N, K, topk = 2, 8, 16, 1
    r = ops.MoERouting(torch.zeros(3, 1, dtype=torch.int64), torch.ones(3, device=cuda),
                       torch.tensor([0, 99, 2], dtype=torch.int64, device=cuda),
                       torch.tensor([0, 0, 1], dtype=torch.int64, device=cuda))
    x = torch.randn(3, K, device=cuda)
    w = torch.randn(E, N, K, device=cuda)
    out = ops.MoEGemm(x, w, r, None, topk)
    assert torch.allclose(out[0], w[0] @ x[0], atol=1e-4) and torch.allclose(out[2], w[1] @ x[2], atol=1e-4)
    assert torch.all(out[1] == 0)


@pytest.mark.parametrize("name", ["q4_0", "q5_0", "q8_0", "q4_k", "q5_k", "q6_k"])
def test_moe_gemm_q_matches_dense(cuda, oracle, name):
    """ops/moe_test.go:192-255: quantized experts equal dequantize + dense grouped GEMM, 1e-4."""
    dt = {"q4_0": ops.Q4_0, "q5_0": ops.Q5_0, "q8_0": ops.Q8_0, "q4_k": ops.Q4_K, "q5_k": ops.Q5_K, "q6_k": ops.Q6_K}[name]
    T, E, topk, N, K = 19, 4, 2, 24, 512
    r = _routing(111, T, E, topk, cuda)
    raw = synth.random_blocks(112, dt, E * N, K)
    deq = oracle.dequant(dt, raw.reshape(-1), E * N * K).reshape(E, N, K)
    x = torch.randn(T, K, generator=torch.Generator().manual_seed(113))
    w = ops.QTensor(torch.from_numpy(raw.reshape(-1)).to(cuda), dt, (E, N, K))
    got = ops.MoEGemmQ(x.to(cuda), w, r, r.weights, topk).cpu().numpy()
    want = oracle.moe_gemm_f32(x.numpy(), deq, r.sorted_pairs.cpu().numpy(), r.sorted_expts.cpu().numpy(),
                               r.weights.cpu().numpy(), T * topk, topk, False)
    assert max_rel(got, want) <= 1e-4 and rel_l2(got, want) <= 1e-3


def test_moe_vs_reference_cuda(cuda):
    """kernels/cuda/src/moe.cu moe_gemm_f32 (grid (E, ceil(N/32)), block 128) on the same routing."""
    if not RefCuda.available("moe"):
        pytest.skip("oracle/_ref/moe.cubin not built")
    ref = RefCuda()
    T, E, topk, N, K = 64, 8, 2, 96, 128
    r = _routing(121, T, E, topk, cuda)
    g = torch.Generator().manual_seed(122)
    x = torch.randn(T, K, generator=g).to(cuda)
    w = (torch.randn(E, N, K, generator=g) * 0.1).to(cuda)
    mine = ops.MoEGemm(x, w, r, r.weights, topk)
    counts = torch.bincount(r.sorted_expts, minlength=E)
    offsets = torch.zeros(E + 1, dtype=torch.int32, device=cuda)
    offsets[1:] = torch.cumsum(counts, 0).to(torch.int32)
    theirs = torch.zeros(T * topk, N, device=cuda)
    ref.launch("moe", "moe_gemm_f32", (E, (N + 31) // 32), (128,),
               [C.c_void_p(x.data_ptr()), C.c_void_p(w.data_ptr()), C.c_void_p(r.sorted_pairs.data_ptr()),
                C.c_void_p(offsets.data_ptr()), C.c_void_p(r.weights.data_ptr()), C.c_void_p(theirs.data_ptr()),
                C.c_int(topk), C.c_ulong(T * topk), C.c_ulong(N), C.c_ulong(K), C.c_int(0)])
    torch.cuda.synchronize()
    assert rel_l2(mine.cpu().numpy(), theirs.cpu().numpy()) <= 1e-3


def _skewed_routing(seed, T, E, topk, dev):
    """Biased router (per-expert bias ~ N(0, 1.5)): some experts get several tiles, some get nothing."""
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(T, E, generator=g) + torch.randn(E, generator=g) * 1.5
    logits[:, E - 1] = -1e9  # the last expert never routed
    return ops.MoERoute(torch.softmax(logits, dim=1).to(dev), topk, True)


def test_moe_grouped_tensor_core_dense_bf16(cuda, oracle):
    """M >= 256 pairs takes the tcgen05 grouped kernel (bf16 operands): same contract, bf16 tolerance."""
    T, E, topk, N, K = 300, 8, 2, 320, 128
    r = _skewed_routing(131, T, E, topk, cuda)
    g = torch.Generator().manual_seed(132)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(E, N, K, generator=g) * 0.1).to(torch.bfloat16)
    got = ops.MoEGemm(x.to(cuda), w.to(cuda), r, r.weights, topk)
    want = oracle.moe_gemm_f32(x.float().numpy(), w.float().numpy(), r.sorted_pairs.cpu().numpy(),
                               r.sorted_expts.cpu().numpy(), r.weights.cpu().numpy(), T * topk, topk, False)
    assert got.dtype == torch.bfloat16 and rel_l2(got.float().cpu().numpy(), want) <= 4e-3
    assert ops.prefill_status(0) == 0


@pytest.mark.parametrize("name", ["q4_k", "q6_k", "q8_0"])
def test_moe_grouped_tensor_core_gguf(cuda, oracle, name):
    dt = {"q4_k": ops.Q4_K, "q6_k": ops.Q6_K, "q8_0": ops.Q8_0}[name]
    T, E, topk, N, K = 400, 6, 2, 264, 512
    r = _skewed_routing(141, T, E, topk, cuda)
    raw = synth.random_blocks(142, dt, E * N, K)
    deq = oracle.dequant(dt, raw.reshape(-1), E * N * K).reshape(E, N, K)
    x = torch.randn(T, K, generator=torch.Generator().manual_seed(143))
    w = ops.QTensor(torch.from_numpy(raw.reshape(-1)).to(cuda), dt, (E, N, K))
    got = ops.MoEGemmQ(x.to(cuda), w, r, r.weights, topk).cpu().numpy()
    want = oracle.moe_gemm_f32(x.numpy(), deq, r.sorted_pairs.cpu().numpy(), r.sorted_expts.cpu().numpy(),
                               r.weights.cpu().numpy(), T * topk, topk, False)
    assert rel_l2(got, want) <= 1e-3
    # second GEMM of a layer: one input row per pair, no routing weights
    h = torch.randn(T * topk, K, generator=torch.Generator().manual_seed(144))
    got2 = ops.MoEGemmQ(h.to(cuda), w, r, None, topk).cpu().numpy()
    want2 = oracle.moe_gemm_f32(h.numpy(), deq, r.sorted_pairs.cpu().numpy(), r.sorted_expts.cpu().numpy(), None,
                                T * topk, topk, True)
    assert rel_l2(got2, want2) <= 1e-3


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-3), (torch.bfloat16, 4e-3)])
def test_moe_gemm_f8block(cuda, oracle, dtype, tol):
    """Block-scaled FP8 experts (128 x 128 blocks) against the per-expert loop the reference runs:
    dequantize each expert (oracle) and take the pair-wise dot products."""
    T, E, topk, N, K, b = 350, 8, 2, 256, 384, 128
    r = _skewed_routing(151, T, E, topk, cuda)
    codes, scale = synth.random_fp8_block(152, E * N, K, b, b)
    deq = oracle.fp8_block_dequant(codes.numpy(), scale.numpy(), b, b).reshape(E, N, K)
    if dtype == torch.bfloat16:
        deq = torch.from_numpy(deq).to(torch.bfloat16).float().numpy()
    x = torch.randn(T, K, generator=torch.Generator().manual_seed(153)).to(dtype)
    got = ops.MoEGemmF8Block(x.to(cuda), codes.reshape(E, N, K).to(cuda), scale.reshape(E, N // b, K // b).to(cuda), b, b, r,
                             r.weights, topk)
    want = oracle.moe_gemm_f32(x.float().numpy(), deq, r.sorted_pairs.cpu().numpy(), r.sorted_expts.cpu().numpy(),
                               r.weights.cpu().numpy(), T * topk, topk, False)
    assert got.dtype == dtype and rel_l2(got.float().cpu().numpy(), want) <= tol
    # rows of the never-routed expert and of pairs that do not exist stay zero
    assert ops.prefill_status(0) == 0
