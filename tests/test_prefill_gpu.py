"""GPU parity of the tensor-core prefill path (matmul_q with M > 64) through the C ABI."""
import numpy as np
import pytest
import torch

from helpers import rel_l2
from light_b200 import ops, synth

pytestmark = pytest.mark.gpu


def _case(dt, M, N, K, seed, cuda, oracle, bf16_x):
    raw = synth.gaussian_weight(seed, dt, N, K).numpy() if seed % 2 else synth.random_blocks(seed, dt, N, K)
    deq = oracle.dequant(dt, raw.reshape(-1), N * K).reshape(N, K).astype(np.float64)
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(seed + 1))
    if bf16_x:
        x = x.to(torch.bfloat16).float()
    w = ops.QTensor(torch.from_numpy(raw.reshape(-1)).to(cuda), dt, (N, K))
    got = ops.MatMulQ(x.to(cuda), w).cpu().numpy()
    want = x.numpy().astype(np.float64) @ deq.T
    return rel_l2(got, want)


@pytest.mark.parametrize("M,N,K", [(65, 256, 256), (128, 256, 1024), (256, 512, 512), (300, 300, 768),
                                   (513, 1000, 2048), (2048, 1024, 4096)])
def test_q4k_prefill_matches_f64_oracle(cuda, oracle, M, N, K):
    """f16 operands, f32 accumulation: with bf16-valued activations (exact in f16) only the single
    rounding of each weight to f16 remains (about 2e-4); the bound is the 1e-3 of the contract."""
    for seed, bf16_x in ((301, True), (302, True), (303, False)):
        err = _case(ops.Q4_K, M, N, K, seed, cuda, oracle, bf16_x)
        assert err <= (5e-4 if bf16_x else 1e-3), (M, N, K, seed, err)
    assert ops.prefill_status(0) == 0


def test_prefill_without_workspace_still_correct(cuda, oracle):
    """Withdrawing the workspace sends the call down the shape-generic kernel: same contract."""
    from light_b200 import _lib

    _lib.check(_lib.lib().light_b200_set_workspace(0, None, 0))
    ops._workspaces.clear()
    N, K, M = 64, 512, 70
    raw = synth.random_blocks(311, ops.Q4_K, N, K)
    deq = oracle.dequant(ops.Q4_K, raw.reshape(-1), N * K).reshape(N, K).astype(np.float64)
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(312))
    from light_b200._lib import lib, check
    import ctypes as C

    xd, wd = x.to(cuda), torch.from_numpy(raw.reshape(-1)).to(cuda)
    out = torch.empty(M, N, device=cuda)
    check(lib().light_b200_matmul_q(ops.Q4_K, C.c_void_p(xd.data_ptr()), C.c_void_p(wd.data_ptr()),
                                    C.c_void_p(out.data_ptr()), M, N, K, 0, None))
    assert rel_l2(out.cpu().numpy(), x.numpy().astype(np.float64) @ deq.T) <= 1e-5


@pytest.mark.parametrize("M,N,K", [(65, 256, 512), (200, 300, 1024), (256, 512, 2048), (1024, 1024, 14336), (70, 40, 768)])
def test_q6k_prefill_matches_f64_oracle(cuda, oracle, M, N, K):
    """Q6_K through the same kernel (K = 768 has rows that are not 4-byte aligned and takes the
    shape-generic kernel instead)."""
    for seed, bf16_x in ((321, True), (322, True), (323, False)):
        err = _case(ops.Q6_K, M, N, K, seed, cuda, oracle, bf16_x)
        assert err <= (5e-4 if bf16_x else 1e-3), (M, N, K, seed, err)
    assert ops.prefill_status(0) == 0


@pytest.mark.parametrize("M,N,K", [(65, 256, 256), (200, 300, 1024), (513, 1000, 2048), (1024, 1024, 14336), (70, 40, 800)])
def test_q80_prefill_matches_f64_oracle(cuda, oracle, M, N, K):
    """Q8_0 through the same kernel (K = 800 is no multiple of 256 and takes the shape-generic kernel)."""
    for seed, bf16_x in ((341, True), (342, False)):
        err = _case(ops.Q8_0, M, N, K, seed, cuda, oracle, bf16_x)
        assert err <= (5e-4 if bf16_x else 1e-3), (M, N, K, seed, err)
    assert ops.prefill_status(0) == 0


def _bf16_round(a: np.ndarray) -> np.ndarray:
    return torch.from_numpy(a.astype(np.float32)).to(torch.bfloat16).float().numpy().astype(np.float64)


@pytest.mark.parametrize("M,N,K,G", [(65, 256, 256, 128), (256, 512, 1024, 128), (300, 200, 512, 64), (1024, 4608, 3584, 128)])
def test_int4_prefill(cuda, oracle, M, N, K, G):
    """GPTQ/AWQ int4 on the tensor cores (config 4 shapes at the end).  bf16 activations: operands are
    the reference's bf16 weight (bit-identical dequantization) and x itself, so only accumulation order
    and the bf16 rounding of the output differ (reference tolerance 3e-2, ops/int4_test.go:80-145);
    f32 activations: f16 operands, 1e-3 relative L2 against the f64 oracle."""
    codes, s, z = synth.random_int4(331, N, K, G)
    w = ops.Int4(torch.from_numpy(codes.view(np.int32)).to(cuda), torch.from_numpy(s).to(cuda),
                 torch.from_numpy(z).to(cuda), G)
    deq = oracle.int4_dequant(codes, s, z, G).astype(np.float64)
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(332))
    got = ops.MatMulInt4(x.to(cuda), w).cpu().numpy()
    assert rel_l2(got, x.numpy().astype(np.float64) @ deq.T) <= 1e-3
    xb = x.to(torch.bfloat16)
    got16 = ops.MatMulInt4(xb.to(cuda), w)
    assert got16.dtype == torch.bfloat16
    want16 = xb.float().numpy().astype(np.float64) @ _bf16_round(deq).T
    assert rel_l2(got16.float().cpu().numpy(), want16) <= 4e-3  # one bf16 rounding of the output
    assert ops.prefill_status(0) == 0


@pytest.mark.parametrize("M,N,K", [(65, 256, 256), (200, 384, 512), (512, 4096, 7168)])
def test_fp8_block_prefill(cuda, oracle, M, N, K):
    """Block-scaled FP8 (128 x 128 blocks; the last shape is a DeepSeek-V3 expert's gate_up) on the
    tensor cores, bf16 and f32 activations."""
    b = 128
    codes, scale = synth.random_fp8_block(341, N, K, b, b)
    deq = oracle.fp8_block_dequant(codes.numpy(), scale.numpy(), b, b).astype(np.float64)
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(342))
    got = ops.MatMulF8Block(x.to(cuda), codes.to(cuda), scale.to(cuda), b, b).cpu().numpy()
    assert rel_l2(got, x.numpy().astype(np.float64) @ deq.T) <= 1e-3
    xb = x.to(torch.bfloat16)
    got16 = ops.MatMulF8Block(xb.to(cuda), codes.to(cuda), scale.to(cuda), b, b)
    want16 = xb.float().numpy().astype(np.float64) @ _bf16_round(deq).T
    assert got16.dtype == torch.bfloat16 and rel_l2(got16.float().cpu().numpy(), want16) <= 4e-3
    assert ops.prefill_status(0) == 0
