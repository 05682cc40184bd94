"""GPU parity of the tensor-core batched-decode kernel (weight rows on the M side of tcgen05.mma, tokens
on N, K split over a thread-block cluster): GGUF from 17 tokens up, int4 and block-scaled FP8 with
bf16 activations from one token up.  The oracle is the f64 product with the CPU-dequantized weights,
as in the reference's own tests (ops/matmul_q_test.go:105-146, ops/int4_test.go:80-145,
ops/fp8_block_test.go:106-186)."""
import numpy as np
import pytest
import torch

from helpers import rel_l2
from light_b200 import ops, synth

pytestmark = pytest.mark.gpu


def _bf16(a: np.ndarray) -> np.ndarray:
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy().astype(np.float64)


@pytest.mark.parametrize("name,dt,N,K", [("q4_k", ops.Q4_K, 300, 4096), ("q4_k", ops.Q4_K, 129, 256), ("q4_k", ops.Q4_K, 1024, 512),
                                          ("q6_k", ops.Q6_K, 300, 14336), ("q6_k", ops.Q6_K, 128, 2048)])
def test_gguf_batched_decode(cuda, oracle, name, dt, N, K):
    """Ragged heights (a last tile of 44 or 1 rows), one to 56 blocks per row (cluster sizes 1 to 8, uneven
    K runs), token counts that fill 32 and 64 MMA columns partly and fully; twice the same bits."""
    raw = synth.gaussian_weight(301, dt, N, K).numpy()
    deq = oracle.dequant(dt, raw.reshape(-1), N * K).reshape(N, K).astype(np.float64)
    w = ops.QTensor(torch.from_numpy(raw.reshape(-1)).to(cuda), dt, (N, K))
    g = torch.Generator().manual_seed(302)
    for M in (17, 32, 40, 64):
        x = torch.randn(M, K, generator=g)
        got = ops.MatMulQ(x.to(cuda), w)
        again = ops.MatMulQ(x.to(cuda), w)
        assert torch.equal(got, again), "the cluster reduction must be deterministic"
        want = x.numpy().astype(np.float64) @ deq.T
        assert rel_l2(got.cpu().numpy(), want) <= 1e-3, (name, N, K, M, rel_l2(got.cpu().numpy(), want))
    assert ops.prefill_status(cuda.index or 0) == 0


@pytest.mark.parametrize("N,K", [(300, 4096), (129, 256), (1024, 768), (2064, 1280), (16, 2048)])
def test_q4k_decode_9_to_32_rows(cuda, oracle, N, K):
    """The register-fed kernel for 9 to 32 activation rows (eight row tiles per CTA, K split over a
    cluster): ragged heights (a last row tile that overlaps the one before, CTAs with fewer than eight
    live tiles, a single tile), one to 16 blocks per row (K runs of uneven length, clusters of 1, 2, 4
    and 8), token counts that fill two and four groups of eight partly and fully; twice the same bits."""
    raw = synth.gaussian_weight(331, ops.Q4_K, N, K).numpy()
    deq = oracle.dequant(ops.Q4_K, raw.reshape(-1), N * K).reshape(N, K).astype(np.float64)
    w = ops.QTensor(torch.from_numpy(raw.reshape(-1)).to(cuda), ops.Q4_K, (N, K))
    g = torch.Generator().manual_seed(332)
    for M in (9, 15, 16, 17, 25, 32):
        x = torch.randn(M, K, generator=g)
        got = ops.MatMulQ(x.to(cuda), w)
        assert torch.equal(got, ops.MatMulQ(x.to(cuda), w)), "the cluster reduction must be deterministic"
        want = x.numpy().astype(np.float64) @ deq.T
        assert rel_l2(got.cpu().numpy(), want) <= 1e-3, (N, K, M, rel_l2(got.cpu().numpy(), want))
    assert ops.prefill_status(cuda.index or 0) == 0


@pytest.mark.parametrize("M", [1, 5, 16, 17, 33, 64])
def test_int4_bf16_decode(cuda, oracle, M):
    """The Qwen2.5-7B W4A16 shape class (K = 3584, group 128, bf16 activations): the operands are the
    reference's bf16 weights bit for bit, so the f64 product of bf16-rounded weights and bf16 x is the
    oracle, up to the one bf16 rounding of the output."""
    N, K, G = 600, 3584, 128
    codes, s, z = synth.random_int4(311, N, K, G)
    w = ops.Int4(torch.from_numpy(codes.view(np.int32)).to(cuda), torch.from_numpy(s).to(cuda), torch.from_numpy(z).to(cuda), G)
    wq = _bf16(oracle.int4_dequant(codes, s, z, G))
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(312)).to(torch.bfloat16)
    got = ops.MatMulInt4(x.to(cuda), w)
    assert got.dtype == torch.bfloat16 and got.shape == (M, N)
    want = x.float().numpy().astype(np.float64) @ wq.T
    assert rel_l2(got.float().cpu().numpy(), want) <= 3e-3
    assert torch.equal(got, ops.MatMulInt4(x.to(cuda), w))


@pytest.mark.parametrize("M", [1, 8, 24, 64])
def test_fp8_block_bf16_decode(cuda, oracle, M):
    """The DeepSeek-V3 expert shape class (K = 7168, 128 x 128 blocks, bf16 activations)."""
    N, K, b = 384, 7168, 128
    codes, scale = synth.random_fp8_block(321, N, K, b, b)
    wq = _bf16(oracle.fp8_block_dequant(codes.numpy(), scale.numpy(), b, b))
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(322)).to(torch.bfloat16)
    got = ops.MatMulF8Block(x.to(cuda), codes.to(cuda), scale.to(cuda), b, b)
    assert got.dtype == torch.bfloat16
    want = x.float().numpy().astype(np.float64) @ wq.T
    assert rel_l2(got.float().cpu().numpy(), want) <= 3e-3
    assert ops.prefill_status(cuda.index or 0) == 0
