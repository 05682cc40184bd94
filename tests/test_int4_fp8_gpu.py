"""GPU parity of the GPTQ/AWQ int4 and block-scaled FP8 paths through the C ABI."""
import ctypes as C

import numpy as np
import pytest
import torch

from helpers import RefCuda, max_rel, rel_l2
from light_b200 import ops, synth

pytestmark = pytest.mark.gpu


def _int4(seed, N, K, G, dev):
    codes, s, z = synth.random_int4(seed, N, K, G)
    w = ops.Int4(torch.from_numpy(codes.view(np.int32)).to(dev), torch.from_numpy(s).to(dev),
                 torch.from_numpy(z).to(dev), G)
    return codes, s, z, w


@pytest.mark.parametrize("G", [32, 128])
def test_int4_dequant_exact(cuda, oracle, G):
    """ops/int4_test.go:47-78: dequantized weight equals the host reference exactly, f32 and bf16;
    the offset form fills one slot of a stacked buffer."""
    N, K = 24, 512
    codes, s, z, w = _int4(81, N, K, G, cuda)
    want = oracle.int4_dequant(codes, s, z, G)
    got = ops.DequantizeInt4(w, torch.float32).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    want16 = oracle.int4_dequant(codes, s, z, G, bf16=True)
    got16 = ops.DequantizeInt4(w, torch.bfloat16).view(torch.int16).cpu().numpy().astype(np.uint16)
    assert np.array_equal(got16, want16)
    stack = torch.full((3, N, K), -1.0, device=cuda)
    ops.DequantizeInt4(w, torch.float32, out=stack, offset=N * K)
    assert np.array_equal(stack[1].cpu().numpy(), want)
    assert torch.all(stack[0] == -1) and torch.all(stack[2] == -1)


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
def test_int4_matmul_vs_f64(cuda, oracle, M):
    """ops/int4_test.go:80-145: tol 1e-4 (f32) / 3e-2 (bf16) relative to 1 + |want|, M in
    {1, 3, 8, 9}; config-4-like group 128."""
    N, K, G = 200, 1024, 128
    codes, s, z, w = _int4(82, N, K, G, cuda)
    deq = oracle.int4_dequant(codes, s, z, G).astype(np.float64)
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(83)).to(torch.bfloat16).float()
    want = x.numpy().astype(np.float64) @ deq.T
    got = ops.MatMulInt4(x.to(cuda), w).cpu().numpy()
    assert max_rel(got, want) <= 1e-4 and rel_l2(got, want) <= 1e-3
    got16 = ops.MatMulInt4(x.to(cuda).to(torch.bfloat16), w)
    assert got16.dtype == torch.bfloat16
    assert max_rel(got16.float().cpu().numpy(), want) <= 3e-2


def test_int4_act_order_and_converters(cuda, oracle):
    """Act-order GPTQ: x's columns are gathered by Perm before the multiply (ops/int4.go:79-85);
    a GPTQ-packed checkpoint converted by the oracle's FromGPTQ restatement feeds the kernel."""
    N, K, G = 64, 256, 128
    codes, s, z = synth.random_int4(84, N, K, G)
    z = np.clip(z, 1, 15)
    c2, s2, z2 = oracle.int4_from_gptq(*synth.to_gptq(codes, s, z), group=G)
    perm = torch.randperm(K, generator=torch.Generator().manual_seed(85))
    w = ops.Int4(torch.from_numpy(c2.view(np.int32)).to(cuda), torch.from_numpy(s2).to(cuda),
                 torch.from_numpy(z2).to(cuda), G, perm=perm.to(cuda))
    x = torch.randn(2, K, generator=torch.Generator().manual_seed(86))
    deq = oracle.int4_dequant(codes, s, z, G).astype(np.float64)
    want = x[:, perm].numpy().astype(np.float64) @ deq.T
    assert max_rel(ops.MatMulInt4(x.to(cuda), w).cpu().numpy(), want) <= 1e-4


def test_int4_vs_reference_cuda(cuda):
    """kernels/cuda/src/int4.cu int4_gemv_f32 / int4_dequant_f32 (launch shapes
    kernels/cuda/int4.go:64-68,98-100) on the same inputs."""
    if not RefCuda.available("int4"):
        pytest.skip("oracle/_ref/int4.cubin not built")
    ref = RefCuda()
    N, K, G = 512, 3584, 128
    codes, s, z, w = _int4(87, N, K, G, cuda)
    for M in (1, 8):
        x = torch.randn(M, K, generator=torch.Generator().manual_seed(88)).to(cuda)
        theirs = torch.zeros(M, N, device=cuda)
        ref.launch("int4", "int4_gemv_f32", ((N + 7) // 8,), (256,),
                   [C.c_void_p(x.data_ptr()), C.c_void_p(w.codes.data_ptr()), C.c_void_p(w.scales.data_ptr()),
                    C.c_void_p(w.zeros.data_ptr()), C.c_void_p(theirs.data_ptr()), C.c_int(M), C.c_int(N), C.c_int(K),
                    C.c_int(G)])
        mine = ops.MatMulInt4(x, w)
        torch.cuda.synchronize()
        assert rel_l2(mine.cpu().numpy(), theirs.cpu().numpy()) <= 1e-3
    theirs = torch.zeros(N, K, device=cuda)
    words = N * K // 8
    ref.launch("int4", "int4_dequant_f32", ((words + 255) // 256,), (256,),
               [C.c_void_p(w.codes.data_ptr()), C.c_void_p(w.scales.data_ptr()), C.c_void_p(w.zeros.data_ptr()),
                C.c_void_p(theirs.data_ptr()), C.c_int(N), C.c_int(K), C.c_int(G)])
    mine = ops.DequantizeInt4(w, torch.float32)
    torch.cuda.synchronize()
    assert torch.equal(mine, theirs)


def test_fp8_block_dequant_exact(cuda, oracle):
    """ops/fp8_block_test.go:16-71: 12 x 32 weight with 4 x 8 blocks and a 128 x 128-block weight,
    exact at f32 and bf16; a block size that does not divide the rows is rejected."""
    for (R, Cc, br, bc, seed) in ((12, 32, 4, 8, 91), (256, 384, 128, 128, 92)):
        codes, scale = synth.random_fp8_block(seed, R, Cc, br, bc, sigma=50.0)
        want = oracle.fp8_block_dequant(codes.numpy(), scale.numpy(), br, bc)
        got = ops.DequantizeF8Block(codes.to(cuda), scale.to(cuda), br, bc, torch.float32).cpu().numpy()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        want16 = oracle.fp8_block_dequant(codes.numpy(), scale.numpy(), br, bc, bf16=True)
        got16 = ops.DequantizeF8Block(codes.to(cuda), scale.to(cuda), br, bc, torch.bfloat16)
        assert np.array_equal(got16.view(torch.int16).cpu().numpy().astype(np.uint16), want16)
    with pytest.raises(ValueError):
        ops.DequantizeF8Block(codes.to(cuda), scale.to(cuda), 5, 128, torch.float32)


def test_fp8_all_codes_decode(cuda, oracle):
    """Every e4m3 code (NaN codes excluded: never a weight) through the GPU decoder with scale 1."""
    codes = torch.tensor([c for c in range(256) if c & 0x7F != 0x7F] + [0, 0], dtype=torch.uint8).reshape(1, 256)
    got = ops.DequantizeF8Block(codes.to(cuda), torch.ones(1, 1, device=cuda), 1, 256, torch.float32).cpu().numpy()
    want = oracle.e4m3_table()[codes.numpy()]
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("M", [1, 3, 8, 9])
def test_fp8_block_matmul_vs_f64(cuda, oracle, M):
    """ops/fp8_block_test.go:106-186: N = 384, K = 512, 128 x 128 blocks, tol 1e-4 / 3e-2."""
    N, K, b = 384, 512, 128
    codes, scale = synth.random_fp8_block(93, N, K, b, b)
    deq = oracle.fp8_block_dequant(codes.numpy(), scale.numpy(), b, b).astype(np.float64)
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(94)).to(torch.bfloat16).float()
    want = x.numpy().astype(np.float64) @ deq.T
    got = ops.MatMulF8Block(x.to(cuda), codes.to(cuda), scale.to(cuda), b, b).cpu().numpy()
    assert max_rel(got, want) <= 1e-4 and rel_l2(got, want) <= 1e-3
    got16 = ops.MatMulF8Block(x.to(cuda).to(torch.bfloat16), codes.to(cuda), scale.to(cuda), b, b)
    assert got16.dtype == torch.bfloat16 and max_rel(got16.float().cpu().numpy(), want) <= 3e-2


def test_fp8_vs_reference_cuda(cuda):
    """kernels/cuda/src/fp8_block.cu fp8_block_gemv_f32 / fp8_block_dequant_f32 on the same inputs."""
    if not RefCuda.available("fp8_block"):
        pytest.skip("oracle/_ref/fp8_block.cubin not built")
    ref = RefCuda()
    N, K, b = 512, 7168, 128
    codes, scale = synth.random_fp8_block(95, N, K, b, b, device="cpu")
    wd, sd = codes.to(cuda), scale.to(cuda)
    for M in (1, 8):
        x = torch.randn(M, K, generator=torch.Generator().manual_seed(96)).to(cuda)
        theirs = torch.zeros(M, N, device=cuda)
        ref.launch("fp8_block", "fp8_block_gemv_f32", ((N + 7) // 8,), (256,),
                   [C.c_void_p(x.data_ptr()), C.c_void_p(wd.data_ptr()), C.c_void_p(sd.data_ptr()),
                    C.c_void_p(theirs.data_ptr()), C.c_int(M), C.c_int(N), C.c_int(K), C.c_int(b), C.c_int(b)])
        mine = ops.MatMulF8Block(x, wd, sd, b, b)
        torch.cuda.synchronize()
        assert rel_l2(mine.cpu().numpy(), theirs.cpu().numpy()) <= 1e-3
    theirs = torch.zeros(N, K, device=cuda)
    n4 = N * K // 4
    ref.launch("fp8_block", "fp8_block_dequant_f32", (min((n4 + 255) // 256, 65535),), (256,),
               [C.c_void_p(wd.data_ptr()), C.c_void_p(sd.data_ptr()), C.c_void_p(theirs.data_ptr()), C.c_int(N),
                C.c_int(K), C.c_int(b), C.c_int(b)])
    mine = ops.DequantizeF8Block(wd, sd, b, b, torch.float32)
    torch.cuda.synchronize()
    assert torch.equal(mine, theirs)


@pytest.mark.parametrize("layout,N,K,G", [("gptq", 600, 3584, 128), ("gptq_v2", 40, 256, 64), ("awq", 600, 3584, 128), ("awq", 8, 64, 32)])
def test_int4_checkpoint_repack_matches_oracle(cuda, oracle, layout, N, K, G):
    """The device converters against the oracle's quant.FromGPTQ / quant.FromAWQ at a Qwen2.5-7B W4A16 shape and at
    ragged tile edges (N, K/8 not multiples of 32)."""
    codes, s, z = synth.random_int4(701, N, K, G)
    if layout == "gptq":
        z[z == 0] = 1.0  # the v1 format stores zero - 1 in four bits
    qw, qz, sc = synth.to_awq(codes, s, z) if layout == "awq" else synth.to_gptq(codes, s, z, v2=layout == "gptq_v2")
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int32) if a.dtype == np.uint32 else np.ascontiguousarray(a)).to(cuda)
    w = ops.Int4FromCheckpoint(t(qw), t(qz), t(sc), G, layout)
    c2, s2, z2 = oracle.int4_from_awq(qw, qz, sc, G) if layout == "awq" else oracle.int4_from_gptq(qw, qz, sc, G, v2=layout == "gptq_v2")
    assert np.array_equal(w.codes.cpu().numpy().view(np.uint32), c2) and np.array_equal(c2, codes)
    assert np.array_equal(w.scales.cpu().numpy(), s2) and np.array_equal(w.zeros.cpu().numpy(), z2)


@pytest.mark.parametrize("N,K,G", [(600, 3584, 128), (16, 256, 64), (37, 2048, 256), (200, 18944, 128)])
def test_int4_one_row_tensor_core_kernel(cuda, oracle, N, K, G):
    """The one-row decode kernel (tensor-core arithmetic on the canonical layout): ragged heights, one to 74
    runs of 256 k, groups of 64 to 256; f32 rows 1..8 (ops/int4_test.go's 1e-4 bound) and bf16 rows 1..3."""
    codes, s, z, w = _int4(801, N, K, G, cuda)
    deq = oracle.int4_dequant(codes, s, z, G).astype(np.float64)
    g = torch.Generator().manual_seed(802)
    for M in (1, 2, 8):
        x = torch.randn(M, K, generator=g)
        got = ops.MatMulInt4(x.to(cuda), w)
        assert torch.equal(got, ops.MatMulInt4(x.to(cuda), w))
        want = x.numpy().astype(np.float64) @ deq.T
        assert max_rel(got.cpu().numpy(), want) <= 1e-4 and rel_l2(got.cpu().numpy(), want) <= 1e-5, (M, rel_l2(got.cpu().numpy(), want))
    for M in (1, 3):
        xb = torch.randn(M, K, generator=g).to(torch.bfloat16)
        got = ops.MatMulInt4(xb.to(cuda), w)
        assert got.dtype == torch.bfloat16
        assert max_rel(got.float().cpu().numpy(), xb.float().numpy().astype(np.float64) @ deq.T) <= 3e-2
    big = torch.randn(1, K, generator=g) * 1e6  # beyond f16 range: the exact power-of-two prescale
    assert rel_l2(ops.MatMulInt4(big.to(cuda), w).cpu().numpy(), big.numpy().astype(np.float64) @ deq.T) <= 1e-5


@pytest.mark.parametrize("N,K,bR,bC", [(384, 7168, 128, 128), (128, 256, 128, 128), (64, 2048, 16, 32), (4096, 512, 128, 256)])
def test_fp8_one_row_tensor_core_kernel(cuda, oracle, N, K, bR, bC):
    """The one-row decode kernel for block-scaled e4m3: every code value (subnormals, both zeros) through the
    bit-shift decode, one to 28 runs of 256 k, block shapes down to 16 x 32; f32 rows against the 1e-4 bound of
    ops/fp8_block_test.go, bf16 rows against 3e-2."""
    rng = np.random.Generator(np.random.Philox(811))
    legal = np.array([c for c in range(256) if (c & 0x7F) != 0x7F], np.uint8)
    codes = torch.from_numpy(legal[rng.integers(0, legal.size, size=(N, K))])
    scale = torch.from_numpy(rng.uniform(1e-4, 2.1e-3, size=(N // bR, K // bC)).astype(np.float32))
    deq = oracle.fp8_block_dequant(codes.numpy(), scale.numpy(), bR, bC).astype(np.float64)
    g = torch.Generator().manual_seed(812)
    for M in (1, 2, 9):
        x = torch.randn(M, K, generator=g)
        got = ops.MatMulF8Block(x.to(cuda), codes.to(cuda), scale.to(cuda), bR, bC)
        assert torch.equal(got, ops.MatMulF8Block(x.to(cuda), codes.to(cuda), scale.to(cuda), bR, bC))
        want = x.numpy().astype(np.float64) @ deq.T
        assert max_rel(got.cpu().numpy(), want) <= 1e-4 and rel_l2(got.cpu().numpy(), want) <= 1e-5, (M, rel_l2(got.cpu().numpy(), want))
    for M in (1, 2):
        xb = torch.randn(M, K, generator=g).to(torch.bfloat16)
        got = ops.MatMulF8Block(xb.to(cuda), codes.to(cuda), scale.to(cuda), bR, bC)
        assert got.dtype == torch.bfloat16
        assert max_rel(got.float().cpu().numpy(), xb.float().numpy().astype(np.float64) @ deq.T) <= 3e-2
