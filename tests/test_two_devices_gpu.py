"""One process driving two GPUs through the C ABI, as the reference's single Go process would: every kernel
attribute (the opt-in to more than 48 KB of dynamic shared memory) and every device symbol address is per
device, so the second device must work after the first has been used.  Skipped on a single-GPU box."""
import numpy as np
import pytest
import torch

from helpers import rel_l2
from light_b200 import ops, synth

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dt,N,K", [(ops.Q4_K, 512, 2048), (ops.Q6_K, 256, 2048), (ops.Q8_0, 256, 1024)])
def test_matmul_q_on_device_1_after_device_0(cuda, oracle, dt, N, K):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    from light_b200 import _lib

    raw = synth.gaussian_weight(77, dt, N, K)
    deq = oracle.dequant(dt, raw.numpy().reshape(-1), N * K).reshape(N, K).astype(np.float64)
    for M in (1, 4, 12, 32, 128):      # one row, token columns, tiles, tcgen05 decode, tcgen05 prefill
        x = torch.randn(M, K, generator=torch.Generator().manual_seed(M))
        want = x.numpy().astype(np.float64) @ deq.T
        for d in (0, 1):
            dev = torch.device("cuda", d)
            _lib.check(_lib.lib().light_b200_init(d))
            with torch.cuda.device(dev):
                got = ops.MatMulQ(x.to(dev), ops.QTensor(raw.reshape(-1).to(dev), dt, (N, K)))
                torch.cuda.synchronize(dev)
            assert rel_l2(got.cpu().numpy(), want) <= 1e-3, (dt, M, d)
    assert ops.prefill_status(0) == 0 and ops.prefill_status(1) == 0


def test_moe_sort_and_attention_on_device_1(cuda):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    for d in (0, 1):
        dev = torch.device("cuda", d)
        with torch.cuda.device(dev):
            ids = torch.randint(0, 64, (5000,), generator=torch.Generator().manual_seed(3)).to(dev)
            got_sp, got_se, _, _ = ops.MoESortPairs(ids, 64)
            se, sp = torch.sort(ids, stable=True)
            torch.cuda.synchronize(dev)
            assert torch.equal(got_se, se) and torch.equal(got_sp, sp), d
            assert ops.moe_route_status(d) == 0
