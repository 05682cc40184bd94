"""Device-side routing against the oracle's restatements of the host router (models/deepseek_route.go:30-133) and
of the expert sort (ops/moe.go:62-99): the chosen experts and their order exactly, the weights to 1e-6, the
sorted pair list bit for bit."""
import numpy as np
import pytest
import torch

from light_b200 import ops

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,E,topk,norm", [(4096, 256, 8, True), (33, 8, 2, True), (5, 64, 6, False), (1, 1000, 32, True)])
def test_route_sigmoid(cuda, oracle, T, E, topk, norm):
    """BASELINE config 5 routing: logits ~ N(0, 1), per-expert bias ~ N(0, 0.5)."""
    g = torch.Generator().manual_seed(900 + T)
    logits, bias = torch.randn(T, E, generator=g), torch.randn(E, generator=g) * 0.5
    want_ids, want_w = oracle.deepseek_route_sigmoid(logits.numpy(), bias.numpy(), topk, norm)
    r = ops.MoERouteSigmoid(logits.to(cuda), bias.to(cuda), topk, norm)
    assert np.array_equal(r.topk_ids.cpu().numpy(), want_ids)
    assert np.max(np.abs(r.weights.cpu().numpy().reshape(T, topk) - want_w)) <= 1e-6
    sp, se = oracle.moe_sort_pairs(want_ids.reshape(-1), E)
    assert np.array_equal(r.sorted_pairs.cpu().numpy(), sp) and np.array_equal(r.sorted_expts.cpu().numpy(), se)
    assert ops.moe_route_status(0) == 0


def test_route_ties_keep_the_lower_expert(cuda, oracle):
    logits = torch.zeros(3, 40)
    logits[1, 7] = logits[1, 39] = 2.0
    want_ids, want_w = oracle.deepseek_route_sigmoid(logits.numpy(), None, 4, True)
    r = ops.MoERouteSigmoid(logits.to(cuda), None, 4, True)
    assert np.array_equal(r.topk_ids.cpu().numpy(), want_ids)
    assert list(want_ids[0]) == [0, 1, 2, 3] and list(want_ids[1][:2]) == [7, 39]
    assert np.max(np.abs(r.weights.cpu().numpy().reshape(3, 4) - want_w)) <= 1e-6


@pytest.mark.parametrize("M,E", [(32768, 256), (10, 4), (1025, 7), (1, 1), (5000, 1024)])
def test_sort_pairs(cuda, oracle, M, E):
    rng = np.random.Generator(np.random.Philox(910 + M))
    ids = np.minimum((rng.exponential(E / 6.0, size=M)).astype(np.int64), E - 1)  # a skewed load
    if M == 10:
        ids = np.array([0, 2, 2, 1, 3, 0, 2, 3, 1, 2], np.int64)  # the fixed ids of ops/int4_test.go's MoE case
    sp, se, counts, offsets = ops.MoESortPairs(torch.from_numpy(ids).to(cuda), E)
    wp, we = oracle.moe_sort_pairs(ids, E)
    assert np.array_equal(sp.cpu().numpy(), wp) and np.array_equal(se.cpu().numpy(), we)
    c = np.bincount(ids, minlength=E)
    assert np.array_equal(counts.cpu().numpy(), c) and np.array_equal(offsets.cpu().numpy(), np.concatenate([[0], np.cumsum(c)]))
    assert ops.moe_route_status(0) == 0
