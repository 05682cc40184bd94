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
    """The DeepSeek-V3 MoE workload's routing: logits ~ N(0, 1), per-expert bias ~ N(0, 0.5)."""
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


@pytest.mark.parametrize("E,topk,n_group,topk_group,sigmoid", [(256, 8, 8, 4, True), (64, 6, 8, 3, False), (160, 6, 1, 1, False), (256, 8, 1, 1, True),
                                                                 (96, 4, 4, 2, True), (33, 5, 1, 1, False)])
def test_deepseek_router_every_branch(cuda, oracle, E, topk, n_group, topk_group, sigmoid):
    """models/deepseek_route.go:30-133: group-limited selection (V3: two best per group; V2: the best), sigmoid + bias
    and softmax scores, ids exact, weights to 1e-6."""
    g = torch.Generator().manual_seed(E + topk)
    T = 300
    logits = torch.randn(T, E, generator=g)
    logits[5] = logits[4]              # equal rows
    logits[7, :8] = 0.25               # ties inside a row: the lower expert id wins
    bias = torch.randn(E, generator=g) * 0.5 if sigmoid else None
    r = ops.MoERouteDeepseek(logits.to(cuda), None if bias is None else bias.to(cuda), topk, n_group, topk_group, sigmoid, True)
    ids, w = oracle.deepseek_route(logits.numpy(), None if bias is None else bias.numpy(), topk, n_group, topk_group, sigmoid, True)
    assert np.array_equal(r.topk_ids.cpu().numpy(), ids)
    assert np.max(np.abs(r.weights.reshape(T, topk).cpu().numpy() - w)) <= 1e-6
    se, sp = torch.sort(r.topk_ids.reshape(-1), stable=True)
    assert torch.equal(r.sorted_expts, se) and torch.equal(r.sorted_pairs, sp)
    assert ops.moe_route_status(0) == 0


@pytest.mark.parametrize("normalize", [True, False])
def test_softmax_route_on_the_device(cuda, oracle, normalize):
    """ops.MoERoute (ops/moe.go:29-71) without torch.topk / torch.sort."""
    T, E, topk = 257, 60, 4
    probs = torch.softmax(torch.randn(T, E, generator=torch.Generator().manual_seed(3)), dim=1)
    probs[9, 3] = probs[9, 11]         # a tie
    r = ops.MoERoute(probs.to(cuda), topk, normalize)
    ids, w = oracle.moe_route_topk(probs.numpy(), topk, normalize)
    assert np.array_equal(r.topk_ids.cpu().numpy(), ids)
    assert np.max(np.abs(r.weights.reshape(T, topk).cpu().numpy() - w)) <= 1e-6
    se, sp = torch.sort(r.topk_ids.reshape(-1), stable=True)
    assert torch.equal(r.sorted_expts, se) and torch.equal(r.sorted_pairs, sp)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_gate_mul_and_combine(cuda, dtype):
    """The unfused sequence's arithmetic (nn/moe.go:206-236, ops/moe.go:206-240): activation rounded, then the product;
    slot rows added one after the other with a rounding per sum."""
    g = torch.Generator().manual_seed(8)
    M, I, topk, N = 96, 72, 4, 40
    h = torch.randn(M, 2 * I, generator=g).to(dtype)
    for gelu in (False, True):
        got = ops.MoEGateMul(h.to(cuda), gelu)
        gv = h[:, :I].float()
        a = (0.5 * gv * (1 + torch.erf(gv / 2 ** 0.5))) if gelu else gv / (1 + torch.exp(-gv))
        want = (a.to(dtype).float() * h[:, I:].float()).to(dtype)
        tol = 1e-6 if dtype == torch.float32 else 2e-2
        assert torch.allclose(got.float().cpu(), want.float(), rtol=tol, atol=tol)
    y = torch.randn(M, N, generator=g).to(dtype)
    got = ops.MoECombine(y.to(cuda), topk)
    v = y.reshape(M // topk, topk, N)
    acc = v[:, 0]
    for s in range(1, topk):
        acc = (acc.float() + v[:, s].float()).to(dtype)
    assert torch.equal(got.cpu(), acc)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_combine_weighted(cuda, dtype):
    """Rows in another order, unweighted: out[t] = sum over slots (slot 0 first, f32) of weight * row(index); pairs whose
    index lies outside the rows contribute nothing; no index = pair order, no weights = 1."""
    g = torch.Generator().manual_seed(21)
    T, topk, N = 37, 3, 48
    M = T * topk
    rows = torch.randn(M + 5, N, generator=g).to(dtype)
    index = torch.randperm(M + 5, generator=g)[:M]
    index[4], index[50] = -1, M + 5
    w = torch.rand(M, generator=g)
    got = ops.MoECombineWeighted(rows.to(cuda), index.to(cuda), w.to(cuda), T, topk).cpu()
    want = torch.zeros(T, N)
    for t in range(T):
        for s in range(topk):
            p = t * topk + s
            if 0 <= int(index[p]) < M + 5:
                want[t] = torch.addcmul(want[t], rows[index[p]].float(), w[p])
    assert got.dtype == torch.float32 and torch.allclose(got, want, rtol=1e-6, atol=1e-6)
    plain = ops.MoECombineWeighted(rows.to(cuda), None, None, T, topk).cpu()
    assert torch.allclose(plain, rows[:M].float().reshape(T, topk, N).sum(1), rtol=1e-6, atol=1e-6)
    with pytest.raises(ValueError, match="no index"):
        ops.MoECombineWeighted(rows[:M - 1].to(cuda), None, None, T, topk)
    with pytest.raises(ValueError, match="index must be"):
        ops.MoECombineWeighted(rows.to(cuda), index[:5].to(cuda), None, T, topk)
