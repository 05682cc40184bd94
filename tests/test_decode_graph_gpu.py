"""The decode-step graph (light_b200.decode.DecodeGraph, the counterpart of models/decode_graph.go) against the same
step computed operator by operator with the CPU oracle: embedding row -> per layer [RMSNorm, q/k/v, RoPE, KV append,
attention, o, RMSNorm, SiLU(gate) * up, down] -> final norm -> lm_head -> argmax, several tokens in a row, eager,
with the norms as launches of their own, and replayed from a CUDA graph."""
import math

import numpy as np
import pytest
import torch

from helpers import rel_l2
from light_b200 import decode, ops, synth

pytestmark = pytest.mark.gpu

H, NH, KH, D, F, V, LAYERS, CAP = 1024, 8, 2, 128, 2048, 1536, 2, 48


def _model(cuda):
    def qt(seed, dt, N, K):
        raw = synth.gaussian_weight(seed, dt, N, K)
        return ops.QTensor(raw.reshape(-1).to(cuda), dt, (N, K)), raw.numpy().reshape(-1)

    layers, raw = [], []
    for l in range(LAYERS):
        ws = {n: qt(500 + 10 * l + i, dt, N, K) for i, (n, dt, N, K) in enumerate(
            [("q", ops.Q4_K, NH * D, H), ("k", ops.Q4_K, KH * D, H), ("v", ops.Q4_K, KH * D, H), ("o", ops.Q4_K, H, NH * D),
             ("gate", ops.Q4_K, F, H), ("up", ops.Q4_K, F, H), ("down", ops.Q6_K, H, F)])}
        g = torch.Generator().manual_seed(600 + l)
        an, fn = 1 + 0.1 * torch.randn(H, generator=g), 1 + 0.1 * torch.randn(H, generator=g)
        layers.append(decode.LlamaLayer(*[ws[n][0] for n in ("q", "k", "v", "o", "gate", "up", "down")], an.to(cuda), fn.to(cuda)))
        raw.append(({n: ws[n][1] for n in ws}, an.numpy(), fn.numpy()))
    on = 1 + 0.1 * torch.randn(H, generator=torch.Generator().manual_seed(700))
    head, head_raw = qt(701, ops.Q6_K, V, H)
    return layers, raw, on, head, head_raw


def _oracle_steps(oracle, raw, on, head_raw, first_token, n_steps):
    """Greedy decode on the CPU: returns the logits of every step and the tokens chosen."""
    shapes = {"q": (ops.Q4_K, NH * D, H), "k": (ops.Q4_K, KH * D, H), "v": (ops.Q4_K, KH * D, H), "o": (ops.Q4_K, H, NH * D),
              "gate": (ops.Q4_K, F, H), "up": (ops.Q4_K, F, H), "down": (ops.Q6_K, H, F)}
    kb = [np.zeros((1, KH, CAP, D), np.float32) for _ in raw]
    vb = [np.zeros((1, KH, CAP, D), np.float32) for _ in raw]
    table = oracle.dequant(ops.Q6_K, head_raw, V * H).reshape(V, H)      # tied embedding: the lm_head rows
    tok, logits_all, toks = first_token, [], []
    mm = lambda name, w, x: oracle.matmul_q(shapes[name][0], x.reshape(1, -1).astype(np.float32), w[name], shapes[name][1])  # noqa: E731
    for pos in range(n_steps):
        h = table[tok].astype(np.float32).copy()
        down = None
        for l, (w, an, fn) in enumerate(raw):
            s = h if down is None else h + down
            y = oracle.rmsnorm(s.reshape(1, -1), an, 1e-5)
            q, k, v = mm("q", w, y), mm("k", w, y), mm("v", w, y)
            pp = np.array([pos], np.int64)
            q = oracle.rope(q.reshape(NH, 1, D), pp, 500000.0).reshape(1, NH, 1, D)
            k = oracle.rope(k.reshape(KH, 1, D), pp, 500000.0).reshape(1, KH, 1, D)
            oracle.kv_append(kb[l], vb[l], k, v.reshape(1, KH, 1, D), pos)
            a = oracle.decode_attn(q, kb[l], vb[l], pos, 1.0 / math.sqrt(D))
            o = mm("o", w, a.reshape(1, -1))
            s2 = s + o.reshape(-1)
            y2 = oracle.rmsnorm(s2.reshape(1, -1), fn, 1e-5)
            gl, ul = mm("gate", w, y2).reshape(-1).astype(np.float64), mm("up", w, y2).reshape(-1).astype(np.float64)
            act = (gl / (1 + np.exp(-gl)) * ul).astype(np.float32)
            down = mm("down", w, act).reshape(-1)
            h = s2
        y = oracle.rmsnorm((h + down).reshape(1, -1), on.numpy(), 1e-5)
        logits = oracle.matmul_q(ops.Q6_K, y, head_raw, V).reshape(-1)
        logits_all.append(logits)
        tok = int(np.argmax(logits))
        toks.append(tok)
    return logits_all, toks


@pytest.mark.parametrize("fold", [True, False])
def test_decode_graph_matches_the_oracle(cuda, oracle, fold):
    layers, raw, on, head, head_raw = _model(cuda)
    cfg = decode.LlamaConfig(hidden=H, n_heads=NH, n_kv_heads=KH, head_dim=D)
    n_steps, first = 6, 17
    want_logits, want_toks = _oracle_steps(oracle, raw, on, head_raw, first, n_steps)
    g = decode.DecodeGraph(cfg, layers, on.to(cuda), head, head, CAP, cuda, fold_norms=fold)
    g.reset(first, 0)
    got = []
    for i in range(n_steps):              # eager
        g.step()
        torch.cuda.synchronize()
        assert rel_l2(g.logits.cpu().numpy().reshape(-1), want_logits[i]) <= 1e-3, (fold, i)
        got.append(int(g.token.item()))
    assert got == want_toks
    assert int(g.pos.item()) == n_steps
    # the same sequence replayed from a CUDA graph, on fresh caches
    g2 = decode.DecodeGraph(cfg, layers, on.to(cuda), head, head, CAP, cuda, fold_norms=fold)
    g2.reset(first, 0)
    g2.capture()
    assert int(g2.token.item()) == first and int(g2.pos.item()) == 0
    toks = g2.generate(n_steps).cpu().tolist()
    assert toks == want_toks
    assert rel_l2(g2.logits.cpu().numpy().reshape(-1), want_logits[-1]) <= 1e-3
    assert ops.decode_attn_status(0) == 0
