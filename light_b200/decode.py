"""The decode step of a Llama-shaped GGUF model as a replayable graph: the place the reference's
models.DecodeGraph holds (models/decode_graph.go:27-230 captures one forward of models/llama.go:1070-1330 and replays
it per token; engine/engine.go:419-565 samples on the device so the token id never visits the host).

    per layer:  add + RMSNorm -> q,k,v (one launch) -> RoPE + KV append + attention (one launch) -> o
                -> add + RMSNorm -> SiLU(gate) * up (one launch) -> down
    then:       add + RMSNorm -> lm_head -> argmax; the next step starts from the embedding row of that token

Every operator is one of this library's C-ABI entry points; with `fold_norms` the RMSNorm (and the residual add
before it) runs inside the q,k,v and gate,up launches (light_b200_matmul_q_fused).  One sequence, one token per
step, F32 activations and KV cache (what the GGUF path of the reference uses, nn/linear.go:214-217).
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from typing import List, Optional

import torch

from . import _lib, ops
from .ops import QTensor


@dataclass
class LlamaLayer:
    """The quantized linears and norm weights of one decoder layer (models/llama.go:40-75)."""
    q: QTensor
    k: QTensor
    v: QTensor
    o: QTensor
    gate: QTensor
    up: QTensor
    down: QTensor
    attn_norm: torch.Tensor
    ffn_norm: torch.Tensor


@dataclass
class LlamaConfig:
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    rope_base: float = 500000.0
    eps: float = 1e-5


class DecodeGraph:
    """One decode step, captured once and replayed per token.

        g = DecodeGraph(cfg, layers, output_norm, lm_head, embedding, kv_capacity, device)
        g.reset(first_token, position=0)
        g.capture()                 # records the step into a CUDA graph (models/decode_graph.go:58-176)
        for _ in range(n): g.step() # one replay per token; g.token holds the sampled id (device I64)
    """

    def __init__(self, cfg: LlamaConfig, layers: List[LlamaLayer], output_norm: torch.Tensor, lm_head: QTensor, embedding: QTensor,
                 kv_capacity: int, device: torch.device, fold_norms: bool = True):
        self.cfg, self.layers, self.device, self.fold_norms = cfg, layers, device, fold_norms
        self.dev_index = device.index if device.index is not None else torch.cuda.current_device()
        self.output_norm, self.lm_head, self.embedding = output_norm, lm_head, embedding
        H, NH, KH, D = cfg.hidden, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
        if NH * D != layers[0].q.shape[0] or KH * D != layers[0].k.shape[0] or layers[0].q.shape[1] != H:
            raise ValueError("DecodeGraph: layer shapes do not match the configuration")
        z = lambda *s: torch.zeros(*s, device=device)  # noqa: E731
        self.vocab = lm_head.shape[0]
        self.h, self.h2, self.xn = z(1, H), z(1, H), z(1, H)
        self.q, self.k, self.v = z(1, NH * D), z(1, KH * D), z(1, KH * D)
        self.attn, self.o, self.act, self.down = z(1, NH, 1, D), z(1, H), z(1, layers[0].gate.shape[0]), z(1, H)
        self.logits = z(1, self.vocab)
        self.token = torch.zeros(1, dtype=torch.int64, device=device)
        self.pos = torch.zeros(1, dtype=torch.int64, device=device)
        self.kbuf = [z(1, KH, kv_capacity, D) for _ in layers]
        self.vbuf = [z(1, KH, kv_capacity, D) for _ in layers]
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        P = lambda t: t.data_ptr()  # noqa: E731
        self._attn_args = [_lib.DecodeAttnArgs(P(self.q), P(self.kbuf[l]), P(self.vbuf[l]), P(self.k), P(self.v), P(self.pos), P(self.attn),
                                               ops.F32, 1, NH, KH, kv_capacity, D, 0, 1.0 / math.sqrt(D), cfg.rope_base) for l in range(len(layers))]
        self._qkv = [((C.c_void_p * 3)(P(L.q.data), P(L.k.data), P(L.v.data)), (C.c_void_p * 3)(P(self.q), P(self.k), P(self.v)),
                      (C.c_int32 * 3)(L.q.shape[0], L.k.shape[0], L.v.shape[0])) for L in layers]
        self._gu = [((C.c_void_p * 2)(P(L.gate.data), P(L.up.data)), (C.c_void_p * 2)(P(self.act), P(self.act)),
                     (C.c_int32 * 2)(L.gate.shape[0], L.up.shape[0])) for L in layers]
        # norms folded into the q,k,v and gate,up launches: the residual stream alternates between two buffers,
        # because the launch that writes the new sum is still reading the old one
        self._folded, cur, other = [], self.h, self.h2
        for l, L in enumerate(layers):
            if l == 0:
                first = (cur, _lib.NormArgs(P(L.attn_norm), None, None, cfg.eps))
            else:
                first = (cur, _lib.NormArgs(P(L.attn_norm), P(self.down), P(other), cfg.eps))
                cur, other = other, cur
            second = (cur, _lib.NormArgs(P(L.ffn_norm), P(self.o), P(other), cfg.eps))
            cur, other = other, cur
            self._folded.append((first, second))
        self._last_h = cur
        self.launches_per_step = (5 if fold_norms else 7) * len(layers) + 4

    def reset(self, token: int, position: int = 0) -> None:
        """Starts a sequence: the token to feed next and the position it will take in the cache."""
        self.token.fill_(int(token))
        self.pos.fill_(int(position))

    def _st(self):
        return C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def forward(self) -> None:
        """Enqueues one step on the current stream: embedding row of `token` -> ... -> logits -> argmax into `token`,
        position advanced by one.  No host synchronisation, no allocation."""
        L, st, d, cfg = _lib.lib(), self._st(), self.dev_index, self.cfg
        P = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
        H = cfg.hidden
        _lib.check(L.light_b200_embedding_q(self.embedding.ggml_type, P(self.embedding.data), P(self.token), P(self.h), 1, self.embedding.shape[0], H, d, st))
        for l, lay in enumerate(self.layers):
            if self.fold_norms and lay.q.ggml_type == ops.Q4_K and lay.gate.ggml_type == ops.Q4_K:
                (x1, n1), (x2, n2) = self._folded[l]
                wp, op, nn = self._qkv[l]
                _lib.check(L.light_b200_matmul_q_fused(ops.Q4_K, P(x1), C.byref(n1), wp, op, nn, 3, 0, H, d, st))
                _lib.check(L.light_b200_decode_attn(C.byref(self._attn_args[l]), d, st))
                _lib.check(L.light_b200_matmul_q(lay.o.ggml_type, P(self.attn), P(lay.o.data), P(self.o), 1, lay.o.shape[0], lay.o.shape[1], d, st))
                wp, op, nn = self._gu[l]
                _lib.check(L.light_b200_matmul_q_fused(ops.Q4_K, P(x2), C.byref(n2), wp, op, nn, 2, 1, H, d, st))
                _lib.check(L.light_b200_matmul_q(lay.down.ggml_type, P(self.act), P(lay.down.data), P(self.down), 1, lay.down.shape[0], lay.down.shape[1], d, st))
            else:
                if not self.fold_norms:
                    _lib.check(L.light_b200_rmsnorm(P(self.h), P(self.down) if l else None, P(lay.attn_norm), P(self.h) if l else None, P(self.xn), ops.F32, 1, H,
                                                    cfg.eps, d, st))
                else:
                    raise ValueError("DecodeGraph: fold_norms needs Q4_K q,k,v and gate,up weights")
                wp, op, nn = self._qkv[l]
                _lib.check(L.light_b200_matmul_q_multi(lay.q.ggml_type, P(self.xn), wp, op, nn, 3, H, d, st))
                _lib.check(L.light_b200_decode_attn(C.byref(self._attn_args[l]), d, st))
                _lib.check(L.light_b200_matmul_q(lay.o.ggml_type, P(self.attn), P(lay.o.data), P(self.o), 1, lay.o.shape[0], lay.o.shape[1], d, st))
                _lib.check(L.light_b200_rmsnorm(P(self.h), P(self.o), P(lay.ffn_norm), P(self.h), P(self.xn), ops.F32, 1, H, cfg.eps, d, st))
                rc = L.light_b200_matmul_q_gated(lay.gate.ggml_type, P(self.xn), P(lay.gate.data), P(lay.up.data), P(self.act), lay.gate.shape[0], H, 1, d, st)
                if rc != 0:  # no fused gate for this format: the unfused sequence, as the reference runs it
                    g = ops.MatMulQ(self.xn, lay.gate)
                    u = ops.MatMulQ(self.xn, lay.up)
                    self.act.copy_(torch.nn.functional.silu(g) * u)
                _lib.check(L.light_b200_matmul_q(lay.down.ggml_type, P(self.act), P(lay.down.data), P(self.down), 1, lay.down.shape[0], lay.down.shape[1], d, st))
        last = self._last_h if self.fold_norms else self.h
        _lib.check(L.light_b200_rmsnorm(P(last), P(self.down), P(self.output_norm), P(self.xn) if self.fold_norms else P(self.h), P(self.xn), ops.F32, 1, H,
                                        cfg.eps, d, st))
        _lib.check(L.light_b200_matmul_q(self.lm_head.ggml_type, P(self.xn), P(self.lm_head.data), P(self.logits), 1, self.vocab, H, d, st))
        _lib.check(L.light_b200_argmax(P(self.logits), P(self.token), 1, self.vocab, d, st))
        _lib.check(L.light_b200_inc_i64(P(self.pos), 1, d, st))

    def capture(self) -> None:
        """Warm up on a side stream, then record forward() into a CUDA graph (models/decode_graph.go:58-176).  The
        warm-up steps are undone: token, position and the cache rows they wrote are restored."""
        tok, pos = self.token.clone(), self.pos.clone()
        s = torch.cuda.Stream(self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(s):
            for _ in range(2):
                self.token.copy_(tok)
                self.pos.copy_(pos)
                self.forward()
        torch.cuda.current_stream(self.device).wait_stream(s)
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        self.token.copy_(tok)
        self.pos.copy_(pos)
        with torch.cuda.graph(g):
            self.forward()
        self.token.copy_(tok)
        self.pos.copy_(pos)
        torch.cuda.synchronize(self.device)
        self.graph = g

    def step(self) -> None:
        """One token: a graph replay when captured (DecodeGraph.Step, models/decode_graph.go:178-205), else eager."""
        if self.graph is not None:
            self.graph.replay()
        else:
            self.forward()

    def generate(self, n: int) -> torch.Tensor:
        """n greedy tokens after the current one; returns them as a device I64 tensor (one synchronisation at the end)."""
        out = torch.empty(n, dtype=torch.int64, device=self.device)
        for i in range(n):
            self.step()
            out[i:i + 1].copy_(self.token)
        return out
