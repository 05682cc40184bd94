"""Host side of the persistent decode chain (light_b200_chain_*): a program of dependent one-row quantized
matrix-vector products -- q,k,v -> o -> gate,up -> down -> ... -> lm_head -- executed by ONE launch per step.

It stands where the reference's models.DecodeGraph stands (models/decode_graph.go:27-230: the decode step
captured once, replayed per token): `DecodeChain` is built once from the operators of a step and `run()` is
the replay.  The reference's graph holds one kernel per operator; here the operators' dependencies are carried
by tagged slots inside one kernel (csrc/decode_chain.cu).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from . import _lib
from .ops import QTensor, _dev


ChainOp = _lib.ChainOp


def _declare(lib):
    """(argtypes come from _lib.SYMBOLS)"""


class DecodeChain:
    """Collects the operators of a decode step, builds the device program, replays it.

        c = DecodeChain(device)
        v_q = c.vec()                                   # a chain vector: handed from operator to operator
        c.matmul([wq, wk, wv], x=h, outs=[q, k, v], out_vecs=[v_q, None, None])
        v_o = c.vec()
        c.matmul([wo], x_vec=v_q, out_vecs=[v_o])
        ...
        c.build(); c.run()                              # run() is stream-ordered and graph-capturable

    Row-split over several GPUs: pass world / rank and, to build(), every rank's arena address (symmetric memory);
    arena_bytes() says how large each must be.
    """

    def __init__(self, device: torch.device, world: int = 1, rank: int = 0):
        self.device, self.world, self.rank = device, world, rank
        self.dev_index = device.index if device.index is not None else torch.cuda.current_device()
        self.ops: list[ChainOp] = []
        self._keep = []
        self.n_vecs = 0
        self.program = None
        _declare(_lib.lib())

    def vec(self) -> int:
        self.n_vecs += 1
        return self.n_vecs - 1

    def matmul(self, ws: Sequence[QTensor], x: Optional[torch.Tensor] = None, x_vec: Optional[int] = None,
               outs: Optional[Sequence[Optional[torch.Tensor]]] = None, out_vecs: Optional[Sequence[Optional[int]]] = None, act: int = 0,
               norm_weight: Optional[torch.Tensor] = None, eps: float = 0.0, res_vec: Optional[int] = None,
               sum_vec: Optional[int] = None) -> None:
        """One operator: out[i] = dequant(ws[i]) . y (or, with act 1 / 2, out[0] = act(ws[0] . y) * (ws[1] . y)),
        y from plain `x` or chain vector `x_vec`, optionally RMS-normalised after adding chain vector res_vec."""
        if not 1 <= len(ws) <= 4:
            raise ValueError(f"DecodeChain.matmul: {len(ws)} weights, want 1..4")
        if (x is None) == (x_vec is None):
            raise ValueError("DecodeChain.matmul: give exactly one of x (plain activations) and x_vec (a chain vector)")
        K = ws[0].shape[1]
        o = ChainOp()
        o.wtype, o.K, o.count, o.act = ws[0].ggml_type, K, len(ws), act
        n_out = 1 if act else len(ws)
        outs = list(outs) if outs is not None else [None] * n_out
        out_vecs = list(out_vecs) if out_vecs is not None else [None] * n_out
        for i, w in enumerate(ws):
            if len(w.shape) != 2 or w.shape[1] != K or w.ggml_type != ws[0].ggml_type or w.device != self.device:
                raise ValueError(f"DecodeChain.matmul: weight {i} must be (N, {K}) of ggml type {ws[0].ggml_type} on {self.device}")
            o.w[i], o.n[i] = w.data.data_ptr(), w.shape[0]
            o.out[i], o.out_vec[i] = None, -1
        for i in range(n_out):
            if outs[i] is not None:
                t = outs[i]
                if t.dtype != torch.float32 or t.numel() != ws[i].shape[0] or not t.is_contiguous() or t.device != self.device:
                    raise ValueError(f"DecodeChain.matmul: out[{i}] must be {ws[i].shape[0]} contiguous F32 values on {self.device}")
                o.out[i] = t.data_ptr()
            if out_vecs[i] is not None:
                o.out_vec[i] = out_vecs[i]
        if x is not None:
            if x.dtype != torch.float32 or x.numel() != K or not x.is_contiguous() or x.device != self.device:
                raise ValueError(f"DecodeChain.matmul: x must be {K} contiguous F32 values on {self.device}")
            o.x, o.x_vec = x.data_ptr(), -1
        else:
            o.x, o.x_vec = None, x_vec
        o.res_vec = -1 if res_vec is None else res_vec
        o.sum_vec = -1 if sum_vec is None else sum_vec
        if norm_weight is not None:
            if norm_weight.dtype != torch.float32 or norm_weight.numel() != K or norm_weight.device != self.device:
                raise ValueError(f"DecodeChain.matmul: norm weight must be {K} F32 values on {self.device}")
            o.norm_weight, o.norm_eps = norm_weight.data_ptr(), eps
        else:
            o.norm_weight, o.norm_eps = None, 0.0
        self._keep.append((ws, outs, x, norm_weight))
        self.ops.append(o)

    def _array(self):
        arr = (ChainOp * len(self.ops))()
        for i, o in enumerate(self.ops):
            arr[i] = o
        return arr

    def arena_bytes(self) -> int:
        n = _lib.lib().light_b200_chain_arena_bytes(self._array(), len(self.ops), self.n_vecs, self.world)
        if n < 0:
            raise ValueError("DecodeChain: a chain vector is written with two different lengths or its index is out of range")
        return int(n)

    def build(self, arenas: Optional[Sequence[int]] = None, arena: Optional[torch.Tensor] = None) -> None:
        """arenas: device address of every rank's arena (world entries, peer-addressable); world == 1: omitted,
        the arena is allocated here."""
        L = _lib.lib()
        nbytes = self.arena_bytes()
        if arenas is None:
            if self.world != 1:
                raise ValueError("DecodeChain.build: with world > 1 pass every rank's arena address")
            self.arena = torch.zeros(nbytes + 256, dtype=torch.uint8, device=self.device)
            base = self.arena.data_ptr()
            arenas = [base + (-base) % 256]
        else:
            self.arena = arena
        pb = L.light_b200_chain_program_bytes(len(self.ops))
        self.program_buf = torch.zeros(pb + 256, dtype=torch.uint8, device=self.device)
        p0 = self.program_buf.data_ptr()
        self.program = p0 + (-p0) % 256
        self.step = torch.zeros(1, dtype=torch.int32, device=self.device)
        ap = (C.c_void_p * self.world)(*arenas)
        st = C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        _lib.check(L.light_b200_chain_build(self._array(), len(self.ops), self.n_vecs, C.c_void_p(self.program), pb, ap, nbytes, self.world,
                                            self.rank, self.dev_index, st))
        torch.cuda.synchronize(self.device)

    def run(self) -> None:
        """One pass over the program on torch's current stream (two launches; graph-capturable)."""
        if self.program is None:
            raise RuntimeError("DecodeChain.run: build() first")
        st = C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        _lib.check(_lib.lib().light_b200_chain_run(C.c_void_p(self.program), C.c_void_p(self.step.data_ptr()), self.dev_index, st))

    def status(self) -> int:
        """0, or 1 if a bounded wait inside the kernel ever gave up on this device (synchronises)."""
        return _lib.lib().light_b200_chain_status(self.dev_index)
