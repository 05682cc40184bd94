#!/usr/bin/env python
"""Benchmark of the quantized-weight matmul path: Llama-3-8B-shape decode at GGUF Q4_K_M.

One step = one decode step's worth of quantized linears for M tokens: 32 layers x
{q, k, v, o, gate, up as Q4_K; down as Q6_K} plus the Q6_K lm_head, 225 fused dequant-matmuls
reading 4.84 GB of block-quantized weights once.  At M = 1 the q/k/v trio and the gate/up pair,
which share their input row, go out as one launch each (matmul_q_multi: 129 launches per step);
--launches single issues all 225 separately.  Weights are random-init from a seed
(N(0, 0.02) before quantization) directly in HBM; activations are N(0, 1).

    python bench.py --gpus N --steps K --warmup W            # this library, rank-per-GPU
    python bench.py --impl reference ...                     # the CPU port of the reference path

Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import math
import os
import statistics
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from light_b200 import _lib, ops, synth  # noqa: E402

HID, FFN, NKV, VOCAB, LAYERS = 4096, 14336, 1024, 128256, 32
# (name, N, K, ggml type) of one decoder layer's linears, in call order
LAYER = [("q", HID, HID, ops.Q4_K), ("k", NKV, HID, ops.Q4_K), ("v", NKV, HID, ops.Q4_K), ("o", HID, HID, ops.Q4_K),
         ("gate", FFN, HID, ops.Q4_K), ("up", FFN, HID, ops.Q4_K), ("down", HID, FFN, ops.Q6_K)]
HEAD = ("lm_head", VOCAB, HID, ops.Q6_K)
# DRAM traffic of the Q4_K decode kernel per algorithmic byte: dram__bytes_read + dram__bytes_write over the
# algorithmic bytes of the three launches of one ncu capture of this kernel on one layer's shapes (every weight
# byte is fetched once).  A constant of the kernel as it stands: it has to be captured again when the kernel changes.
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = 89.78 / 89.86


def weight_bytes(N, K, dt):
    return N * synth.row_bytes(dt, K)


def algorithmic_bytes(N, K, dt, M):
    """weights once + activations in + outputs out."""
    return weight_bytes(N, K, dt) + M * K * 4 + M * N * 4


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with NVML while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._t = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            try:
                uuid = "GPU-" + str(torch.cuda.get_device_properties(index).uuid)
                self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                get = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
                r = get(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.005)

    def __enter__(self):
        if self.nv:
            self._t = threading.Thread(target=self._run, daemon=True)
            self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._t:
            self._t.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["nvml unavailable"]}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


class Chain:
    """The quantized linears of one decode step on one GPU, each weight row-split over `world` ranks."""

    # Linears that share their input row and are issued as ONE launch at M = 1, as the reference's
    # decode step does for BF16 weights (ops.LinearMulti for q/k/v, models/llama.go:1085; gate and
    # up, models/llama.go:1300): keyed by the first member's name.
    GROUPS = {"q": ("q", "k", "v"), "gate": ("gate", "up")}

    def __init__(self, device, M, rank=0, world=1, layers=LAYERS, seed=0, share=None, fused=True):
        self.device, self.M, self.rank, self.world = device, M, rank, world
        self.fused = fused and M <= 64  # q,k,v and gate,up as one launch each: one row, or the batched-decode kernels (2 .. 64 rows)
        self._multi = {}
        self.lin = []  # (name, N_local, N, K, dt, weight bytes tensor)
        if share is not None:  # same weights, another token count
            self.lin = share.lin
        else:
            for l in range(layers):
                for i, (name, N, K, dt) in enumerate(LAYER):
                    self.lin.append(self._make(f"l{l}.{name}", N, K, dt, seed * 100003 + l * 16 + i))
            self.lin.append(self._make(*HEAD, seed * 100003 + 99991))
        g = torch.Generator(device=device)
        g.manual_seed(seed + 7)
        self.x = {HID: torch.randn(M, HID, generator=g, device=device), FFN: torch.randn(M, FFN, generator=g, device=device)}
        self.out = [torch.empty(M, e[2], device=device) for e in self.lin]  # full-width outputs (gathered when world > 1)
        self.local = [torch.empty(M, e[1], device=device) for e in self.lin] if world > 1 else self.out
        self.dev_index = device.index or 0
        if M > 1:  # the batched-decode kernels stage x and keep their split-K partial sums in the library's workspace
            ops.ensure_workspace(self.dev_index, int(_lib.lib().light_b200_matmul_q_workspace_bytes(M, FFN)))
        self.peer, self.fx, self.dc, self.gather_kind = None, None, None, "none"
        self.attn = None
        if world > 1:
            from light_b200 import tp

            self.gidx = [i for i, e in enumerate(self.lin) if e[0].split(".")[-1] in self.GATHERED]
            self.gather_kind = "nccl"
            mode = os.environ.get("LIGHT_B200_TP_GATHER", "fused")
            if mode in ("chain", "fused", "peer"):
                try:
                    in_chain = mode == "chain" and self.fused and M == 1  # the whole step as one persistent launch per rank
                    fused = (mode == "fused" or in_chain) and self.fused and M == 1  # the in-launch exchange serves one activation row
                    pidx = [i for i in self.gidx if not fused or self.lin[i][0] == HEAD[0]]  # gathered by the gather kernel
                    self.peer = tp.PeerGather(device)
                    outs = self.peer.plan([(M, self.lin[i][2]) for i in pidx])
                    for j, i in enumerate(pidx):
                        self.out[i] = outs[j]
                    self.pidx = pidx
                    self.gather_kind = "peer"
                    if in_chain:
                        self._plan_chain(tp)
                        self.gather_kind = "inside one persistent launch per rank (tagged slots stored into every rank's arena; logits: peer-store gather kernel)"
                    elif fused:
                        self._plan_fused(tp)
                        self.gather_kind = "fused into the matmul launches (logits: peer-store gather kernel)"
                except Exception as e:  # noqa: BLE001  (no peer mapping on this box: NCCL does the gathers)
                    print(f"[bench] peer-memory exchange unavailable ({type(e).__name__}: {e}); using NCCL", file=sys.stderr)
                    self.peer, self.fx = None, None
                    self.gather_kind = "nccl"

    def _plan_fused(self, tp):
        """Receive buffers and per-launch arguments of the in-launch exchange: every launch but the first
        takes its activations from the exchanged output before it (a real dependent chain: q -> o -> gate ->
        down -> next layer's q ... -> lm_head), the logits are gathered by the gather kernel."""
        fidx = [i for i in self.gidx if self.lin[i][0] != HEAD[0]]
        fx = tp.FusedExchange(self.device)
        fx.plan([self.lin[i][2] for i in fidx])
        self.launch_args, prev = [], None
        for idx in self.plan():
            K = self.lin[idx[0]][3]
            x_from = prev if prev is not None and self.lin[fidx[prev]][2] == K else None
            outs_to = [fidx.index(i) if i in fidx else None for i in idx]
            n = len(idx)
            self.launch_args.append((fx.args(x_from, outs_to), x_from is None,
                                     (C.c_void_p * n)(*[self.lin[i][5].data_ptr() for i in idx]),
                                     (C.c_void_p * n)(*[self.local[i].data_ptr() for i in idx]),
                                     (C.c_int32 * n)(*[self.lin[i][1] for i in idx])))
            for o in outs_to:
                if o is not None:
                    prev = o
        self.fx = fx

    def _plan_chain(self, tp):
        """The same dependent chain (q -> o -> gate -> down -> next layer's q ... -> lm_head) as ONE persistent launch
        per rank (light_b200_chain_*): every exchanged output is a chain vector in symmetric memory that all ranks
        store their rows into; the logits stay row-local and are gathered by the gather kernel."""
        from light_b200 import chain as lbchain

        dc = lbchain.DecodeChain(self.device, world=self.world, rank=self.rank)
        vecs = {n: dc.vec() for n in ("q", "o", "gate", "down")}
        prev = None
        for idx in self.plan():
            names = [self.lin[i][0].split(".")[-1] for i in idx]
            K, dt = self.lin[idx[0]][3], self.lin[idx[0]][4]
            ws = [ops.QTensor(self.lin[i][5].reshape(-1), dt, (self.lin[i][1], K)) for i in idx]
            outs = [self.local[i].reshape(-1) for i in idx]
            out_vecs = [vecs.get(n) for n in names]
            kw = dict(x=self.x[K].reshape(-1)) if prev is None or prev[1] != K else dict(x_vec=prev[0])
            dc.matmul(ws, outs=outs, out_vecs=out_vecs, **kw)
            for n, i in zip(names, idx):
                if n in vecs:
                    prev = (vecs[n], self.lin[i][2])
        tp.build_chain_symmetric(dc)
        self.dc = dc

    def enable_attention(self, kv_len=1024):
        """Adds the decode-step attention of configs[1] (32 query / 8 KV heads of dim 128, KV length
        kv_len, f32 cache, one sequence per activation row) after every layer's q,k,v launch: one
        light_b200_decode_attn launch that appends the new k, v at the last position and attends."""
        assert self.world == 1
        NHQ, NHK, HD = 32, NKV // 128, 128
        by = {e[0]: i for i, e in enumerate(self.lin)}
        self.pos = torch.tensor([kv_len - 1], dtype=torch.int64, device=self.device)
        self.attn, self.attn_bytes = {}, 0
        g = torch.Generator(device=self.device)
        g.manual_seed(11)
        for l in range(sum(1 for e in self.lin if e[0].endswith(".q"))):
            kb = torch.randn(self.M, NHK, kv_len, HD, generator=g, device=self.device)
            vb = torch.randn(self.M, NHK, kv_len, HD, generator=g, device=self.device)
            out = torch.empty(self.M, NHQ, 1, HD, device=self.device)
            q, k, v = (self.out[by[f"l{l}.{n}"]] for n in ("q", "k", "v"))
            a = _lib.DecodeAttnArgs(q.data_ptr(), kb.data_ptr(), vb.data_ptr(), k.data_ptr(), v.data_ptr(), self.pos.data_ptr(),
                                    out.data_ptr(), ops.F32, self.M, NHQ, NHK, kv_len, HD, 0, 1.0 / math.sqrt(HD))
            self.attn[by[f"l{l}.v"]] = (a, kb, vb, out)  # issued after the launch that produces v
            self.attn_bytes += 2 * kb.numel() * 4

    def _make(self, name, N, K, dt, seed):
        assert N % self.world == 0
        nl = N // self.world
        # every rank draws only its own rows (a row split is a byte slice of the block layout)
        w = synth.gaussian_weight(seed * 8 + self.rank, dt, nl, K, device=self.device)
        return (name, nl, N, K, dt, w)

    def launch(self, i, stream):
        name, nl, N, K, dt, w = self.lin[i]
        _lib.check(_lib.lib().light_b200_matmul_q(dt, C.c_void_p(self.x[K].data_ptr()), C.c_void_p(w.data_ptr()),
                                                  C.c_void_p(self.local[i].data_ptr()), self.M, nl, K, self.dev_index,
                                                  C.c_void_p(stream)))

    def launch_multi(self, idx, stream):
        """The linears idx (same x, same type) in one matmul_q_multi launch."""
        key = idx[0]
        if key not in self._multi:
            n = len(idx)
            self._multi[key] = ((C.c_void_p * n)(*[self.lin[i][5].data_ptr() for i in idx]),
                                (C.c_void_p * n)(*[self.local[i].data_ptr() for i in idx]),
                                (C.c_int32 * n)(*[self.lin[i][1] for i in idx]))
        wp, op, nn = self._multi[key]
        _, _, _, K, dt, _ = self.lin[key]
        _lib.check(_lib.lib().light_b200_matmul_q_multi_rows(dt, C.c_void_p(self.x[K].data_ptr()), wp, op, nn, len(idx), self.M, K,
                                                             self.dev_index, C.c_void_p(stream)))

    def plan(self, only=None):
        """The launches of one step: lists of indices into self.lin, one list per launch."""
        out, i = [], 0
        while i < len(self.lin):
            e = self.lin[i]
            if only is not None and e[4] != only:
                i += 1
                continue
            grp = self.GROUPS.get(e[0].split(".")[-1]) if self.fused else None
            k = len(grp) if grp else 1
            out.append(list(range(i, i + k)))
            i += k
        return out

    # Outputs the next operator needs in full on every rank (the rest stay row-local): the attention
    # output (q stands in for it here: k, v and the heads they feed are rank-local), o, the MLP
    # activation (gate stands in for silu(gate) * up), down, and the logits.
    GATHERED = ("q", "o", "gate", "down", "lm_head")

    def step(self, only=None):
        from light_b200 import tp

        st = torch.cuda.current_stream(self.device).cuda_stream
        n = 0
        if self.peer is not None and only is None:
            self.peer.step_begin()
        if self.fx is not None and only is None:
            self.fx.step_begin()
        if self.dc is not None and only is None:
            self.dc.run()
            n = 2
            li_head = len(self.lin) - 1
            self.peer.gather(self.pidx.index(li_head), self.local[li_head])
            return n + 1
        for li, idx in enumerate(self.plan(only)):
            if self.fx is not None and only is None:
                args, plain_x, wp, op, nn = self.launch_args[li]
                _, _, _, K, dt, _ = self.lin[idx[0]]
                _lib.check(_lib.lib().light_b200_matmul_q_tp(dt, C.c_void_p(self.x[K].data_ptr() if plain_x else 0), wp, op, nn,
                                                             len(idx), K, C.byref(args), self.dev_index, C.c_void_p(st)))
            elif len(idx) > 1:
                self.launch_multi(idx, st)
            else:
                self.launch(idx[0], st)
            n += 1
            if self.attn and only is None and idx[-1] in self.attn:
                _lib.check(_lib.lib().light_b200_decode_attn(C.byref(self.attn[idx[-1]][0]), self.dev_index, C.c_void_p(st)))
                n += 1
            for i in idx:
                if self.world > 1 and only is None and self.lin[i][0].split(".")[-1] in self.GATHERED:
                    if self.peer is not None and i in self.pidx:
                        self.peer.gather(self.pidx.index(i), self.local[i])
                    elif self.peer is None:
                        tp.all_gather_columns(self.local[i], self.out[i])
        return n

    def bytes_per_step(self, only=None):
        return sum(algorithmic_bytes(e[1], e[3], e[4], self.M) for e in self.lin if only is None or e[4] == only)

    def launches(self, only=None):
        if self.dc is not None and only is None:
            return 4  # step words of the chain and of the gather, the persistent chain kernel, the logits gather
        return len(self.plan(only))

    def reference_logits(self):
        """The same dependent chain, one launch per linear and an NCCL all-gather after every exchanged output: what
        the exchange inside the launches must reproduce."""
        from light_b200 import tp

        prev, logits = None, None
        for idx in self.plan():
            K, dt = self.lin[idx[0]][3], self.lin[idx[0]][4]
            x = self.x[K] if prev is None or prev.shape[1] != K else prev
            for i in idx:
                name = self.lin[i][0].split(".")[-1]
                y = ops.MatMulQ(x, ops.QTensor(self.lin[i][5].reshape(-1), dt, (self.lin[i][1], K)))
                if name in self.GATHERED:
                    full = tp.all_gather_columns(y)
                    if name == HEAD[0]:
                        logits = full
                    else:
                        prev = full
        return logits



def full_step_graph(chain, kv_len=1024, fold_norms=True):
    """configs[1]'s whole decode step at M = 1 on the chain's weights as a light_b200.decode.DecodeGraph (the
    counterpart of models/decode_graph.go): embedding row of the last sampled token -> 32 layers of [norm, q/k/v,
    RoPE + KV append + attention, o, norm, SiLU(gate) * up, down] -> final norm -> lm_head -> argmax.  The KV cache
    holds kv_len - 1 earlier positions (f32) and grows by one per replay."""
    from light_b200 import decode

    by = {e[0]: e for e in chain.lin}
    qt = lambda e: ops.QTensor(e[5].reshape(-1), e[4], (e[1], e[3]))  # noqa: E731
    n_layers = sum(1 for e in chain.lin if e[0].endswith(".q"))
    ones = torch.ones(HID, device=chain.device)
    layers = [decode.LlamaLayer(*[qt(by[f"l{l}.{n}"]) for n in ("q", "k", "v", "o", "gate", "up", "down")], ones, ones) for l in range(n_layers)]
    cfg = decode.LlamaConfig(hidden=HID, n_heads=32, n_kv_heads=NKV // 128, head_dim=128)
    g = decode.DecodeGraph(cfg, layers, ones, qt(by[HEAD[0]]), qt(by[HEAD[0]]), kv_len + 256, chain.device, fold_norms=fold_norms)
    gen = torch.Generator(device=chain.device)
    gen.manual_seed(21)
    for kb, vb in zip(g.kbuf, g.vbuf):   # a cache with content, as after kv_len - 1 decoded tokens
        kb[:, :, :kv_len - 1].copy_(torch.randn(1, NKV // 128, kv_len - 1, 128, generator=gen, device=chain.device))
        vb[:, :, :kv_len - 1].copy_(torch.randn(1, NKV // 128, kv_len - 1, 128, generator=gen, device=chain.device))
    g.reset(1, kv_len - 1)
    g.capture()
    return g


def capture(fn, device):
    """Warm up on a side stream, then capture fn() into a CUDA graph (as the reference's decode loop
    replays its step, models/decode_graph.go:58-205)."""
    s = torch.cuda.Stream(device)
    s.wait_stream(torch.cuda.current_stream(device))
    with torch.cuda.stream(s):
        for _ in range(2):
            fn()
    torch.cuda.current_stream(device).wait_stream(s)
    torch.cuda.synchronize(device)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    return g


def timed(replay, steps, warmup, device, barrier):
    for _ in range(warmup):
        replay()
    torch.cuda.synchronize(device)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        replay()
    e1.record()
    torch.cuda.synchronize(device)
    barrier()
    return e0.elapsed_time(e1)  # ms


def cpu_reference(M, threads, steps, warmup, budget_s=150.0):
    """The reference's CPU implementation of the path (kernels/cpu/quant_matmul.go matmulQCPU: AVX2 row
    decoders, 48-row tiles, 4x3 FMA tiles, static chunks over all host threads), as restated in
    oracle/light_oracle.c.  One step = the 225 linears of a decode step when `steps` of them fit the time
    budget; otherwise the first L of the 32 layers plus lm_head's share, and the step time is scaled by 32 / L.
    Four distinct layers' weights are rotated (551 MB: beyond the host's last-level cache).
    Returns (tok/s, seconds per whole step, seconds per timed step, layers per timed step, description)."""
    from oracle import binding as ob

    rng = np.random.Generator(np.random.Philox(5))
    xs = {HID: rng.standard_normal((M, HID)).astype(np.float32), FFN: rng.standard_normal((M, FFN)).astype(np.float32)}
    # decode time does not depend on the code values: random blocks stand in for quantized Gaussians here
    rot = [[(N, K, dt, synth.random_blocks(900 + 16 * r + i, dt, N, K)) for i, (_, N, K, dt) in enumerate(LAYER)] for r in range(4)]
    _, NH, KH, dth = HEAD
    head = synth.random_blocks(999, dth, NH, KH)

    def layers(n, first=0):
        for l in range(first, first + n):
            for N, K, dt, w in rot[l % 4]:
                ob.matmul_q(dt, xs[K], w, N, threads=threads)

    def head_rows(frac):
        n = max(48, int(NH * frac) // 48 * 48)
        ob.matmul_q(dth, xs[KH], head[:n], n, threads=threads)

    layers(1)
    t0 = time.perf_counter()
    layers(2, 1)
    t_layer = (time.perf_counter() - t0) / 2
    est_full = LAYERS * t_layer * (1 + weight_bytes(NH, KH, dth) / (LAYERS * sum(weight_bytes(N, K, dt) for _, N, K, dt in LAYER)))
    L = LAYERS if (steps + warmup) * est_full <= budget_s else max(1, min(LAYERS, int(budget_s / ((steps + warmup) * est_full) * LAYERS)))

    def step():
        layers(L)
        head_rows(L / LAYERS)

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    t_timed = (time.perf_counter() - t0) / steps
    t_step = t_timed * LAYERS / L
    what = "the whole step: 32 layers x 7 linears + lm_head (4.84 GB of weights)" if L == LAYERS else \
        f"{L} of 32 layers + {L}/32 of lm_head's rows per timed step, scaled by 32/{L}"
    return M / t_step, t_step, t_timed, L, f"{steps} timed steps of {what}; M={M}; AVX2 row decoders: {bool(ob.lib().lo_uses_avx2())}"


def extras(chain, device, args):
    """Side measurements on the same weights, reported next to the headline (not part of `value`):
    batched decode at the other token counts of configs[1], and the prefill matmuls of configs[2]."""
    out = {"decode_tokens_per_s": {}, "prefill_m2048": {}}
    steps = max(5, min(20, args.steps))
    if args.only_extra == "chain":
        return {"decode_m1_dependent_chain_one_launch": chain_kernel_extras(chain, device, steps)}
    if chain.fused:  # the same step with one launch per linear
        c = Chain(device, 1, share=chain, fused=False)
        g = capture(c.step, device)
        ms = timed(g.replay, steps, 3, device, lambda: None) / steps
        out["decode_m1_one_launch_per_linear"] = {"launches": c.launches(), "ms_per_step": ms, "tok_s": 1 / (ms * 1e-3)}
        del g, c
    for M in (8, 32, 64):
        c = Chain(device, M, share=chain)
        g = capture(c.step, device)
        ms = timed(g.replay, steps, 3, device, lambda: None) / steps
        out["decode_tokens_per_s"][str(M)] = {"ms_per_step": ms, "tok_s": M / (ms * 1e-3),
                                              "weights_gbs": c.bytes_per_step() / (ms * 1e-3) / 1e9}
        del g, c
    # the same steps with the attention of configs[1] between the q,k,v and o launches (KV length 1024, f32 cache):
    # what the linear chain leaves out of a decode step besides norms, rope and the residual adds
    out["decode_with_attention_kv1024"] = {}
    for M in (1, 8, 32, 64):
        c = Chain(device, M, share=chain, fused=chain.fused)
        c.enable_attention(1024)
        g = capture(c.step, device)
        ms = timed(g.replay, steps, 3, device, lambda: None) / steps
        base = out["decode_tokens_per_s"][str(M)]["ms_per_step"] if M > 1 else None
        out["decode_with_attention_kv1024"][str(M)] = {"ms_per_step": ms, "tok_s": M / (ms * 1e-3), "kv_bytes_per_step": c.attn_bytes,
                                                       "attention_us_per_layer": None if base is None else (ms - base) * 1e3 / len(c.attn)}
        del g, c
    if chain.world == 1 and chain.M == 1:
        logits = []
        for key, fold in (("decode_m1_full_step_kv1024", True), ("decode_m1_full_step_kv1024_norms_as_launches", False)):
            fs = full_step_graph(chain, 1024, fold)
            for _ in range(3):
                fs.step()
            torch.cuda.synchronize(device)
            fs.reset(1, 1023)
            ms = timed(fs.step, steps, 0, device, lambda: None) / steps  # a closed loop: every replay decodes the token the last one sampled
            fs.reset(1, 1023)
            fs.step()  # one step from a known token and position, for the comparison of the two variants
            torch.cuda.synchronize(device)
            out[key] = {"launches": fs.launches_per_step, "ms_per_step": ms, "tok_s": 1 / (ms * 1e-3),
                        "logits_finite": bool(torch.isfinite(fs.logits).all().item()), "sampled_token": int(fs.token.item())}
            logits.append(fs.logits.clone())
            del fs
        d = (logits[0] - logits[1]).norm() / logits[1].norm()
        out["decode_m1_full_step_kv1024"]["rel_l2_of_logits_against_norms_as_launches"] = float(d)
        out["decode_m1_full_step_kv1024"]["parity"] = "tests/test_decode_graph_gpu.py: this class against the CPU oracle, operator by operator"
    assert ops.decode_attn_status(device.index or 0) == 0
    # the Q4_K decode kernel on one matrix large enough that the cost of a launch does not matter (the vocabulary
    # projection's shape, 295 MB as Q4_K): its streaming rate, next to the launch-bound average of a step
    big = synth.gaussian_weight(4242, ops.Q4_K, VOCAB, HID, device=device)
    qt = ops.QTensor(big.reshape(-1), ops.Q4_K, (VOCAB, HID))
    xb = chain.x[HID][:1]
    ops.MatMulQ(xb, qt)
    ms = timed(lambda: ops.MatMulQ(xb, qt), 20, 3, device, lambda: None) / 20
    nbytes = algorithmic_bytes(VOCAB, HID, ops.Q4_K, 1)
    peak, _ = load_peaks()
    out["q4k_gemv_one_large_matrix"] = {"shape": [VOCAB, HID], "bytes": nbytes, "us": ms * 1e3, "gbs": nbytes / (ms * 1e-3) / 1e9,
                                        "frac_of_measured_hbm": nbytes / (ms * 1e-3) / 1e9 / peak}
    del big, qt
    # the other weight formats of the path at one activation row, on shapes of configs[3] / [4] (weights rotated so
    # that L2 does not hold them): bytes of weights (+ scales) per launch over the time of a launch
    out["other_formats_m1"] = {}
    peak, _ = load_peaks()

    def rotate(make, call, nbytes, key):
        R = max(2, min(24, int(1.0e9 // nbytes) + 1))
        ws = [make(i) for i in range(R)]
        g = capture(lambda: [call(w) for w in ws], device)
        ms = timed(g.replay, 5, 2, device, lambda: None) / 5 / R
        del g
        out["other_formats_m1"][key] = {"us": ms * 1e3, "gbs": nbytes / (ms * 1e-3) / 1e9, "frac_of_measured_hbm": nbytes / (ms * 1e-3) / 1e9 / peak}

    x4, x35, x71 = torch.randn(1, HID, device=device), torch.randn(1, 3584, device=device), torch.randn(1, 7168, device=device)
    x35b = x35.to(torch.bfloat16)
    rotate(lambda i: ops.QTensor(synth.gaussian_weight(7000 + i, ops.Q8_0, FFN, HID, device=device).reshape(-1), ops.Q8_0, (FFN, HID)),
           lambda w: ops.MatMulQ(x4, w), FFN * HID // 32 * 34, "q8_0_14336x4096")
    i4 = synth.random_int4(7100, 18944, 3584, 128)
    i4d = [torch.from_numpy(a.view(np.int32) if a.dtype == np.uint32 else a).to(device) for a in i4]
    rotate(lambda i: ops.Int4(i4d[0].clone(), i4d[1], i4d[2], 128), lambda w: ops.MatMulInt4(x35, w), 18944 * 3584 // 2 + 2 * 18944 * 28 * 4,
           "int4_g128_18944x3584_f32")
    rotate(lambda i: ops.Int4(i4d[0].clone(), i4d[1], i4d[2], 128), lambda w: ops.MatMulInt4(x35b, w),
           18944 * 3584 // 2 + 2 * 18944 * 28 * 4, "int4_g128_18944x3584_bf16")
    rotate(lambda i: synth.random_fp8_block(7200 + i, 4096, 7168, device=device), lambda w: ops.MatMulF8Block(x71, w[0], w[1], 128, 128),
           4096 * 7168 + 32 * 56 * 4, "fp8_block128_4096x7168_f32")
    # the same formats with bf16 activations at 16 rows (token tiles over activations staged once)
    x71b = torch.randn(16, 7168, device=device).to(torch.bfloat16)
    rotate(lambda i: synth.random_fp8_block(7300 + i, 18432, 7168, device=device), lambda w: ops.MatMulF8Block(x71b, w[0], w[1], 128, 128),
           18432 * 7168 + 144 * 56 * 4, "fp8_block128_18432x7168_bf16_16rows")
    M = 2048
    by = {e[0]: e for e in chain.lin}
    qkv = torch.cat([by["l0.q"][5], by["l0.k"][5], by["l0.v"][5]])          # fused rows: a byte concatenation
    gate_up = torch.cat([by["l0.gate"][5], by["l0.up"][5]])
    shapes = [("qkv", qkv, HID + 2 * NKV, HID, ops.Q4_K), ("o", by["l0.o"][5], HID, HID, ops.Q4_K),
              ("gate_up", gate_up, 2 * FFN, HID, ops.Q4_K), ("down", by["l0.down"][5], HID, FFN, ops.Q6_K)]
    for name, w, N, K, dt in shapes:
        x = torch.randn(M, K, device=device).to(torch.bfloat16).float()
        qt = ops.QTensor(w.reshape(-1), dt, (N, K))
        ops.MatMulQ(x, qt)
        ms = timed(lambda: ops.MatMulQ(x, qt), 10, 3, device, lambda: None) / 10
        out["prefill_m2048"][name] = {"ms": ms, "tflops": 2.0 * M * N * K / (ms * 1e-3) / 1e12}
    peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else {}
    if "bf16_tflops_sustained" in peaks:
        tot_f = sum(2.0 * M * N * K for _, _, N, K, _ in shapes)
        tot_t = sum(v["ms"] for v in out["prefill_m2048"].values()) * 1e-3
        out["prefill_m2048"]["all_four"] = {"tflops": tot_f / tot_t / 1e12,
                                            "frac_of_measured_sustained_bf16": tot_f / tot_t / 1e12 / peaks["bf16_tflops_sustained"]}
    out["int4_w4a16_qwen7b_shapes"] = int4_extras(device, peak, peaks)
    out["moe_fp8_deepseek_v3_layer"] = moe_extras(device, peaks)
    if chain.world == 1 and chain.M == 1:
        out["decode_m1_dependent_chain_one_launch"] = chain_kernel_extras(chain, device, steps)
    out["tensor_core_status"] = ops.prefill_status(device.index or 0)
    return out


def int4_extras(device, hbm_peak, peaks):
    """configs[3]: GPTQ / AWQ-style 4-bit weights, group 128, at Qwen2.5-7B shapes, 16-bit activations, M = 1, 16, 256 and
    4096: microseconds per call with the weights rotated through more than L2 holds, and the roofline that bounds
    each (HBM for the decode sizes, the tensor pipe for 256 and 4096 rows)."""
    res = {}
    tf_peak = peaks.get("bf16_tflops")
    for name, N, K in (("qkv_4608x3584", 4608, 3584), ("gate_up_37888x3584", 37888, 3584), ("down_3584x18944", 3584, 18944)):
        codes, s, z = synth.random_int4(7300 + N % 97, N, K, 128)
        base = [torch.from_numpy(a.view(np.int32) if a.dtype == np.uint32 else a).to(device) for a in (codes, s, z)]
        nbytes = N * K // 2 + 2 * N * (K // 128) * 4
        R = max(2, min(16, int(0.6e9 // nbytes) + 1))
        ws = [ops.Int4(base[0].clone(), base[1], base[2], 128) for _ in range(R)]
        res[name] = {}
        for M in (1, 16, 256, 4096):
            x = torch.randn(M, K, device=device).to(torch.bfloat16)
            ops.MatMulInt4(x, ws[0])
            g = capture(lambda: [ops.MatMulInt4(x, w) for w in ws], device)
            ms = timed(g.replay, 5, 2, device, lambda: None) / 5 / R
            del g
            e = {"us": ms * 1e3}
            if M <= 16:
                e["gbs"] = nbytes / (ms * 1e-3) / 1e9
                e["frac_of_measured_hbm"] = e["gbs"] / hbm_peak
            else:
                e["tflops"] = 2.0 * M * N * K / (ms * 1e-3) / 1e12
                if tf_peak:
                    e["frac_of_measured_bf16_burst"] = e["tflops"] / tf_peak
            res[name][str(M)] = e
        del ws, base
        torch.cuda.empty_cache()
    return res


def moe_extras(device, peaks):
    """configs[4] on one GPU: a DeepSeek-V3-shaped sparse block, 256 routed experts with block-scaled FP8 weights
    (128 x 128 blocks), hidden 7168, expert width 2048, 4096 bf16 tokens routed top-8 by the sigmoid + bias router
    (bias ~ N(0, 0.5): a skewed load).  Router, counting sort, grouped gate-up matmul, SiLU gate, grouped down matmul
    with the routing weights, combine: every step a launch of this library.  Needs about 12 GB; skipped with less."""
    E, H, I, T, topk, b = 256, 7168, 2048, 4096, 8, 128
    free, _ = torch.cuda.mem_get_info(device)
    if free < 16 * (1 << 30):
        return {"skipped": "needs about 12 GB of free device memory"}
    w1, s1 = synth.random_fp8_block(7401, E * 2 * I, H, b, b, device=device)
    w2, s2 = synth.random_fp8_block(7402, E * H, I, b, b, device=device)
    w1, s1 = w1.reshape(E, 2 * I, H), s1.reshape(E, 2 * I // b, H // b)
    w2, s2 = w2.reshape(E, H, I), s2.reshape(E, H // b, I // b)
    g = torch.Generator(device=device)
    g.manual_seed(7403)
    x = (torch.randn(T, H, generator=g, device=device) * 0.05).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g, device=device)
    bias = torch.randn(E, generator=g, device=device) * 0.5
    state = {}

    def layer():
        r = ops.MoERouteSigmoid(logits, bias, topk, True)
        h = ops.MoEGemmF8Block(x, w1, s1, b, b, r, None, topk)
        y = ops.MoEGemmF8Block(ops.MoEGateMul(h), w2, s2, b, b, r, r.weights, topk)
        state["out"], state["r"] = ops.MoECombine(y, topk), r

    layer()
    torch.cuda.synchronize(device)
    r = state["r"]
    cnt = torch.bincount(r.sorted_expts, minlength=E)
    ms = timed(layer, 5, 2, device, lambda: None) / 5
    M = T * topk
    hh = ops.MoEGateMul(ops.MoEGemmF8Block(x, w1, s1, b, b, r, None, topk))
    ms1 = timed(lambda: ops.MoEGemmF8Block(x, w1, s1, b, b, r, None, topk), 5, 2, device, lambda: None) / 5
    ms2 = timed(lambda: ops.MoEGemmF8Block(hh, w2, s2, b, b, r, r.weights, topk), 5, 2, device, lambda: None) / 5
    f1, f2 = 2.0 * M * 2 * I * H, 2.0 * M * H * I
    res = {"tokens": T, "pairs_per_expert_min_mean_max": [int(cnt.min()), float(cnt.float().mean()), int(cnt.max())],
           "layer_ms": ms, "tokens_per_s": T / (ms * 1e-3), "layer_tflops": (f1 + f2) / (ms * 1e-3) / 1e12,
           "gate_up_matmul": {"ms": ms1, "tflops": f1 / (ms1 * 1e-3) / 1e12}, "down_matmul": {"ms": ms2, "tflops": f2 / (ms2 * 1e-3) / 1e12},
           "finite": bool(torch.isfinite(state["out"].float()).all().item()), "route_status": ops.moe_route_status(device.index or 0)}
    if "bf16_tflops" in peaks:  # the experts are expanded to bf16 for the tensor core: the bf16 peak bounds the matmuls
        res["layer_frac_of_measured_bf16_burst"] = res["layer_tflops"] / peaks["bf16_tflops"]
    # the same block for one decode step's tokens (few pairs per expert: the warp-per-column kernel)
    xd = x[:8].contiguous()
    rd = ops.MoERouteSigmoid(logits[:8].contiguous(), bias, topk, True)

    def small():
        h = ops.MoEGemmF8Block(xd, w1, s1, b, b, rd, None, topk)
        return ops.MoECombine(ops.MoEGemmF8Block(ops.MoEGateMul(h), w2, s2, b, b, rd, rd.weights, topk), topk)

    small()
    msd = timed(small, 5, 2, device, lambda: None) / 5
    touched = 8 * topk * (2 * I * H + H * I)  # bytes of expert weights 64 pairs read (distinct experts assumed)
    res["decode_8_tokens"] = {"ms": msd, "expert_bytes": touched, "gbs": touched / (msd * 1e-3) / 1e9}
    del w1, w2, s1, s2
    torch.cuda.empty_cache()
    return res


def moe_ep_extras(device, world, rank, barrier):
    """configs[4] with its 256 experts sharded over the ranks (256 / world each): 4096 tokens in total, 4096 / world
    brought by every rank, routed top-8 by the sigmoid + bias router; tokens travel to their experts' ranks by
    all-to-all (NCCL over NVLink), run through this library's grouped block-FP8 matmuls there, travel back and are
    summed with the routing weights (light_b200.tp.ExpertParallel).  Times are CUDA events, max over ranks."""
    import torch.distributed as dist
    from light_b200 import tp

    E, H, I, T, topk, b = 256, 7168, 2048, 4096 // world, 8, 128
    if E % world:
        return {"skipped": f"256 experts do not split over {world} ranks"}
    El = E // world
    free = torch.tensor([torch.cuda.mem_get_info(device)[0]], device=device, dtype=torch.float64)
    dist.all_reduce(free, op=dist.ReduceOp.MIN)
    if float(free.item()) < El * 3 * I * H * 1.3 + (4 << 30):
        return {"skipped": "not enough free device memory for this rank's experts"}
    w1, s1 = synth.random_fp8_block(7401 + 10 * rank, El * 2 * I, H, b, b, device=device)
    w2, s2 = synth.random_fp8_block(7402 + 10 * rank, El * H, I, b, b, device=device)
    w1, s1 = w1.reshape(El, 2 * I, H), s1.reshape(El, 2 * I // b, H // b)
    w2, s2 = w2.reshape(El, H, I), s2.reshape(El, H // b, I // b)
    g = torch.Generator(device=device)
    g.manual_seed(7403 + rank)
    x = (torch.randn(T, H, generator=g, device=device) * 0.05).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g, device=device)
    gb = torch.Generator(device=device)
    gb.manual_seed(7404)  # the router bias is the layer's: the same on every rank
    bias = torch.randn(E, generator=gb, device=device) * 0.5
    ep = tp.ExpertParallel(E)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    seen = {}

    def ffn(rows, order, le):
        seen["rows"] = rows.shape[0]
        ev[0].record()
        r = ops.MoERouting(None, None, order.contiguous(), le.contiguous())
        h = ops.MoEGemmF8Block(rows, w1, s1, b, b, r, None, 1)
        y = ops.MoEGemmF8Block(ops.MoEGateMul(h), w2, s2, b, b, r, None, 1)
        ev[1].record()
        return y

    def layer():
        r = ops.MoERouteSigmoid(logits, bias, topk, True)
        seen["out"] = ep.forward(x, r.topk_ids, r.weights.reshape(T, topk), ffn, routing=r)

    layer()
    n = 5
    ms = timed(layer, n, 2, device, barrier) / n
    ms_ffn = ev[0].elapsed_time(ev[1])  # the last step's local matmuls
    t = torch.tensor([ms, ms_ffn, float(seen["rows"]), -float(seen["rows"])], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    fin = torch.tensor([float(torch.isfinite(seen["out"]).all().item()), -float(ops.moe_route_status(device.index or 0))], device=device)
    dist.all_reduce(fin, op=dist.ReduceOp.MIN)
    ms, ms_ffn = float(t[0]), float(t[1])
    flops = 2.0 * 4096 * topk * 3 * I * H
    res = {"experts_per_rank": El, "tokens_total": 4096, "tokens_per_rank": T,
           "pairs_received_per_rank_min_max": [int(-float(t[3])), int(float(t[2]))],
           "layer_ms": ms, "tokens_per_s": 4096 / (ms * 1e-3), "layer_tflops_all_ranks": flops / (ms * 1e-3) / 1e12,
           "local_matmuls_ms_slowest_rank": ms_ffn, "exchange_and_host_ms": ms - ms_ffn,
           "dispatch_bytes_per_rank": T * topk * H * 2, "combine_bytes_per_rank": T * topk * H * 2,
           "exchange": "torch.distributed.all_to_all_single (NCCL) for the rows out, the expert ids out, the results back; the split sizes of all ranks in one all-gather read once on the host; weighted slot sum as one launch",
           "finite": bool(fin[0].item() > 0), "route_status": int(-float(fin[1]))}
    del w1, w2, s1, s2
    torch.cuda.empty_cache()
    return res


def chain_kernel_extras(chain, device, steps):
    """The M = 1 step as ONE persistent launch: the 129 operators as a device-side program with the RMS norms and the
    residual adds folded in, every operator reading the vector the one before wrote (a dependent chain, unlike the
    headline's launches, which all read fixed inputs)."""
    from light_b200 import chain as dchain

    dc = dchain.DecodeChain(device)
    vq, vo, va, vd, vh = dc.vec(), dc.vec(), dc.vec(), dc.vec(), [dc.vec(), dc.vec()]
    qt = lambda e: ops.QTensor(e[5].reshape(-1), e[4], (e[2], e[3]))  # noqa: E731
    by_layer = {}
    for i, e in enumerate(chain.lin):
        by_layer.setdefault(e[0].split(".")[0], []).append(i)
    outs = {"logits": torch.empty(VOCAB, device=device)}
    nw = torch.ones(HID, device=device)
    h0 = chain.x[HID][0].contiguous()
    cur = None  # the chain vector that holds the residual stream
    for name, idx in by_layer.items():
        if name == "lm_head":
            last = vh[0] if cur == vh[1] else vh[1]
            dc.matmul([qt(chain.lin[idx[0]])], x_vec=cur, res_vec=vd, sum_vec=last, outs=[outs["logits"]], norm_weight=nw, eps=1e-5)
            continue
        q, k, v, o_, gate, up, down = [chain.lin[i] for i in idx]
        # decoder layer: norm(h + down) -> q,k,v (q stands in for the attention output) -> o -> norm(h' + o) -> act(gate) * up -> down
        if cur is None:
            dc.matmul([qt(q), qt(k), qt(v)], x=h0, out_vecs=[vq, None, None], norm_weight=nw, eps=1e-5)
            dc.matmul([qt(o_)], x_vec=vq, out_vecs=[vo])
            dc.matmul([qt(gate), qt(up)], x=h0, res_vec=vo, sum_vec=vh[1], act=1, out_vecs=[va], norm_weight=nw, eps=1e-5)
            cur = vh[1]
        else:
            other = vh[0] if cur == vh[1] else vh[1]
            dc.matmul([qt(q), qt(k), qt(v)], x_vec=cur, res_vec=vd, sum_vec=other, out_vecs=[vq, None, None], norm_weight=nw, eps=1e-5)
            dc.matmul([qt(o_)], x_vec=vq, out_vecs=[vo])
            dc.matmul([qt(gate), qt(up)], x_vec=other, res_vec=vo, sum_vec=cur, act=1, out_vecs=[va], norm_weight=nw, eps=1e-5)
        dc.matmul([qt(down)], x_vec=va, out_vecs=[vd])
    try:
        dc.build()
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"{type(e).__name__}: {e}"}
    for _ in range(3):
        dc.run()
    torch.cuda.synchronize(device)
    ms = timed(dc.run, steps, 0, device, lambda: None) / steps
    return {"operators": len(dc.ops), "launches": 2, "ms_per_step": ms, "tok_s": 1 / (ms * 1e-3), "status": dc.status(),
            "logits_finite": bool(torch.isfinite(outs["logits"]).all().item())}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="light_b200", choices=["light_b200", "reference"])
    ap.add_argument("--tokens", type=int, default=1, help="tokens per decode step (M)")
    ap.add_argument("--layers", type=int, default=LAYERS, help="decoder layers (default: the full 32)")
    ap.add_argument("--launches", default="fused", choices=["fused", "single"],
                    help="fused: q/k/v and gate/up of a layer as one launch each at M=1; single: one launch per linear")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the batched-decode and prefill side measurements")
    ap.add_argument("--only-extra", default="", help="run a single side measurement (for a small profiling case): chain")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    M = args.tokens
    metric, unit = "llama3_8b_q4_k_m_decode_tokens_per_s", "tok/s"
    workload = (f"configs[1]: Llama-3-8B-shape decoder at GGUF Q4_K_M, batched decode M={M}, the 225 quantized "
                f"linears of one step (32 x [q,k,v,o,gate,up Q4_K; down Q6_K] + Q6_K lm_head), linear chain only"
                + ("; q,k,v and gate,up of a layer issued as one launch each" if args.launches == "fused" and M == 1 else ""))

    if args.impl == "reference":
        if rank != 0:
            return 0
        threads = os.cpu_count() or 1
        v, t_step, t_timed, L, sample = cpu_reference(M, threads, args.steps, min(args.warmup, 3))
        print(json.dumps({
            "impl": "reference", "metric": metric, "value": v, "unit": unit, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": t_timed * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload},
            "cpu_baseline": {"value": v, "unit": unit, "cores": threads, "kind": "port", "sample": sample,
                             "layers_per_timed_step": L, "ms_per_whole_step": t_step * 1e3},
            "e2e": {"value": v, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }))
        return 0

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback")
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)
        barrier = lambda: dist.barrier()  # noqa: E731
    else:
        barrier = lambda: None  # noqa: E731
    _lib.check(_lib.lib().light_b200_init(local))

    chain = Chain(device, M, rank, world, layers=args.layers, fused=args.launches == "fused")
    torch.cuda.synchronize(device)
    barrier()
    launches_per_step = chain.launches()
    graph = capture(chain.step, device)

    with ClockSampler(local) as clk:
        ms = timed(graph.replay, args.steps, args.warmup, device, barrier)
    t = torch.tensor([ms], device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    ms_per_step = ms / args.steps
    value = M / (ms_per_step * 1e-3)

    # ---- roofline of the dominant kernel: the Q4_K decode GEMV, alone in a graph of its own
    peak, peak_kind = load_peaks()
    g4 = capture(lambda: chain.step(only=ops.Q4_K), device)
    ms4 = timed(g4.replay, args.steps, max(3, args.warmup), device, barrier)
    n4 = chain.launches(ops.Q4_K)
    b4 = chain.bytes_per_step(ops.Q4_K) / n4
    us4 = ms4 * 1e3 / (args.steps * n4)
    achieved = b4 / (us4 * 1e-6) / 1e9
    g6 = capture(lambda: chain.step(only=ops.Q6_K), device)
    ms6 = timed(g6.replay, args.steps, max(3, args.warmup), device, barrier)
    n6 = chain.launches(ops.Q6_K)
    gbs6 = chain.bytes_per_step(ops.Q6_K) / (ms6 * 1e-3 / args.steps) / 1e9
    roofline = {"bound": "hbm", "kernel": "q4k_gemv_mma_kernel", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "peak_source": f"of {peak_kind}", "traffic": b4 * NCU_TRAFFIC_PER_ALGORITHMIC_BYTE,
                "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of this kernel's three launch shapes on the "
                                  "1-layer case (89.78 MB) over their algorithmic bytes (89.86 MB), scaled to the mean launch",
                "bytes_per_launch": b4, "us_per_launch": us4, "launches_per_step": n4,
                "timed": "all Q4_K launches of a step in a graph of their own",
                "q6k_gemv_gbs": gbs6, "q6k_launches_per_step": n6,
                "whole_step_gbs": chain.bytes_per_step() / (ms_per_step * 1e-3) / 1e9}

    # ---- end to end: host activations in, logits out, every step
    hx = {k: v.cpu().pin_memory() for k, v in chain.x.items()}
    hlog = torch.empty(M, VOCAB).pin_memory()
    h2d = sum(v.numel() * 4 for v in hx.values())
    d2h = hlog.numel() * 4

    def e2e_step():
        for k in hx:
            chain.x[k].copy_(hx[k], non_blocking=True)
        graph.replay()
        hlog.copy_(chain.out[-1], non_blocking=True)
        torch.cuda.current_stream(device).synchronize()

    ms_e = timed(e2e_step, args.steps, max(3, args.warmup), device, barrier)
    te = torch.tensor([ms_e], device=device)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_val = M / (float(te.item()) / args.steps * 1e-3)

    line = {
        "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32 activations x Q4_K/Q6_K weights, f32 accumulate", "data": "synthetic",
        "config": {"workload": workload, "tokens_per_step": M, "layers": args.layers,
                   "weights_bytes_per_step": sum(weight_bytes(e[2], e[3], e[4]) for e in chain.lin),
                   "parallelism": f"rows of every weight split over {world} GPU(s)" + (f", all-gather ({chain.gather_kind}) of the attention output, o, the MLP activation, down and the logits (129 per step)" if world > 1 else ""),
                   "l2": "inputs (4.84 GB of weights per step) exceed the 126 MB L2", "launch": "CUDA graph replay"},
        "roofline": roofline,
        "e2e": {"value": e2e_val, "unit": unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clk.summary(),
    }
    if world == 1 and not args.no_extras:
        line["extras"] = ex = extras(chain, device, args)
        # the side measurements a reader looks for first, lifted out of `extras` (same numbers)
        line["also_measured"] = None if args.only_extra else {
            "batched_decode_tok_s": {k: round(v["tok_s"], 1) for k, v in ex["decode_tokens_per_s"].items()},
            "whole_decode_step_kv1024_tok_s": round(ex["decode_m1_full_step_kv1024"]["tok_s"], 1) if "decode_m1_full_step_kv1024" in ex else None,
            "prefill_m2048_frac_of_sustained_bf16": ex["prefill_m2048"].get("all_four", {}).get("frac_of_measured_sustained_bf16"),
        }
    if world > 1 and chain.peer is not None:
        # correctness of the exchange that was just timed: rank 0's logits against the NCCL-gathered chain
        graph.replay()
        torch.cuda.synchronize(device)
        got = chain.out[-1].clone()
        want = chain.reference_logits()
        torch.cuda.synchronize(device)
        rel = float(((got.double() - want.double()).norm() / want.double().norm()).item())  # (the chain's values grow far beyond f32's square root)
        st = chain.peer.status() | (chain.dc.status() if chain.dc is not None else 0)
        check = torch.tensor([rel, float(st)], device=device)
        dist.all_reduce(check, op=dist.ReduceOp.MAX)
        line["tp_check"] = {"rel_l2_vs_nccl_chain_max_over_ranks": float(check[0].item()), "comm_status": int(check[1].item()),
                            "finite": bool(torch.isfinite(got).all().item())}
    peer_bad = world > 1 and chain.peer is not None and chain.peer.status() != 0  # (one status word covers both exchanges)
    ep_stuck = False
    if world > 1 and not args.no_extras:
        # Last, and under a deadline on every rank: a side measurement must not be able to keep the line above from
        # being printed (a rank that fails alone would leave the others waiting in the next all-to-all).
        got = {}

        def ep_work():
            try:
                torch.cuda.set_device(device)
                got["v"] = moe_ep_extras(device, world, rank, barrier)
            except Exception as e:  # noqa: BLE001
                got["v"] = {"error": repr(e)[:300]}

        th = threading.Thread(target=ep_work, daemon=True)
        th.start()
        th.join(180)
        ep_stuck = "v" not in got
        line["moe_fp8_deepseek_v3_layer_expert_parallel"] = got.get("v", {"error": "no result within 180 s"})
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            v, t_step, _, _, sample = cpu_reference(M, threads, 3, 1)
            line["cpu_baseline"] = {"value": v, "unit": unit, "cores": threads, "kind": "port", "sample": sample}
        print(json.dumps(line), flush=True)
    if peer_bad:
        print("[bench] a bounded wait on a peer gave up: the N-GPU number above is not valid", file=sys.stderr)
    if world > 1:
        # Graphs that captured NCCL kernels must be gone before the communicator is torn down; and a
        # communicator that will not finish tearing down must not keep the job alive.
        sys.stdout.flush()
        if not ep_stuck:
            del graph
            torch.cuda.synchronize(device)
            dist.barrier()
        os._exit(0)
    return 0


if __name__ == "__main__":
    sys.exit(main())
