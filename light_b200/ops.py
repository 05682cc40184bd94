"""Host side of the operator API for the quantized-weight matmul path.

Mirrors the reference's `ops` package for this path -- same names, argument meaning and error
behaviour (ops/matmul_q.go, ops/int4.go, ops/fp8_block.go, ops/moe.go) -- on top of the C ABI in
include/light_b200.h.  Tensors are torch CUDA tensors used only as device buffers; every op
allocates its output, as the reference ops do, and enqueues on torch's current stream.

There is no CPU path and no PyTorch fallback: a tensor that is not on a CUDA device is an
error, and so is a missing shared library.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from . import _lib
from ._lib import BF16, F16, F32, Q4_0, Q4_K, Q5_0, Q5_K, Q6_K, Q8_0, Light200Error, MoeArgs  # noqa: F401

GGUF_NAMES = {Q4_0: "Q4_0", Q5_0: "Q5_0", Q8_0: "Q8_0", Q4_K: "Q4_K", Q5_K: "Q5_K", Q6_K: "Q6_K"}
_ACT = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}


def block_elems(ggml_type: int) -> int:
    """dtype.DType.BlockElems (dtype/dtype.go:76-83)."""
    return _lib.lib().light_b200_block_elems(ggml_type)


def block_bytes(ggml_type: int) -> int:
    """dtype.DType.BlockBytes (dtype/dtype.go:85-91)."""
    return _lib.lib().light_b200_block_bytes(ggml_type)


@dataclass
class QTensor:
    """A GGUF block-quantized tensor kept in its on-disk layout: `data` is uint8 with the rows'
    blocks back to back; `shape` is the logical (N, K) or (E, N, K) (gguf/reader.go:237-251)."""
    data: torch.Tensor
    ggml_type: int
    shape: tuple

    def __post_init__(self):
        be, bb = block_elems(self.ggml_type), block_bytes(self.ggml_type)
        if be == 0:
            raise ValueError(f"QTensor: ggml type {self.ggml_type} is not a supported quantized dtype")
        n = 1
        for d in self.shape:
            n *= d
        if self.shape[-1] % be:
            raise ValueError(f"QTensor: inner dim {self.shape[-1]} not a multiple of {GGUF_NAMES[self.ggml_type]} "
                             f"block size {be}")
        if self.data.dtype != torch.uint8 or self.data.numel() != n // be * bb:
            raise ValueError(f"QTensor: {self.data.numel()} bytes of {self.data.dtype} for shape {self.shape}, "
                             f"expected {n // be * bb} uint8")

    @property
    def device(self):
        return self.data.device


@dataclass
class Int4:
    """quant.Int4 (quant/int4.go:12-31): codes u32 (N, K/8) held as int32, scales / zeros f32
    (N, K/G), group G, optional act-order permutation (K,) int64."""
    codes: torch.Tensor
    scales: torch.Tensor
    zeros: torch.Tensor
    group: int
    perm: Optional[torch.Tensor] = None

    def N(self) -> int:
        return self.codes.shape[0]

    def K(self) -> int:
        return self.codes.shape[1] * 8


@dataclass
class MoERouting:
    """ops.MoERouting (ops/moe.go:13-22)."""
    topk_ids: torch.Tensor      # (T, topk) int64
    weights: torch.Tensor       # (M,) f32
    sorted_pairs: torch.Tensor  # (M,) int64, pair ids in expert order
    sorted_expts: torch.Tensor  # (M,) int64, non-decreasing


def _dev(t: torch.Tensor, what: str) -> int:
    if not t.is_cuda:
        raise ValueError(f"{what}: tensor is on {t.device}; this library has CUDA kernels only")
    return t.device.index if t.device.index is not None else torch.cuda.current_device()


def _stream(device: int) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> C.c_void_p:
    return C.c_void_p(0 if t is None else t.data_ptr())


# --------------------------------------------------------------------------- workspace

_workspaces = {}  # device index -> torch uint8 buffer handed to the library
_retired = []     # buffers that were outgrown: a captured graph may still hold their address (scratch stays valid scratch)


def ensure_workspace(device_index: int, nbytes: int) -> None:
    """Keeps one reusable device buffer per GPU registered with the library (the counterpart of the
    reference's per-device weight scratch, ops/fp8_block.go:105-154); grows it when a call needs more."""
    cur = _workspaces.get(device_index)
    if cur is not None and cur.numel() - 1024 >= nbytes:
        return
    # 64 MB to begin with: what batched decode (22 MB) and a 2048-row prefill of the widest layer's f16 copy need.  A
    # buffer that is outgrown is kept, not freed: launches already captured in a CUDA graph go on using its address, and
    # every call writes what it reads there, so they stay correct.
    if cur is not None:
        _retired.append(cur)
    buf = torch.empty(max(nbytes, 64 << 20) + 1024, dtype=torch.uint8, device=torch.device("cuda", device_index))
    off = (-buf.data_ptr()) % 1024
    _lib.check(_lib.lib().light_b200_set_workspace(device_index, C.c_void_p(buf.data_ptr() + off), buf.numel() - 1024))
    _workspaces[device_index] = buf


def prefill_status(device_index: int = 0) -> int:
    """0 unless a bounded wait inside a tensor-core kernel gave up on this device."""
    return _lib.lib().light_b200_prefill_status(device_index)


# --------------------------------------------------------------------------- GGUF

def MatMulQ(x: torch.Tensor, w: QTensor) -> torch.Tensor:
    """ops.MatMulQ (ops/matmul_q.go:27-75): out (M, N) f32 = x (M, K) f32 . dequant(w (N, K))^T."""
    if x.dim() != 2 or len(w.shape) != 2:
        raise ValueError(f"MatMulQ: want x (M,K) and w (N,K); got {tuple(x.shape)}, {tuple(w.shape)}")
    if x.dtype != torch.float32:
        raise ValueError(f"MatMulQ: x must be F32, got {x.dtype}")
    if x.device != w.device:
        raise ValueError(f"MatMulQ: x on {x.device}, w on {w.device}")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise ValueError(f"MatMulQ: inner dim mismatch (x K={K}, w K={w.shape[1]})")
    dev = _dev(x, "MatMulQ")
    xc = x.contiguous()
    if M > 1:  # the batched paths keep an f16 copy of x (and split-K partial sums) in the workspace
        ensure_workspace(dev, int(_lib.lib().light_b200_matmul_q_workspace_bytes(M, K)))
    out = torch.empty((M, N), dtype=torch.float32, device=x.device)
    _lib.check(_lib.lib().light_b200_matmul_q(w.ggml_type, _ptr(xc), _ptr(w.data), _ptr(out), M, N, K, dev,
                                              _stream(dev)))
    return out


def _one_row(x: torch.Tensor, op: str) -> int:
    if x.dtype != torch.float32:
        raise ValueError(f"{op}: x must be F32, got {x.dtype}")
    K = x.shape[-1]
    if x.numel() != K:
        raise ValueError(f"{op}: x must be one row, got {tuple(x.shape)}")
    return K


def MatMulQMulti(x: torch.Tensor, ws: Sequence[QTensor], outs: Optional[Sequence[torch.Tensor]] = None) -> list:
    """The quantized twin of ops.LinearMulti (ops/gemv.go:21-78): f32 activations (one row, or a small batch
    (M, K)) against up to four quantized weights of one type that share K (the q/k/v trio, gate and up), in one
    launch for one row and for 2..8 rows of Q4_K.  Returns one (..., N_i) f32 tensor per weight (written into
    `outs` when given)."""
    if not 1 <= len(ws) <= 4:
        raise ValueError(f"MatMulQMulti: {len(ws)} weights, want 1..4")
    if x.dtype != torch.float32:
        raise ValueError(f"MatMulQMulti: x must be F32, got {x.dtype}")
    K = x.shape[-1]
    M = x.numel() // K
    for i, w in enumerate(ws):
        if len(w.shape) != 2 or w.shape[1] != K or w.ggml_type != ws[0].ggml_type or w.device != x.device:
            raise ValueError(f"MatMulQMulti: weight {i} must be (N, {K}) of type {ws[0].ggml_type} on {x.device}")
    dev = _dev(x, "MatMulQMulti")
    xc = x.contiguous()
    lead = tuple(x.shape[:-1])
    if outs is None:
        outs = [torch.empty(lead + (w.shape[0],), dtype=torch.float32, device=x.device) for w in ws]
    n = len(ws)
    wp = (C.c_void_p * n)(*[w.data.data_ptr() for w in ws])
    op = (C.c_void_p * n)(*[o.data_ptr() for o in outs])
    nn = (C.c_int32 * n)(*[w.shape[0] for w in ws])
    if M > 1:
        ensure_workspace(dev, int(_lib.lib().light_b200_matmul_q_workspace_bytes(M, K)))
    _lib.check(_lib.lib().light_b200_matmul_q_multi_rows(ws[0].ggml_type, _ptr(xc), wp, op, nn, n, M, K, dev, _stream(dev)))
    return list(outs)


def MatMulQGated(x: torch.Tensor, wg: QTensor, wu: QTensor, gelu: bool = False, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The quantized twin of ops.GatedLinear (ops/gemv.go:80-140): act(x . wg^T) * (x . wu^T) for one
    f32 activation row, act = SiLU or (gelu) GELU-erf, in one launch.  Raises when the fused kernel
    does not apply; the caller then runs MatMulQ twice and the activation itself, as the reference
    does without gemv_gated."""
    K = _one_row(x, "MatMulQGated")
    for w in (wg, wu):
        if len(w.shape) != 2 or w.shape[1] != K or w.shape[0] != wg.shape[0] or w.ggml_type != wg.ggml_type or w.device != x.device:
            raise ValueError(f"MatMulQGated: weights must be (N, {K}) of one type on {x.device}")
    dev = _dev(x, "MatMulQGated")
    xc = x.contiguous()
    N = wg.shape[0]
    if out is None:
        out = torch.empty(tuple(x.shape[:-1]) + (N,), dtype=torch.float32, device=x.device)
    _lib.check(_lib.lib().light_b200_matmul_q_gated(wg.ggml_type, _ptr(xc), _ptr(wg.data), _ptr(wu.data), _ptr(out), N, K,
                                                    2 if gelu else 1, dev, _stream(dev)))
    return out


def LinearMulti(x: torch.Tensor, ws: Sequence[torch.Tensor], out_dtype: torch.dtype = torch.bfloat16) -> list:
    """ops.LinearMulti (ops/gemv.go:21-78): one BF16 activation row against up to four (N_i, K) BF16 weights in one
    launch; outputs at BF16 or F32."""
    if len(ws) == 0:
        raise ValueError("LinearMulti: no weights")
    K = x.shape[-1]
    if x.dtype != torch.bfloat16 or x.numel() != K:
        raise ValueError(f"LinearMulti: x must be one BF16 row, got {x.dtype} {tuple(x.shape)}")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise ValueError(f"LinearMulti: outDT {out_dtype}")
    for i, w in enumerate(ws):
        if w.dim() != 2 or w.shape[1] != K or w.dtype != torch.bfloat16 or w.device != x.device:
            raise ValueError(f"LinearMulti: weight {i} must be (N, {K}) BF16 on {x.device}, got {tuple(w.shape)} {w.dtype} on {w.device}")
    if len(ws) > 4 or K % 8:
        raise ValueError(f"LinearMulti: K {K} / {len(ws)} weights unsupported by the fused kernel")
    dev = _dev(x, "LinearMulti")
    xc = x.contiguous()
    wc = [w.contiguous() for w in ws]
    lead = tuple(x.shape[:-1])
    outs = [torch.empty(lead + (w.shape[0],), dtype=out_dtype, device=x.device) for w in ws]
    n = len(ws)
    wp = (C.c_void_p * n)(*[w.data_ptr() for w in wc])
    op = (C.c_void_p * n)(*[o.data_ptr() for o in outs])
    nn = (C.c_int32 * n)(*[w.shape[0] for w in ws])
    _lib.check(_lib.lib().light_b200_gemv_multi(_ptr(xc), wp, op, nn, n, K, int(out_dtype == torch.float32), dev, _stream(dev)))
    return outs


def GatedLinear(x: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, gelu: bool = False) -> torch.Tensor:
    """ops.GatedLinear (ops/gemv.go:80-140): act(x . wg^T) * (x . wu^T) for one BF16 row, BF16 weights, act SiLU or
    GELU-erf, with the BF16 roundings of the unfused sequence."""
    K = x.shape[-1]
    if x.dtype != torch.bfloat16 or x.numel() != K:
        raise ValueError(f"GatedLinear: x must be one BF16 row, got {x.dtype} {tuple(x.shape)}")
    for w in (wg, wu):
        if w.dim() != 2 or w.shape[1] != K or w.shape[0] != wg.shape[0] or w.dtype != torch.bfloat16 or w.device != x.device:
            raise ValueError(f"GatedLinear: weights must be (N, {K}) BF16 on {x.device}, got {tuple(wg.shape)} / {tuple(wu.shape)}")
    dev = _dev(x, "GatedLinear")
    out = torch.empty(tuple(x.shape[:-1]) + (wg.shape[0],), dtype=torch.bfloat16, device=x.device)
    _lib.check(_lib.lib().light_b200_gemv_gated(_ptr(x.contiguous()), _ptr(wg.contiguous()), _ptr(wu.contiguous()), _ptr(out), wg.shape[0], K,
                                                int(gelu), dev, _stream(dev)))
    return out


def NormMatMulQ(x: torch.Tensor, norm_weight: torch.Tensor, eps: float, ws: Sequence[QTensor], residual: Optional[torch.Tensor] = None,
                gate: Optional[str] = None):
    """RMSNorm(x [+ residual]) followed by LinearMulti (gate None) or GatedLinear (gate "silu" / "gelu") over Q4_K
    weights, as one launch (light_b200_matmul_q_fused).  One activation row.  Returns the list of outputs (one
    tensor for a gated pair), and with a residual also the sum x + residual."""
    K = _one_row(x, "NormMatMulQ")
    act = {None: 0, "silu": 1, "gelu": 2}[gate]
    if act and len(ws) != 2:
        raise ValueError("ops.NormMatMulQ: a gated launch takes exactly the gate and the up matrix")
    if norm_weight.shape != (K,) or norm_weight.dtype != torch.float32 or (residual is not None and residual.numel() != K):
        raise ValueError(f"ops.NormMatMulQ: norm weight {tuple(norm_weight.shape)} / residual against K = {K}")
    for w in ws:
        if len(w.shape) != 2 or w.shape[1] != K or w.ggml_type != ws[0].ggml_type:
            raise ValueError(f"ops.NormMatMulQ: weight {w.shape} against K = {K}")
    dev = _dev(x, "NormMatMulQ")
    xc = x.contiguous()
    total = torch.empty_like(xc) if residual is not None else None
    rc = residual.contiguous() if residual is not None else None
    nw = norm_weight.contiguous()
    outs = [torch.empty(tuple(x.shape[:-1]) + (w.shape[0],), dtype=torch.float32, device=x.device) for w in (ws[:1] if act else ws)]
    n = len(ws)
    na = _lib.NormArgs(_ptr(nw), _ptr(rc), _ptr(total), float(eps))
    wp = (C.c_void_p * n)(*[w.data.data_ptr() for w in ws])
    op = (C.c_void_p * n)(*[outs[0 if act else i].data_ptr() for i in range(n)])
    nn = (C.c_int32 * n)(*[w.shape[0] for w in ws])
    _lib.check(_lib.lib().light_b200_matmul_q_fused(ws[0].ggml_type, _ptr(xc), C.byref(na), wp, op, nn, n, act, K, dev, _stream(dev)))
    res = outs[0] if act else outs
    return res if residual is None else (res, total)


def Dequantize(w: QTensor) -> torch.Tensor:
    """quant.Dequantize on a CUDA tensor (quant/cuda_hook.go:28-46): blocks -> f32, same shape."""
    dev = _dev(w.data, "Dequantize")
    n = 1
    for d in w.shape:
        n *= d
    out = torch.empty(w.shape, dtype=torch.float32, device=w.device)
    _lib.check(_lib.lib().light_b200_dequant(w.ggml_type, _ptr(w.data), _ptr(out), n, dev, _stream(dev)))
    return out


def MatMulW8A8(x: torch.Tensor, wq: torch.Tensor, ws: torch.Tensor) -> torch.Tensor:
    """ops.MatMulW8A8 (ops/matmul_w8a8.go:13-63): x F32 (M, K), wq I8 (N, K), ws F32 (N,) -> F32 (M, N); the rows of x
    are quantised to int8 on the device, the products accumulate in int32."""
    if x.dim() != 2 or wq.dim() != 2 or ws.dim() != 1:
        raise ValueError(f"ops.MatMulW8A8: want x (M,K), wq (N,K), ws (N,); got {tuple(x.shape)}, {tuple(wq.shape)}, {tuple(ws.shape)}")
    if x.dtype != torch.float32 or wq.dtype != torch.int8 or ws.dtype != torch.float32:
        raise ValueError(f"ops.MatMulW8A8: dtypes must be x=F32, wq=I8, ws=F32 (got {x.dtype}, {wq.dtype}, {ws.dtype})")
    M, K = x.shape
    N = wq.shape[0]
    if wq.shape[1] != K or ws.shape[0] != N:
        raise ValueError(f"ops.MatMulW8A8: x {tuple(x.shape)}, wq {tuple(wq.shape)}, ws {tuple(ws.shape)} do not agree")
    dev = _dev(x, "MatMulW8A8")
    out = torch.empty((M, N), dtype=torch.float32, device=x.device)
    xq = torch.empty((M, K), dtype=torch.int8, device=x.device)
    xs = torch.empty((M,), dtype=torch.float32, device=x.device)
    _lib.check(_lib.lib().light_b200_matmul_w8a8(_ptr(x.contiguous()), _ptr(wq.contiguous()), _ptr(ws.contiguous()), _ptr(out), _ptr(xq), _ptr(xs),
                                                 M, N, K, dev, _stream(dev)))
    return out


def EmbeddingQ(table: QTensor, ids: torch.Tensor) -> torch.Tensor:
    """nn.Embedding over a quantized table (nn/embedding.go; nn/embedding_test.go:127): only the gathered rows are
    dequantized.  table (V, K) blocks, ids I64 of any shape -> f32 ids.shape + (K,)."""
    if len(table.shape) != 2:
        raise ValueError(f"ops.EmbeddingQ: table shape {table.shape}, want (V, K)")
    if ids.dtype != torch.int64:
        raise ValueError(f"ops.EmbeddingQ: ids must be I64, got {ids.dtype}")
    dev = _dev(table.data, "EmbeddingQ")
    V, K = table.shape
    flat = ids.contiguous().reshape(-1)
    out = torch.empty((flat.numel(), K), dtype=torch.float32, device=table.device)
    _lib.check(_lib.lib().light_b200_embedding_q(table.ggml_type, _ptr(table.data), _ptr(flat), _ptr(out), flat.numel(), V, K, dev, _stream(dev)))
    return out.reshape(tuple(ids.shape) + (K,))


# --------------------------------------------------------------------------- int4

def Int4FromCheckpoint(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor, group: int, layout: str) -> "Int4":
    """quant.FromGPTQ (ordered groups) / quant.FromAWQ (quant/int4.go:103-261) on the device: layout "gptq",
    "gptq_v2" or "awq"; qweight / qzeros I32, scales F32 (K/G, N)."""
    kind = {"gptq": 0, "gptq_v2": 1, "awq": 2}[layout]
    if qweight.dim() != 2 or qzeros.dim() != 2 or scales.dim() != 2:
        raise ValueError("quant.From%s: rank-2 qweight / qzeros / scales expected" % ("AWQ" if kind == 2 else "GPTQ"))
    K, N = (qweight.shape[0], qweight.shape[1] * 8) if kind == 2 else (qweight.shape[0] * 8, qweight.shape[1])
    if group <= 0:
        group = K
    if K % group or tuple(scales.shape) != (K // group, N) or tuple(qzeros.shape) != (K // group, N // 8) or scales.dtype != torch.float32:
        raise ValueError(f"quant.From{'AWQ' if kind == 2 else 'GPTQ'}: qweight {tuple(qweight.shape)}, qzeros {tuple(qzeros.shape)}, "
                         f"scales {tuple(scales.shape)}, group {group} inconsistent")
    dev = _dev(qweight, "Int4FromCheckpoint")
    codes = torch.empty((N, K // 8), dtype=torch.int32, device=qweight.device)
    s = torch.empty((N, K // group), dtype=torch.float32, device=qweight.device)
    z = torch.empty_like(s)
    _lib.check(_lib.lib().light_b200_int4_repack(_ptr(qweight.contiguous()), _ptr(qzeros.contiguous()), _ptr(scales.contiguous()), _ptr(codes),
                                                 _ptr(s), _ptr(z), N, K, group, kind, dev, _stream(dev)))
    return Int4(codes, s, z, group)


def DequantizeInt4(w: Int4, out_dtype: torch.dtype, out: Optional[torch.Tensor] = None, offset: int = 0) -> torch.Tensor:
    """ops.DequantizeInt4 / dequantizeInt4At (ops/int4.go:13-57): (N, K) at F32 or BF16; with
    `out` given, writes `offset` elements into it (one slot of a stacked buffer)."""
    if w.group <= 0 or w.K() % w.group:
        raise ValueError(f"ops.DequantizeInt4: group {w.group} does not divide K {w.K()}")
    if out_dtype not in (torch.float32, torch.bfloat16):
        raise ValueError(f"ops.DequantizeInt4: output {out_dtype}, want F32 or BF16")
    dev = _dev(w.codes, "DequantizeInt4")
    if out is None:
        out = torch.zeros((w.N(), w.K()), dtype=out_dtype, device=w.codes.device)
    _lib.check(_lib.lib().light_b200_int4_dequant(_ptr(w.codes.contiguous()), _ptr(w.scales.contiguous()),
                                                  _ptr(w.zeros.contiguous()), _ptr(out), _ACT[out_dtype], w.N(), w.K(),
                                                  w.group, offset, dev, _stream(dev)))
    return out


def GatherColumns(x: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """gatherColumns (ops/int4.go:129-147): x (M, K) -> x[:, idx], one launch."""
    if x.dim() != 2 or idx.dtype != torch.int64 or idx.numel() != x.shape[1] or x.dtype not in _ACT:
        raise ValueError(f"gather_columns: x {tuple(x.shape)} {x.dtype}, idx {tuple(idx.shape)} {idx.dtype}")
    dev = _dev(x, "GatherColumns")
    out = torch.empty_like(x, memory_format=torch.contiguous_format)
    _lib.check(_lib.lib().light_b200_gather_columns(_ptr(x.contiguous()), _ptr(idx.contiguous()), _ptr(out), _ACT[x.dtype], x.shape[0], x.shape[1], dev,
                                                    _stream(dev)))
    return out


def ConcatInt4(a: Int4, b: Int4) -> Int4:
    """concatInt4 (models/int4_load.go:226-244): two weights stacked along N (gate over up); same K, same group, no act-order."""
    if a.group != b.group or a.K() != b.K() or a.perm is not None or b.perm is not None:
        raise ValueError(f"concatInt4: incompatible gate / up (group {a.group} / {b.group}, act-order {a.perm is not None} / {b.perm is not None})")
    return Int4(torch.cat([a.codes, b.codes], 0), torch.cat([a.scales, b.scales], 0), torch.cat([a.zeros, b.zeros], 0), a.group)


def MoEInt4(x: torch.Tensor, gate_up: Sequence[Int4], down: Sequence[Int4], route: MoERouting, topk: int, gelu: bool = False) -> torch.Tensor:
    """ops.MoEInt4 (ops/int4.go:157-268): a sparse block over 4-bit experts.  Only the experts the routing uses are
    expanded (light_b200_int4_dequant into one stacked buffer at x's dtype), the routing is renumbered onto them, and
    the two grouped matmuls, the gate and the combine run as for dense experts."""
    if x.dim() != 2 or len(gate_up) == 0 or len(gate_up) != len(down):
        raise ValueError(f"ops.MoEInt4: x {tuple(x.shape)}, {len(gate_up)} gate-up / {len(down)} down experts")
    T, H = x.shape
    I2, I = gate_up[0].N(), down[0].K()
    if gate_up[0].K() != H or down[0].N() != H or I2 != 2 * I:
        raise ValueError(f"ops.MoEInt4: expert shapes gate-up ({I2}, {gate_up[0].K()}), down ({down[0].N()}, {I}) for hidden {H}")
    ids = route.topk_ids.reshape(-1)
    if int(ids.min()) < 0 or int(ids.max()) >= len(gate_up):
        raise ValueError("ops.MoEInt4: expert out of range")
    used, compact = torch.unique(ids, return_inverse=True)   # the experts in use, and every pair's slot among them
    U = used.numel()
    gu = torch.empty((U, I2, H), dtype=x.dtype, device=x.device)
    dn = torch.empty((U, H, I), dtype=x.dtype, device=x.device)
    for s, e in enumerate(used.tolist()):
        DequantizeInt4(gate_up[e], x.dtype, out=gu, offset=s * I2 * H)
        DequantizeInt4(down[e], x.dtype, out=dn, offset=s * H * I)
    r = MoERouteFromIDs(compact.reshape(-1), route.weights, T, topk)
    h = MoEGemm(x.contiguous(), gu, r, None, topk)
    pair = MoEGemm(MoEGateMul(h, gelu), dn, r, r.weights, topk)
    return MoECombine(pair, topk)


def MatMulInt4(x: torch.Tensor, w: Int4) -> torch.Tensor:
    """ops.MatMulInt4 (ops/int4.go:66-127): x (M, K) F32 or BF16 -> (M, N) at x's dtype."""
    if x.dim() != 2 or x.shape[1] != w.K():
        raise ValueError(f"ops.MatMulInt4: x {tuple(x.shape)}, weight ({w.N()}, {w.K()})")
    if x.dtype not in (torch.float32, torch.bfloat16):
        raise ValueError(f"ops.MatMulInt4: activations {x.dtype}, want F32 or BF16")
    dev = _dev(x, "MatMulInt4")
    xc = x.contiguous()
    if w.perm is not None:  # act-order GPTQ: gather x's columns into the weight's K order (ops/int4.go:129-147)
        xc = GatherColumns(xc, w.perm)
    M, N = x.shape[0], w.N()
    if M > 64 or (4 <= M and x.dtype == torch.bfloat16):
        # tensor-core path: f16 copy of x (f32 activations) and the persistent kernel's partial tiles; 4 to 64 bf16 rows:
        # token tiles over activations staged once
        ensure_workspace(dev, int(_lib.lib().light_b200_matmul_q_workspace_bytes(M, w.K())))
    out = torch.zeros((M, N), dtype=x.dtype, device=x.device)
    _lib.check(_lib.lib().light_b200_int4_gemv(_ptr(xc), _ptr(w.codes.contiguous()), _ptr(w.scales.contiguous()),
                                               _ptr(w.zeros.contiguous()), _ptr(out), _ACT[x.dtype], M, N, w.K(),
                                               w.group, dev, _stream(dev)))
    return out


# --------------------------------------------------------------------------- block-scaled FP8

def DequantizeF8Block(w: torch.Tensor, scale: torch.Tensor, block_r: int, block_c: int,
                      out_dtype: torch.dtype) -> torch.Tensor:
    """ops.DequantizeF8Block (ops/fp8_block.go:13-60): e4m3 codes (R, C) (uint8 or float8_e4m3fn),
    f32 scale (R/bR, C/bC) -> (R, C) at F32 or BF16."""
    if w.dim() != 2 or scale.dim() != 2:
        raise ValueError("ops.DequantizeF8Block: rank-2 weight and scale expected")
    R, Cc = w.shape
    if block_r <= 0 or block_c <= 0 or R % block_r or Cc % block_c or tuple(scale.shape) != (R // block_r, Cc // block_c):
        raise ValueError(f"ops.DequantizeF8Block: weight {tuple(w.shape)}, scale {tuple(scale.shape)}, "
                         f"block ({block_r}, {block_c}) inconsistent")
    dev = _dev(w, "DequantizeF8Block")
    out = torch.empty((R, Cc), dtype=out_dtype, device=w.device)
    if out_dtype not in (torch.float32, torch.bfloat16):
        raise ValueError(f"ops.DequantizeF8Block: output {out_dtype}, want F32 or BF16")
    _lib.check(_lib.lib().light_b200_fp8_block_dequant(_ptr(w.contiguous()), _ptr(scale.contiguous()), _ptr(out),
                                                       _ACT[out_dtype], R, Cc, block_r, block_c, dev, _stream(dev)))
    return out


def MatMulF8Block(x: torch.Tensor, w: torch.Tensor, scale: torch.Tensor, block_r: int, block_c: int) -> torch.Tensor:
    """ops.MatMulF8Block (ops/fp8_block.go:165-233): x (M, K) F32 or BF16 -> (M, N) at x's dtype."""
    if x.dim() != 2 or w.dim() != 2 or x.shape[1] != w.shape[1]:
        raise ValueError(f"ops.MatMulF8Block: x {tuple(x.shape)}, w {tuple(w.shape)}")
    if x.dtype not in (torch.float32, torch.bfloat16):
        raise ValueError(f"ops.MatMulF8Block: activations {x.dtype}, want F32 or BF16")
    M, K = x.shape
    N = w.shape[0]
    dev = _dev(x, "MatMulF8Block")
    if M > 64 or (4 <= M and x.dtype == torch.bfloat16):  # (as in MatMulInt4)
        ensure_workspace(dev, int(_lib.lib().light_b200_matmul_q_workspace_bytes(M, K)))
    out = torch.zeros((M, N), dtype=x.dtype, device=x.device)
    _lib.check(_lib.lib().light_b200_fp8_block_gemv(_ptr(x.contiguous()), _ptr(w.contiguous()),
                                                    _ptr(scale.contiguous()), _ptr(out), _ACT[x.dtype], M, N, K,
                                                    block_r, block_c, dev, _stream(dev)))
    return out


# --------------------------------------------------------------------------- MoE

def MoERouteFromIDs(ids: torch.Tensor, weights: torch.Tensor, T: int, topk: int) -> MoERouting:
    """ops.MoERouteFromIDs (ops/moe.go:73-99): explicit top-k selection -> expert-sorted pairs."""
    if ids.numel() != T * topk or weights.numel() != T * topk:
        raise ValueError(f"moe_route: {ids.numel()} ids / {weights.numel()} weights for {T} x {topk}")
    flat = ids.reshape(T * topk).to(torch.int64)
    sorted_expts, sorted_pairs = torch.sort(flat, stable=True)
    return MoERouting(ids.reshape(T, topk), weights.reshape(T * topk).float(), sorted_pairs, sorted_expts)


def MoERoute(probs: torch.Tensor, topk: int, normalize: bool) -> MoERouting:
    """ops.MoERoute (ops/moe.go:29-71): router probabilities (T, E) F32 -> the k largest experts per token, their
    probabilities (renormalised when `normalize`), and the pairs sorted by expert.  Selection and sort run on the
    device (light_b200_moe_route_topk + light_b200_moe_sort_pairs); ties keep the lower expert id."""
    if probs.dim() != 2 or probs.dtype != torch.float32:
        raise ValueError(f"moe_route: probs must be (T, E) F32, got {tuple(probs.shape)} {probs.dtype}")
    T, E = probs.shape
    if topk < 1 or topk > E:
        raise ValueError(f"moe_route: topk {topk} out of range [1, {E}]")
    dev = _dev(probs, "MoERoute")
    ids = torch.empty((T, topk), dtype=torch.int64, device=probs.device)
    w = torch.empty((T, topk), dtype=torch.float32, device=probs.device)
    _lib.check(_lib.lib().light_b200_moe_route_topk(_ptr(probs.contiguous()), _ptr(ids), _ptr(w), T, E, topk, int(normalize), dev, _stream(dev)))
    sp, se, _, _ = MoESortPairs(ids.reshape(-1), E)
    return MoERouting(ids, w.reshape(-1), sp, se)


def MoERouteDeepseek(logits: torch.Tensor, bias: Optional[torch.Tensor], topk: int, n_group: int = 1, topk_group: int = 1, sigmoid: bool = True,
                     norm_topk: bool = True) -> MoERouting:
    """The DeepSeek router on the device, every branch of models/deepseek_route.go:30-133 (sigmoid + bias or softmax
    scores, group-limited selection, stable top-k), followed by the expert sort of ops.MoERouteFromIDs."""
    if logits.dim() != 2 or logits.dtype != torch.float32:
        raise ValueError(f"deepseek router: logits must be (T, E) F32, got {tuple(logits.shape)} {logits.dtype}")
    T, E = logits.shape
    n_group = max(1, n_group)
    if E % n_group:
        raise ValueError(f"deepseek router: {E} experts not divisible into {n_group} groups")
    if topk < 1 or topk > E:
        raise ValueError(f"moe_route: topk {topk} out of range [1, {E}]")
    dev = _dev(logits, "MoERouteDeepseek")
    ids = torch.empty((T, topk), dtype=torch.int64, device=logits.device)
    w = torch.empty((T, topk), dtype=torch.float32, device=logits.device)
    _lib.check(_lib.lib().light_b200_moe_route_deepseek(_ptr(logits.contiguous()), _ptr(None if bias is None else bias.contiguous()), _ptr(ids), _ptr(w),
                                                        T, E, topk, n_group, topk_group, int(sigmoid), int(norm_topk), dev, _stream(dev)))
    sp, se, _, _ = MoESortPairs(ids.reshape(-1), E)
    return MoERouting(ids, w.reshape(-1), sp, se)


def MoERouteSigmoid(logits: torch.Tensor, bias: Optional[torch.Tensor], topk: int, norm_topk: bool = True, E_sort: Optional[int] = None) -> MoERouting:
    """The DeepSeek-V3 router (models/deepseek_route.go:30-133, sigmoid branch, one group) and the expert sort of
    ops.MoERouteFromIDs (ops/moe.go:73-99), both on the device: logits (T, E) F32, bias (E) F32 or None."""
    if logits.dim() != 2 or logits.dtype != torch.float32:
        raise ValueError(f"moe_route: logits must be (T, E) F32, got {tuple(logits.shape)} {logits.dtype}")
    T, E = logits.shape
    if topk < 1 or topk > E:
        raise ValueError(f"moe_route: topk {topk} out of range [1, {E}]")
    dev = _dev(logits, "MoERouteSigmoid")
    ids = torch.empty((T, topk), dtype=torch.int64, device=logits.device)
    w = torch.empty((T, topk), dtype=torch.float32, device=logits.device)
    _lib.check(_lib.lib().light_b200_moe_route_sigmoid(_ptr(logits.contiguous()), _ptr(None if bias is None else bias.contiguous()), _ptr(ids),
                                                       _ptr(w), T, E, topk, int(norm_topk), dev, _stream(dev)))
    sp, se, _, _ = MoESortPairs(ids.reshape(-1), E)
    return MoERouting(ids, w.reshape(-1), sp, se)


def MoESortPairs(ids: torch.Tensor, E: int):
    """Expert-sorted pairs with their counts and offsets: (sorted_pairs, sorted_expts, counts, offsets)."""
    if ids.dtype != torch.int64 or ids.dim() != 1:
        raise ValueError(f"moe_sort_pairs: ids must be 1-D I64, got {ids.dtype} {tuple(ids.shape)}")
    dev = _dev(ids, "MoESortPairs")
    M = ids.numel()
    sp, se = torch.empty_like(ids), torch.empty_like(ids)
    counts = torch.empty(E, dtype=torch.int32, device=ids.device)
    offsets = torch.empty(E + 1, dtype=torch.int32, device=ids.device)
    scratch = torch.empty(M + (M + 1023) // 1024 * E + 1, dtype=torch.int32, device=ids.device)
    _lib.check(_lib.lib().light_b200_moe_sort_pairs(_ptr(ids.contiguous()), _ptr(counts), _ptr(offsets), _ptr(sp), _ptr(se), _ptr(scratch), M, E, dev,
                                                    _stream(dev)))
    return sp, se, counts, offsets


def moe_route_status(device_index: int = 0) -> int:
    """1 if an expert id outside [0, E) ever reached MoESortPairs on this device (synchronises)."""
    return _lib.lib().light_b200_moe_route_status(device_index)


def _moe_dispatch(op: str, key_dtype: int, quant: bool, inp: torch.Tensor, weights, wshape, routing: MoERouting,
                  topk_weights: Optional[torch.Tensor], topk: int, out_dtype: torch.dtype, f8=None) -> torch.Tensor:
    """moeGemmDispatch (ops/moe.go:124-204)."""
    if inp.dim() != 2 or len(wshape) != 3:
        raise ValueError(f"{op}: input (rows, K) and weights (E, N, K) required, got {tuple(inp.shape)} / {tuple(wshape)}")
    E, N, K = wshape
    if inp.shape[1] != K:
        raise ValueError(f"{op}: input K {inp.shape[1]} != weights K {K}")
    M = routing.sorted_pairs.shape[0]
    if routing.sorted_expts.shape[0] != M or routing.sorted_pairs.dtype != torch.int64 or \
            routing.sorted_expts.dtype != torch.int64:
        raise ValueError(f"{op}: routing must hold M I64 pair ids and M I64 expert ids")
    if inp.shape[0] == M:
        row_per_pair = True
    elif inp.shape[0] == M // topk:
        row_per_pair = False
    else:
        raise ValueError(f"{op}: input rows {inp.shape[0]} must be M={M} (per pair) or M/topk={M // topk} (per token)")
    if topk_weights is not None and (topk_weights.dtype != torch.float32 or topk_weights.numel() != M):
        raise ValueError(f"{op}: topkWeights must be F32 with {M} elements")
    dev = _dev(inp, op)
    inc = inp.contiguous()
    if M >= 256:  # tensor-core grouped path: the token rows gathered in expert order, the persistent kernel's partial tiles
        ensure_workspace(dev, int(_lib.lib().light_b200_matmul_q_workspace_bytes(M, K)))
    counts = torch.zeros(E, dtype=torch.int32, device=inp.device)
    offsets = torch.zeros(E + 1, dtype=torch.int32, device=inp.device)
    out = torch.zeros((M, N), dtype=out_dtype, device=inp.device)
    a = MoeArgs(input=inc.data_ptr(), weights=weights.data_ptr(), sorted_pairs=routing.sorted_pairs.contiguous().data_ptr(),
                expert_ids=routing.sorted_expts.contiguous().data_ptr(), counts=counts.data_ptr(),
                offsets=offsets.data_ptr(),
                topk_weights=0 if topk_weights is None else topk_weights.contiguous().data_ptr(), out=out.data_ptr(),
                M=M, size_m=M, E=E, N=N, K=K, topk=topk, row_per_pair=int(row_per_pair), dtype=key_dtype)
    if f8 is not None:
        scale, bR, bC = f8
        _lib.check(_lib.lib().light_b200_moe_gemm_f8block(C.byref(a), _ptr(scale.contiguous()), bR, bC, dev, _stream(dev)))
        return out
    fn = _lib.lib().light_b200_moe_gemm_q if quant else _lib.lib().light_b200_moe_gemm
    _lib.check(fn(C.byref(a), dev, _stream(dev)))
    return out


def MoEGemm(inp: torch.Tensor, weights: torch.Tensor, routing: MoERouting, topk_weights: Optional[torch.Tensor],
            topk: int) -> torch.Tensor:
    """ops.MoEGemm (ops/moe.go:101-122): dense stacked experts (E, N, K) at input's dtype."""
    if inp.dim() != 2 or weights.dim() != 3:
        raise ValueError(f"moe_gemm: input (rows, K) and weights (E, N, K) required, got {tuple(inp.shape)} / "
                         f"{tuple(weights.shape)}")
    if inp.dtype != weights.dtype:
        raise ValueError(f"moe_gemm: input {inp.dtype} / weights {weights.dtype} dtype mismatch")
    if inp.dtype not in _ACT:
        raise ValueError(f"moe_gemm: unsupported dtype {inp.dtype}")
    return _moe_dispatch("moe_gemm", _ACT[inp.dtype], False, inp, weights.contiguous(), tuple(weights.shape), routing,
                         topk_weights, topk, inp.dtype)


def MoEGemmQ(x: torch.Tensor, w: QTensor, routing: MoERouting, topk_weights: Optional[torch.Tensor],
             topk: int) -> torch.Tensor:
    """ops.MoEGemmQ (ops/moe.go:242-265): GGUF block-quantized experts (E, N, K), x f32, out f32."""
    if x.dtype != torch.float32:
        raise ValueError(f"moe_gemm_q: x must be F32, got {x.dtype}")
    if len(w.shape) != 3:
        raise ValueError(f"moe_gemm_q: w must be a quantized (E, N, K) tensor, got {tuple(w.shape)}")
    return _moe_dispatch("moe_gemm_q", w.ggml_type, True, x, w.data, tuple(w.shape), routing, topk_weights, topk,
                         torch.float32)


def MoEGemmF8Block(x: torch.Tensor, w: torch.Tensor, scale: torch.Tensor, block_r: int, block_c: int,
                   routing: MoERouting, topk_weights: Optional[torch.Tensor], topk: int) -> torch.Tensor:
    """Grouped matmul over block-scaled FP8 experts: w e4m3 codes (E, N, K) (uint8 or float8_e4m3fn), scale
    f32 (E, N/bR, K/bC), x F32 or BF16 (rows per token or per pair), output (M, N) at x's dtype.  The
    reference runs this as a host loop over experts (models/moe_routed.go:34-79: IndexSelect, one
    ops.MatMulF8Block per expert, scatter); the contract per pair is the same as MoEGemm's."""
    if x.dtype not in (torch.float32, torch.bfloat16):
        raise ValueError(f"moe_gemm_f8block: activations {x.dtype}, want F32 or BF16")
    if w.dim() != 3 or scale.dim() != 3:
        raise ValueError(f"moe_gemm_f8block: w (E, N, K) and scale (E, N/bR, K/bC) required, got {tuple(w.shape)} / "
                         f"{tuple(scale.shape)}")
    E, N, K = w.shape
    if block_r <= 0 or block_c <= 0 or N % block_r or K % block_c or tuple(scale.shape) != (E, N // block_r, K // block_c):
        raise ValueError(f"moe_gemm_f8block: weight {tuple(w.shape)}, scale {tuple(scale.shape)}, block ({block_r}, {block_c}) "
                         "inconsistent")
    return _moe_dispatch("moe_gemm_f8block", _ACT[x.dtype], False, x, w.contiguous(), (E, N, K), routing, topk_weights, topk,
                         x.dtype, f8=(scale, block_r, block_c))


def MoECombine(pair_out: torch.Tensor, topk: int) -> torch.Tensor:
    """ops.MoECombine (ops/moe.go:206-240): sum of the topk slot rows, (M, N) -> (T, N), slot 0 first, every sum
    rounded to the tensor's dtype (the reference adds the slots one after the other with its Add kernel): one launch."""
    M, N = pair_out.shape
    if M % topk:
        raise ValueError(f"moe_combine: {M} rows not divisible by topk {topk}")
    if pair_out.dtype not in _ACT or N % 8:
        raise ValueError(f"moe_combine: dtype {pair_out.dtype} / N {N} (a multiple of 8) unsupported")
    dev = _dev(pair_out, "MoECombine")
    out = torch.empty((M // topk, N), dtype=pair_out.dtype, device=pair_out.device)
    _lib.check(_lib.lib().light_b200_moe_combine(_ptr(pair_out.contiguous()), _ptr(out), _ACT[pair_out.dtype], M // topk, N, topk, dev, _stream(dev)))
    return out


def MoECombineWeighted(rows: torch.Tensor, index: Optional[torch.Tensor], weights: Optional[torch.Tensor], tokens: int, topk: int) -> torch.Tensor:
    """out f32 (tokens, N)[t] = sum over the token's slots, slot 0 first, of weights[t * topk + s] * rows[index[t * topk + s]]:
    the combine of a sparse block whose expert rows arrive unweighted and in another order (experts sharded over GPUs,
    tp.ExpertParallel); the arithmetic of MoEGemm's weighted epilogue followed by MoECombine (ops/moe.go:121-240), in f32.
    index int64 per pair (None: pair p is row p; outside [0, rows) drops the pair), weights f32 per pair (None: 1)."""
    if rows.dim() != 2 or rows.dtype not in _ACT or rows.shape[1] % 8:
        raise ValueError(f"moe_combine_weighted: rows {tuple(rows.shape)} {rows.dtype}: want (R, N), N a multiple of 8, F32 / BF16 / F16")
    M = tokens * topk
    for name, t, dt in (("index", index, torch.int64), ("weights", weights, torch.float32)):
        if t is not None and (t.dtype != dt or t.numel() != M or t.device != rows.device):
            raise ValueError(f"moe_combine_weighted: {name} must be {dt} with {M} elements on {rows.device}")
    if index is None and rows.shape[0] < M:
        raise ValueError(f"moe_combine_weighted: {rows.shape[0]} rows for {M} pairs and no index")
    dev = _dev(rows, "MoECombineWeighted")
    rows = rows.contiguous()
    out = torch.empty((tokens, rows.shape[1]), dtype=torch.float32, device=rows.device)
    _lib.check(_lib.lib().light_b200_moe_combine_weighted(_ptr(rows), _ptr(None if index is None else index.contiguous()),
                                                          _ptr(None if weights is None else weights.contiguous()), _ptr(out), _ACT[rows.dtype],
                                                          tokens, rows.shape[1], topk, rows.shape[0], dev, _stream(dev)))
    return out


def MoEGateMul(h: torch.Tensor, gelu: bool = False) -> torch.Tensor:
    """The step between the two grouped matmuls of a sparse block (nn/moe.go:206-224): h (M, 2 I) -> act(h[:, :I]) * h[:, I:],
    act SiLU or GELU-erf, the activation rounded to the tensor's dtype before the product: one launch."""
    if h.dim() != 2 or h.shape[1] % 16 or h.dtype not in _ACT:
        raise ValueError(f"moe_gate_mul: want (M, 2 I) with I a multiple of 8 at F32 / BF16 / F16, got {tuple(h.shape)} {h.dtype}")
    M, I2 = h.shape
    dev = _dev(h, "MoEGateMul")
    out = torch.empty((M, I2 // 2), dtype=h.dtype, device=h.device)
    _lib.check(_lib.lib().light_b200_moe_gate_mul(_ptr(h.contiguous()), _ptr(out), _ACT[h.dtype], M, I2 // 2, int(gelu), dev, _stream(dev)))
    return out


# --------------------------------------------------------------------------- decode-step attention

def _check_pos(pos: torch.Tensor, like: torch.Tensor, op: str) -> None:
    if pos.dtype != torch.int64 or pos.numel() != 1:
        raise ValueError(f"ops.{op}: position must be a one-element I64 tensor, got {pos.dtype} {tuple(pos.shape)}")
    if pos.device != like.device:
        raise ValueError(f"ops.{op}: position on {pos.device}, tensors on {like.device}")


def _check_cache(kbuf: torch.Tensor, vbuf: torch.Tensor, op: str) -> None:
    if kbuf.dim() != 4 or kbuf.shape != vbuf.shape:
        raise ValueError(f"ops.{op}: want buffers (B, KH, cap, HD), got {tuple(kbuf.shape)} / {tuple(vbuf.shape)}")
    if not kbuf.is_contiguous() or not vbuf.is_contiguous():
        raise ValueError(f"ops.{op}: buffers must be contiguous")


def KVAppend(kbuf: torch.Tensor, vbuf: torch.Tensor, k: torch.Tensor, v: torch.Tensor, pos: torch.Tensor) -> None:
    """ops.KVAppend (ops/decode_attn.go:13-62): k, v (B, KH, 1, HD) into the buffers (B, KH, cap, HD) at the
    position held on the device."""
    _check_cache(kbuf, vbuf, "KVAppend")
    if k.dim() != 4 or k.shape[2] != 1 or k.shape != v.shape:
        raise ValueError(f"ops.KVAppend: want k / v (B, KH, 1, HD), got {tuple(k.shape)} / {tuple(v.shape)}")
    if (kbuf.shape[0], kbuf.shape[1], kbuf.shape[3]) != (k.shape[0], k.shape[1], k.shape[3]):
        raise ValueError(f"ops.KVAppend: k {tuple(k.shape)} does not fit buffer {tuple(kbuf.shape)}")
    if k.dtype != kbuf.dtype or v.dtype != vbuf.dtype or k.dtype not in (torch.float32, torch.bfloat16):
        raise ValueError(f"ops.KVAppend: dtype mismatch ({k.dtype} into {kbuf.dtype})")
    _check_pos(pos, kbuf, "KVAppend")
    dev = _dev(kbuf, "KVAppend")
    B, KH, cap, D = kbuf.shape
    _lib.check(_lib.lib().light_b200_kv_append(_ptr(k.contiguous()), _ptr(v.contiguous()), _ptr(kbuf), _ptr(vbuf), _ptr(pos),
                                               _ACT[k.dtype], B, KH, D, cap, dev, _stream(dev)))


def DecodeAttention(q: torch.Tensor, kbuf: torch.Tensor, vbuf: torch.Tensor, pos: torch.Tensor, scale: float, window: int = 0,
                    k_new: Optional[torch.Tensor] = None, v_new: Optional[torch.Tensor] = None, rope_base: float = 0.0) -> torch.Tensor:
    """ops.DecodeAttention (ops/decode_attn.go:64-170): q (B, NH, 1, HD) against the first pos + 1 keys of the
    buffers -> (B, NH, 1, HD).  With k_new / v_new (B, KH, 1, HD) the same launch appends them at pos first
    (KVCache.decodeAttend, models/llama.go:1156-1160, does the two ops back to back); with rope_base the launch
    also rotates q and k_new at that position (the two ops.RoPE calls before it, models/llama.go:1136-1146)."""
    _check_cache(kbuf, vbuf, "DecodeAttention")
    if q.dim() != 4 or q.shape[2] != 1:
        raise ValueError(f"ops.DecodeAttention: want q (B, NH, 1, HD), got {tuple(q.shape)}")
    B, NH, _, D = q.shape
    KH, cap = kbuf.shape[1], kbuf.shape[2]
    if kbuf.shape[0] != B or kbuf.shape[3] != D or KH == 0 or NH % KH:
        raise ValueError(f"ops.DecodeAttention: q {tuple(q.shape)} against buffers {tuple(kbuf.shape)}")
    if q.dtype != kbuf.dtype or q.dtype != vbuf.dtype or q.dtype not in (torch.float32, torch.bfloat16):
        raise ValueError(f"ops.DecodeAttention: dtype mismatch q {q.dtype} k {kbuf.dtype} v {vbuf.dtype}")
    if (k_new is None) != (v_new is None):
        raise ValueError("ops.DecodeAttention: k_new and v_new come together")
    if k_new is not None and (tuple(k_new.shape) != (B, KH, 1, D) or k_new.shape != v_new.shape or k_new.dtype != q.dtype or v_new.dtype != q.dtype):
        raise ValueError(f"ops.DecodeAttention: k_new {tuple(k_new.shape)} {k_new.dtype} against buffers {tuple(kbuf.shape)}")
    _check_pos(pos, q, "DecodeAttention")
    dev = _dev(q, "DecodeAttention")
    out = torch.empty((B, NH, 1, D), dtype=q.dtype, device=q.device)
    qc = q.contiguous()
    kn = k_new.contiguous() if k_new is not None else None
    vn = v_new.contiguous() if v_new is not None else None
    a = _lib.DecodeAttnArgs(_ptr(qc), _ptr(kbuf), _ptr(vbuf), _ptr(kn), _ptr(vn), _ptr(pos), _ptr(out), _ACT[q.dtype], B, NH, KH, cap, D,
                            int(window), float(scale), float(rope_base))
    _lib.check(_lib.lib().light_b200_decode_attn(C.byref(a), dev, _stream(dev)))
    return out


def IncrementI64(t: torch.Tensor) -> None:
    """ops.IncrementI64 (ops/decode_attn.go:184-205): adds one to every element in place."""
    if t.dtype != torch.int64 or not t.is_contiguous():
        raise ValueError(f"ops.IncrementI64: want a contiguous I64 tensor, got {t.dtype} {tuple(t.shape)}")
    dev = _dev(t, "IncrementI64")
    _lib.check(_lib.lib().light_b200_inc_i64(_ptr(t), t.numel(), dev, _stream(dev)))


def RMSNorm(x: torch.Tensor, weight: torch.Tensor, eps: float, residual: Optional[torch.Tensor] = None):
    """ops.RMSNorm (ops/norm.go:69-111): y = x * rsqrt(mean(x^2, -1) + eps) * weight.  With `residual`, the sum
    x + residual is normalised and returned as well: (y, sum), the ops.Add before the norm in the same launch."""
    if x.device != weight.device:
        raise ValueError("ops.RMSNorm: device mismatch")
    if x.dtype != weight.dtype:
        raise ValueError(f"ops.RMSNorm: dtype mismatch (x={x.dtype}, weight={weight.dtype}) -- cast at load time")
    if x.dtype not in (torch.float32, torch.bfloat16):
        raise ValueError(f"ops.RMSNorm: dtype {x.dtype} unsupported (F32/BF16)")
    if weight.dim() != 1 or weight.shape[0] != x.shape[-1]:
        raise ValueError(f"ops.RMSNorm: weight shape {tuple(weight.shape)} incompatible with x last dim {x.shape[-1]}")
    if residual is not None and (residual.shape != x.shape or residual.dtype != x.dtype):
        raise ValueError(f"ops.RMSNorm: residual {tuple(residual.shape)} {residual.dtype} against x {tuple(x.shape)} {x.dtype}")
    dev = _dev(x, "RMSNorm")
    xc, wc = x.contiguous(), weight.contiguous()
    rc = residual.contiguous() if residual is not None else None
    out = torch.empty_like(xc)
    total = torch.empty_like(xc) if residual is not None else None
    cols = x.shape[-1]
    _lib.check(_lib.lib().light_b200_rmsnorm(_ptr(xc), _ptr(rc), _ptr(wc), _ptr(total), _ptr(out), _ACT[x.dtype], xc.numel() // cols, cols,
                                             float(eps), dev, _stream(dev)))
    return out if residual is None else (out, total)


def RoPE(x: torch.Tensor, positions: torch.Tensor, base: float) -> torch.Tensor:
    """ops.RoPE (ops/rope.go:30-77): x (..., seqLen, headDim), positions (seqLen,) I64, rotate-half pairing."""
    if x.dim() < 2:
        raise ValueError(f"ops.RoPE: x rank must be >= 2 (got {x.dim()})")
    if x.dtype not in (torch.float32, torch.bfloat16):
        raise ValueError(f"ops.RoPE: dtype {x.dtype} unsupported (F32/BF16)")
    if positions.dtype != torch.int64 or positions.dim() != 1:
        raise ValueError("ops.RoPE: positions must be 1-D I64")
    head_dim, seq_len = x.shape[-1], x.shape[-2]
    if head_dim % 2:
        raise ValueError(f"ops.RoPE: headDim must be even (got {head_dim})")
    if positions.shape[0] != seq_len:
        raise ValueError(f"ops.RoPE: positions length {positions.shape[0]} != seqLen {seq_len}")
    dev = _dev(x, "RoPE")
    xc = x.contiguous()
    out = torch.empty_like(xc)
    _lib.check(_lib.lib().light_b200_rope(_ptr(xc), _ptr(positions.contiguous()), _ptr(out), _ACT[x.dtype], xc.numel() // head_dim, seq_len,
                                          head_dim, float(base), dev, _stream(dev)))
    return out


def Argmax(x: torch.Tensor) -> torch.Tensor:
    """ops.Argmax over the last axis (ops/argmax.go:14-60): F32 (..., cols) -> I64 (...), lowest index among equals."""
    if x.dtype != torch.float32 or x.dim() < 1:
        raise ValueError(f"ops.Argmax: want an F32 tensor, got {x.dtype} {tuple(x.shape)}")
    dev = _dev(x, "Argmax")
    xc = x.contiguous()
    cols = x.shape[-1]
    out = torch.empty(x.shape[:-1], dtype=torch.int64, device=x.device)
    _lib.check(_lib.lib().light_b200_argmax(_ptr(xc), _ptr(out), xc.numel() // cols, cols, dev, _stream(dev)))
    return out


def decode_attn_status(device_index: int = 0) -> int:
    """1 if a decode-attention or append launch ever saw a position outside the cache (synchronises)."""
    return _lib.lib().light_b200_decode_attn_status(device_index)
