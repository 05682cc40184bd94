"""GGUF container reader: the host side of loading quantized weights (reference gguf/reader.go:23-264,
gguf/types.go:9-110).  Little-endian header `GGUF` (0x46554747), versions 2-3, metadata key/values, a tensor
table (name, dims innermost-first, ggml type, offset), then the data section at the next multiple of
`general.alignment` (default 32).  Tensor bytes are returned untouched: the block formats go to the device as they
lie on disk, nothing is repacked (models/llama_gguf.go:32-151).

`write()` produces such a file from in-memory tensors; the tests use it, as the reference's own tests build their
inputs in memory (gguf/reader_test.go).
"""
from __future__ import annotations

import struct
from dataclasses import dataclass
from typing import Any, BinaryIO, Dict, List, Sequence, Tuple

MAGIC = 0x46554747
MIN_VERSION, MAX_VERSION = 2, 3
MAX_RANK, MAX_ARRAY_DEPTH, MAX_ALIGN = 16, 8, 1 << 30

# value types (gguf/types.go:20-34)
T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64 = range(13)
_SCALAR = {T_U8: "<B", T_I8: "<b", T_U16: "<H", T_I16: "<h", T_U32: "<I", T_I32: "<i", T_F32: "<f", T_U64: "<Q", T_I64: "<q", T_F64: "<d"}

# ggml tensor types -> (name, elements per block, bytes per block)  (gguf/types.go:38-110, dtype/dtype.go:53-102)
GGML_TYPES = {
    0: ("F32", 1, 4), 1: ("F16", 1, 2), 2: ("Q4_0", 32, 18), 3: ("Q4_1", 32, 20), 6: ("Q5_0", 32, 22), 7: ("Q5_1", 32, 24),
    8: ("Q8_0", 32, 34), 9: ("Q8_1", 32, 36), 10: ("Q2_K", 256, 84), 11: ("Q3_K", 256, 110), 12: ("Q4_K", 256, 144),
    13: ("Q5_K", 256, 176), 14: ("Q6_K", 256, 210), 15: ("Q8_K", 256, 292), 24: ("I8", 1, 1), 25: ("I16", 1, 2),
    26: ("I32", 1, 4), 27: ("I64", 1, 8), 28: ("F64", 1, 8), 30: ("BF16", 1, 2),
}


class GGUFError(ValueError):
    pass


@dataclass
class TensorInfo:
    name: str
    ggml_type: int
    dims: List[int]   # innermost first, as stored
    offset: int       # relative to the data section
    nbytes: int

    @property
    def shape_row_major(self) -> Tuple[int, ...]:
        """Dims reversed (outermost first), the order TensorRowMajor hands to tensor.FromBytes (gguf/reader.go:237-251)."""
        return tuple(reversed(self.dims))


class _Cursor:
    def __init__(self, f: BinaryIO, size: int):
        self.f, self.size, self.pos = f, size, 0

    def take(self, n: int) -> bytes:
        if n < 0 or self.pos + n > self.size:
            raise GGUFError(f"gguf: read of {n} bytes at {self.pos} past end of {self.size}-byte input")
        self.f.seek(self.pos)
        b = self.f.read(n)
        if len(b) != n:
            raise GGUFError(f"gguf: short read at {self.pos}")
        self.pos += n
        return b

    def scalar(self, fmt: str):
        return struct.unpack(fmt, self.take(struct.calcsize(fmt)))[0]

    def string(self) -> str:
        n = self.scalar("<Q")
        if n > self.size - self.pos:
            raise GGUFError(f"gguf: string of {n} bytes past end of input")
        return self.take(n).decode("utf-8", errors="replace")

    def value(self, vtype: int, depth: int) -> Any:
        if vtype in _SCALAR:
            return self.scalar(_SCALAR[vtype])
        if vtype == T_BOOL:
            return self.scalar("<B") != 0
        if vtype == T_STR:
            return self.string()
        if vtype == T_ARR:
            if depth >= MAX_ARRAY_DEPTH:
                raise GGUFError(f"gguf: arrays nested deeper than {MAX_ARRAY_DEPTH}")
            et, n = self.scalar("<I"), self.scalar("<Q")
            if n > self.size - self.pos:  # every element takes at least one byte
                raise GGUFError(f"gguf: array of {n} elements past end of input")
            return [self.value(et, depth + 1) for _ in range(n)]
        raise GGUFError(f"gguf: unknown value type {vtype}")


class File:
    """gguf.File (gguf/reader.go:31-191): Version, Meta (in declaration order), Tensors (in declaration order)."""

    def __init__(self, f: BinaryIO):
        f.seek(0, 2)
        r = _Cursor(f, f.tell())
        self._f = f
        magic = r.scalar("<I")
        if magic != MAGIC:
            raise GGUFError(f"gguf: bad magic {magic:#x} (want {MAGIC:#x})")
        self.version = r.scalar("<I")
        if not MIN_VERSION <= self.version <= MAX_VERSION:
            raise GGUFError(f"gguf: version {self.version} not in [{MIN_VERSION}, {MAX_VERSION}]")
        n_tensors, n_kv = r.scalar("<Q"), r.scalar("<Q")
        if n_kv * 13 > r.size or n_tensors * 24 > r.size:
            raise GGUFError("gguf: metadata or tensor count larger than the input")
        self.meta: Dict[str, Any] = {}
        for _ in range(n_kv):
            key = r.string()
            self.meta[key] = r.value(r.scalar("<I"), 0)
        self.tensors: Dict[str, TensorInfo] = {}
        for _ in range(n_tensors):
            name = r.string()
            nd = r.scalar("<I")
            if nd > MAX_RANK:
                raise GGUFError(f"gguf: tensor[{name!r}] rank {nd} exceeds {MAX_RANK}")
            dims = [r.scalar("<Q") for _ in range(nd)]
            gt = r.scalar("<I")
            if gt not in GGML_TYPES:
                raise GGUFError(f"gguf: tensor[{name!r}]: unsupported ggml type {gt}")
            off = r.scalar("<Q")
            n = 1
            for d in dims:
                n *= d
            _, be, bb = GGML_TYPES[gt]
            blocks = 0 if n == 0 else (n - 1) // be + 1
            self.tensors[name] = TensorInfo(name, gt, dims, off, blocks * bb)
        align = 32
        a = self.meta.get("general.alignment")
        if isinstance(a, int) and not isinstance(a, bool) and a > 0:
            align = a
        if align > MAX_ALIGN:
            raise GGUFError(f"gguf: general.alignment {align} exceeds {MAX_ALIGN}")
        self.data_base = (r.pos + align - 1) // align * align
        for t in self.tensors.values():
            end = self.data_base + t.offset + t.nbytes
            if end > r.size:
                raise GGUFError(f"gguf: tensor[{t.name!r}] data [{self.data_base + t.offset}, {end}) past end of {r.size}-byte input")

    def tensor_bytes(self, name: str) -> bytes:
        """File.TensorBytes: the tensor's payload exactly as stored."""
        t = self.tensors.get(name)
        if t is None:
            raise GGUFError(f"gguf: tensor {name!r} not found")
        self._f.seek(self.data_base + t.offset)
        b = self._f.read(t.nbytes)
        if len(b) != t.nbytes:
            raise GGUFError(f"gguf: read tensor {name!r}: short read")
        return b

    def qtensor(self, name: str, device):
        """File.TensorRowMajor for a block-quantized weight: an ops.QTensor (N, K) on `device`, bytes untouched."""
        import numpy as np
        import torch

        from . import ops

        t = self.tensors[name] if name in self.tensors else None
        if t is None:
            raise GGUFError(f"gguf: tensor {name!r} not found")
        if t.ggml_type not in ops.GGUF_NAMES:
            raise GGUFError(f"gguf: tensor {name!r} has ggml type {t.ggml_type}, which has no fused kernel")
        raw = torch.from_numpy(np.frombuffer(self.tensor_bytes(name), dtype=np.uint8).copy())
        return ops.QTensor(raw.to(device), t.ggml_type, t.shape_row_major)


    def _row_bytes(self, t: TensorInfo) -> int:
        _, be, bb = GGML_TYPES[t.ggml_type]
        if t.dims[0] % be:
            raise GGUFError(f"gguf: tensor {t.name!r}: inner dim {t.dims[0]} is not a whole number of {be}-element blocks")
        return t.dims[0] // be * bb

    def qtensor_unpermuted(self, name: str, heads: int, device):
        """loadGGUFLinearWeightUnpermuted (models/llama_gguf.go:343-382): a llama attn_q / attn_k weight with the
        converter's row interleave undone.  File row h*hd + 2i + s holds the row h*hd + s*hd/2 + i of the original
        checkpoint; a row is a whole run of blocks, so the rows move as bytes and stay quantized."""
        import numpy as np
        import torch

        from . import ops

        t = self.tensors.get(name)
        if t is None:
            raise GGUFError(f"gguf: tensor {name!r} not found")
        if len(t.dims) != 2 or heads <= 0 or t.dims[1] % (2 * heads):
            raise GGUFError(f"gguf: tensor {name!r} dims {t.dims} cannot be un-permuted over {heads} heads")
        rb = self._row_bytes(t)
        N = t.dims[1]
        if rb * N != t.nbytes:
            raise GGUFError(f"{name}: {t.nbytes} bytes, want {N} rows x {rb}")
        rows = np.frombuffer(self.tensor_bytes(name), dtype=np.uint8).reshape(N, rb)
        out = unpermute_rows(rows, heads)
        return ops.QTensor(torch.from_numpy(out.reshape(-1)).to(device), t.ggml_type, (N, t.dims[0]))

    def moe_gate_up(self, gate_name: str, up_name: str, device):
        """The fused (E, 2 I, H) expert tensor of loadGGUFMoE (models/llama_gguf.go:153-216): expert e's gate rows
        followed by its up rows, concatenated as bytes (a row is a whole number of blocks)."""
        import numpy as np
        import torch

        from . import ops

        gi, ui = self.tensors.get(gate_name), self.tensors.get(up_name)
        if gi is None:
            raise GGUFError(f"{gate_name} missing")
        if ui is None or ui.ggml_type != gi.ggml_type or len(gi.dims) != 3 or ui.dims != gi.dims:
            raise GGUFError(f"{up_name} missing or mismatched")
        H, I, E = gi.dims
        slab = self._row_bytes(gi) * I
        gb = np.frombuffer(self.tensor_bytes(gate_name), dtype=np.uint8).reshape(E, slab)
        ub = np.frombuffer(self.tensor_bytes(up_name), dtype=np.uint8).reshape(E, slab)
        fused = concat_expert_slabs(gb, ub)
        return ops.QTensor(torch.from_numpy(fused.reshape(-1)).to(device), gi.ggml_type, (E, 2 * I, H))


def unpermute_rows(rows, heads: int):
    """rows (N, row_bytes) uint8 -> the same rows with dst h*hd + s*hd/2 + i taken from src h*hd + 2i + s."""
    import numpy as np

    N = rows.shape[0]
    hd = N // heads
    half = hd // 2
    # src index as a (heads, half, 2) array read in (heads, 2, half) order
    src = np.arange(N).reshape(heads, half, 2).transpose(0, 2, 1).reshape(-1)
    return np.ascontiguousarray(rows[src])


def concat_expert_slabs(gate, up):
    """gate, up (E, slab_bytes) uint8 -> (E, 2 * slab_bytes): every expert's gate slab, then its up slab."""
    import numpy as np

    return np.ascontiguousarray(np.concatenate([gate, up], axis=1))


def open_file(path: str) -> File:
    return File(open(path, "rb"))


def _enc_value(v: Any) -> Tuple[int, bytes]:
    if isinstance(v, bool):
        return T_BOOL, struct.pack("<B", int(v))
    if isinstance(v, int):
        return (T_U32, struct.pack("<I", v)) if 0 <= v < 2**32 else (T_I64, struct.pack("<q", v))
    if isinstance(v, float):
        return T_F32, struct.pack("<f", v)
    if isinstance(v, str):
        b = v.encode()
        return T_STR, struct.pack("<Q", len(b)) + b
    if isinstance(v, (list, tuple)):
        encs = [_enc_value(x) for x in v]
        et = encs[0][0] if encs else T_U32
        if any(e[0] != et for e in encs):
            raise GGUFError("gguf: arrays hold one element type")
        return T_ARR, struct.pack("<IQ", et, len(encs)) + b"".join(e[1] for e in encs)
    raise GGUFError(f"gguf: cannot encode {type(v).__name__}")


def write(f: BinaryIO, meta: Dict[str, Any], tensors: Sequence[Tuple[str, int, Sequence[int], bytes]], version: int = 3) -> None:
    """Writes a GGUF file: tensors are (name, ggml type, dims innermost-first, payload bytes)."""
    align = int(meta.get("general.alignment", 32))
    head = struct.pack("<IIQQ", MAGIC, version, len(tensors), len(meta))
    for k, v in meta.items():
        kb = k.encode()
        vt, vb = _enc_value(v)
        head += struct.pack("<Q", len(kb)) + kb + struct.pack("<I", vt) + vb
    off, table, blobs = 0, b"", []
    for name, gt, dims, payload in tensors:
        nb = name.encode()
        table += struct.pack("<Q", len(nb)) + nb + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        table += struct.pack("<IQ", gt, off)
        blobs.append((off, payload))
        off = (off + len(payload) + align - 1) // align * align
    f.write(head + table)
    base = (len(head) + len(table) + align - 1) // align * align
    f.write(b"\0" * (base - len(head) - len(table)))
    for o, payload in blobs:
        f.seek(base + o)
        f.write(payload)
