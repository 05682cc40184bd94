"""safetensors container reader / writer: the host side of loading GPTQ / AWQ 4-bit and block-scaled FP8 checkpoints
(reference safetensors/safetensors.go:42-262, safetensors/multi.go:16-55).

Layout: u64 little-endian header length, a JSON object {name: {dtype, shape, data_offsets}} with an optional
`__metadata__` string map, then the data section; offsets are relative to it.  Every entry is checked before anything
is read (safetensors.go:109-141): known dtype, non-negative dims, no overflow of the element or byte count,
0 <= lo <= hi, hi - lo equal to what shape and dtype imply, hi inside the data section.  Tensors come back as torch
tensors on the requested device with the bytes untouched (F8_E4M3 as torch.float8_e4m3fn, F8_E8M0 as uint8).
"""
from __future__ import annotations

import json
import os
import struct
from typing import BinaryIO, Dict, Optional, Sequence, Tuple

MAX_HEADER_LEN = 100_000_000
_MAX_INT = (1 << 63) - 1

# name -> (torch dtype name, bytes per element)  (safetensors.go:264-300)
_DTYPES = {
    "F64": ("float64", 8), "F32": ("float32", 4), "F16": ("float16", 2), "BF16": ("bfloat16", 2), "F8_E4M3": ("float8_e4m3fn", 1),
    "F8_E8M0": ("uint8", 1), "I64": ("int64", 8), "I32": ("int32", 4), "I16": ("int16", 2), "I8": ("int8", 1), "U8": ("uint8", 1),
    "U16": ("uint16", 2), "U32": ("uint32", 4), "U64": ("uint64", 8),
}


class SafetensorsError(ValueError):
    pass


def _size_of(f: BinaryIO) -> int:
    try:
        cur = f.tell()
        end = f.seek(0, os.SEEK_END)
        f.seek(cur)
        return end
    except (OSError, ValueError):
        return -1


def _read_header(f: BinaryIO):
    size = _size_of(f)
    f.seek(0)
    lb = f.read(8)
    if len(lb) != 8:
        raise SafetensorsError("safetensors: read header length: short read")
    (raw_len,) = struct.unpack("<Q", lb)
    limit = size - 8 if size >= 8 else MAX_HEADER_LEN
    if raw_len == 0 or raw_len > limit:
        raise SafetensorsError(f"safetensors: implausible header length {raw_len}")
    buf = f.read(raw_len)
    if len(buf) != raw_len:
        raise SafetensorsError("safetensors: read header: short read")
    try:
        raw = json.loads(buf)
    except (ValueError, UnicodeDecodeError) as e:
        raise SafetensorsError(f"safetensors: parse header JSON: {e}") from None
    if not isinstance(raw, dict):
        raise SafetensorsError("safetensors: parse header JSON: not an object")
    meta: Optional[Dict[str, str]] = None
    infos = {}
    for name, v in raw.items():
        if name == "__metadata__":
            if not isinstance(v, dict) or not all(isinstance(x, str) for x in v.values()):
                raise SafetensorsError("safetensors: parse __metadata__: want a string map")
            meta = v
            continue
        if (not isinstance(v, dict) or not isinstance(v.get("dtype"), str) or not isinstance(v.get("shape"), list)
                or not isinstance(v.get("data_offsets"), list) or len(v["data_offsets"]) != 2
                or not all(isinstance(d, int) and not isinstance(d, bool) for d in v["shape"] + v["data_offsets"])
                or not all(-_MAX_INT - 1 <= d <= _MAX_INT for d in v["shape"] + v["data_offsets"])):
            raise SafetensorsError(f"safetensors: parse {name!r}: malformed entry")
        infos[name] = (v["dtype"], list(v["shape"]), (v["data_offsets"][0], v["data_offsets"][1]))
    data_start = 8 + raw_len
    return infos, meta, data_start, (size - data_start if size >= 0 else -1)


def _check(name: str, info, data_len: int) -> Tuple[str, int]:
    dt, shape, (lo, hi) = info
    if dt.upper() not in _DTYPES:
        raise SafetensorsError(f"safetensors: tensor {name!r}: unsupported safetensors dtype {dt!r}")
    tname, esize = _DTYPES[dt.upper()]
    n = 1
    for i, d in enumerate(shape):
        if d < 0:
            raise SafetensorsError(f"safetensors: tensor {name!r}: negative dim {d} at axis {i}")
        if d != 0 and n > _MAX_INT // d:
            raise SafetensorsError(f"safetensors: tensor {name!r}: shape {shape} overflows")
        n *= d
    if n > _MAX_INT // esize:
        raise SafetensorsError(f"safetensors: tensor {name!r}: {dt} {shape} byte size overflows")
    if lo < 0 or hi < lo:
        raise SafetensorsError(f"safetensors: tensor {name!r}: bad byte range [{lo}, {hi})")
    if hi - lo != n * esize:
        raise SafetensorsError(f"safetensors: tensor {name!r}: header says {hi - lo} bytes, shape/dtype imply {n * esize}")
    if data_len >= 0 and hi > data_len:
        raise SafetensorsError(f"safetensors: tensor {name!r}: byte range [{lo}, {hi}) past the {data_len}-byte data section")
    return tname, n


def _read_entry(f: BinaryIO, name: str, info, data_start: int, device):
    import numpy as np
    import torch

    dt, shape, (lo, hi) = info
    tname, _ = _DTYPES[dt.upper()]
    f.seek(data_start + lo)
    buf = f.read(hi - lo)
    if len(buf) != hi - lo:
        raise SafetensorsError(f"safetensors: read {name!r}: short read")
    raw = torch.from_numpy(np.frombuffer(buf, dtype=np.uint8).copy())
    t = raw.view(getattr(torch, tname)).reshape(shape) if raw.numel() else torch.empty(shape, dtype=getattr(torch, tname))
    return t.to(device)


def header(f: BinaryIO):
    """safetensors.Header: ({name: (dtype, shape, (lo, hi))}, metadata) without touching the data section."""
    infos, meta, _, _ = _read_header(f)
    return infos, meta


def load(f: BinaryIO, device="cpu"):
    """safetensors.Load: every tensor of the file on `device`, plus the metadata map (None when absent)."""
    infos, meta, data_start, data_len = _read_header(f)
    for name, info in infos.items():
        _check(name, info, data_len)
    return {name: _read_entry(f, name, info, data_start, device) for name, info in infos.items()}, meta


def load_tensor(f: BinaryIO, name: str, device="cpu"):
    """safetensors.LoadTensor: one tensor by name; only its bytes are read."""
    infos, _, data_start, data_len = _read_header(f)
    if name not in infos:
        raise SafetensorsError(f"safetensors: no tensor named {name!r}")
    _check(name, infos[name], data_len)
    return _read_entry(f, name, infos[name], data_start, device)


def load_files(paths: Sequence[str], device="cpu"):
    """safetensors.LoadFiles (multi.go:16-55): the union of several shards; a name in two shards is an error; the
    metadata is the first shard's."""
    if not paths:
        raise SafetensorsError("safetensors.LoadFiles: no paths")
    out, first_meta = {}, None
    for i, p in enumerate(paths):
        try:
            with open(p, "rb") as f:
                shard, meta = load(f, device)
        except OSError as e:
            raise SafetensorsError(f"safetensors.LoadFiles: open {p}: {e}") from None
        except SafetensorsError as e:
            raise SafetensorsError(f"safetensors.LoadFiles: load {p}: {e}") from None
        if i == 0:
            first_meta = meta
        for name, t in shard.items():
            if name in out:
                raise SafetensorsError(f"safetensors.LoadFiles: tensor {name!r} present in multiple shards")
            out[name] = t
    return out, first_meta


def write(f: BinaryIO, tensors: Dict[str, "object"], metadata: Optional[Dict[str, str]] = None) -> None:
    """safetensors.Write (safetensors.go:193-262): names in sorted order, data back to back in that order, compact
    JSON header.  Tensors must be contiguous CPU torch tensors of a dtype the format names."""
    import torch

    rev = {getattr(torch, t): k for k, (t, _) in _DTYPES.items() if k != "F8_E8M0"}
    names = []
    for n, t in tensors.items():
        if n == "__metadata__":
            raise SafetensorsError(f"safetensors.Write: tensor name {n!r} is reserved")
        if t.dtype not in rev:
            raise SafetensorsError(f"safetensors.Write: tensor {n!r}: dtype {t.dtype} has no safetensors encoding")
        if t.device.type != "cpu":
            raise SafetensorsError(f"safetensors.Write: tensor {n!r} not on CPU")
        if not t.is_contiguous():
            raise SafetensorsError(f"safetensors.Write: tensor {n!r} not contiguous")
        names.append(n)
    names.sort()
    hdr: Dict[str, object] = {}
    if metadata:
        hdr["__metadata__"] = dict(metadata)
    off = 0
    for n in names:
        t = tensors[n]
        size = t.numel() * t.element_size()
        hdr[n] = {"dtype": rev[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + size]}
        off += size
    hj = json.dumps(hdr, separators=(",", ":")).encode()
    f.write(struct.pack("<Q", len(hj)))
    f.write(hj)
    for n in names:
        t = tensors[n]
        f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b"")


def take_int4(hf: Dict[str, "object"], mod: str, method: str, group: int, device, v2: bool = False):
    """takeInt4 (models/int4_load.go:169-207): the 4-bit module `mod` of a loaded checkpoint (qweight, qzeros, scales and,
    for GPTQ, g_idx) -> ops.Int4 on `device`, removing those tensors from `hf`.  `method` is "gptq" or "awq", `v2` the
    checkpoint_format "gptq_v2"; the repack into the (N, K/8) row layout runs on the device (light_b200_int4_repack).
    A g_idx that is not the ordered k // group (quant/int4.go:122-151, 177-195): K is sorted stably by group, qweight's
    rows are taken in that order before the repack, and the order is kept as the weight's activation permutation."""
    import torch

    from . import ops

    def take(name):
        if name not in hf:
            raise SafetensorsError(f"{method}: missing tensor {name!r}")
        return hf.pop(name)

    qw, qz, sc = take(mod + ".qweight").to(device), take(mod + ".qzeros").to(device), take(mod + ".scales").to(device).float()
    if method != "gptq":
        return ops.Int4FromCheckpoint(qw, qz, sc, group, "awq")
    perm = None
    gi = hf.pop(mod + ".g_idx", None)
    if gi is not None:
        K = qw.shape[0] * 8
        g = gi.to(torch.int64).cpu()
        gsz = group if group > 0 else K
        if g.numel() != K:
            raise SafetensorsError(f"quant.FromGPTQ: g_idx has {g.numel()} entries for K {K}")
        if not torch.equal(g, torch.arange(K) // gsz):
            perm = torch.sort(g, stable=True).indices
            if not torch.equal(g[perm], torch.arange(K) // gsz):
                raise SafetensorsError(f"quant.FromGPTQ: g_idx groups are not all of size {gsz}")
            perm = perm.to(device)
            shifts = (torch.arange(8, device=qw.device, dtype=torch.int32) * 4).view(1, 8, 1)
            rows = ((qw.view(torch.int32).unsqueeze(1) >> shifts) & 0xF).reshape(K, -1).index_select(0, perm)    # (K, N) nibbles in sorted order
            packed = (rows.reshape(K // 8, 8, -1).to(torch.int64) << shifts.to(torch.int64)).sum(1)
            qw = torch.where(packed >= 1 << 31, packed - (1 << 32), packed).to(torch.int32)    # the same 32 bits as I32
    w = ops.Int4FromCheckpoint(qw, qz, sc, group, "gptq_v2" if v2 else "gptq")
    w.perm = perm
    return w
