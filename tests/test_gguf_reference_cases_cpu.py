"""The GGUF reader against byte streams assembled field by field, independently of light_b200.gguf.write(): the
malformed inputs the reference lists (gguf/validate_test.go:48-88: counts, ranks, products and offsets that the
input cannot hold must be errors, never allocations or crashes) and the valid files its tests build from explicit
fields (gguf/gguf_test.go:26-160: scalar metadata of every kind, a string array, an F32 tensor of dims [2, 3],
a hand-built Q4_0 block; gguf/validate_test.go:92-130: two tensors, the second read back)."""
import io
import struct

import numpy as np
import pytest

from light_b200 import gguf

U64_MAX, U32_MAX, I64_MAX = (1 << 64) - 1, (1 << 32) - 1, (1 << 63) - 1


def stream(n_tensors, n_kv, body=b"", version=3):
    """gguf/validate_test.go:23-30 (ggufStream)."""
    return struct.pack("<IIQQ", 0x46554747, version, n_tensors, n_kv) + body


def s(text):
    b = text.encode()
    return struct.pack("<Q", len(b)) + b


def tensor_info(name, dims, off, ggml_type=0):
    """gguf/validate_test.go:37-46 (tensorInfo)."""
    return s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", ggml_type, off)


def array_kv(elem_type, n):
    return s("k") + struct.pack("<IIQ", gguf.T_ARR, elem_type, n)


NESTED = s("deep") + struct.pack("<I", gguf.T_ARR) + b"".join(struct.pack("<IQ", gguf.T_ARR, 1) for _ in range(100))

MALFORMED = {
    "array count MaxUint64": stream(0, 1, array_kv(gguf.T_U8, U64_MAX)),
    "array of u64 too long": stream(0, 1, array_kv(gguf.T_U64, 4) + bytes(16)),
    "array of arrays too big": stream(0, 1, array_kv(gguf.T_ARR, 1 << 40)),
    "kv count MaxUint64": stream(0, U64_MAX),
    "tensor count MaxUint64": stream(U64_MAX, 0),
    "deep nesting": stream(0, 1, NESTED),
    "huge rank": stream(1, 0, s("t") + struct.pack("<I", U32_MAX)),
    "dims product overflow": stream(1, 0, tensor_info("t", [1 << 32, 1 << 32], 0)),
    "byte size overflow": stream(1, 0, tensor_info("t", [1 << 62], 0)),
    "offset overflow": stream(1, 0, tensor_info("t", [1], U64_MAX - 2)),
    "offset near MaxInt64": stream(1, 0, tensor_info("t", [4], I64_MAX - 8)),
    "string length too big": stream(0, 1, struct.pack("<Q", 1 << 29)),
    "tensor data past end of input": stream(1, 0, tensor_info("t", [1000], 0)),
    "bad magic": bytes(32),
    "version 1": stream(0, 0, version=1),
    "version 4": stream(0, 0, version=4),
    "unknown ggml type": stream(1, 0, tensor_info("t", [32], 0, ggml_type=99) + bytes(64)),
    "unknown value type": stream(0, 1, s("k") + struct.pack("<I", 77) + bytes(8)),
    "truncated header": struct.pack("<II", 0x46554747, 3),
}


@pytest.mark.parametrize("name", sorted(MALFORMED))
def test_malformed_inputs_are_errors(name):
    with pytest.raises(gguf.GGUFError):
        gguf.File(io.BytesIO(MALFORMED[name]))


def _kv(key, vtype, payload):
    return s(key) + struct.pack("<I", vtype) + payload


def _pad(b, align):
    return b + bytes((-len(b)) % align)


def q4_0_block(scale, vals):
    """quant/others_test.go (buildQ4_0BlockRaw): f16 scale, then byte j = (vals[j] + 8) | (vals[j + 16] + 8) << 4."""
    out = bytearray(np.float16(scale).tobytes())
    for j in range(16):
        out.append(((vals[j] + 8) & 0xF) | (((vals[j + 16] + 8) & 0xF) << 4))
    return bytes(out)


@pytest.mark.parametrize("align", [32, 64])
def test_file_assembled_from_explicit_fields(align, oracle):
    """The contents of TestGGUFRoundTripScalar / TestGGUFQuantTensorLoadsAndDequantizes / TestSizedRoundTrip in one file."""
    kvs = [
        _kv("general.name", gguf.T_STR, s("toy-model")),
        _kv("general.architecture_version", gguf.T_U32, struct.pack("<I", 1)),
        _kv("block_count", gguf.T_I64, struct.pack("<q", 4)),
        _kv("rope_theta", gguf.T_F32, struct.pack("<f", 10000.0)),
        _kv("is_quantized", gguf.T_BOOL, b"\x01"),
        _kv("tokenizer.tokens", gguf.T_ARR, struct.pack("<IQ", gguf.T_STR, 2) + s("hello") + s("world")),
        _kv("small", gguf.T_I8, struct.pack("<b", -3)),
        _kv("wide", gguf.T_F64, struct.pack("<d", 2.5)),
        _kv("general.alignment", gguf.T_U32, struct.pack("<I", align)),
    ]
    f32 = np.arange(1, 7, dtype="<f4").tobytes()                 # dims [2, 3] as the test passes them
    vals = [(i % 16) - 8 for i in range(32)]
    q4 = q4_0_block(0.5, vals)
    b_vals = np.array([4, 5], dtype="<f4").tobytes()
    payloads = [("weight", [2, 3], 0, f32), ("w", [32], 2, q4), ("b", [2], 0, b_vals)]
    table, data = b"", b""
    for name, dims, gt, blob in payloads:
        table += tensor_info(name, dims, len(data), ggml_type=gt)
        data = _pad(data + blob, align)
    head = _pad(stream(len(payloads), len(kvs), b"".join(kvs) + table), align)
    f = gguf.File(io.BytesIO(head + data))
    assert f.version == 3
    assert f.meta["general.name"] == "toy-model" and f.meta["block_count"] == 4 and f.meta["rope_theta"] == 10000.0
    assert f.meta["is_quantized"] is True and f.meta["tokenizer.tokens"] == ["hello", "world"]
    assert f.meta["small"] == -3 and f.meta["wide"] == 2.5 and f.meta["general.architecture_version"] == 1
    assert list(f.meta)[:2] == ["general.name", "general.architecture_version"]       # declaration order (KeyOrder)
    assert list(f.tensors) == ["weight", "w", "b"]                                      # declaration order (Order)
    assert f.data_base == len(head)
    w = f.tensors["weight"]
    assert w.dims == [2, 3] and w.shape_row_major == (3, 2) and w.nbytes == 24
    assert np.array_equal(np.frombuffer(f.tensor_bytes("weight"), "<f4"), np.arange(1, 7, dtype=np.float32))
    assert np.array_equal(np.frombuffer(f.tensor_bytes("b"), "<f4"), np.array([4, 5], np.float32))
    # the Q4_0 block: bytes untouched, and the decoder gives scale * value (|error| <= 1e-5, the reference's bound)
    raw = f.tensor_bytes("w")
    assert raw == q4 and f.tensors["w"].ggml_type == 2 and f.tensors["w"].nbytes == 18
    deq = oracle.dequant(2, np.frombuffer(raw, np.uint8), 32)
    assert np.max(np.abs(deq - 0.5 * np.array(vals, np.float32))) <= 1e-5
    with pytest.raises(gguf.GGUFError):
        f.tensor_bytes("nope")


def test_header_only_file():
    """TestGGUFEmptyFile: zero tensors; here the alignment key is absent, so the default of 32 applies."""
    f = gguf.File(io.BytesIO(stream(0, 0)))
    assert f.tensors == {} and f.meta == {} and f.data_base == 32
    f2 = gguf.File(io.BytesIO(stream(0, 0, version=2)))
    assert f2.version == 2


def test_alignment_rules():
    """gguf/reader.go:166-176: a non-positive or non-integer general.alignment keeps 32; one above 2^30 is an error."""
    ok = stream(0, 1, _kv("general.alignment", gguf.T_I32, struct.pack("<i", -8)))
    assert gguf.File(io.BytesIO(ok)).data_base % 32 == 0
    big = stream(0, 1, _kv("general.alignment", gguf.T_U64, struct.pack("<Q", 1 << 31)))
    with pytest.raises(gguf.GGUFError):
        gguf.File(io.BytesIO(big))
