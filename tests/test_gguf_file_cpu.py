"""The GGUF container reader (gguf/reader.go:23-264 mirrored in light_b200/gguf.py) on files built in memory:
header, metadata of every value kind, the tensor table, data-section alignment, untouched payload bytes, and the
reader's refusals (bad magic, versions outside 2-3, truncated data)."""
import io
import struct

import numpy as np
import pytest

from light_b200 import gguf, ops, synth


def _file(align=None, version=3):
    w1 = synth.random_blocks(950, ops.Q4_K, 8, 512)   # (N = 8, K = 512): dims on disk are (512, 8)
    w2 = synth.random_blocks(951, ops.Q6_K, 3, 256)
    f32 = np.arange(6, dtype=np.float32)
    meta = {"general.architecture": "llama", "llama.block_count": 2, "llama.rope.freq_base": 500000.0, "flag": True,
            "tokenizer.ggml.tokens": ["a", "b", "c"], "big": -(2**40), "nested": [[1, 2], [3, 4]]}
    if align:
        meta["general.alignment"] = align
    buf = io.BytesIO()
    gguf.write(buf, meta, [("blk.0.attn_q.weight", ops.Q4_K, (512, 8), w1.tobytes()), ("blk.0.ffn_down.weight", ops.Q6_K, (256, 3), w2.tobytes()),
                            ("norm", 0, (6,), f32.tobytes())], version=version)
    return buf, meta, w1, w2, f32


@pytest.mark.parametrize("align", [None, 64, 4096])
def test_round_trip(align):
    buf, meta, w1, w2, f32 = _file(align)
    f = gguf.File(buf)
    assert f.version == 3 and list(f.meta) == list(meta)
    assert f.meta["llama.block_count"] == 2 and f.meta["flag"] is True and f.meta["big"] == -(2**40)
    assert f.meta["tokenizer.ggml.tokens"] == ["a", "b", "c"] and f.meta["nested"] == [[1, 2], [3, 4]]
    assert abs(f.meta["llama.rope.freq_base"] - 500000.0) < 1e-3
    assert f.data_base % (align or 32) == 0
    t = f.tensors["blk.0.attn_q.weight"]
    assert t.dims == [512, 8] and t.shape_row_major == (8, 512) and t.nbytes == 8 * 2 * 144
    assert f.tensor_bytes("blk.0.attn_q.weight") == w1.tobytes()
    assert f.tensor_bytes("blk.0.ffn_down.weight") == w2.tobytes() and f.tensors["blk.0.ffn_down.weight"].nbytes == 3 * 210
    assert np.array_equal(np.frombuffer(f.tensor_bytes("norm"), np.float32), f32)
    assert list(f.tensors) == ["blk.0.attn_q.weight", "blk.0.ffn_down.weight", "norm"]


def test_refusals():
    buf, *_ = _file()
    raw = buf.getvalue()
    with pytest.raises(gguf.GGUFError, match="bad magic"):
        gguf.File(io.BytesIO(b"GGML" + raw[4:]))
    with pytest.raises(gguf.GGUFError, match="version"):
        gguf.File(io.BytesIO(raw[:4] + struct.pack("<I", 1) + raw[8:]))
    with pytest.raises(gguf.GGUFError, match="past end"):
        gguf.File(io.BytesIO(raw[:-100]))
    with pytest.raises(gguf.GGUFError, match="not found"):
        gguf.File(io.BytesIO(raw)).tensor_bytes("missing")
    assert gguf.File(_file(version=2)[0]).version == 2


def test_payload_feeds_the_oracle(oracle):
    """The bytes read back decode to the same weights as the bytes written (nothing is repacked on the way)."""
    buf, _, w1, _, _ = _file()
    f = gguf.File(buf)
    raw = np.frombuffer(f.tensor_bytes("blk.0.attn_q.weight"), np.uint8)
    assert np.array_equal(oracle.dequant(ops.Q4_K, raw, 8 * 512), oracle.dequant(ops.Q4_K, w1.reshape(-1), 8 * 512))
