"""Loader-side helpers that sit in front of the quantized matmuls.

GGUF (models/llama_gguf.go:153-216, 343-382): the llama attn_q / attn_k row un-permute and the per-expert gate / up
concatenation, both on raw block bytes.  safetensors (safetensors/safetensors.go, safetensors/validate_test.go): round
trips, and the reference's list of malformed headers, each of which must be refused before anything is read."""
import io
import json
import struct

import numpy as np
import pytest
import torch

from light_b200 import gguf, ops, safetensors, synth


def _gguf_with(tensors):
    buf = io.BytesIO()
    gguf.write(buf, {"general.architecture": "llama"}, tensors)
    return gguf.File(buf)


@pytest.mark.parametrize("dt,K", [(ops.Q4_K, 512), (ops.Q6_K, 256), (ops.Q8_0, 64)])
def test_unpermute_rows_inverts_the_converter(dt, K, oracle):
    """The converter reshapes (heads, 2, hd/2, K) -> swap(1, 2): file row h*hd + 2i + s holds row h*hd + s*hd/2 + i.
    Decoding the un-permuted bytes gives the original rows."""
    heads, hd = 3, 8
    N = heads * hd
    orig = synth.random_blocks(31, dt, N, K)                      # (N, row_bytes) as the checkpoint has them
    rows = orig.reshape(N, -1)
    file_rows = rows.reshape(heads, 2, hd // 2, -1).swapaxes(1, 2).reshape(N, -1)     # what the converter writes
    assert not np.array_equal(file_rows, rows)
    f = _gguf_with([("blk.0.attn_q.weight", dt, (K, N), np.ascontiguousarray(file_rows).tobytes())])
    got = gguf.unpermute_rows(np.frombuffer(f.tensor_bytes("blk.0.attn_q.weight"), np.uint8).reshape(N, -1), heads)
    assert np.array_equal(got, rows)
    # row by row, as the reference's loop states it
    half = hd // 2
    for h in range(heads):
        for s in range(2):
            for i in range(half):
                assert np.array_equal(got[h * hd + s * half + i], file_rows[h * hd + 2 * i + s])
    want = oracle.dequant(dt, rows.reshape(-1), N * K)
    assert np.array_equal(oracle.dequant(dt, got.reshape(-1), N * K), want)
    q = f.qtensor_unpermuted("blk.0.attn_q.weight", heads, "cpu")
    assert q.shape == (N, K) and np.array_equal(q.data.numpy(), rows.reshape(-1))


def test_unpermute_refusals():
    w = synth.random_blocks(32, ops.Q4_K, 6, 256)
    f = _gguf_with([("q", ops.Q4_K, (256, 6), w.tobytes())])
    with pytest.raises(gguf.GGUFError, match="not found"):
        f.qtensor_unpermuted("missing", 2, "cpu")
    with pytest.raises(gguf.GGUFError, match="cannot be un-permuted"):
        f.qtensor_unpermuted("q", 4, "cpu")          # 6 rows do not split into 4 heads of an even size


def test_moe_gate_up_concat(oracle):
    """(E, I, H) gate and up -> (E, 2 I, H): expert e's gate rows then its up rows, byte for byte."""
    E, I, H = 4, 6, 512
    gate = synth.random_blocks(33, ops.Q4_K, E * I, H)
    up = synth.random_blocks(34, ops.Q4_K, E * I, H)
    f = _gguf_with([("blk.1.ffn_gate_exps.weight", ops.Q4_K, (H, I, E), gate.tobytes()), ("blk.1.ffn_up_exps.weight", ops.Q4_K, (H, I, E), up.tobytes()),
                    ("blk.1.ffn_up_other.weight", ops.Q6_K, (H, I, E), synth.random_blocks(35, ops.Q6_K, E * I, H).tobytes())])
    q = f.moe_gate_up("blk.1.ffn_gate_exps.weight", "blk.1.ffn_up_exps.weight", "cpu")
    assert q.shape == (E, 2 * I, H) and q.ggml_type == ops.Q4_K
    rb = H // 256 * 144
    fused = q.data.numpy().reshape(E, 2 * I, rb)
    g3, u3 = gate.reshape(E, I, rb), up.reshape(E, I, rb)
    for e in range(E):
        assert np.array_equal(fused[e, :I], g3[e]) and np.array_equal(fused[e, I:], u3[e])
    d = oracle.dequant(ops.Q4_K, q.data.numpy(), E * 2 * I * H).reshape(E, 2 * I, H)
    assert np.array_equal(d[2, I + 1], oracle.dequant(ops.Q4_K, u3[2, 1], H))
    with pytest.raises(gguf.GGUFError, match="missing or mismatched"):
        f.moe_gate_up("blk.1.ffn_gate_exps.weight", "blk.1.ffn_up_other.weight", "cpu")
    with pytest.raises(gguf.GGUFError, match="missing"):
        f.moe_gate_up("nope", "blk.1.ffn_up_exps.weight", "cpu")


# --------------------------------------------------------------------------- safetensors

def _raw(header: str, data: bytes = b"") -> bytes:
    h = header.encode()
    return struct.pack("<Q", len(h)) + h + data


def test_safetensors_round_trip(tmp_path):
    g = torch.Generator().manual_seed(5)
    tensors = {
        "model.layers.0.q_proj.qweight": torch.randint(-2**31, 2**31 - 1, (16, 8), generator=g, dtype=torch.int64).to(torch.int32),
        "model.layers.0.q_proj.scales": torch.randn(2, 8, generator=g).to(torch.float16),
        "w.fp8": torch.randn(4, 128, generator=g).to(torch.float8_e4m3fn),
        "w.scale_inv": torch.rand(1, 1, generator=g),
        "bf": torch.randn(3, 5, generator=g).to(torch.bfloat16),
        "empty": torch.zeros(0, 4),
        "ids": torch.arange(7, dtype=torch.int64),
    }
    buf = io.BytesIO()
    safetensors.write(buf, tensors, {"format": "pt"})
    raw = buf.getvalue()
    (hl,) = struct.unpack("<Q", raw[:8])
    hdr = json.loads(raw[8:8 + hl])
    assert hdr["__metadata__"] == {"format": "pt"}
    names = [n for n in hdr if n != "__metadata__"]
    assert names == sorted(names)                                   # data laid out in name order, back to back
    off = 0
    for n in names:
        assert hdr[n]["data_offsets"][0] == off
        off = hdr[n]["data_offsets"][1]
    assert off == len(raw) - 8 - hl and hdr["w.fp8"]["dtype"] == "F8_E4M3" and hdr["empty"]["data_offsets"][0] == hdr["empty"]["data_offsets"][1]
    got, meta = safetensors.load(io.BytesIO(raw))
    assert meta == {"format": "pt"} and set(got) == set(tensors)
    for n, t in tensors.items():
        assert got[n].dtype == t.dtype and got[n].shape == t.shape, n
        assert torch.equal(got[n].reshape(-1).view(torch.uint8), t.reshape(-1).view(torch.uint8)) if t.numel() else True, n
    one = safetensors.load_tensor(io.BytesIO(raw), "bf")
    assert torch.equal(one, tensors["bf"])
    with pytest.raises(safetensors.SafetensorsError, match="no tensor named"):
        safetensors.load_tensor(io.BytesIO(raw), "nope")
    infos, _ = safetensors.header(io.BytesIO(raw))
    assert infos["ids"] == ("I64", [7], tuple(hdr["ids"]["data_offsets"]))
    # two shards: union; a duplicate name is refused
    p1, p2 = tmp_path / "a.safetensors", tmp_path / "b.safetensors"
    with open(p1, "wb") as f:
        safetensors.write(f, {"x": torch.ones(2)}, {"shard": "1"})
    with open(p2, "wb") as f:
        safetensors.write(f, {"y": torch.zeros(3)})
    both, meta = safetensors.load_files([str(p1), str(p2)])
    assert set(both) == {"x", "y"} and meta == {"shard": "1"}
    with pytest.raises(safetensors.SafetensorsError, match="multiple shards"):
        safetensors.load_files([str(p1), str(p1)])
    with pytest.raises(safetensors.SafetensorsError, match="no paths"):
        safetensors.load_files([])


def test_safetensors_write_refusals():
    with pytest.raises(safetensors.SafetensorsError, match="reserved"):
        safetensors.write(io.BytesIO(), {"__metadata__": torch.ones(1)})
    with pytest.raises(safetensors.SafetensorsError, match="not contiguous"):
        safetensors.write(io.BytesIO(), {"t": torch.ones(4, 4).t()[1:]})
    with pytest.raises(safetensors.SafetensorsError, match="no safetensors encoding"):
        safetensors.write(io.BytesIO(), {"c": torch.ones(2, dtype=torch.complex64)})


# The malformed headers the reference's reader must refuse (safetensors/validate_test.go:66-78), four data bytes behind each.
MALFORMED = {
    "reversed range": '{"x":{"dtype":"F32","shape":[1],"data_offsets":[4,0]}}',
    "negative offsets": '{"x":{"dtype":"F32","shape":[1],"data_offsets":[-12,-8]}}',
    "very negative": '{"x":{"dtype":"F32","shape":[1],"data_offsets":[-9000000000000000000,-8999999999999999996]}}',
    "negative dim": '{"x":{"dtype":"F32","shape":[-1],"data_offsets":[0,0]}}',
    "negative dim pair": '{"x":{"dtype":"F32","shape":[-1,-4],"data_offsets":[0,16]}}',
    "shape overflow": '{"x":{"dtype":"F32","shape":[4611686018427387904,4],"data_offsets":[0,0]}}',
    "byte size overflow": '{"x":{"dtype":"F64","shape":[2305843009213693952],"data_offsets":[0,0]}}',
    "past data end": '{"x":{"dtype":"F32","shape":[1000000000],"data_offsets":[0,4000000000]}}',
    "bad dtype": '{"x":{"dtype":"Q9","shape":[1],"data_offsets":[0,4]}}',
    "size mismatch": '{"x":{"dtype":"F32","shape":[2],"data_offsets":[0,4]}}',
}


@pytest.mark.parametrize("name", sorted(MALFORMED))
def test_safetensors_malformed_headers(name, tmp_path):
    raw = _raw(MALFORMED[name], bytes([1, 2, 3, 4]))
    with pytest.raises(safetensors.SafetensorsError):
        safetensors.load(io.BytesIO(raw))
    with pytest.raises(safetensors.SafetensorsError):
        safetensors.load_tensor(io.BytesIO(raw), "x")
    p = tmp_path / "m.safetensors"
    p.write_bytes(raw)
    with pytest.raises(safetensors.SafetensorsError):
        safetensors.load_files([str(p)])


@pytest.mark.parametrize("n", [1 << 31, 1 << 40, (1 << 63) + 5, (1 << 64) - 1, 0])
def test_safetensors_header_length_is_bounded(n):
    with pytest.raises(safetensors.SafetensorsError, match="implausible header length"):
        safetensors.header(io.BytesIO(struct.pack("<Q", n) + b"{}"))


def test_safetensors_header_garbage():
    for h in ("[1,2]", '{"x":3}', '{"x":{"dtype":"F32","shape":[1.5],"data_offsets":[0,4]}}', '{"__metadata__":{"a":1}}', "{not json"):
        with pytest.raises(safetensors.SafetensorsError):
            safetensors.load(io.BytesIO(_raw(h, b"\0\0\0\0")))
    ok, _ = safetensors.load(io.BytesIO(_raw('{"x":{"dtype":"f32","shape":[1],"data_offsets":[0,4]}}', struct.pack("<f", 2.5))))
    assert ok["x"].item() == 2.5                   # dtype names are matched without regard to case
