"""The load-side format step on the CPU: GGUF header reader and geometry gate against synthetic files whose metadata
and tensor table follow the shipped model's (tools/check_gguf.py:24-67 in the reference), and the numpy statement of
the PTQ1_0 packing used as the checker of the device kernels."""
import numpy as np
import pytest

from bonsai_b200 import gguf, synth


def model_table(layers=64):
    """(name, dims, type) of every tensor the gate looks at, with 1-element stand-ins for the data."""
    t = [("output.weight", [5120, 248320], gguf.GGML_TYPE_PQ2_0), ("token_embd.weight", [5120, 248320], gguf.GGML_TYPE_PQ2_0)]
    for i in range(layers):
        t += [(f"blk.{i}.attn_norm.weight", [5120], gguf.GGML_TYPE_F32), (f"blk.{i}.post_attention_norm.weight", [5120], gguf.GGML_TYPE_F32),
              (f"blk.{i}.ffn_down.weight", [17408, 5120], gguf.GGML_TYPE_PQ2_0), (f"blk.{i}.ffn_gate.weight", [5120, 17408], gguf.GGML_TYPE_PQ2_0),
              (f"blk.{i}.ffn_up.weight", [5120, 17408], gguf.GGML_TYPE_PQ2_0)]
        if (i + 1) % 4 == 0:
            t += [(f"blk.{i}.attn_q.weight", [5120, 12288], gguf.GGML_TYPE_PQ2_0), (f"blk.{i}.attn_k.weight", [5120, 1024], gguf.GGML_TYPE_PQ2_0),
                  (f"blk.{i}.attn_v.weight", [5120, 1024], gguf.GGML_TYPE_PQ2_0), (f"blk.{i}.attn_output.weight", [6144, 5120], gguf.GGML_TYPE_PQ2_0)]
        else:
            t += [(f"blk.{i}.attn_qkv.weight", [5120, 10240], gguf.GGML_TYPE_PQ2_0), (f"blk.{i}.attn_gate.weight", [5120, 6144], gguf.GGML_TYPE_PQ2_0),
                  (f"blk.{i}.ssm_out.weight", [6144, 5120], gguf.GGML_TYPE_PQ2_0)]
    return t


def header_only(kv, table):
    """A header whose tensor table is complete and whose data section is absent (the gate reads no data)."""
    import struct

    def s(x):
        b = x.encode()
        return struct.pack("<Q", len(b)) + b
    out = bytearray(b"GGUF" + struct.pack("<IQQ", 3, len(table), len(kv)))
    for k, v in kv.items():
        out += s(k) + (struct.pack("<I", 8) + s(v) if isinstance(v, str) else struct.pack("<II", 4, v))
    off = 0
    for name, dims, tt in table:
        out += s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", tt, off)
        off += (gguf.tensor_nbytes(dims, tt) + 31) // 32 * 32
    return bytes(out)


def test_gate_accepts_the_model_geometry():
    h = gguf.read_header(header_only(gguf.EXPECT_KV, model_table()))
    assert not h.truncated and len(h.tensors) == 2 + 64 * 5 + 48 * 3 + 16 * 4
    assert gguf.check_geometry(h) == []
    # PQ2_0 bytes of the linear layers the decode step streams: 401 mat-vecs (output.weight once, not token_embd)
    total = sum(t["nbytes"] for n, t in h.tensors.items() if t["type"] == gguf.GGML_TYPE_PQ2_0 and n != "token_embd.weight")
    assert total == 6799564800
    assert h.data_start % 32 == 0


def test_gate_names_what_is_wrong():
    kv = dict(gguf.EXPECT_KV)
    kv["qwen35.embedding_length"] = 4096
    table = model_table()
    table[5] = ("blk.0.ffn_gate.weight", [5120, 17408], gguf.GGML_TYPE_F16)          # wrong type
    table = [t for t in table if t[0] != "blk.7.attn_k.weight"]                      # 15 instead of 16
    table.append(("blk.64.nextn.eh_proj.weight", [5120, 5120], gguf.GGML_TYPE_PQ2_0))   # a multi-token-prediction block
    problems = "\n".join(gguf.check_geometry(gguf.read_header(header_only(kv, table))))
    assert "qwen35.embedding_length" in problems and "blk.X.ffn_gate.weight" in problems
    assert "blk.X.attn_k.weight" in problems and "nextn" in problems


def test_truncated_header_is_reported_not_fatal():
    full = header_only(gguf.EXPECT_KV, model_table())
    h = gguf.read_header(full[:len(full) // 2])
    assert h.truncated and 0 < len(h.tensors) < 500
    with pytest.raises(ValueError):
        gguf.read_header(b"GGML" + full[4:])


def test_write_read_round_trip(tmp_path):
    W = synth.pq2_0_weights(16, 1024, seed=1)
    norm = np.arange(1024, dtype=np.float32)
    p = tmp_path / "tiny.gguf"
    gguf.write_gguf(p, {"general.architecture": "qwen35", "qwen35.block_count": 1},
                    [("blk.0.ffn_up.weight", [1024, 16], gguf.GGML_TYPE_PQ2_0, W), ("blk.0.attn_norm.weight", [1024], gguf.GGML_TYPE_F32, norm)])
    h = gguf.read_header(p)
    assert h.kv["qwen35.block_count"] == 1 and h.tensors["blk.0.ffn_up.weight"]["dims"] == [1024, 16]
    assert np.array_equal(gguf.read_tensor(h, p, "blk.0.ffn_up.weight"), W)
    assert np.array_equal(gguf.read_tensor(h, p, "blk.0.attn_norm.weight"), norm)
    assert (h.data_start + h.tensors["blk.0.attn_norm.weight"]["offset"]) % 32 == 0
    assert gguf.check_geometry(h) != []                      # not the 27B model


def test_ptq1_numpy_statement_round_trips(port):
    from oracle.oracle import ptq1_pack, ptq1_unpack
    W = synth.pq2_0_weights(8, 1024, seed=3)
    blocks = W.reshape(-1, 34).copy()
    q = blocks[:, 2:].astype(np.int64)
    fields = [(q >> f) & 3 for f in (0, 2, 4, 6)]
    fields = [np.where(c == 3, 1, c) for c in fields]                   # a strictly ternary copy: code 3 (+2) becomes 1
    blocks[:, 2:] = (fields[0] | (fields[1] << 2) | (fields[2] << 4) | (fields[3] << 6)).astype(np.uint8)
    packed, bad = ptq1_pack(blocks.reshape(-1))
    assert bad == 0 and packed.size == blocks.shape[0] * 28
    assert np.array_equal(ptq1_unpack(packed), blocks.reshape(-1))
    # same weights: dequantised values agree
    assert np.array_equal(port.dequantize_pq2_0(ptq1_unpack(packed)), port.dequantize_pq2_0(blocks.reshape(-1)))
    _, bad = ptq1_pack(W)
    assert bad == int(sum((((W.reshape(-1, 34)[:, 2:] >> f) & 3) == 3).sum() for f in (0, 2, 4, 6)))
