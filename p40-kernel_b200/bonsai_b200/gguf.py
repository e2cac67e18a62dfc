"""The on-disk format on the load side of the path: GGUF header reader, geometry gate, tensor upload and repack.

What the reference does with a model file before any kernel runs: tools/check_gguf.py:22-62 asserts that the file's
metadata and tensor table match the geometry its kernels are built for (include/bonsai_model.h:29-59), and the
runner uploads every PQ2_0 tensor and may re-lay it with bonsai_p40_repack (docs/REPACK.md).  This module is that
step for the sm_100a library:

    hdr = gguf.read_header(path)            # metadata, tensor table, data offset
    problems = gguf.check_geometry(hdr)     # [] when the file is the 27B model the kernels expect
    W = gguf.upload(hdr, path, "blk.0.ffn_up.weight", repack=True)     # device tensor, optionally repacked

`write_gguf` writes a small file of the same format (tests, synthetic models).  Format facts used (GGUF v3): magic
"GGUF", u32 version, u64 tensor count, u64 metadata count; strings are u64 length + bytes; a tensor entry is name, u32
rank, u64 dims (innermost first: dims[0] = n_in), u32 type, u64 offset relative to the data section, which starts at
the next multiple of `general.alignment` (default 32) after the header.
"""
import re
import struct

import numpy as np

GGML_TYPE_F32, GGML_TYPE_F16, GGML_TYPE_BF16, GGML_TYPE_PQ2_0 = 0, 1, 30, 142      # tools/check_gguf.py:18-21
PQ2_0_BLOCK_BYTES, PQ2_0_BLOCK_WEIGHTS = 34, 128

# metadata the kernels rely on (tools/check_gguf.py:24-43; include/bonsai_model.h:29-52)
EXPECT_KV = {
    "general.architecture": "qwen35",
    "qwen35.block_count": 64,
    "qwen35.embedding_length": 5120,
    "qwen35.feed_forward_length": 17408,
    "qwen35.attention.head_count": 24,
    "qwen35.attention.head_count_kv": 4,
    "qwen35.attention.key_length": 256,
    "qwen35.attention.value_length": 256,
    "qwen35.full_attention_interval": 4,
    "qwen35.ssm.conv_kernel": 4,
    "qwen35.ssm.state_size": 128,
    "qwen35.ssm.group_count": 16,
    "qwen35.ssm.time_step_rank": 48,
    "qwen35.ssm.inner_size": 6144,
    "qwen35.rope.dimension_count": 64,
    "prism.hadamard.block_size": 1024,
    "prism.hadamard.transform": "normalized-sylvester-walsh-hadamard",
    "prism.hadamard.axis": "input-last-dimension",
}
# tensor name (layer number replaced by X) -> (n_in, n_out or None, type, count or None)   (tools/check_gguf.py:45-67)
EXPECT_TENSORS = {
    "output.weight": (5120, 248320, GGML_TYPE_PQ2_0, None),
    "token_embd.weight": (5120, 248320, GGML_TYPE_PQ2_0, None),
    "blk.X.attn_norm.weight": (5120, None, GGML_TYPE_F32, 64),
    "blk.X.post_attention_norm.weight": (5120, None, GGML_TYPE_F32, None),
    "blk.X.ffn_down.weight": (17408, 5120, GGML_TYPE_PQ2_0, None),
    "blk.X.ffn_gate.weight": (5120, 17408, GGML_TYPE_PQ2_0, None),
    "blk.X.ffn_up.weight": (5120, 17408, GGML_TYPE_PQ2_0, None),
    "blk.X.attn_qkv.weight": (5120, 10240, GGML_TYPE_PQ2_0, 48),
    "blk.X.attn_gate.weight": (5120, 6144, GGML_TYPE_PQ2_0, 48),
    "blk.X.ssm_out.weight": (6144, 5120, GGML_TYPE_PQ2_0, 48),
    "blk.X.attn_q.weight": (5120, 12288, GGML_TYPE_PQ2_0, 16),
    "blk.X.attn_k.weight": (5120, 1024, GGML_TYPE_PQ2_0, 16),
    "blk.X.attn_v.weight": (5120, 1024, GGML_TYPE_PQ2_0, 16),
    "blk.X.attn_output.weight": (6144, 5120, GGML_TYPE_PQ2_0, 16),
}

_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
_T_STRING, _T_ARRAY = 8, 9


class Header:
    """version, kv (dict), tensors (name -> dict(dims, type, offset, nbytes)), data_start, truncated."""


def tensor_nbytes(dims, ggml_type):
    n = 1
    for d in dims:
        n *= d
    if ggml_type == GGML_TYPE_PQ2_0:
        if dims[0] % PQ2_0_BLOCK_WEIGHTS:
            raise ValueError(f"PQ2_0 tensor with n_in = {dims[0]}, not a multiple of 128")
        return n // PQ2_0_BLOCK_WEIGHTS * PQ2_0_BLOCK_BYTES
    return n * {GGML_TYPE_F32: 4, GGML_TYPE_F16: 2, GGML_TYPE_BF16: 2}.get(ggml_type, 0)


def read_header(path_or_bytes):
    """Parses the header of a GGUF file (or of its first bytes: a truncated tensor table is reported, not fatal)."""
    if isinstance(path_or_bytes, (bytes, bytearray, memoryview)):
        buf = bytes(path_or_bytes)
    else:
        with open(path_or_bytes, "rb") as f:
            buf = f.read(64 << 20)          # headers of the 27B file are ~11 MB (its data starts at byte 11 120 992)
    pos = 0

    def take(fmt):
        nonlocal pos
        v = struct.unpack_from(fmt, buf, pos)[0]
        pos += struct.calcsize(fmt)
        return v

    def string():
        nonlocal pos
        n = take("<Q")
        if pos + n > len(buf):
            raise struct.error("string runs past the buffer")
        s = buf[pos:pos + n].decode("utf-8", "replace")
        pos += n
        return s

    def value(t):
        if t in _SCALAR:
            return take(_SCALAR[t])
        if t == _T_STRING:
            return string()
        if t == _T_ARRAY:
            at, n = take("<I"), take("<Q")
            return [value(at) for _ in range(n)]
        raise ValueError(f"unknown metadata type {t}")

    h = Header()
    if buf[:4] != b"GGUF":
        raise ValueError(f"not a GGUF file (magic {buf[:4]!r})")
    pos = 4
    h.version, n_tensors, n_kv = take("<I"), take("<Q"), take("<Q")
    h.kv, h.tensors, h.truncated = {}, {}, False
    try:
        for _ in range(n_kv):
            k = string()
            h.kv[k] = value(take("<I"))
        for _ in range(n_tensors):
            name = string()
            nd = take("<I")
            dims = [take("<Q") for _ in range(nd)]
            tt, off = take("<I"), take("<Q")
            h.tensors[name] = {"dims": dims, "type": tt, "offset": off, "nbytes": tensor_nbytes(dims, tt)}
    except struct.error:
        h.truncated = True
    align = int(h.kv.get("general.alignment", 32))
    h.data_start = (pos + align - 1) // align * align
    return h


def check_geometry(h):
    """The gate of tools/check_gguf.py:107-165: returns the list of mismatches ([] = the file is the model the kernels
    were built for).  A file that carries a multi-token-prediction block is refused as there (docs/MTP.md)."""
    problems = []
    for k, want in EXPECT_KV.items():
        if h.kv.get(k) != want:
            problems.append(f"{k}: got {h.kv.get(k)!r}, want {want!r}")
    groups = {}
    for name, t in h.tensors.items():
        if re.search(r"nextn|mtp|draft|eagle", name, re.I):
            problems.append(f"{name}: multi-token-prediction tensors are not supported")
            continue
        g = re.sub(r"blk\.\d+\.", "blk.X.", name)
        groups.setdefault((g, tuple(t["dims"]), t["type"]), 0)
        groups[(g, tuple(t["dims"]), t["type"])] += 1
    for (g, dims, tt), cnt in sorted(groups.items()):
        exp = EXPECT_TENSORS.get(g)
        if exp is None:
            continue
        n_in, n_out, etype, count = exp
        ok = dims[0] == n_in and (n_out is None or (len(dims) > 1 and dims[1] == n_out)) and tt == etype
        ok = ok and (count is None or cnt == count)
        if not ok:
            problems.append(f"{g}: dims={list(dims)} type={tt} x{cnt}, want ({n_in}, {n_out}) type={etype} x{count}")
    # what the kernels themselves need of every PQ2_0 tensor (include/bonsai_p40.h: rows of whole 128-weight blocks;
    # bulk copies: 16-byte aligned data; the repacked layout: n_in / 128 a multiple of 8)
    for name, t in h.tensors.items():
        if t["type"] == GGML_TYPE_PQ2_0 and (h.data_start + t["offset"]) % 2:
            problems.append(f"{name}: data at an odd file offset")
    return problems


def read_tensor(h, path, name):
    """The tensor's bytes as a numpy array (uint8 for PQ2_0, the element type otherwise)."""
    t = h.tensors[name]
    with open(path, "rb") as f:
        f.seek(h.data_start + t["offset"])
        raw = f.read(t["nbytes"])
    if len(raw) != t["nbytes"]:
        raise IOError(f"{name}: file ends inside the tensor")
    dt = {GGML_TYPE_F32: np.float32, GGML_TYPE_F16: np.float16}.get(t["type"], np.uint8)
    return np.frombuffer(raw, dtype=dt).copy()


def upload(h, path, name, repack=False):
    """Tensor -> pinned host buffer -> device (torch's allocator returns 256-byte aligned memory, so rows are 16-byte
    aligned whenever n_in / 128 is even).  With repack=True a PQ2_0 tensor is re-laid on the device by
    bonsai_p40_repack (needs n_in / 128 a multiple of 8); returns the device tensor (uint8 for PQ2_0)."""
    import torch
    import bonsai_b200 as bb
    t = h.tensors[name]
    hostbuf = torch.from_numpy(read_tensor(h, path, name)).pin_memory()
    dev = hostbuf.cuda(non_blocking=True)
    if repack:
        if t["type"] != GGML_TYPE_PQ2_0:
            raise ValueError(f"{name} is not a PQ2_0 tensor")
        n_in, n_out = t["dims"][0], t["dims"][1]
        out = torch.empty_like(dev)
        rc = bb.repack(dev, out, n_out, n_in)
        if rc != 0:
            raise RuntimeError(f"bonsai_p40_repack refused {name} ({n_in} x {n_out}): {rc}")
        dev = out
    torch.cuda.current_stream().synchronize()      # the pinned buffer may go
    return dev


# ---- writer (tests, synthetic models) -----------------------------------------------------------------------
def write_gguf(path, kv, tensors, alignment=32):
    """kv: dict of str -> (str | int); tensors: list of (name, dims, ggml_type, numpy array of the raw bytes)."""
    def s(x):
        b = x.encode()
        return struct.pack("<Q", len(b)) + b
    out = bytearray(b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(kv)))
    for k, v in kv.items():
        out += s(k)
        if isinstance(v, str):
            out += struct.pack("<I", _T_STRING) + s(v)
        else:
            out += struct.pack("<II", 4, int(v))
    blobs, off = [], 0
    for name, dims, tt, data in tensors:
        raw = np.ascontiguousarray(data).view(np.uint8).reshape(-1).tobytes()
        assert len(raw) == tensor_nbytes(dims, tt), name
        out += s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        out += struct.pack("<IQ", tt, off)
        blobs.append((off, raw))
        off = (off + len(raw) + alignment - 1) // alignment * alignment
    start = (len(out) + alignment - 1) // alignment * alignment
    out += b"\0" * (start - len(out))
    for o, raw in blobs:
        out += b"\0" * (start + o - len(out)) + raw
    with open(path, "wb") as f:
        f.write(out)
