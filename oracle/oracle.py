"""ctypes access to the CPU checkers (TEST INFRASTRUCTURE).

`Oracle("port")` loads this repository's C restatement (oracle/libbonsai_oracle.so);
`Oracle("reference")` loads the reference's own headers compiled by oracle/build_oracle.py
(oracle/_ref/libbonsai_ref.so).  Both expose the same numpy-level methods so a test can run
one against the other.  Only tests, the smoke check and the benchmark's CPU-baseline leg may
import this module; the CUDA library has no dependency on it.
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
PORT_SO = os.path.join(HERE, "libbonsai_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "libbonsai_ref.so")

W_BYTES = 34
A_BYTES = 36


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def ptq1_pack(pq2):
    """PQ2_0 blocks (34 bytes) -> PTQ1_0 blocks (28 bytes: qs[24] five base-3 digits per byte, qh[2] four digits per
    byte, fp16 d), the packing the reference describes in docs/NEXT_STEPS.md:76-83; digit order: weight j < 120 is digit
    j % 5 of byte j / 5, least significant first.  Returns (bytes, number of weights with code 3, stored as code 2)."""
    b = np.ascontiguousarray(pq2, dtype=np.uint8).reshape(-1, W_BYTES)
    codes = np.stack([(b[:, 2:] >> f) & 3 for f in (0, 2, 4, 6)], axis=2).reshape(b.shape[0], 128).astype(np.int64)
    bad = int((codes == 3).sum())
    codes = np.minimum(codes, 2)
    out = np.zeros((b.shape[0], 28), dtype=np.uint8)
    out[:, :24] = (codes[:, :120].reshape(-1, 24, 5) * (3 ** np.arange(5))).sum(2)
    out[:, 24:26] = (codes[:, 120:].reshape(-1, 2, 4) * (3 ** np.arange(4))).sum(2)
    out[:, 26:28] = b[:, 0:2]
    return out.reshape(-1), bad


def ptq1_unpack(ptq):
    p = np.ascontiguousarray(ptq, dtype=np.uint8).reshape(-1, 28).astype(np.int64)
    codes = np.zeros((p.shape[0], 128), dtype=np.int64)
    for k in range(5):
        codes[:, k:120:5] = (p[:, :24] // 3 ** k) % 3
    for k in range(4):
        codes[:, 120 + k::4] = (p[:, 24:26] // 3 ** k) % 3
    out = np.zeros((p.shape[0], W_BYTES), dtype=np.uint8)
    out[:, 0:2] = p[:, 26:28]
    c = codes.reshape(-1, 32, 4)
    out[:, 2:] = c[:, :, 0] | (c[:, :, 1] << 2) | (c[:, :, 2] << 4) | (c[:, :, 3] << 6)
    return out.reshape(-1)


def reference_available():
    return os.path.exists(REF_SO)


class Oracle:
    def __init__(self, kind="port"):
        self.kind = kind
        if kind == "port":
            if not os.path.exists(PORT_SO):
                from .build_oracle import build_oracle
                build_oracle()
            self.lib, self.pre = C.CDLL(PORT_SO), "bo_"
        elif kind == "reference":
            if not os.path.exists(REF_SO):
                raise FileNotFoundError("oracle/_ref/libbonsai_ref.so is not built (run oracle/build_oracle.py)")
            self.lib, self.pre = C.CDLL(REF_SO), "ref_"
        else:
            raise ValueError(kind)
        f = self._fn
        f("f16_to_f32", C.c_float, [C.c_uint16])
        f("f32_to_f16", C.c_uint16, [C.c_float])
        f("quantize_q8_1", None, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int])
        f("quantize_pq2_0", None, [C.c_void_p, C.c_void_p, C.c_int64])
        f("dequantize_pq2_0", None, [C.c_void_p, C.c_void_p, C.c_int64])
        f("fwht_blocks", None, [C.c_void_p, C.c_void_p, C.c_int64])
        f("chunk_dot", C.c_float, [C.c_void_p, C.c_void_p, C.c_int])
        f("row_dot", C.c_float, [C.c_void_p, C.c_void_p, C.c_int64])
        f("gemv", None, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64])
        f("gemm", None, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64])
        f("gemv_mt", C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int])
        f("gemm_mt", C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int])
        f("repack_row", None, [C.c_void_p, C.c_int, C.c_void_p])
        f("unpack_row", None, [C.c_void_p, C.c_int, C.c_void_p])
        f("repack_unit_sumi", C.c_int32, [C.c_void_p, C.c_void_p, C.c_int, C.c_int])
        f("repack_row_dot", C.c_float, [C.c_void_p, C.c_void_p, C.c_int])
        f("rmsnorm", None, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_float])
        f("swiglu", None, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64])
        f("gdn_step", None, [C.c_void_p] * 7 + [C.c_int] * 4)
        f("kv_quantize_row_q8_0", None, [C.c_void_p, C.c_void_p, C.c_int])
        f("kv_dequantize_row_q8_0", None, [C.c_void_p, C.c_void_p, C.c_int])
        f("kv_score", C.c_float, [C.c_void_p, C.c_void_p, C.c_int])
        if kind == "reference":
            f("kv_block_index", C.c_int64, [C.c_int] * 5)
            f("kv_total_bytes", C.c_int64, [C.c_int])
            f("kv_gdn_bytes", C.c_int64, [])
        if kind == "port":
            f("kv_attn_decode", None, [C.c_void_p] * 4 + [C.c_int] * 5 + [C.c_float])
            f("attn", None, [C.c_void_p] * 4 + [C.c_int] * 4 + [C.c_float])
            f("chunk_sumi", C.c_int32, [C.c_void_p, C.c_void_p, C.c_int])
            f("row_chunk_sums", None, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p])

    def _fn(self, name, res, args):
        fn = getattr(self.lib, self.pre + name)
        fn.restype, fn.argtypes = res, args
        setattr(self, "_" + name, fn)

    # ---- scalars -----------------------------------------------------------------------
    def f16_to_f32(self, h):
        return float(self._f16_to_f32(int(h)))

    def f32_to_f16(self, f):
        return int(self._f32_to_f16(float(np.float32(f))))

    # ---- activation side -----------------------------------------------------------------
    def quantize_q8_1(self, x, permute=True):
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.zeros(x.size // 32 * A_BYTES, dtype=np.uint8)
        self._quantize_q8_1(_p(x), _p(out), x.size, int(permute))
        return out

    def fwht_blocks(self, x, signs=None):
        y = np.array(x, dtype=np.float32, copy=True).reshape(-1)
        s = None if signs is None else np.ascontiguousarray(signs, dtype=np.float32)
        self._fwht_blocks(_p(y), None if s is None else _p(s), y.size)
        return y

    def quantize_batch_chunk_major(self, X):
        """X: fp32 [n_tok][n_in] -> Q8_1 bytes laid out [n_in/32][n_tok][36], each token quantised
        alone (the layout the mat-mul consumes)."""
        X = np.ascontiguousarray(X, dtype=np.float32)
        n_tok, n_in = X.shape
        per_tok = np.stack([self.quantize_q8_1(X[t]).reshape(n_in // 32, A_BYTES) for t in range(n_tok)], axis=1)
        return np.ascontiguousarray(per_tok).reshape(-1)

    # ---- weight side -----------------------------------------------------------------------
    def quantize_pq2_0(self, w):
        w = np.ascontiguousarray(w, dtype=np.float32)
        out = np.zeros(w.size // 128 * W_BYTES, dtype=np.uint8)
        self._quantize_pq2_0(_p(w), _p(out), w.size)
        return out

    def dequantize_pq2_0(self, wq):
        wq = np.ascontiguousarray(wq, dtype=np.uint8)
        y = np.zeros(wq.size // W_BYTES * 128, dtype=np.float32)
        self._dequantize_pq2_0(_p(wq), _p(y), y.size)
        return y

    # ---- dots ------------------------------------------------------------------------------
    def chunk_dot(self, wblk, ablk, iqs):
        wblk = np.ascontiguousarray(wblk, dtype=np.uint8)
        ablk = np.ascontiguousarray(ablk, dtype=np.uint8)
        return np.float32(self._chunk_dot(_p(wblk), _p(ablk), iqs))

    def row_chunk_sums(self, wrow, xq, n_in):
        """int32 per-chunk sums of one row.  The reference exposes them only through the repacked
        layout, so the reference flavour repacks the row first."""
        wrow = np.ascontiguousarray(wrow, dtype=np.uint8)
        xq = np.ascontiguousarray(xq, dtype=np.uint8)
        out = np.zeros(n_in // 32, dtype=np.int32)
        if self.kind == "port":
            self._row_chunk_sums(_p(wrow), _p(xq), n_in, _p(out))
            return out
        nb = n_in // 128
        rp = self.repack_row(wrow, nb)
        for u in range(4 * nb):
            out[4 * (u % nb) + u // nb] = self._repack_unit_sumi(_p(rp), _p(xq), nb, u)
        return out

    def gemv(self, W, xq, n_out, n_in, threads=1):
        W = np.ascontiguousarray(W, dtype=np.uint8)
        xq = np.ascontiguousarray(xq, dtype=np.uint8)
        y = np.zeros(n_out, dtype=np.float32)
        if threads > 1:
            self._gemv_mt(_p(W), _p(xq), _p(y), n_out, n_in, threads)
        else:
            self._gemv(_p(W), _p(xq), _p(y), n_out, n_in)
        return y

    def gemm(self, W, Xq, n_out, n_in, n_tok, threads=1):
        W = np.ascontiguousarray(W, dtype=np.uint8)
        Xq = np.ascontiguousarray(Xq, dtype=np.uint8)
        Y = np.zeros((n_out, n_tok), dtype=np.float32)
        if threads > 1:
            self._gemm_mt(_p(W), _p(Xq), _p(Y), n_out, n_in, n_tok, threads)
        else:
            self._gemm(_p(W), _p(Xq), _p(Y), n_out, n_in, n_tok)
        return Y

    # ---- repacked layout ----------------------------------------------------------------------
    def repack_row(self, wrow, nb):
        wrow = np.ascontiguousarray(wrow, dtype=np.uint8)
        out = np.zeros(W_BYTES * nb, dtype=np.uint8)
        self._repack_row(_p(wrow), nb, _p(out))
        return out

    def unpack_row(self, row, nb):
        row = np.ascontiguousarray(row, dtype=np.uint8)
        out = np.zeros(W_BYTES * nb, dtype=np.uint8)
        self._unpack_row(_p(row), nb, _p(out))
        return out

    def repack(self, W, n_out, n_in):
        nb = n_in // 128
        W = np.ascontiguousarray(W, dtype=np.uint8).reshape(n_out, W_BYTES * nb)
        return np.concatenate([self.repack_row(W[r], nb) for r in range(n_out)])

    def repack_row_dot(self, row, xq, nb):
        row = np.ascontiguousarray(row, dtype=np.uint8)
        xq = np.ascontiguousarray(xq, dtype=np.uint8)
        return np.float32(self._repack_row_dot(_p(row), _p(xq), nb))

    def gemv_repack(self, Wr, x, n_out, n_in):
        """Fused entry semantics: quantise fp32 x (not rotated), then repacked row dots."""
        nb = n_in // 128
        xq = self.quantize_q8_1(x)
        Wr = np.ascontiguousarray(Wr, dtype=np.uint8).reshape(n_out, W_BYTES * nb)
        return np.array([self.repack_row_dot(Wr[r], xq, nb) for r in range(n_out)], dtype=np.float32)

    # ---- the operators beside the mat-vec path ---------------------------------------------------------
    def rmsnorm(self, x, w, eps):
        x = np.ascontiguousarray(x, dtype=np.float32)
        w = np.ascontiguousarray(w, dtype=np.float32)
        x2 = x.reshape(-1, w.size)
        y = np.zeros_like(x2)
        self._rmsnorm(_p(x2), _p(w), _p(y), x2.shape[0], x2.shape[1], float(eps))
        return y.reshape(x.shape)

    def swiglu(self, gate, up):
        gate = np.ascontiguousarray(gate, dtype=np.float32)
        up = np.ascontiguousarray(up, dtype=np.float32)
        y = np.zeros_like(gate)
        self._swiglu(_p(gate), _p(up), _p(y), gate.size)
        return y

    def gdn_step(self, state, q, k, v, g, beta, n_k_heads, n_v_heads, K, V):
        """Returns (new state, out); `state` is not modified."""
        S = np.array(state, dtype=np.float32, copy=True)
        a = [np.ascontiguousarray(t, dtype=np.float32) for t in (q, k, v, g, beta)]
        out = np.zeros(n_v_heads * V, dtype=np.float32)
        self._gdn_step(_p(S), _p(a[0]), _p(a[1]), _p(a[2]), _p(a[3]), _p(a[4]), _p(out), n_k_heads, n_v_heads, K, V)
        return S, out

    def attn(self, q, k, v, n_tok, n_head, n_head_kv, D, scale):
        a = [np.ascontiguousarray(t, dtype=np.float32) for t in (q, k, v)]
        out = np.zeros(n_tok * n_head * D, dtype=np.float32)
        self._attn(_p(a[0]), _p(a[1]), _p(a[2]), _p(out), n_tok, n_head, n_head_kv, D, float(scale))
        return out

    # ---- K/V cache --------------------------------------------------------------------------------------
    def kv_quantize_row(self, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.zeros(x.size // 32 * 34, dtype=np.uint8)
        self._kv_quantize_row_q8_0(_p(x), _p(out), x.size)
        return out

    def kv_dequantize_row(self, blocks):
        blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
        y = np.zeros(blocks.size // 34 * 32, dtype=np.float32)
        self._kv_dequantize_row_q8_0(_p(blocks), _p(y), y.size)
        return y

    def kv_score(self, q8, k8):
        q8 = np.ascontiguousarray(q8, dtype=np.uint8)
        k8 = np.ascontiguousarray(k8, dtype=np.uint8)
        return np.float32(self._kv_score(_p(q8), _p(k8), q8.size // 34))

    def kv_attn_decode(self, K, V, q, capacity, layer, pos, n_head=24, n_kv_head=4, scale=0.0625):
        K = np.ascontiguousarray(K, dtype=np.uint8)
        V = np.ascontiguousarray(V, dtype=np.uint8)
        q = np.ascontiguousarray(q, dtype=np.float32)
        out = np.zeros(n_head * 256, dtype=np.float32)
        self._kv_attn_decode(_p(K), _p(V), _p(q), _p(out), capacity, layer, pos, n_head, n_kv_head, float(scale))
        return out

