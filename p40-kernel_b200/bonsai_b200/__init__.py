"""Python access to libbonsai_p40.so (the sm_100a build) through its C ABI.

The functions mirror include/bonsai_p40.h and include/bonsai_b200_ext.h one to one: same names
(minus the prefix), same argument order, same integer return codes.  Tensors are torch CUDA tensors
used only as device memory; the stream passed to the library is torch's current stream, so
torch.cuda.Event timing brackets the library's kernels.

There is no CPU fallback: importing works without a GPU (the symbols are checked), every compute
call requires CUDA tensors and raises otherwise.
"""
import ctypes as C
import os

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_PKG_DIR)
# the in-tree build; BONSAI_B200_LIB names another build of the same library (A/B timing of two builds in one process tree)
LIB_PATH = os.environ.get("BONSAI_B200_LIB") or os.path.join(_ROOT, "libbonsai_p40.so")

W_BLOCK_BYTES = 34
A_BLOCK_BYTES = 36

_lib = None

_VP, _I64, _INT, _U64, _F = C.c_void_p, C.c_int64, C.c_int, C.c_uint64, C.c_float

#: every exported symbol with its C signature (also what the symbol-presence test checks)
SIGNATURES = {
    "bonsai_p40_gemv": (_INT, [_VP, _VP, _VP, _I64, _I64, _VP]),
    "bonsai_p40_quant_activations": (_INT, [_VP, _VP, _I64, _VP]),
    "bonsai_p40_gemm": (_INT, [_VP, _VP, _VP, _I64, _I64, _I64, _VP]),
    "bonsai_p40_repack": (_INT, [_VP, _VP, _I64, _I64, _VP]),
    "bonsai_p40_gemv_repack": (_INT, [_VP, _VP, _VP, _I64, _I64, _VP]),
    "bonsai_p40_fwht": (_INT, [_VP, _VP, _I64, _VP]),
    "bonsai_p40_rmsnorm": (_INT, [_VP, _VP, _VP, _I64, _I64, _F, _VP]),
    "bonsai_p40_gdn_step": (_INT, [_VP] * 7 + [_INT] * 4 + [_VP]),
    "bonsai_p40_attn": (_INT, [_VP] * 4 + [_INT] * 4 + [_F, _VP]),
    "bonsai_b200_fwht_quant": (_INT, [_VP, _VP, _VP, _VP, _I64, _VP]),
    "bonsai_b200_linear": (_INT, [_VP, _VP, _VP, _VP, _VP, _I64, _I64, _VP]),
    "bonsai_b200_linear_static": (_INT, [_VP, _VP, _VP, _VP, _I64, _I64, _VP]),
    "bonsai_b200_swiglu": (_INT, [_VP, _VP, _VP, _I64, _VP]),
    "bonsai_b200_quant_batch": (_INT, [_VP, _VP, _VP, _I64, _I64, _INT, _VP]),
    "bonsai_b200_gemv_chunk_sums": (_INT, [_VP, _VP, _VP, _I64, _I64, _I64, _VP]),
    "bonsai_b200_gemv_dump": (_INT, [_VP, _VP, _VP, _VP, _I64, _I64, _VP]),
    "bonsai_b200_gemm_dump": (_INT, [_VP, _VP, _VP, _VP, _I64, _I64, _I64, _VP]),
    "bonsai_b200_gemm_reserve": (_INT, [_I64, _I64, _VP]),
    "bonsai_b200_gemm_release": (_INT, []),
    "bonsai_b200_ptq1_pack": (_INT, [_VP, _VP, _I64, _VP, _VP]),
    "bonsai_b200_ptq1_unpack": (_INT, [_VP, _VP, _I64, _VP]),
    "bonsai_b200_synth_pq2_0": (_INT, [_VP, _I64, _I64, _U64, _VP]),
    "bonsai_b200_stream_probe": (_INT, [_VP, _I64, _INT, _VP, _VP]),
    "bonsai_b200_chain_create": (_INT, [_VP, _I64, _VP]),
    "bonsai_b200_chain_create_tp": (_INT, [_VP, _I64, _INT, _INT, _VP, _I64, _I64, _I64, _VP]),
    "bonsai_b200_chain_run": (_INT, [_VP, _VP]),
    "bonsai_b200_chain_destroy": (_INT, [_VP]),
    "bonsai_b200_chain_info": (_INT, [_VP, _VP]),
    "bonsai_b200_kv_arrays": (_INT, [_VP, _VP, _VP, _VP]),
    "bonsai_kv_bytes": (_I64, [_INT]),
    "bonsai_kv_gdn_bytes": (_I64, []),
    "bonsai_kv_create": (_VP, [_INT, _VP]),
    "bonsai_kv_free": (None, [_VP]),
    "bonsai_kv_reset": (None, [_VP, _VP]),
    "bonsai_kv_append": (_INT, [_VP, _INT, _INT, _VP, _VP, _VP]),
    "bonsai_kv_append_batch": (_INT, [_VP, _INT, _INT, _INT, _VP, _VP, _VP]),
    "bonsai_kv_attn_decode": (_INT, [_VP, _INT, _INT, _VP, _VP, _VP]),
    "bonsai_kv_gdn_state": (_VP, [_VP, _INT]),
    "bonsai_b200_set_option": (_INT, [C.c_char_p, _I64]),
    "bonsai_b200_device_status": (_INT, []),
    "bonsai_b200_clear_status": (_INT, []),
    "bonsai_b200_version": (_INT, []),
}


def lib():
    """Loads the shared library once.  Fails loudly when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python {os.path.join(_ROOT, 'build.py')}` "
                "(there is no fallback path)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def _stream():
    import torch
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _dev(t, name):
    if t is None:
        return None
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: this library has no CPU path")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    return C.c_void_p(t.data_ptr())


def set_option(key, value):
    return lib().bonsai_b200_set_option(key.encode(), int(value))


def device_status():
    return lib().bonsai_b200_device_status()


def clear_status():
    return lib().bonsai_b200_clear_status()


def version():
    return lib().bonsai_b200_version()


# ---- include/bonsai_p40.h ------------------------------------------------------------------------
def gemv(W, xq, y, n_out, n_in):
    return lib().bonsai_p40_gemv(_dev(W, "W"), _dev(xq, "xq"), _dev(y, "y"), n_out, n_in, _stream())


def quant_activations(x, out, n):
    return lib().bonsai_p40_quant_activations(_dev(x, "x"), _dev(out, "out"), n, _stream())


def gemm(W, Xq, Y, n_out, n_in, n_tok):
    return lib().bonsai_p40_gemm(_dev(W, "W"), _dev(Xq, "Xq"), _dev(Y, "Y"), n_out, n_in, n_tok, _stream())


def repack(src, dst, n_out, n_in):
    return lib().bonsai_p40_repack(_dev(src, "src"), _dev(dst, "dst"), n_out, n_in, _stream())


def gemv_repack(W, x, y, n_out, n_in):
    return lib().bonsai_p40_gemv_repack(_dev(W, "W"), _dev(x, "x"), _dev(y, "y"), n_out, n_in, _stream())


def rmsnorm(x, w, y, n_rows, n, eps):
    return lib().bonsai_p40_rmsnorm(_dev(x, "x"), _dev(w, "w"), _dev(y, "y"), n_rows, n, eps, _stream())


def gdn_step(state, q, k, v, g, beta, out, n_k_heads, n_v_heads, K, V):
    return lib().bonsai_p40_gdn_step(_dev(state, "state"), _dev(q, "q"), _dev(k, "k"), _dev(v, "v"), _dev(g, "g"),
                                     _dev(beta, "beta"), _dev(out, "out"), n_k_heads, n_v_heads, K, V, _stream())


def attn(q, k, v, out, n_tok, n_head, n_head_kv, head_dim, scale):
    return lib().bonsai_p40_attn(_dev(q, "q"), _dev(k, "k"), _dev(v, "v"), _dev(out, "out"), n_tok, n_head, n_head_kv,
                                 head_dim, scale, _stream())


def fwht(x, signs, n):
    return lib().bonsai_p40_fwht(_dev(x, "x"), _dev(signs, "signs"), n, _stream())


# ---- include/bonsai_b200_ext.h ---------------------------------------------------------------------
def fwht_quant(x, signs, xq, x_rot, n):
    return lib().bonsai_b200_fwht_quant(_dev(x, "x"), _dev(signs, "signs"), _dev(xq, "xq"), _dev(x_rot, "x_rot"), n,
                                        _stream())


def swiglu(gate, up, y, n):
    return lib().bonsai_b200_swiglu(_dev(gate, "gate"), _dev(up, "up"), _dev(y, "y"), n, _stream())


def quant_batch(X, signs, Xq, n_in, n_tok, rotate):
    return lib().bonsai_b200_quant_batch(_dev(X, "X"), _dev(signs, "signs"), _dev(Xq, "Xq"), n_in, n_tok,
                                         int(bool(rotate)), _stream())


def gemv_chunk_sums(W, xq, out, row0, n_rows, n_in):
    return lib().bonsai_b200_gemv_chunk_sums(_dev(W, "W"), _dev(xq, "xq"), _dev(out, "out"), row0, n_rows, n_in,
                                             _stream())


def gemv_dump(W, xq, y, sums, n_out, n_in):
    return lib().bonsai_b200_gemv_dump(_dev(W, "W"), _dev(xq, "xq"), _dev(y, "y"), _dev(sums, "sums"), n_out, n_in, _stream())


def gemm_dump(W, Xq, Y, sums, n_out, n_in, n_tok):
    return lib().bonsai_b200_gemm_dump(_dev(W, "W"), _dev(Xq, "Xq"), _dev(Y, "Y"), _dev(sums, "sums"), n_out, n_in, n_tok,
                                       _stream())


def gemm_reserve(n_in, n_tok):
    return lib().bonsai_b200_gemm_reserve(n_in, n_tok, _stream())


def gemm_release():
    return lib().bonsai_b200_gemm_release()


def ptq1_pack(src, dst, n_blocks, code3_count):
    return lib().bonsai_b200_ptq1_pack(_dev(src, "src"), _dev(dst, "dst"), n_blocks, _dev(code3_count, "code3_count"), _stream())


def ptq1_unpack(src, dst, n_blocks):
    return lib().bonsai_b200_ptq1_unpack(_dev(src, "src"), _dev(dst, "dst"), n_blocks, _stream())


def synth_pq2_0(W, first_block, n_blocks, seed):
    return lib().bonsai_b200_synth_pq2_0(_dev(W, "W"), first_block, n_blocks, seed, _stream())


def stream_probe(buf, nbytes, mode, sink):
    return lib().bonsai_b200_stream_probe(_dev(buf, "buf"), nbytes, mode, _dev(sink, "sink"), _stream())


def linear(W, x, signs, y, xq_scratch, n_out, n_in):
    return lib().bonsai_b200_linear(_dev(W, "W"), _dev(x, "x"), _dev(signs, "signs"), _dev(y, "y"),
                                    _dev(xq_scratch, "xq_scratch"), n_out, n_in, _stream())


def linear_static(W, x, signs, y, n_out, n_in):
    """The projection whose scratch lives inside the library (no allocation, n_in <= 32768)."""
    return lib().bonsai_b200_linear_static(_dev(W, "W"), _dev(x, "x"), _dev(signs, "signs"), _dev(y, "y"), n_out,
                                           n_in, _stream())


# ---- a list of projections in one launch -------------------------------------------------------------
OP_ROTATE, OP_DEPENDS, OP_SAME_INPUT, OP_RMSNORM, OP_SWIGLU, OP_RESCALE = 1, 2, 4, 8, 16, 32


class Op(C.Structure):
    """struct bonsai_b200_op"""
    _fields_ = [("W", C.c_void_p), ("x", C.c_void_p), ("signs", C.c_void_p), ("y", C.c_void_p),
                ("n_out", C.c_int64), ("n_in", C.c_int64), ("flags", C.c_uint32), ("reserved", C.c_uint32),
                ("aux", C.c_void_p), ("eps", C.c_float), ("src_len", C.c_uint32)]


class Chain:
    """bonsai_b200_chain_create / _create_tp / _run / _destroy.  `ops` is a list of (W, x, signs, y, n_out, n_in,
    flags[, aux[, eps[, src_len]]]) with CUDA tensors; the tensors are kept alive by the object.  With `peers` (a peer.PeerBuffer whose
    tensor holds every y) the list runs over the row slices of several ranks."""

    def __init__(self, ops, peers=None, wait_limit_us=0):
        self._keep = [t for op in ops for t in (*op[:4], *op[7:8]) if t is not None]
        arr = (Op * len(ops))()
        for o, op in zip(arr, ops):
            W, x, signs, y, n_out, n_in, flags = op[:7]
            aux = op[7] if len(op) > 7 else None
            o.W, o.x, o.y = _dev(W, "W").value, _dev(x, "x").value, _dev(y, "y").value
            o.signs = _dev(signs, "signs").value if signs is not None else None
            o.aux = _dev(aux, "aux").value if aux is not None else None
            o.eps = float(op[8]) if len(op) > 8 else 0.0
            o.src_len = int(op[9]) if len(op) > 9 else 0
            o.n_out, o.n_in, o.flags, o.reserved = n_out, n_in, flags, 0
        self._h = C.c_void_p()
        if peers is None:
            rc = lib().bonsai_b200_chain_create(C.cast(arr, C.c_void_p), len(ops), C.byref(self._h))
        else:       # several ranks: `peers` is a bonsai_b200.peer.PeerBuffer that holds every y of the list
            self._keep.append(peers)
            bases = (C.c_void_p * peers.world)(*peers.ptrs)
            rc = lib().bonsai_b200_chain_create_tp(C.cast(arr, C.c_void_p), len(ops), peers.rank, peers.world,
                                                  C.cast(bases, C.c_void_p), peers.total_bytes,
                                                  peers.counter_offset, wait_limit_us, C.byref(self._h))
        if rc != 0:
            self._h = C.c_void_p()
            raise RuntimeError(f"bonsai_b200_chain_create returned {rc}")
        self.n_ops = len(ops)

    def run(self):
        return lib().bonsai_b200_chain_run(self._h, _stream())

    def info(self):
        out = (C.c_int64 * 4)()
        rc = lib().bonsai_b200_chain_info(self._h, C.cast(out, C.c_void_p))
        if rc != 0:
            raise RuntimeError(f"bonsai_b200_chain_info returned {rc}")
        return {"threads": out[0], "nslot": out[1], "slot_bytes": out[2], "ctas": out[3]}

    def close(self):
        if self._h:
            lib().bonsai_b200_chain_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ---- include/bonsai_kv.h ---------------------------------------------------------------------------------
class KVCache:
    """bonsai_kv_create / _free and the calls on the handle.  Geometry of the 27B model: 16 cached layers, 4 kv heads,
    24 query heads, head dimension 256; 48 delta-net layers with [48][128][128] fp32 state."""
    N_LAYERS, N_KV_HEADS, N_HEADS, HEAD_DIM = 16, 4, 24, 256

    def __init__(self, capacity):
        self._h = lib().bonsai_kv_create(int(capacity), _stream())
        if not self._h:
            raise RuntimeError("bonsai_kv_create failed")
        self.capacity = capacity

    def append(self, layer, pos, k, v):
        return lib().bonsai_kv_append(self._h, layer, pos, _dev(k, "k"), _dev(v, "v"), _stream())

    def append_batch(self, layer, pos0, n_tok, k, v):
        return lib().bonsai_kv_append_batch(self._h, layer, pos0, n_tok, _dev(k, "k"), _dev(v, "v"), _stream())

    def attn_decode(self, layer, pos, q, out):
        return lib().bonsai_kv_attn_decode(self._h, layer, pos, _dev(q, "q"), _dev(out, "out"), _stream())

    def gdn_state(self, layer):
        return lib().bonsai_kv_gdn_state(self._h, layer)

    def reset(self):
        lib().bonsai_kv_reset(self._h, _stream())

    def arrays(self):
        """(K pointer, V pointer, bytes of each) on the device."""
        k, v, n = C.c_void_p(), C.c_void_p(), C.c_int64()
        assert lib().bonsai_b200_kv_arrays(self._h, C.byref(k), C.byref(v), C.byref(n)) == 0
        return k.value, v.value, n.value

    def close(self):
        if self._h:
            lib().bonsai_kv_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

