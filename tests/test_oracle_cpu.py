"""CPU suite: the C restatement against the committed golden vectors (made by the reference's own
host code) and, where oracle/_ref is present, against that code directly."""
import numpy as np
import pytest

from bonsai_b200 import synth


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


# ---- golden vectors -----------------------------------------------------------------------------
def test_f32_to_f16_golden(port, golden):
    got = np.array([port.f32_to_f16(v) for v in golden["f32_bits"].view(np.float32)], dtype=np.uint16)
    assert np.array_equal(got, golden["f16_bits"])


def test_f16_widen_golden(port, golden):
    got = np.array([np.float32(port.f16_to_f32(h)).view(np.uint32) for h in range(0, 65536, 37)], dtype=np.uint32)
    want = golden["f16_widen_bits"]
    nan = (want & 0x7F800000 == 0x7F800000) & (want & 0x7FFFFF != 0)
    assert np.array_equal(got[~nan], want[~nan])


def test_fwht_golden(port, golden):
    assert np.array_equal(bits(port.fwht_blocks(golden["x"])), golden["fwht_plain"])
    assert np.array_equal(bits(port.fwht_blocks(golden["x"], golden["signs"])), golden["fwht_signed"])


def test_quantiser_golden(port, golden):
    x = golden["x"]
    assert np.array_equal(port.quantize_q8_1(x, True), golden["q_raw_perm"])
    assert np.array_equal(port.quantize_q8_1(x, False), golden["q_raw_plain"])
    assert np.array_equal(port.quantize_q8_1(port.fwht_blocks(x, golden["signs"]), True), golden["q_rot_perm"])
    assert np.array_equal(port.quantize_q8_1(golden["x_ties"], True), golden["q_ties"])


def test_quantiser_ties_round_away(golden):
    # the tie vector quantises 0.5 -> 1, -0.5 -> -1, 2.5 -> 3 ... (ties away, not to even)
    q = golden["q_ties"][4:].view(np.int8)
    inv = [16 * (j >> 4) + 4 * (j & 3) + ((j >> 2) & 3) for j in range(32)]
    plain = np.empty(32, dtype=np.int8)
    for pos, src in enumerate(inv):
        plain[src] = q[pos]
    assert list(plain[:9]) == [127, 1, -1, 2, -2, 3, -3, 127, -127]


def test_gemv_golden(port, golden):
    y = port.gemv(golden["W"], golden["xq"], 12, 1024)
    assert np.array_equal(bits(y), golden["gemv_y"])
    assert np.array_equal(port.row_chunk_sums(golden["W"][3 * 272:4 * 272], golden["xq"], 1024),
                          golden["chunk_sums_row3"])
    assert np.array_equal(bits(port.gemv(golden["W"], golden["xq"], 12, 1024, threads=4)), golden["gemv_y"])


def test_gemm_golden(port, golden):
    assert np.array_equal(port.quantize_batch_chunk_major(golden["X"]), golden["Xq"])
    Y = port.gemm(golden["Wg"], golden["Xq"], 16, 256, 5)
    assert np.array_equal(bits(Y).reshape(-1), golden["gemm_Y"].reshape(-1))
    Ymt = port.gemm(golden["Wg"], golden["Xq"], 16, 256, 5, threads=3)
    assert np.array_equal(bits(Ymt).reshape(-1), golden["gemm_Y"].reshape(-1))


def test_repack_golden(port, golden):
    rp = port.repack(golden["W"], 12, 1024)
    assert np.array_equal(rp, golden["W_repacked"])
    for r in range(12):
        assert np.array_equal(port.unpack_row(rp[r * 272:(r + 1) * 272], 8), golden["W"][r * 272:(r + 1) * 272])
    y = port.gemv_repack(rp, golden["x"][:1024], 12, 1024)
    assert np.array_equal(bits(y), golden["gemv_repack_y"])


def test_weight_quantiser_golden(port, golden):
    assert np.array_equal(port.quantize_pq2_0(golden["w_float"]), golden["w_quant"])
    assert np.array_equal(bits(port.dequantize_pq2_0(golden["w_quant"])), golden["w_dequant"])


# ---- properties the reference's own tests assert (tests/test_p40.cpp sections 1, 2, 12) -------------
def test_fwht_involution_and_sylvester(port):
    x = synth.activations(1024, seed=7)
    twice = port.fwht_blocks(port.fwht_blocks(x))
    assert np.abs(twice - x).mean() < 1e-4
    i = np.arange(1024)
    sign = 1.0 - 2.0 * (np.bitwise_count(i[:, None] & i[None, :]) & 1)
    naive = (sign @ x.astype(np.float64)) / 32.0
    assert np.abs(port.fwht_blocks(x) - naive).max() < 1e-3


def test_permuted_layout_is_a_permutation(port):
    x = synth.activations(5120, seed=3) * 3.0
    perm = port.quantize_q8_1(x, True).reshape(-1, 36)
    plain = port.quantize_q8_1(x, False).reshape(-1, 36)
    src = [16 * (j >> 4) + 4 * (j & 3) + ((j >> 2) & 3) for j in range(32)]
    assert np.array_equal(perm[:, :4], plain[:, :4])
    assert np.array_equal(perm[:, 4:], plain[:, 4:][:, src])


def test_row_dot_matches_exact_integer_reference(port):
    n = 5120
    W = synth.pq2_0_weights(1, n, seed=1234)
    x = synth.activations(n, seed=1234) * 3.0
    perm = port.quantize_q8_1(x, True)
    plain = port.quantize_q8_1(x, False).reshape(-1, 36)
    got = port.gemv(W, perm, 1, n)[0]
    blocks = W.reshape(-1, 34)
    exact = 0.0
    for b in range(n // 128):
        dw = float(blocks[b, :2].view(np.float16)[0])
        codes = ((blocks[b, 2:, None] >> (2 * np.arange(4))) & 3).reshape(-1).astype(np.int64) - 1
        for c in range(4):
            a = plain[4 * b + c]
            da = float(a[:2].view(np.float16)[0])
            exact += dw * da * float((codes[32 * c:32 * c + 32] * a[4:].view(np.int8).astype(np.int64)).sum())
    assert abs(got - exact) <= 1e-2


def test_repack_geometry(port):
    for n_in in (5120, 17408, 6144, 10240, 12288, 1024):
        nb = n_in // 128
        assert nb % 8 == 0 and (2 * nb) % 16 == 0
        row = synth.pq2_0_weights(1, n_in, seed=nb)
        rp = port.repack_row(row, nb)
        assert rp.size == 34 * nb
        assert np.array_equal(port.unpack_row(rp, nb), row)
        # unit u = plane * nb + block holds code bytes 8*plane..8*plane+7 of that block
        blocks = row.reshape(nb, 34)
        units = rp[2 * nb:].reshape(4, nb, 8)
        for p in range(4):
            assert np.array_equal(units[p], blocks[:, 2 + 8 * p:10 + 8 * p])
        assert np.array_equal(rp[:2 * nb].reshape(nb, 2), blocks[:, :2])


def test_repack_dot_close_to_plain_dot(port):
    n_in, nb = 5120, 40
    W = synth.pq2_0_weights(3, n_in, seed=31337)
    x = synth.activations(n_in, seed=31337) * 3.0
    xq = port.quantize_q8_1(x, True)
    plain = port.gemv(W, xq, 3, n_in)
    rp = port.repack(W, 3, n_in)
    via = port.gemv_repack(rp, x, 3, n_in)
    assert np.abs(plain - via).max() <= 1e-3       # same integers, different fp32 order


# ---- the restatement against the reference build itself, on fresh inputs ------------------------------
@pytest.mark.parametrize("n_out,n_in,seed", [(5, 5120, 4242), (3, 17408, 1), (9, 1024, 2), (2, 6144, 3), (4, 384, 4)])
def test_port_equals_reference(port, ref, n_out, n_in, seed):
    W = synth.pq2_0_weights(n_out, n_in, seed=seed)
    x = synth.activations(n_in, seed=seed) * 2.0
    sg = synth.signs(n_in, seed=seed)
    if n_in % 1024 == 0:
        xr_p, xr_r = port.fwht_blocks(x, sg), ref.fwht_blocks(x, sg)
        assert np.array_equal(bits(xr_p), bits(xr_r))
        x = xr_r
    qp, qr = port.quantize_q8_1(x), ref.quantize_q8_1(x)
    assert np.array_equal(qp, qr)
    assert np.array_equal(bits(port.gemv(W, qp, n_out, n_in)), bits(ref.gemv(W, qr, n_out, n_in)))
    assert np.array_equal(port.row_chunk_sums(W[:34 * n_in // 128], qp, n_in),
                          ref.row_chunk_sums(W[:34 * n_in // 128], qr, n_in))
    if (n_in // 128) % 8 == 0:
        rp_p, rp_r = port.repack(W, n_out, n_in), ref.repack(W, n_out, n_in)
        assert np.array_equal(rp_p, rp_r)
        nb = n_in // 128
        for r in range(n_out):
            row = rp_p[r * 34 * nb:(r + 1) * 34 * nb]
            assert port.repack_row_dot(row, qp, nb).view(np.uint32) == ref.repack_row_dot(row, qr, nb).view(np.uint32)


def test_port_gemm_equals_reference(port, ref):
    n_out, n_in, n_tok = 64, 256, 5
    W = synth.pq2_0_weights(n_out, n_in, seed=31337)
    X = synth.activations(n_in, seed=31337, batch=n_tok) * 3.0
    Xq = port.quantize_batch_chunk_major(X)
    assert np.array_equal(Xq, ref.quantize_batch_chunk_major(X))
    assert np.array_equal(bits(port.gemm(W, Xq, n_out, n_in, n_tok)), bits(ref.gemm(W, Xq, n_out, n_in, n_tok)))


def test_port_f32_to_f16_equals_reference_dense(port, ref):
    rng = np.random.default_rng(9)
    vals = rng.integers(0, 2 ** 32, size=20000, dtype=np.uint64).astype(np.uint32).view(np.float32)
    for v in vals:
        assert port.f32_to_f16(v) == ref.f32_to_f16(v)


def test_port_ops_equal_reference(port, ref):
    """RMSNorm, SwiGLU and the delta-net step of the C restatement against the reference's src/ops.h, bit for bit."""
    rng = np.random.default_rng(11)
    x = rng.uniform(-2, 2, size=(3, 5120)).astype(np.float32)
    w = rng.uniform(0, 2, size=5120).astype(np.float32)
    assert np.array_equal(port.rmsnorm(x, w, 1e-6).view(np.uint32), ref.rmsnorm(x, w, 1e-6).view(np.uint32))
    g = rng.uniform(-4, 4, size=17408).astype(np.float32)
    u = rng.uniform(-2, 2, size=17408).astype(np.float32)
    assert np.array_equal(port.swiglu(g, u).view(np.uint32), ref.swiglu(g, u).view(np.uint32))
    S = (rng.uniform(-1, 1, size=(8, 128, 128)) * 0.1).astype(np.float32)
    q, k = rng.uniform(-1, 1, size=(2, 4, 128)).astype(np.float32)
    v = rng.uniform(-1, 1, size=(8, 128)).astype(np.float32)
    gg = (-rng.uniform(0.1, 1, size=8)).astype(np.float32)
    b = rng.uniform(0.1, 1, size=8).astype(np.float32)
    a, c = port.gdn_step(S, q, k, v, gg, b, 4, 8, 128, 128), ref.gdn_step(S, q, k, v, gg, b, 4, 8, 128, 128)
    assert np.array_equal(a[0].view(np.uint32), c[0].view(np.uint32)) and np.array_equal(a[1].view(np.uint32), c[1].view(np.uint32))


def test_port_kv_core_equals_reference(port, ref):
    """Q8_0 row quantiser, dequantiser and block score of src/kv_cache.h:100-145, bit for bit; exact ties and zeros."""
    rng = np.random.default_rng(12)
    x = (rng.standard_normal(4096) * 5).astype(np.float32)
    x[:32] = 0.0
    x[32:64] = np.arange(32, dtype=np.float32) + 0.5          # amax 31.5: many exact .5 ties after scaling
    a, b = port.kv_quantize_row(x), ref.kv_quantize_row(x)
    assert np.array_equal(a, b)
    assert np.array_equal(port.kv_dequantize_row(a).view(np.uint32), ref.kv_dequantize_row(a).view(np.uint32))
    for i in range(0, 16):
        qa, ka = a[i * 272:(i + 1) * 272], a[(15 - i) * 272:(16 - i) * 272]
        assert port.kv_score(qa, ka).view(np.uint32) == ref.kv_score(qa, ka).view(np.uint32)


def test_attention_recurrence_matches_full_softmax(port):
    """The online-softmax recurrence of the checker against a double-precision full softmax (the reference's own test of
    the recurrence, tests/test_p40.cpp:264-309, uses 1e-4)."""
    rng = np.random.default_rng(13)
    n_tok, n_head, n_kv, D = 33, 6, 2, 256
    q = rng.uniform(-1, 1, size=(n_tok, n_head, D)).astype(np.float32)
    k = rng.uniform(-1, 1, size=(n_tok, n_kv, D)).astype(np.float32)
    v = rng.uniform(-1, 1, size=(n_tok, n_kv, D)).astype(np.float32)
    scale = 1.0 / 16.0
    got = port.attn(q, k, v, n_tok, n_head, n_kv, D, scale).reshape(n_tok, n_head, D)
    for qi in (0, 7, 32):
        for h in (0, 5):
            kvh = h // (n_head // n_kv)
            s = (k[:qi + 1, kvh].astype(np.float64) @ q[qi, h].astype(np.float64)) * scale
            p = np.exp(s - s.max())
            want = (p[:, None] * v[:qi + 1, kvh].astype(np.float64)).sum(0) / p.sum()
            assert float(np.abs(got[qi, h] - want).max()) < 1e-5

