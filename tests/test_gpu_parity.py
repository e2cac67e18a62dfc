"""GPU parity: every entry point of the C ABI against the CPU checker, on the same inputs.

Bars: Q8_1 blocks, rotated fp32 values, int32 chunk sums and repacked bytes are compared bit for
bit.  fp32 outputs of the mat-vec are held to REL_TOL = 1e-5 (the bound the path states: max-abs
error over max |y| of the vector) in the default streaming order, whose per-chunk terms are the
host's bit for bit but are added in a fixed tree order; with the option gemv_order = 1, and for the
repacked mat-vec and the mat-mul always, the kernels keep the host's summation order and the
outputs are compared bit for bit as well.
"""
import numpy as np
import pytest

from bonsai_b200 import synth

pytestmark = pytest.mark.gpu

REL_TOL = 1e-5   # fp32 outputs: max |got - want| <= REL_TOL * max |want| per vector


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.detach().cpu().numpy()


def assert_close(got, want):
    scale = float(np.abs(want).max()) or 1.0
    err = float(np.abs(got.astype(np.float64) - want.astype(np.float64)).max())
    assert err <= REL_TOL * scale, f"max-abs {err:.3e} vs bound {REL_TOL * scale:.3e}"
    return err


def assert_close_and_exact(got, want):
    err = assert_close(got, want)
    assert np.array_equal(bits(got), bits(want)), f"not bit-identical (max-abs {err:.3e})"


class host_order:
    """Runs the mat-vec in the host's term-by-term summation order (bit-identical outputs)."""

    def __init__(self, gpu):
        self.gpu = gpu

    def __enter__(self):
        assert self.gpu.set_option("gemv_order", 1) == 0

    def __exit__(self, *a):
        self.gpu.set_option("gemv_order", 0)
        self.gpu.set_option("gemv_variant", -1)


# ---- activation side ---------------------------------------------------------------------------
@pytest.mark.parametrize("n", [32, 64, 1024, 5120, 17408, 32768])
def test_quantiser_bytes(gpu, port, n):
    import torch
    x = synth.activations(n, seed=n) * 2.5
    x[: min(32, n)] = 0.0
    out = torch.zeros(n // 32 * 36, dtype=torch.uint8, device="cuda")
    assert gpu.quant_activations(dev(x), out, n) == 0
    assert np.array_equal(host(out), port.quantize_q8_1(x, True))


def test_quantiser_golden_and_ties(gpu, golden):
    import torch
    for xin, want in ((golden["x"], golden["q_raw_perm"]), (golden["x_ties"], golden["q_ties"])):
        out = torch.zeros(want.size, dtype=torch.uint8, device="cuda")
        assert gpu.quant_activations(dev(xin), out, xin.size) == 0
        assert np.array_equal(host(out), want)


def test_quantiser_fp16_scale_ties(gpu, port):
    # chunks whose scale amax/127 falls exactly between two fp16 values: the host rounds away
    import torch
    n = 32 * 64
    x = np.zeros(n, dtype=np.float32)
    for c in range(64):
        half = np.uint32(0x3C00 + 16 * c)                              # an fp16 value
        tie = ((int(half) & 0x3FF) << 13 | ((int(half) >> 10) + 112) << 23 | 0x1000)
        d = np.array([tie], dtype=np.uint32).view(np.float32)[0]
        x[32 * c] = np.float32(d) * np.float32(127.0)
        x[32 * c + 1:32 * c + 32] = synth.activations(31, seed=c) * 0.1
    out = torch.zeros(n // 32 * 36, dtype=torch.uint8, device="cuda")
    assert gpu.quant_activations(dev(x), out, n) == 0
    assert np.array_equal(host(out), port.quantize_q8_1(x, True))


@pytest.mark.parametrize("n", [1024, 5120, 17408])
@pytest.mark.parametrize("signed", [False, True])
def test_fwht_bits(gpu, port, n, signed):
    import torch
    x = synth.activations(n, seed=n + 1)
    sg = synth.signs(n, seed=n) if signed else None
    want = port.fwht_blocks(x, sg)
    xd = dev(x)
    assert gpu.fwht(xd, None if sg is None else dev(sg), n) == 0
    assert np.array_equal(bits(host(xd)), bits(want))
    # fused rotation + quantiser: same bytes as the two calls, input left untouched
    xin = dev(x)
    xq = torch.zeros(n // 32 * 36, dtype=torch.uint8, device="cuda")
    xr = torch.zeros(n, dtype=torch.float32, device="cuda")
    assert gpu.fwht_quant(xin, None if sg is None else dev(sg), xq, xr, n) == 0
    assert np.array_equal(bits(host(xin)), bits(x))
    assert np.array_equal(bits(host(xr)), bits(want))
    assert np.array_equal(host(xq), port.quantize_q8_1(want, True))


def test_fwht_golden(gpu, golden):
    xd = dev(golden["x"])
    assert gpu.fwht(xd, dev(golden["signs"]), 2048) == 0
    assert np.array_equal(bits(host(xd)), golden["fwht_signed"])


@pytest.mark.parametrize("n_tok,n_in,rotate", [(5, 256, False), (1, 1024, True), (3, 2048, True), (17, 5120, True),
                                               (33, 384, False)])
def test_quant_batch_chunk_major(gpu, port, n_tok, n_in, rotate):
    import torch
    X = synth.activations(n_in, seed=n_tok, batch=n_tok) * 1.7
    sg = synth.signs(n_in, seed=3) if rotate else None
    Xr = np.stack([port.fwht_blocks(X[t], sg) for t in range(n_tok)]) if rotate else X
    want = port.quantize_batch_chunk_major(Xr)
    Xq = torch.zeros(want.size, dtype=torch.uint8, device="cuda")
    assert gpu.quant_batch(dev(X), None if sg is None else dev(sg), Xq, n_in, n_tok, rotate) == 0
    assert np.array_equal(host(Xq), want)


# ---- mat-vec --------------------------------------------------------------------------------------
GEMV_SHAPES = [(1, 128), (5, 5120), (31, 384), (33, 1024), (64, 17408), (130, 6144), (257, 256), (1024, 5120),
               (7, 32768), (300, 32768), (9000, 2048), (4097, 768), (20000, 256)]


def run_gemv(gpu, W, xq, n_out, n_in):
    import torch
    y = torch.full((n_out,), -12345.0, dtype=torch.float32, device="cuda")
    assert gpu.gemv(dev(W), dev(xq), y, n_out, n_in) == 0
    return host(y)


@pytest.mark.parametrize("n_out,n_in", GEMV_SHAPES)
def test_gemv_both_orders(gpu, port, n_out, n_in):
    W = synth.pq2_0_weights(n_out, n_in, seed=n_out)
    x = synth.activations(n_in, seed=n_in)
    xq = port.quantize_q8_1(x, True)
    want = port.gemv(W, xq, n_out, n_in, threads=4)
    assert_close(run_gemv(gpu, W, xq, n_out, n_in), want)
    with host_order(gpu):
        assert_close_and_exact(run_gemv(gpu, W, xq, n_out, n_in), want)


@pytest.mark.parametrize("variant", [0, 1000, 2000, 3000, 100, 300, 400, 500, 10, 70, 50, 1, 2, 1113, 1040])
@pytest.mark.parametrize("n_out,n_in", [(5, 5120), (203, 5120), (100, 17408), (37, 1024), (6000, 5120), (2500, 17408),
                                        (1500, 6144), (700, 8192), (130, 2304)])
def test_gemv_stream_every_tiling(gpu, port, variant, n_out, n_in):
    """Segment length, tile height, thread count and ring depth of the streaming kernel: the result
    stays within the bound, and is the SAME bits for every tiling that shares a segment length
    (the summation tree depends on nothing else)."""
    W = synth.pq2_0_weights(n_out, n_in, seed=variant + n_out)
    xq = port.quantize_q8_1(synth.activations(n_in, seed=variant), True)
    want = port.gemv(W, xq, n_out, n_in, threads=4)
    try:
        assert gpu.set_option("gemv_variant", variant) == 0
        got = run_gemv(gpu, W, xq, n_out, n_in)
        assert_close(got, want)
        again = run_gemv(gpu, W, xq, n_out, n_in)
        assert np.array_equal(bits(got), bits(again))        # deterministic from launch to launch
    finally:
        gpu.set_option("gemv_variant", -1)


@pytest.mark.parametrize("variant", [0, 10000, 20000, 11000, 12000, 15000, 16000, 10100, 10200, 10500, 10010, 10020,
                                     10001, 10002, 10003, 25100, 5510, 110000, 210010, 300020, 110030])
@pytest.mark.parametrize("n_out,n_in", [(5, 5120), (203, 5120), (100, 17408), (37, 1024), (6000, 5120), (2500, 17408)])
def test_gemv_every_tiling(gpu, port, variant, n_out, n_in):
    """Rows per lane (1/2/4), segment length, tile height, adder warps and ring depth change only
    the schedule, never a bit of y.  The two large shapes wrap the ring several times."""
    W = synth.pq2_0_weights(n_out, n_in, seed=variant + n_out)
    xq = port.quantize_q8_1(synth.activations(n_in, seed=variant), True)
    want = port.gemv(W, xq, n_out, n_in, threads=4)
    with host_order(gpu):
        assert gpu.set_option("gemv_variant", variant) == 0
        assert_close_and_exact(run_gemv(gpu, W, xq, n_out, n_in), want)


@pytest.mark.parametrize("order", [0, 1])
def test_gemv_programmatic_launch_same_bits(gpu, port, order):
    import torch
    n_out, n_in = 640, 5120
    W = synth.pq2_0_weights(n_out, n_in, seed=77)
    x = synth.activations(n_in, seed=77)
    want = port.gemv(W, port.quantize_q8_1(port.fwht_blocks(x), True), n_out, n_in, threads=4)
    Wd, xd = dev(W), dev(x)
    xq = torch.zeros(n_in // 32 * 36, dtype=torch.uint8, device="cuda")
    y = torch.zeros(n_out, dtype=torch.float32, device="cuda")
    try:
        gpu.set_option("gemv_order", order)
        assert gpu.gemv(Wd, dev(port.quantize_q8_1(port.fwht_blocks(x), True)), y, n_out, n_in) == 0
        plain = host(y).copy()
        gpu.set_option("pdl", 1)
        for _ in range(5):   # back-to-back dependent chains on one stream
            assert gpu.fwht_quant(xd, None, xq, None, n_in) == 0
            assert gpu.gemv(Wd, xq, y, n_out, n_in) == 0
        torch.cuda.synchronize()
        assert np.array_equal(bits(host(y)), bits(plain))
        (assert_close_and_exact if order else assert_close)(host(y), want)
    finally:
        gpu.set_option("pdl", 0)
        gpu.set_option("gemv_order", 0)


MMA_SHAPES = [(5, 5120), (16, 256), (203, 5120), (100, 17408), (37, 1024), (2400, 5120), (700, 17408), (1500, 6144),
              (130, 2304), (33, 8192), (4, 256), (250, 10240)]


@pytest.mark.parametrize("n_out,n_in", MMA_SHAPES)
def test_gemv_tensor_core_body_ints_and_bound(gpu, port, n_out, n_in):
    """The mat-vec whose integer products run on mma.sync (gemv_order = 2): the int32 chunk sums that the kernel
    itself formed (bonsai_b200_gemv_dump) equal the host's bit for bit on every row and chunk; y stays within the
    bound; the plain entry point gives the same bits as the dumping one; rows give the same bits wherever they sit
    in the matrix (a row slice, as a rank of a row-partitioned run would hold it)."""
    import torch
    W = synth.pq2_0_weights(n_out, n_in, seed=n_out + 3)
    x = synth.activations(n_in, seed=n_out + 3)
    xq = port.quantize_q8_1(port.fwht_blocks(x) if n_in % 1024 == 0 else x, True)
    Wd, xqd = dev(W), dev(xq)
    y = torch.full((n_out,), 7.0, dtype=torch.float32, device="cuda")
    sums = torch.full((n_out, n_in // 32), -12345, dtype=torch.int32, device="cuda")
    assert gpu.gemv_dump(Wd, xqd, y, sums, n_out, n_in) == 0
    want = port.gemv(W, xq, n_out, n_in)
    assert_close(host(y), want)
    row_bytes = n_in // 128 * 34
    got_sums = host(sums)
    for r in sorted({r for r in (0, 1, 7, 8, 15, 16, n_out // 2, n_out - 1) if r < n_out}):
        want_sums = port.row_chunk_sums(W[r * row_bytes:(r + 1) * row_bytes], xq, n_in)
        assert np.array_equal(got_sums[r], want_sums), r
    try:
        assert gpu.set_option("gemv_order", 2) == 0
        y2 = torch.zeros(n_out, dtype=torch.float32, device="cuda")
        assert gpu.gemv(Wd, xqd, y2, n_out, n_in) == 0
        assert np.array_equal(bits(host(y2)), bits(host(y)))
        if n_out >= 40:
            lo, hi = 16 + 3, n_out - 2          # a slice that starts in the middle of a 16-row group
            ys = torch.zeros(hi - lo, dtype=torch.float32, device="cuda")
            Ws = dev(W[lo * row_bytes:hi * row_bytes]) if (lo * row_bytes) % 16 else Wd[lo * row_bytes:hi * row_bytes]
            assert gpu.gemv(Ws, xqd, ys, hi - lo, n_in) == 0
            assert np.array_equal(bits(host(ys)), bits(host(y)[lo:hi]))
    finally:
        gpu.set_option("gemv_order", 0)
    assert gpu.device_status() == 0


def test_gemv_unaligned_weights_take_the_generic_kernel(gpu, port):
    import torch
    n_out, n_in = 19, 1024
    W = synth.pq2_0_weights(n_out, n_in, seed=8)
    xq = port.quantize_q8_1(synth.activations(n_in, seed=8), True)
    buf = torch.zeros(W.size + 16, dtype=torch.uint8, device="cuda")
    buf[2:2 + W.size] = dev(W)
    y = torch.zeros(n_out, dtype=torch.float32, device="cuda")
    assert gpu.gemv(buf[2:], dev(xq), y, n_out, n_in) == 0
    assert_close_and_exact(host(y), port.gemv(W, xq, n_out, n_in))      # the fallback keeps the host order


def test_gemv_golden(gpu, golden):
    want = golden["gemv_y"].view(np.float32)
    assert_close(run_gemv(gpu, golden["W"], golden["xq"], 12, 1024), want)
    with host_order(gpu):
        got = run_gemv(gpu, golden["W"], golden["xq"], 12, 1024)
    assert np.array_equal(bits(got), golden["gemv_y"])


def test_chunk_sums_int_exact(gpu, port, golden):
    import torch
    n_out, n_in = 40, 5120
    W = synth.pq2_0_weights(n_out, n_in, seed=21)
    xq = port.quantize_q8_1(synth.activations(n_in, seed=21) * 4.0, True)
    out = torch.zeros((6, n_in // 32), dtype=torch.int32, device="cuda")
    assert gpu.gemv_chunk_sums(dev(W), dev(xq), out, 17, 6, n_in) == 0
    rb = 34 * n_in // 128
    for i in range(6):
        assert np.array_equal(host(out)[i], port.row_chunk_sums(W[(17 + i) * rb:(18 + i) * rb], xq, n_in))
    g = torch.zeros((1, 32), dtype=torch.int32, device="cuda")
    assert gpu.gemv_chunk_sums(dev(golden["W"]), dev(golden["xq"]), g, 3, 1, 1024) == 0
    assert np.array_equal(host(g)[0], golden["chunk_sums_row3"])


@pytest.mark.parametrize("n_in,n_out", [(5120, 5120), (5120, 1024), (5120, 17408), (17408, 5120)])
def test_gemv_full_layer_shapes(gpu, port, n_in, n_out):
    """The projection shapes of one transformer layer at full size, rotated + quantised on the GPU;
    the whole output is checked (the CPU checker needs well under a second per shape)."""
    import torch
    W = synth.pq2_0_weights(n_out, n_in, seed=0)
    x = synth.activations(n_in, seed=0)
    xq = torch.zeros(n_in // 32 * 36, dtype=torch.uint8, device="cuda")
    assert gpu.fwht_quant(dev(x), None, xq, None, n_in) == 0
    want_xq = port.quantize_q8_1(port.fwht_blocks(x), True)
    assert np.array_equal(host(xq), want_xq)
    y = torch.zeros(n_out, dtype=torch.float32, device="cuda")
    Wd = dev(W)
    want = port.gemv(W, want_xq, n_out, n_in, threads=8)
    assert gpu.gemv(Wd, xq, y, n_out, n_in) == 0
    err = assert_close(host(y), want)
    print(f"n_in={n_in} n_out={n_out}: max-abs {err:.3e}, max|y| {np.abs(want).max():.3f}")
    with host_order(gpu):
        assert gpu.gemv(Wd, xq, y, n_out, n_in) == 0
        assert_close_and_exact(host(y), want)


def test_gemv_linearity_in_the_weight_scale(gpu, port):
    """Size-independent property: doubling every fp16 block scale doubles y exactly."""
    n_out, n_in = 300, 5120
    W = synth.pq2_0_weights(n_out, n_in, seed=9).reshape(-1, 34).copy()
    xq = port.quantize_q8_1(synth.activations(n_in, seed=9), True)
    y1 = run_gemv(gpu, W.reshape(-1), xq, n_out, n_in)
    d = W[:, :2].copy().view(np.float16)
    W[:, :2] = (d * np.float16(2.0)).view(np.uint8)
    y2 = run_gemv(gpu, W.reshape(-1), xq, n_out, n_in)
    assert np.array_equal(bits(y2), bits(y1 * np.float32(2.0)))


@pytest.mark.parametrize("n_out,n_in,signed", [(640, 5120, False), (300, 17408, True), (9, 1024, True)])
def test_linear_one_call(gpu, port, n_out, n_in, signed):
    """Rotation + quantiser + mat-vec through the single entry point with a caller-provided scratch."""
    import torch
    W = synth.pq2_0_weights(n_out, n_in, seed=n_out)
    x = synth.activations(n_in, seed=n_out)
    sg = synth.signs(n_in, seed=1) if signed else None
    scratch = torch.zeros(n_in // 32 * 36, dtype=torch.uint8, device="cuda")
    y = torch.zeros(n_out, dtype=torch.float32, device="cuda")
    xd = dev(x)
    Wd, sd = dev(W), None if sg is None else dev(sg)
    assert gpu.linear(Wd, xd, sd, y, scratch, n_out, n_in) == 0          # default: two launches
    want_xq = port.quantize_q8_1(port.fwht_blocks(x, sg), True)
    assert np.array_equal(host(scratch), want_xq)
    assert np.array_equal(bits(host(xd)), bits(x))
    assert_close(host(y), port.gemv(W, want_xq, n_out, n_in, threads=4))
    fused = host(y).copy()
    try:
        gpu.set_option("fuse_linear", 1)                                  # one kernel, rotation in its prologue: same bits
        y.zero_()
        scratch.zero_()
        assert gpu.linear(Wd, xd, sd, y, scratch, n_out, n_in) == 0
    finally:
        gpu.set_option("fuse_linear", 0)
    assert np.array_equal(host(scratch), want_xq)
    assert np.array_equal(bits(host(y)), bits(fused))
    assert gpu.linear(Wd, xd, None, y, scratch, n_out, 1000) == 1


# ---- repacked layout ----------------------------------------------------------------------------------
@pytest.mark.parametrize("n_out,n_in", [(12, 1024), (5, 5120), (67, 17408), (300, 6144)])
def test_repack_bytes_and_gemv(gpu, port, n_out, n_in):
    import torch
    W = synth.pq2_0_weights(n_out, n_in, seed=n_in)
    x = synth.activations(n_in, seed=n_out) * 1.3
    Wr = torch.zeros(W.size, dtype=torch.uint8, device="cuda")
    assert gpu.repack(dev(W), Wr, n_out, n_in) == 0
    want_r = port.repack(W, n_out, n_in)
    assert np.array_equal(host(Wr), want_r)
    y = torch.zeros(n_out, dtype=torch.float32, device="cuda")
    want = port.gemv_repack(want_r, x, n_out, n_in)
    assert gpu.gemv_repack(Wr, dev(x), y, n_out, n_in) == 0          # default: terms of a row added by a warp, fixed tree
    assert_close(host(y), want)
    y2 = torch.zeros(n_out, dtype=torch.float32, device="cuda")
    assert gpu.gemv_repack(Wr, dev(x), y2, n_out, n_in) == 0
    assert np.array_equal(bits(host(y2)), bits(host(y)))               # ... the same bits on every launch
    with host_order(gpu):                                              # unit order: the bits of repack_row_dot
        assert gpu.gemv_repack(Wr, dev(x), y, n_out, n_in) == 0
    assert_close_and_exact(host(y), want)


def test_repack_source_two_byte_aligned(gpu, port):
    # a source that is only 2-byte aligned takes the kernel with 2-byte loads: the same bytes
    import torch
    n_out, n_in = 67, 2048
    W = synth.pq2_0_weights(n_out, n_in, seed=9)
    buf = torch.zeros(W.size + 16, dtype=torch.uint8, device="cuda")
    buf[2:2 + W.size] = dev(W)
    Wr = torch.zeros(W.size, dtype=torch.uint8, device="cuda")
    assert gpu.repack(buf[2:], Wr, n_out, n_in) == 0
    assert np.array_equal(host(Wr), port.repack(W, n_out, n_in))
    assert gpu.repack(buf[1:], Wr, n_out, n_in) == 1


def test_repack_golden(gpu, golden):
    import torch
    Wr = torch.zeros(golden["W"].size, dtype=torch.uint8, device="cuda")
    assert gpu.repack(dev(golden["W"]), Wr, 12, 1024) == 0
    assert np.array_equal(host(Wr), golden["W_repacked"])
    y = torch.zeros(12, dtype=torch.float32, device="cuda")
    with host_order(gpu):
        assert gpu.gemv_repack(Wr, dev(golden["x"][:1024]), y, 12, 1024) == 0
    assert np.array_equal(bits(host(y)), golden["gemv_repack_y"])


@pytest.mark.parametrize("variant", [1, 1011, 2311])
def test_gemv_repack_every_tiling(gpu, port, variant):
    import torch
    n_out, n_in = 101, 5120
    W = synth.pq2_0_weights(n_out, n_in, seed=variant)
    x = synth.activations(n_in, seed=variant)
    want_r = port.repack(W, n_out, n_in)
    y = torch.zeros(n_out, dtype=torch.float32, device="cuda")
    want = port.gemv_repack(want_r, x, n_out, n_in)
    try:
        gpu.set_option("gemv_variant", variant)
        assert gpu.gemv_repack(dev(want_r), dev(x), y, n_out, n_in) == 0
        assert_close(host(y), want)
        with host_order(gpu):
            assert gpu.gemv_repack(dev(want_r), dev(x), y, n_out, n_in) == 0
    finally:
        gpu.set_option("gemv_variant", -1)
    assert_close_and_exact(host(y), want)


# ---- mat-mul ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("n_out,n_in,n_tok", [(64, 256, 5), (5, 128, 1), (70, 384, 33), (256, 5120, 17), (130, 1024, 64),
                                              (96, 17408, 8)])
def test_gemm_bits(gpu, port, n_out, n_in, n_tok):
    import torch
    W = synth.pq2_0_weights(n_out, n_in, seed=n_tok)
    X = synth.activations(n_in, seed=n_out, batch=n_tok)
    Xq = port.quantize_batch_chunk_major(X)
    Y = torch.full((n_out, n_tok), 777.0, dtype=torch.float32, device="cuda")
    try:
        assert gpu.set_option("gemm_path", 0) == 0          # the integer SIMT kernel: the host loop's bits
        assert gpu.gemm(dev(W), dev(Xq), Y, n_out, n_in, n_tok) == 0
    finally:
        gpu.set_option("gemm_path", -1)
    assert_close_and_exact(host(Y), port.gemm(W, Xq, n_out, n_in, n_tok, threads=8))


@pytest.mark.parametrize("n_in,n_out,n_tok", [(17408, 5120, 8), (5120, 17408, 1), (5120, 17408, 8), (2048, 20000, 5)])
def test_row_partition_assembles_full_result(gpu, port, n_in, n_out, n_tok):
    """The multi-GPU split on one device: 8 ranks' row slices (contiguous byte ranges of W), each
    multiplied on its own, written where an all-gather would put them, equal the unsplit result bit
    for bit (batch 8 through the mat-mul entry point, batch 1 through the mat-vec)."""
    import torch
    from bonsai_b200 import partition
    W = synth.pq2_0_weights(n_out, n_in, seed=3)
    X = synth.activations(n_in, seed=4, batch=n_tok)
    Wd = dev(W)
    if n_tok == 1:
        xq = port.quantize_q8_1(X.reshape(-1), True)
        want = port.gemv(W, xq, n_out, n_in, threads=8)
        xqd = dev(xq)
        y = torch.zeros(n_out, device="cuda")
        with host_order(gpu):
            for r in range(8):
                lo, hi = partition.row_slice(n_out, r, 8)
                b0, b1 = partition.byte_slice(n_out, n_in, r, 8)
                assert gpu.gemv(Wd[b0:b1], xqd, y[lo:hi], hi - lo, n_in) == 0
        assert_close_and_exact(host(y), want)
    else:
        # batch 8 takes the streaming small-batch kernel: within the bound of the host loop, and the slices give the
        # bits of the unsplit call (a row's sum does not depend on where the row sits)
        Xq = port.quantize_batch_chunk_major(X)
        want = port.gemm(W, Xq, n_out, n_in, n_tok, threads=8)
        Xqd = dev(Xq)
        Y = torch.zeros(n_out, n_tok, device="cuda")
        for r in range(8):
            lo, hi = partition.row_slice(n_out, r, 8)
            b0, b1 = partition.byte_slice(n_out, n_in, r, 8)
            assert gpu.gemm(Wd[b0:b1], Xqd, Y[lo:hi], hi - lo, n_in, n_tok) == 0
        assert_close(host(Y), want)
        Yu = torch.zeros(n_out, n_tok, device="cuda")
        assert gpu.gemm(Wd, Xqd, Yu, n_out, n_in, n_tok) == 0
        assert np.array_equal(bits(host(Y)), bits(host(Yu)))


@pytest.mark.parametrize("n_out,n_in,n_tok", [(128, 128, 64), (64, 256, 5), (300, 5120, 100), (1024, 5120, 512), (200, 17408, 130),
                                              (129, 384, 65)])
def test_gemm_simt_kernel_keeps_the_host_bits(gpu, port, n_out, n_in, n_tok):
    """Integer SIMT kernel (gemm_path 0): bit-identical to the host loop, on full tiles, ragged rows, ragged
    tokens and odd block counts."""
    import torch
    W = synth.pq2_0_weights(n_out, n_in, seed=n_tok)
    X = synth.activations(n_in, seed=n_out, batch=n_tok)
    Xq = port.quantize_batch_chunk_major(X)
    Y = torch.full((n_out, n_tok), 777.0, dtype=torch.float32, device="cuda")
    try:
        assert gpu.set_option("gemm_path", 0) == 0
        assert gpu.gemm(dev(W), dev(Xq), Y, n_out, n_in, n_tok) == 0
        torch.cuda.synchronize()
    finally:
        gpu.set_option("gemm_path", -1)
    assert_close_and_exact(host(Y), port.gemm(W, Xq, n_out, n_in, n_tok, threads=8))
    assert gpu.device_status() == 0


def _chunk_ints(port, W, Xq, n_out, n_in, n_tok, rows, toks):
    """The host loop's int32 (sum code * a - sum a) for the given rows and tokens: [len(rows)][len(toks)][n_in/32]."""
    nch = n_in // 32
    row_bytes = n_in // 128 * 34
    xb = Xq.reshape(nch, n_tok, 36)
    out = np.zeros((len(rows), len(toks), nch), dtype=np.int32)
    for j, t in enumerate(toks):
        xq_t = np.ascontiguousarray(xb[:, t, :]).reshape(-1)
        for i, r in enumerate(rows):
            out[i, j] = port.row_chunk_sums(W[r * row_bytes:(r + 1) * row_bytes], xq_t, n_in)
    return out


@pytest.mark.parametrize("n_out,n_in,n_tok", [(128, 128, 64), (64, 256, 5), (300, 1024, 100), (256, 5120, 128), (129, 384, 65),
                                              (6400, 256, 384), (19072, 256, 130), (203, 5120, 8), (100, 17408, 8),
                                              (37, 1024, 2), (1500, 6144, 3), (130, 2304, 7), (33, 8192, 8),
                                              (40000, 4096, 8), (38500, 256, 3), (300, 1024, 9), (200, 5120, 33)])
def test_gemm_tensor_core_ints_and_bound(gpu, port, n_out, n_in, n_tok):
    """The two tensor-core mat-muls -- tcgen05 for token batches (gemm_path 1), mma.sync with the weights streamed once
    for 2 .. 8 tokens (gemm_path 2) -- : the int32 the tensor core produced for every (row, token, chunk) -- written out
    by bonsai_b200_gemm_dump -- equals the host loop's integer bit for bit on sampled rows and tokens, and Y is
    within 1e-5 of max |Y| of the host loop (fp32 side: fused multiply-adds per block, see csrc/gemm_tc.cuh); the
    plain entry point gives the same Y bits as the dumping one.  Full tiles, ragged rows and tokens, odd block
    counts, tile counts that do not divide over the SMs (tiles cut in two between neighbouring CTAs), and for the
    small-batch kernel more than 16 row groups per CTA (several batches of groups, with and without row segments)."""
    import torch
    W = synth.pq2_0_weights(n_out, n_in, seed=n_tok + 1)
    X = synth.activations(n_in, seed=n_out, batch=n_tok)
    Xq = port.quantize_batch_chunk_major(X)
    Wd, Xqd = dev(W), dev(Xq)
    nch = n_in // 32
    Y = torch.full((n_out, n_tok), 777.0, dtype=torch.float32, device="cuda")
    sums = torch.full((n_out, n_tok, nch), -12345, dtype=torch.int32, device="cuda")
    assert gpu.gemm_dump(Wd, Xqd, Y, sums, n_out, n_in, n_tok) == 0
    torch.cuda.synchronize()
    want = port.gemm(W, Xq, n_out, n_in, n_tok, threads=8)
    assert_close(host(Y), want)
    rows = sorted({0, 1, 31, 32, 127 % n_out, 128 % n_out, n_out // 2, n_out - 1})
    toks = sorted({0, 1, 15, 16, 31, 32, 63, 127, 128, n_tok // 2, n_tok - 1} & set(range(n_tok)))
    got = host(sums)[np.ix_(rows, toks)]
    assert np.array_equal(got, _chunk_ints(port, W, Xq, n_out, n_in, n_tok, rows, toks))
    assert not (host(sums) == -12345).any()          # every (row, token, chunk) was produced
    Y2 = torch.full((n_out, n_tok), 555.0, dtype=torch.float32, device="cuda")
    try:
        assert gpu.set_option("gemm_path", 2 if n_tok <= 8 else 3) == 0
        assert gpu.gemm(Wd, Xqd, Y2, n_out, n_in, n_tok) == 0
        torch.cuda.synchronize()
    finally:
        gpu.set_option("gemm_path", -1)
    assert np.array_equal(bits(host(Y2)), bits(host(Y)))
    assert gpu.device_status() == 0


@pytest.mark.parametrize("n_out,n_in,n_tok", [(203, 5120, 9), (100, 17408, 16), (1500, 6144, 12), (40000, 4096, 13),
                                              (33, 1024, 10)])
def test_gemm_small_batch_up_to_16_tokens(gpu, port, n_out, n_in, n_tok):
    """9 .. 16 tokens through the streaming kernel (two token groups per code extraction; the default for matrices of up
    to ~100 MB, gemm_path 2 asks for it): Y within 1e-5 of max |Y| of the host loop, every element written, the same
    bits on a second call and from the default dispatch."""
    import torch
    W = synth.pq2_0_weights(n_out, n_in, seed=n_tok + 5)
    X = synth.activations(n_in, seed=n_out + 2, batch=n_tok)
    Xq = port.quantize_batch_chunk_major(X)
    Wd, Xqd = dev(W), dev(Xq)
    Y = torch.full((n_out, n_tok), float("nan"), dtype=torch.float32, device="cuda")
    Y2 = torch.full((n_out, n_tok), float("nan"), dtype=torch.float32, device="cuda")
    try:
        assert gpu.set_option("gemm_path", 2) == 0
        assert gpu.gemm(Wd, Xqd, Y, n_out, n_in, n_tok) == 0
    finally:
        gpu.set_option("gemm_path", -1)
    assert gpu.gemm(Wd, Xqd, Y2, n_out, n_in, n_tok) == 0
    torch.cuda.synchronize()
    assert gpu.device_status() == 0
    assert np.isfinite(host(Y)).all()
    assert_close(host(Y), port.gemm(W, Xq, n_out, n_in, n_tok, threads=8))
    assert np.array_equal(bits(host(Y2)), bits(host(Y)))


def test_gemm_small_batch_word_aligned_activations(gpu, port):
    """Xq that is only 4-byte aligned: the small-batch kernel stages the blocks with plain loads; same Y bits."""
    import torch
    n_out, n_in, n_tok = 200, 5120, 6
    W = synth.pq2_0_weights(n_out, n_in, seed=21)
    X = synth.activations(n_in, seed=22, batch=n_tok)
    Xq = port.quantize_batch_chunk_major(X)
    Wd = dev(W)
    buf = torch.zeros(Xq.size + 16, dtype=torch.uint8, device="cuda")
    buf[4:4 + Xq.size] = dev(Xq)
    Y = torch.zeros(n_out, n_tok, device="cuda")
    Y2 = torch.zeros(n_out, n_tok, device="cuda")
    assert gpu.gemm(Wd, dev(Xq), Y, n_out, n_in, n_tok) == 0
    assert gpu.gemm(Wd, buf[4:], Y2, n_out, n_in, n_tok) == 0
    assert_close(host(Y), port.gemm(W, Xq, n_out, n_in, n_tok, threads=8))
    assert np.array_equal(bits(host(Y2)), bits(host(Y)))
    assert gpu.device_status() == 0


@pytest.mark.parametrize("n_out,n_in,n_tok", [(128, 1024, 64), (300, 1024, 100), (256, 5120, 128), (129, 2048, 65),
                                              (6400, 1024, 384), (19072, 1024, 130), (1000, 17408, 48), (5120, 5120, 512),
                                              (700, 5120, 9), (260, 17408, 20), (5120, 2048, 47)])
def test_gemm_tensor_core_fp16_bound(gpu, port, n_out, n_in, n_tok):
    """The fp16 tensor-core mat-mul (gemm_path 1: activations split into two fp16 planes, whole blocks accumulated in
    tensor memory, csrc/gemm_tc16.cuh): Y within 1e-5 of max |Y| of the host loop on sampled rows, every element
    written, the same bits on a second call.  Full tiles, ragged rows and tokens, tiles cut in two between CTAs; a
    second shape on the same stream (the scratch grows), and large activation ranges (per-token power-of-two scale)."""
    import torch
    W = synth.pq2_0_weights(n_out, n_in, seed=n_tok + 3)
    X = synth.activations(n_in, seed=n_out + 1, batch=n_tok)
    X[::3] *= 1000.0                                    # tokens of very different magnitude
    X[1::7] *= 1e-4
    Xq = port.quantize_batch_chunk_major(X)
    Wd, Xqd = dev(W), dev(Xq)
    Y = torch.full((n_out, n_tok), float("nan"), dtype=torch.float32, device="cuda")
    Y2 = torch.full((n_out, n_tok), float("nan"), dtype=torch.float32, device="cuda")
    try:
        assert gpu.set_option("gemm_path", 1) == 0
        assert gpu.gemm(Wd, Xqd, Y, n_out, n_in, n_tok) == 0
        assert gpu.gemm(Wd, Xqd, Y2, n_out, n_in, n_tok) == 0
        torch.cuda.synchronize()
    finally:
        gpu.set_option("gemm_path", -1)
    assert gpu.device_status() == 0
    y = host(Y)
    assert np.isfinite(y).all()
    assert np.array_equal(bits(y), bits(host(Y2)))
    rows = np.unique(np.concatenate([np.arange(min(n_out, 130)), np.arange(max(0, n_out - 130), n_out),
                                     np.linspace(0, n_out - 1, 64).astype(np.int64)]))
    row_bytes = n_in // 128 * 34
    Wsub = np.concatenate([W[r * row_bytes:(r + 1) * row_bytes] for r in rows])
    want = port.gemm(Wsub, Xq, len(rows), n_in, n_tok, threads=8)
    # the bound is per token: tokens differ by seven orders of magnitude here
    for t in range(n_tok):
        ref = want[:, t]
        err = np.abs(y[rows, t] - ref).max()
        assert err <= 1e-5 * max(np.abs(ref).max(), 1e-30), (t, err, np.abs(ref).max())


def test_gemm_default_dispatch(gpu, port):
    """By token count: one token is the mat-vec; 2 .. 16 the streaming small-batch kernel; more the tcgen05 kernel."""
    import torch
    n_out, n_in = 256, 1024
    W = synth.pq2_0_weights(n_out, n_in, seed=9)
    for n_tok, exact in ((1, False), (8, False), (9, False), (20, False), (47, False), (512, False)):
        X = synth.activations(n_in, seed=n_tok, batch=n_tok)
        Xq = port.quantize_batch_chunk_major(X)
        Y = torch.zeros((n_out, n_tok), dtype=torch.float32, device="cuda")
        assert gpu.gemm(dev(W), dev(Xq), Y, n_out, n_in, n_tok) == 0
        want = port.gemm(W, Xq, n_out, n_in, n_tok, threads=8)
        if exact:
            assert_close_and_exact(host(Y), want)
        else:
            assert_close(host(Y), want)


def test_gemm_golden(gpu, golden):
    import torch
    Y = torch.zeros((16, 5), dtype=torch.float32, device="cuda")
    try:
        assert gpu.set_option("gemm_path", 0) == 0          # the kernel that keeps the host loop's bits
        assert gpu.gemm(dev(golden["Wg"]), dev(golden["Xq"]), Y, 16, 256, 5) == 0
    finally:
        gpu.set_option("gemm_path", -1)
    assert np.array_equal(bits(host(Y)).reshape(-1), golden["gemm_Y"].reshape(-1))


def test_gemm_one_token_equals_gemv(gpu, port):
    import torch
    n_out, n_in = 200, 5120
    W = synth.pq2_0_weights(n_out, n_in, seed=4)
    xq = port.quantize_q8_1(synth.activations(n_in, seed=4), True)
    # one token is the mat-vec: the same bits as bonsai_p40_gemv, in its default order and in the host's
    Y = torch.zeros((n_out, 1), dtype=torch.float32, device="cuda")
    assert gpu.gemm(dev(W), dev(xq), Y, n_out, n_in, 1) == 0
    assert np.array_equal(bits(host(Y)).reshape(-1), bits(run_gemv(gpu, W, xq, n_out, n_in)))
    with host_order(gpu):
        assert gpu.gemm(dev(W), dev(xq), Y, n_out, n_in, 1) == 0
        assert np.array_equal(bits(host(Y)).reshape(-1), bits(run_gemv(gpu, W, xq, n_out, n_in)))
        assert_close_and_exact(host(Y).reshape(-1), port.gemv(W, xq, n_out, n_in, threads=4))
    try:                                                # the integer SIMT kernel keeps the host's bits at any token count
        assert gpu.set_option("gemm_path", 0) == 0
        assert gpu.gemm(dev(W), dev(xq), Y, n_out, n_in, 1) == 0
    finally:
        gpu.set_option("gemm_path", -1)
    assert_close_and_exact(host(Y).reshape(-1), port.gemv(W, xq, n_out, n_in, threads=4))


# ---- synthetic weights, status ----------------------------------------------------------------------------
def test_synthetic_weights_distribution_and_slices(gpu):
    import torch
    nblk = 40 * 2048
    W = torch.zeros(nblk * 34, dtype=torch.uint8, device="cuda")
    assert gpu.synth_pq2_0(W, 0, nblk, 0) == 0
    w = host(W).reshape(nblk, 34)
    codes = ((w[:, 2:, None] >> (2 * np.arange(4))) & 3).reshape(-1)
    freq = np.bincount(codes, minlength=4) / codes.size
    assert abs(freq[0] - 0.33) < 0.005 and abs(freq[1] - 0.34) < 0.005 and abs(freq[2] - 0.33) < 0.005
    assert 0.0005 < freq[3] < 0.0015
    d = w[:, :2].copy().view(np.float16).astype(np.float64).reshape(-1)
    assert (d >= 0).all() and abs(d.mean() - 0.02 * np.sqrt(2 / np.pi)) < 0.001
    # a slice regenerated alone equals the same blocks of the full tensor
    part = torch.zeros(100 * 34, dtype=torch.uint8, device="cuda")
    assert gpu.synth_pq2_0(part, 5000, 100, 0) == 0
    assert np.array_equal(host(part), w[5000:5100].reshape(-1))
    other = torch.zeros(100 * 34, dtype=torch.uint8, device="cuda")
    assert gpu.synth_pq2_0(other, 5000, 100, 1) == 0
    assert not np.array_equal(host(other), host(part))


@pytest.mark.parametrize("offset", [1, 2, 3])
def test_float_vectors_at_odd_offsets(gpu, port, offset):
    """The reference takes any float pointer (src/kernels/elementwise_p40.cu:75-80, gemv_p40.cu:200-208,
    gemv_repack_p40.cu:209-220): a vector that starts `offset` floats into an allocation is only 4-byte aligned
    and must give the same bytes as an aligned one."""
    import torch
    n = 5120
    x = synth.activations(n, seed=31)
    sg = synth.signs(n, seed=31)
    holder = torch.zeros(n + 8, dtype=torch.float32, device="cuda")
    sholder = torch.zeros(n + 8, dtype=torch.float32, device="cuda")
    xv, sv = holder[offset:offset + n], sholder[offset:offset + n]
    xv.copy_(dev(x)); sv.copy_(dev(sg))
    assert xv.data_ptr() % 16 != 0
    # quantiser
    out = torch.zeros(n // 32 * 36, dtype=torch.uint8, device="cuda")
    assert gpu.quant_activations(xv, out, n) == 0
    assert np.array_equal(host(out), port.quantize_q8_1(x, True))
    # rotation in place, with signs
    assert gpu.fwht(xv, sv, n) == 0
    assert np.array_equal(bits(host(xv)), bits(port.fwht_blocks(x, sg)))
    assert holder[offset - 1].item() == 0.0 and holder[offset + n].item() == 0.0      # neighbours untouched
    # rotation + quantiser in one launch, rotated copy at an odd offset too
    xv.copy_(dev(x))
    rot = torch.zeros(n + 8, dtype=torch.float32, device="cuda")
    assert gpu.fwht_quant(xv, sv, out, rot[offset:offset + n], n) == 0
    want_rot = port.fwht_blocks(x, sg)
    assert np.array_equal(bits(host(rot[offset:offset + n])), bits(want_rot))
    assert np.array_equal(host(out), port.quantize_q8_1(want_rot, True))
    # repacked mat-vec takes the fp32 vector itself
    n_out = 96
    W = synth.pq2_0_weights(n_out, n, seed=32)
    Wr = torch.zeros(W.size, dtype=torch.uint8, device="cuda")
    assert gpu.repack(dev(W), Wr, n_out, n) == 0
    y = torch.zeros(n_out, device="cuda")
    y_al = torch.zeros(n_out, device="cuda")
    # default order: a 16-byte aligned vector takes the streaming kernel, another one the resident kernel -- two fixed
    # trees over the same terms; in host order both run the same kernel and agree to the bit
    assert gpu.gemv_repack(Wr, xv, y, n_out, n) == 0
    assert gpu.gemv_repack(Wr, dev(x), y_al, n_out, n) == 0
    assert_close(host(y), host(y_al))
    with host_order(gpu):
        assert gpu.gemv_repack(Wr, xv, y, n_out, n) == 0
        assert gpu.gemv_repack(Wr, dev(x), y_al, n_out, n) == 0
    assert np.array_equal(bits(host(y)), bits(host(y_al)))
    assert_close_and_exact(host(y), port.gemv_repack(port.repack(W, n_out, n), x, n_out, n))
    # a pointer that is not even float-aligned is refused
    raw = torch.zeros(4 * n + 64, dtype=torch.uint8, device="cuda")
    assert gpu.lib().bonsai_p40_fwht(raw.data_ptr() + 2, None, 1024, None) == 1
    assert gpu.lib().bonsai_p40_quant_activations(raw.data_ptr() + 2, out.data_ptr(), 1024, None) == 1


def test_rejections_and_stubs_on_device(gpu):
    import torch
    z = torch.zeros(4096, dtype=torch.float32, device="cuda")
    b = torch.zeros(8192, dtype=torch.uint8, device="cuda")
    assert gpu.gemv(b, b, z, 4, 100) == 1
    assert gpu.gemv(b, b, z, 0, 128) == 0
    assert gpu.quant_activations(z, b, 48) == 1
    assert gpu.fwht(z, None, 1000) == 1
    assert gpu.repack(b, b, 4, 128) == 1
    assert gpu.gemv_repack(b, z, z, 4, 640) == 1
    assert gpu.gemm(b, b, z, 4, 100, 2) == 1


def test_no_bounded_wait_gave_up(gpu):
    assert gpu.device_status() == 0


def test_gemm_in_a_captured_graph_after_reserve(gpu, port):
    """A caller that captures graphs reserves the mat-mul's scratch for the capturing stream first
    (bonsai_b200_gemm_reserve); the captured launch then runs, replay after replay, with the same bits as the plain
    call, and within the bound of the host loop.  Without the reservation a captured call still gives a result within
    the bound (the integer tensor-core kernel, which needs no scratch)."""
    import torch
    n_out, n_in, n_tok = 384, 2048, 96
    W = synth.pq2_0_weights(n_out, n_in, seed=21)
    X = synth.activations(n_in, seed=22, batch=n_tok)
    Xq = port.quantize_batch_chunk_major(X)
    Wd, Xqd = dev(W), dev(Xq)
    want = port.gemm(W, Xq, n_out, n_in, n_tok, threads=8)
    Y_plain = torch.zeros((n_out, n_tok), dtype=torch.float32, device="cuda")
    assert gpu.gemm(Wd, Xqd, Y_plain, n_out, n_in, n_tok) == 0
    torch.cuda.synchronize()
    assert_close(host(Y_plain), want)
    for reserve in (False, True):
        side = torch.cuda.Stream()
        Y = torch.zeros((n_out, n_tok), dtype=torch.float32, device="cuda")
        graph = torch.cuda.CUDAGraph()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            if reserve:
                assert gpu.gemm_reserve(n_in, n_tok) == 0
            with torch.cuda.graph(graph, stream=side):
                assert gpu.gemm(Wd, Xqd, Y, n_out, n_in, n_tok) == 0
        torch.cuda.current_stream().wait_stream(side)
        for _ in range(3):
            Y.fill_(777.0)
            graph.replay()
            torch.cuda.synchronize()
            assert_close(host(Y), want)
            if reserve:
                assert np.array_equal(bits(host(Y)), bits(host(Y_plain)))
    assert gpu.gemm_reserve(100, 8) == 1 and gpu.gemm_reserve(1024, 0) == 1
    del graph
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    assert gpu.gemm_release() == 0                      # the buffers go back to the device ...
    assert torch.cuda.mem_get_info()[0] > free0
    Y3 = torch.zeros((n_out, n_tok), dtype=torch.float32, device="cuda")
    assert gpu.gemm(Wd, Xqd, Y3, n_out, n_in, n_tok) == 0       # ... and the next call gets a new one
    torch.cuda.synchronize()
    assert np.array_equal(bits(host(Y3)), bits(host(Y_plain)))
    assert gpu.device_status() == 0


@pytest.mark.parametrize("tile", [64, 128])
def test_gemm_fp16_both_tile_widths(gpu, port, tile):
    """The fp16 tensor-core mat-mul is built for token tiles of 64 and of 128 (picked by token count); each forced on a
    batch the other would normally take: ragged rows and tokens, bound against the host loop."""
    import torch
    for n_out, n_in, n_tok in ((300, 2048, 100), (129, 1024, 513)):
        W = synth.pq2_0_weights(n_out, n_in, seed=tile + n_tok)
        X = synth.activations(n_in, seed=n_out, batch=n_tok)
        Xq = port.quantize_batch_chunk_major(X)
        Y = torch.full((n_out, n_tok), float("nan"), dtype=torch.float32, device="cuda")
        try:
            assert gpu.set_option("gemm_tile", tile) == 0
            assert gpu.set_option("gemm_path", 1) == 0
            assert gpu.gemm(dev(W), dev(Xq), Y, n_out, n_in, n_tok) == 0
            torch.cuda.synchronize()
        finally:
            gpu.set_option("gemm_tile", 0)
            gpu.set_option("gemm_path", -1)
        assert_close(host(Y), port.gemm(W, Xq, n_out, n_in, n_tok, threads=8))
    assert gpu.device_status() == 0
