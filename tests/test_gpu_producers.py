"""The producers fused into the list kernel's prologue (RMSNorm / SwiGLU -> signs -> FWHT -> Q8_1, and the exact
power-of-two glue of the synthetic decode step), and the decode step itself with values flowing from op to op.

Bars.  Fused against unfused on the GPU (bonsai_p40_rmsnorm / bonsai_b200_swiglu, then the same op without the flag):
every output bit for bit -- the fused prologue performs the same operations in the same order, so the Q8_1 blocks it
builds in shared memory are the bytes the two-step form writes to memory.  Against the CPU checker: the fp32
intermediate within 1e-5 (tests/test_gpu_ops.py), and for the rescale glue, whose arithmetic is exact, the whole op:
Q8_1 bytes exact, int32 chunk sums exact, y within 1e-5 of max |y|, the checker being fed the GPU's own previous output.
"""
import numpy as np
import pytest

from bonsai_b200 import synth

pytestmark = pytest.mark.gpu

REL_TOL = 1e-5


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.detach().cpu().numpy()


def glue(y_prev, n_in):
    """x[j] = y_prev[j mod len] * 2^-e, e = floor(log2(max |y_prev|)); unscaled when the maximum is zero or subnormal."""
    m = float(np.abs(y_prev).max())
    scale = np.float32(1.0)
    if m >= np.finfo(np.float32).tiny:
        _, ex = np.frexp(np.float32(m))          # m = mant * 2^ex, mant in [0.5, 1)
        scale = np.ldexp(np.float32(1.0), -(int(ex) - 1)).astype(np.float32)
    idx = np.arange(n_in) % y_prev.size
    return (y_prev[idx] * scale).astype(np.float32)


def test_rmsnorm_producer_equals_the_two_step_form(gpu, port):
    import torch
    n_in, n_mid, n_out = 5120, 5120, 700
    W0 = synth.pq2_0_weights(n_mid, n_in, seed=61)
    W1 = synth.pq2_0_weights(n_out, n_mid, seed=62)
    x = synth.activations(n_in, seed=61)
    sg = synth.signs(n_mid, seed=61)
    w = (np.random.default_rng(61).uniform(0.5, 1.5, size=n_mid)).astype(np.float32)
    W0d, W1d, xd, sgd, wd = dev(W0), dev(W1), dev(x), dev(sg), dev(w)
    eps = 1e-6
    # fused: op 0 normalises the external vector, op 1 the output of op 0 (a wait in between)
    y0 = torch.zeros(n_mid, device="cuda")
    y1 = torch.zeros(n_out, device="cuda")
    chain = gpu.Chain([(W0d, xd, None, y0, n_mid, n_in, gpu.OP_ROTATE | gpu.OP_RMSNORM, wd, eps),
                       (W1d, y0, sgd, y1, n_out, n_mid, gpu.OP_ROTATE | gpu.OP_DEPENDS | gpu.OP_RMSNORM, wd, eps)])
    assert chain.run() == 0
    torch.cuda.synchronize()
    # two-step form
    scratch = torch.zeros(n_in // 32 * 36, dtype=torch.uint8, device="cuda")
    xn = torch.zeros(n_in, device="cuda")
    r0 = torch.zeros(n_mid, device="cuda")
    r1 = torch.zeros(n_out, device="cuda")
    assert gpu.rmsnorm(xd, wd, xn, 1, n_in, eps) == 0
    assert gpu.linear(W0d, xn, None, r0, scratch, n_mid, n_in) == 0
    assert gpu.rmsnorm(r0, wd, xn, 1, n_mid, eps) == 0
    assert gpu.linear(W1d, xn, sgd, r1, scratch, n_out, n_mid) == 0
    torch.cuda.synchronize()
    assert np.array_equal(bits(host(y0)), bits(host(r0)))
    assert np.array_equal(bits(host(y1)), bits(host(r1)))
    # and the normalised vector itself against the checker
    want = port.rmsnorm(host(r0), w, eps)
    got = host(xn)
    assert float(np.abs(got - want).max()) <= REL_TOL * float(np.abs(want).max())
    chain.close()
    assert gpu.device_status() == 0


def test_swiglu_producer_equals_the_two_step_form(gpu, port):
    """gate and up projections share an input; the down projection reads silu(gate) * up.  17408 floats: the wide-input
    path, where CTA b rotates block b for the whole grid."""
    import torch
    n_in, n_ff, n_out = 5120, 17408, 640
    Wg = synth.pq2_0_weights(n_ff, n_in, seed=71)
    Wu = synth.pq2_0_weights(n_ff, n_in, seed=72)
    Wd_ = synth.pq2_0_weights(n_out, n_ff, seed=73)
    x = synth.activations(n_in, seed=71)
    Wgd, Wud, Wdd, xd = dev(Wg), dev(Wu), dev(Wd_), dev(x)
    g = torch.zeros(n_ff, device="cuda")
    u = torch.zeros(n_ff, device="cuda")
    y = torch.zeros(n_out, device="cuda")
    chain = gpu.Chain([(Wgd, xd, None, g, n_ff, n_in, gpu.OP_ROTATE),
                       (Wud, xd, None, u, n_ff, n_in, gpu.OP_ROTATE | gpu.OP_SAME_INPUT),
                       (Wdd, g, None, y, n_out, n_ff, gpu.OP_ROTATE | gpu.OP_DEPENDS | gpu.OP_SWIGLU, u)])
    for _ in range(2):
        assert chain.run() == 0
    torch.cuda.synchronize()
    scratch = torch.zeros(n_ff // 32 * 36, dtype=torch.uint8, device="cuda")
    act = torch.zeros(n_ff, device="cuda")
    r = torch.zeros(n_out, device="cuda")
    assert gpu.swiglu(g, u, act, n_ff) == 0
    assert gpu.linear(Wdd, act, None, r, scratch, n_out, n_ff) == 0
    torch.cuda.synchronize()
    assert np.array_equal(bits(host(y)), bits(host(r)))
    want = port.swiglu(host(g), host(u))
    assert float(np.abs(host(act) - want).max()) <= REL_TOL * float(np.abs(want).max())
    chain.close()
    assert gpu.device_status() == 0


def test_rescale_glue_lets_values_flow(gpu, port):
    """A short dependent list with the glue between the ops, one shared input and a wrap (1024 -> 6144)."""
    import torch
    shapes = [(5120, 6144), (6144, 17408), (17408, 5120), (5120, 1024), (5120, 2048), (6144, 300)]
    same = {4: True}                 # op 4 shares op 3's input
    Ws = [synth.pq2_0_weights(n_out, n_in, seed=80 + i) for i, (n_in, n_out) in enumerate(shapes)]
    Wd = [dev(W) for W in Ws]
    x0 = synth.activations(5120, seed=80)
    ys = [torch.zeros(n_out, device="cuda") for _, n_out in shapes]
    ops = []
    src = {1: 0, 2: 1, 3: 2, 4: 2, 5: 3}
    for i, (n_in, n_out) in enumerate(shapes):
        if i == 0:
            ops.append((Wd[i], dev(x0), None, ys[i], n_out, n_in, gpu.OP_ROTATE))
        else:
            p = src[i]
            fl = gpu.OP_ROTATE | gpu.OP_RESCALE | (gpu.OP_SAME_INPUT if same.get(i) else gpu.OP_DEPENDS)
            ops.append((Wd[i], ys[p], None, ys[i], n_out, n_in, fl, None, 0.0, shapes[p][1]))
    chain = gpu.Chain(ops)
    for _ in range(2):                # the recorded maxima are reset by every run
        assert chain.run() == 0
    torch.cuda.synchronize()
    # per op against the per-matrix entry point on the glue'd vector (bits) and against the checker
    worst = 0.0
    for i, (n_in, n_out) in enumerate(shapes):
        x_i = x0 if i == 0 else glue(host(ys[src[i]]), n_in)
        scratch = torch.zeros(n_in // 32 * 36, dtype=torch.uint8, device="cuda")
        r = torch.zeros(n_out, device="cuda")
        assert gpu.linear(Wd[i], dev(x_i), None, r, scratch, n_out, n_in) == 0
        torch.cuda.synchronize()
        assert np.array_equal(bits(host(ys[i])), bits(host(r))), i
        want_xq = port.quantize_q8_1(port.fwht_blocks(x_i), True)
        assert np.array_equal(host(scratch), want_xq), i
        want = port.gemv(Ws[i], want_xq, n_out, n_in, threads=4)
        worst = max(worst, float(np.abs(host(ys[i]).astype(np.float64) - want).max()) / float(np.abs(want).max()))
    assert worst <= REL_TOL, worst
    chain.close()
    assert gpu.device_status() == 0


def test_producer_rejections(gpu):
    import ctypes as C
    import torch
    W = torch.zeros(8 * 8 * 34, dtype=torch.uint8, device="cuda")
    x = torch.zeros(1024, device="cuda")
    y = torch.zeros(8, device="cuda")
    aux = torch.zeros(1024, device="cuda")

    def create(flags, aux_t=None, eps=0.0, src_len=0, n_in=1024, xt=None):
        op = (gpu.Op * 1)()
        op[0].W, op[0].x, op[0].signs, op[0].y = W.data_ptr(), (xt if xt is not None else x).data_ptr(), None, y.data_ptr()
        op[0].n_out, op[0].n_in, op[0].flags, op[0].reserved = 8, n_in, flags, 0
        op[0].aux = aux_t.data_ptr() if aux_t is not None else None
        op[0].eps, op[0].src_len = eps, src_len
        h = C.c_void_p()
        rc = gpu.lib().bonsai_b200_chain_create(C.cast(op, C.c_void_p), 1, C.byref(h))
        if rc == 0:
            assert gpu.lib().bonsai_b200_chain_destroy(h) == 0
        return rc
    assert create(gpu.OP_ROTATE | gpu.OP_RMSNORM, aux, 1e-6) == 0
    assert create(gpu.OP_ROTATE | gpu.OP_SWIGLU, aux) == 0
    assert create(gpu.OP_RMSNORM, aux, 1e-6) == 1                                 # producers need OP_ROTATE
    assert create(gpu.OP_ROTATE | gpu.OP_RMSNORM) == 1                            # no weights
    assert create(gpu.OP_ROTATE | gpu.OP_RMSNORM | gpu.OP_SWIGLU, aux, 1e-6) == 1  # one producer per op
    assert create(gpu.OP_ROTATE, aux) == 1                                        # aux without a producer
    assert create(gpu.OP_ROTATE, None, 1e-6) == 1                                 # eps without RMSNorm
    assert create(gpu.OP_ROTATE | gpu.OP_RESCALE, None, 0.0, 1024) == 1           # x is no earlier op's output
    assert create(gpu.OP_ROTATE, None, 0.0, 1024) == 1                            # src_len without the flag
    assert create(64 | gpu.OP_ROTATE) == 1                                        # unknown flag


def test_decode_step_values_flow(gpu, port):
    """The 401 projections of one decoded token (6.8 GB of synthetic weights) as ONE list launch with the exact glue
    between them; every op is then checked on its own with the checker fed the GPU's own previous output: Q8_1 bytes,
    int32 chunk sums of sampled rows, y of those rows within 1e-5 of max |y|."""
    import torch
    import bench
    shapes = bench.model_gemvs()
    assert len(shapes) == 401 and sum(bench.weight_bytes(a, b) for a, b in shapes) == 6799564800
    free, _ = torch.cuda.mem_get_info()
    if free < 12 << 30:
        pytest.skip("needs 12 GB of free device memory")
    ops, ys, Ws = bench.decode_ops(torch, gpu, shapes, seed=0, flow=True)
    chain = gpu.Chain(ops)
    assert chain.run() == 0
    torch.cuda.synchronize()
    assert gpu.device_status() == 0
    x0 = host(ops[0][1])
    row_bytes = lambda i: shapes[i][0] // 128 * 34
    W_rows_of = lambda i, r: host(Ws[i][r * row_bytes(i):(r + 1) * row_bytes(i)])
    same = {i: bool(ops[i][6] & gpu.OP_SAME_INPUT) for i in range(len(ops))}
    worst = 0.0
    x_cur = None
    for i, (n_in, n_out) in enumerate(shapes):
        if i == 0:
            x_cur = x0
        elif not same[i]:
            x_cur = glue(host(ys[i - 1]), n_in)
        want_xq = port.quantize_q8_1(port.fwht_blocks(x_cur), True)
        xq = torch.zeros(n_in // 32 * 36, dtype=torch.uint8, device="cuda")
        assert gpu.fwht_quant(dev(x_cur), None, xq, None, n_in) == 0
        assert np.array_equal(host(xq), want_xq), i
        got_y = host(ys[i])
        assert np.isfinite(got_y).all() and float(np.abs(got_y).max()) > 0.0, i
        scale = float(np.abs(got_y).max())
        sums = torch.zeros(1, n_in // 32, dtype=torch.int32, device="cuda")
        for r in sorted({0, n_out // 2, n_out - 1}):
            wrow = W_rows_of(i, r)
            want = port.gemv(wrow, want_xq, 1, n_in)[0]
            worst = max(worst, abs(float(got_y[r]) - float(want)) / scale)
            assert gpu.gemv_chunk_sums(Ws[i], xq, sums, r, 1, n_in) == 0
            assert np.array_equal(host(sums)[0], port.row_chunk_sums(wrow, want_xq, n_in)), (i, r)
    assert worst <= REL_TOL, worst
    chain.close()
