"""GPU parity of the one-launch list of projections (bonsai_b200_chain_*): every op's output must be
the SAME BITS as the per-matrix entry points give (bonsai_p40_gemv after bonsai_b200_fwht_quant), which
in turn are held to the CPU checker; dependent ops are also checked end to end against the checker."""
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


@pytest.fixture(params=[512, 640, 768])
def threads(gpu, request):
    """Threads per CTA of the persistent kernel; the wider ones stage fewer blocks per lane, i.e. use
    shorter row segments -- the per-matrix kernel is given the same segment length so that both sum in
    the same tree."""
    assert gpu.set_option("chain_threads", request.param) == 0
    assert gpu.set_option("gemv_variant", {512: -1, 640: 100, 768: 200}[request.param]) == 0
    yield request.param
    gpu.set_option("chain_threads", 512)
    gpu.set_option("gemv_variant", -1)


SHAPES = [(5, 5120), (203, 5120), (100, 17408), (37, 1024), (6000, 5120), (2500, 17408), (1500, 6144), (700, 8192),
          (130, 2304), (5120, 5120), (1024, 5120), (4, 256)]


def test_independent_q8_ops_equal_per_matrix_calls(gpu, port, threads):
    import torch
    ops, wants = [], []
    for i, (n_out, n_in) in enumerate(SHAPES):
        W = dev(synth.pq2_0_weights(n_out, n_in, seed=100 + i))
        xq_h = port.quantize_q8_1(synth.activations(n_in, seed=i), True)
        xq = dev(xq_h)
        y_ref = torch.zeros(n_out, device="cuda")
        assert gpu.gemv(W, xq, y_ref, n_out, n_in) == 0
        wants.append(host(y_ref))
        y = torch.full((n_out,), -777.0, device="cuda")
        ops.append((W, xq, None, y, n_out, n_in, 0))
    # two more ops that reuse the last op's quantised vector
    last = ops[-1]
    for i, n_out in enumerate([77, 8]):
        W = dev(synth.pq2_0_weights(n_out, last[5], seed=900 + i))
        y_ref = torch.zeros(n_out, device="cuda")
        assert gpu.gemv(W, last[1], y_ref, n_out, last[5]) == 0
        wants.append(host(y_ref))
        ops.append((W, last[1], None, torch.full((n_out,), -777.0, device="cuda"), n_out, last[5], gpu.OP_SAME_INPUT))
    chain = gpu.Chain(ops)
    info = chain.info()
    assert info["threads"] == threads and info["nslot"] >= 3
    for _ in range(2):                      # twice: the arrival counter and every barrier start over
        for op in ops:
            op[3].fill_(-777.0)
        assert chain.run() == 0
        torch.cuda.synchronize()
        for op, want in zip(ops, wants):
            assert np.array_equal(bits(host(op[3])), bits(want)), (op[4], op[5])
    chain.close()
    assert gpu.device_status() == 0


def test_rotate_ops_and_shared_inputs(gpu, port, threads):
    """fp32 inputs rotated and quantised inside the launch; k/v-style ops reuse the previous op's vector."""
    import torch
    n_in = 5120
    x = synth.activations(n_in, seed=3)
    sg = synth.signs(n_in, seed=4)
    xd, sd = dev(x), dev(sg)
    xq_want = port.quantize_q8_1(port.fwht_blocks(x, sg), True)
    x2 = synth.activations(17408, seed=5)
    x2d = dev(x2)
    xq2_want = port.quantize_q8_1(port.fwht_blocks(x2, None), True)
    ops, wants = [], []
    for i, n_out in enumerate([1000, 1024, 36, 7]):
        Wh = synth.pq2_0_weights(n_out, n_in, seed=200 + i)
        y = torch.zeros(n_out, device="cuda")
        ops.append((dev(Wh), xd, sd, y, n_out, n_in, gpu.OP_ROTATE | (gpu.OP_SAME_INPUT if i else 0)))
        wants.append(port.gemv(Wh, xq_want, n_out, n_in, threads=4))
    for i, n_out in enumerate([300, 5]):
        Wh = synth.pq2_0_weights(n_out, 17408, seed=300 + i)
        y = torch.zeros(n_out, device="cuda")
        ops.append((dev(Wh), x2d, None, y, n_out, 17408, gpu.OP_ROTATE | (gpu.OP_SAME_INPUT if i else 0)))
        wants.append(port.gemv(Wh, xq2_want, n_out, 17408, threads=4))
    chain = gpu.Chain(ops)
    assert chain.run() == 0
    torch.cuda.synchronize()
    scratch = torch.zeros(17408 // 32 * 36, dtype=torch.uint8, device="cuda")
    for op, want in zip(ops, wants):
        W, x_, s_, y, n_out, n_in_, _ = op
        got = host(y)
        scale = float(np.abs(want).max()) or 1.0
        assert float(np.abs(got.astype(np.float64) - want).max()) <= REL_TOL * scale
        y2 = torch.zeros(n_out, device="cuda")
        assert gpu.linear(W, x_, s_, y2, scratch, n_out, n_in_) == 0
        assert np.array_equal(bits(got), bits(host(y2)))
    chain.close()
    assert gpu.device_status() == 0


def test_dependent_ops_flow_through_the_launch(gpu, port, threads):
    """y of one op is the x of the next (which waits for every row of it), five ops deep, twice."""
    import torch
    widths = [5120, 6144, 1024, 17408, 5120, 2048]       # op i: widths[i] -> widths[i + 1]
    x0 = synth.activations(widths[0], seed=11)
    bufs = [dev(x0)] + [torch.zeros(w, device="cuda") for w in widths[1:]]
    Ws = [synth.pq2_0_weights(widths[i + 1], widths[i], seed=400 + i) for i in range(5)]
    # the second consumer of bufs[1] shares its input with op 1
    W_side = synth.pq2_0_weights(333, widths[1], seed=499)
    y_side = torch.zeros(333, device="cuda")
    ops = []
    for i in range(5):
        ops.append((dev(Ws[i]), bufs[i], None, bufs[i + 1], widths[i + 1], widths[i],
                    gpu.OP_ROTATE | (gpu.OP_DEPENDS if i else 0)))
        if i == 1:
            ops.append((dev(W_side), bufs[1], None, y_side, 333, widths[1], gpu.OP_ROTATE | gpu.OP_SAME_INPUT))
    chain = gpu.Chain(ops)
    # the same flow through the per-matrix entry points
    ref = [dev(x0)] + [torch.zeros(w, device="cuda") for w in widths[1:]]
    scratch = torch.zeros(17408 // 32 * 36, dtype=torch.uint8, device="cuda")
    for i in range(5):
        assert gpu.linear(dev(Ws[i]), ref[i], None, ref[i + 1], scratch, widths[i + 1], widths[i]) == 0
    side_ref = torch.zeros(333, device="cuda")
    assert gpu.linear(dev(W_side), ref[1], None, side_ref, scratch, 333, widths[1]) == 0
    for _ in range(2):
        for b in bufs[1:]:
            b.zero_()
        y_side.zero_()
        assert chain.run() == 0
        torch.cuda.synchronize()
        for i in range(1, 6):
            assert np.array_equal(bits(host(bufs[i])), bits(host(ref[i]))), i
        assert np.array_equal(bits(host(y_side)), bits(host(side_ref)))
    # and the first hop against the checker
    want = port.gemv(Ws[0], port.quantize_q8_1(port.fwht_blocks(x0, None), True), widths[1], widths[0], threads=4)
    got = host(bufs[1])
    assert float(np.abs(got.astype(np.float64) - want).max()) <= REL_TOL * float(np.abs(want).max())
    chain.close()
    assert gpu.device_status() == 0


def test_long_mixed_list_in_a_graph(gpu, port):
    """60 ops (more than the record ring and many laps of the tile ring), replayed from a CUDA graph."""
    import torch
    rng = np.random.default_rng(7)
    shapes = [(int(rng.integers(1, 900)), int(rng.choice([256, 1024, 2048, 5120, 6144]))) for _ in range(60)]
    ops, wants = [], []
    scratch = torch.zeros(6144 // 32 * 36, dtype=torch.uint8, device="cuda")
    for i, (n_out, n_in) in enumerate(shapes):
        W = dev(synth.pq2_0_weights(n_out, n_in, seed=500 + i))
        y = torch.zeros(n_out, device="cuda")
        y_ref = torch.zeros(n_out, device="cuda")
        if i % 3 == 0 and n_in % 1024 == 0:
            x = dev(synth.activations(n_in, seed=i))
            assert gpu.linear(W, x, None, y_ref, scratch, n_out, n_in) == 0
            ops.append((W, x, None, y, n_out, n_in, gpu.OP_ROTATE))
        else:
            xq = dev(port.quantize_q8_1(synth.activations(n_in, seed=i), True))
            assert gpu.gemv(W, xq, y_ref, n_out, n_in) == 0
            ops.append((W, xq, None, y, n_out, n_in, 0))
        wants.append(host(y_ref))
    chain = gpu.Chain(ops)
    assert chain.run() == 0                 # warm-up outside the capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            assert chain.run() == 0
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(3):
        for op in ops:
            op[3].zero_()
        graph.replay()
        torch.cuda.synchronize()
        for op, want in zip(ops, wants):
            assert np.array_equal(bits(host(op[3])), bits(want))
    chain.close()
    assert gpu.device_status() == 0


def test_chain_rejections(gpu):
    import torch
    W = torch.zeros(8 * 2 * 34, dtype=torch.uint8, device="cuda")
    x = torch.zeros(1024, device="cuda")
    y = torch.zeros(8, device="cuda")
    ok = (W, x, None, y, 8, 256, 0)
    gpu.Chain([ok]).close()
    for bad in [(W, x, None, y, 8, 128, 0),                       # odd block count
                (W, x, None, y, 8, 256, gpu.OP_ROTATE),           # rotation needs whole 1024-blocks
                (W, x, None, y, 8, 256, gpu.OP_DEPENDS),          # a dependent op must quantise fp32
                (W, x, None, y, 8, 256, gpu.OP_SAME_INPUT),       # nothing before it
                (W, x, None, y, 0, 256, 0),
                (W, x, None, y, 8, 256, 64)]:
        with pytest.raises(RuntimeError):
            gpu.Chain([bad])
    with pytest.raises(RuntimeError):
        gpu.Chain([ok, (W, y, None, y, 8, 256, gpu.OP_SAME_INPUT)])   # not the same input


@pytest.mark.parametrize("seg,variant", [(24, 200), (16, 300), (8, 400)])
def test_shorter_segments_match_the_per_matrix_tiling(gpu, port, seg, variant):
    """chain_seg changes the summation tree exactly as the per-matrix kernel's segment option does."""
    import torch
    ops, wants = [], []
    try:
        assert gpu.set_option("chain_seg", seg) == 0
        assert gpu.set_option("gemv_variant", variant) == 0
        for i, (n_out, n_in) in enumerate([(203, 5120), (100, 17408), (130, 2304), (64, 6144)]):
            W = dev(synth.pq2_0_weights(n_out, n_in, seed=600 + i))
            xq = dev(port.quantize_q8_1(synth.activations(n_in, seed=i), True))
            y_ref = torch.zeros(n_out, device="cuda")
            assert gpu.gemv(W, xq, y_ref, n_out, n_in) == 0
            wants.append(host(y_ref))
            ops.append((W, xq, None, torch.zeros(n_out, device="cuda"), n_out, n_in, 0))
        chain = gpu.Chain(ops)
        assert chain.run() == 0
        torch.cuda.synchronize()
        for op, want in zip(ops, wants):
            assert np.array_equal(bits(host(op[3])), bits(want))
        chain.close()
    finally:
        gpu.set_option("chain_seg", 40)
        gpu.set_option("gemv_variant", -1)
    assert gpu.device_status() == 0


@pytest.mark.parametrize("seed", [1, 2])
def test_random_lists_with_dependencies(gpu, port, threads, seed):
    """Random lists: Q8_1 and fp32 inputs, shared inputs, ops that read earlier ops' outputs (of any
    width, so wide inputs take the rotate-once-for-the-grid path too).  Dependencies only point
    backwards, so the same ops issued one by one through the per-matrix entry points are the answer."""
    import torch
    rng = np.random.default_rng(seed)
    widths = [1024, 2048, 5120, 6144, 9216, 17408]
    ext = {w: dev(synth.activations(w, seed=seed * 100 + w)) for w in widths}          # vectors from outside the list
    ext_q = {w: dev(port.quantize_q8_1(synth.activations(w, seed=seed * 100 + w + 1), True)) for w in widths}
    produced = {}                                   # width -> (chain buffer, reference buffer) written by an earlier op
    scratch = torch.zeros(max(widths) // 32 * 36, dtype=torch.uint8, device="cuda")
    ops, refs = [], []
    prev = None
    for i in range(40):
        if prev is not None and rng.random() < 0.2:
            kind, n_in, x, x_ref = prev                                  # same input as the op before
            flags = (gpu.OP_ROTATE if kind != "q8" else 0) | gpu.OP_SAME_INPUT
        else:
            n_in = int(rng.choice(list(produced) if produced and rng.random() < 0.5 else [1024, 1024, 2048, 2048, 5120, 6144]))
            if n_in in produced and rng.random() < 0.7:
                kind, (x, x_ref), flags = "dep", produced[n_in], gpu.OP_ROTATE | gpu.OP_DEPENDS
            elif rng.random() < 0.5:
                kind, x, x_ref, flags = "q8", ext_q[n_in], ext_q[n_in], 0
            else:
                kind, x, x_ref, flags = "rot", ext[n_in], ext[n_in], gpu.OP_ROTATE
        if n_in <= 2048 and rng.random() < 0.5:
            n_out = int(rng.choice([9216, 17408]))                       # wide outputs only from narrow inputs: small matrices
        elif rng.random() < 0.5:
            n_out = int(rng.choice([1024, 2048, 5120, 6144]))
        else:
            n_out = int(rng.integers(1, 700))
        W = dev(synth.pq2_0_weights(n_out, n_in, seed=seed * 1000 + i))
        y, y_ref = torch.zeros(n_out, device="cuda"), torch.zeros(n_out, device="cuda")
        if kind == "q8":
            assert gpu.gemv(W, x_ref, y_ref, n_out, n_in) == 0
        else:
            assert gpu.linear(W, x_ref, None, y_ref, scratch, n_out, n_in) == 0
        ops.append((W, x, None, y, n_out, n_in, flags))
        refs.append(y_ref)
        if n_out in widths:
            produced[n_out] = (y, y_ref)
        prev = (kind, n_in, x, x_ref)
    chain = gpu.Chain(ops)
    for _ in range(2):
        for op in ops:
            op[3].fill_(-3.0)
        assert chain.run() == 0
        torch.cuda.synchronize()
        for i, (op, want) in enumerate(zip(ops, refs)):
            assert np.array_equal(bits(host(op[3])), bits(host(want))), (i, op[4], op[5], op[6])
    chain.close()
    assert gpu.device_status() == 0


def _one_op_chain_tp(gpu, y_ptr, bases, rank, world, total, offset, limit=0, n_out=8):
    import ctypes as C
    import torch
    W = torch.zeros(n_out * 2 * 34, dtype=torch.uint8, device="cuda")
    x = torch.zeros(1024, device="cuda")
    op = (gpu.Op * 1)()
    op[0].W, op[0].x, op[0].signs, op[0].y = W.data_ptr(), x.data_ptr(), None, y_ptr
    op[0].n_out, op[0].n_in, op[0].flags, op[0].reserved = n_out, 256, 0, 0
    arr = (C.c_void_p * len(bases))(*bases)
    h = C.c_void_p()
    rc = gpu.lib().bonsai_b200_chain_create_tp(C.cast(op, C.c_void_p), 1, rank, world, C.cast(arr, C.c_void_p), total,
                                              offset, limit, C.byref(h))
    if rc == 0:
        assert gpu.lib().bonsai_b200_chain_destroy(h) == 0
    return rc


def test_several_rank_form_checks_its_arguments(gpu):
    """bonsai_b200_chain_create_tp on one device: creation only (nothing is launched, so the second
    'rank' can be the same buffer).  Refused: bad rank counts, ranks and counter offsets; a counter block
    that does not fit in the buffer; a mapping that is not 16-byte aligned; an output that does not lie
    inside the peer-mapped buffer in front of the counters (the kernel stores it into every other GPU at
    the same offset, so it would leave the mapping there)."""
    import torch
    buf = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    other = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    base = buf.data_ptr()

    def create(rank, world, offset, y=base, total=2048 + 64, bases=(base, base), n_out=8):
        return _one_op_chain_tp(gpu, y, list(bases), rank, world, total, offset, n_out=n_out)
    assert create(0, 2, 2048) == 0
    assert create(1, 2, 2048) == 0
    assert create(0, 2, 2048, y=base + 2048 - 32) == 0      # the last 8 floats in front of the counters
    assert create(0, 1, 2048) == 1          # one rank: use bonsai_b200_chain_create
    assert create(2, 2, 2048) == 1          # rank out of range
    assert create(0, 9, 2048) == 1          # more ranks than the kernel addresses
    assert create(0, 2, 2050) == 1          # counters must sit on a 64-byte boundary
    assert create(0, 2, -64) == 1
    assert create(0, 2, 2048, total=2048 + 63) == 1                      # counter block runs past the buffer
    assert create(0, 2, 2048, y=base + 2048 - 28) == 1                   # output overlaps the counters
    assert create(0, 2, 2048, y=base + 2048) == 1                        # output behind the buffer's payload
    assert create(0, 2, 2048, y=other.data_ptr()) == 1                   # output in another allocation
    assert create(0, 2, 2048, y=base, n_out=520) == 1                    # 2080 bytes do not fit in 2048
    assert create(0, 2, 2048, bases=(base, base + 8)) == 1               # unaligned mapping of a peer
    assert create(1, 2, 2048, y=base + 8 + 64, bases=(base, base + 8)) == 1


def test_a_rank_that_never_comes_makes_the_wait_run_out(gpu, port):
    """Failure detection without a fault: a two-rank list whose second 'rank' is a second buffer on the same GPU that
    no kernel ever signals.  The launch must end by itself within the wait limit (3 ms), the status word must
    say that a wait for other ranks ran out, clearing must work, and a normal list must pass parity afterwards."""
    import time
    import torch
    n_in, n_out = 1024, 64
    W = synth.pq2_0_weights(n_out, n_in, seed=5)
    x = synth.activations(n_in, seed=5)
    Wd, xd = dev(W), dev(x)
    payload = 4096

    class TwoBuffers:            # what bonsai_b200.peer.PeerBuffer provides, without a second process
        rank, world, counter_offset, total_bytes = 0, 2, payload, payload + 64

    mine = torch.zeros(payload + 64, dtype=torch.uint8, device="cuda")
    nobody = torch.zeros(payload + 64, dtype=torch.uint8, device="cuda")
    TwoBuffers.ptrs = [mine.data_ptr(), nobody.data_ptr()]
    y = mine[:n_out * 4].view(torch.float32)
    assert gpu.device_status() == 0
    chain = gpu.Chain([(Wd, xd, None, y, n_out, n_in, gpu.OP_ROTATE)], peers=TwoBuffers, wait_limit_us=3000)
    t0 = time.perf_counter()
    assert chain.run() == 0
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 5.0
    assert gpu.device_status() == 2                      # STATUS_GRID_TIMEOUT: the wait for the other rank ran out
    # the rows were computed and also stored into the other buffer before the wait
    scratch = torch.zeros(n_in // 32 * 36, dtype=torch.uint8, device="cuda")
    ref = torch.zeros(n_out, device="cuda")
    assert gpu.linear(Wd, xd, None, ref, scratch, n_out, n_in) == 0
    torch.cuda.synchronize()
    assert torch.equal(y, ref) and torch.equal(nobody[:n_out * 4].view(torch.float32), ref)
    chain.close()
    assert gpu.clear_status() == 0
    assert gpu.device_status() == 0
    # the context is intact: a one-rank list gives the per-matrix bits
    y2 = torch.zeros(n_out, device="cuda")
    chain = gpu.Chain([(Wd, xd, None, y2, n_out, n_in, gpu.OP_ROTATE)])
    assert chain.run() == 0
    torch.cuda.synchronize()
    assert torch.equal(y2, ref)
    want = port.gemv(W, port.quantize_q8_1(port.fwht_blocks(x), True), n_out, n_in)
    assert float(np.abs(host(y2).astype(np.float64) - want).max()) <= REL_TOL * float(np.abs(want).max())
    chain.close()
    assert gpu.device_status() == 0
