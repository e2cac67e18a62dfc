#!/usr/bin/env python
"""Benchmark of the PQ2_0 decode mat-vec on B200, one JSON line per run.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--sets S]

Workload ("layer_sweep"): the batch-1 projection shapes of one transformer layer,
n_in x n_out = 5120x5120, 5120x1024, 5120x17408, 17408x5120, PQ2_0 weights with the checkpoint's
code distribution, Q8_1 activations from FWHT-rotated N(0,1) vectors.  `--sets S` independent copies
of the four matrices are resident in HBM (S = 8 -> 446 MB, larger than the 126 MB L2) and one sweep is
one pass over all of them, so every launch streams its weights from HBM.  A step is `sweeps_per_step`
sweeps (chosen so that the timed region lasts at least 50 ms; 1 when --steps is large enough).

value   : PQ2_0 weight bytes of all launches / device time (CUDA events, max over ranks), GB/s.
--call  : "list" (default) hands a sweep's mat-vecs to bonsai_b200_chain_run, ONE persistent launch that
          streams the matrices back to back; "matrix" calls bonsai_p40_gemv once per matrix (the
          reference's ABI unchanged).  In list mode the per-matrix figure is measured too and
          reported under "per_matrix_abi".
e2e     : the same metric with HOST buffers: the sweep's fp32 activation vectors are copied from
          pinned host memory (one block), rotated + quantised (one call) + multiplied through the C
          ABI, and the outputs are copied back, all inside the timed region.  Weights stay resident
          (they are model state).  Same data plane between ranks as `value`.
roofline: algorithmic bytes (weights + Q8_1 vectors + fp32 outputs) of a launch / its duration, against the
          measured HBM copy bandwidth, the nominal 8 TB/s and a read-only streaming probe run here.
parity  : after the timed loop every output vector of the last sweep (on every rank: the gathered
          vector) is compared bit for bit with bonsai_p40_gemv on the UNSPLIT matrix.
N > 1   : every matrix is split by output rows over the ranks (strong scaling: the total work is fixed); the
          slices are assembled either by one NCCL all-gather per sweep or by the kernel itself (stores into
          every rank's peer-mapped buffer); --gather auto times both here and keeps the faster.
secondary: row-partitioned batch of 8 (every N); on one GPU also the decode step (401 mat-vecs of one token, values
          flowing), the prefill mat-mul (512 tokens) and the repacked-layout mat-vec; each with its own parity check.
--impl reference : the reference's own host implementation of the same path on this box's CPU
          cores (oracle/_ref when it was built, else the C restatement in oracle/).
"""
import argparse
import json
import math
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "p40-kernel_b200"))

LAYER_SHAPES = [(5120, 5120), (5120, 1024), (5120, 17408), (17408, 5120)]   # (n_in, n_out)
METRIC = "pq2_0_gemv_weight_stream"
UNIT = "GB/s"
DTYPE = "int8xint2->int32, fp32 scale"
NOMINAL_HBM_GBS = 8000.0
MIN_TIMED_MS = 50.0


def weight_bytes(n_in, n_out):
    return n_out * (n_in // 128) * 34


def algorithmic_bytes(n_in, n_out, batch=1):
    return weight_bytes(n_in, n_out) + batch * ((n_in // 32) * 36 + 4 * n_out)


def measured_peaks():
    try:
        d = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


def env_ranks():
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")),
            int(os.environ.get("LOCAL_RANK", "0")))


# ---------------------------------------------------------------------------------------------------
class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.stop_flag, self.sm, self.reasons, self.max_sm = index, threading.Event(), [], set(), None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_sm = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def sample(self):
        nv = self.nv
        self.sm.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
        r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
        names = {"hw_slowdown": nv.nvmlClocksThrottleReasonHwSlowdown,
                 "hw_thermal_slowdown": nv.nvmlClocksThrottleReasonHwThermalSlowdown,
                 "sw_thermal_slowdown": nv.nvmlClocksThrottleReasonSwThermalSlowdown,
                 "sw_power_cap": nv.nvmlClocksThrottleReasonSwPowerCap}
        for k, bit in names.items():
            if r & bit:
                self.reasons.add(k)

    def run(self):
        if self.nv is None:
            return
        while not self.stop_flag.is_set():
            try:
                self.sample()
            except Exception:
                return
            time.sleep(0.003)

    def result(self):
        self.stop_flag.set()
        self.join(timeout=2)
        if not self.sm:
            return {"sm_mhz": None, "sm_max_mhz": self.max_sm, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(self.sm), "sm_max_mhz": self.max_sm, "reasons": sorted(self.reasons),
                "samples": len(self.sm)}


# ---- timing on the device ---------------------------------------------------------------------------
def graph_of(torch, fn):
    """Runs fn once eagerly on the capture stream (validates it, warms caches, lets the library allocate the scratch
    it keeps per stream: nothing may be allocated during capture), then captures it; returns the replay function."""
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=side):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    return graph.replay


def device_ms(torch, run, n, dist=None):
    """Device time of n calls of run(), max over ranks.  One untimed call goes first and the start event is
    recorded on the stream right behind it, with no host synchronisation in between: the ranks of a
    several-GPU step meet on the device in that call (its collective or its closing rendezvous), so the skew
    of the host-side barrier is outside the measurement."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    run()
    e0.record()
    for _ in range(n):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if dist is not None:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def timed(torch, fn, steps, warmup, dist=None, sampler_index=None, use_graph=True):
    """Times `steps` steps of fn; a step is `reps` calls, reps chosen so that the region lasts >= 50 ms.
    Returns (ms, reps, clocks)."""
    run = graph_of(torch, fn) if use_graph else fn
    for _ in range(max(0, warmup)):
        run()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
    est = device_ms(torch, run, 3, dist) / 3.0
    reps = max(1, int(math.ceil(MIN_TIMED_MS / max(1e-6, steps * est))))
    sampler = ClockSampler(sampler_index) if sampler_index is not None else None
    if sampler:
        sampler.start()
    ms = device_ms(torch, run, steps * reps, dist)
    clocks = sampler.result() if sampler else None
    return ms, reps, clocks


# ---------------------------------------------------------------------------------------------------
def cpu_arm(threads):
    """The CPU checker on one layer sweep (FWHT + quantise + mat-vec per shape)."""
    from oracle.oracle import Oracle, reference_available
    from bonsai_b200 import synth
    kind = "reference" if reference_available() else "port"
    orc = Oracle(kind)
    mats = [(n_in, n_out, synth.pq2_0_weights(n_out, n_in, seed=i)) for i, (n_in, n_out) in enumerate(LAYER_SHAPES)]
    xs = {n_in: synth.activations(n_in, seed=0) for n_in, _ in LAYER_SHAPES}

    def sweep():
        for n_in, n_out, W in mats:
            xq = orc.quantize_q8_1(orc.fwht_blocks(xs[n_in]), True)
            orc.gemv(W, xq, n_out, n_in, threads=threads)

    return kind, sweep, sum(weight_bytes(a, b) for a, b in LAYER_SHAPES)


def run_reference(args):
    rank, _, _ = env_ranks()
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    kind, sweep, wbytes = cpu_arm(threads)
    warm = max(1, min(args.warmup, 20))
    for _ in range(warm):
        sweep()
    steps = max(1, min(args.steps, 50))
    t0 = time.perf_counter()
    for _ in range(steps):
        sweep()
    dt = time.perf_counter() - t0
    val = wbytes * steps / dt / 1e9
    sample = f"one layer sweep (4 mat-vecs, {wbytes} weight bytes) per step, FWHT+Q8_1 on the CPU included"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warm, "ms_per_step": dt / steps * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": DTYPE,
        "data": "synthetic", "config": {"workload": "layer_sweep", "shapes_nin_nout": LAYER_SHAPES, "batch": 1},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ---------------------------------------------------------------------------------------------------
def stream_probe_gbs(torch, bb, nbytes=1 << 30):
    """Read-only streaming ceilings measured here: 16-byte loads (mode 0) and bulk copies into a shared-memory
    ring (mode 1) over a buffer much larger than L2, best of 5."""
    buf = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    buf.fill_(1)
    sink = torch.zeros(4, dtype=torch.uint8, device="cuda")
    out = {}
    for mode, name in ((0, "ld16"), (1, "bulk")):
        best = None
        for i in range(7):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            rc = bb.stream_probe(buf, nbytes, mode, sink)
            e1.record()
            torch.cuda.synchronize()
            if rc != 0:
                best = None
                break
            if i >= 2:
                ms = e0.elapsed_time(e1)
                best = ms if best is None else min(best, ms)
        out[name] = None if best is None else nbytes / (best * 1e-3) / 1e9
    del buf
    return out


def apply_opts(args, bb):
    """--opt KEY=VALUE: library options by name (bonsai_b200_set_option), for sweeps."""
    for kv in getattr(args, "opt", []):
        key, _, val = kv.partition("=")
        if bb.set_option(key, int(val)) != 0:
            raise SystemExit(f"--opt {kv}: the library does not know this key (tuning keys need the tuning build)")


def run_b200(args):
    import torch
    import bonsai_b200 as bb
    from bonsai_b200 import partition

    rank, world, local = env_ranks()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    bb.lib()
    if args.pdl >= 0:
        bb.set_option("pdl", args.pdl)
    if args.order >= 0:
        bb.set_option("gemv_order", args.order)
    apply_opts(args, bb)

    sets = args.sets
    # ---- resident tensors: weights generated on the device, row slice of this rank only ----------
    mats = []               # (n_in, n_out, rows, W_slice, first_block_of_the_whole_matrix)
    blk_base = 0
    for s in range(sets):
        for n_in, n_out in LAYER_SHAPES:
            r_lo, r_hi = partition.row_slice(n_out, rank, world)
            rows = r_hi - r_lo
            nblk_row = n_in // 128
            W = torch.empty(rows * nblk_row * 34, dtype=torch.uint8, device="cuda")
            assert bb.synth_pq2_0(W, blk_base + r_lo * nblk_row, rows * nblk_row, args.seed) == 0
            mats.append((n_in, n_out, rows, W, blk_base))
            blk_base += n_out * nblk_row
    xq, xdev = {}, {}
    for n_in in sorted({a for a, _ in LAYER_SHAPES}):
        g = torch.Generator(device="cpu").manual_seed(args.seed + n_in)
        xdev[n_in] = torch.randn(n_in, generator=g, dtype=torch.float32).cuda()
        xq[n_in] = torch.empty(n_in // 32 * 36, dtype=torch.uint8, device="cuda")
        assert bb.fwht_quant(xdev[n_in], None, xq[n_in], None, n_in) == 0
    torch.cuda.synchronize()

    use_list = args.call == "list"
    # one sweep's outputs, rank-major when gathered: gathered[r] holds rank r's slice of every matrix, in
    # matrix order; `slice_off[i]` is where matrix i's slice starts inside a rank's part
    slice_off, off = [], 0
    for m in mats:
        slice_off.append(off)
        off += m[2]
    part = off
    y_local = torch.zeros(part, dtype=torch.float32, device="cuda")
    y_gathered = torch.zeros(world * part, dtype=torch.float32, device="cuda") if world > 1 else None

    # host buffers of the end-to-end leg: one pinned block with every activation vector of a sweep, one
    # pinned block for every output of a sweep (one copy each way per sweep)
    x_off, off = [], 0
    for m in mats:
        x_off.append(off)
        off += m[0]
    pin_x = torch.empty(off, dtype=torch.float32).pin_memory()
    for m, o in zip(mats, x_off):
        pin_x[o:o + m[0]] = xdev[m[0]].cpu()
    dev_x = torch.empty(off, dtype=torch.float32, device="cuda")
    xq_all = torch.empty(off // 32 * 36, dtype=torch.uint8, device="cuda")
    pin_y = torch.empty(world * part, dtype=torch.float32).pin_memory()

    def same_input_flag(i):     # consecutive matrices that read the same resident Q8_1 vector share its tables
        return bb.OP_SAME_INPUT if i and mats[i - 1][0] == mats[i][0] else 0

    def ops_resident(ybuf, base):
        return [(W, xq[n_in], None, ybuf[base + o:base + o + rows], rows, n_in, same_input_flag(i))
                for i, ((n_in, n_out, rows, W, _), o) in enumerate(zip(mats, slice_off))]

    def ops_e2e(ybuf, base, xq_buf):
        # end to end: the sweep's vectors arrive as one host block; FWHT-1024 and the quantiser work on 1024-
        # and 32-element blocks, so ONE bonsai_b200_fwht_quant call over the concatenation rotates and quantises
        # every vector (vector i's Q8_1 blocks start at byte x_off[i] / 32 * 36)
        return [(W, xq_buf[xo // 32 * 36:(xo + n_in) // 32 * 36], None, ybuf[base + o:base + o + rows], rows, n_in, 0)
                for (n_in, n_out, rows, W, _), o, xo in zip(mats, slice_off, x_off)]

    peer_ok = False
    if use_list and world > 1 and args.gather in ("auto", "peer"):
        try:                                    # the peer mapping needs the CUDA runtime bindings (same on every rank)
            import cuda.bindings.runtime       # noqa: F401
            peer_ok = True
        except Exception:
            if args.gather == "peer":
                raise
    chain = chain_e2e = None
    peers = {}
    if use_list:
        chain = bb.Chain(ops_resident(y_local, 0))
        chain_e2e = bb.Chain(ops_e2e(y_local, 0, xq_all))
    if peer_ok:
        from bonsai_b200.peer import PeerBuffer
        for key in ("value", "e2e"):          # one buffer (outputs + counters) per chain
            pb = PeerBuffer(world * part * 4, dist, rank, world)
            yp = pb.tensor.view(torch.float32)
            ch = bb.Chain(ops_resident(yp, rank * part) if key == "value" else ops_e2e(yp, rank * part, xq_all), peers=pb)
            peers[key] = (pb, yp, ch)

    # ---- the candidates for one sweep ------------------------------------------------------------------
    def sweep_matrix():
        for i, (n_in, n_out, rows, W, _) in enumerate(mats):
            rc = bb.gemv(W, xq[n_in], y_local[slice_off[i]:slice_off[i] + rows], rows, n_in)
            assert rc == 0
        if world > 1:
            dist.all_gather_into_tensor(y_gathered, y_local)

    def sweep_list_nccl():
        assert chain.run() == 0
        if world > 1:
            dist.all_gather_into_tensor(y_gathered, y_local)

    def sweep_list_peer():
        assert peers["value"][2].run() == 0

    def e2e_matrix():
        dev_x.copy_(pin_x, non_blocking=True)
        assert bb.fwht_quant(dev_x, None, xq_all, None, dev_x.numel()) == 0
        for i, (n_in, n_out, rows, W, _) in enumerate(mats):
            xo = x_off[i]
            assert bb.gemv(W, xq_all[xo // 32 * 36:(xo + n_in) // 32 * 36], y_local[slice_off[i]:slice_off[i] + rows],
                           rows, n_in) == 0
        if world > 1:
            dist.all_gather_into_tensor(y_gathered, y_local)
            pin_y.copy_(y_gathered, non_blocking=True)
        else:
            pin_y.copy_(y_local, non_blocking=True)

    def e2e_list_nccl():
        dev_x.copy_(pin_x, non_blocking=True)
        assert bb.fwht_quant(dev_x, None, xq_all, None, dev_x.numel()) == 0
        assert chain_e2e.run() == 0
        if world > 1:
            dist.all_gather_into_tensor(y_gathered, y_local)
            pin_y.copy_(y_gathered, non_blocking=True)
        else:
            pin_y.copy_(y_local, non_blocking=True)

    def e2e_list_peer():
        dev_x.copy_(pin_x, non_blocking=True)
        assert bb.fwht_quant(dev_x, None, xq_all, None, dev_x.numel()) == 0
        assert peers["e2e"][2].run() == 0
        pin_y.copy_(peers["e2e"][1], non_blocking=True)

    # ---- which data plane between the ranks: measured here, not assumed ----------------------------------
    gather, gather_probe = ("none" if world == 1 else "nccl"), None
    if use_list and world > 1:
        if args.gather == "auto" and peer_ok:
            gather_probe = {}
            for name, fn in (("nccl", sweep_list_nccl), ("peer", sweep_list_peer)):
                run = graph_of(torch, fn)
                for _ in range(5):
                    run()
                torch.cuda.synchronize()
                dist.barrier()
                gather_probe[name] = device_ms(torch, run, 40, dist) / 40 * 1e3        # us per sweep, max over ranks
            gather = min(gather_probe, key=gather_probe.get)
        elif args.gather == "peer" and peer_ok:
            gather = "peer"
    if not use_list:
        sweep_fn, e2e_fn = sweep_matrix, e2e_matrix
    elif gather == "peer":
        sweep_fn, e2e_fn = sweep_list_peer, e2e_list_peer
    else:
        sweep_fn, e2e_fn = sweep_list_nccl, e2e_list_nccl
    launches_per_sweep = 1 if use_list else len(mats)

    def e2e_pipelined(steps, warmup):
        """The end-to-end sweep on three streams with two buffer sets: sweep i's host->device copy, its
        launches and its device->host copy run on their own streams, ordered by events, so that the
        copies of neighbouring sweeps overlap the mat-vecs (every sweep still copies its inputs in and its
        outputs out inside the timed region).  One GPU, list mode.  Returns (ms, sweeps)."""
        s_in, s_k, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        dx = [dev_x, torch.empty_like(dev_x)]
        xa = [xq_all, torch.empty_like(xq_all)]
        yl = [y_local, torch.zeros_like(y_local)]
        py = [pin_y, torch.empty_like(pin_y).pin_memory()]
        chains = [chain_e2e, bb.Chain(ops_e2e(yl[1], 0, xa[1]))]
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_k = [torch.cuda.Event() for _ in range(2)]
        ev_out = [torch.cuda.Event() for _ in range(2)]
        torch.cuda.synchronize()

        def run(n, first):
            for i in range(first, first + n):
                b = i & 1
                with torch.cuda.stream(s_in):
                    if i >= 2:
                        s_in.wait_event(ev_k[b])            # the launches of sweep i - 2 have read this input buffer
                    dx[b].copy_(pin_x, non_blocking=True)
                    ev_in[b].record(s_in)
                with torch.cuda.stream(s_k):
                    s_k.wait_event(ev_in[b])
                    if i >= 2:
                        s_k.wait_event(ev_out[b])           # sweep i - 2's outputs have left this buffer
                    assert bb.fwht_quant(dx[b], None, xa[b], None, dx[b].numel()) == 0
                    assert chains[b].run() == 0
                    ev_k[b].record(s_k)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_k[b])
                    py[b].copy_(yl[b], non_blocking=True)
                    ev_out[b].record(s_out)
        run(4, 0)
        torch.cuda.synchronize()
        # 32 sweeps per graph (the three streams fork from and join the capturing stream); replays serialise,
        # so one sweep in 32 starts without a neighbour to overlap with
        per_graph = 32
        graph, cap = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        with torch.cuda.graph(graph, stream=cap):
            for st in (s_in, s_k, s_out):
                st.wait_stream(cap)
            run(per_graph, 0)
            for st in (s_in, s_k, s_out):
                cap.wait_stream(st)
        for _ in range(max(1, warmup // per_graph)):
            graph.replay()
        torch.cuda.synchronize()
        est = device_ms(torch, graph.replay, 2) / 2
        replays = max(1, steps // per_graph, int(math.ceil(MIN_TIMED_MS / max(1e-6, est))))
        ms = device_ms(torch, graph.replay, replays)
        chains[1].close()
        return ms, replays * per_graph

    total_w = sum(weight_bytes(a, b) for a, b in LAYER_SHAPES) * sets
    total_alg = sum(algorithmic_bytes(a, b // world) for a, b in LAYER_SHAPES) * sets      # per rank and sweep
    ms, reps, clocks = timed(torch, sweep_fn, args.steps, args.warmup, dist, local, not args.no_graph)
    sweeps = args.steps * reps
    value = total_w * sweeps / (ms * 1e-3) / 1e9

    # ---- parity of what was just timed: every output vector against the per-matrix call on the unsplit matrix --
    def full_vector(src, i):
        rows = mats[i][2]
        if world == 1:
            return src[slice_off[i]:slice_off[i] + rows]
        return torch.cat([src[r * part + slice_off[i]:r * part + slice_off[i] + rows] for r in range(world)])

    def check_outputs(src):
        bad, worst = 0, 0.0
        for i, (n_in, n_out, rows, W, first) in enumerate(mats):
            if world == 1:
                Wf = W
            else:
                Wf = torch.empty(n_out * (n_in // 128) * 34, dtype=torch.uint8, device="cuda")
                assert bb.synth_pq2_0(Wf, first, n_out * (n_in // 128), args.seed) == 0
            want = torch.empty(n_out, dtype=torch.float32, device="cuda")
            assert bb.gemv(Wf, xq[n_in], want, n_out, n_in) == 0
            got = full_vector(src, i)
            if not torch.equal(got.view(torch.int32), want.view(torch.int32)):
                bad += 1
                worst = max(worst, float((got - want).abs().max().item()))
        return bad, worst

    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    timed_out = y_local if world == 1 else (peers["value"][1] if (use_list and gather == "peer") else y_gathered)
    bad, worst = check_outputs(timed_out)

    # ---- end to end ------------------------------------------------------------------------------------
    e2e_steps = max(1, args.steps // 4)
    ms_e, reps_e, _ = timed(torch, e2e_fn, e2e_steps, max(3, args.warmup // 4), dist, None, not args.no_graph)
    e2e_value = total_w * e2e_steps * reps_e / (ms_e * 1e-3) / 1e9
    e2e_mode, e2e_serial = "one stream: copy in, launches, copy out, in order", None
    torch.cuda.synchronize()
    bad_e, worst_e = check_outputs(pin_y.cuda())
    if use_list and world == 1 and not args.no_graph:
        ms_p, sweeps_p = e2e_pipelined(e2e_steps, max(8, args.warmup // 4))
        e2e_serial = e2e_value
        e2e_value = total_w * sweeps_p / (ms_p * 1e-3) / 1e9
        e2e_mode = "three streams, two buffer sets: the copies of neighbouring sweeps overlap the launches"
    if dist is not None:
        t = torch.tensor([bad + bad_e, worst, worst_e], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        bad_all, worst_all = int(t[0].item()), float(max(t[1].item(), t[2].item()))
    else:
        bad_all, worst_all = bad + bad_e, max(worst, worst_e)

    per_matrix = None
    if use_list:        # the unchanged per-matrix ABI on the same tensors, for comparison
        ms_m, reps_m, _ = timed(torch, sweep_matrix, e2e_steps, max(3, args.warmup // 4), dist, None, not args.no_graph)
        per_matrix = {"call": "bonsai_p40_gemv per matrix" + (" + all-gather per sweep" if world > 1 else ""),
                      "value": total_w * e2e_steps * reps_m / (ms_m * 1e-3) / 1e9, "unit": UNIT,
                      "ms_per_sweep": ms_m / (e2e_steps * reps_m), "gpu_launches_per_sweep": len(mats)}
    split = None
    if use_list and world > 1:      # where a sweep's time goes on the all-gather plane: the launch alone, the collective alone
        def only_matvec():
            assert chain.run() == 0

        def only_gather():
            dist.all_gather_into_tensor(y_gathered, y_local)
        ms_k, reps_k, _ = timed(torch, only_matvec, e2e_steps, 3, dist, None, not args.no_graph)
        ms_g, reps_g, _ = timed(torch, only_gather, e2e_steps, 3, dist, None, not args.no_graph)
        split = {"matvec_us_per_sweep": ms_k / (e2e_steps * reps_k) * 1e3,
                 "allgather_us_per_sweep": ms_g / (e2e_steps * reps_g) * 1e3,
                 "allgather_bytes_per_rank": int(y_local.numel() * 4)}
    status = bb.device_status()

    peak, bf16_peak, peak_kind = measured_peaks()
    probe = stream_probe_gbs(torch, bb) if rank == 0 else None
    launch_alg = total_alg / launches_per_sweep
    launch_us = ms * 1e3 / (sweeps * launches_per_sweep)
    achieved = launch_alg / (launch_us * 1e-6) / 1e9
    traffic, traffic_kind = None, None
    if world == 1:          # DRAM bytes per launch from the committed ncu capture of the same kernel form, scaled by bytes
        name = "gemv_chain_traffic.json" if use_list else "gemv_stream_traffic.json"
        try:
            t = json.load(open(os.path.join(ROOT, "profiles", name)))
            traffic = t["dram_bytes_per_launch"] / t["algorithmic_bytes_per_launch"] * launch_alg
            traffic_kind = f"scaled from the committed ncu capture profiles/{name} (N = 1); not measured in this run"
        except Exception:
            pass
    roof = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": UNIT, "frac": achieved / peak,
            "peak_kind": peak_kind + " HBM copy bandwidth", "frac_nominal": achieved / NOMINAL_HBM_GBS,
            "nominal_peak": NOMINAL_HBM_GBS, "traffic": traffic, "traffic_kind": traffic_kind,
            "avg_launch_us": launch_us, "algorithmic_bytes_per_launch": launch_alg,
            "kernel": "gemv_chain_kernel" if use_list else "gemv_stream_kernel"}
    if probe:
        best = max([v for v in probe.values() if v] or [0.0])
        roof["probe_gbs"] = probe
        roof["frac_probe"] = achieved / best if best else None
    if world == 1:
        par = "single"
    elif not use_list or gather == "nccl":
        par = f"rows/{world} + one NCCL all-gather per sweep"
    else:
        par = f"rows/{world}, outputs stored into every rank's buffer by the kernel (peer-mapped memory, no collective)"
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
        "config": {"workload": "layer_sweep", "shapes_nin_nout": LAYER_SHAPES, "batch": 1, "sets": sets,
                   "sweeps_per_step": reps, "us_per_sweep": ms * 1e3 / sweeps,
                   "resident_weight_bytes": total_w,
                   "l2": ("inputs larger than L2" if total_w / world > 126e6 else
                          f"the rank's slice ({total_w / world / 1e6:.0f} MB) is smaller than the 126 MB L2: weights may be served from it"),
                   "parallelism": par, "gather": gather, "gather_probe_us_per_sweep": gather_probe, "pdl": args.pdl,
                   "fp32_order": "host-sequential" if args.order == 1 else "fixed-tree",
                   "launch": "eager" if args.no_graph else "cuda_graph_per_sweep",
                   "call": "bonsai_b200_chain_run: the sweep's mat-vecs as one persistent launch" if use_list
                           else "bonsai_p40_gemv per matrix"},
        "gpu_launches": sweeps * launches_per_sweep,
        "clocks": clocks,
        "parity": {"checked": 2 * len(mats), "mismatches": bad_all, "max_abs": worst_all,
                   "against": "bonsai_p40_gemv on the unsplit matrix, bit for bit; timed leg and end-to-end leg, every rank"},
        "e2e": {"value": e2e_value, "unit": UNIT,
                "h2d_bytes_per_step": int(pin_x.numel() * 4) * reps_e, "d2h_bytes_per_step": int(pin_y.numel() * 4) * reps_e,
                "sweeps_per_step": reps_e, "mode": e2e_mode, "one_stream_value": e2e_serial},
        "roofline": roof,
        "device_status": status,
    }
    if per_matrix is not None:
        line["per_matrix_abi"] = per_matrix
    if split is not None:
        line["split"] = split
    if not args.no_secondary:
        sec = {}
        legs = [("batch8", batch_leg)]              # at every N; the others on one GPU
        if world == 1:
            legs += [("batch16", lambda a, t, b, d: batch_leg(a, t, b, d, n_tok=16)),
                     ("batch32", lambda a, t, b, d: batch_leg(a, t, b, d, n_tok=32)),
                     ("decode_step", decode_step_leg), ("prefill", prefill_leg), ("repack_gemv", repack_leg),
                     ("beside_the_path", beside_leg)]
        for name, leg in legs:
            try:
                sec[name] = leg(args, torch, bb, dist)
            except Exception as e:                 # a failing secondary leg must not hide the headline
                if dist is not None:
                    raise                          # several ranks: an exception on one rank must not leave the others waiting
                sec[name] = {"error": f"{type(e).__name__}: {e}"[:300]}
        line["secondary"] = sec
    if world == 1 and not args.no_cpu:
        threads = os.cpu_count() or 1
        kind, sweep, wbytes = cpu_arm(threads)
        sweep()
        n, t0 = 0, time.perf_counter()
        while time.perf_counter() - t0 < args.cpu_seconds:
            sweep()
            n += 1
        dt = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": wbytes * n / dt / 1e9, "unit": UNIT, "cores": threads, "kind": kind,
                                "sample": f"{n} layer sweeps (4 mat-vecs each, FWHT+Q8_1 included) in {dt:.1f} s"}
        _, sweep1, _ = cpu_arm(1)             # the same code on one host thread
        t0 = time.perf_counter()
        sweep1()
        dt1 = time.perf_counter() - t0
        line["cpu_baseline"]["single_thread"] = {"value": wbytes / dt1 / 1e9, "unit": UNIT,
                                                 "sample": f"1 layer sweep in {dt1:.2f} s"}
    if rank == 0:
        print(json.dumps(line))
    for pb, _, ch in peers.values():
        ch.close()
        pb.close(dist)
    if dist is not None:
        dist.destroy_process_group()
    if bad_all or status != 0:
        raise SystemExit(f"parity or status failure: mismatches={bad_all} max_abs={worst_all:.3e} status={status}")


# ---- the decode step ---------------------------------------------------------------------------------
def model_gemvs():
    """(n_in, n_out) of every PQ2_0 mat-vec of one decoded token, in layer order: 64 layers (48 linear-
    attention, every 4th full attention) plus the output head -- 401 mat-vecs, 6.8 GB of weights
    (reference: include/bonsai_model.h:29-59, tools/check_gguf.py:45-62)."""
    out = []
    for layer in range(64):
        if (layer + 1) % 4 == 0:
            out += [(5120, 12288), (5120, 1024), (5120, 1024), (6144, 5120)]
        else:
            out += [(5120, 10240), (5120, 6144), (6144, 5120)]
        out += [(5120, 17408), (5120, 17408), (17408, 5120)]
    out.append((5120, 248320))
    return out


def decode_ops(torch, bb, shapes, seed, flow, rank=0, world=1, y_all=None):
    """The op list of one decoded token.  flow=True (one rank): op i reads the output of op i - 1 through the exact
    power-of-two glue (x_i[j] = y_{i-1}[j mod N_{i-1}] * 2^-e, e = floor(log2(max |y_{i-1}|))), projections of equal
    input width that follow each other share one input.  flow=False: every op rotates and quantises a resident
    vector of its input width; the waits between the ops are the same.  Returns (ops, outputs, weights)."""
    from bonsai_b200 import partition
    ws, rows_of, first = [], [], 0
    for n_in, n_out in shapes:
        lo, hi = partition.row_slice(n_out, rank, world)
        nblk_row = n_in // 128
        W = torch.empty((hi - lo) * nblk_row * 34, dtype=torch.uint8, device="cuda")
        assert bb.synth_pq2_0(W, first + lo * nblk_row, (hi - lo) * nblk_row, seed) == 0
        first += n_out * nblk_row
        ws.append(W)
        rows_of.append(hi - lo)
    g = torch.Generator(device="cpu").manual_seed(seed)
    xs = {k: torch.randn(k, generator=g).cuda() for k in sorted({a for a, _ in shapes})}
    y_off, off = [], 0
    for _, n_out in shapes:
        y_off.append(off)
        off += n_out
    if y_all is None:
        y_all = torch.zeros(off, dtype=torch.float32, device="cuda")
    ys = [y_all[o:o + n] for o, (_, n) in zip(y_off, shapes)]
    ops = []
    for i, ((n_in, n_out), W) in enumerate(zip(shapes, ws)):
        r = rows_of[i]
        same = i > 0 and shapes[i - 1][0] == n_in
        fl = bb.OP_ROTATE | (bb.OP_SAME_INPUT if same else (bb.OP_DEPENDS if i else 0))
        ysl = ys[i][rank * r:(rank + 1) * r]
        if flow and same:           # the previous op's input, prepared the same way
            ops.append((W, ops[i - 1][1], None, ysl, r, n_in, fl | (ops[i - 1][6] & bb.OP_RESCALE), None, 0.0, ops[i - 1][9]))
        elif flow and i > 0:
            ops.append((W, ys[i - 1], None, ysl, r, n_in, fl | bb.OP_RESCALE, None, 0.0, shapes[i - 1][1]))
        else:
            ops.append((W, xs[n_in], None, ysl, r, n_in, fl, None, 0.0, 0))
    return ops, ys, ws


def glue_vector(torch, y_prev, n_in):
    """The glue of decode_ops(flow=True), with torch on the device: exact (a power-of-two factor, an index map)."""
    m = y_prev.abs().max()
    scale = torch.ones((), device=y_prev.device)
    if float(m.item()) >= 1.1754943508222875e-38:
        _, ex = torch.frexp(m)
        scale = torch.ldexp(scale, -(ex - 1))
    idx = torch.arange(n_in, device=y_prev.device) % y_prev.numel()
    return (y_prev[idx] * scale).contiguous()


def decode_step_leg(args, torch, bb, dist):
    """The 401 projections of one decoded token (6.8 GB of PQ2_0 weights) as ONE list launch per token
    (bonsai_b200_chain_run), replayed as one CUDA graph: tokens/s and weight GB/s.  On one GPU the values flow: each
    projection rotates and quantises the previous projection's output (exact power-of-two glue), projections that read
    the same vector share its quantised form, every other projection waits for all rows of the projections before
    it.  With N > 1 every matrix is split by output rows; the outputs reach every rank by peer stores inside the kernel
    (list) or by an all-gather behind every projection (per-matrix calls), and every projection reads a resident
    vector (the glue needs the maximum over all ranks' rows, which the kernel records on one rank only).
    Parity: every projection's output of the timed launch against the per-matrix call (bonsai_b200_linear) on the
    unsplit matrix and the same input vector -- for flowing values the glue'd previous output -- bit for bit."""
    rank, world, local = env_ranks()
    if dist is None:
        world, rank = 1, 0
    bb.set_option("pdl", max(args.pdl, 0))
    shapes = model_gemvs()
    use_list = args.call == "list"
    flow = use_list and world == 1
    peer_buf, chain, y_all = None, None, None
    if use_list and world > 1:
        from bonsai_b200.peer import PeerBuffer
        peer_buf = PeerBuffer(sum(n for _, n in shapes) * 4, dist, rank, world)
        y_all = peer_buf.tensor.view(torch.float32)
    ops, ys, ws = decode_ops(torch, bb, shapes, args.seed, flow, rank, world, y_all)
    xq = {k: torch.empty(k // 32 * 36, dtype=torch.uint8, device="cuda") for k in sorted({a for a, _ in shapes})}
    launches_per_token = len(shapes)
    if use_list:
        chain = bb.Chain(ops, peers=peer_buf)
        launches_per_token = 1

        def token():
            assert chain.run() == 0
    else:
        def token():
            for (W, x, _, ysl, r, n_in, *_), yv in zip(ops, ys):
                assert bb.linear(W, x, None, ysl, xq[n_in], r, n_in) == 0    # rotation + quantiser + mat-vec
                if world > 1:
                    dist.all_gather_into_tensor(yv, ysl)

    steps = max(3, min(args.steps, 30))
    warm = max(3, min(args.warmup, 5))
    ms, reps, clocks = timed(torch, token, steps, warm, dist, local, True)
    ms_tok = ms / (steps * reps)
    # parity: the per-matrix call on the unsplit matrix and the same input vector, every projection
    bad, worst = 0, 0.0
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    first, x_cur = 0, None
    for i, (n_in, n_out) in enumerate(shapes):
        nblk = n_out * (n_in // 128)
        if world == 1:
            Wf = ws[i]
        else:
            Wf = torch.empty(nblk * 34, dtype=torch.uint8, device="cuda")
            assert bb.synth_pq2_0(Wf, first, nblk, args.seed) == 0
        first += nblk
        if not flow or i == 0:
            x_cur = ops[i][1]
        elif not (ops[i][6] & bb.OP_SAME_INPUT):
            x_cur = glue_vector(torch, ys[i - 1], n_in)
        want = torch.empty(n_out, dtype=torch.float32, device="cuda")
        assert bb.linear(Wf, x_cur, None, want, xq[n_in], n_out, n_in) == 0
        got = ys[i]
        if not torch.equal(got.view(torch.int32), want.view(torch.int32)):
            bad += 1
            worst = max(worst, float((got - want).abs().max().item()))
        del Wf
    if dist is not None:
        t = torch.tensor([bad, worst], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        bad, worst = int(t[0].item()), float(t[1].item())
    wbytes = sum(weight_bytes(a, b) for a, b in shapes)
    peak, _, peak_kind = measured_peaks()
    gbs = wbytes / (ms_tok * 1e-3) / 1e9
    status = bb.device_status()
    call = ("bonsai_b200_chain_run, one launch per token" + (" and rank, outputs stored into every rank's buffer "
            "by the kernel" if world > 1 else "") if launches_per_token == 1 else
            "bonsai_b200_linear per matrix" + (", then an all-gather" if world > 1 else ""))
    out = {"metric": "decode_tokens_per_s", "value": 1e3 / ms_tok, "unit": "tokens/s", "ms_per_token": ms_tok,
           "weight_gbs": gbs, "matvecs": len(shapes), "weight_bytes": wbytes, "call": call, "values_flow": flow,
           "gpu_launches": launches_per_token * steps * reps, "steps": steps, "tokens_per_step": reps,
           "frac": gbs / world / peak, "frac_nominal": gbs / world / NOMINAL_HBM_GBS, "peak_kind": peak_kind,
           "parity": {"checked": len(shapes), "mismatches": bad, "max_abs": worst,
                      "against": "bonsai_b200_linear on the unsplit matrix and the same input, bit for bit"},
           "clocks": clocks, "device_status": status}
    if chain is not None:
        chain.close()
    if peer_buf is not None:
        peer_buf.close(dist)
    return out


def run_decode_step(args):
    import torch
    import bonsai_b200 as bb
    rank, world, local = env_ranks()
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    bb.lib()
    apply_opts(args, bb)
    leg = decode_step_leg(args, torch, bb, dist)
    if rank == 0:
        peak, _, peak_kind = measured_peaks()
        print(json.dumps({
            "metric": "decode_tokens_per_s", "value": leg["value"], "unit": "tokens/s", "n_gpus": world, "steps": leg["steps"],
            "warmup": max(3, min(args.warmup, 5)), "ms_per_step": leg["ms_per_token"] * leg["tokens_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
            "config": {"workload": "decode_step", "matvecs": leg["matvecs"], "weight_bytes": leg["weight_bytes"], "batch": 1,
                       "pdl": args.pdl, "l2": "inputs larger than L2", "launch": "cuda_graph_per_token", "call": leg["call"],
                       "values_flow": leg["values_flow"],
                       "tokens_per_step": leg["tokens_per_step"],
                       "parallelism": "single" if world == 1 else f"rows/{world}"},
            "gpu_launches": leg["gpu_launches"], "clocks": leg["clocks"], "parity": leg["parity"],
            "roofline": {"bound": "hbm", "achieved": leg["weight_gbs"] / world, "peak": peak, "unit": "GB/s",
                         "frac": leg["frac"], "frac_nominal": leg["frac_nominal"], "peak_kind": peak_kind, "traffic": None},
            "device_status": leg["device_status"]}))
    if dist is not None:
        dist.destroy_process_group()
    if leg["parity"]["mismatches"] or leg["device_status"] != 0:
        raise SystemExit("parity or status failure in the decode step")


# ---- prefill -----------------------------------------------------------------------------------------
def prefill_leg(args, torch, bb, dist):
    """M = 512 tokens through the two large projections; a step = token-batch rotation + quantiser into the
    chunk-major layout, then the tensor-core mat-mul, for both matrices.  Parity: 256 output rows of each matrix
    against the integer SIMT kernel (which keeps the host loop's bits), bound 1e-5 x max |Y|."""
    n_tok = 512
    mats = []
    for n_in, n_out in [(5120, 17408), (17408, 5120)]:
        nblk = n_out * (n_in // 128)
        W = torch.empty(nblk * 34, dtype=torch.uint8, device="cuda")
        assert bb.synth_pq2_0(W, 0, nblk, args.seed) == 0
        X = torch.randn(n_tok, n_in, device="cuda")
        Xq = torch.empty(n_in // 32 * n_tok * 36, dtype=torch.uint8, device="cuda")
        Y = torch.empty(n_out, n_tok, device="cuda")
        mats.append((n_in, n_out, W, X, Xq, Y))

    path = getattr(args, "gemm_path", -1)
    bb.set_option("gemm_path", path)

    def step():
        for n_in, n_out, W, X, Xq, Y in mats:
            assert bb.quant_batch(X, None, Xq, n_in, n_tok, True) == 0
            assert bb.gemm(W, Xq, Y, n_out, n_in, n_tok) == 0

    steps = max(3, min(args.steps, 30))
    ms, reps, clocks = timed(torch, step, steps, max(3, min(args.warmup, 5)), None, 0, True)
    ms_step = ms / (steps * reps)
    # the mat-mul alone (without the quantiser launches), per matrix
    per = []
    for n_in, n_out, W, X, Xq, Y in mats:
        def only(W=W, Xq=Xq, Y=Y, n_out=n_out, n_in=n_in):
            assert bb.gemm(W, Xq, Y, n_out, n_in, n_tok) == 0
        m, r, _ = timed(torch, only, steps, 3, None, None, True)
        per.append({"n_in": n_in, "n_out": n_out, "us": m / (steps * r) * 1e3,
                    "tops": 2.0 * n_tok * n_in * n_out / (m / (steps * r) * 1e-3) / 1e12})
    # parity on a row subset: the same rows through the integer SIMT kernel
    bad, worst_rel = 0, 0.0
    rows = 256
    try:
        for n_in, n_out, W, X, Xq, Y in mats:
            r0 = (n_out // 2) // 128 * 128
            Wsub = W[r0 * (n_in // 128) * 34:(r0 + rows) * (n_in // 128) * 34]
            Yref = torch.empty(rows, n_tok, device="cuda")
            bb.set_option("gemm_path", 0)
            assert bb.gemm(Wsub, Xq, Yref, rows, n_in, n_tok) == 0
            bb.set_option("gemm_path", path)
            torch.cuda.synchronize()
            got = Y[r0:r0 + rows]
            rel = float(((got - Yref).abs().max() / Yref.abs().max()).item())
            worst_rel = max(worst_rel, rel)
            if not rel <= 1e-5:
                bad += 1
    finally:
        bb.set_option("gemm_path", -1)
    ops = sum(2.0 * n_tok * a * b for a, b, *_ in mats)
    tops = ops / (ms_step * 1e-3) / 1e12
    _, bf16, kind = measured_peaks()
    # The default kernel runs fp16 MMAs, two per useful product (the activations are split into two exact fp16 halves):
    # the denominator is the measured dense bf16 peak, and the kernel's own ceiling is half of it.  The integer
    # tensor-core kernel (--gemm-path 3) is held against twice that peak (int8).
    fp16_form = path in (-1, 1)
    peak = bf16 if fp16_form else 2.0 * bf16
    # a dense int8 figure measured here, beside the denominator above: the library's int8 mat-mul (cuBLASLt through
    # torch._int_mm) on 8192^3, best of 10 -- a measuring stick, not on the path
    int8_lib = None
    try:
        n = 8192
        a = torch.randint(-3, 4, (n, n), dtype=torch.int8, device="cuda")
        b = torch.randint(-3, 4, (n, n), dtype=torch.int8, device="cuda").t()
        for _ in range(3):
            torch._int_mm(a, b)
        best = 1e9
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._int_mm(a, b)
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        int8_lib = 2.0 * n ** 3 / (best * 1e-3) / 1e12
    except Exception:
        pass
    return {"metric": "pq2_0_prefill_gemm", "value": tops, "unit": "TOPS", "n_tok": n_tok, "ms_per_step": ms_step,
            "steps": steps, "passes_per_step": reps, "gpu_launches": 4 * steps * reps, "per_matrix": per,
            "frac": tops / peak, "peak": peak,
            "peak_kind": (f"{kind} dense bf16; the kernel issues two fp16 MMAs per useful product, its ceiling is half"
                          if fp16_form else f"2 x {kind} dense bf16 (int8)"),
            "kernel": "gemm_tc16_kernel (fp16 split)" if fp16_form else ("gemm_tc_kernel (int8)" if path == 3 else f"gemm_path {path}"),
            "dtype": ("fp16 x fp16 -> fp32 (tcgen05), activations int8 x fp16 split exactly into two fp16" if fp16_form
                      else "int8 x int8 -> int32 (tcgen05), fp32 scale"),
            "library_int8_dense_tops_measured": int8_lib,
            "parity": {"checked_rows_per_matrix": rows, "mismatches": bad, "max_rel_to_max_abs": worst_rel, "bound": 1e-5,
                       "against": "the integer SIMT mat-mul (host-loop bits) on the same rows"},
            "clocks": clocks, "device_status": bb.device_status()}


def run_prefill(args):
    import torch
    import bonsai_b200 as bb
    torch.cuda.set_device(0)
    bb.lib()
    apply_opts(args, bb)
    leg = prefill_leg(args, torch, bb, None)
    print(json.dumps({
        "metric": leg["metric"], "value": leg["value"], "unit": "TOPS", "n_gpus": 1, "steps": leg["steps"],
        "warmup": max(3, min(args.warmup, 5)), "ms_per_step": leg["ms_per_step"] * leg["passes_per_step"],
        "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": leg["dtype"], "data": "synthetic",
        "config": {"workload": "prefill", "kernel": leg["kernel"], "n_tok": leg["n_tok"], "shapes_nin_nout": [[5120, 17408], [17408, 5120]],
                   "launch": "cuda_graph_per_step", "passes_per_step": leg["passes_per_step"], "per_matrix": leg["per_matrix"]},
        "gpu_launches": leg["gpu_launches"], "clocks": leg["clocks"], "parity": leg["parity"],
        "roofline": {"bound": "tensor", "achieved": leg["value"], "peak": leg["peak"], "unit": "TOPS", "frac": leg["frac"],
                     "peak_kind": leg["peak_kind"], "traffic": None,
                     "library_int8_dense_tops_measured": leg["library_int8_dense_tops_measured"]},
        "device_status": leg["device_status"]}))
    if leg["parity"]["mismatches"] or leg["device_status"] != 0:
        raise SystemExit("parity or status failure in the prefill leg")


# ---- repacked-layout mat-vec ---------------------------------------------------------------------------
def repack_leg(args, torch, bb, dist):
    """bonsai_p40_gemv_repack (fused quantiser + mat-vec over the aligned repacked layout) on the four layer
    shapes, 8 resident copies each (larger than L2), one launch per matrix.  Parity: the repacked bytes round-trip
    is covered by the tests; here y is compared with bonsai_p40_gemv on the un-repacked matrix (same terms, other
    summation order): bound 1e-5 x max |y|."""
    sets = args.sets
    mats, total_w = [], 0
    for s in range(sets):
        for j, (n_in, n_out) in enumerate(LAYER_SHAPES):
            nblk = n_out * (n_in // 128)
            W = torch.empty(nblk * 34, dtype=torch.uint8, device="cuda")
            assert bb.synth_pq2_0(W, (s * 4 + j) * 1000003, nblk, args.seed) == 0
            Wr = torch.empty_like(W)
            assert bb.repack(W, Wr, n_out, n_in) == 0
            mats.append((n_in, n_out, W if s == 0 else None, Wr))
            total_w += nblk * 34
    g = torch.Generator(device="cpu").manual_seed(args.seed + 7)
    xs = {k: torch.randn(k, generator=g).cuda() for k in sorted({a for a, _ in LAYER_SHAPES})}
    ys = {n: torch.empty(n, device="cuda") for n in {b for _, b in LAYER_SHAPES}}

    def sweep():
        for n_in, n_out, _, Wr in mats:
            assert bb.gemv_repack(Wr, xs[n_in], ys[n_out], n_out, n_in) == 0

    steps = max(3, min(args.steps, 50))
    ms, reps, _ = timed(torch, sweep, steps, 3, None, None, True)
    gbs = total_w * steps * reps / (ms * 1e-3) / 1e9
    bad, worst = 0, 0.0
    for n_in, n_out, W, Wr in mats[:4]:
        xq = torch.empty(n_in // 32 * 36, dtype=torch.uint8, device="cuda")
        assert bb.quant_activations(xs[n_in], xq, n_in) == 0
        want = torch.empty(n_out, device="cuda")
        got = torch.empty(n_out, device="cuda")
        assert bb.gemv(W, xq, want, n_out, n_in) == 0
        assert bb.gemv_repack(Wr, xs[n_in], got, n_out, n_in) == 0
        torch.cuda.synchronize()
        rel = float(((got - want).abs().max() / want.abs().max()).item())
        worst = max(worst, rel)
        if not rel <= 1e-5:
            bad += 1
    peak, _, kind = measured_peaks()
    return {"metric": "pq2_0_gemv_repack_weight_stream", "value": gbs, "unit": UNIT, "us_per_sweep": ms * 1e3 / (steps * reps),
            "gpu_launches": len(mats) * steps * reps, "frac": gbs / peak, "frac_nominal": gbs / NOMINAL_HBM_GBS,
            "peak_kind": kind, "call": "bonsai_p40_gemv_repack per matrix (quantiser fused)",
            "parity": {"checked": 4, "mismatches": bad, "max_rel_to_max_abs": worst, "bound": 1e-5,
                       "against": "bonsai_p40_gemv on the un-repacked matrix"},
            "device_status": bb.device_status()}


# ---- the operators, the cache and the load-time steps beside the mat-vec path ------------------------------------
def beside_leg(args, torch, bb, dist):
    """Device-timed throughput of the rows next to the hot path, each on a working set larger than L2 and against the
    bound that applies (HBM bytes that must move, or fp32 FLOP/s for the causal attention): RMSNorm, the gated delta-net
    step over the 48 layers' state, causal attention of a 2048-token prefill, K/V append and decode attention at 32 768
    cached positions over the 16 cached layers, PQ2_0 -> repacked layout, PQ2_0 <-> PTQ1_0.  Results are checked against
    the CPU checker by tests/test_gpu_ops.py, test_gpu_kv.py, test_gpu_load.py; here only the status word is read."""
    peak, _, kind = measured_peaks()
    out = {}

    def rate(fn, nbytes, launches, steps=5):
        ms, reps, _ = timed(torch, fn, steps, 2, None, None, True)
        us = ms * 1e3 / (steps * reps)
        return {"GB/s": nbytes / us / 1e3, "us": us, "frac": nbytes / us / 1e3 / peak, "gpu_launches": launches}

    g = torch.Generator(device="cpu").manual_seed(args.seed + 21)
    # RMSNorm: 8192 rows of 5120 (168 MB in, 168 MB out)
    rows, n = 8192, 5120
    x = torch.randn(rows, n, generator=g).cuda()
    w = torch.randn(n, generator=g).cuda()
    y = torch.empty_like(x)
    out["rmsnorm_8192x5120"] = rate(lambda: bb.rmsnorm(x, w, y, rows, n, 1e-6), 2 * rows * n * 4, 1)
    del x, y
    # delta-net step: 48 layers x [48 heads][128][128] fp32 state, read and written once (151 MB each way)
    layers, nk, nv, K, V = 48, 16, 48, 128, 128
    st = [torch.randn(nv, K, V, generator=g).cuda() * 0.01 for _ in range(layers)]
    q = torch.randn(nk, K, generator=g).cuda()
    k = torch.randn(nk, K, generator=g).cuda() * 0.1
    v = torch.randn(nv, V, generator=g).cuda()
    gg = -torch.rand(nv, generator=g).cuda()
    be = torch.rand(nv, generator=g).cuda()
    o = torch.empty(nv, V, device="cuda")

    def gdn():
        for s_ in st:
            assert bb.gdn_step(s_, q, k, v, gg, be, o, nk, nv, K, V) == 0
    out["gdn_step_48_layers"] = rate(gdn, 2 * layers * nv * K * V * 4, layers)
    del st
    # causal attention, prefill of 2048 tokens: 24 heads over 4 kv heads, head dimension 256, fp32 on the CUDA cores
    T, H, HKV, D = 2048, 24, 4, 256
    qa = torch.randn(T, H, D, generator=g).cuda()
    ka = torch.randn(T, HKV, D, generator=g).cuda()
    va = torch.randn(T, HKV, D, generator=g).cuda()
    oa = torch.empty_like(qa)
    ms, reps, _ = timed(torch, lambda: bb.attn(qa, ka, va, oa, T, H, HKV, D, 1.0 / 16.0), 3, 1, None, None, True)
    us = ms * 1e3 / (3 * reps)
    flops = 4.0 * H * D * (T * (T + 1) / 2)
    out["attn_prefill_2048"] = {"TFLOP/s": flops / us / 1e6, "us": us, "bound": "fp32 FMA on the CUDA cores (no tensor cores: "
                                "the reference's kernel and its test are fp32)", "gpu_launches": 1}
    del qa, ka, va, oa
    # K/V cache: 32 768 positions in every one of the 16 cached layers (1.14 GB of Q8_0 blocks)
    P = 32768
    kv = bb.KVCache(P)
    try:
        chunk = 4096
        kk = torch.randn(chunk, 4, 256, generator=g).cuda()
        vv = torch.randn(chunk, 4, 256, generator=g).cuda()

        def fill():
            for layer in range(16):
                for p0 in range(0, P, chunk):
                    assert kv.append_batch(layer, p0, chunk, kk, vv) == 0
        # bytes that must move: fp32 rows in (2 x 4 x 256 x 4 per position), Q8_0 blocks out (2 x 4 x 272)
        out["kv_append_16x32768"] = rate(fill, 16 * P * (2 * 4 * 256 * 4 + 2 * 4 * 272), 16 * (P // chunk), steps=2)
        qd = torch.randn(24, 256, generator=g).cuda()
        od = torch.empty(24, 256, device="cuda")

        def decode():
            for layer in range(16):
                assert kv.attn_decode(layer, P - 1, qd, od) == 0
        out["kv_attn_decode_16_layers_at_32768"] = rate(decode, 16 * P * 2 * 4 * 272, 32)
    finally:
        kv.close()
    # load-time steps on 5120 x 17408 x 8 copies (190 MB of PQ2_0): repack (read + write), PTQ1_0 pack and unpack
    n_in, n_out, copies = 5120, 17408, 8
    nblk = n_out * (n_in // 128) * copies
    W = torch.empty(nblk * 34, dtype=torch.uint8, device="cuda")
    assert bb.synth_pq2_0(W, 0, nblk, args.seed + 5) == 0
    Wr = torch.empty_like(W)
    out["repack_5120x17408x8"] = rate(lambda: bb.repack(W, Wr, n_out * copies, n_in), 2 * nblk * 34, 1)
    Pk = torch.empty(nblk * 28, dtype=torch.uint8, device="cuda")
    c3 = torch.zeros(1, dtype=torch.int64, device="cuda")
    out["ptq1_pack"] = rate(lambda: bb.ptq1_pack(W, Pk, nblk, c3), nblk * (34 + 28), 1)
    out["ptq1_unpack"] = rate(lambda: bb.ptq1_unpack(Pk, Wr, nblk), nblk * (34 + 28), 1)
    return {"metric": "rows_beside_the_path", "peak_GB/s": peak, "peak_kind": kind, "rows": out,
            "gpu_launches": sum(v["gpu_launches"] for v in out.values()), "device_status": bb.device_status()}


# ---- row-partitioned small batch -----------------------------------------------------------------------
def batch_leg(args, torch, bb, dist, n_tok=8):
    """The two large projections (5120 -> 17408, 17408 -> 5120) with a batch of n_tok activation vectors: every rank
    multiplies its row slice through bonsai_p40_gemm (2 .. 16 tokens: the kernel that streams the weights once for all
    tokens; more: the tensor cores), an NCCL all-gather assembles Y[n_out][n_tok].  `--sets` copies of each matrix are
    resident.  Reports weight GB/s (weight bytes of all launches / time) and token-weight GB/s (x n_tok).  Parity: the assembled Y of the last sweep
    against the same entry point on the unsplit matrix, bit for bit (a row's sum does not depend on the split)."""
    from bonsai_b200 import partition
    rank, world, local = env_ranks()
    if dist is None:
        world, rank = 1, 0
    shapes = [(5120, 17408), (17408, 5120)]
    mats, total_w, first = [], 0, 0
    for s_ in range(args.sets):
        for n_in, n_out in shapes:
            lo, hi = partition.row_slice(n_out, rank, world)
            nblk_row = n_in // 128
            W = torch.empty((hi - lo) * nblk_row * 34, dtype=torch.uint8, device="cuda")
            assert bb.synth_pq2_0(W, first + lo * nblk_row, (hi - lo) * nblk_row, args.seed + 17) == 0
            mats.append((n_in, n_out, lo, hi, W, first))
            first += n_out * nblk_row
            total_w += n_out * nblk_row * 34
    g = torch.Generator(device="cpu").manual_seed(args.seed + 8)
    Xq = {}
    for n_in in sorted({a for a, _ in shapes}):
        X = torch.randn(n_tok, n_in, generator=g).cuda()
        Xq[n_in] = torch.empty(n_in // 32 * n_tok * 36, dtype=torch.uint8, device="cuda")
        assert bb.quant_batch(X, None, Xq[n_in], n_in, n_tok, True) == 0
    Y = {n_out: torch.zeros(n_out, n_tok, device="cuda") for _, n_out in shapes}

    def sweep():
        for n_in, n_out, lo, hi, W, _ in mats:
            assert bb.gemm(W, Xq[n_in], Y[n_out][lo:hi], hi - lo, n_in, n_tok) == 0
            if world > 1:
                dist.all_gather_into_tensor(Y[n_out], Y[n_out][lo:hi])

    steps = max(3, min(args.steps, 50))
    ms, reps, _ = timed(torch, sweep, steps, 3, dist, None, True)
    us = ms * 1e3 / (steps * reps)
    gbs = total_w / (us * 1e-6) / 1e9
    bad, worst = 0, 0.0
    torch.cuda.synchronize()
    for n_in, n_out, lo, hi, W, first_blk in mats[-2:]:             # the copies the last sweep left in Y
        nblk = n_out * (n_in // 128)
        Wf = torch.empty(nblk * 34, dtype=torch.uint8, device="cuda")
        assert bb.synth_pq2_0(Wf, first_blk, nblk, args.seed + 17) == 0
        want = torch.zeros(n_out, n_tok, device="cuda")
        assert bb.gemm(Wf, Xq[n_in], want, n_out, n_in, n_tok) == 0
        if not torch.equal(Y[n_out].view(torch.int32), want.view(torch.int32)):
            bad += 1
            worst = max(worst, float((Y[n_out] - want).abs().max().item()))
    if dist is not None:
        t = torch.tensor([bad, worst], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        bad, worst = int(t[0].item()), float(t[1].item())
    peak, _, kind = measured_peaks()
    kernels_per_call = 1 if n_tok <= 16 else 3      # streaming kernel; tensor cores: two launches prepare the fp16 planes
    return {"metric": f"pq2_0_gemm_batch{n_tok}_weight_stream", "value": gbs, "unit": UNIT, "n_tok": n_tok, "us_per_sweep": us,
            "token_weight_gbs": gbs * n_tok, "gpu_launches": len(mats) * steps * reps * kernels_per_call,
            "frac": gbs / world / peak, "peak_kind": kind, "resident_weight_bytes": total_w,
            "call": f"bonsai_p40_gemm ({n_tok} tokens) per matrix slice" + (" + NCCL all-gather" if world > 1 else ""),
            "parity": {"checked": 2, "mismatches": bad, "max_abs": worst,
                       "against": "bonsai_p40_gemm on the unsplit matrix, bit for bit, every rank"},
            "device_status": bb.device_status()}


def run_single(args):
    """One shape, `--copies` distinct weight tensors, one plain launch per copy: the command the ncu
    captures under profiles/ are taken with (nothing is timed here)."""
    import torch
    import bonsai_b200 as bb
    n_in, n_out = args.single
    torch.cuda.set_device(0)
    bb.lib()
    bb.set_option("pdl", max(args.pdl, 0))
    if args.order >= 0:
        bb.set_option("gemv_order", args.order)
    nblk = n_out * (n_in // 128)
    Ws = []
    for c in range(args.copies):
        W = torch.empty(nblk * 34, dtype=torch.uint8, device="cuda")
        assert bb.synth_pq2_0(W, c * nblk, nblk, args.seed) == 0
        Ws.append(W)
    x = torch.randn(n_in, device="cuda")
    xq = torch.empty(n_in // 32 * 36, dtype=torch.uint8, device="cuda")
    y = torch.empty(n_out, device="cuda")
    assert bb.fwht_quant(x, None, xq, None, n_in) == 0
    torch.cuda.synchronize()
    for W in Ws:
        assert bb.gemv(W, xq, y, n_out, n_in) == 0
    torch.cuda.synchronize()
    print(json.dumps({"single": [n_in, n_out], "copies": args.copies, "device_status": bb.device_status()}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--sets", type=int, default=8)
    ap.add_argument("--workload", default="layer_sweep", choices=["layer_sweep", "decode_step", "prefill"],
                    help="layer_sweep (default, the headline metric), decode_step (401 mat-vecs of one token), "
                         "prefill (512-token mat-mul)")
    ap.add_argument("--call", default="list", choices=["list", "matrix"],
                    help="list (default): a sweep's mat-vecs as one persistent launch (bonsai_b200_chain_run); "
                         "matrix: one bonsai_p40_gemv launch per matrix")
    ap.add_argument("--gather", default="auto", choices=["auto", "peer", "nccl"],
                    help="N > 1, list mode: nccl = one all-gather per sweep; peer = the kernel stores its outputs into "
                         "every rank's buffer (CUDA IPC mapping, no collective); auto = both are timed at start-up on the "
                         "box the benchmark runs on and the faster one is used for `value` and `e2e`")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--pdl", type=int, default=1, help="0 plain launches, 1 programmatic launches (weights of the next "
                    "mat-vec stream while the previous kernel drains)")
    ap.add_argument("--cpu-seconds", type=float, default=8.0)
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="skip the decode-step / prefill / repack legs of the default line")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from Python instead of replaying a graph")
    ap.add_argument("--single", type=int, nargs=2, metavar=("N_IN", "N_OUT"), help="profiling aid: launch one shape only")
    ap.add_argument("--copies", type=int, default=8)
    ap.add_argument("--gemm-path", type=int, default=-1, help="prefill workload: -1 default kernel choice, 3 the integer "
                    "tensor-core kernel, 0 the integer SIMT kernel (bonsai_b200_set_option gemm_path)")
    ap.add_argument("--opt", action="append", default=[], metavar="KEY=VALUE",
                    help="bonsai_b200_set_option(KEY, VALUE) before anything is built; may be given several times")
    ap.add_argument("--order", type=int, default=-1, help="1: the mat-vec that keeps the host's summation order")
    args = ap.parse_args()
    if args.single:
        return run_single(args)
    if args.impl == "reference":
        return run_reference(args)
    if args.workload == "decode_step":
        return run_decode_step(args)
    if args.workload == "prefill":
        return run_prefill(args)
    run_b200(args)


if __name__ == "__main__":
    main()
