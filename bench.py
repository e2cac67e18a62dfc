#!/usr/bin/env python
"""Benchmark of the PQ2_0 decode mat-vec on B200, one JSON line per run.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--sets S]

Workload ("layer_sweep"): the batch-1 projection shapes of one transformer layer,
n_in x n_out = 5120x5120, 5120x1024, 5120x17408, 17408x5120, PQ2_0 weights with the checkpoint's
code distribution, Q8_1 activations from FWHT-rotated N(0,1) vectors.  `--sets S` independent copies
of the four matrices are resident in HBM (S = 8 -> 446 MB, larger than the 126 MB L2) and a step is
one pass over all of them, so every launch streams its weights from HBM.

value   : PQ2_0 weight bytes of all launches / device time (CUDA events, max over ranks), GB/s.
--call  : "list" (default) hands the step's mat-vecs to bonsai_b200_chain_run, ONE persistent launch that
          streams the matrices back to back; "matrix" calls bonsai_p40_gemv once per matrix (the
          reference's ABI unchanged).  In list mode the per-matrix figure is measured too and
          reported under "per_matrix_abi".
e2e     : the same metric with HOST buffers: the step's fp32 activation vectors are copied from
          pinned host memory (one block), rotated + quantised (one call) + multiplied through the C
          ABI, and the outputs are copied back, all inside the timed region.  Weights stay resident
          (they are model state).
roofline: algorithmic bytes (weights + Q8_1 vectors + fp32 outputs) of a launch / its duration,
          against the measured HBM copy bandwidth.
N > 1   : every matrix is split by output rows over the ranks; each rank multiplies its slices and
          an NCCL all-gather assembles the outputs (strong scaling: the total work is fixed).
--impl reference : the reference's own host implementation of the same path on this box's CPU
          cores (oracle/_ref when it was built, else the C restatement in oracle/).
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "p40-kernel_b200"))

LAYER_SHAPES = [(5120, 5120), (5120, 1024), (5120, 17408), (17408, 5120)]   # (n_in, n_out)
METRIC = "pq2_0_gemv_weight_stream"
UNIT = "GB/s"


def weight_bytes(n_in, n_out):
    return n_out * (n_in // 128) * 34


def algorithmic_bytes(n_in, n_out):
    return weight_bytes(n_in, n_out) + (n_in // 32) * 36 + 4 * n_out


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


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
            time.sleep(0.005)

    def result(self):
        self.stop_flag.set()
        self.join(timeout=2)
        if not self.sm:
            return {"sm_mhz": None, "sm_max_mhz": self.max_sm, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(self.sm), "sm_max_mhz": self.max_sm, "reasons": sorted(self.reasons),
                "samples": len(self.sm)}


# ---------------------------------------------------------------------------------------------------
def cpu_arm(args, threads):
    """Times the CPU checker on one layer sweep (FWHT + quantise + mat-vec per shape)."""
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
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    kind, sweep, wbytes = cpu_arm(args, threads)
    for _ in range(max(1, min(args.warmup, 3))):
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
        "warmup": min(args.warmup, 3), "ms_per_step": dt / steps * 1e3, "higher_is_better": True,
        "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "int8xint2->int32, fp32 scale",
        "data": "synthetic", "config": {"workload": "layer_sweep", "shapes_nin_nout": LAYER_SHAPES, "batch": 1},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ---------------------------------------------------------------------------------------------------
def run_b200(args):
    import torch
    import bonsai_b200 as bb
    from bonsai_b200 import partition

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
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
    if args.variant >= -1:
        bb.set_option("gemv_variant", args.variant)
    if args.order >= 0:
        bb.set_option("gemv_order", args.order)

    sets = args.sets
    # ---- resident tensors: weights generated on the device, row slice of this rank only ----------
    mats = []
    blk_base = 0
    for s in range(sets):
        for n_in, n_out in LAYER_SHAPES:
            r_lo, r_hi = partition.row_slice(n_out, rank, world)
            rows = r_hi - r_lo
            nblk_row = n_in // 128
            W = torch.empty(rows * nblk_row * 34, dtype=torch.uint8, device="cuda")
            first = blk_base + rank * rows * nblk_row
            assert bb.synth_pq2_0(W, first, rows * nblk_row, args.seed) == 0
            blk_base += n_out * nblk_row
            y = torch.zeros(n_out, dtype=torch.float32, device="cuda")
            mats.append((n_in, n_out, rows, W, y))
    xq = {}
    xdev = {}
    for n_in in sorted({a for a, _ in LAYER_SHAPES}):
        g = torch.Generator(device="cpu").manual_seed(args.seed + n_in)
        xh = torch.randn(n_in, generator=g, dtype=torch.float32)
        xdev[n_in] = xh.cuda()
        xq[n_in] = torch.empty(n_in // 32 * 36, dtype=torch.uint8, device="cuda")
        assert bb.fwht_quant(xdev[n_in], None, xq[n_in], None, n_in) == 0
    torch.cuda.synchronize()

    use_list = args.call == "list"

    def step_matrix():
        n = 0
        for n_in, n_out, rows, W, y in mats:
            ys = y[rank * rows:(rank + 1) * rows]
            rc = bb.gemv(W, xq[n_in], ys, rows, n_in)
            n += 1
            if world > 1:
                dist.all_gather_into_tensor(y, ys)
        return n

    # host buffers for the end-to-end leg: one pinned block with every activation vector of a step,
    # one pinned block for every output of a step (one copy each way per step)
    x_off, off = [], 0
    for n_in, n_out, rows, W, y in mats:
        x_off.append(off)
        off += n_in
    pin_x = torch.empty(off, dtype=torch.float32).pin_memory()
    for (n_in, *_), o in zip(mats, x_off):
        pin_x[o:o + n_in] = xdev[n_in].cpu()
    dev_x = torch.empty(off, dtype=torch.float32, device="cuda")
    y_all = torch.zeros(sum(m[1] for m in mats), dtype=torch.float32, device="cuda")
    pin_y = torch.empty(y_all.numel(), dtype=torch.float32).pin_memory()
    y_off, off = [], 0
    for m in mats:
        y_off.append(off)
        off += m[1]
    xq_e2e = [torch.empty(m[0] // 32 * 36, dtype=torch.uint8, device="cuda") for m in mats]

    # list mode: the whole step is ONE launch of the persistent kernel (bonsai_b200_chain_run); with
    # several ranks every rank multiplies its row slices and one all-gather moves all of them
    # (rank-major: gathered[r] holds rank r's slice of every matrix, in matrix order)
    slice_off, off = [], 0
    for m in mats:
        slice_off.append(off)
        off += m[2]
    y_local = torch.zeros(off, dtype=torch.float32, device="cuda")
    y_gathered = torch.zeros(world * off, dtype=torch.float32, device="cuda") if world > 1 else None
    chain = chain_e2e = chain_tp = peer_buf = None
    gather = args.gather if args.gather != "auto" else ("peer" if world >= 4 else "nccl")
    if args.gather == "auto" and gather == "peer":
        try:                                    # the peer mapping needs the CUDA runtime bindings (same on every rank)
            import cuda.bindings.runtime       # noqa: F401
        except Exception:
            gather = "nccl"
    if use_list and world > 1 and gather == "peer":
        # the gathered outputs live in a buffer that every rank has mapped (CUDA IPC): the kernel's epilogue stores
        # each y element into every rank's copy, so there is no collective at all
        from bonsai_b200.peer import PeerBuffer
        peer_buf = PeerBuffer(world * off * 4, dist, rank, world)
        y_peer = peer_buf.tensor.view(torch.float32)
        chain_tp = bb.Chain([(W, xq[n_in], None, y_peer[rank * off + o:rank * off + o + rows], rows, n_in,
                              bb.OP_SAME_INPUT if i and mats[i - 1][0] == n_in else 0)
                             for i, ((n_in, n_out, rows, W, y), o) in enumerate(zip(mats, slice_off))], peers=peer_buf)
    if use_list:
        # consecutive matrices that read the same resident Q8_1 vector say so (its shared-memory copy is reused)
        chain = bb.Chain([(W, xq[n_in], None, y_local[o:o + rows], rows, n_in,
                           bb.OP_SAME_INPUT if i and mats[i - 1][0] == n_in else 0)
                          for i, ((n_in, n_out, rows, W, y), o) in enumerate(zip(mats, slice_off))])
        # end to end: the step's activation vectors arrive as one host block; FWHT-1024 and the quantiser
        # work on 1024- and 32-element blocks, so ONE bonsai_b200_fwht_quant call over the concatenation
        # rotates and quantises every vector (vector i's Q8_1 blocks start at byte x_off[i] / 32 * 36)
        xq_all = torch.empty(dev_x.numel() // 32 * 36, dtype=torch.uint8, device="cuda")
        chain_e2e = bb.Chain([(W, xq_all[xo // 32 * 36:(xo + n_in) // 32 * 36], None, y_local[o:o + rows], rows, n_in, 0)
                              for (n_in, n_out, rows, W, y), o, xo in zip(mats, slice_off, x_off)])

    def step_list():
        if chain_tp is not None:
            assert chain_tp.run() == 0
            return 1
        assert chain.run() == 0
        if world > 1:
            dist.all_gather_into_tensor(y_gathered, y_local)
        return 1

    def step_list_e2e():
        dev_x.copy_(pin_x, non_blocking=True)
        assert bb.fwht_quant(dev_x, None, xq_all, None, dev_x.numel()) == 0
        assert chain_e2e.run() == 0
        if world > 1:
            dist.all_gather_into_tensor(y_gathered, y_local)
            pin_y.copy_(y_gathered, non_blocking=True)
        else:
            pin_y.copy_(y_local, non_blocking=True)
        return 1

    def e2e_pipelined(steps, warmup):
        """The end-to-end step on three streams with two buffer sets: step i's host->device copy, its
        launches and its device->host copy run on their own streams, ordered by events, so that the
        copies of neighbouring steps overlap the mat-vecs (every step still copies its inputs in and its
        outputs out inside the timed region).  One GPU, list mode."""
        s_in, s_k, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        dx = [dev_x, torch.empty_like(dev_x)]
        xa = [xq_all, torch.empty_like(xq_all)]
        yl = [y_local, torch.zeros_like(y_local)]
        py = [pin_y, torch.empty_like(pin_y).pin_memory()]
        chains = [chain_e2e,
                  bb.Chain([(W, xa[1][xo // 32 * 36:(xo + n_in) // 32 * 36], None, yl[1][o:o + rows], rows, n_in, 0)
                            for (n_in, n_out, rows, W, y), o, xo in zip(mats, slice_off, x_off)])]
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_k = [torch.cuda.Event() for _ in range(2)]
        ev_out = [torch.cuda.Event() for _ in range(2)]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()

        def run(n, first):
            for i in range(first, first + n):
                b = i & 1
                with torch.cuda.stream(s_in):
                    if i >= 2:
                        s_in.wait_event(ev_k[b])            # the launches of step i - 2 have read this input buffer
                    dx[b].copy_(pin_x, non_blocking=True)
                    ev_in[b].record(s_in)
                with torch.cuda.stream(s_k):
                    s_k.wait_event(ev_in[b])
                    if i >= 2:
                        s_k.wait_event(ev_out[b])           # step i - 2's outputs have left this buffer
                    assert bb.fwht_quant(dx[b], None, xa[b], None, dx[b].numel()) == 0
                    assert chains[b].run() == 0
                    ev_k[b].record(s_k)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_k[b])
                    py[b].copy_(yl[b], non_blocking=True)
                    ev_out[b].record(s_out)
        run(4, 0)
        torch.cuda.synchronize()
        if args.no_graph:
            e0.record(s_in)
            run(steps, 0)
            s_out.wait_stream(s_in)
            s_out.wait_stream(s_k)
            e1.record(s_out)
            torch.cuda.synchronize()
            return e0.elapsed_time(e1), steps
        # eight steps per graph (the three streams fork from and join the capturing stream); replays serialise,
        # so one step in eight starts without a neighbour to overlap with
        per_graph = 8
        graph, cap = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        with torch.cuda.graph(graph, stream=cap):
            for st in (s_in, s_k, s_out):
                st.wait_stream(cap)
            run(per_graph, 0)
            for st in (s_in, s_k, s_out):
                cap.wait_stream(st)
        replays = max(1, steps // per_graph)
        for _ in range(max(1, warmup // per_graph)):
            graph.replay()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(replays):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1), replays * per_graph

    def step_e2e():
        n = 0
        dev_x.copy_(pin_x, non_blocking=True)
        for i, (n_in, n_out, rows, W, y) in enumerate(mats):
            xi = dev_x[x_off[i]:x_off[i] + n_in]
            yo = y_all[y_off[i]:y_off[i] + n_out]
            ys = yo[rank * rows:(rank + 1) * rows]
            bb.linear(W, xi, None, ys, xq_e2e[i], rows, n_in)       # rotation + quantiser + mat-vec, one kernel
            n += 1
            if world > 1:
                dist.all_gather_into_tensor(yo, ys)
        pin_y.copy_(y_all, non_blocking=True)
        return n

    def timed(step_fn, steps, warmup, sample_clocks):
        """Captures one step in a CUDA graph (launch overhead of ~30 small kernels would otherwise
        dominate), replays it `warmup` then `steps` times, and times the replays on the device."""
        per_step = step_fn()                      # eager once: validates return path, warms caches
        torch.cuda.synchronize()
        run = step_fn
        if not args.no_graph:
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side):
                    step_fn()
            torch.cuda.current_stream().wait_stream(side)
            run = graph.replay
        for _ in range(warmup):
            run()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()
        sampler = ClockSampler(local) if sample_clocks else None
        if sampler:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            run()
        e1.record()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        clocks = sampler.result() if sampler else None
        if dist is not None:
            t = torch.tensor([ms], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, per_step * steps, clocks

    total_w = sum(weight_bytes(a, b) for a, b in LAYER_SHAPES) * sets
    total_alg = sum(algorithmic_bytes(a, b // world) for a, b in LAYER_SHAPES) * sets
    ms, launches, clocks = timed(step_list if use_list else step_matrix, args.steps, args.warmup, True)
    value = total_w * args.steps / (ms * 1e-3) / 1e9
    e2e_steps = max(1, args.steps // 4)
    ms_e, _, _ = timed(step_list_e2e if use_list else step_e2e, e2e_steps, max(3, args.warmup // 4), False)
    e2e_value = total_w * e2e_steps / (ms_e * 1e-3) / 1e9
    e2e_mode, e2e_serial = "one stream: copy in, launches, copy out, in order", None
    if use_list and world == 1:
        ms_p, steps_p = e2e_pipelined(e2e_steps, max(8, args.warmup // 4))
        e2e_serial = e2e_value
        e2e_value = total_w * steps_p / (ms_p * 1e-3) / 1e9
        e2e_mode = "three streams, two buffer sets: the copies of neighbouring steps overlap the launches"
    per_matrix = None
    if use_list:        # the unchanged per-matrix ABI on the same tensors, for comparison
        ms_m, launches_m, _ = timed(step_matrix, e2e_steps, max(3, args.warmup // 4), False)
        per_matrix = {"call": "bonsai_p40_gemv per matrix", "value": total_w * e2e_steps / (ms_m * 1e-3) / 1e9,
                      "unit": UNIT, "ms_per_step": ms_m / e2e_steps, "gpu_launches_per_step": launches_m // e2e_steps}
    split = None
    if use_list and world > 1 and chain_tp is None:      # where the step's time goes: the mat-vec launch alone, the all-gather alone
        def only_matvec():
            assert chain.run() == 0
            return 1

        def only_gather():
            dist.all_gather_into_tensor(y_gathered, y_local)
            return 1
        ms_k, _, _ = timed(only_matvec, e2e_steps, 3, False)
        ms_g, _, _ = timed(only_gather, e2e_steps, 3, False)
        split = {"matvec_ms_per_step": ms_k / e2e_steps, "allgather_ms_per_step": ms_g / e2e_steps,
                 "allgather_bytes_per_rank": int(y_local.numel() * 4)}
    status = bb.device_status()
    launches_per_step = launches // args.steps

    peak, peak_kind = measured_peak_gbs()
    traffic = None
    try:        # DRAM bytes per launch from the committed ncu capture, scaled by the bytes a launch streams
        t = json.load(open(os.path.join(ROOT, "profiles", "gemv_chain_traffic.json" if use_list else "gemv_stream_traffic.json")))
        traffic = t["dram_bytes_per_launch"] / t["algorithmic_bytes_per_launch"] * (total_alg / launches_per_step)
    except Exception:
        pass
    achieved = total_alg * args.steps / (ms * 1e-3) / 1e9     # per-rank algorithmic bytes / per-launch time
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong" if world > 1 else "weak",
        "vs_baseline": None, "dtype": "int8xint2->int32, fp32 scale", "data": "synthetic",
        "config": {"workload": "layer_sweep", "shapes_nin_nout": LAYER_SHAPES, "batch": 1, "sets": sets,
                   "resident_weight_bytes": total_w, "l2": "inputs larger than L2" if total_w > 126e6 else "fits L2",
                   "parallelism": ("single" if world == 1 else f"rows/{world}, outputs stored into every rank's buffer by the "
                                   "kernel (peer-mapped memory, no collective)" if chain_tp is not None
                                   else f"rows/{world}+allgather"), "pdl": args.pdl,
                   "fp32_order": "host-sequential" if args.order == 1 else "fixed-tree", "variant": args.variant,
                   "launch": "eager" if args.no_graph else "cuda_graph_per_step",
                   "call": "bonsai_b200_chain_run: the step's mat-vecs as one persistent launch" if use_list
                           else "bonsai_p40_gemv per matrix"},
        "gpu_launches": launches,
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": UNIT,
                "h2d_bytes_per_step": int(pin_x.numel() * 4), "d2h_bytes_per_step": int(pin_y.numel() * 4),
                "mode": e2e_mode, "one_stream_value": e2e_serial},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": UNIT, "frac": achieved / peak,
                     "peak_kind": peak_kind, "traffic": traffic,
                     "avg_launch_us": ms * 1e3 / max(1, launches),
                     "algorithmic_bytes_per_launch_avg": total_alg / launches_per_step},
        "device_status": status,
    }
    if per_matrix is not None:
        line["per_matrix_abi"] = per_matrix
    if split is not None:
        line["split"] = split
    if world == 1 and not args.no_cpu:
        threads = os.cpu_count() or 1
        kind, sweep, wbytes = cpu_arm(args, threads)
        sweep()
        reps, t0 = 0, time.perf_counter()
        while time.perf_counter() - t0 < args.cpu_seconds:
            sweep()
            reps += 1
        dt = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": wbytes * reps / dt / 1e9, "unit": UNIT, "cores": threads, "kind": kind,
                                "sample": f"{reps} layer sweeps (4 mat-vecs each, FWHT+Q8_1 included) in {dt:.1f} s"}
        _, sweep1, _ = cpu_arm(args, 1)             # the same code on one host thread
        t0 = time.perf_counter()
        sweep1()
        dt1 = time.perf_counter() - t0
        line["cpu_baseline"]["single_thread"] = {"value": wbytes / dt1 / 1e9, "unit": UNIT,
                                                 "sample": f"1 layer sweep in {dt1:.2f} s"}
    if rank == 0:
        print(json.dumps(line))
    if peer_buf is not None:
        chain_tp.close()
        peer_buf.close(dist)
    if dist is not None:
        dist.destroy_process_group()


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


def _graph_time(torch, fn, steps, warmup):
    fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(warmup):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def run_decode_step(args):
    """BASELINE config 2: the 401 projections of one decoded token, each the rotation + Q8_1 quantiser of a
    resident fp32 vector of its input width followed by the mat-vec (the values do not flow from one
    projection to the next; the waits do), replayed as one CUDA graph.  Reports tokens/s and weight GB/s.
    With N > 1 every matrix is split by output rows and every projection is followed by the all-gather of
    its output (per-matrix calls: a list launch cannot span a collective, and one launch per group of
    projections that share an input measured slower, 82 against 127 tokens/s at N = 2)."""
    import torch
    import bonsai_b200 as bb
    from bonsai_b200 import partition
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    bb.lib()
    bb.set_option("pdl", max(args.pdl, 0))
    shapes = model_gemvs()
    ws, rows_of, first = [], [], 0
    for n_in, n_out in shapes:
        lo, hi = partition.row_slice(n_out, rank, world)
        nblk_row = n_in // 128
        W = torch.empty((hi - lo) * nblk_row * 34, dtype=torch.uint8, device="cuda")
        assert bb.synth_pq2_0(W, first + lo * nblk_row, (hi - lo) * nblk_row, args.seed) == 0
        first += n_out * nblk_row
        ws.append(W)
        rows_of.append(hi - lo)
    g = torch.Generator(device="cpu").manual_seed(args.seed)
    xs = {k: torch.randn(k, generator=g).cuda() for k in sorted({a for a, _ in shapes})}
    xq = {k: torch.empty(k // 32 * 36, dtype=torch.uint8, device="cuda") for k in xs}
    ys = {n: torch.empty(n, device="cuda") for n in {b for _, b in shapes}}

    launches_per_token = len(shapes)
    peer_buf = None
    peer_ok = args.gather == "peer"
    if args.gather == "auto":
        try:
            import cuda.bindings.runtime       # noqa: F401
            peer_ok = True
        except Exception:
            peer_ok = False
    if args.call == "list" and world > 1 and peer_ok:
        # one launch per token and rank: every rank multiplies its rows of every projection and stores them into
        # every rank's copy of the output vectors; a projection that waits, waits for the rows of every rank
        from bonsai_b200.peer import PeerBuffer
        outs = sorted({b for _, b in shapes})
        base, off = {}, 0
        for n in outs:
            base[n] = off
            off += n
        peer_buf = PeerBuffer(off * 4, dist, rank, world)
        y_peer = peer_buf.tensor.view(torch.float32)
        ops, prev = [], None
        for i, ((n_in, n_out), W) in enumerate(zip(shapes, ws)):
            r = rows_of[i]
            fl = bb.OP_ROTATE | (bb.OP_SAME_INPUT if prev == n_in and i else (bb.OP_DEPENDS if i else 0))
            ops.append((W, xs[n_in], None, y_peer[base[n_out] + rank * r:base[n_out] + (rank + 1) * r], r, n_in, fl))
            prev = n_in
        chain = bb.Chain(ops, peers=peer_buf)
        launches_per_token = 1

        def token():
            assert chain.run() == 0
    elif args.call == "list" and world == 1:
        # one launch per token: projections that read the same vector share its quantised form, every
        # other projection waits for all rows of the projections before it (its input is an output
        # of the step in the real model; here the values do not flow, the waits do)
        ops, prev = [], None
        for i, ((n_in, n_out), W) in enumerate(zip(shapes, ws)):
            fl = bb.OP_ROTATE | (bb.OP_SAME_INPUT if prev == n_in and i else (bb.OP_DEPENDS if i else 0))
            ops.append((W, xs[n_in], None, ys[n_out], n_out, n_in, fl))
            prev = n_in
        chain = bb.Chain(ops)
        launches_per_token = 1

        def token():
            assert chain.run() == 0
    else:
        def token():
            for i, ((n_in, n_out), W) in enumerate(zip(shapes, ws)):
                r = rows_of[i]
                ysl = ys[n_out][rank * r:(rank + 1) * r]
                bb.linear(W, xs[n_in], None, ysl, xq[n_in], r, n_in)    # rotation + quantiser + mat-vec
                if world > 1:
                    dist.all_gather_into_tensor(ys[n_out], ysl)

    steps = max(3, min(args.steps, 50))
    warm = max(3, min(args.warmup, 5))
    sampler = ClockSampler(local)
    sampler.start()
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
    ms = _graph_time(torch, token, steps, warm)
    clocks = sampler.result()
    if dist is not None:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    wbytes = sum(weight_bytes(a, b) for a, b in shapes)
    peak, peak_kind = measured_peak_gbs()
    gbs = wbytes / (ms * 1e-3) / 1e9
    status = bb.device_status()
    if rank == 0:
        call = ("bonsai_b200_chain_run, one launch per token" + (" and rank, outputs stored into every rank's buffer "
                "by the kernel" if world > 1 else "") if launches_per_token == 1 else
                "bonsai_b200_linear per matrix" + (", then an all-gather" if world > 1 else ""))
        print(json.dumps({
            "metric": "decode_tokens_per_s", "value": 1e3 / ms, "unit": "tokens/s", "n_gpus": world, "steps": steps,
            "warmup": warm, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong" if world > 1 else "weak",
            "vs_baseline": None, "dtype": "int8xint2->int32, fp32 scale", "data": "synthetic",
            "config": {"workload": "decode_step", "matvecs": len(shapes), "weight_bytes": wbytes, "batch": 1, "pdl": args.pdl,
                       "l2": "inputs larger than L2", "launch": "cuda_graph_per_step", "call": call,
                       "parallelism": ("single" if world == 1 else f"rows/{world}, peer stores in the kernel" if peer_buf is not None
                                       else f"rows/{world}+allgather")},
            "gpu_launches": launches_per_token * steps, "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": gbs / world, "peak": peak, "unit": "GB/s", "frac": gbs / world / peak,
                         "peak_kind": peak_kind, "traffic": None},
            "device_status": status}))
    if peer_buf is not None:
        chain.close()
        peer_buf.close(dist)
    if dist is not None:
        dist.destroy_process_group()


def run_prefill(args):
    """BASELINE config 3: M = 512 tokens through the two large projections; a step = token-batch rotation +
    quantiser into the chunk-major layout, then the tensor-core mat-mul, for both matrices."""
    import torch
    import bonsai_b200 as bb
    torch.cuda.set_device(0)
    bb.lib()
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

    def step():
        for n_in, n_out, W, X, Xq, Y in mats:
            assert bb.quant_batch(X, None, Xq, n_in, n_tok, True) == 0
            assert bb.gemm(W, Xq, Y, n_out, n_in, n_tok) == 0

    steps = max(3, min(args.steps, 30))
    sampler = ClockSampler(0)
    sampler.start()
    ms = _graph_time(torch, step, steps, max(3, min(args.warmup, 5)))
    clocks = sampler.result()
    ops = sum(2.0 * n_tok * a * b for a, b, *_ in mats)
    tops = ops / (ms * 1e-3) / 1e12
    try:
        bf16 = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"])
        peak, kind = 2.0 * bf16, "2 x measured dense bf16"
    except Exception:
        peak, kind = 2.0 * 1590.0, "2 x fallback dense bf16"
    # a dense int8 figure measured here, for reference beside the denominator above: the library's int8
    # mat-mul (cuBLASLt through torch._int_mm) on 8192^3, best of 10 -- a measuring stick, not on the path
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
    print(json.dumps({
        "metric": "pq2_0_prefill_gemm", "value": tops, "unit": "TOPS", "n_gpus": 1, "steps": steps,
        "warmup": max(3, min(args.warmup, 5)), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8 x int8 -> int32 (tcgen05), fp32 scale", "data": "synthetic",
        "config": {"workload": "prefill", "n_tok": n_tok, "shapes_nin_nout": [[5120, 17408], [17408, 5120]],
                   "launch": "cuda_graph_per_step"},
        "gpu_launches": 4 * steps, "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": tops, "peak": peak, "unit": "TOPS", "frac": tops / peak,
                     "peak_kind": kind, "traffic": None, "library_int8_dense_tops_measured": int8_lib},
        "device_status": bb.device_status()}))


def run_single(args):
    """One shape, `--copies` distinct weight tensors, one plain launch per copy: the command the ncu
    captures under profiles/ are taken with (nothing is timed here)."""
    import torch
    import bonsai_b200 as bb
    n_in, n_out = args.single
    torch.cuda.set_device(0)
    bb.lib()
    bb.set_option("pdl", max(args.pdl, 0))
    if args.variant >= -1:
        bb.set_option("gemv_variant", args.variant)
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
                    help="list (default): the step's mat-vecs as one persistent launch (bonsai_b200_chain_run); "
                         "matrix: one bonsai_p40_gemv launch per matrix")
    ap.add_argument("--gather", default="auto", choices=["auto", "peer", "nccl"],
                    help="N > 1, list mode: nccl = one all-gather per step; peer = the kernel stores its outputs into "
                         "every rank's buffer (CUDA IPC mapping, no collective); auto = what measured faster: peer for "
                         "the decode step and for the layer sweep at N >= 4, nccl for the layer sweep at N = 2")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--pdl", type=int, default=1, help="0 plain launches, 1 programmatic launches (weights of the next "
                    "mat-vec stream while the previous kernel drains)")
    ap.add_argument("--variant", type=int, default=-2, help="-2 leave the library default")
    ap.add_argument("--cpu-seconds", type=float, default=8.0)
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from Python instead of replaying a graph")
    ap.add_argument("--single", type=int, nargs=2, metavar=("N_IN", "N_OUT"), help="profiling aid: launch one shape only")
    ap.add_argument("--copies", type=int, default=8)
    ap.add_argument("--order", type=int, default=-1, help="1: the mat-vec that keeps the host's summation order")
    args = ap.parse_args()
    if args.single:
        return run_single(args)
    if args.workload == "decode_step" and args.impl == "b200":
        return run_decode_step(args)
    if args.workload == "prefill" and args.impl == "b200":
        return run_prefill(args)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
