"""Worker of test_gpu_tp.py: one process per GPU (torch.distributed.run), a list with dependent, shared-input and
Q8_1 ops over row slices, outputs stored into every rank's buffer by the kernel; every rank compares every full
output vector with the per-matrix entry points on the unsplit matrices, bit for bit, and sampled rows of every op
with the CPU checker (1e-5 of the largest output)."""
import os, sys
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT); sys.path.insert(0, os.path.join(ROOT, "p40-kernel_b200"))
import numpy as np, torch, torch.distributed as dist
import bonsai_b200 as bb
from bonsai_b200 import synth, partition
from bonsai_b200.peer import PeerBuffer

rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"]); local = int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local)
dist.init_process_group("gloo")
bb.lib()
def dev(a): return torch.from_numpy(np.ascontiguousarray(a)).cuda()

widths = [5120, 6144, 17408, 5120, 2048, 1024]      # op i: widths[i] -> widths[i+1], each depends on the one before
n_ops = len(widths) - 1
x0 = synth.activations(widths[0], seed=7)
Ws = [synth.pq2_0_weights(widths[i + 1], widths[i], seed=40 + i) for i in range(n_ops)]
# a side op that shares op 1's input, and two independent Q8 ops
W_side = synth.pq2_0_weights(4096, widths[1], seed=77)
xq_ext = synth.activations(5120, seed=9)
W_q = synth.pq2_0_weights(1024, 5120, seed=78)

# reference on this rank, full matrices, per-matrix calls
scratch = torch.zeros(17408 // 32 * 36, dtype=torch.uint8, device="cuda")
ref = [dev(x0)] + [torch.zeros(w, device="cuda") for w in widths[1:]]
for i in range(n_ops):
    assert bb.linear(dev(Ws[i]), ref[i], None, ref[i + 1], scratch, widths[i + 1], widths[i]) == 0
side_ref = torch.zeros(4096, device="cuda"); assert bb.linear(dev(W_side), ref[1], None, side_ref, scratch, 4096, widths[1]) == 0
xq_d = torch.empty(5120 // 32 * 36, dtype=torch.uint8, device="cuda"); assert bb.fwht_quant(dev(xq_ext), None, xq_d, None, 5120) == 0
q_ref = torch.zeros(1024, device="cuda"); assert bb.gemv(dev(W_q), xq_d, q_ref, 1024, 5120) == 0
torch.cuda.synchronize()

# peer buffer: [y1 .. y5 | side | q]
sizes = widths[1:] + [4096, 1024]
offs = np.concatenate([[0], np.cumsum(sizes)]).astype(int)
pb = PeerBuffer(int(offs[-1]) * 4, dist, rank, world)
buf = pb.tensor.view(torch.float32)
def region(k): return buf[offs[k]:offs[k + 1]]
def wslice(W, n_out, n_in):
    b0, b1 = partition.byte_slice(n_out, n_in, rank, world)
    return dev(W.reshape(-1)[b0:b1])
def yslice(k, n_out):
    lo, hi = partition.row_slice(n_out, rank, world)
    return region(k)[lo:hi], hi - lo

ops = []
x_in = dev(x0)
for i in range(n_ops):
    ys, rows = yslice(i, widths[i + 1])
    src = x_in if i == 0 else region(i - 1)
    ops.append((wslice(Ws[i], widths[i + 1], widths[i]), src, None, ys, rows, widths[i], bb.OP_ROTATE | (bb.OP_DEPENDS if i else 0)))
    if i == 1:
        ys2, rows2 = yslice(n_ops, 4096)
        ops.append((wslice(W_side, 4096, widths[1]), src, None, ys2, rows2, widths[1], bb.OP_ROTATE | bb.OP_SAME_INPUT))
ys3, rows3 = yslice(n_ops + 1, 1024)
ops.append((wslice(W_q, 1024, 5120), xq_d, None, ys3, rows3, 5120, 0))
chain = bb.Chain(ops, peers=pb)
ok = True
for it in range(3):
    assert chain.run() == 0
    torch.cuda.synchronize(); dist.barrier()
    for i in range(n_ops):
        same = torch.equal(region(i), ref[i + 1]); ok &= same
        if not same: print(f"rank {rank} it {it}: op {i} differs, max abs {(region(i) - ref[i + 1]).abs().max().item():.3e}")
    ok &= torch.equal(region(n_ops), side_ref) and torch.equal(region(n_ops + 1), q_ref)
    dist.barrier()
# timing: graph replay
g = torch.cuda.CUDAGraph(); st = torch.cuda.Stream(); st.wait_stream(torch.cuda.current_stream())
with torch.cuda.stream(st):
    with torch.cuda.graph(g, stream=st):
        chain.run()
torch.cuda.current_stream().wait_stream(st)
dist.barrier()
for _ in range(5): g.replay()
torch.cuda.synchronize(); dist.barrier()
e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
e0.record()
for _ in range(50): g.replay()
e1.record(); torch.cuda.synchronize()
for i in range(n_ops):
    ok &= torch.equal(region(i), ref[i + 1])
# ... and directly against the CPU checker, not only through the one-GPU entry points: sampled rows of every op of the
# dependent run, the checker fed this rank's own input of the op (the previous op's assembled output)
from oracle.oracle import Oracle
orc = Oracle("port")
for i in range(n_ops):
    n_in_i, n_out_i = widths[i], widths[i + 1]
    x_i = x0 if i == 0 else region(i - 1).cpu().numpy()
    xq_i = orc.quantize_q8_1(orc.fwht_blocks(np.ascontiguousarray(x_i, dtype=np.float32)), True)
    rows = np.unique(np.linspace(0, n_out_i - 1, 48).astype(np.int64))
    row_bytes = n_in_i // 128 * 34
    Wsub = np.concatenate([Ws[i].reshape(-1)[r * row_bytes:(r + 1) * row_bytes] for r in rows])
    want = orc.gemv(Wsub, xq_i, len(rows), n_in_i)
    got = region(i).cpu().numpy()[rows]
    err = float(np.abs(got - want).max()); bound = 1e-5 * float(np.abs(want).max())
    if not err <= bound:
        ok = False
        print(f"rank {rank}: op {i} differs from the CPU checker: {err:.3e} > {bound:.3e}")
status = bb.device_status()
print(f"rank {rank}: ok={ok} status={status} {e0.elapsed_time(e1)/50*1e3:.1f} us per run of {len(ops)} ops", flush=True)
dist.barrier()
chain.close(); pb.close(dist)
dist.destroy_process_group()
sys.exit(0 if ok and status == 0 else 1)
