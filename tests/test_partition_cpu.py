"""Row-partitioned mat-vec on CPU ranks (gloo, world size 2): every rank multiplies its row slice with the
CPU checker, an all-gather assembles y, and the result equals the unpartitioned product bit for bit.
Covers the host logic of the multi-GPU path (slice arithmetic, alignment, in-place gather)."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, n_out, n_in, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "p40-kernel_b200"))
    import torch
    import torch.distributed as dist
    from bonsai_b200 import partition, synth
    from oracle.oracle import Oracle

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    orc = Oracle("port")
    W = synth.pq2_0_weights(n_out, n_in, seed=3)                  # every rank can regenerate any slice
    xq = orc.quantize_q8_1(orc.fwht_blocks(synth.activations(n_in, seed=3)), True)
    b_lo, b_hi = partition.byte_slice(n_out, n_in, rank, world)
    r_lo, r_hi = partition.row_slice(n_out, rank, world)
    assert b_lo % 16 == 0                                           # the slice starts aligned for bulk copies
    y = torch.zeros(n_out, dtype=torch.float32)
    y[r_lo:r_hi] = torch.from_numpy(orc.gemv(W[b_lo:b_hi], xq, r_hi - r_lo, n_in))
    partition.gather_rows(dist, y, rank, world)
    np.save(os.path.join(out_dir, f"y{rank}.npy"), y.numpy())
    dist.destroy_process_group()


@pytest.mark.parametrize("n_out,n_in", [(64, 5120), (40, 17408)])
def test_row_partition_gloo(tmp_path, port, n_out, n_in):
    import torch.multiprocessing as mp
    from bonsai_b200 import synth
    world = 2
    tcp = 29500 + (os.getpid() + n_out) % 2000
    mp.spawn(_worker, args=(world, tcp, n_out, n_in, str(tmp_path)), nprocs=world, join=True)
    W = synth.pq2_0_weights(n_out, n_in, seed=3)
    xq = port.quantize_q8_1(port.fwht_blocks(synth.activations(n_in, seed=3)), True)
    want = port.gemv(W, xq, n_out, n_in)
    for r in range(world):
        got = np.load(tmp_path / f"y{r}.npy")
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_slices_cover_and_align():
    from bonsai_b200 import partition
    for n_out, n_in in [(5120, 5120), (17408, 5120), (5120, 17408), (1024, 5120), (248320, 5120)]:
        for world in (1, 2, 4, 8):
            edges = [partition.byte_slice(n_out, n_in, r, world) for r in range(world)]
            assert edges[0][0] == 0 and edges[-1][1] == n_out * (n_in // 128) * 34
            for (a, b), (c, d) in zip(edges, edges[1:]):
                assert b == c
            assert all(lo % 16 == 0 for lo, _ in edges)
    with pytest.raises(ValueError):
        partition.row_slice(10, 0, 4)


def _ledger_worker(rank, world, port, skip_step, out_dir):
    sys.path.insert(0, os.path.join(ROOT, "p40-kernel_b200"))
    import json
    from datetime import timedelta
    import torch.distributed as dist
    from bonsai_b200 import partition

    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=timedelta(seconds=20))
    ledger = partition.StepLedger(store, rank, world)
    launched, seen_late = [], {}
    for step in (1, 2, 3):
        if rank == 1 and step == skip_step:
            break                                   # this rank leaves between steps: it never announces `step`
        ledger.announce(step)
        late = ledger.laggards(step, timeout_s=0.5)
        if late:
            seen_late[step] = late
            break                                   # do not launch: a peer is missing
        launched.append(step)                       # stands for bonsai_b200_chain_run of this step
    with open(os.path.join(out_dir, f"ledger{rank}.json"), "w") as f:
        json.dump({"launched": launched, "late": seen_late}, f)
    store.set(f"done/{rank}", "1")
    if rank == 0:                                   # the store's owner stays until everybody has written
        store.wait([f"done/{r}" for r in range(world)])


def test_a_rank_that_skips_a_step_is_named_before_the_launch(tmp_path):
    """Rank 1 of 2 leaves before step 2.  Rank 0 learns it on the host (no device wait is started), names rank 1 and
    launches nothing further; both launched step 1."""
    import json
    import torch.multiprocessing as mp
    tcp = 31500 + os.getpid() % 2000
    mp.spawn(_ledger_worker, args=(2, tcp, 2, str(tmp_path)), nprocs=2, join=True)
    r0 = json.load(open(tmp_path / "ledger0.json"))
    r1 = json.load(open(tmp_path / "ledger1.json"))
    assert r0["launched"] == [1] and r0["late"] == {"2": [1]}
    assert r1["launched"] == [1] and r1["late"] == {}
