"""The projection entry point that allocates nothing (bonsai_b200_linear_static).

Collected last on purpose (file name), so that a run that stops at the first failure has already run
everything else.  Called through the C ABI and compared with the existing entry point that takes a
caller-provided scratch (bonsai_b200_linear): the two launch the same kernels, so the outputs must be
the same bits, and both must stay within the mat-vec tolerance of the CPU checker.  Two calls in a row
with different shapes check that what the first call left in the shared array does not leak into the
second.
"""
import numpy as np
import pytest

from bonsai_b200 import synth

pytestmark = pytest.mark.gpu

REL_TOL = 1e-5      # same bound as tests/test_gpu_parity.py: max |got - want| <= REL_TOL * max |want|


def _project_both_ways(gpu, port, n_out, n_in, seed, signed):
    import torch
    W = synth.pq2_0_weights(n_out, n_in, seed=seed)
    x = synth.activations(n_in, seed=seed)
    sg = synth.signs(n_in, seed=seed) if signed else None
    Wd, xd = torch.from_numpy(W).cuda(), torch.from_numpy(x).cuda()
    sd = None if sg is None else torch.from_numpy(sg).cuda()
    y_static = torch.full((n_out,), 123.0, dtype=torch.float32, device="cuda")
    y_scratch = torch.full((n_out,), 456.0, dtype=torch.float32, device="cuda")
    scratch = torch.zeros(n_in // 32 * 36, dtype=torch.uint8, device="cuda")
    assert gpu.linear_static(Wd, xd, sd, y_static, n_out, n_in) == 0
    assert gpu.linear(Wd, xd, sd, y_scratch, scratch, n_out, n_in) == 0
    torch.cuda.synchronize()
    got, ref = y_static.cpu().numpy(), y_scratch.cpu().numpy()
    want = port.gemv(W, port.quantize_q8_1(port.fwht_blocks(x, sg), True), n_out, n_in, threads=4)
    scale = float(np.abs(want).max()) or 1.0
    assert float(np.abs(got.astype(np.float64) - ref).max()) <= REL_TOL * scale
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
    assert float(np.abs(got.astype(np.float64) - want).max()) <= REL_TOL * scale
    assert np.array_equal(xd.cpu().numpy().view(np.uint32), x.view(np.uint32))      # input untouched


def test_static_scratch_projection_two_calls_in_a_row(gpu, port):
    _project_both_ways(gpu, port, n_out=700, n_in=17408, seed=21, signed=True)      # fills 544 blocks of the array
    _project_both_ways(gpu, port, n_out=1030, n_in=5120, seed=22, signed=False)     # then only the first 160
    _project_both_ways(gpu, port, n_out=64, n_in=32768, seed=23, signed=True)       # the largest size it takes
    assert gpu.device_status() == 0


def test_static_scratch_projection_takes_no_device_memory(gpu):
    """What the name promises: device memory in use is the same before and after a call (the first call on the
    device has happened above or happens here, before the measurement; nothing else allocates in between)."""
    import torch
    n_out, n_in = 256, 17408
    Wd = torch.from_numpy(synth.pq2_0_weights(n_out, n_in, seed=24)).cuda()
    xd = torch.from_numpy(synth.activations(n_in, seed=24)).cuda()
    y = torch.zeros(n_out, dtype=torch.float32, device="cuda")
    assert gpu.linear_static(Wd, xd, None, y, n_out, n_in) == 0         # set-up call: resolves the array's address
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(2):
        assert gpu.linear_static(Wd, xd, None, y, n_out, n_in) == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, (free_before, free_after)


def test_static_scratch_projection_rejects_what_does_not_fit(gpu):
    import torch
    z = torch.zeros(8, dtype=torch.float32, device="cuda")
    b = torch.zeros(64, dtype=torch.uint8, device="cuda")
    too_large = gpu.lib().bonsai_b200_linear_static(b.data_ptr(), z.data_ptr(), None, z.data_ptr(), 4, 32768 + 1024, None)
    assert too_large == 2                                                            # BONSAI_B200_ETOOLARGE
    assert gpu.linear_static(b, z, None, z, 4, 1000) == 1                            # not a multiple of 1024
    assert gpu.linear_static(b, z, None, z, 0, 1024) == 1
