"""The load-time format steps on the GPU: GGUF tensor -> upload -> bonsai_p40_repack -> mat-vec, and the PTQ1_0
packing (device kernels against the numpy statement, byte for byte; lossless round trip)."""
import numpy as np
import pytest

from bonsai_b200 import gguf, synth

pytestmark = pytest.mark.gpu


def host(t):
    return t.detach().cpu().numpy()


def test_gguf_upload_repack_matvec(gpu, port, tmp_path):
    import torch
    n_in, n_out = 5120, 96
    W = synth.pq2_0_weights(n_out, n_in, seed=5)
    x = synth.activations(n_in, seed=5)
    p = tmp_path / "one.gguf"
    gguf.write_gguf(p, {"general.architecture": "qwen35"}, [("blk.0.ffn_up.weight", [n_in, n_out], gguf.GGML_TYPE_PQ2_0, W)])
    h = gguf.read_header(p)
    raw = gguf.upload(h, p, "blk.0.ffn_up.weight")
    assert np.array_equal(host(raw), W)
    rep = gguf.upload(h, p, "blk.0.ffn_up.weight", repack=True)
    assert np.array_equal(host(rep), port.repack(W, n_out, n_in))             # the bytes of repack_row_pq2_0
    y = torch.zeros(n_out, device="cuda")
    want = port.gemv_repack(port.repack(W, n_out, n_in), x, n_out, n_in)
    assert gpu.gemv_repack(rep, torch.from_numpy(x).cuda(), y, n_out, n_in) == 0
    assert np.abs(host(y) - want).max() <= 1e-5 * np.abs(want).max()          # default: a fixed tree order
    try:
        assert gpu.set_option("gemv_order", 1) == 0
        assert gpu.gemv_repack(rep, torch.from_numpy(x).cuda(), y, n_out, n_in) == 0
    finally:
        gpu.set_option("gemv_order", 0)
    assert np.array_equal(host(y).view(np.uint32), want.view(np.uint32))      # gemv_order 1 keeps the host's order


@pytest.mark.parametrize("n_blocks", [1, 7, 4096, 100003])
def test_ptq1_pack_unpack(gpu, n_blocks):
    import torch
    from oracle.oracle import ptq1_pack, ptq1_unpack
    W = synth.pq2_0_weights(n_blocks, 128, seed=n_blocks)                      # n_blocks rows of one block: code 3 at p = 0.001
    Wd = torch.from_numpy(W).cuda()
    packed = torch.zeros(n_blocks * 28, dtype=torch.uint8, device="cuda")
    count = torch.zeros(1, dtype=torch.int64, device="cuda")
    assert gpu.ptq1_pack(Wd, packed, n_blocks, count) == 0
    want, bad = ptq1_pack(W)
    assert np.array_equal(host(packed), want)
    assert int(count.item()) == bad
    back = torch.zeros_like(Wd)
    assert gpu.ptq1_unpack(packed, back, n_blocks) == 0
    assert np.array_equal(host(back), ptq1_unpack(want))
    if bad == 0:
        assert np.array_equal(host(back), W)                                   # lossless when no weight is +2
    assert packed.numel() * 34 == Wd.numel() * 28                              # 17.6 % fewer bytes
