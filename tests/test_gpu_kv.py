"""GPU parity of the K/V cache path (include/bonsai_kv.h): sizing, append (Q8_0 bytes exact against the host
quantiser, src/kv_cache.h:100-117, at the block index of src/kv_cache.h:81-84) and single-query decode attention over
the cache (1e-5 of the largest output against the position-by-position host recurrence on the SAME cache bytes)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

N_LAYERS, N_KV, N_HEADS, D = 16, 4, 24, 256


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.detach().cpu().numpy()


def cache_bytes(gpu, kv):
    """The K and V arrays as numpy uint8 (device -> host)."""
    import torch
    kp, vp, n = kv.arrays()

    class Raw:
        def __init__(self, ptr):
            self.__cuda_array_interface__ = {"shape": (n,), "typestr": "|u1", "data": (int(ptr), False), "version": 3}
    return host(torch.as_tensor(Raw(kp), device="cuda")), host(torch.as_tensor(Raw(vp), device="cuda"))


def test_sizes(gpu, ref):
    L = gpu.lib()
    for cap in (1, 4096, 262144, 500000):
        assert L.bonsai_kv_bytes(cap) == ref._kv_total_bytes(min(cap, 262144))
    assert L.bonsai_kv_bytes(0) == 0 and L.bonsai_kv_bytes(-5) == 0
    assert L.bonsai_kv_gdn_bytes() == ref._kv_gdn_bytes() == 48 * 48 * 128 * 128 * 4
    assert L.bonsai_kv_bytes(262144) == 2 * 16 * 4 * 262144 * 8 * 34


def test_append_bytes_and_layout(gpu, port):
    import torch
    cap = 700
    kv = gpu.KVCache(cap)
    rng = np.random.default_rng(1)
    written = {}
    for layer, pos0, n_tok in ((0, 0, 1), (3, 5, 37), (15, cap - 3, 3), (3, 0, 5)):
        k = (rng.standard_normal((n_tok, N_KV, D)) * rng.uniform(0.01, 30)).astype(np.float32)
        v = (rng.standard_normal((n_tok, N_KV, D)) * rng.uniform(0.01, 30)).astype(np.float32)
        k[0, 0, :32] = 0.0                                  # an all-zero block: scale 0, values 0
        k[0, 1, 32:64] = np.float32(63.5) / 127 * 127       # exact ties at .5 are rounded away from zero
        rc = kv.append(layer, pos0, dev(k[0]), dev(v[0])) if n_tok == 1 else kv.append_batch(layer, pos0, n_tok, dev(k), dev(v))
        assert rc == 0
        for t in range(n_tok):
            for h in range(N_KV):
                written[(layer, h, pos0 + t)] = (k[t, h], v[t, h])
    torch.cuda.synchronize()
    Kb, Vb = cache_bytes(gpu, kv)
    for (layer, h, pos), (kr, vr) in written.items():
        off = ((layer * N_KV + h) * cap + pos) * 8 * 34
        assert np.array_equal(Kb[off:off + 272], port.kv_quantize_row(kr)), (layer, h, pos)
        assert np.array_equal(Vb[off:off + 272], port.kv_quantize_row(vr)), (layer, h, pos)
    # rejections (src/kernels/kv_p40.cu:319-321)
    z = torch.zeros(N_KV * D, device="cuda")
    assert kv.append(16, 0, z, z) == 1 and kv.append(-1, 0, z, z) == 1
    assert kv.append(0, cap, z, z) == 1 and kv.append_batch(0, cap - 1, 2, z, z) == 1 and kv.append_batch(0, 0, 0, z, z) == 1
    assert kv.gdn_state(0) is not None and kv.gdn_state(47) is not None and kv.gdn_state(48) is None
    kv.close()


@pytest.mark.parametrize("pos", [0, 1, 31, 32, 255, 256, 300, 2100])
def test_attn_decode(gpu, port, pos):
    import torch
    cap, layer = 2304, 7
    kv = gpu.KVCache(cap)
    rng = np.random.default_rng(pos)
    n = pos + 1
    k = rng.uniform(-1, 1, size=(n, N_KV, D)).astype(np.float32)
    v = rng.uniform(-1, 1, size=(n, N_KV, D)).astype(np.float32)
    # a few positions that dominate the softmax, spread over the tiles and splits
    q = rng.uniform(-1, 1, size=(N_HEADS, D)).astype(np.float32)
    for j in (0, n // 2, n - 1):
        k[j, :, :] = 3.0 * q[::6][:, :] / np.abs(q[::6]).max()
    assert kv.append_batch(layer, 0, n, dev(k), dev(v)) == 0
    out = torch.zeros(N_HEADS * D, device="cuda")
    assert kv.attn_decode(layer, pos, dev(q), out) == 0
    torch.cuda.synchronize()
    Kb, Vb = cache_bytes(gpu, kv)
    got = host(out).astype(np.float64)
    # (a) the exact value of the same arithmetic: quantised query x the cache bytes, softmax and value sum in float64
    exact = np.zeros((N_HEADS, D))
    for h in range(N_HEADS):
        kvh = h // (N_HEADS // N_KV)
        off = (layer * N_KV + kvh) * cap * 272
        kd = port.kv_dequantize_row(Kb[off:off + n * 272]).reshape(n, D).astype(np.float64)
        vd = port.kv_dequantize_row(Vb[off:off + n * 272]).reshape(n, D).astype(np.float64)
        qd = port.kv_dequantize_row(port.kv_quantize_row(q[h])).astype(np.float64)
        sc = kd @ qd * 0.0625
        pw = np.exp(sc - sc.max())
        exact[h] = (pw[:, None] * vd).sum(0) / pw.sum()
    err = float(np.abs(got - exact.reshape(-1)).max())
    assert err <= 1e-5 * float(np.abs(exact).max()), (err, float(np.abs(exact).max()))
    # (b) the host's fp32 recurrence, position by position (its own rounding grows with the position count: the
    # reference's test of the recurrence allows 1e-4, tests/test_p40.cpp:308)
    want = port.kv_attn_decode(Kb, Vb, q, cap, layer, pos)
    assert float(np.abs(got - want).max()) <= 1e-4 * float(np.abs(want).max())
    assert kv.attn_decode(16, 0, dev(q), out) == 1 and kv.attn_decode(0, cap, dev(q), out) == 1
    assert gpu.device_status() == 0
    kv.close()


def test_state_is_zeroed_and_reset(gpu):
    import torch
    kv = gpu.KVCache(64)
    torch.cuda.synchronize()
    ptr = kv.gdn_state(5)
    n = 48 * 128 * 128

    class Raw:
        __cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (int(ptr), False), "version": 3}
    st = torch.as_tensor(Raw(), device="cuda")
    assert float(st.abs().max().item()) == 0.0
    st.fill_(2.0)
    kv.reset()
    torch.cuda.synchronize()
    assert float(st.abs().max().item()) == 0.0
    kv.close()
