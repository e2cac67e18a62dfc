"""GPU parity of the operators beside the mat-vec path: bonsai_p40_rmsnorm, _gdn_step, _attn against the CPU
checker (the reference's src/ops.h through oracle/_ref where it is built; the C restatement otherwise).

Bound: 1e-5 of the largest reference value per tensor (the reference's own tests use 1e-4 against a double-precision
formula, tests/test_p40.cpp:168-171,232-233,308): long sums are added in a fixed tree order on the device and
sequentially on the host, and exp() is the device's.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

REL_TOL = 1e-5


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.detach().cpu().numpy()


def close(got, want, tol=REL_TOL):
    scale = float(np.abs(want).max()) or 1.0
    err = float(np.abs(got.astype(np.float64) - want.astype(np.float64)).max())
    assert err <= tol * scale, f"max-abs {err:.3e} vs bound {tol * scale:.3e}"


@pytest.mark.parametrize("n_rows,n", [(1, 5120), (7, 5120), (3, 6144), (2, 1000), (5, 37), (1, 70000)])
def test_rmsnorm(gpu, port, n_rows, n):
    import torch
    rng = np.random.default_rng(n)
    x = rng.uniform(-2, 2, size=(n_rows, n)).astype(np.float32)
    w = (rng.uniform(-2, 2, size=n) * 0.5 + 1.0).astype(np.float32)
    y = torch.zeros(n_rows, n, dtype=torch.float32, device="cuda")
    assert gpu.rmsnorm(dev(x), dev(w), y, n_rows, n, 1e-6) == 0
    close(host(y), port.rmsnorm(x, w, 1e-6))
    # a row at an odd float offset (the reference takes any pointer)
    holder = torch.zeros(n + 3, dtype=torch.float32, device="cuda")
    holder[1:n + 1].copy_(dev(x[0]))
    y1 = torch.zeros(n, dtype=torch.float32, device="cuda")
    assert gpu.rmsnorm(holder[1:n + 1], dev(w), y1, 1, n, 1e-6) == 0
    assert np.array_equal(host(y1).view(np.uint32), host(y)[0].view(np.uint32))


def test_rmsnorm_matches_the_reference_headers(gpu, ref):
    import torch
    rng = np.random.default_rng(5)
    x = rng.uniform(-2, 2, size=(4, 5120)).astype(np.float32)
    w = rng.uniform(0, 2, size=5120).astype(np.float32)
    y = torch.zeros(4, 5120, dtype=torch.float32, device="cuda")
    assert gpu.rmsnorm(dev(x), dev(w), y, 4, 5120, 1e-6) == 0
    close(host(y), ref.rmsnorm(x, w, 1e-6))


@pytest.mark.parametrize("n_k,n_v,K,V", [(16, 48, 128, 128), (4, 8, 128, 128), (2, 2, 64, 32), (1, 3, 100, 96)])
def test_gdn_step(gpu, port, n_k, n_v, K, V):
    import torch
    rng = np.random.default_rng(K + V + n_v)
    S = (rng.uniform(-1, 1, size=(n_v, K, V)) * 0.1).astype(np.float32)
    q = rng.uniform(-1, 1, size=(n_k, K)).astype(np.float32)
    k = rng.uniform(-1, 1, size=(n_k, K)).astype(np.float32)
    v = rng.uniform(-1, 1, size=(n_v, V)).astype(np.float32)
    g = (-rng.uniform(0.05, 1.0, size=n_v)).astype(np.float32)
    beta = rng.uniform(0.1, 1.0, size=n_v).astype(np.float32)
    want_S, want_out = port.gdn_step(S, q, k, v, g, beta, n_k, n_v, K, V)
    Sd = dev(S)
    out = torch.zeros(n_v * V, dtype=torch.float32, device="cuda")
    assert gpu.gdn_step(Sd, dev(q), dev(k), dev(v), dev(g), dev(beta), out, n_k, n_v, K, V) == 0
    close(host(Sd), want_S)
    close(host(out), want_out)
    # two more steps: the state keeps following the host recurrence
    for _ in range(2):
        want_S, want_out = port.gdn_step(want_S, q, k, v, g, beta, n_k, n_v, K, V)
        assert gpu.gdn_step(Sd, dev(q), dev(k), dev(v), dev(g), dev(beta), out, n_k, n_v, K, V) == 0
    close(host(Sd), want_S, 3e-5)
    close(host(out), want_out, 3e-5)


@pytest.mark.parametrize("n_tok,n_head,n_head_kv", [(1, 24, 4), (64, 24, 4), (37, 6, 2), (130, 4, 4)])
def test_attn(gpu, port, n_tok, n_head, n_head_kv):
    import torch
    D = 256
    rng = np.random.default_rng(n_tok)
    q = rng.uniform(-1, 1, size=(n_tok, n_head, D)).astype(np.float32)
    k = rng.uniform(-1, 1, size=(n_tok, n_head_kv, D)).astype(np.float32)
    v = rng.uniform(-1, 1, size=(n_tok, n_head_kv, D)).astype(np.float32)
    scale = 1.0 / np.sqrt(D)
    out = torch.zeros(n_tok * n_head * D, dtype=torch.float32, device="cuda")
    assert gpu.attn(dev(q), dev(k), dev(v), out, n_tok, n_head, n_head_kv, D, scale) == 0
    close(host(out), port.attn(q, k, v, n_tok, n_head, n_head_kv, D, scale))
    assert gpu.device_status() == 0
