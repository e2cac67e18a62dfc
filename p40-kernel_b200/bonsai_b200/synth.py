"""Seeded synthetic stand-ins for the model's tensors (host side, numpy).

Weights follow the value distribution of the shipped checkpoint: 2-bit codes drawn per element
from {0, 1, 2} with p = {0.33, 0.34, 0.33} plus code 3 at p = 0.001, one fp16 scale
|N(0, 0.02)| per 128-weight block, packed as 34-byte PQ2_0 blocks (element j of a block lives in
code byte j / 4, bits 2 * (j % 4)).  Activations are fp32 N(0, 1).
"""
import numpy as np

W_BYTES = 34
A_BYTES = 36
CODE_P = np.array([0.33, 0.34, 0.33, 0.001], dtype=np.float64)


def pq2_0_weights(n_out, n_in, seed=0):
    """Returns uint8 [n_out * (n_in / 128) * 34]: row-major rows of PQ2_0 blocks."""
    assert n_in % 128 == 0
    rng = np.random.default_rng(seed)
    nblk = n_out * (n_in // 128)
    codes = rng.choice(4, size=(nblk, 32, 4), p=CODE_P / CODE_P.sum()).astype(np.uint8)
    packed = codes[..., 0] | (codes[..., 1] << 2) | (codes[..., 2] << 4) | (codes[..., 3] << 6)
    d = np.abs(rng.normal(0.0, 0.02, size=nblk)).astype(np.float16)
    out = np.empty((nblk, W_BYTES), dtype=np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(nblk, 2)
    out[:, 2:] = packed
    return out.reshape(-1)


def activations(n, seed=0, batch=None):
    rng = np.random.default_rng(seed + 1_000_003)
    shape = (n,) if batch is None else (batch, n)
    return rng.standard_normal(shape).astype(np.float32)


def signs(n, seed=0):
    rng = np.random.default_rng(seed + 2_000_003)
    return np.where(rng.random(n) < 0.5, -1.0, 1.0).astype(np.float32)
