"""Regenerates tests/golden/pq2_golden.npz from the REFERENCE's own host code.

Run where a reference checkout is mounted: oracle/build_oracle.py compiles oracle/ref_shim.cpp
against the reference headers (oracle/_ref/libbonsai_ref.so) and every output stored below is what
that library returned.  Inputs are stored next to the outputs, so checking the vectors needs
neither the reference nor a particular numpy random stream.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "p40-kernel_b200"))

from bonsai_b200 import synth  # noqa: E402
from oracle.build_oracle import build_reference  # noqa: E402
from oracle.oracle import Oracle  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "pq2_golden.npz")


def main():
    if build_reference() is None:
        sys.exit("no reference checkout: cannot regenerate golden vectors")
    ref = Oracle("reference")
    rng = np.random.default_rng(20240607)
    g = {}

    # fp32 -> fp16 (host rounding rule): random patterns, exact ties, subnormal range, overflow edge
    rand = rng.integers(0, 2 ** 32, size=1500, dtype=np.uint64).astype(np.uint32)
    ties = (rng.integers(0x38800000 >> 13, 0x47800000 >> 13, size=700, dtype=np.uint64).astype(np.uint32) << 13) | 0x1000
    subn = rng.integers(0x33000000, 0x38800000, size=700, dtype=np.uint64).astype(np.uint32)
    edge = np.array([0, 0x80000000, 0x477FE000, 0x477FF000, 0x477FEFFF, 0x7F800000, 0xFF800000, 0x7FC00000,
                     0x33000000, 0x33000001, 0x32FFFFFF, 0x387FC000, 0x387FE000, 0x38800000], dtype=np.uint32)
    bits = np.concatenate([rand, ties, ties | 0x80000000, subn, edge]).astype(np.uint32)
    g["f32_bits"] = bits
    g["f16_bits"] = np.array([ref.f32_to_f16(v) for v in bits.view(np.float32)], dtype=np.uint16)
    g["f16_widen_bits"] = np.array([np.float32(ref.f16_to_f32(h)).view(np.uint32) for h in range(0, 65536, 37)],
                                   dtype=np.uint32)

    # rotation + quantiser
    x = synth.activations(2048, seed=11)
    x[5] = 0.0
    x[64:96] = 0.0                       # an all-zero chunk: d = 0, id = 0
    x[100] = 3.5 * x[100]
    sg = synth.signs(2048, seed=11)
    g["x"], g["signs"] = x, sg
    g["fwht_plain"] = ref.fwht_blocks(x).view(np.uint32)
    g["fwht_signed"] = ref.fwht_blocks(x, sg).view(np.uint32)
    g["q_raw_perm"] = ref.quantize_q8_1(x, True)
    g["q_raw_plain"] = ref.quantize_q8_1(x, False)
    g["q_rot_perm"] = ref.quantize_q8_1(ref.fwht_blocks(x, sg), True)
    # values that land exactly on .5 after scaling: amax = 127 makes id = 1
    t = np.zeros(32, dtype=np.float32)
    t[0] = 127.0
    t[1:9] = [0.5, -0.5, 1.5, -1.5, 2.5, -2.5, 126.5, -126.5]
    g["x_ties"], g["q_ties"] = t, ref.quantize_q8_1(t, True)

    # mat-vec: 12 rows x 1024 (8 blocks per row), with code 3 present
    W = synth.pq2_0_weights(12, 1024, seed=5)
    xq = ref.quantize_q8_1(ref.fwht_blocks(x[:1024], sg[:1024]), True)
    g["W"], g["xq"] = W, xq
    g["gemv_y"] = ref.gemv(W, xq, 12, 1024).view(np.uint32)
    g["chunk_sums_row3"] = ref.row_chunk_sums(W[3 * 8 * 34:4 * 8 * 34], xq, 1024)

    # mat-mul: 16 rows x 256 x 5 tokens, chunk-major activations
    Wg = synth.pq2_0_weights(16, 256, seed=6)
    X = synth.activations(256, seed=6, batch=5)
    Xq = ref.quantize_batch_chunk_major(X)
    g["Wg"], g["X"], g["Xq"] = Wg, X, Xq
    g["gemm_Y"] = ref.gemm(Wg, Xq, 16, 256, 5).view(np.uint32)

    # repacked layout
    g["W_repacked"] = ref.repack(W, 12, 1024)
    xq_raw = ref.quantize_q8_1(x[:1024], True)
    g["gemv_repack_y"] = np.array([ref.repack_row_dot(g["W_repacked"][r * 272:(r + 1) * 272], xq_raw, 8)
                                   for r in range(12)], dtype=np.float32).view(np.uint32)

    # weight quantiser / dequantiser
    wf = (rng.standard_normal(512) * 0.7).astype(np.float32)
    g["w_float"] = wf
    g["w_quant"] = ref.quantize_pq2_0(wf)
    g["w_dequant"] = ref.dequantize_pq2_0(g["w_quant"]).view(np.uint32)

    np.savez_compressed(OUT, **g)
    print(OUT, os.path.getsize(OUT), "bytes")


if __name__ == "__main__":
    main()
