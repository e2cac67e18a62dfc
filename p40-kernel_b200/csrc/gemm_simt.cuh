// gemm_simt.cuh -- mat-mul Y[n_out][n_tok] = W . X on the integer SIMT pipe (dp4a).
//
// Serves token counts too small to fill a tensor-core tile and every shape the tensor-core
// kernel does not take.  Replaces, for sm_100a, gemm_pq2_0_p40_kernel
// (src/kernels/gemm_p40.cu:44-139); per (row, token) the terms (dw * da) * (float)sumi are added
// block by block, chunk by chunk, which is the order of the reference's host loop
// (tests/test_p40.cpp:460-467), so Y is bit-identical to it.
//
// Tile: 64 rows x 32 tokens per CTA of 256 threads; thread = (row, group of 8 tokens).  Per weight
// block the CTA stages 64 x 34 weight bytes and the 4 x 32 activation blocks of the tile, so each
// code word is unpacked once per row and reused by 8 tokens, and activation words are read as
// warp-wide broadcasts.
#pragma once

#include "common.cuh"

namespace b200 {

constexpr int GS_ROWS = 64, GS_TOKS = 32, GS_TPT = 8;   // tokens per thread

__global__ void __launch_bounds__(256) gemm_simt_kernel(const uint8_t *__restrict__ W, const uint32_t *__restrict__ Xq,
                                                        float *__restrict__ Y, int n_out, int nblocks, int n_tok) {
    __shared__ uint32_t ws[GS_ROWS][9];                       // 34 bytes + 2 pad per row; odd word stride
    __shared__ __align__(16) int aq[4][GS_TOKS][8];           // int8 words
    __shared__ float ad[4][GS_TOKS];
    __shared__ int as64[4][GS_TOKS];

    const int row_l = threadIdx.x & (GS_ROWS - 1);
    const int tg = threadIdx.x >> 6;                          // 0..3, constant inside a warp
    const int row0 = blockIdx.x * GS_ROWS, tok0 = blockIdx.y * GS_TOKS;
    const int row = row0 + row_l;

    float acc[GS_TPT];
#pragma unroll
    for (int j = 0; j < GS_TPT; ++j) acc[j] = 0.0f;

    for (int b = 0; b < nblocks; ++b) {
        __syncthreads();
        // weights: 64 rows x 17 halfwords
        for (int i = threadIdx.x; i < GS_ROWS * 17; i += blockDim.x) {
            const int r = i / 17, h = i - r * 17;
            const int gr = min(row0 + r, n_out - 1);
            reinterpret_cast<unsigned short *>(&ws[r][0])[h] =
                (unsigned short)ldg_nc_u16(W + ((size_t)gr * nblocks + b) * W_BLOCK_BYTES + 2 * h);
        }
        // activations: 4 chunks x 32 tokens x 9 words (token-contiguous in the chunk-major layout)
        for (int i = threadIdx.x; i < 4 * GS_TOKS * 9; i += blockDim.x) {
            const int c = i / (GS_TOKS * 9), rem = i - c * (GS_TOKS * 9);
            const int t = rem / 9, w = rem - t * 9;
            uint32_t v = 0;
            if (tok0 + t < n_tok) v = __ldg(Xq + 9 * ((size_t)(4 * b + c) * n_tok + tok0 + t) + w);
            if (w == 0) {
                ad[c][t] = f16_bits_to_f32(v & 0xFFFFu);
                as64[c][t] = -64 * (int)(short)(v >> 16);
            } else {
                aq[c][t][w - 1] = (int)v;
            }
        }
        __syncthreads();

        const float dw = f16_bits_to_f32(ws[row_l][0] & 0xFFFFu);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const uint32_t c0 = __funnelshift_r(ws[row_l][2 * c], ws[row_l][2 * c + 1], 16);
            const uint32_t c1 = __funnelshift_r(ws[row_l][2 * c + 1], ws[row_l][2 * c + 2], 16);
#pragma unroll
            for (int j = 0; j < GS_TPT; ++j) {
                const int t = tg * GS_TPT + j;
                const int4 lo = *reinterpret_cast<const int4 *>(&aq[c][t][0]);
                const int4 hi = *reinterpret_cast<const int4 *>(&aq[c][t][4]);
                const int a[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
                const int sumi = chunk_sumi_scaled(c0, c1, a, as64[c][t]);
                acc[j] = __fadd_rn(acc[j], __fmul_rn(__fmul_rn(dw, ad[c][t]), (float)sumi));
            }
        }
    }
    if (row < n_out) {
#pragma unroll
        for (int j = 0; j < GS_TPT; ++j) {
            const int t = tok0 + tg * GS_TPT + j;
            if (t < n_tok) Y[(size_t)row * n_tok + t] = acc[j];
        }
    }
}

}  // namespace b200
