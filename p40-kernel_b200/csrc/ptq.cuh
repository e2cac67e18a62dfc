// ptq.cuh -- the denser ternary packing PTQ1_0 (28 bytes per 128 weights) beside PQ2_0 (34 bytes).
//
// The reference only describes it (docs/NEXT_STEPS.md:76-83): the same ternary values and the same fp16 scale per 128
// weights as PQ2_0, five base-3 digits per byte instead of four 2-bit fields -- qs[24] (5 trits per byte: weights
// 0..119), qh[2] (4 trits per byte: weights 120..127), d (fp16) = 24 + 2 + 2 bytes.  Lossless exactly when no weight
// uses PQ2_0's fourth code (+2), which the reference found to be the case for the shipped checkpoint
// (docs/NEXT_STEPS.md:106-116).  The code that defines the byte order lives in a third-party fork that is not part of
// the reference checkout, so the order used here is this library's own: weight j < 120 is digit j % 5 of byte j / 5
// (digit k has weight 3^k), weight 120 + j is digit j % 4 of qh[j / 4]; a digit is the PQ2_0 code (0, 1, 2 = -1, 0, +1).
#pragma once

#include "common.cuh"

namespace b200 {

constexpr int PTQ_BLOCK_BYTES = 28;

// One thread per block.  `code3` counts the weights whose PQ2_0 code is 3 (not representable: stored as code 2).
__global__ void __launch_bounds__(256) ptq1_pack_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, long long n_blocks,
                                                        unsigned long long *__restrict__ code3) {
    unsigned int bad = 0;
    for (long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x; b < n_blocks; b += (long long)gridDim.x * blockDim.x) {
        const uint8_t *s = src + b * W_BLOCK_BYTES;
        uint8_t *d = dst + b * PTQ_BLOCK_BYTES;
        uint8_t code[128];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint32_t h = ldg_nc_u16(s + 2 + 2 * i);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                uint32_t c = (h >> (2 * k)) & 3u;
                if (c == 3u) { ++bad; c = 2u; }
                code[8 * i + k] = (uint8_t)c;
            }
        }
        unsigned short out[14];
        uint8_t *ob = reinterpret_cast<uint8_t *>(out);
#pragma unroll
        for (int i = 0; i < 24; ++i)
            ob[i] = (uint8_t)(code[5 * i] + 3 * code[5 * i + 1] + 9 * code[5 * i + 2] + 27 * code[5 * i + 3] + 81 * code[5 * i + 4]);
#pragma unroll
        for (int i = 0; i < 2; ++i)
            ob[24 + i] = (uint8_t)(code[120 + 4 * i] + 3 * code[121 + 4 * i] + 9 * code[122 + 4 * i] + 27 * code[123 + 4 * i]);
        out[13] = (unsigned short)ldg_nc_u16(s);
#pragma unroll
        for (int i = 0; i < 14; ++i) reinterpret_cast<unsigned short *>(d)[i] = out[i];     // 28-byte blocks start on even addresses
    }
    if (bad) atomicAdd(code3, (unsigned long long)bad);
}

__global__ void __launch_bounds__(256) ptq1_unpack_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, long long n_blocks) {
    for (long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x; b < n_blocks; b += (long long)gridDim.x * blockDim.x) {
        const uint8_t *s = src + b * PTQ_BLOCK_BYTES;
        uint8_t code[128];
#pragma unroll
        for (int i = 0; i < 13; ++i) {
            const uint32_t h = ldg_nc_u16(s + 2 * i);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                uint32_t v = (h >> (8 * half)) & 0xFFu;
                const int byte = 2 * i + half;
                if (byte < 24) {
#pragma unroll
                    for (int k = 0; k < 5; ++k) { code[5 * byte + k] = (uint8_t)(v % 3u); v /= 3u; }
                } else {
#pragma unroll
                    for (int k = 0; k < 4; ++k) { code[120 + 4 * (byte - 24) + k] = (uint8_t)(v % 3u); v /= 3u; }
                }
            }
        }
        unsigned short *d = reinterpret_cast<unsigned short *>(dst + b * W_BLOCK_BYTES);
        d[0] = (unsigned short)ldg_nc_u16(s + 26);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            uint32_t h = 0;
#pragma unroll
            for (int k = 0; k < 8; ++k) h |= (uint32_t)code[8 * i + k] << (2 * k);
            d[1 + i] = (unsigned short)h;
        }
    }
}

}  // namespace b200
