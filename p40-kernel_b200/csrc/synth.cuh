// synth.cuh -- counter-based synthetic PQ2_0 weights generated on the device.
//
// Benchmark support, not part of the numeric path: fills a weight tensor whose value
// distribution copies the shipped checkpoint (ternary codes, code 3 all but absent) so that
// multi-gigabyte decode chains need no host generation or PCIe upload.  Halfword h of block i
// depends only on (seed, first_block + i, h), so any slice of a tensor can be regenerated.
#pragma once

#include "common.cuh"

namespace b200 {

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// 16 uniform bits -> code with p(3) = 65/65536, p(0) = p(2) = 21605/65536, p(1) = 22261/65536.
__device__ __forceinline__ uint32_t code_from_u16(uint32_t u) {
    return u < 65u ? 3u : (u < 21670u ? 0u : (u < 43931u ? 1u : 2u));
}

__global__ void __launch_bounds__(256) synth_pq2_kernel(unsigned short *__restrict__ W, long long first_block,
                                                        long long n_blocks, unsigned long long seed) {
    const long long total = n_blocks * 17;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long blk = i / 17;
        const int h = (int)(i - blk * 17);
        const unsigned long long ctr = (unsigned long long)(first_block + blk) * 32ull + (unsigned long long)h;
        const unsigned long long r0 = mix64(seed * 0xD1342543DE82EF95ull + 2 * ctr);
        unsigned short out;
        if (h == 0) {
            int s = 0;
#pragma unroll
            for (int k = 0; k < 8; ++k) s += (int)((r0 >> (8 * k)) & 0xFF);
            const float z = __fmul_rn((float)(s - 1020), 1.0f / 209.03f);   // ~N(0,1): sum of 8 uniform bytes
            out = __half_as_ushort(__float2half_rn(__fmul_rn(fabsf(z), 0.02f)));
        } else {
            const unsigned long long r1 = mix64(seed * 0xD1342543DE82EF95ull + 2 * ctr + 1);
            uint32_t v = 0;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                v |= code_from_u16((uint32_t)(r0 >> (16 * k)) & 0xFFFFu) << (2 * k);
                v |= code_from_u16((uint32_t)(r1 >> (16 * k)) & 0xFFFFu) << (8 + 2 * k);
            }
            out = (unsigned short)v;
        }
        W[i] = out;
    }
}

}  // namespace b200
