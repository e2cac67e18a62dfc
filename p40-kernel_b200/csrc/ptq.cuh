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
constexpr int PTQ_CTA_BLOCKS = 256;            // blocks per CTA pass = threads per CTA

// Both directions: a CTA stages 256 blocks in shared memory with coalesced 4-byte accesses (source runs are 2-byte
// aligned: the first and last halfword of a run are moved singly), every thread converts one block with table look-ups
// (ten bits = five 2-bit codes <-> one byte), and the CTA writes the result back the same way.  A thread per block with
// halfword accesses to global memory and a division chain per byte ran at a tenth of the memory bandwidth.

// global (2-byte aligned) -> shared (4-byte aligned buffer), `bytes` even
__device__ __forceinline__ void ptq_stage_in(uint8_t *sm, const uint8_t *g, int bytes) {
    const int head = (int)((4 - (reinterpret_cast<uintptr_t>(g) & 3u)) & 3u);          // 0 or 2
    if (threadIdx.x == 0 && head && bytes >= 2) *reinterpret_cast<unsigned short *>(sm + 2) = *reinterpret_cast<const unsigned short *>(g);
    // the shared image is shifted so that global word k lands on a word: image offset = 4 - head for head != 0, else 0
    const int shift = head ? 4 - head : 0;
    const int words = (bytes - head) >> 2;
    const uint32_t *gw = reinterpret_cast<const uint32_t *>(g + head);
    uint32_t *sw = reinterpret_cast<uint32_t *>(sm + shift + head);
    for (int i = threadIdx.x; i < words; i += blockDim.x) sw[i] = __ldg(gw + i);
    const int tail = bytes - head - 4 * words;                                            // 0 or 2
    if (threadIdx.x == 32 && tail) *reinterpret_cast<unsigned short *>(sm + shift + head + 4 * words) =
                                       *reinterpret_cast<const unsigned short *>(g + head + 4 * words);
}
__device__ __forceinline__ int ptq_image_shift(const uint8_t *g) { return (reinterpret_cast<uintptr_t>(g) & 3u) ? 2 : 0; }
// shared -> global, mirror of the above
__device__ __forceinline__ void ptq_stage_out(uint8_t *g, const uint8_t *sm, int bytes) {
    const int head = (int)((4 - (reinterpret_cast<uintptr_t>(g) & 3u)) & 3u);
    const int shift = head ? 4 - head : 0;
    if (threadIdx.x == 0 && head && bytes >= 2) *reinterpret_cast<unsigned short *>(g) = *reinterpret_cast<const unsigned short *>(sm + 2);
    const int words = (bytes - head) >> 2;
    uint32_t *gw = reinterpret_cast<uint32_t *>(g + head);
    const uint32_t *sw = reinterpret_cast<const uint32_t *>(sm + shift + head);
    for (int i = threadIdx.x; i < words; i += blockDim.x) gw[i] = sw[i];
    const int tail = bytes - head - 4 * words;
    if (threadIdx.x == 32 && tail) *reinterpret_cast<unsigned short *>(g + head + 4 * words) =
                                       *reinterpret_cast<const unsigned short *>(sm + shift + head + 4 * words);
}

// `code3` counts the weights whose PQ2_0 code is 3 (not representable: stored as code 2).
__global__ void __launch_bounds__(PTQ_CTA_BLOCKS) ptq1_pack_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, long long n_blocks,
                                                                   unsigned long long *__restrict__ code3) {
    __shared__ __align__(16) uint8_t in[PTQ_CTA_BLOCKS * W_BLOCK_BYTES + 8];
    __shared__ __align__(16) uint8_t out[PTQ_CTA_BLOCKS * PTQ_BLOCK_BYTES + 8];
    __shared__ unsigned short lut[1024];        // ten bits (five codes, least significant first) -> byte | (count of code 3) << 8
    for (int i = threadIdx.x; i < 1024; i += blockDim.x) {
        unsigned v = 0, w = 1, bad = 0;
        for (int k = 0; k < 5; ++k, w *= 3) {
            unsigned c = (i >> (2 * k)) & 3u;
            if (c == 3u) { ++bad; c = 2u; }
            v += c * w;
        }
        lut[i] = (unsigned short)(v | (bad << 8));
    }
    unsigned int bad = 0;
    for (long long b0 = (long long)blockIdx.x * PTQ_CTA_BLOCKS; b0 < n_blocks; b0 += (long long)gridDim.x * PTQ_CTA_BLOCKS) {
        const int nb = (int)min((long long)PTQ_CTA_BLOCKS, n_blocks - b0);
        const uint8_t *g = src + b0 * W_BLOCK_BYTES;
        uint8_t *gd = dst + b0 * PTQ_BLOCK_BYTES;
        __syncthreads();                                        // the table; the buffers of the previous pass
        ptq_stage_in(in, g, nb * W_BLOCK_BYTES);
        __syncthreads();
        if ((int)threadIdx.x < nb) {
            const unsigned short *s16 = reinterpret_cast<const unsigned short *>(in + ptq_image_shift(g) + threadIdx.x * W_BLOCK_BYTES);
            unsigned short *d16 = reinterpret_cast<unsigned short *>(out + ptq_image_shift(gd) + threadIdx.x * PTQ_BLOCK_BYTES);
            uint32_t w[8];                                      // the 256 code bits
#pragma unroll
            for (int i = 0; i < 8; ++i) w[i] = (uint32_t)s16[1 + 2 * i] | ((uint32_t)s16[2 + 2 * i] << 16);
            uint32_t ob[13];
#pragma unroll
            for (int i = 0; i < 12; ++i) {                      // bytes 2 i, 2 i + 1: bits 20 i .. 20 i + 19
                const int bit = 20 * i, wi = bit >> 5, sh = bit & 31;
                const uint32_t twenty = (sh <= 12 ? (w[wi] >> sh) : __funnelshift_r(w[wi], w[wi + 1 < 8 ? wi + 1 : 7], sh)) & 0xFFFFFu;
                const unsigned a = lut[twenty & 1023u], c = lut[twenty >> 10];
                bad += (a >> 8) + (c >> 8);
                ob[i] = (a & 0xFFu) | ((c & 0xFFu) << 8);
            }
            {                                                   // qh: weights 120..127 = the last 16 bits, four codes per byte
                const uint32_t sixteen = w[7] >> 16;
                const unsigned a = lut[sixteen & 255u], c = lut[sixteen >> 8];
                bad += (a >> 8) + (c >> 8);
                ob[12] = (a & 0xFFu) | ((c & 0xFFu) << 8);
            }
#pragma unroll
            for (int i = 0; i < 13; ++i) d16[i] = (unsigned short)ob[i];
            d16[13] = s16[0];
        }
        __syncthreads();
        ptq_stage_out(gd, out, nb * PTQ_BLOCK_BYTES);
    }
    // one addition per CTA (one per thread onto the same word serialised into most of the kernel's time)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) bad += __shfl_xor_sync(0xffffffffu, bad, o);
    __shared__ unsigned int wsum[PTQ_CTA_BLOCKS / 32];
    __syncthreads();
    if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = bad;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long total = 0;
        for (int i = 0; i < PTQ_CTA_BLOCKS / 32; ++i) total += wsum[i];
        if (total) atomicAdd(code3, total);
    }
}

__global__ void __launch_bounds__(PTQ_CTA_BLOCKS) ptq1_unpack_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, long long n_blocks) {
    __shared__ __align__(16) uint8_t in[PTQ_CTA_BLOCKS * PTQ_BLOCK_BYTES + 8];
    __shared__ __align__(16) uint8_t out[PTQ_CTA_BLOCKS * W_BLOCK_BYTES + 8];
    __shared__ unsigned short lut[256];         // byte -> ten bits (five base-3 digits as 2-bit codes, least significant first)
    for (int i = threadIdx.x; i < 256; i += blockDim.x) {
        unsigned v = (unsigned)i, bits = 0;
        for (int k = 0; k < 5; ++k) { bits |= (v % 3u) << (2 * k); v /= 3u; }
        lut[i] = (unsigned short)bits;
    }
    for (long long b0 = (long long)blockIdx.x * PTQ_CTA_BLOCKS; b0 < n_blocks; b0 += (long long)gridDim.x * PTQ_CTA_BLOCKS) {
        const int nb = (int)min((long long)PTQ_CTA_BLOCKS, n_blocks - b0);
        const uint8_t *g = src + b0 * PTQ_BLOCK_BYTES;
        uint8_t *gd = dst + b0 * W_BLOCK_BYTES;
        __syncthreads();
        ptq_stage_in(in, g, nb * PTQ_BLOCK_BYTES);
        __syncthreads();
        if ((int)threadIdx.x < nb) {
            const unsigned short *s16 = reinterpret_cast<const unsigned short *>(in + ptq_image_shift(g) + threadIdx.x * PTQ_BLOCK_BYTES);
            unsigned short *d16 = reinterpret_cast<unsigned short *>(out + ptq_image_shift(gd) + threadIdx.x * W_BLOCK_BYTES);
            uint32_t w[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) w[i] = 0;
#pragma unroll
            for (int i = 0; i < 12; ++i) {                      // bytes 2 i, 2 i + 1 -> bits 20 i .. 20 i + 19
                const unsigned h = s16[i];
                const uint32_t twenty = (uint32_t)lut[h & 0xFFu] | ((uint32_t)lut[h >> 8] << 10);
                const int bit = 20 * i, wi = bit >> 5, sh = bit & 31;
                w[wi] |= twenty << sh;
                if (sh > 12) w[wi + 1 < 8 ? wi + 1 : 7] |= twenty >> (32 - sh);
            }
            {
                const unsigned h = s16[12];
                w[7] |= ((uint32_t)(lut[h & 0xFFu] & 0xFFu) | ((uint32_t)(lut[h >> 8] & 0xFFu) << 8)) << 16;
            }
            d16[0] = s16[13];
#pragma unroll
            for (int i = 0; i < 8; ++i) { d16[1 + 2 * i] = (unsigned short)w[i]; d16[2 + 2 * i] = (unsigned short)(w[i] >> 16); }
        }
        __syncthreads();
        ptq_stage_out(gd, out, nb * W_BLOCK_BYTES);
    }
}

}  // namespace b200
