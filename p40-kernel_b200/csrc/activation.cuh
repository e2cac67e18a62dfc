// activation.cuh -- FWHT-1024 rotation and the Q8_1 quantiser (activation side of the path).
//
// Replaces, for sm_100a: fwht_1024_p40_kernel (src/kernels/elementwise_p40.cu:17-41) and
// quant_q8_1_pq2_kernel (src/kernels/gemv_p40.cu:168-196).  Output bytes follow the reference's
// HOST functions: fwht_blocks (src/fwht.h:20-42) and quantize_row_q8_1(..., permute = true)
// (src/pq2_0.h:99-126).
//
// Both kernels are a handful of warps of latency-bound work (<= 70 KB in, <= 20 KB out per
// decode vector), so the design goal is one launch and no shared-memory round trips:
//   * rotation: one warp per 1024-block, 32 values per lane in registers; the ten butterfly
//     stages run in the host's order (h = 1, 2, ..., 512), each output produced by exactly one
//     a + b or a - b with a the lower-index operand, so the fp32 bits equal the host's;
//   * quantiser: eight lanes per 32-chunk, four values per lane (the same register layout the
//     rotation leaves behind, which is what lets the two fuse without a shuffle stage between).
#pragma once

#include "common.cuh"

namespace b200 {

// ---- quantiser core: 8 consecutive lanes own one 32-chunk, lane g (0..7) holds x[4g..4g+3] ----
// Returns through `word` the Q8_1 data word this lane stores (word index g of qs) and through
// `header` the d|s word (valid on every lane of the group).
__device__ __forceinline__ void quantise_chunk_8lanes(const float (&v)[4], int lane, uint32_t &word, uint32_t &header) {
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float d = __fdiv_rn(amax, 127.0f);
    const float id = d > 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    int sum = 0;
    uint32_t packed = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        int q = round_ties_away(__fmul_rn(v[e], id));
        q = max(-127, min(127, q));
        sum += q;
        packed |= ((uint32_t)q & 0xFFu) << (8 * e);
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    // 4x4 byte transpose among the four lanes of each half-group: element j = 4g + e lands at
    // position 16*(j>>4) + 4*(j&3) + ((j>>2)&3) = byte (g&3) of word 4*(g>>2) + e, so this lane
    // (word g) gathers byte (g&3) from the lanes of its half-group.
    const int m = lane & 3;
    const int base = lane & ~3;
    word = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t other = __shfl_sync(0xffffffffu, packed, base + k);
        word |= ((other >> (8 * m)) & 0xFFu) << (8 * k);
    }
    header = f32_to_f16_bits_ties_away(d) | (((uint32_t)sum & 0xFFFFu) << 16);
}

// Four consecutive floats: one 16-byte access when the caller's pointer allows it (VEC), else four 4-byte
// accesses -- the reference takes any float pointer (src/kernels/elementwise_p40.cu:75-80, gemv_p40.cu:200-208).
template <bool VEC>
__device__ __forceinline__ float4 load_f4(const float *p) {
    if (VEC) return *reinterpret_cast<const float4 *>(p);
    return make_float4(p[0], p[1], p[2], p[3]);
}
template <bool VEC>
__device__ __forceinline__ void store_f4(float *p, float4 v) {
    if (VEC) { *reinterpret_cast<float4 *>(p) = v; return; }
    p[0] = v.x; p[1] = v.y; p[2] = v.z; p[3] = v.w;
}

// One thread per four inputs.  X is [n_tok][n_in]; output block index = chunk * tok_stride + tok
// (tok_stride = 1 with n_tok = 1 gives the plain vector layout).
template <bool VEC>
__global__ void __launch_bounds__(256) quant_q8_1_kernel(const float *__restrict__ X, uint32_t *__restrict__ out,
                                                         int n_in, int n_tok) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    const int lane = threadIdx.x & 31;
    const int per_tok = n_in >> 2;
    const long long total = (long long)per_tok * n_tok;
    const long long stride = (long long)gridDim.x * blockDim.x;
    // whole warps iterate together: total is a multiple of 8 and a warp covers 32 threads
    for (long long i0 = (long long)blockIdx.x * blockDim.x + (threadIdx.x & ~31); i0 < total; i0 += stride) {
        const long long i = i0 + lane;
        const bool live = i < total;
        const long long ic = live ? i : total - 1;
        const int tok = (int)(ic / per_tok);
        const int g4 = (int)(ic - (long long)tok * per_tok);
        const float4 f = load_f4<VEC>(X + (size_t)tok * n_in + 4 * (size_t)g4);
        const float v[4] = {f.x, f.y, f.z, f.w};
        uint32_t word, header;
        quantise_chunk_8lanes(v, lane, word, header);
        if (live) {
            const int chunk = g4 >> 3;
            uint32_t *blk = out + 9 * ((size_t)chunk * n_tok + tok);
            blk[1 + (lane & 7)] = word;
            if ((lane & 7) == 0) blk[0] = header;
        }
    }
}

// ---- rotation: one warp per 1024-block ---------------------------------------------------------
// Lane l holds v[r][e] = element r*128 + 4*l + e (r = 0..7, e = 0..3): index bits 0-1 are e,
// bits 2-6 the lane, bits 7-9 r.
__device__ __forceinline__ void fwht1024_warp(float (&v)[8][4], int lane) {
#pragma unroll
    for (int r = 0; r < 8; ++r) {   // h = 1, 2: inside the lane
        float a = v[r][0], b = v[r][1], c = v[r][2], d = v[r][3];
        float s0 = __fadd_rn(a, b), s1 = __fsub_rn(a, b), s2 = __fadd_rn(c, d), s3 = __fsub_rn(c, d);
        v[r][0] = __fadd_rn(s0, s2); v[r][2] = __fsub_rn(s0, s2);
        v[r][1] = __fadd_rn(s1, s3); v[r][3] = __fsub_rn(s1, s3);
    }
#pragma unroll
    for (int s = 0; s < 5; ++s) {   // h = 4 .. 64: across lanes
        const bool upper = (lane >> s) & 1;
#pragma unroll
        for (int r = 0; r < 8; ++r)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float mine = v[r][e];
                const float other = __shfl_xor_sync(0xffffffffu, mine, 1 << s);
                v[r][e] = upper ? __fsub_rn(other, mine) : __fadd_rn(mine, other);
            }
    }
#pragma unroll
    for (int s = 0; s < 3; ++s) {   // h = 128, 256, 512: across r
#pragma unroll
        for (int r = 0; r < 8; ++r)
            if (!((r >> s) & 1)) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float a = v[r][e], b = v[r | (1 << s)][e];
                    v[r][e] = __fadd_rn(a, b);
                    v[r | (1 << s)][e] = __fsub_rn(a, b);
                }
            }
    }
#pragma unroll
    for (int r = 0; r < 8; ++r)
#pragma unroll
        for (int e = 0; e < 4; ++e) v[r][e] = __fmul_rn(v[r][e], 0.03125f);
}

// ---- rotation split over warps: one warp per 128-element slice ----------------------------------
// A 1024-block is eight slices r = 0..7 of 128 consecutive elements; lane l of the slice's warp holds
// elements 4l .. 4l+3.  The butterflies with h = 1 .. 64 stay inside a slice (front); those with
// h = 128, 256, 512 combine the eight slices element by element (back), through shared memory.  Every
// output is still produced by the same a + b / a - b as in fwht1024_warp, stage by stage, so the bits
// are the same: a - b is computed as (-b) + a ... with IEEE addition that is the same rounding.
__device__ __forceinline__ void fwht_slice_front(float (&v)[4], int lane) {
    {
        const float a = v[0], b = v[1], c = v[2], d = v[3];
        const float s0 = __fadd_rn(a, b), s1 = __fsub_rn(a, b), s2 = __fadd_rn(c, d), s3 = __fsub_rn(c, d);
        v[0] = __fadd_rn(s0, s2); v[2] = __fsub_rn(s0, s2);
        v[1] = __fadd_rn(s1, s3); v[3] = __fsub_rn(s1, s3);
    }
#pragma unroll
    for (int s = 0; s < 5; ++s) {
        const bool upper = (lane >> s) & 1;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float mine = v[e];
            const float other = __shfl_xor_sync(0xffffffffu, mine, 1 << s);
            v[e] = upper ? __fsub_rn(other, mine) : __fadd_rn(mine, other);
        }
    }
}
// `block` points at the eight front-transformed slices of one 1024-block ([8][32] float4); returns
// slice r of the finished rotation (scaled by 1/32) for this lane.
__device__ __forceinline__ void fwht_slice_back(const float4 *block, int r, int lane, float (&out)[4]) {
    float a[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float4 f = block[(r ^ j) * 32 + lane];
        a[j][0] = f.x; a[j][1] = f.y; a[j][2] = f.z; a[j][3] = f.w;
    }
    // the element at index q of a pair (q, q | h) becomes a_lower + a_upper, the upper one a_lower - a_upper;
    // with m = sign mask when this slice is the upper one:  new(q) = partner + (own ^ m)
    const uint32_t m0 = (r & 1) ? 0x80000000u : 0u, m1 = (r & 2) ? 0x80000000u : 0u, m2 = (r & 4) ? 0x80000000u : 0u;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        float u[4];      // h = 128 at slices r, r^2, r^4, r^6
#pragma unroll
        for (int k = 0; k < 4; ++k)
            u[k] = __fadd_rn(a[2 * k + 1][e], __uint_as_float(__float_as_uint(a[2 * k][e]) ^ m0));
        // h = 256 at slices r (u[0] with u[1]) and r^4 (u[2] with u[3])
        const float w0 = __fadd_rn(u[1], __uint_as_float(__float_as_uint(u[0]) ^ m1));
        const float w1 = __fadd_rn(u[3], __uint_as_float(__float_as_uint(u[2]) ^ m1));
        // h = 512 at slice r
        out[e] = __fmul_rn(__fadd_rn(w1, __uint_as_float(__float_as_uint(w0) ^ m2)), 0.03125f);
    }
}

// blocks = n_tok * (n_in / 1024) warps.  X [n_tok][n_in] read-only; x_rot (nullable, may alias X)
// receives the rotated values; xq (nullable) the Q8_1 blocks at chunk * n_tok + tok.
template <bool VEC>
__global__ void __launch_bounds__(128) fwht_quant_kernel(const float *X, const float *__restrict__ signs, float *x_rot,
                                                         uint32_t *__restrict__ xq, int n_in, int n_tok) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    const int lane = threadIdx.x & 31;
    const int blocks_per_tok = n_in / FWHT_N;
    const long long nwarps = (long long)blocks_per_tok * n_tok;
    const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w >= nwarps) return;
    const int tok = (int)(w / blocks_per_tok);
    const int blk = (int)(w - (long long)tok * blocks_per_tok);
    const size_t base = (size_t)tok * n_in + (size_t)blk * FWHT_N;

    float v[8][4];
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        const float4 f = load_f4<VEC>(X + base + r * 128 + 4 * lane);
        v[r][0] = f.x; v[r][1] = f.y; v[r][2] = f.z; v[r][3] = f.w;
    }
    if (signs) {
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            const float4 s = load_f4<VEC>(signs + (size_t)blk * FWHT_N + r * 128 + 4 * lane);
            v[r][0] = __fmul_rn(v[r][0], s.x); v[r][1] = __fmul_rn(v[r][1], s.y);
            v[r][2] = __fmul_rn(v[r][2], s.z); v[r][3] = __fmul_rn(v[r][3], s.w);
        }
    }
    fwht1024_warp(v, lane);
    if (x_rot) {
#pragma unroll
        for (int r = 0; r < 8; ++r)
            store_f4<VEC>(x_rot + base + r * 128 + 4 * lane, make_float4(v[r][0], v[r][1], v[r][2], v[r][3]));
    }
    if (xq) {
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            uint32_t word, header;
            quantise_chunk_8lanes(v[r], lane, word, header);
            const int chunk = blk * 32 + r * 4 + (lane >> 3);
            uint32_t *dst = xq + 9 * ((size_t)chunk * n_tok + tok);
            dst[1 + (lane & 7)] = word;
            if ((lane & 7) == 0) dst[0] = header;
        }
    }
}

}  // namespace b200
