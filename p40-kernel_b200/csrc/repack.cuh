// repack.cuh -- the aligned repacked weight layout and the fused quantise + mat-vec over it.
//
// Layout of one row, nb = n_in/128 blocks, nb % 8 == 0 (src/pq2_0_repack.h:16-57): nb fp16 scales,
// then 4 planes of nb 8-byte units; unit u = plane * nb + block holds code bytes 8*plane..8*plane+7
// of that block and meets activation chunk 4*block + plane.  Row stride stays 34 * nb.
//
// Replaces, for sm_100a, repack_pq2_0_kernel and gemv_repack_p40_kernel
// (src/kernels/gemv_repack_p40.cu:165-192, 91-162).  The output row value is the reference's host
// function repack_row_dot (src/pq2_0_repack.h:122-138): terms (dw * da) * (float)sumi added in
// UNIT order, i.e. plane-major -- a different fp32 order from the plain mat-vec.  The kernel of this file keeps that
// order when asked to (bonsai_b200_set_option("gemv_order", 1): bit-identical, its whole share resident in shared
// memory) and otherwise adds the terms of a row by a warp; the DEFAULT of bonsai_p40_gemv_repack is the streaming
// kernel of gemv_stream.cuh (REPACK form: ring of tiles, 8-byte aligned unit loads, the lane order of the plain
// mat-vec, to whose result it is bit-identical) whenever the vector is 16-byte aligned and n_in a multiple of 1024.
#pragma once

#include "activation.cuh"
#include "gemv.cuh"

namespace b200 {

constexpr int RP_REC_WORDS = 12;   // 8 words int8 + fp32 scale + int32 (-64*s) + 2 pad: stride 48 B

// One thread per 8-byte unit; destination stores are aligned and coalesced.
__global__ void __launch_bounds__(256) repack_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst,
                                                     long long n_out, int nb) {
    const long long total = n_out * 4 * nb;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long row = i / (4 * nb);
        const int u = (int)(i - row * 4 * nb);
        const int p = u / nb, b = u - p * nb;
        const uint8_t *s = src + ((size_t)row * nb + b) * W_BLOCK_BYTES;
        uint8_t *drow = dst + (size_t)row * nb * W_BLOCK_BYTES;
        const uint8_t *cp = s + 2 + 8 * p;   // 2-byte aligned source
        uint2 v;
        v.x = ldg_nc_u16(cp) | (ldg_nc_u16(cp + 2) << 16);
        v.y = ldg_nc_u16(cp + 4) | (ldg_nc_u16(cp + 6) << 16);
        *reinterpret_cast<uint2 *>(drow + 2 * nb + 8 * (size_t)u) = v;
        if (p == 0) *reinterpret_cast<unsigned short *>(drow + 2 * b) = (unsigned short)ldg_nc_u16(s);
    }
}

// The same with both sides moved as 16-byte words: a row of either layout is 34 * nb bytes, a multiple of 16 when
// nb % 8 == 0, so a run of rows is one aligned range.  A CTA stages rows_per_pass source rows in shared memory, then
// every thread builds one 16-byte destination word (8 scales, or two units of one plane) from 2-byte shared reads;
// consecutive threads read blocks 68 bytes = 17 words apart, which no two lanes share a bank on.
constexpr int RPK_SMEM_BYTES = 32 * 1024;

__global__ void __launch_bounds__(256) repack_staged_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst,
                                                            long long n_out, int nb, int rows_per_pass) {
    extern __shared__ __align__(16) uint8_t rpk_sm[];
    const int row_bytes = nb * W_BLOCK_BYTES;
    const int wpr = row_bytes / 16, scale_words = nb / 8;
    const long long passes = (n_out + rows_per_pass - 1) / rows_per_pass;
    for (long long ps = blockIdx.x; ps < passes; ps += gridDim.x) {
        const long long r0 = ps * rows_per_pass;
        const int rows = (int)((n_out - r0 < rows_per_pass) ? (n_out - r0) : rows_per_pass);
        const int words = rows * wpr;
        const uint4 *s4 = reinterpret_cast<const uint4 *>(src + (size_t)r0 * row_bytes);
        uint4 *d4 = reinterpret_cast<uint4 *>(dst + (size_t)r0 * row_bytes);
        for (int i = threadIdx.x; i < words; i += 256) reinterpret_cast<uint4 *>(rpk_sm)[i] = __ldg(s4 + i);
        __syncthreads();
        for (int i = threadIdx.x; i < words; i += 256) {
            const int r = i / wpr, w = i - r * wpr;
            const unsigned short *rs = reinterpret_cast<const unsigned short *>(rpk_sm + (size_t)r * row_bytes);
            uint4 v;
            if (w < scale_words) {
                const unsigned short *q = rs + 17 * 8 * w;   // a block is 17 half-words
                v.x = q[0] | ((uint32_t)q[17] << 16);
                v.y = q[34] | ((uint32_t)q[51] << 16);
                v.z = q[68] | ((uint32_t)q[85] << 16);
                v.w = q[102] | ((uint32_t)q[119] << 16);
            } else {
                const int u = 2 * (w - scale_words);
                const int p = u / nb, b = u - p * nb;
                const unsigned short *q = rs + 17 * b + 1 + 4 * p;
                v.x = q[0] | ((uint32_t)q[1] << 16);
                v.y = q[2] | ((uint32_t)q[3] << 16);
                v.z = q[17] | ((uint32_t)q[18] << 16);
                v.w = q[19] | ((uint32_t)q[20] << 16);
            }
            d4[i] = v;
        }
        __syncthreads();
    }
}

// TREE: the terms of a row are added by a warp (lane l adds units l, l + 32, ... in ascending order, then a 5-step
// butterfly) -- a fixed order like that of the default mat-vec, within 1e-5 of repack_row_dot; !TREE: by one lane in
// unit order, bit-identical to repack_row_dot (bonsai_b200_set_option("gemv_order", 1)), several times slower.
template <int RR, bool VEC, bool TREE>
__global__ void __launch_bounds__(256) gemv_repack_kernel(const uint8_t *__restrict__ W, const float *__restrict__ x,
                                                          float *__restrict__ y, int n_out, int nb, int rows_per_cta,
                                                          int rows_per_stage) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem);
    uint32_t *act = reinterpret_cast<uint32_t *>(smem + GEMV_BAR_BYTES);   // 4*nb records, indexed by unit
    uint32_t *wsm = act + (size_t)4 * nb * RP_REC_WORDS;

    const int row0 = blockIdx.x * rows_per_cta;
    const int rows_here = min(rows_per_cta, n_out - row0);
    const size_t row_bytes = (size_t)nb * W_BLOCK_BYTES;               // multiple of 16 (nb % 8 == 0)
    const int row_words = (int)(row_bytes / 4);
    const int nstages = (rows_here + rows_per_stage - 1) / rows_per_stage;

    if (threadIdx.x == 0) {
        for (int s = 0; s < nstages; ++s) mbar_init(&bars[s], 1);
        mbar_fence_init();
        const uint64_t pol = policy_evict_first();
        for (int s = 0; s < nstages; ++s) {
            const int r_begin = s * rows_per_stage;
            const int r_cnt = min(rows_per_stage, rows_here - r_begin);
            const uint32_t bytes = (uint32_t)(r_cnt * row_bytes);
            mbar_expect_tx(&bars[s], bytes);
            bulk_g2s(reinterpret_cast<uint8_t *>(wsm) + (size_t)r_begin * row_bytes,
                     W + ((size_t)row0 + r_begin) * row_bytes, bytes, &bars[s], pol);
        }
    }
    pdl_launch_dependents();
    pdl_wait_prior_grid();

    // fused quantiser: 8 lanes per 32-chunk, record of chunk 4*b + p stored at unit p*nb + b.
    // Loads run four iterations ahead of the shuffles that consume them.
    {
        const int lane = threadIdx.x & 31;
        const int ngroups4 = nb * 32;   // float4 groups in x: a multiple of 32, so whole warps are live
        for (int i0 = threadIdx.x & ~31; i0 < ngroups4; i0 += 4 * blockDim.x) {
            float4 f[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const int i = i0 + b * blockDim.x + lane;
                f[b] = i < ngroups4 ? load_f4<VEC>(x + 4 * (size_t)i) : make_float4(0, 0, 0, 0);
            }
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const int i = i0 + b * blockDim.x + lane;
                if (i0 + b * blockDim.x >= ngroups4) break;   // warp-uniform
                const float v[4] = {f[b].x, f[b].y, f[b].z, f[b].w};
                uint32_t word, header;
                quantise_chunk_8lanes(v, lane, word, header);
                const int chunk = i >> 3;
                uint32_t *rec = act + ((chunk & 3) * nb + (chunk >> 2)) * RP_REC_WORDS;
                rec[lane & 7] = word;
                if ((lane & 7) == 0) {
                    rec[8] = __float_as_uint(f16_bits_to_f32(header & 0xFFFFu));
                    rec[9] = (uint32_t)(-64 * (int)(short)(header >> 16));
                }
            }
        }
    }
    __syncthreads();

    const int nunits = 4 * nb;
    const int codes_w = nb / 2;        // word offset of the code planes inside a row
    const int ngroups = (rows_here + RR - 1) / RR;
    const int nitems = ngroups * nunits;
    for (int item = threadIdx.x; item < nitems; item += blockDim.x) {
        const int g = item / nunits, u = item - g * nunits;
        const int r_first = g * RR;
        if (!mbar_wait_bounded(&bars[r_first / rows_per_stage], 0)) break;
        const uint32_t *rec = act + u * RP_REC_WORDS;
        const int4 lo = *reinterpret_cast<const int4 *>(rec);
        const int4 hi = *reinterpret_cast<const int4 *>(rec + 4);
        const int a[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        const uint2 sc = *reinterpret_cast<const uint2 *>(rec + 8);
        const float da = __uint_as_float(sc.x);
        const int b = u % nb;
#pragma unroll
        for (int rr = 0; rr < RR; ++rr) {
            if (r_first + rr >= rows_here) break;
            uint32_t *row = wsm + (size_t)(r_first + rr) * row_words;
            const uint2 codes = *reinterpret_cast<const uint2 *>(row + codes_w + 2 * u);
            const uint32_t dbits = reinterpret_cast<const unsigned short *>(row)[b];
            const int sumi = chunk_sumi_scaled(codes.x, codes.y, a, (int)sc.y);
            // (dw * da) * sumi: the association of repack_unit_dot (src/pq2_0_repack.h:125-128)
            const float term = __fmul_rn(__fmul_rn(f16_bits_to_f32(dbits), da), (float)sumi);
            reinterpret_cast<float *>(row)[codes_w + 2 * u] = term;
        }
    }
    __syncthreads();

    if (TREE) {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
        for (int r = warp; r < rows_here; r += nwarp) {
            const float *base = reinterpret_cast<const float *>(wsm) + (size_t)r * row_words + codes_w;
            float acc = 0.0f;
            for (int u = lane; u < nunits; u += 32) acc = __fadd_rn(acc, base[2 * u]);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, o));
            if (lane == 0) y[row0 + r] = acc;
        }
        return;
    }
    // one lane per row: terms added in unit order, four loads in flight per step
    int skew, max_skew;
    row_skew(row_words, threadIdx.x & 31, skew, max_skew);
    for (int r = threadIdx.x; r < rows_here; r += blockDim.x) {
        const float *base = reinterpret_cast<const float *>(wsm) + (size_t)r * row_words + codes_w;
        float acc = 0.0f;
        for (int k = 0; k < nb + max_skew; ++k) {       // nunits / 4 = nb steps
            const int s4 = k - skew;
            if (s4 >= 0 && s4 < nb) {
                float t[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) t[j] = base[2 * (4 * s4 + j)];
#pragma unroll
                for (int j = 0; j < 4; ++j) acc = __fadd_rn(acc, t[j]);
            }
        }
        y[row0 + r] = acc;
    }
}

}  // namespace b200
