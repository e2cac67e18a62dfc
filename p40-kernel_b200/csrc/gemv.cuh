// gemv.cuh -- decode mat-vec y = W . x over PQ2_0 weights and permuted Q8_1 activations.
//
// Replaces, for sm_100a, gemv_pq2_0_p40_kernel (src/kernels/gemv_p40.cu:82-165).  The value of
// every output row is the reference's host function pq2_0_row_dot_perm (src/pq2_0.h:183-191):
// int32 chunk sums, each scaled as (dw * da) * (float)sumi, added in fp32 in block-then-chunk
// order.  This kernel keeps that order, so y is bit-identical to the host, not merely close.
//
// Shape of the kernel (B200: the op is a pure stream of 34-byte blocks from HBM):
//   * a CTA owns a run of consecutive rows.  Rows are contiguous in memory and 16-byte aligned
//     when n_in/128 is even, so the run is ONE aligned span; it is fetched by a few 1-D bulk
//     async copies (TMA, no multicast) into shared memory, one mbarrier per stage, all issued by
//     one thread before anything else happens -- before the wait on the previous kernel of the
//     stream when the launch is programmatic, because weights never depend on it;
//   * the Q8_1 vector is re-laid in shared memory as one 336-byte record per 256 activations
//     (8 chunks x 32 int8, 8 scales as fp32, 8 values of -64*s), a stride that keeps 16-byte
//     loads of neighbouring lanes in different banks;
//   * an item is one pair of weight blocks (68 bytes = 17 words) for RR consecutive rows.  A lane
//     reads its 17 words at stride 17 -- conflict-free -- funnel-shifts the 2-byte-offset codes of
//     the even block, and runs 16 dp4a per chunk with the activation registers shared by RR rows;
//   * the fp32 term of each chunk overwrites the first 8 words of the item's own weight bytes;
//     after the CTA's items are done, one lane per row adds the row's terms in order.
#pragma once

#include "common.cuh"

namespace b200 {

constexpr int GEMV_MAX_STAGES = 16;
constexpr int ACT_REC_WORDS = 84;   // 64 words int8 + 8 fp32 scales + 8 int32 (-64*s) + 4 pad

struct GemvPlan {
    int rows_per_cta;     // multiple of RR
    int rows_per_stage;   // multiple of 4 (keeps every bulk copy 16-byte aligned)
    int threads;
    int rr;
    int smem_bytes;
};

// Re-lay the Q8_1 vector (global, 9 words per chunk) into padded per-pair records.
__device__ __forceinline__ void stage_activations(const uint32_t *__restrict__ xq, uint32_t *rec, int nchunks) {
    for (int i = threadIdx.x; i < nchunks * 9; i += blockDim.x) {
        const int chunk = i / 9, w = i - chunk * 9;
        const uint32_t v = __ldg(xq + i);
        uint32_t *r = rec + (chunk >> 3) * ACT_REC_WORDS;
        const int cc = chunk & 7;
        if (w == 0) {
            r[64 + cc] = __float_as_uint(f16_bits_to_f32(v & 0xFFFFu));
            r[72 + cc] = (uint32_t)(-64 * (int)(short)(v >> 16));
        } else {
            r[cc * 8 + (w - 1)] = v;
        }
    }
}

// Sequential fp32 sum of a row's terms, one lane per row.  `row_words` is the distance between
// rows in words; lanes whose rows fall in the same bank start a few steps apart (skew) so that
// their loads hit different banks.  term(i) gives the word offset of term i inside the row.
template <typename TermOffset>
__device__ __forceinline__ float ordered_row_sum(const float *row_base, int nterms, int skew, int max_skew,
                                                 TermOffset term) {
    float acc = 0.0f;
    for (int k = 0; k < nterms + max_skew; ++k) {
        const int i = k - skew;
        if (i >= 0 && i < nterms) acc = __fadd_rn(acc, row_base[term(i)]);
    }
    return acc;
}

__host__ __device__ inline int gcd_int(int a, int b) { while (b) { int t = a % b; a = b; b = t; } return a; }

template <int RR>
__global__ void __launch_bounds__(256, 1) gemv_pq2_kernel(const uint8_t *__restrict__ W, const uint32_t *__restrict__ xq,
                                                       float *__restrict__ y, int n_out, int npairs, int rows_per_cta,
                                                       int rows_per_stage) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem);                       // GEMV_MAX_STAGES barriers
    uint32_t *act = reinterpret_cast<uint32_t *>(smem + 128);                  // npairs records
    uint32_t *wsm = act + (size_t)npairs * ACT_REC_WORDS;                      // rows_per_cta * 17 * npairs words

    const int row0 = blockIdx.x * rows_per_cta;
    const int rows_here = min(rows_per_cta, n_out - row0);
    const int row_words = 17 * npairs;
    const size_t row_bytes = (size_t)row_words * 4;
    const int nstages = (rows_here + rows_per_stage - 1) / rows_per_stage;

    if (threadIdx.x == 0) {
        for (int s = 0; s < nstages; ++s) mbar_init(&bars[s], 1);
        mbar_fence_init();
        const uint64_t pol = policy_evict_first();
        const uint8_t *src = W + (size_t)row0 * row_bytes;
        for (int s = 0; s < nstages; ++s) {
            const int r_begin = s * rows_per_stage;
            const int r_cnt = min(rows_per_stage, rows_here - r_begin);
            const uint32_t bytes = (uint32_t)(r_cnt * row_bytes);
            const uint32_t bulk = bytes & ~15u;
            uint8_t *dst = reinterpret_cast<uint8_t *>(wsm) + (size_t)r_begin * row_bytes;
            if (bulk) {
                mbar_expect_tx(&bars[s], bulk);
                bulk_g2s(dst, src + (size_t)r_begin * row_bytes, bulk, &bars[s], pol);
            } else {
                mbar_expect_tx(&bars[s], 0);
            }
            // a ragged last stage (row count not a multiple of 4) leaves < 16 bytes for plain loads
            for (uint32_t o = bulk; o < bytes; o += 4)
                *reinterpret_cast<uint32_t *>(dst + o) = ldg_nc_u32(src + (size_t)r_begin * row_bytes + o);
        }
    }
    pdl_launch_dependents();
    pdl_wait_prior_grid();          // activations (and y) belong to the previous kernel until here
    stage_activations(xq, act, npairs * 8);
    __syncthreads();                // records + barrier inits + ragged-tail words visible to all

    const int ngroups = (rows_here + RR - 1) / RR;
    const int nitems = ngroups * npairs;
    for (int item = threadIdx.x; item < nitems; item += blockDim.x) {
        const int g = item / npairs, q = item - g * npairs;
        const int r_first = g * RR;
        // every row of the group lies in one stage when rows_per_stage % RR == 0
        if (!mbar_wait_bounded(&bars[r_first / rows_per_stage], 0)) break;

        uint32_t w[RR][17];
#pragma unroll
        for (int rr = 0; rr < RR; ++rr) {
            // rows past the end of a ragged group re-read the group's first row (never stored)
            const int r = (r_first + rr < rows_here) ? r_first + rr : r_first;
            const uint32_t *p = wsm + (size_t)r * row_words + 17 * q;
#pragma unroll
            for (int j = 0; j < 17; ++j) w[rr][j] = p[j];
        }
        const uint32_t *rec = act + q * ACT_REC_WORDS;
        float dw[RR][2];
#pragma unroll
        for (int rr = 0; rr < RR; ++rr) {
            dw[rr][0] = f16_bits_to_f32(w[rr][0] & 0xFFFFu);
            dw[rr][1] = f16_bits_to_f32(w[rr][8] >> 16);
        }
        const int4 sc0 = *reinterpret_cast<const int4 *>(rec + 64), sc1 = *reinterpret_cast<const int4 *>(rec + 68);
        const int4 in0 = *reinterpret_cast<const int4 *>(rec + 72), in1 = *reinterpret_cast<const int4 *>(rec + 76);
        const int scale_bits[8] = {sc0.x, sc0.y, sc0.z, sc0.w, sc1.x, sc1.y, sc1.z, sc1.w};
        const int inits[8] = {in0.x, in0.y, in0.z, in0.w, in1.x, in1.y, in1.z, in1.w};
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) {
            const int4 lo = *reinterpret_cast<const int4 *>(rec + cc * 8);
            const int4 hi = *reinterpret_cast<const int4 *>(rec + cc * 8 + 4);
            const int a[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
            const float da = __int_as_float(scale_bits[cc]);
            const int init = inits[cc];
#pragma unroll
            for (int rr = 0; rr < RR; ++rr) {
                uint32_t c0, c1;
                if (cc < 4) {   // even block: codes start 2 bytes into word 0
                    c0 = __funnelshift_r(w[rr][2 * cc], w[rr][2 * cc + 1], 16);
                    c1 = __funnelshift_r(w[rr][2 * cc + 1], w[rr][2 * cc + 2], 16);
                } else {        // odd block: codes are word-aligned from word 9
                    c0 = w[rr][2 * cc + 1];
                    c1 = w[rr][2 * cc + 2];
                }
                const int sumi = chunk_sumi_scaled(c0, c1, a, init);
                const float term = __fmul_rn(__fmul_rn(dw[rr][cc >> 2], da), (float)sumi);
                if (r_first + rr < rows_here)
                    reinterpret_cast<float *>(wsm)[(size_t)(r_first + rr) * row_words + 17 * q + cc] = term;
            }
        }
    }
    __syncthreads();

    // one lane per row: ordered sum of the 8 * npairs terms
    const int bank_step = row_words & 31;
    const int distinct = 32 / gcd_int(bank_step == 0 ? 32 : bank_step, 32);   // rows before banks repeat
    const int max_skew = (32 / distinct) - 1;
    for (int r = threadIdx.x; r < rows_here; r += blockDim.x) {
        const int skew = (r & 31) / distinct;
        const float *base = reinterpret_cast<const float *>(wsm) + (size_t)r * row_words;
        y[row0 + r] = ordered_row_sum(base, 8 * npairs, skew, max_skew,
                                      [](int i) { return 17 * (i >> 3) + (i & 7); });
    }
}

// ---- fallback for shapes the staged kernel does not take (odd block count, unaligned W) ---------
// One warp per row, 2-byte loads straight from global, same term order.
__global__ void __launch_bounds__(256) gemv_pq2_generic_kernel(const uint8_t *__restrict__ W,
                                                               const uint8_t *__restrict__ xq, float *__restrict__ y,
                                                               int n_out, int nblocks) {
    constexpr int SEG = 512;                     // chunks summed per pass
    __shared__ float terms[8][SEG];
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row = blockIdx.x * 8 + warp;
    if (row >= n_out) return;
    const uint8_t *wrow = W + (size_t)row * nblocks * W_BLOCK_BYTES;
    const int nchunks = nblocks * 4;
    float acc = 0.0f;
    for (int c0 = 0; c0 < nchunks; c0 += SEG) {
        const int n = min(SEG, nchunks - c0);
        for (int i = lane; i < n; i += 32) {
            const int c = c0 + i;
            const uint8_t *wb = wrow + (size_t)(c >> 2) * W_BLOCK_BYTES;
            const uint8_t *cp = wb + 2 + 8 * (c & 3);
            const uint32_t c0w = ldg_nc_u16(cp) | (ldg_nc_u16(cp + 2) << 16);
            const uint32_t c1w = ldg_nc_u16(cp + 4) | (ldg_nc_u16(cp + 6) << 16);
            const uint32_t *ab = reinterpret_cast<const uint32_t *>(xq + (size_t)c * A_BLOCK_BYTES);
            const uint32_t hdr = __ldg(ab);
            int a[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) a[k] = (int)__ldg(ab + 1 + k);
            const int sumi = chunk_sumi_scaled(c0w, c1w, a, -64 * (int)(short)(hdr >> 16));
            const float d = __fmul_rn(f16_bits_to_f32(ldg_nc_u16(wb)), f16_bits_to_f32(hdr & 0xFFFFu));
            terms[warp][i] = __fmul_rn(d, (float)sumi);
        }
        __syncwarp();
        if (lane == 0)
            for (int i = 0; i < n; ++i) acc = __fadd_rn(acc, terms[warp][i]);
        __syncwarp();
    }
    if (lane == 0) y[row] = acc;
}

// ---- parity probe: raw int32 chunk sums ---------------------------------------------------------
__global__ void __launch_bounds__(256) gemv_chunk_sums_kernel(const uint8_t *__restrict__ W,
                                                              const uint8_t *__restrict__ xq, int32_t *__restrict__ out,
                                                              long long row0, int n_rows, int nblocks) {
    const int nchunks = nblocks * 4;
    const long long total = (long long)n_rows * nchunks;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(i / nchunks), c = (int)(i - (long long)r * nchunks);
        const uint8_t *wb = W + ((size_t)(row0 + r) * nblocks + (c >> 2)) * W_BLOCK_BYTES;
        const uint8_t *cp = wb + 2 + 8 * (c & 3);
        const uint32_t c0w = ldg_nc_u16(cp) | (ldg_nc_u16(cp + 2) << 16);
        const uint32_t c1w = ldg_nc_u16(cp + 4) | (ldg_nc_u16(cp + 6) << 16);
        const uint32_t *ab = reinterpret_cast<const uint32_t *>(xq + (size_t)c * A_BLOCK_BYTES);
        int a[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) a[k] = (int)__ldg(ab + 1 + k);
        out[i] = chunk_sumi_scaled(c0w, c1w, a, -64 * (int)(short)(__ldg(ab) >> 16));
    }
}

}  // namespace b200
