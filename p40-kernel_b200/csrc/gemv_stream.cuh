// gemv_stream.cuh -- the default decode mat-vec: y = W . x, PQ2_0 weights x permuted Q8_1 activations.
//
// Replaces, for sm_100a, gemv_pq2_0_p40_kernel (src/kernels/gemv_p40.cu:82-165).  Every int32 chunk
// sum and every fp32 term (dw * da) * (float)sumi equals the reference's host code
// (src/pq2_0.h:149-172) bit for bit; the terms of a row are added in a fixed, launch-independent
// order that differs from the host's sequential one (each of 8 lanes adds the terms of every 8th
// block in ascending order, then a 3-step butterfly joins the lanes, then row segments are joined
// in ascending order), like the reference's own device kernel, whose lanes stride over blocks and
// tree-reduce (src/kernels/gemv_p40.cu:104,155-159).  The kernel that keeps the host's order term by
// term is gemv_ring_kernel (gemv.cuh), selectable at run time.
//
// Shape (B200): one persistent CTA per SM streams its run of rows through a ring of shared-memory
// slots fed by 1-D bulk async copies (TMA, CTA-local); it stays under half of an SM's shared
// memory so that, with programmatic launches, the next kernel's CTA is resident and prefetching
// while this one drains.  A tile is (a few row quads) x (a row segment of <= 40 blocks); a task is
// one quad of one tile, taken by one warp: lane = (row of the quad, one of 8 block lanes), the lane
// owns blocks bl, bl + 8, ... of the segment.  It first copies its blocks into registers and gives
// the slot back, so shared memory holds bytes in flight rather than bytes being multiplied; then it
// multiplies from registers.  Neighbouring lanes read neighbouring 34-byte blocks (conflict-free up
// to the row stride), the four lanes of a block lane read the same activation bytes (one
// broadcast): no term buffers, no ordered adder, about 30 instructions per 32 weights.
#pragma once

#include "activation.cuh"
#include "common.cuh"
#include "gemv.cuh"

namespace b200 {

constexpr int STREAM_STEPS = 5;         // blocks per lane and task: segments hold at most 8 * 5 = 40 blocks
constexpr int STREAM_ACT_WORDS = 36;    // per block: 4 chunks x 8 words int8, 4 pad (stride 144 B: 8 blocks, 8 bank groups)

struct StreamParams {
    int n_out, nb;         // rows, blocks per row
    int rows_per_cta;      // multiple of 4
    int tr;                // rows per tile, multiple of 4: a tile is tr whole rows, one contiguous copy
    int nseg;              // segments per row; segment j starts at block j * seg_blocks
    int seg_blocks;        // blocks per segment (<= 8 * STREAM_STEPS), the last one takes the remainder
    int nslot;
    int tpt;               // tasks per tile = (tr / 4) * nseg
    uint32_t magic_tpt, magic_nseg, magic_nslot;   // ceil(2^32 / d), 0 for d == 1
};

// The multiply of one task when every block lane owns exactly STEPS blocks of the segment (segment
// length a multiple of 8 -- always the case when n_in is a multiple of 1024): no per-lane bounds, and
// every shared-memory address is the lane's base plus a compile-time offset (block b = bl + 8k sits
// 272 k bytes = 68 k words after block bl; its activation record 288 k words after that of bl).
// `release` runs between the copy into registers and the multiply: it hands the ring slot back.
// Same terms in the same order as the general loop below, so the bits do not depend on which runs.
template <int STEPS, typename Release>
__device__ __forceinline__ float stream_task_full(const uint8_t *rowp, int bl, int gb0, const uint32_t *act_q,
                                                  const float *act_s, const int *act_i, Release release) {
    const uint32_t *xw = reinterpret_cast<const uint32_t *>(rowp) + ((W_BLOCK_BYTES * bl + 2) >> 2);
    const uint8_t *dp = rowp + W_BLOCK_BYTES * bl;
    uint32_t x[STEPS][9];
    float dw[STEPS];
#pragma unroll
    for (int k = 0; k < STEPS; ++k) {
#pragma unroll
        for (int i = 0; i < 9; ++i) x[k][i] = xw[68 * k + i];
        dw[k] = f16_bits_to_f32(*reinterpret_cast<const unsigned short *>(dp + 272 * k));
    }
    release();
    const uint32_t sh = (gb0 & 1) ? 0u : 16u;           // codes start two bytes into a word for even blocks
    const uint32_t *aq = act_q + gb0 * STREAM_ACT_WORDS;
    const float *as = act_s + 4 * gb0;
    const int *ai = act_i + 4 * gb0;
    float acc = 0.0f;
#pragma unroll
    for (int k = 0; k < STEPS; ++k) {
        const float4 sc = *reinterpret_cast<const float4 *>(as + 32 * k);
        const int4 in = *reinterpret_cast<const int4 *>(ai + 32 * k);
        const float scale[4] = {sc.x, sc.y, sc.z, sc.w};
        const int inits[4] = {in.x, in.y, in.z, in.w};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int4 lo = *reinterpret_cast<const int4 *>(aq + 8 * STREAM_ACT_WORDS * k + c * 8);
            const int4 hi = *reinterpret_cast<const int4 *>(aq + 8 * STREAM_ACT_WORDS * k + c * 8 + 4);
            const int a[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
            const uint32_t c0 = __funnelshift_r(x[k][2 * c], x[k][2 * c + 1], sh);
            const uint32_t c1 = __funnelshift_r(x[k][2 * c + 1], x[k][2 * c + 2], sh);
            const int sumi = chunk_sumi_scaled(c0, c1, a, inits[c]);
            acc = __fadd_rn(acc, __fmul_rn(__fmul_rn(dw[k], scale[c]), (float)sumi));
        }
    }
    return acc;
}

// The general task: a last segment of any length (a lane past the end re-reads the last block and
// skips its terms).
template <int MAXSTEPS, typename Release>
__device__ __forceinline__ float stream_task_ragged(const uint8_t *rowp, int bl, int b0, int blocks, const uint32_t *act_q,
                                                    const float *act_s, const int *act_i, Release release) {
    uint32_t x[MAXSTEPS][9];
    float dw[MAXSTEPS];
#pragma unroll
    for (int k = 0; k < MAXSTEPS; ++k) {
        const int b = min(bl + 8 * k, blocks - 1);
        const uint32_t *xw = reinterpret_cast<const uint32_t *>(rowp) + ((W_BLOCK_BYTES * b + 2) >> 2);
#pragma unroll
        for (int i = 0; i < 9; ++i) x[k][i] = xw[i];
        dw[k] = f16_bits_to_f32(*reinterpret_cast<const unsigned short *>(rowp + W_BLOCK_BYTES * b));
    }
    release();
    float acc = 0.0f;
#pragma unroll
    for (int k = 0; k < MAXSTEPS; ++k) {
        const int b = bl + 8 * k;
        if (b < blocks) {
            const int gb = b0 + b;
            const uint32_t sh = (gb & 1) ? 0u : 16u;
            const float4 sc = *reinterpret_cast<const float4 *>(act_s + 4 * gb);
            const int4 in = *reinterpret_cast<const int4 *>(act_i + 4 * gb);
            const float scale[4] = {sc.x, sc.y, sc.z, sc.w};
            const int inits[4] = {in.x, in.y, in.z, in.w};
            const uint32_t *aq = act_q + gb * STREAM_ACT_WORDS;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int4 lo = *reinterpret_cast<const int4 *>(aq + c * 8);
                const int4 hi = *reinterpret_cast<const int4 *>(aq + c * 8 + 4);
                const int a[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
                const uint32_t c0 = __funnelshift_r(x[k][2 * c], x[k][2 * c + 1], sh);
                const uint32_t c1 = __funnelshift_r(x[k][2 * c + 1], x[k][2 * c + 2], sh);
                const int sumi = chunk_sumi_scaled(c0, c1, a, inits[c]);
                acc = __fadd_rn(acc, __fmul_rn(__fmul_rn(dw[k], scale[c]), (float)sumi));
            }
        }
    }
    return acc;
}

// One task: dispatches on the segment length (warp-uniform).  MAXSTEPS bounds the blocks a lane
// stages in registers (segments hold at most 8 * MAXSTEPS blocks).
template <int MAXSTEPS, typename Release>
__device__ __forceinline__ float stream_task(const uint8_t *rowp, int bl, int b0, int blocks, const uint32_t *act_q,
                                             const float *act_s, const int *act_i, Release release) {
    if ((blocks & 7) == 0) {
        const int steps = blocks >> 3;
        if (MAXSTEPS >= 5 && steps == 5) return stream_task_full<(MAXSTEPS >= 5 ? 5 : 1)>(rowp, bl, b0 + bl, act_q, act_s, act_i, release);
        if (MAXSTEPS >= 4 && steps == 4) return stream_task_full<(MAXSTEPS >= 4 ? 4 : 1)>(rowp, bl, b0 + bl, act_q, act_s, act_i, release);
        if (MAXSTEPS >= 3 && steps == 3) return stream_task_full<(MAXSTEPS >= 3 ? 3 : 1)>(rowp, bl, b0 + bl, act_q, act_s, act_i, release);
        if (MAXSTEPS >= 2 && steps == 2) return stream_task_full<(MAXSTEPS >= 2 ? 2 : 1)>(rowp, bl, b0 + bl, act_q, act_s, act_i, release);
        if (steps == 1) return stream_task_full<1>(rowp, bl, b0 + bl, act_q, act_s, act_i, release);
    }
    return stream_task_ragged<MAXSTEPS>(rowp, bl, b0, blocks, act_q, act_s, act_i, release);
}

// The same task over the REPACKED row layout (repack.cuh: nb fp16 scales, then four planes of nb 8-byte units; the
// unit of plane p and block b holds the codes that meet activation chunk 4 b + p): `row` is the start of the row in
// the slot, gb the block index in the row.  Eight-byte aligned loads, no funnel shifts; same terms (dw * da) * sumi,
// added per lane in ascending block and chunk order like the tasks above.
template <int MAXSTEPS, typename Release>
__device__ __forceinline__ float stream_task_repack(const uint8_t *row, int nb, int bl, int b0, int blocks, const uint32_t *act_q,
                                                    const float *act_s, const int *act_i, Release release) {
    uint2 cw[MAXSTEPS][4];
    float dw[MAXSTEPS];
    const unsigned short *sc16 = reinterpret_cast<const unsigned short *>(row);
    const uint2 *units = reinterpret_cast<const uint2 *>(row + 2 * nb);
#pragma unroll
    for (int k = 0; k < MAXSTEPS; ++k) {
        const int gb = b0 + min(bl + 8 * k, blocks - 1);
        dw[k] = f16_bits_to_f32(sc16[gb]);
#pragma unroll
        for (int p = 0; p < 4; ++p) cw[k][p] = units[p * nb + gb];
    }
    release();
    float acc = 0.0f;
#pragma unroll
    for (int k = 0; k < MAXSTEPS; ++k) {
        const int b = bl + 8 * k;
        if (b < blocks) {
            const int gb = b0 + b;
            const float4 sc = *reinterpret_cast<const float4 *>(act_s + 4 * gb);
            const int4 in = *reinterpret_cast<const int4 *>(act_i + 4 * gb);
            const float scale[4] = {sc.x, sc.y, sc.z, sc.w};
            const int inits[4] = {in.x, in.y, in.z, in.w};
            const uint32_t *aq = act_q + gb * STREAM_ACT_WORDS;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int4 lo = *reinterpret_cast<const int4 *>(aq + c * 8);
                const int4 hi = *reinterpret_cast<const int4 *>(aq + c * 8 + 4);
                const int a[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
                const int sumi = chunk_sumi_scaled(cw[k][c].x, cw[k][c].y, a, inits[c]);
                acc = __fadd_rn(acc, __fmul_rn(__fmul_rn(dw[k], scale[c]), (float)sumi));
            }
        }
    }
    return acc;
}

// Shared memory: [full[256] | done[256]] [act int8: nb * 36 words] [act scale: nb * 4 floats]
// [act -64*sum: nb * 4 ints] [partials: rows_per_cta * nseg floats] [quad counters: rows_per_cta / 4]
// [task counter] [ring: nslot * (tr * 34 * nb + 16)].
//   full[t] : tile t has landed in slot t % nslot             (1 arrival + copy bytes)
//   done[t] : every task of tile t has copied its blocks out   (live quads * nseg arrivals)
// Both are single-use (parity 0), so a warp that skipped tiles can never read a stale phase.
//
// FUSED = true is the one-launch projection: the CTA takes the fp32 activation vector instead of Q8_1
// blocks, rotates it (FWHT-1024, one warp per 1024-block) and quantises it straight into its own
// shared-memory tables while its first weight tiles are in flight; CTA 0 also writes the Q8_1 blocks
// to `xq_out` so that the caller's scratch holds what the two-launch form would have left there.
// REPACK = true (with FUSED) is bonsai_p40_gemv_repack: W is in the repacked layout and x is quantised WITHOUT a
// rotation (src/kernels/gemv_repack_p40.cu:91-162 fuses exactly that).
template <bool FUSED, bool REPACK = false>
__global__ void __launch_bounds__(512, 1) gemv_stream_kernel(const uint8_t *__restrict__ W, const uint32_t *__restrict__ xq,
                                                             float *__restrict__ y, const StreamParams P,
                                                             const float *__restrict__ x, const float *__restrict__ signs,
                                                             uint32_t *__restrict__ xq_out) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);
    uint64_t *done = full + RING_MAX_TILES;
    uint32_t *act_q = reinterpret_cast<uint32_t *>(smem + 2 * RING_MAX_TILES * 8);
    float *act_s = reinterpret_cast<float *>(act_q + (size_t)P.nb * STREAM_ACT_WORDS);
    int *act_i = reinterpret_cast<int *>(act_s + (size_t)P.nb * 4);
    float *partial = reinterpret_cast<float *>(act_i + (size_t)P.nb * 4);
    int *quad_count = reinterpret_cast<int *>(partial + (size_t)P.rows_per_cta * P.nseg);
    int *next_task = quad_count + ((P.rows_per_cta / 4 + 3) & ~3);
    uint8_t *ring = reinterpret_cast<uint8_t *>(next_task + 4);
    const size_t row_bytes = (size_t)P.nb * W_BLOCK_BYTES;
    const int slot_bytes = P.tr * (int)row_bytes + 16;

    const int row0 = blockIdx.x * P.rows_per_cta;
    const int rows_here = min(P.rows_per_cta, P.n_out - row0);
    if (rows_here <= 0) return;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int nwarps = blockDim.x >> 5;
    const int compute_warps = nwarps - 1;
    const int ntiles = (rows_here + P.tr - 1) / P.tr;
    const uint64_t pol = policy_evict_first();
    const uint8_t *src = W + (size_t)row0 * row_bytes;

    // Issues tile t (whole rows, contiguous in memory) into its slot; called by one lane.  A ragged
    // last tile can leave < 16 bytes for plain loads; they are stored before the arrive, which
    // releases them to the waiters together with the copied bytes.
    auto issue_tile = [&](int t) {
        // the slot was read through ordinary loads: order them before the asynchronous overwrite
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        const int slot = t - (int)fast_div((uint32_t)t, P.magic_nslot) * P.nslot;
        const int r_begin = t * P.tr;
        const int r_cnt = min(P.tr, rows_here - r_begin);
        uint8_t *dst = ring + (size_t)slot * slot_bytes;
        const uint32_t bytes = (uint32_t)(r_cnt * row_bytes);
        const uint32_t bulk = bytes & ~15u;
        const uint8_t *s = src + (size_t)r_begin * row_bytes;
        for (uint32_t o = bulk; o < bytes; o += 4) *reinterpret_cast<uint32_t *>(dst + o) = ldg_nc_u32(s + o);
        mbar_expect_tx(&full[t], bulk);
        if (bulk) bulk_g2s(dst, s, bulk, &full[t], pol);
    };

    // ---- prologue: barriers, two tiles, activations, the rest of the ring (issue order = return order)
    const int first_fill = min(P.nslot, ntiles);
    if (wid == compute_warps) {
        for (int t = lane; t < ntiles; t += 32) {
            const int r_cnt = min(P.tr, rows_here - t * P.tr);
            mbar_init(&full[t], 1);
            mbar_init(&done[t], (uint32_t)(((r_cnt + 3) / 4) * P.nseg));
        }
        mbar_fence_init();
        __syncwarp();
        if (lane == 0)
            for (int t = 0; t < min(2, first_fill); ++t) issue_tile(t);
    }
    for (int i = threadIdx.x; i < P.rows_per_cta / 4; i += blockDim.x) quad_count[i] = 0;
    if (threadIdx.x == 0) *next_task = 0;
    pdl_launch_dependents();
    pdl_wait_prior_grid();              // activations (and y) belong to the previous kernel until here
    if (FUSED) {
        // rotation + quantiser in the prologue: nb / 8 blocks of 1024 activations over the compute warps
        const int nfb = P.nb >> 3;
        bool first = true;
        for (int fb0 = 0; fb0 < nfb || first; fb0 += compute_warps) {
            const int fb = fb0 + wid;
            const bool live = wid < compute_warps && fb < nfb;
            float v[8][4];
            if (live) {
#pragma unroll
                for (int r = 0; r < 8; ++r) {
                    const float4 f = *reinterpret_cast<const float4 *>(x + (size_t)fb * FWHT_N + r * 128 + 4 * lane);
                    v[r][0] = f.x; v[r][1] = f.y; v[r][2] = f.z; v[r][3] = f.w;
                }
            }
            if (first) {
                // every warp has issued its first loads: the rest of the ring may queue behind them
                __syncthreads();
                if (wid == compute_warps && lane == 0)
                    for (int t = 2; t < first_fill; ++t) issue_tile(t);
                first = false;
            }
            if (live) {
                if (!REPACK && signs) {
#pragma unroll
                    for (int r = 0; r < 8; ++r) {
                        const float4 sg = *reinterpret_cast<const float4 *>(signs + (size_t)fb * FWHT_N + r * 128 + 4 * lane);
                        v[r][0] = __fmul_rn(v[r][0], sg.x); v[r][1] = __fmul_rn(v[r][1], sg.y);
                        v[r][2] = __fmul_rn(v[r][2], sg.z); v[r][3] = __fmul_rn(v[r][3], sg.w);
                    }
                }
                if (!REPACK) fwht1024_warp(v, lane);
#pragma unroll
                for (int r = 0; r < 8; ++r) {
                    uint32_t word, header;
                    quantise_chunk_8lanes(v[r], lane, word, header);
                    const int chunk = fb * 32 + r * 4 + (lane >> 3);
                    act_q[(chunk >> 2) * STREAM_ACT_WORDS + (chunk & 3) * 8 + (lane & 7)] = word;
                    if ((lane & 7) == 0) {
                        act_s[chunk] = f16_bits_to_f32(header & 0xFFFFu);
                        act_i[chunk] = -64 * (int)(short)(header >> 16);
                    }
                    if (blockIdx.x == 0 && xq_out) {
                        xq_out[9 * chunk + 1 + (lane & 7)] = word;
                        if ((lane & 7) == 0) xq_out[9 * chunk] = header;
                    }
                }
            }
        }
    } else {
        const int nchunks = P.nb * 4;
        uint32_t v[9];
        const bool mine = (int)threadIdx.x < nchunks;
        if (mine) act_chunk_load(xq, threadIdx.x, v);
        if (wid == compute_warps && lane == 0)
            for (int t = 2; t < first_fill; ++t) issue_tile(t);
        for (int chunk = threadIdx.x; chunk < nchunks; chunk += blockDim.x) {
            if (chunk != (int)threadIdx.x) act_chunk_load(xq, chunk, v);
            uint32_t *q = act_q + (chunk >> 2) * STREAM_ACT_WORDS + (chunk & 3) * 8;
            *reinterpret_cast<uint4 *>(q) = make_uint4(v[1], v[2], v[3], v[4]);
            *reinterpret_cast<uint4 *>(q + 4) = make_uint4(v[5], v[6], v[7], v[8]);
            act_s[chunk] = f16_bits_to_f32(v[0] & 0xFFFFu);
            act_i[chunk] = -64 * (int)(short)(v[0] >> 16);
        }
    }
    __syncthreads();                    // activation arrays, counters and barrier inits visible to all

    if (wid < compute_warps) {
        const int rr = lane & 3, bl = lane >> 2;
        const int ntasks = ntiles * P.tpt;
        for (;;) {
            // tasks are handed out in order to whichever warp is free, so a landed tile never waits
            // for one particular warp
            int task = 0;
            if (lane == 0) task = atomicAdd(next_task, 1);
            task = __shfl_sync(0xffffffffu, task, 0);
            if (task >= ntasks) break;
            const int t = (int)fast_div((uint32_t)task, P.magic_tpt);
            const int local = task - t * P.tpt;
            const int quad = (int)fast_div((uint32_t)local, P.magic_nseg);  // quad inside the tile
            const int j = local - quad * P.nseg;                            // segment of the row
            const int r_quad = t * P.tr + quad * 4;                         // first row of the quad (CTA-local)
            if (r_quad >= rows_here) continue;                              // padding quad of a ragged last tile
            const int slot = t - (int)fast_div((uint32_t)t, P.magic_nslot) * P.nslot;
            if (!mbar_wait_bounded(&full[t], 0)) break;
            const int b0 = j * P.seg_blocks;
            const int blocks = min(P.seg_blocks, P.nb - b0);
            // a row past the end of a ragged quad reads stale slot bytes; its sum is never stored
            const uint8_t *rowp = ring + (size_t)slot * slot_bytes + (size_t)(quad * 4 + rr) * row_bytes +
                                  (size_t)b0 * W_BLOCK_BYTES;

            // Phase A: the lane pulls its blocks (every 8th of the segment, at most STREAM_STEPS of them)
            // into registers and the warp hands the slot back at once -- the ring then holds bytes in
            // flight, not bytes being multiplied.  32 code bytes start at byte 34*b + 2 of the row: two
            // bytes into a word for even b, word-aligned for odd b; nine words cover them either way and
            // a funnel shift by 16 or 0 aligns them.  Phase B multiplies from registers against the
            // broadcast activation words.  (rowp is word-aligned: rows start on a word since nb is even,
            // and so do segments since seg_blocks is even.)
            auto release = [&]() {
                __syncwarp();
                if (lane == 0) mbar_arrive(&done[t]);   // release: every lane's loads above are complete
            };
            float acc = REPACK ? stream_task_repack<STREAM_STEPS>(ring + (size_t)slot * slot_bytes + (size_t)(quad * 4 + rr) * row_bytes,
                                                                  P.nb, bl, b0, blocks, act_q, act_s, act_i, release)
                               : stream_task<STREAM_STEPS>(rowp, bl, b0, blocks, act_q, act_s, act_i, release);
            acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 4));
            acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 8));
            acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 16));
            const int r = r_quad + rr;
            if (P.nseg == 1) {
                if (bl == 0 && r < rows_here) y[row0 + r] = acc;
            } else {
                // segments finish in any order: the warp that completes a quad's last one adds the
                // partial sums in ascending segment order
                if (bl == 0) partial[r * P.nseg + j] = acc;
                __syncwarp();
                int last = 0;
                if (lane == 0) {
                    __threadfence_block();
                    last = atomicAdd(&quad_count[r_quad >> 2], 1) == P.nseg - 1;
                }
                last = __shfl_sync(0xffffffffu, last, 0);
                if (last) {
                    __threadfence_block();
                    if (bl == 0 && r < rows_here) {
                        float total = partial[r * P.nseg];
                        for (int sgm = 1; sgm < P.nseg; ++sgm) total = __fadd_rn(total, partial[r * P.nseg + sgm]);
                        y[row0 + r] = total;
                    }
                }
            }
        }
    } else if (lane == 0) {
        // ---- copy warp: a slot is refilled as soon as every task of its previous tile has copied out --
        for (int t = first_fill; t < ntiles; ++t) {
            if (!mbar_wait_bounded(&done[t - P.nslot], 0)) return;
            issue_tile(t);
        }
    }
}

}  // namespace b200
