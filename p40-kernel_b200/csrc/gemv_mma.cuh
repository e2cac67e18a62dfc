// gemv_mma.cuh -- decode mat-vec with the integer products on the warp-level tensor-core instruction.
//
// Same job as gemv_stream_kernel (replaces gemv_pq2_0_p40_kernel, src/kernels/gemv_p40.cu:82-165): every int32
// chunk sum equals the reference's host code (src/pq2_0.h:149-169) bit for bit, every fp32 term is
// (dw * da) * (float)sumi as on the host (src/pq2_0.h:170-171), and the terms of a row are added in a fixed order
// that depends only on the row's length (below), never on the launch, the CTA or the position of the row.
//
// Why: the dp4a body is bound by instruction issue (8 masks + 8 dp4a + 4 joins + loads of the activation words per
// 32 weights and lane).  mma.sync.m16n8k32 (u8 x s8 -> s32) multiplies 16 weight rows by one K = 32 byte slice for
// 8 output columns in ONE instruction, and batch 1 leaves 7 of the 8 columns unused -- so the columns are given
// to eight different 32-weight CHUNKS instead:
//   * K slice of one instruction = field f (bits 2f, 2f+1 of every code byte) of the eight code words of one
//     weight block, masked IN PLACE (one AND per register, no shift: the byte holds 4^f * code);
//   * B = the int8 activations of the block's four chunks, chunk c only in column c ("block diagonal"), so
//     column c receives the sum over chunk c alone; a second block fills columns 4..7 of the same accumulators;
//   * the four fields have four accumulator sets, joined exactly as the dp4a body joins them:
//     64 * sumi = C3 + 4 C2 + 16 C1 + 64 C0 (C3 starts at -64 * s, which subtracts the activation sum);
//   * the factor 64 is taken out by the activation scale, stored as da / 64 (a power of two: every product and the
//     term are the host's bits).
// The B registers depend on the block pair only, not on the row, and every lane ends up with four useful sums
// (2 rows x 2 chunks), so conversion and scaling run on full warps.
//
// Work split: a tile is 16 consecutive rows x one row segment (<= 40 blocks, one or 16 bulk copies into a ring
// slot); an item is one block pair of a tile, items go round-robin to the compute warps.  Per item: B registers
// (1 load + 16 ANDs), 12 loads of code words, 32 ANDs, 8 MMAs, 12 joins, 20 for conversion, scales and adds.
// Summation order of a row: inside a pair, lane t of 4 adds chunks 2t, 2t+1 (ascending), a 2-step butterfly joins
// the 4 lanes; pairs are added in ascending order, then segments in ascending order.
#pragma once

#include "common.cuh"
#include "gemv.cuh"

namespace b200 {

constexpr int MMA_C = 15;                          // compute warps
constexpr int MMA_THREADS = (MMA_C + 2) * 32;      // + copy warp + adder warp
constexpr int MMA_MAX_SLOTS = 12;
constexpr int MMA_SEG_MAX = 40;                    // blocks per row segment (multiple of 8)
constexpr int MMA_GROUP_RING = 8;                  // row groups whose segment sums can be pending at once

struct MmaGeom {
    int n_out, nb;
    int ngroups;             // row groups of 16
    int nseg, seg_q, seg_r;  // segments in units of 8 blocks: segment j has seg_q + (j < seg_r) units (nseg == 1: nb blocks)
    int stride;              // bytes between the rows of a tile in its slot (multiple of 16)
    int contiguous;          // 1: a tile is one bulk copy (whole rows, stride == row bytes)
    int nslot, slot_bytes;
    int pairs_max;           // block pairs in the longest segment
    uint32_t magic_pairs, magic_nseg, magic_nslot;
};

__host__ __device__ inline int mma_seg_start(const MmaGeom &P, int j) {   // first block of segment j
    return P.nseg == 1 ? 0 : 8 * (j * P.seg_q + (j < P.seg_r ? j : P.seg_r));
}
__host__ __device__ inline int mma_seg_len(const MmaGeom &P, int j) {     // blocks of segment j
    return P.nseg == 1 ? P.nb : 8 * (P.seg_q + (j < P.seg_r ? 1 : 0));
}
// Shared memory in front of the ring: barriers, activation words (32 B per chunk), {da / 64, -64 s} per chunk,
// pair sums of every slot, segment sums of the row groups in flight.
__host__ __device__ inline size_t mma_fixed_bytes(const MmaGeom &P, int nslot) {
    const size_t b = 512 + (size_t)P.nb * 4 * 40 + (size_t)nslot * P.pairs_max * 64 + MMA_GROUP_RING * 64;
    return (b + 127) & ~(size_t)127;
}

__device__ __forceinline__ void mma_u8s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1, const int (&c)[4]) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]));
}
__device__ __forceinline__ void mbar_arrive_n(uint64_t *bar, uint32_t n) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(n) : "memory");
}

// The B operands of one block pair for lane (g = lane / 4, t = lane % 4): column g of the accumulators belongs to
// chunk g of the pair (block g / 4, chunk g % 4 of it).  Code word wi of a block (wi = t for the first K half,
// 4 + t for the second) belongs to chunk wi / 2 and is word wi % 2 of it, whose field f meets activation word
// 4 * (wi % 2) + f (src/pq2_0.h:158-166) -- for both halves that is word 4 * (t % 2) + f of the lane's own chunk,
// placed in the half whose chunk it is, zero elsewhere.
struct MmaPairB {
    uint32_t b[2][4][2];     // [block of the pair][field][K half]
    float da[2];             // da / 64 of chunks 2t, 2t + 1 of the pair (the lane's accumulator columns)
    int init[2];             // -64 * s of the same chunks
};
__device__ __forceinline__ void mma_pair_setup(MmaPairB &B, const uint32_t *actw, const uint32_t *tab2, int pair, int g, int t,
                                               const uint32_t (&m)[2][2]) {
    const uint4 v = *reinterpret_cast<const uint4 *>(actw + (size_t)(8 * pair + g) * 8 + 4 * (t & 1));
    const uint4 s = *reinterpret_cast<const uint4 *>(tab2 + (size_t)(8 * pair + 2 * t) * 2);
    const uint32_t vf[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int bl = 0; bl < 2; ++bl)
#pragma unroll
        for (int f = 0; f < 4; ++f) {
            B.b[bl][f][0] = vf[f] & m[bl][0];
            B.b[bl][f][1] = vf[f] & m[bl][1];
        }
    B.da[0] = __uint_as_float(s.x);
    B.init[0] = (int)s.y;
    B.da[1] = __uint_as_float(s.z);
    B.init[1] = (int)s.w;
}

// One block pair of 16 rows.  `rows` points at the pair in row 0 of the tile (byte address in shared memory, a
// multiple of 4: segments start at an even block), rows are `stride` bytes apart.  Returns through sum[0], sum[1]
// the lane's fp32 sums for rows g and g + 8 (its two chunk columns of the pair), through J the joined integers
// 64 * sumi of (row g, chunk 2t), (row g, chunk 2t + 1), (row g + 8, chunk 2t), (row g + 8, chunk 2t + 1).
__device__ __forceinline__ void mma_pair_rows(const uint8_t *rows, int stride, int g, int t, const MmaPairB &B,
                                              float (&sum)[2], int (&J)[4]) {
    const uint8_t *r0 = rows + (size_t)g * stride;
    const uint8_t *r1 = r0 + 8 * (size_t)stride;
    // first block: its codes start 2 bytes into a word; second block: word-aligned, 36 bytes on
    uint32_t e[2][4], o[2][2];
    {
        const uint32_t *p0 = reinterpret_cast<const uint32_t *>(r0), *p1 = reinterpret_cast<const uint32_t *>(r1);
        e[0][0] = p0[t]; e[0][1] = p0[t + 1]; e[0][2] = p0[t + 4]; e[0][3] = p0[t + 5];
        e[1][0] = p1[t]; e[1][1] = p1[t + 1]; e[1][2] = p1[t + 4]; e[1][3] = p1[t + 5];
        o[0][0] = p0[9 + t]; o[0][1] = p0[13 + t];
        o[1][0] = p1[9 + t]; o[1][1] = p1[13 + t];
    }
    const unsigned short d0 = *reinterpret_cast<const unsigned short *>(r0 + 34 * (t >> 1));
    const unsigned short d1 = *reinterpret_cast<const unsigned short *>(r1 + 34 * (t >> 1));
    uint32_t w[2][4];        // [block][row g word t, row g+8 word t, row g word 4+t, row g+8 word 4+t]: the A register order
    w[0][0] = __funnelshift_r(e[0][0], e[0][1], 16);
    w[0][1] = __funnelshift_r(e[1][0], e[1][1], 16);
    w[0][2] = __funnelshift_r(e[0][2], e[0][3], 16);
    w[0][3] = __funnelshift_r(e[1][2], e[1][3], 16);
    w[1][0] = o[0][0]; w[1][1] = o[1][0]; w[1][2] = o[0][1]; w[1][3] = o[1][1];
    int c[4][4];
#pragma unroll
    for (int f = 0; f < 4; ++f) {
        const uint32_t mask = 0x03030303u << (2 * f);
        const int zero[4] = {0, 0, 0, 0};
        const int init[4] = {B.init[0], B.init[1], B.init[0], B.init[1]};
        const uint32_t a0[4] = {w[0][0] & mask, w[0][1] & mask, w[0][2] & mask, w[0][3] & mask};
        const uint32_t a1[4] = {w[1][0] & mask, w[1][1] & mask, w[1][2] & mask, w[1][3] & mask};
        int mid[4];
        if (f == 3) mma_u8s8(mid, a0, B.b[0][f][0], B.b[0][f][1], init);
        else mma_u8s8(mid, a0, B.b[0][f][0], B.b[0][f][1], zero);
        mma_u8s8(c[f], a1, B.b[1][f][0], B.b[1][f][1], mid);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) J[i] = c[3][i] + c[2][i] * 4 + c[1][i] * 16 + c[0][i] * 64;
    const float dw0 = f16_bits_to_f32(d0), dw1 = f16_bits_to_f32(d1);
    const float t0 = __fmul_rn(__fmul_rn(dw0, B.da[0]), (float)J[0]);
    const float t1 = __fmul_rn(__fmul_rn(dw0, B.da[1]), (float)J[1]);
    const float t2 = __fmul_rn(__fmul_rn(dw1, B.da[0]), (float)J[2]);
    const float t3 = __fmul_rn(__fmul_rn(dw1, B.da[1]), (float)J[3]);
    sum[0] = __fadd_rn(t0, t1);
    sum[1] = __fadd_rn(t2, t3);
}

// DUMP: also writes the int32 chunk sums (sum code * a - sum a) of every row to dump[row][n_in / 32] (parity probe).
template <bool DUMP>
__global__ void __launch_bounds__(MMA_THREADS, 1) gemv_mma_kernel(const uint8_t *__restrict__ W, const uint32_t *__restrict__ xq,
                                                                 float *__restrict__ y, const MmaGeom P,
                                                                 int32_t *__restrict__ dump) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);       // [12] tile landed in slot
    uint64_t *done = full + MMA_MAX_SLOTS;                      // [12] every compute warp is through with the slot's tile
    uint64_t *freeb = done + MMA_MAX_SLOTS;                     // [12] the adder warp has read them: the slot may be refilled
    uint32_t *actw = reinterpret_cast<uint32_t *>(smem + 512);
    uint32_t *tab2 = actw + (size_t)P.nb * 4 * 8;
    float *pairsum = reinterpret_cast<float *>(tab2 + (size_t)P.nb * 4 * 2);
    float *gacc = pairsum + (size_t)P.nslot * P.pairs_max * 16;
    uint8_t *ring = smem + mma_fixed_bytes(P, P.nslot);

    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int my_groups = ((int)blockIdx.x < P.ngroups) ? (P.ngroups - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const int ntiles = my_groups * P.nseg;
    const size_t row_bytes = (size_t)P.nb * W_BLOCK_BYTES;
    const uint64_t pol = policy_evict_first();

    // tile T of this CTA -> (row group, segment)
    auto tile_of = [&](int T, int &gi, int &j) {
        const int k = (int)fast_div((uint32_t)T, P.magic_nseg);
        j = T - k * P.nseg;
        gi = (int)blockIdx.x + k * (int)gridDim.x;
    };
    auto issue_tile = [&](int T) {          // whole copy warp
        int gi, j;
        tile_of(T, gi, j);
        const int slot = T - (int)fast_div((uint32_t)T, P.magic_nslot) * P.nslot;
        const int r_cnt = min(16, P.n_out - 16 * gi);
        const int sb = mma_seg_start(P, j), sl = mma_seg_len(P, j);
        uint8_t *dst = ring + (size_t)slot * P.slot_bytes;
        const uint8_t *src = W + (size_t)16 * gi * row_bytes + (size_t)sb * W_BLOCK_BYTES;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");       // the slot was read through ordinary loads
        if (lane == 0) {
            if (P.contiguous) {
                // a ragged last group of rows whose length is no multiple of 16 bytes (n_in / 128 not a multiple of
                // 8): the last few bytes by plain loads, stored before the arrive that releases them to the waiters
                const uint32_t bytes = (uint32_t)(r_cnt * row_bytes), bulk = bytes & ~15u;
                for (uint32_t o = bulk; o < bytes; o += 4) *reinterpret_cast<uint32_t *>(dst + o) = ldg_nc_u32(src + o);
                mbar_expect_tx(&full[slot], bulk);
                if (bulk) bulk_g2s(dst, src, bulk, &full[slot], pol);
            } else {
                mbar_expect_tx(&full[slot], (uint32_t)((size_t)r_cnt * sl * W_BLOCK_BYTES));
            }
        }
        __syncwarp();
        if (!P.contiguous && lane < r_cnt)
            bulk_g2s(dst + (size_t)lane * P.stride, src + (size_t)lane * row_bytes, (uint32_t)(sl * W_BLOCK_BYTES), &full[slot], pol);
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < MMA_MAX_SLOTS; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&done[s], MMA_C);
            mbar_init(&freeb[s], 1);
        }
        mbar_fence_init();
    }
    __syncthreads();
    const int first_fill = min(P.nslot, ntiles);
    if (wid == MMA_C)
        for (int T = 0; T < min(2, first_fill); ++T) issue_tile(T);        // weights never depend on the kernel before
    pdl_launch_dependents();
    pdl_wait_prior_grid();              // activations (and y) belong to the previous kernel until here
    {
        const int nchunks = P.nb * 4;
        for (int c0 = 0; c0 < nchunks; c0 += MMA_THREADS) {
            const int chunk = c0 + (int)threadIdx.x;
            uint32_t v[9];
            if (chunk < nchunks) act_chunk_load(xq, chunk, v);
            if (c0 == 0 && wid == MMA_C)
                for (int T = 2; T < first_fill; ++T) issue_tile(T);         // the rest of the ring queues behind the activations
            if (chunk < nchunks) {
                *reinterpret_cast<uint4 *>(actw + (size_t)chunk * 8) = make_uint4(v[1], v[2], v[3], v[4]);
                *reinterpret_cast<uint4 *>(actw + (size_t)chunk * 8 + 4) = make_uint4(v[5], v[6], v[7], v[8]);
                tab2[2 * chunk] = __float_as_uint(__fmul_rn(f16_bits_to_f32(v[0] & 0xFFFFu), 0.015625f));
                tab2[2 * chunk + 1] = (uint32_t)(-64 * (int)(short)(v[0] >> 16));
            }
        }
    }
    __syncthreads();

    if (wid < MMA_C) {
        // ================================ compute warps ================================
        const int g = lane >> 2, t = lane & 3;
        uint32_t m[2][2];
#pragma unroll
        for (int bl = 0; bl < 2; ++bl) {
            m[bl][0] = ((g >> 2) == bl && (g & 3) == (t >> 1)) ? 0xFFFFFFFFu : 0u;
            m[bl][1] = ((g >> 2) == bl && (g & 3) == 2 + (t >> 1)) ? 0xFFFFFFFFu : 0u;
        }
        // Every warp goes through EVERY tile in order: waits for it to land, works on the pairs that fall to it (pair p
        // of tile T is item T * pairs_max + p, items go round-robin over the warps), then arrives on the tile's `done`
        // barrier.  A slot's barriers are reused every nslot tiles and a phase is told from the one before only by its
        // parity, so no warp may be two phases away when it asks; here none can: the slot is refilled only after all
        // warps have arrived for its tile, and a warp arrives only after it has seen the tile land.
        for (int T = 0; T < ntiles; ++T) {
            int gi, j;
            tile_of(T, gi, j);
            const int sb = mma_seg_start(P, j), sl = mma_seg_len(P, j);
            const int lap = (int)fast_div((uint32_t)T, P.magic_nslot);
            const int slot = T - lap * P.nslot;
            if (!mbar_wait_bounded(&full[slot], (uint32_t)(lap & 1))) break;
            int p = wid - (int)((unsigned)(T * P.pairs_max) % (unsigned)MMA_C);
            if (p < 0) p += MMA_C;
            for (; p < (sl >> 1); p += MMA_C) {
                MmaPairB B;
                mma_pair_setup(B, actw, tab2, (sb >> 1) + p, g, t, m);
                float sum[2];
                int J[4];
                mma_pair_rows(ring + (size_t)slot * P.slot_bytes + (size_t)68 * p, P.stride, g, t, B, sum, J);
                if (DUMP) {
                    const int chunk = 8 * ((sb >> 1) + p) + 2 * t;
                    const int r0 = 16 * gi + g, r1 = r0 + 8;
                    const size_t nch = (size_t)P.nb * 4;
                    if (r0 < P.n_out) { dump[r0 * nch + chunk] = J[0] >> 6; dump[r0 * nch + chunk + 1] = J[1] >> 6; }
                    if (r1 < P.n_out) { dump[r1 * nch + chunk] = J[2] >> 6; dump[r1 * nch + chunk + 1] = J[3] >> 6; }
                }
#pragma unroll
                for (int k = 0; k < 2; ++k) {
                    sum[k] = __fadd_rn(sum[k], __shfl_xor_sync(0xffffffffu, sum[k], 1));
                    sum[k] = __fadd_rn(sum[k], __shfl_xor_sync(0xffffffffu, sum[k], 2));
                }
                float *ps = pairsum + ((size_t)slot * P.pairs_max + p) * 16;
                if (t == 0) { ps[g] = sum[0]; ps[g + 8] = sum[1]; }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&done[slot]);            // release: the loads of the slot and the sums above are complete
        }
    } else if (wid == MMA_C) {
        // ================================ copy warp ================================
        for (int T = first_fill; T < ntiles; ++T) {
            const int lap = (int)fast_div((uint32_t)T, P.magic_nslot);
            const int slot = T - lap * P.nslot;
            if (!mbar_wait_bounded(&freeb[slot], (uint32_t)((lap - 1) & 1))) return;
            issue_tile(T);
        }
    } else {
        // ================================ adder warp ================================
        // pair sums of a tile in ascending pair order, segments of a row group in ascending order
        for (int T = 0; T < ntiles; ++T) {
            int gi, j;
            tile_of(T, gi, j);
            const int lap = (int)fast_div((uint32_t)T, P.magic_nslot);
            const int slot = T - lap * P.nslot;
            if (!mbar_wait_bounded(&done[slot], (uint32_t)(lap & 1))) return;
            const int pairs = mma_seg_len(P, j) >> 1;
            const int row = 16 * gi + lane;
            if (lane < 16) {
                const float *ps = pairsum + (size_t)slot * P.pairs_max * 16 + lane;
                float s = ps[0];
                for (int p = 1; p < pairs; ++p) s = __fadd_rn(s, ps[p * 16]);
                if (P.nseg > 1) {
                    float *ga = gacc + ((T / P.nseg) & (MMA_GROUP_RING - 1)) * 16 + lane;
                    if (j > 0) s = __fadd_rn(*ga, s);
                    *ga = s;
                }
                if (j == P.nseg - 1 && row < P.n_out) y[row] = s;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&freeb[slot]);
        }
    }
}

// ---- small token batches (2 .. 8 tokens): the same ring, the eight accumulator columns given to the tokens ----------
// Replaces gemm_pq2_0_p40_kernel (src/kernels/gemm_p40.cu:44-139) for the token counts between the mat-vec and a
// tensor-core tile -- the band the reference names as missing (docs/MTP.md:58): weights are streamed ONCE for all
// tokens.  One instruction = 16 rows x one 32-weight chunk x 8 tokens: A = the chunk's codes extracted to bytes (field t
// of the chunk's two code words for lane t of 4: the permuted order of src/pq2_0.h:158-166, so activation words t and
// 4 + t are the matching B rows), C starts at -s (the activation sum), so D is the host's int32 sumi
// (src/pq2_0.h:149-169) bit for bit.  Terms (dw * da) * (float)sumi as on the host, added in ascending chunk order
// inside a quarter of a row segment, quarters and segments in ascending order.
// Shared memory: int8 activation words [chunk][token 0..7][8] and the Q8_1 header words [chunk][token]; tokens past
// n_tok are zero.  Xq is the chunk-major layout of bonsai_p40_gemm: block (chunk, tok) at chunk * n_tok + tok.
constexpr int MMA_ITEMS = 4;          // items (quarters of a segment) per tile

__host__ __device__ inline size_t mmab_fixed_bytes(const MmaGeom &P, int nslot) {
    const size_t b = 512 + (size_t)P.nb * 4 * 288 + (size_t)nslot * MMA_ITEMS * 512 + MMA_GROUP_RING * 512;
    return (b + 127) & ~(size_t)127;
}

template <bool DUMP>
__global__ void __launch_bounds__(MMA_THREADS, 1) gemm_mma_kernel(const uint8_t *__restrict__ W, const uint32_t *__restrict__ Xq,
                                                                 float *__restrict__ Y, const MmaGeom P, const int n_tok,
                                                                 int32_t *__restrict__ dump) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);
    uint64_t *done = full + MMA_MAX_SLOTS;
    uint64_t *freeb = done + MMA_MAX_SLOTS;
    uint32_t *actb = reinterpret_cast<uint32_t *>(smem + 512);                 // [chunk][tok][8]
    uint32_t *hdr = actb + (size_t)P.nb * 4 * 64;                              // [chunk][tok]
    float *itemsum = reinterpret_cast<float *>(hdr + (size_t)P.nb * 4 * 8);   // [slot][item][row 16][tok 8]
    float *gacc = itemsum + (size_t)P.nslot * MMA_ITEMS * 128;
    uint8_t *ring = smem + mmab_fixed_bytes(P, P.nslot);

    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int my_groups = ((int)blockIdx.x < P.ngroups) ? (P.ngroups - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const int ntiles = my_groups * P.nseg;
    const size_t row_bytes = (size_t)P.nb * W_BLOCK_BYTES;
    const uint64_t pol = policy_evict_first();
    const int ppi = (P.pairs_max + MMA_ITEMS - 1) / MMA_ITEMS;                 // pairs per item

    auto tile_of = [&](int T, int &gi, int &j) {
        const int k = (int)fast_div((uint32_t)T, P.magic_nseg);
        j = T - k * P.nseg;
        gi = (int)blockIdx.x + k * (int)gridDim.x;
    };
    auto issue_tile = [&](int T) {          // whole copy warp
        int gi, j;
        tile_of(T, gi, j);
        const int slot = T - (int)fast_div((uint32_t)T, P.magic_nslot) * P.nslot;
        const int r_cnt = min(16, P.n_out - 16 * gi);
        const int sb = mma_seg_start(P, j), sl = mma_seg_len(P, j);
        uint8_t *dst = ring + (size_t)slot * P.slot_bytes;
        const uint8_t *src = W + (size_t)16 * gi * row_bytes + (size_t)sb * W_BLOCK_BYTES;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        if (lane == 0) {
            if (P.contiguous) {
                const uint32_t bytes = (uint32_t)(r_cnt * row_bytes), bulk = bytes & ~15u;
                for (uint32_t o = bulk; o < bytes; o += 4) *reinterpret_cast<uint32_t *>(dst + o) = ldg_nc_u32(src + o);
                mbar_expect_tx(&full[slot], bulk);
                if (bulk) bulk_g2s(dst, src, bulk, &full[slot], pol);
            } else {
                mbar_expect_tx(&full[slot], (uint32_t)((size_t)r_cnt * sl * W_BLOCK_BYTES));
            }
        }
        __syncwarp();
        if (!P.contiguous && lane < r_cnt)
            bulk_g2s(dst + (size_t)lane * P.stride, src + (size_t)lane * row_bytes, (uint32_t)(sl * W_BLOCK_BYTES), &full[slot], pol);
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < MMA_MAX_SLOTS; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&done[s], MMA_C);
            mbar_init(&freeb[s], 1);
        }
        mbar_fence_init();
    }
    __syncthreads();
    const int first_fill = min(P.nslot, ntiles);
    if (wid == MMA_C)
        for (int T = 0; T < min(2, first_fill); ++T) issue_tile(T);
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    {
        const int total = P.nb * 4 * 8;                 // (chunk, token slot)
        for (int i = threadIdx.x; i < total; i += MMA_THREADS) {
            const int chunk = i >> 3, tok = i & 7;
            uint32_t v[9];
#pragma unroll
            for (int w = 0; w < 9; ++w) v[w] = tok < n_tok ? __ldg(Xq + 9 * ((size_t)chunk * n_tok + tok) + w) : 0u;
            *reinterpret_cast<uint4 *>(actb + (size_t)i * 8) = make_uint4(v[1], v[2], v[3], v[4]);
            *reinterpret_cast<uint4 *>(actb + (size_t)i * 8 + 4) = make_uint4(v[5], v[6], v[7], v[8]);
            hdr[i] = v[0];
        }
        if (wid == MMA_C)
            for (int T = 2; T < first_fill; ++T) issue_tile(T);
    }
    __syncthreads();

    if (wid < MMA_C) {
        const int g = lane >> 2, t = lane & 3;
        const size_t nch = (size_t)P.nb * 4;
        // every warp goes through every tile in order (see gemv_mma_kernel); item k of tile T is item T * 4 + k
        for (int T = 0; T < ntiles; ++T) {
            int gi, j;
            tile_of(T, gi, j);
            const int sb = mma_seg_start(P, j), sl = mma_seg_len(P, j);
            const int lap = (int)fast_div((uint32_t)T, P.magic_nslot);
            const int slot = T - lap * P.nslot;
            if (!mbar_wait_bounded(&full[slot], (uint32_t)(lap & 1))) break;
            int k = wid - (int)((unsigned)(T * MMA_ITEMS) % (unsigned)MMA_C);
            if (k < 0) k += MMA_C;
            for (; k < MMA_ITEMS; k += MMA_C) {
                const int p_lo = k * ppi, p_hi = min((k + 1) * ppi, sl >> 1);
                if (p_lo >= p_hi) continue;                     // a short segment has fewer items; the adder skips them too
                float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                for (int p = p_lo; p < p_hi; ++p) {
                    const uint8_t *r0 = ring + (size_t)slot * P.slot_bytes + (size_t)68 * p + (size_t)g * P.stride;
                    const uint8_t *r1 = r0 + 8 * (size_t)P.stride;
                    const uint32_t *p0 = reinterpret_cast<const uint32_t *>(r0), *p1 = reinterpret_cast<const uint32_t *>(r1);
                    uint32_t e0[17], e1[17];                        // the pair's 17 words of rows g and g + 8
    #pragma unroll
                    for (int i = 0; i < 17; ++i) { e0[i] = p0[i]; e1[i] = p1[i]; }
    #pragma unroll
                    for (int bl = 0; bl < 2; ++bl) {
                        const float dw0 = f16_bits_to_f32(bl ? (e0[8] >> 16) : (e0[0] & 0xFFFFu));
                        const float dw1 = f16_bits_to_f32(bl ? (e1[8] >> 16) : (e1[0] & 0xFFFFu));
    #pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            uint32_t w[4];                          // row g word 0, row g + 8 word 0, row g word 1, row g + 8 word 1
                            if (bl == 0) {                          // codes start two bytes into word 0
                                w[0] = __funnelshift_r(e0[2 * c], e0[2 * c + 1], 16);
                                w[1] = __funnelshift_r(e1[2 * c], e1[2 * c + 1], 16);
                                w[2] = __funnelshift_r(e0[2 * c + 1], e0[2 * c + 2], 16);
                                w[3] = __funnelshift_r(e1[2 * c + 1], e1[2 * c + 2], 16);
                            } else {                                // word-aligned from word 9 on
                                w[0] = e0[9 + 2 * c]; w[1] = e1[9 + 2 * c]; w[2] = e0[10 + 2 * c]; w[3] = e1[10 + 2 * c];
                            }
                            uint32_t a[4];
    #pragma unroll
                            for (int i = 0; i < 4; ++i) a[i] = (w[i] >> (2 * t)) & 0x03030303u;
                            const int ci = 4 * (sb + 2 * p + bl) + c;
                            const uint32_t *ab = actb + ((size_t)ci * 8 + g) * 8;
                            const uint2 hh = *reinterpret_cast<const uint2 *>(hdr + (size_t)ci * 8 + 2 * t);
                            const int cin[4] = {-(int)(short)(hh.x >> 16), -(int)(short)(hh.y >> 16), -(int)(short)(hh.x >> 16),
                                                -(int)(short)(hh.y >> 16)};
                            int d[4];
                            mma_u8s8(d, a, ab[t], ab[4 + t], cin);
                            const float da0 = f16_bits_to_f32(hh.x & 0xFFFFu), da1 = f16_bits_to_f32(hh.y & 0xFFFFu);
                            acc[0] = __fadd_rn(acc[0], __fmul_rn(__fmul_rn(dw0, da0), (float)d[0]));
                            acc[1] = __fadd_rn(acc[1], __fmul_rn(__fmul_rn(dw0, da1), (float)d[1]));
                            acc[2] = __fadd_rn(acc[2], __fmul_rn(__fmul_rn(dw1, da0), (float)d[2]));
                            acc[3] = __fadd_rn(acc[3], __fmul_rn(__fmul_rn(dw1, da1), (float)d[3]));
                            if (DUMP) {
                                const int ra = 16 * gi + g, rb = ra + 8, ta = 2 * t, tb = ta + 1;
                                if (ra < P.n_out && ta < n_tok) dump[((size_t)ra * n_tok + ta) * nch + ci] = d[0];
                                if (ra < P.n_out && tb < n_tok) dump[((size_t)ra * n_tok + tb) * nch + ci] = d[1];
                                if (rb < P.n_out && ta < n_tok) dump[((size_t)rb * n_tok + ta) * nch + ci] = d[2];
                                if (rb < P.n_out && tb < n_tok) dump[((size_t)rb * n_tok + tb) * nch + ci] = d[3];
                            }
                        }
                    }
                }
                float *is = itemsum + ((size_t)slot * MMA_ITEMS + k) * 128;
                *reinterpret_cast<float2 *>(is + g * 8 + 2 * t) = make_float2(acc[0], acc[1]);
                *reinterpret_cast<float2 *>(is + (g + 8) * 8 + 2 * t) = make_float2(acc[2], acc[3]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&done[slot]);
        }
    } else if (wid == MMA_C) {
        for (int T = first_fill; T < ntiles; ++T) {
            const int lap = (int)fast_div((uint32_t)T, P.magic_nslot);
            const int slot = T - lap * P.nslot;
            if (!mbar_wait_bounded(&freeb[slot], (uint32_t)((lap - 1) & 1))) return;
            issue_tile(T);
        }
    } else {
        // adder warp: lane l owns outputs (row l / 2, tokens 4 * (l % 2) .. + 3) of the tile
        for (int T = 0; T < ntiles; ++T) {
            int gi, j;
            tile_of(T, gi, j);
            const int lap = (int)fast_div((uint32_t)T, P.magic_nslot);
            const int slot = T - lap * P.nslot;
            if (!mbar_wait_bounded(&done[slot], (uint32_t)(lap & 1))) return;
            const int items = ((mma_seg_len(P, j) >> 1) + ppi - 1) / ppi;
            const float *is = itemsum + (size_t)slot * MMA_ITEMS * 128 + 4 * lane;
            float4 s = *reinterpret_cast<const float4 *>(is);
            for (int k = 1; k < items; ++k) {
                const float4 v = *reinterpret_cast<const float4 *>(is + k * 128);
                s.x = __fadd_rn(s.x, v.x); s.y = __fadd_rn(s.y, v.y); s.z = __fadd_rn(s.z, v.z); s.w = __fadd_rn(s.w, v.w);
            }
            if (P.nseg > 1) {
                float4 *ga = reinterpret_cast<float4 *>(gacc + ((T / P.nseg) & (MMA_GROUP_RING - 1)) * 128) + lane;
                if (j > 0) {
                    const float4 o = *ga;
                    s.x = __fadd_rn(o.x, s.x); s.y = __fadd_rn(o.y, s.y); s.z = __fadd_rn(o.z, s.z); s.w = __fadd_rn(o.w, s.w);
                }
                *ga = s;
            }
            if (j == P.nseg - 1) {
                const int row = 16 * gi + (lane >> 1), tok0 = 4 * (lane & 1);
                if (row < P.n_out) {
                    const float out[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        if (tok0 + e < n_tok) Y[(size_t)row * n_tok + tok0 + e] = out[e];
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&freeb[slot]);
        }
    }
}

}  // namespace b200
