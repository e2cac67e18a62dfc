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

#include <cuda.h>          // CUtensorMap (type only: the encoder is looked up at run time)

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
    asm(
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

// ---- small token batches (1 .. 16 tokens): the eight accumulator columns given to the tokens --------------------------
// Replaces gemm_pq2_0_p40_kernel (src/kernels/gemm_p40.cu:44-139) for the token counts between the mat-vec and a
// tensor-core tile -- the band the reference names as missing (docs/MTP.md:58): weights are streamed ONCE for all
// tokens.  One instruction = 16 rows x one 32-weight chunk x 8 tokens: A = the chunk's codes extracted to bytes (field t
// of the chunk's two code words for lane t of 4: the permuted order of src/pq2_0.h:158-166, so activation words t and
// 4 + t are the matching B rows); with C = -s (the activation sum) D would be the host's int32 sumi
// (src/pq2_0.h:149-169) bit for bit, and it is that plus a constant: C starts at 0x4B400000 - s, so
// D = 0x4B400000 + sumi, which read as a float is 12582912 + sumi exactly (|sumi| <= 8192), and one subtraction gives
// (float)sumi without a conversion instruction.  Terms (dw * da) * (float)sumi as on the host, added in ascending
// chunk order inside an item, items and segments in ascending order.
//
// The kernel is bound by the shared-memory data pipe (loads of code words, of activation words and of the decoded
// headers: ~12 wavefronts per MMA with one MMA per chunk), so a chunk's operand loads serve as many MMAs as fit:
// NRG = 2 row groups of 16 rows (up to 8 tokens) or NTG = 2 token groups (9 .. 16 tokens).
//
// Work of a CTA: its row groups in batches of MMAB_GB; inside a batch the SEGMENT loop is the outer one -- tile T =
// (batch, segment j, NRG neighbouring groups of the batch) -- so only the Q8_1 blocks of one segment have to be in
// shared memory (three buffers, filled by bulk copies straight from Xq, whose chunk-major layout -- block (chunk, tok)
// at chunk * n_tok + tok, 9 words -- is read as it is; a lane whose token is past n_tok reads a neighbour's block and
// its accumulator column is never stored), and the ring of weight tiles gets the rest.  A group's part of a tile is ONE
// copy: a 2-D tiled copy of 16 rows x one segment (<= 24 blocks; box = `stride` bytes, 16 * odd so that the 8 rows one
// load touches lie in different banks; what the box takes past the segment or the matrix is never read), or, for rows
// that are not a multiple of 8 blocks, one bulk copy of 16 whole rows.  An item is `ppi` block pairs of a tile; the
// items of a tile add their sums into the slot's sums one after the other in item order (a counter passes the turn),
// the last one joins them to the groups' earlier segments and hands the slot back.
constexpr int MMAB_C = 22;            // compute warps: item I = items * tile + k belongs to warp I % MMAB_C
constexpr int MMAB_THREADS = (MMAB_C + 2) * 32;      // + weight warp + activation warp
constexpr int MMAB_SEG_UNITS = 3;     // segment <= 3 units of 8 blocks
constexpr int MMAB_GB = 16;           // row groups per batch
constexpr int MMAB_MAGIC = 0x4B400000;

struct MmabGeom {
    int n_out, nb;
    int ngroups;             // row groups of 16
    int nseg, seg_q, seg_r;  // segments in units of 8 blocks: segment j has seg_q + (j < seg_r) units (nseg == 1: nb blocks)
    int stride;              // bytes between the rows of a tile in its slot
    int tiled;               // 1: a group's rows come by one 2-D tiled copy; 0: by one bulk copy of whole rows (nseg == 1)
    int nslot, slot_bytes;   // a slot holds nrg groups of 16 rows
    int pairs_max;           // block pairs in the longest segment
    int items, ppi;          // items per tile, block pairs per item
    int act_bufs, act_buf_bytes;   // a buffer = the segment's Q8_1 blocks, then {da, 0x4B400000 - s} of every (chunk, token)
    int act_tab_off;               // bytes from a buffer's start to that table
    int ntg, nrg;                  // token groups of 8, row groups of 16 that share a chunk's operand loads
    uint32_t magic_nslot, magic_bt, magic_items;   // division by nslot, by the tiles of a full batch, by items
};
__host__ __device__ inline int mmab_seg_start(const MmabGeom &P, int j) {
    return P.nseg == 1 ? 0 : 8 * (j * P.seg_q + (j < P.seg_r ? j : P.seg_r));
}
__host__ __device__ inline int mmab_seg_len(const MmabGeom &P, int j) {
    return P.nseg == 1 ? P.nb : 8 * (P.seg_q + (j < P.seg_r ? 1 : 0));
}
// Shared memory in front of the ring: barriers and counters, activation buffers, the sums of every slot's tile, the sums
// of a batch's groups.
__host__ __device__ inline size_t mmab_fixed_bytes(const MmabGeom &P, int nslot) {
    const size_t b = 512 + (size_t)P.act_bufs * P.act_buf_bytes + ((size_t)nslot * P.nrg + MMAB_GB) * 512 * P.ntg;
    return (b + 127) & ~(size_t)127;
}
__device__ __forceinline__ void mmab_tile_copy(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}

template <bool DUMP, int NTG, int NRG>
__global__ void __launch_bounds__(MMAB_THREADS, 1) gemm_mma_kernel(const uint8_t *__restrict__ W, const uint32_t *__restrict__ Xq,
                                                                  float *__restrict__ Y, const MmabGeom P, const int n_tok,
                                                                  int32_t *__restrict__ dump,
                                                                  const __grid_constant__ CUtensorMap wmap) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);                       // [12] a tile has landed
    uint64_t *freeb = full + MMA_MAX_SLOTS;                                    // [12] its sums are taken: the slot may be refilled
    uint64_t *actfull = freeb + MMA_MAX_SLOTS;                                 // [3] a segment's Q8_1 blocks have landed
    // [0] weight tiles given out so far, [1] steps whose Q8_1 blocks have landed and whose headers are decoded, [2] steps
    // whose blocks have been asked for.  A compute warp visits only its own tiles, so before it tests a tile's barrier
    // by parity it makes sure the copy it waits for has been ISSUED: that implies the barrier's previous phase is
    // complete, and the phase after cannot complete before the warp is through.  Everything else a warp can fall
    // behind on is a counter that only grows (or a turn number).
    volatile int *issued = reinterpret_cast<volatile int *>(smem + 256);
    volatile int *turn = reinterpret_cast<volatile int *>(smem + 272);         // [12] the item whose turn it is to add into the slot's sums
    volatile int *gstage = reinterpret_cast<volatile int *>(smem + 320);       // [16] next segment of the batch's group l
    int *stepdone = reinterpret_cast<int *>(smem + 384);                       // [4] tiles of step q taken, at q % 4
    uint8_t *actbuf = smem + 512;
    float *tsum = reinterpret_cast<float *>(actbuf + (size_t)P.act_bufs * P.act_buf_bytes);   // [slot][row group][token group][row 16][tok 8]
    float *gacc = tsum + (size_t)P.nslot * NRG * NTG * 128;                    // [group of the batch][token group][row 16][tok 8]
    uint8_t *ring = smem + mmab_fixed_bytes(P, P.nslot);

    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int mg = ((int)blockIdx.x < P.ngroups) ? (P.ngroups - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    constexpr int GBP = MMAB_GB / NRG;                                          // tiles per segment of a full batch
    const int batch_tiles = GBP * P.nseg;
    const int nbatch = (mg + MMAB_GB - 1) / MMAB_GB;
    const int gb_last = mg - (nbatch - 1) * MMAB_GB;                           // groups of the last batch (mg > 0)
    const int gbp_last = (gb_last + NRG - 1) / NRG;
    const int ntiles = mg > 0 ? (nbatch - 1) * batch_tiles + P.nseg * gbp_last : 0;
    const uint32_t magic_lastp = gbp_last > 1 ? (uint32_t)(((1ull << 32) + (uint32_t)gbp_last - 1) / (uint32_t)gbp_last) : 0u;
    const size_t row_bytes = (size_t)P.nb * W_BLOCK_BYTES;
    const int group_bytes = 16 * P.stride;

    // tile T -> batch b, segment j, tile pl of the segment, step q (segments counted through the batches), groups of the
    // batch gb; the divisions are multiplications
    auto tile_of = [&](int T, int &b, int &j, int &pl, int &q, int &gb) {
        b = (int)fast_div((uint32_t)T, P.magic_bt);
        const int r = T - b * batch_tiles;
        if (b < nbatch - 1) {
            gb = MMAB_GB;
            j = r / GBP;
            pl = r - j * GBP;
        } else {
            gb = gb_last;
            j = (int)fast_div((uint32_t)r, magic_lastp);
            pl = r - j * gbp_last;
        }
        q = b * P.nseg + j;
    };
    auto group_index = [&](int b, int l) { return (int)blockIdx.x + (b * MMAB_GB + l) * (int)gridDim.x; };
    auto slot_of = [&](int T, int &lap) {
        lap = (int)fast_div((uint32_t)T, P.magic_nslot);
        return T - lap * P.nslot;
    };
    auto third = [](int q) { return (int)(((uint32_t)q * 0xAAABu) >> 17); };   // q / 3 for q < 65536
    // One lane gives out a tile.  No proxy fence: the slot was only READ by the compute warps, and their last reads
    // are ordered before this copy by the barrier the weight warp waited on.
    auto issue_tile = [&](int T) {
        int b, j, pl, q, gb, lap;
        tile_of(T, b, j, pl, q, gb);
        const int slot = slot_of(T, lap);
        uint8_t *dst = ring + (size_t)slot * P.slot_bytes;
        const int present = min(NRG, gb - NRG * pl);
        if (P.tiled) {
            mbar_expect_tx(&full[slot], (uint32_t)(present * group_bytes));
            for (int h = 0; h < present; ++h)
                mmab_tile_copy(dst + (size_t)h * group_bytes, &wmap, (mmab_seg_start(P, j) >> 3) * 68,
                               16 * group_index(b, NRG * pl + h), &full[slot]);
        } else {
            const uint64_t pol = policy_evict_first();
            uint32_t total = 0;
            for (int h = 0; h < present; ++h) {
                const int gi = group_index(b, NRG * pl + h);
                const int r_cnt = min(16, P.n_out - 16 * gi);
                const uint8_t *src = W + (size_t)16 * gi * row_bytes;
                uint8_t *d = dst + (size_t)h * group_bytes;
                const uint32_t bytes = (uint32_t)(r_cnt * row_bytes), bulk = bytes & ~15u;
                for (uint32_t o = bulk; o < bytes; o += 4) *reinterpret_cast<uint32_t *>(d + o) = ldg_nc_u32(src + o);
                total += bulk;
            }
            mbar_expect_tx(&full[slot], total);
            for (int h = 0; h < present; ++h) {
                const int gi = group_index(b, NRG * pl + h);
                const int r_cnt = min(16, P.n_out - 16 * gi);
                const uint32_t bulk = (uint32_t)(r_cnt * row_bytes) & ~15u;
                if (bulk) bulk_g2s(dst + (size_t)h * group_bytes, W + (size_t)16 * gi * row_bytes, bulk, &full[slot], pol);
            }
        }
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < MMA_MAX_SLOTS; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&freeb[s], 1);
            turn[s] = 0;
        }
        for (int s = 0; s < 3; ++s) mbar_init(&actfull[s], 1);
        for (int s = 0; s < MMAB_GB; ++s) gstage[s] = 0;
        for (int s = 0; s < 4; ++s) stepdone[s] = 0;
        issued[0] = 0;
        issued[1] = 0;
        issued[2] = 0;
        mbar_fence_init();
        if (P.tiled) asm volatile("prefetch.tensormap [%0];" ::"l"(&wmap) : "memory");
    }
    __syncthreads();
    // The weights do not depend on the launch before this one: two tiles go out at once.  The rest of the first fill
    // goes out after the first step's Q8_1 blocks have been asked for -- copies complete in the order they were issued,
    // and nothing can be multiplied before those blocks are there.
    const int first_fill = min(P.nslot, ntiles), early = min(2, first_fill);
    if (wid == MMAB_C) {
        if (lane < early) issue_tile(lane);
        __syncwarp();
        if (lane == 0) issued[0] = early;
    }
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    auto wait_count = [&](volatile int *c, int need) -> bool {
        for (uint32_t n = 0; n < (1u << 22); ++n) {
            if (*c >= need) return true;
            __nanosleep(64);
        }
        atomicExch(&g_device_status, STATUS_MBARRIER_TIMEOUT);
        return false;
    };
    auto wait_equal = [&](volatile int *c, int want) -> bool {
        for (uint32_t n = 0; n < (1u << 22); ++n) {
            if (*c == want) return true;
            __nanosleep(32);
        }
        atomicExch(&g_device_status, STATUS_MBARRIER_TIMEOUT);
        return false;
    };

    if (wid < MMAB_C) {
        const int g = lane >> 2, t = lane & 3;
        const size_t nch = (size_t)P.nb * 4;
        const int cstride = 9 * n_tok;                                  // words from a chunk's blocks to the next chunk's
        const int off_b = 9 * g + 1 + t;                                // the lane's token: int8 words t and 4 + t
        const int off_h = 4 * t;                                        // {da, c} of tokens 2t and 2t + 1 in a chunk's table row (8 NTG tokens)
        const int sh0 = 16 + 2 * t, sh1 = 2 * t;
        int q_seen = -1;
        const int nitems = P.items * ntiles;
        for (int I = wid; I < nitems; I += MMAB_C) {
            const int T = (int)fast_div((uint32_t)I, P.magic_items), k = I - T * P.items;
            int b, j, pl, q, gb, lap;
            tile_of(T, b, j, pl, q, gb);
            const int sb = mmab_seg_start(P, j), sl = mmab_seg_len(P, j);
            const int ab = P.nseg > 1 ? q - 3 * third(q) : 0;
            if (P.nseg > 1 ? q != q_seen : q_seen < 0) {        // the step's blocks have landed and their headers are decoded
                if (!wait_count(&issued[1], P.nseg > 1 ? q + 1 : 1)) break;
                __threadfence_block();
                q_seen = q;
            }
            const uint32_t *act = reinterpret_cast<const uint32_t *>(actbuf + (size_t)ab * P.act_buf_bytes);
            const int slot = slot_of(T, lap);
            if (!wait_count(&issued[0], T + 1)) break;
            if (!mbar_wait_bounded(&full[slot], (uint32_t)(lap & 1))) break;
            const int p_lo = k * P.ppi, p_hi = min(p_lo + P.ppi, sl >> 1);      // empty in a short segment
            float acc[NRG][NTG][4];
#pragma unroll
            for (int h = 0; h < NRG; ++h)
#pragma unroll
                for (int u = 0; u < NTG; ++u) acc[h][u][0] = acc[h][u][1] = acc[h][u][2] = acc[h][u][3] = 0.0f;
            if (p_lo < p_hi) {
                const uint8_t *r0 = ring + (size_t)slot * P.slot_bytes + (size_t)68 * p_lo + (size_t)g * P.stride;
                const uint32_t *pb = act + (size_t)8 * p_lo * cstride + off_b;
                const uint32_t *ph = act + P.act_tab_off / 4 + (size_t)8 * p_lo * 16 * NTG + off_h;
                for (int p = p_lo; p < p_hi; ++p, r0 += 68) {
#pragma unroll
                    for (int bl = 0; bl < 2; ++bl) {
                        // the block's 9 words of rows g and g + 8 of every row group: block 0 = words 0 .. 8 of the pair
                        // (codes from byte 2 on), block 1 = words 8 .. 16 (scale in the high half of word 8, codes word-aligned)
                        uint32_t e[NRG][2][9];
#pragma unroll
                        for (int h = 0; h < NRG; ++h) {
                            const uint32_t *w0 = reinterpret_cast<const uint32_t *>(r0 + (size_t)h * group_bytes) + 8 * bl;
                            const uint32_t *w1 = reinterpret_cast<const uint32_t *>(r0 + (size_t)h * group_bytes + 8 * (size_t)P.stride) + 8 * bl;
#pragma unroll
                            for (int i = 0; i < 9; ++i) { e[h][0][i] = w0[i]; e[h][1][i] = w1[i]; }
                        }
                        float dw[NRG][2];
#pragma unroll
                        for (int h = 0; h < NRG; ++h) {
                            dw[h][0] = f16_bits_to_f32(bl ? (e[h][0][0] >> 16) : (e[h][0][0] & 0xFFFFu));
                            dw[h][1] = f16_bits_to_f32(bl ? (e[h][1][0] >> 16) : (e[h][1][0] & 0xFFFFu));
                        }
#pragma unroll
                        for (int c = 0; c < 4; ++c, pb += cstride, ph += 16 * NTG) {
                            uint32_t bw[NTG][2];
                            uint4 hv[NTG];
#pragma unroll
                            for (int u = 0; u < NTG; ++u) {
                                bw[u][0] = pb[72 * u];
                                bw[u][1] = pb[72 * u + 4];
                                hv[u] = *reinterpret_cast<const uint4 *>(ph + 16 * u);
                            }
#pragma unroll
                            for (int h = 0; h < NRG; ++h) {
                                uint32_t a[4];      // row g word 0, row g + 8 word 0, row g word 1, row g + 8 word 1: field t
                                if (bl == 0) {      // one funnel shift aligns and takes the field
                                    a[0] = __funnelshift_r(e[h][0][2 * c], e[h][0][2 * c + 1], sh0);
                                    a[1] = __funnelshift_r(e[h][1][2 * c], e[h][1][2 * c + 1], sh0);
                                    a[2] = __funnelshift_r(e[h][0][2 * c + 1], e[h][0][2 * c + 2], sh0);
                                    a[3] = __funnelshift_r(e[h][1][2 * c + 1], e[h][1][2 * c + 2], sh0);
                                } else {
                                    a[0] = e[h][0][1 + 2 * c] >> sh1; a[1] = e[h][1][1 + 2 * c] >> sh1;
                                    a[2] = e[h][0][2 + 2 * c] >> sh1; a[3] = e[h][1][2 + 2 * c] >> sh1;
                                }
#pragma unroll
                                for (int i = 0; i < 4; ++i) a[i] &= 0x03030303u;
#pragma unroll
                                for (int u = 0; u < NTG; ++u) {
                                    const int cin[4] = {(int)hv[u].y, (int)hv[u].w, (int)hv[u].y, (int)hv[u].w};
                                    int d[4];
                                    mma_u8s8(d, a, bw[u][0], bw[u][1], cin);
                                    const float da0 = __uint_as_float(hv[u].x), da1 = __uint_as_float(hv[u].z);
                                    const float f0 = __fsub_rn(__int_as_float(d[0]), 12582912.0f), f1 = __fsub_rn(__int_as_float(d[1]), 12582912.0f);
                                    const float f2 = __fsub_rn(__int_as_float(d[2]), 12582912.0f), f3 = __fsub_rn(__int_as_float(d[3]), 12582912.0f);
                                    acc[h][u][0] = __fadd_rn(acc[h][u][0], __fmul_rn(__fmul_rn(dw[h][0], da0), f0));
                                    acc[h][u][1] = __fadd_rn(acc[h][u][1], __fmul_rn(__fmul_rn(dw[h][0], da1), f1));
                                    acc[h][u][2] = __fadd_rn(acc[h][u][2], __fmul_rn(__fmul_rn(dw[h][1], da0), f2));
                                    acc[h][u][3] = __fadd_rn(acc[h][u][3], __fmul_rn(__fmul_rn(dw[h][1], da1), f3));
                                    if (DUMP && u == 0 && NRG * pl + h < gb) {
                                        const int ci = 4 * (sb + 2 * p + bl) + c;
                                        const int ra = 16 * group_index(b, NRG * pl + h) + g, rb = ra + 8, ta = 2 * t, tb = ta + 1;
                                        if (ra < P.n_out && ta < n_tok) dump[((size_t)ra * n_tok + ta) * nch + ci] = d[0] - MMAB_MAGIC;
                                        if (ra < P.n_out && tb < n_tok) dump[((size_t)ra * n_tok + tb) * nch + ci] = d[1] - MMAB_MAGIC;
                                        if (rb < P.n_out && ta < n_tok) dump[((size_t)rb * n_tok + ta) * nch + ci] = d[2] - MMAB_MAGIC;
                                        if (rb < P.n_out && tb < n_tok) dump[((size_t)rb * n_tok + tb) * nch + ci] = d[3] - MMAB_MAGIC;
                                    }
                                }
                            }
                        }
                    }
                }
            }
            // the items of a tile add into the slot's sums in item order: wait for the turn, add, pass it on
            if (!wait_equal(&turn[slot], k)) break;
            __threadfence_block();
            if (p_lo < p_hi) {
#pragma unroll
                for (int h = 0; h < NRG; ++h)
#pragma unroll
                    for (int u = 0; u < NTG; ++u) {
                        float *ts = tsum + (((size_t)slot * NRG + h) * NTG + u) * 128;
                        float2 *lo = reinterpret_cast<float2 *>(ts + g * 8 + 2 * t), *hi = reinterpret_cast<float2 *>(ts + (g + 8) * 8 + 2 * t);
                        float2 vlo = make_float2(acc[h][u][0], acc[h][u][1]), vhi = make_float2(acc[h][u][2], acc[h][u][3]);
                        if (k > 0) {
                            const float2 olo = *lo, ohi = *hi;
                            vlo.x = __fadd_rn(olo.x, vlo.x); vlo.y = __fadd_rn(olo.y, vlo.y);
                            vhi.x = __fadd_rn(ohi.x, vhi.x); vhi.y = __fadd_rn(ohi.y, vhi.y);
                        }
                        *lo = vlo;
                        *hi = vhi;
                    }
            }
            __syncwarp();
            if (k < P.items - 1) {
                if (lane == 0) {
                    __threadfence_block();
                    turn[slot] = k + 1;
                }
                continue;
            }
            // the last item: the tile's sums join the groups' earlier segments (ascending: wait for the segment before)
            __threadfence_block();
#pragma unroll
            for (int h = 0; h < NRG; ++h) {
                const int l = NRG * pl + h;
                if (l >= gb) break;
                if (P.nseg > 1) {
                    if (!wait_equal(&gstage[l], j)) break;
                    __threadfence_block();
                }
                const int gi = group_index(b, l);
#pragma unroll
                for (int u = 0; u < NTG; ++u) {
                    // lane owns outputs (row lane / 2, tokens 4 * (lane % 2) .. + 3) of the token group
                    float4 s = *(reinterpret_cast<const float4 *>(tsum + (((size_t)slot * NRG + h) * NTG + u) * 128) + lane);
                    if (P.nseg > 1) {
                        float4 *ga = reinterpret_cast<float4 *>(gacc + ((size_t)l * NTG + u) * 128) + lane;
                        if (j > 0) {
                            const float4 o = *ga;
                            s.x = __fadd_rn(o.x, s.x); s.y = __fadd_rn(o.y, s.y); s.z = __fadd_rn(o.z, s.z); s.w = __fadd_rn(o.w, s.w);
                        }
                        if (j < P.nseg - 1) *ga = s;
                    }
                    if (j == P.nseg - 1) {
                        const int row = 16 * gi + (lane >> 1), tok0 = 8 * u + 4 * (lane & 1);
                        if (row < P.n_out) {
                            const float out[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
                            for (int e2 = 0; e2 < 4; ++e2)
                                if (tok0 + e2 < n_tok) Y[(size_t)row * n_tok + tok0 + e2] = out[e2];
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) {
                turn[slot] = 0;
                __threadfence_block();
                if (P.nseg > 1) {
                    for (int h = 0; h < NRG && NRG * pl + h < gb; ++h) gstage[NRG * pl + h] = (j == P.nseg - 1) ? 0 : j + 1;
                    atomicAdd(&stepdone[q & 3], 1);
                }
                mbar_arrive(&freeb[slot]);
            }
        }
    } else if (wid == MMAB_C) {
        // weight warp: the rest of the first fill, then (one lane) every tile when its slot's previous tile is taken
        if (ntiles > 0 && !wait_count(&issued[2], 1)) return;
        if (lane >= early && lane < first_fill) issue_tile(lane);
        __syncwarp();
        if (lane == 0) issued[0] = first_fill;
        if (lane == 0)
            for (int T = first_fill; T < ntiles; ++T) {
                int lap;
                const int slot = slot_of(T, lap);
                if (!mbar_wait_bounded(&freeb[slot], (uint32_t)((lap - 1) & 1))) break;
                issue_tile(T);
                issued[0] = T + 1;
            }
    } else {
        // activation warp: a step's Q8_1 blocks are asked for up to two steps ahead (three buffers; a buffer is free when
        // every tile of the step three before is taken), and when they have landed their headers are decoded once for
        // all compute warps: {da as fp32, 0x4B400000 - s} per (chunk, token)
        const bool bulk_ok = (reinterpret_cast<uintptr_t>(Xq) & 15u) == 0;
        const uint64_t keep = policy_evict_normal();            // every CTA reads the same blocks: they stay in L2
        const int nsteps = P.nseg > 1 ? nbatch * P.nseg : (mg > 0 ? 1 : 0);
        auto tiles_of_step = [&](int s) { return s / P.nseg < nbatch - 1 ? GBP : gbp_last; };
        int qa = 0;
        bool ok = true;
        auto ask = [&](bool block) -> bool {                    // the blocks of step qa; false: its buffer is still in use
            if (qa >= 3) {
                volatile int *cnt = stepdone + ((qa - 3) & 3);
                const int need = tiles_of_step(qa - 3);
                if (block) {
                    if (!wait_equal(cnt, need)) { ok = false; return false; }
                } else if (*cnt != need) {
                    return false;
                }
                __syncwarp();
                if (lane == 0) *cnt = 0;
            }
            const int j = P.nseg > 1 ? qa % P.nseg : 0;
            const int ab = P.nseg > 1 ? qa - 3 * third(qa) : 0;
            const uint32_t bytes = (uint32_t)mmab_seg_len(P, j) * 4u * (uint32_t)n_tok * 36u;
            const uint8_t *src = reinterpret_cast<const uint8_t *>(Xq) + (size_t)mmab_seg_start(P, j) * 4 * n_tok * 36;
            uint8_t *dst = actbuf + (size_t)ab * P.act_buf_bytes;
            if (bulk_ok) {
                constexpr uint32_t PIECE = 4096;                // several copies in flight land sooner than one long one
                if (lane == 0) mbar_expect_tx(&actfull[ab], bytes);
                __syncwarp();
                for (uint32_t o = lane * PIECE; o < bytes; o += 32 * PIECE)
                    bulk_g2s(dst + o, src + o, min(PIECE, bytes - o), &actfull[ab], keep);
            } else {                                            // a vector that is only word-aligned: plain loads
                for (uint32_t i = lane; i < bytes / 4; i += 32)
                    reinterpret_cast<uint32_t *>(dst)[i] = __ldg(reinterpret_cast<const uint32_t *>(src) + i);
                __syncwarp();
                if (lane == 0) mbar_arrive(&actfull[ab]);
            }
            ++qa;
            if (lane == 0) issued[2] = qa;
            return true;
        };
        for (int qc = 0; qc < nsteps && ok; ++qc) {
            while (qa < nsteps && qa <= qc + 2 && ask(qa == qc)) {}
            if (!ok) break;
            const int q3 = third(qc);
            const int ab = P.nseg > 1 ? qc - 3 * q3 : 0;
            if (!mbar_wait_bounded(&actfull[ab], P.nseg > 1 ? (uint32_t)(q3 & 1) : 0u)) break;
            const int j = P.nseg > 1 ? qc % P.nseg : 0;
            const uint32_t *blk = reinterpret_cast<const uint32_t *>(actbuf + (size_t)ab * P.act_buf_bytes);
            uint2 *tab = reinterpret_cast<uint2 *>(actbuf + (size_t)ab * P.act_buf_bytes + P.act_tab_off);
            // record i = chunk * TPC + tok (TPC = 8 NTG table entries per chunk): the lane's token is lane % TPC, its
            // chunks lane / TPC, + 32 / TPC, ...; all loads of a round first
            constexpr int TPC = 8 * NTG, CPW = 32 / TPC;
            const int n = mmab_seg_len(P, j) * 4 * TPC;
            const int tok = lane & (TPC - 1);
            const uint32_t *src_h = blk + (size_t)((lane / TPC) * n_tok + tok) * 9;
            constexpr int CONV_UNROLL = 24;
            for (int i0 = lane; i0 < n; i0 += 32 * CONV_UNROLL, src_h += (size_t)CPW * CONV_UNROLL * n_tok * 9) {
                uint32_t h[CONV_UNROLL];
#pragma unroll
                for (int u = 0; u < CONV_UNROLL; ++u)
                    h[u] = (i0 + 32 * u < n && tok < n_tok) ? src_h[(size_t)CPW * u * n_tok * 9] : 0u;
#pragma unroll
                for (int u = 0; u < CONV_UNROLL; ++u)
                    if (i0 + 32 * u < n)
                        tab[i0 + 32 * u] = make_uint2(__float_as_uint(f16_bits_to_f32(h[u] & 0xFFFFu)), (uint32_t)(MMAB_MAGIC - ((int)h[u] >> 16)));
            }
            __syncwarp();
            if (lane == 0) {
                __threadfence_block();
                issued[1] = qc + 1;
            }
        }
    }
}

}  // namespace b200
