// gemm_tc.cuh -- prefill mat-mul Y[n_out][n_tok] = W . X on the 5th-generation tensor cores.
//
// Replaces, for sm_100a, gemm_pq2_0_p40_kernel (src/kernels/gemm_p40.cu:44-139).  The contraction is a real dense
// one, so the integer dot products run as tcgen05.mma.kind::i8 with int32 accumulators in tensor memory.  Every
// 32-weight chunk has its own fp16 x fp16 scale, so chunks cannot be summed inside the tensor core: each K = 32 MMA
// writes its own TMEM columns (accumulate off) and the epilogue warps read the int32 tile back (tcgen05.ld) and
// fold it into fp32 registers.  The integers are exact: weights are expanded to signed bytes code - 1, so one MMA
// gives sum(code * a) - sum(a) of the chunk, the very int32 of the host loop (tests/test_p40.cpp:460-467,
// src/pq2_0.h:149-169).  The fp32 side uses the tolerance the path states (1e-5 of max |Y|) to spend two
// instructions per output and chunk instead of five: per block  s = da0*v0 + da1*v1 + da2*v2 + da3*v3  by fused
// multiply-adds, then  acc += dw * s  -- the host computes (dw*da_c)*v_c term by term; same sums, other roundings.
// (The integer SIMT kernel, gemm_simt.cuh, keeps the host's bits; bonsai_b200_set_option("gemm_path", 0).)
//
// CTA tile: 128 weight rows x 64 tokens, one CTA per SM (it owns the SM's 512 TMEM columns: two halves of 4 chunks x
// 64 columns, i.e. the chunk results of two whole weight blocks: the tensor core fills one half while the epilogue
// drains the other),
// K stepped one weight block (4 chunks = 4 MMAs of M 128 x N 64 x K 32) at a time:
//   warps 0-15  : epilogue; warp w owns TMEM lanes 32 * (w % 4) .. (one weight row per thread) and tokens
//                 16 * (w / 4) .. + 15: 16 accumulators + 16 block sums per thread
//   warps 16-19 : producers; thread p expands the 2-bit codes of row p of the block to int8 (code - 1) in the
//                 K-major 128-byte-swizzled layout the MMA reads (a row = the block's 128 bytes) and copies the int8
//                 activations and the scale of token p (p < 64) for the block's four chunks
//   warp 20     : one thread issues the MMAs and commits them to mbarriers; the warp owns the TMEM allocation
//   warp 21     : (TMA form) bulk async copies of the raw bytes into shared memory, two buffers each: the weight
//                 rows 8 blocks (272 bytes, a 16-byte multiple) at a time, the Q8_1 blocks of the tile's tokens one
//                 weight block at a time -- the producers then read shared memory instead of issuing a 2-byte
//                 global load per halfword of a 34-byte block (which made them the bottleneck: 1.8 us per block).
//                 Needs n_in / 128 a multiple of 8, n_tok a multiple of 4, 16-byte aligned W and Xq; every other
//                 shape takes the form whose producers load from global memory themselves.
// The byte order inside a chunk is the permuted one on both sides: field k of a 16-code word holds the four codes
// that the activation quantiser stored as word k (src/pq2_0.h:120-125, 158-166).
//
// Work split ("stream-K"): the (tile, weight block) iterations of the whole problem are cut into one contiguous
// range per CTA, so every SM gets the same work whatever the tile count (160 tiles on 148 SMs would otherwise take
// two rounds).  A tile cut in two has its later K part computed FIRST by the CTA whose range starts inside it: that
// CTA writes its partial sums to Y and raises a flag; the CTA whose range ends inside the tile computes the earlier
// K part LAST, waits for the flag (bounded; normally long since raised) and stores early + late.  One fixed order,
// so Y does not depend on timing.  Flags live in a small static array, one set per launch in flight (8 sets, chosen
// by the launch number); the reader lowers a flag once it has seen it.
// Every wait is bounded; on a time-out the CTA still reaches the common exit and frees its TMEM.
#pragma once

#include "common.cuh"

#include <cuda.h>          // CUtensorMap (type only: the encoder is looked up at run time)

namespace b200 {

constexpr int TC_M = 128, TC_N = 64;
constexpr int TC_TMEM_STAGES = 8;                          // chunk results in flight in tensor memory: 8 x 64 columns = two whole blocks
constexpr int TC_STAGES = 4;                               // shared-memory stages (one weight block each)
constexpr int TC_XBUFS = 4;                                // raw Q8_1 buffers in flight (TMA form): bulk copies take ~1 us to land
constexpr int TC_A_BYTES = 4 * TC_M * 32;                  // 4 chunks x 128 rows x 32 bytes
constexpr int TC_B_BYTES = 4 * TC_N * 32;                  // 4 chunks x 64 tokens x 32 bytes
constexpr int TC_STAGE_BYTES = TC_A_BYTES + TC_B_BYTES;                 // operands of one weight block: a multiple of 1024
constexpr int TC_SCALE_BYTES = TC_M * 4 + 4 * TC_N * 4;                 // dw[128], da[4][64] of the block
constexpr int TC_EPI_WARPS = 16, TC_PRODA_WARPS = 4, TC_PRODB_WARPS = 2;
constexpr int TC_EPI_THREADS = TC_EPI_WARPS * 32, TC_PRODA_THREADS = TC_PRODA_WARPS * 32, TC_PRODB_THREADS = TC_PRODB_WARPS * 32;
constexpr int TC_THREADS = TC_EPI_THREADS + TC_PRODA_THREADS + TC_PRODB_THREADS + 64;       // + issuer warp + loader warp
constexpr int TC_WBUFS = 2;                                // raw weight pieces in flight (TMA form)
constexpr int TC_WRAW_BYTES = TC_M * 272;                  // raw PQ2_0 bytes of 8 consecutive blocks of 128 rows
constexpr int TC_XRAW_BYTES = 4 * TC_N * A_BLOCK_BYTES;    // raw Q8_1 blocks of 4 chunks x 64 tokens
constexpr int TC_SMEM_BYTES = 2048 + TC_STAGES * (TC_STAGE_BYTES + TC_SCALE_BYTES);   // barriers + slack to align to 1024
constexpr int TC_SMEM_BYTES_TMA = TC_SMEM_BYTES + TC_WBUFS * TC_WRAW_BYTES + TC_XBUFS * TC_XRAW_BYTES;
constexpr int TC_FLAG_SETS = 8, TC_MAX_CTAS = 256;

// Partial-tile flags: set `epoch % 8`, word = CTA that wrote the partial; raised by the writer, lowered by the reader.
__device__ unsigned int g_gemm_flags[TC_FLAG_SETS][TC_MAX_CTAS];

// Shared-memory matrix descriptor, K-major, 128-byte swizzle: a row of the operand is the 128 bytes of one weight
// block (four K = 32 chunks side by side), eight rows make a 1024-byte atom, and inside an atom the 16-byte piece j
// of row r sits at piece j ^ (r % 8).  Operand bases are 1024-byte aligned; a chunk is selected by advancing the
// start address by 32 bytes.  (The unswizzled core-matrix layout was read by the tensor core at a fraction of the
// shared-memory bandwidth: 550-700 cycles per K = 32 instruction, measured, against ~100 for this one.)
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: D = int32, A and B signed 8-bit, both K-major, N = 128, M = 128.
constexpr uint32_t TC_IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((TC_N >> 3) << 17) | ((TC_M >> 4) << 24);

__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(TC_IDESC), "r"(0u), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_ld16(uint32_t taddr, int (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_ld8(uint32_t taddr, int (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];\n"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tc_epi_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(TC_EPI_THREADS) : "memory"); }

// Block J of a row's raw 272-byte piece, from the 48-byte window that starts at byte 32 J: the fp16 scale is halfword J
// of the window, the eight code words follow it.
template <int J>
__device__ __forceinline__ void tc_pick(const uint32_t (&L)[12], uint32_t &dbits, uint32_t (&w)[8]) {
    dbits = (J & 1) ? (L[J >> 1] >> 16) : (L[J >> 1] & 0xFFFFu);
#pragma unroll
    for (int k = 0; k < 8; ++k)
        w[k] = (J & 1) ? L[((J + 1) >> 1) + k] : __funnelshift_r(L[(J >> 1) + k], L[(J >> 1) + k + 1], 16);
}

struct TcStage {
    uint8_t *a, *b;      // 128 / 64 rows x 128 bytes, swizzled
    float *dw;           // [128] weight scale of the block, per row
    float *da;           // [4][128] activation scale per chunk and token
};
__device__ __forceinline__ TcStage tc_stage(uint8_t *base, int s) {
    uint8_t *p = base + (size_t)s * TC_STAGE_BYTES;
    TcStage st;
    st.a = p;
    st.b = p + TC_A_BYTES;
    st.dw = reinterpret_cast<float *>(base + (size_t)TC_STAGES * TC_STAGE_BYTES + (size_t)s * TC_SCALE_BYTES);
    st.da = st.dw + TC_M;
    return st;
}

struct TcParams {
    int n_out, nblocks, n_tok;
    int tiles_tok, n_tiles;          // token tiles per row tile, tiles in all (token tile runs fastest)
    int stream_k;                    // 1: contiguous ranges of (tile, block) iterations; 0: whole tiles, round-robin
    unsigned int epoch;              // launch number, never 0 (flag set = epoch % 8)
    long long total_it;              // n_tiles * nblocks
};

// The CTA's next piece of work: blocks [kb0, kb1) of `tile`.  Every role walks the same sequence.
struct TcWalk {
    long long it, it_end;
    int tile_rr;
    __device__ __forceinline__ void start(const TcParams &P) {
        if (P.stream_k) {
            it = P.total_it * (long long)blockIdx.x / (long long)gridDim.x;
            it_end = P.total_it * ((long long)blockIdx.x + 1) / (long long)gridDim.x;
        } else {
            tile_rr = (int)blockIdx.x;
        }
    }
    __device__ __forceinline__ bool next(const TcParams &P, int &tile, int &kb0, int &kb1) {
        if (P.stream_k) {
            if (it >= it_end) return false;
            tile = (int)(it / P.nblocks);
            kb0 = (int)(it - (long long)tile * P.nblocks);
            const long long left = it_end - it;
            kb1 = (int)min((long long)P.nblocks, (long long)kb0 + left);
            it += kb1 - kb0;
            return true;
        }
        if (tile_rr >= P.n_tiles) return false;
        tile = tile_rr;
        kb0 = 0;
        kb1 = P.nblocks;
        tile_rr += (int)gridDim.x;
        return true;
    }
};

// DUMP: also writes the int32 value of every (row, token, chunk) to dump[(row * n_tok + tok) * (4 * nblocks) + chunk].
template <bool DUMP, bool TMA>
__global__ void __launch_bounds__(TC_THREADS, 1) gemm_tc_kernel(const uint8_t *__restrict__ W, const uint32_t *__restrict__ Xq,
                                                                float *Y, const TcParams P, int32_t *__restrict__ dump,
                                                                const __grid_constant__ CUtensorMap wmap) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);               // [4] producers -> issuer
    uint64_t *released = full + TC_STAGES;                              // [4] tensor core + epilogue -> producers
    uint64_t *mma_done = released + TC_STAGES;                          // [8, 2 used] tensor core -> epilogue: a block's four chunk results are there
    uint64_t *tmem_empty = mma_done + TC_TMEM_STAGES;                   // [8, 2 used] epilogue -> issuer: the block's columns are in registers
    uint64_t *wfull = tmem_empty + TC_TMEM_STAGES;                      // [3] loader -> producers: 8 blocks of weight rows landed
    uint64_t *wfree = wfull + TC_WBUFS;                                 // [3] producers -> loader
    uint64_t *xfull = wfree + TC_WBUFS;                                      // [4] loader -> producers: a block's Q8_1 blocks landed
    uint64_t *xfree = xfull + TC_XBUFS;                                 // [4] producers -> loader
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(xfree + TC_XBUFS);
    uint8_t *stages = smem + 1024 + ((1024u - (smem_u32(smem) & 1023u)) & 1023u);      // operands start on a 1024-byte boundary
    uint8_t *wraw = stages + TC_STAGES * (TC_STAGE_BYTES + TC_SCALE_BYTES);
    uint8_t *xraw = wraw + TC_WBUFS * TC_WRAW_BYTES;

    const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nblocks = P.nblocks, n_tok = P.n_tok, n_out = P.n_out;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; ++s) { mbar_init(&full[s], TC_PRODA_THREADS + TC_PRODB_THREADS); mbar_init(&released[s], 1 + TC_EPI_WARPS); }
        for (int s = 0; s < TC_TMEM_STAGES; ++s) { mbar_init(&mma_done[s], 1); mbar_init(&tmem_empty[s], TC_EPI_WARPS); }
        for (int s = 0; s < TC_WBUFS; ++s) { mbar_init(&wfull[s], 1); mbar_init(&wfree[s], TC_PRODA_THREADS); }
        for (int s = 0; s < TC_XBUFS; ++s) { mbar_init(&xfull[s], 1); mbar_init(&xfree[s], TC_PRODB_THREADS); }
        mbar_fence_init();
    }
    if (wid == TC_EPI_WARPS + TC_PRODA_WARPS + TC_PRODB_WARPS) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    TcWalk walk;
    walk.start(P);
    int tile, kb0, kb1;

    if (wid < TC_EPI_WARPS) {
        // ---------------- epilogue: one weight row per thread, 16 tokens ----------------
        const int q = wid & 3, cg = wid >> 2;
        const int row_l = 32 * q + lane;
        unsigned int *flags = g_gemm_flags[P.epoch & (TC_FLAG_SETS - 1)];
        bool ok = true;
        int n = 0;                              // weight blocks consumed by this CTA so far
        while (ok && walk.next(P, tile, kb0, kb1)) {
            const int rt = tile / P.tiles_tok, tt = tile - rt * P.tiles_tok;
            const int row = rt * TC_M + row_l, tokb = tt * TC_N + 16 * cg;
            float acc[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[j] = 0.0f;
            const uint32_t tlane = tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(16 * cg);
            for (int kb = kb0; kb < kb1 && ok; ++kb, ++n) {
                const int s = n % TC_STAGES;
                const TcStage st = tc_stage(stages, s);
                // Block n lives in half n % 2 of tensor memory (chunk c in columns 64 c ..): the tensor core fills one half
                // while this loop drains the other.  One barrier round per BLOCK, not per chunk: every barrier operation
                // goes through the shared-memory pipe, and with 21 warps polling it a single one was seen to cost the
                // issuing thread ~300 cycles.  The load of the next chunk is in flight while the current one is folded in.
                const int hb = n & 1;
                float accb[16];
                int v[2][16];
                if (!mbar_wait_bounded(&mma_done[hb], (uint32_t)((n >> 1) & 1), 20, 80)) { ok = false; break; }
                tc_fence_after();
                const uint32_t tblk = tlane + (uint32_t)(hb * 4 * TC_N);
                tc_ld16(tblk, v[0]);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    tc_ld_wait();
                    if (c < 3) {
                        tc_ld16(tblk + (uint32_t)((c + 1) * TC_N), v[(c + 1) & 1]);
                    } else {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&tmem_empty[hb]);    // all four chunks are in registers: the half may be overwritten
                    }
                    const float4 *da4 = reinterpret_cast<const float4 *>(st.da + c * TC_N + 16 * cg);
#pragma unroll
                    for (int g4 = 0; g4 < 4; ++g4) {
                        const float4 d = da4[g4];
                        const float dd[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float f = (float)v[c & 1][4 * g4 + e];
                            accb[4 * g4 + e] = (c == 0) ? __fmul_rn(dd[e], f) : __fmaf_rn(dd[e], f, accb[4 * g4 + e]);
                        }
                    }
                    if (DUMP && row < n_out) {
#pragma unroll
                        for (int e = 0; e < 16; ++e) {
                            const int tok = tokb + e;
                            if (tok < n_tok) dump[((size_t)row * n_tok + tok) * (4 * (size_t)nblocks) + 4 * kb + c] = v[c & 1][e];
                        }
                    }
                }
                if (!ok) break;
                const float dw = st.dw[row_l];          // written by the producers: read behind the waits above
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[j] = __fmaf_rn(dw, accb[j], acc[j]);
                __syncwarp();
                if (lane == 0) mbar_arrive(&released[s]);          // the scale tables of this stage are free
            }
            if (!ok) break;
            // ---- the tile (or this CTA's part of it) is done
            const bool late_part = kb0 > 0, early_part = kb1 < nblocks;
            float *yrow = Y + (size_t)row * n_tok + tokb;
            const bool vec = (n_tok & 3) == 0 && (reinterpret_cast<uintptr_t>(Y) & 15u) == 0;
            if (early_part) {
                // the CTA after this one computed the later blocks of this tile first and left them in Y
                if (threadIdx.x == 0) {
                    const unsigned int *f = flags + blockIdx.x + 1;
                    uint32_t ns = 64;
                    bool there = false;
                    for (uint32_t k = 0; k < (1u << 22); ++k) {
                        unsigned int v;
                        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
                        if (v != 0u) { there = true; break; }
                        __nanosleep(ns);
                        ns = min(ns * 2, 1024u);
                    }
                    if (!there) atomicExch(&g_device_status, STATUS_GRID_TIMEOUT);
                    // this CTA is the flag's only reader: lowered here, it is down again for the next launch that uses
                    // the set (a replayed CUDA graph carries the same launch number every time)
                    *const_cast<volatile unsigned int *>(f) = 0u;
                }
                tc_epi_barrier();
                if (row < n_out) {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (tokb + j < n_tok) acc[j] = __fadd_rn(acc[j], __ldcg(yrow + j));
                }
            }
            if (row < n_out) {
                if (vec) {
#pragma unroll
                    for (int j = 0; j < 16; j += 4)
                        if (tokb + j < n_tok) *reinterpret_cast<float4 *>(yrow + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (tokb + j < n_tok) yrow[j] = acc[j];
                }
            }
            if (late_part) {
                __threadfence();
                tc_epi_barrier();
                if (threadIdx.x == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(flags + blockIdx.x), "r"(P.epoch) : "memory");
            }
        }
    } else if (wid < TC_EPI_WARPS + TC_PRODA_WARPS) {
        // ---------------- weight producers: thread p expands the 2-bit codes of row p of the block ----------------
        const int p = threadIdx.x - TC_EPI_THREADS;            // 0..127
        const uint32_t a_off = (uint32_t)(p * 128), sw = (uint32_t)(p & 7);    // row p of the operand, its swizzle key
        bool ok = true;
        int n = 0, oct = 0;                     // weight blocks / pieces of up to 8 blocks handled so far
        while (ok && walk.next(P, tile, kb0, kb1)) {
            const int rt = tile / P.tiles_tok;
            const int row = min(rt * TC_M + p, n_out - 1);      // rows past the end repeat the last one (never stored)
            const uint8_t *wrow = W + (size_t)row * nblocks * W_BLOCK_BYTES;
            for (int kb = kb0; kb < kb1; ++kb, ++n) {
                const int s = n % TC_STAGES;
                uint32_t w[8], dbits;
                int wbuf = 0;
                if (TMA) {
                    // raw bytes from shared memory: the loader warp copied them there
                    if (kb == kb0 || (kb & 7) == 0) {
                        if (!mbar_wait_bounded(&wfull[oct % TC_WBUFS], (uint32_t)((oct / TC_WBUFS) & 1))) { ok = false; break; }
                        ++oct;
                    }
                    wbuf = (oct - 1) % TC_WBUFS;
                    // Block j of the row's 272-byte piece starts at byte 34 j = 32 j + 2 j: the 48-byte window at 32 j holds
                    // it at halfword j.  Three 16-byte loads (rows are 68 words apart: eight lanes cover all 32 banks), then
                    // the nine words are picked out with compile-time indices, one case per j (j is the same for the warp).
                    const int j = kb & 7;
                    const uint4 *wr = reinterpret_cast<const uint4 *>(wraw + (size_t)wbuf * TC_WRAW_BYTES + (size_t)p * 272 + (size_t)j * 32);
                    const uint4 q0 = wr[0], q1 = wr[1], q2 = wr[2];
                    const uint32_t L[12] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w, q2.x, q2.y, q2.z, q2.w};
                    switch (j) {
                        case 0: tc_pick<0>(L, dbits, w); break;
                        case 1: tc_pick<1>(L, dbits, w); break;
                        case 2: tc_pick<2>(L, dbits, w); break;
                        case 3: tc_pick<3>(L, dbits, w); break;
                        case 4: tc_pick<4>(L, dbits, w); break;
                        case 5: tc_pick<5>(L, dbits, w); break;
                        case 6: tc_pick<6>(L, dbits, w); break;
                        default: tc_pick<7>(L, dbits, w); break;
                    }
                } else {
                    // all loads of this thread are issued before the wait and before anything is stored
                    const uint8_t *wb = wrow + (size_t)kb * W_BLOCK_BYTES;
                    uint32_t h[17];
#pragma unroll
                    for (int i = 0; i < 17; ++i) h[i] = ldg_nc_u16(wb + 2 * i);
                    dbits = h[0];
#pragma unroll
                    for (int k = 0; k < 8; ++k) w[k] = h[1 + 2 * k] | (h[2 + 2 * k] << 16);
                }
                if (!mbar_wait_bounded(&released[s], (uint32_t)(((n / TC_STAGES) & 1) ^ 1))) { ok = false; break; }
                const TcStage st = tc_stage(stages, s);
                st.dw[p] = f16_bits_to_f32(dbits);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const uint32_t w0 = w[2 * c], w1 = w[2 * c + 1];
                    // field k of a word -> four codes 0..3 -> signed bytes code - 1 (add 0x7F per byte, flip the top bit)
                    uint4 lo, hi;
                    lo.x = ((w0 & 0x03030303u) + 0x7F7F7F7Fu) ^ 0x80808080u;
                    lo.y = (((w0 >> 2) & 0x03030303u) + 0x7F7F7F7Fu) ^ 0x80808080u;
                    lo.z = (((w0 >> 4) & 0x03030303u) + 0x7F7F7F7Fu) ^ 0x80808080u;
                    lo.w = (((w0 >> 6) & 0x03030303u) + 0x7F7F7F7Fu) ^ 0x80808080u;
                    hi.x = ((w1 & 0x03030303u) + 0x7F7F7F7Fu) ^ 0x80808080u;
                    hi.y = (((w1 >> 2) & 0x03030303u) + 0x7F7F7F7Fu) ^ 0x80808080u;
                    hi.z = (((w1 >> 4) & 0x03030303u) + 0x7F7F7F7Fu) ^ 0x80808080u;
                    hi.w = (((w1 >> 6) & 0x03030303u) + 0x7F7F7F7Fu) ^ 0x80808080u;
                    *reinterpret_cast<uint4 *>(st.a + a_off + ((uint32_t)(2 * c) ^ sw) * 16) = lo;          // bytes 0..15 of the chunk
                    *reinterpret_cast<uint4 *>(st.a + a_off + ((uint32_t)(2 * c + 1) ^ sw) * 16) = hi;      // bytes 16..31
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");    // the tensor core reads through the async proxy
                mbar_arrive(&full[s]);
                if (TMA && ((kb & 7) == 7 || kb == kb1 - 1)) mbar_arrive(&wfree[wbuf]);        // the piece is used up
            }
        }
    } else if (wid < TC_EPI_WARPS + TC_PRODA_WARPS + TC_PRODB_WARPS) {
        // ---------------- activation producers: thread t lays out the int8 values and the scales of token t ----------------
        const int t = threadIdx.x - TC_EPI_THREADS - TC_PRODA_THREADS;          // 0..63
        const uint32_t b_off = (uint32_t)(t * 128), sw = (uint32_t)(t & 7);
        bool ok = true;
        int n = 0;
        while (ok && walk.next(P, tile, kb0, kb1)) {
            const int rt = tile / P.tiles_tok, tt = tile - rt * P.tiles_tok;
            const int tok = tt * TC_N + t;
            const bool tok_ok = tok < n_tok;
            for (int kb = kb0; kb < kb1; ++kb, ++n) {
                const int s = n % TC_STAGES;
                uint32_t av[4][9];
                if (TMA) {
                    if (!mbar_wait_bounded(&xfull[n % TC_XBUFS], (uint32_t)((n / TC_XBUFS) & 1))) { ok = false; break; }
                    const uint32_t *xr = reinterpret_cast<const uint32_t *>(xraw + (size_t)(n % TC_XBUFS) * TC_XRAW_BYTES) + 9 * t;
#pragma unroll
                    for (int c = 0; c < 4; ++c)
#pragma unroll
                        for (int k = 0; k < 9; ++k) av[c][k] = tok_ok ? xr[c * (TC_N * 9) + k] : 0u;
                } else {
#pragma unroll
                    for (int c = 0; c < 4; ++c)
#pragma unroll
                        for (int k = 0; k < 9; ++k)
                            av[c][k] = tok_ok ? __ldg(Xq + 9 * ((size_t)(4 * kb + c) * n_tok + tok) + k) : 0u;
                }
                if (!mbar_wait_bounded(&released[s], (uint32_t)(((n / TC_STAGES) & 1) ^ 1))) { ok = false; break; }
                const TcStage st = tc_stage(stages, s);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    *reinterpret_cast<uint4 *>(st.b + b_off + ((uint32_t)(2 * c) ^ sw) * 16) = make_uint4(av[c][1], av[c][2], av[c][3], av[c][4]);
                    *reinterpret_cast<uint4 *>(st.b + b_off + ((uint32_t)(2 * c + 1) ^ sw) * 16) = make_uint4(av[c][5], av[c][6], av[c][7], av[c][8]);
                    st.da[c * TC_N + t] = f16_bits_to_f32(av[c][0] & 0xFFFFu);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(&full[s]);
                if (TMA) mbar_arrive(&xfree[n % TC_XBUFS]);                                 // the raw bytes are in the stage
            }
        }
    } else if (wid == TC_EPI_WARPS + TC_PRODA_WARPS + TC_PRODB_WARPS + 1) {
        // ---------------- loader (TMA form): raw weight rows and raw Q8_1 blocks into shared memory ----------------
        // Two cursors over the same sequence of work: weight pieces (up to 8 blocks of 128 rows, three buffers: a piece
        // takes several microseconds to arrive under load, so it is asked for two pieces ahead) and activation blocks
        // (four buffers).  Neither waits for the other: each is issued as soon as its buffer is free.
        if (TMA) {
            const uint64_t pol_x = policy_evict_last_or_default();
            TcWalk wwalk = walk;
            int w_tile = 0, w_kb = 0, w_kb1 = 0, oct = 0;
            int x_tile = 0, x_kb = 0, x_kb1 = 0, n = 0;
            bool w_more = wwalk.next(P, w_tile, w_kb, w_kb1), x_more = walk.next(P, x_tile, x_kb, x_kb1);
            uint32_t idle = 0;
            while (w_more || x_more) {
                bool moved = false;
                if (w_more && mbar_test(&wfree[oct % TC_WBUFS], (uint32_t)(((oct / TC_WBUFS) & 1) ^ 1))) {
                    const int wb = oct % TC_WBUFS;
                    const int rt = w_tile / P.tiles_tok;
                    if (lane == 0) {
                        // one tiled copy for the whole piece: box = 68 words x 128 rows of the matrix seen as [n_out][row words];
                        // rows past the end arrive as zeros and count towards the bytes like the others.  (128 row copies of
                        // 272 bytes each kept the copy unit busy for ~11 000 cycles per piece.)
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        mbar_expect_tx(&wfull[wb], (uint32_t)TC_WRAW_BYTES);
                        asm volatile(
                            "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                            ::"r"(smem_u32(wraw + (size_t)wb * TC_WRAW_BYTES)), "l"(&wmap), "r"((w_kb >> 3) * 68), "r"(rt * TC_M),
                              "r"(smem_u32(&wfull[wb]))
                            : "memory");
                    }
                    __syncwarp();
                    ++oct;
                    w_kb = min(w_kb1, (w_kb | 7) + 1);
                    if (w_kb >= w_kb1) w_more = wwalk.next(P, w_tile, w_kb, w_kb1);
                    moved = true;
                }
                if (x_more && mbar_test(&xfree[n % TC_XBUFS], (uint32_t)(((n / TC_XBUFS) & 1) ^ 1))) {
                    const int xb = n % TC_XBUFS;
                    const int rt = x_tile / P.tiles_tok, tt = x_tile - rt * P.tiles_tok;
                    const int toks_valid = min(TC_N, n_tok - tt * TC_N);
                    if (lane == 0) {
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        const uint32_t bytes = (uint32_t)toks_valid * A_BLOCK_BYTES;       // a multiple of 16: n_tok % 4 == 0
                        mbar_expect_tx(&xfull[xb], 4u * bytes);
                        for (int c = 0; c < 4; ++c)
                            bulk_g2s(xraw + (size_t)xb * TC_XRAW_BYTES + (size_t)c * (TC_N * A_BLOCK_BYTES),
                                     reinterpret_cast<const uint8_t *>(Xq) + ((size_t)(4 * x_kb + c) * n_tok + (size_t)tt * TC_N) * A_BLOCK_BYTES,
                                     bytes, &xfull[xb], pol_x);
                    }
                    __syncwarp();
                    ++n;
                    if (++x_kb >= x_kb1) x_more = walk.next(P, x_tile, x_kb, x_kb1);
                    moved = true;
                }
                if (moved) {
                    idle = 0;
                } else {
                    __nanosleep(64);
                    if (++idle > (1u << 22)) {                  // ~0.3 s without a free buffer: give up, report
                        if (lane == 0) atomicExch(&g_device_status, STATUS_MBARRIER_TIMEOUT);
                        break;
                    }
                }
            }
        }
    } else if (lane == 0) {
        // ---------------- issuer: four K = 32 MMAs per weight block ----------------
        bool ok = true;
        int n = 0;
        while (ok && walk.next(P, tile, kb0, kb1)) {
            for (int kb = kb0; kb < kb1; ++kb, ++n) {
                const int s = n % TC_STAGES;
                if (!mbar_wait_hot(&full[s], (uint32_t)((n / TC_STAGES) & 1))) { ok = false; break; }
                const TcStage st = tc_stage(stages, s);
                const int hb = n & 1;
                if (!mbar_wait_hot(&tmem_empty[hb], (uint32_t)(((n >> 1) & 1) ^ 1))) { ok = false; break; }
                tc_fence_after();
                const uint32_t a0 = smem_u32(st.a), b0 = smem_u32(st.b);
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    tc_mma_i8(tmem_base + (uint32_t)((4 * hb + c) * TC_N), tc_smem_desc(a0 + 32u * c), tc_smem_desc(b0 + 32u * c));
                tc_commit(&mma_done[hb]);
                tc_commit(&released[s]);        // arrives when the four MMAs above have read the stage
            }
        }
    }
    // common exit: every role arrives here, also after a time-out, so the TMEM columns are always freed
    tc_fence_before();
    __syncthreads();
    if (wid == TC_EPI_WARPS + TC_PRODA_WARPS + TC_PRODB_WARPS) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

}  // namespace b200
