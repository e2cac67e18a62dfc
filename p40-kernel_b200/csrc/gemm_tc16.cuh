// gemm_tc16.cuh -- prefill mat-mul with the WHOLE contraction on the tensor cores (tcgen05.mma.kind::f16).
//
// gemm_tc.cuh keeps the integers of the host loop (one int8 MMA per 32-weight chunk, the per-chunk scales folded in
// by the CUDA cores) and is bound by exactly that fold: ~5400 warp instructions per 128 x 64 x 128 unit, 70 % of the
// issue slots, the tensor pipe 6.5 % busy.  This kernel moves the per-chunk activation scale to the OTHER side of the
// tensor core.  The dequantised activation  xh = da * a  (fp16 scale x int8, 18 significant bits) is split once per
// call into two fp16 numbers H + L = xh * 2^S exactly (S per token, a power of two that puts the token's largest
// value just under 2^15; L is the exact remainder, and where it underflows the loss is below 2^-38 of the token's
// largest value), the codes go to the tensor core as fp16 -1, 0, 1, 2, and one accumulator in tensor memory
// collects  sum_k (code_k - 1) * (H_k + L_k)  over a whole 128-weight block: products are exact, sums are the tensor
// core's fp32.  The CUDA cores are left with one fused multiply-add per output and BLOCK (the fp16 weight scale) and
// the expansion of the codes: 2900 warp instructions per unit against 5400, and the tensor pipe 44 % busy.
// Accuracy: the only roundings are the tensor core's fp32 additions inside a block (256 terms) and one fp32 FMA per
// block, against the host's one rounding per chunk term: Y is held to 1e-5 of max |Y| like the integer kernel's
// (measured ~1e-6); the INTEGERS of the host loop are not formed here: bonsai_b200_gemm_dump and
// bonsai_b200_set_option("gemm_path", 3) keep the integer kernel.
// Oracle: tests/test_p40.cpp:438-467 + src/pq2_0.h:149-169 (the host loop); kernel replaced: src/kernels/gemm_p40.cu:44-139.
//
// CTA tile 128 rows x 64 tokens, one CTA per SM, K stepped one weight block at a time = 16 MMAs (M 128, N 64, K 16):
// two K halves of 64 values x {H, L} x four K = 16 steps, all into one 64-column accumulator (4 in flight).
//   warps 0-7   : epilogue: per block two tcgen05.ld of 16 columns, acc += dw * D (one row x 32 tokens per thread)
//   warps 8-23  : code producers: thread (row p, K half g), every second block: 64 two-bit codes -> 64 fp16 with byte
//                 permutes (the fp16 patterns of -1, 0, 1, 2 differ only in their high byte), written to tensor memory
//   warps 24-25 : issuers (alternate blocks)
//   warps 26-27 : loaders (tiled TMA copies): weight pieces of 8 blocks x 128 rows; per block two boxes of 64 values x
//                 64 tokens x {H, L}, landing swizzled as the MMA reads them
// Work split, partial tiles and time-outs as in gemm_tc.cuh (same walk, same flag words).
// Every role that feeds the tensor core is a serial chain per block, and each in turn was the kernel's period until it
// was split or shortened (measured with per-role cycle stamps): descriptors built per MMA in a one-lane branch (70
// cycles per MMA; now two adds in warp-uniform code), one loader polling two rings (1000 cycles per unit; now two
// loader warps with blocking waits and one barrier round per block), both operands in shared memory (the tensor
// core's operand reads; now A in tensor memory), every producer warp on every block (1300 cycles; now alternate blocks).
#pragma once

#include "gemm_tc.cuh"

namespace b200 {

constexpr int T16_M = 128;
// Operands move in units of one K half of a weight block (64 values).  The codes (A) never touch shared memory: the
// producers write the fp16 values straight into TENSOR memory (tcgen05.st, lane = weight row, 32 columns per unit) and
// the MMA takes A from there -- with both operands in shared memory the tensor core's operand reads alone (6 KB per
// 128 x 64 x 16 MMA, 96 KB per block) ate 3/4 of the shared-memory bandwidth of the block's whole time budget.  The
// activations (B: the H and L planes of the tile's tokens) land in a shared-memory ring by TMA, asked for as far ahead
// as the ring allows: the boxes come from L2 and take ~1000-1500 cycles.
constexpr int T16_NA = 8;                                  // A ring: half-block units in tensor memory
constexpr int T16_A_COL0 = 256, T16_A_UNIT_COLS = 32;      // tensor memory: accumulators in columns 0..255, then 8 A units x 32
constexpr int T16_WBUFS = 2;
constexpr int T16_DWRING = 8;                              // weight scales of the last 8 blocks (epilogue lags the producers)
constexpr int T16_ISSUERS = 2;                             // issuing warps: warp k takes the blocks n with n % 2 == k
// The token width of a tile is a template parameter: 128 tokens per tile halve the code expansion per output (the
// kernel's busiest part) and are used for large batches; 64 keep small batches from padding.
template <int TN>
struct T16C {
    static constexpr int N = TN;
    static constexpr int ACC = 256 / TN;                                    // accumulators in flight (TN columns each)
    static constexpr int EPI_WARPS = TN / 8;                                // 4 lane quarters x (TN / 32) column groups of 32 tokens
    static constexpr int PROD_SETS = TN == 64 ? 2 : 1;                      // sets of producer warps on alternate blocks
    static constexpr int PROD_WARPS = 8 * PROD_SETS;                        // 4 row quarters x 2 K halves per set
    static constexpr int EPI_THREADS = EPI_WARPS * 32, PROD_THREADS = PROD_WARPS * 32;
    static constexpr int THREADS = EPI_THREADS + PROD_THREADS + 32 * (T16_ISSUERS + 2);      // + two loader warps
    static constexpr int BUNIT = TN * 256;                                  // B bytes of one K half: {H, L} x TN tokens x 128 bytes
    static constexpr int NB = (128 * 1024) / (2 * BUNIT);                   // B ring: whole blocks, 128 KB in all
    static constexpr int SMEM_BYTES = 2048 + NB * 2 * BUNIT + T16_DWRING * T16_M * 4 + T16_WBUFS * TC_WRAW_BYTES;
    // instruction descriptor: D = fp32, A and B fp16, both K-major, N = TN, M = 128
    static constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(T16_M >> 4) << 24);
};


// The descriptors' upper words are the same for every operand of this kernel (128-byte swizzle, 1024 bytes between
// 8-row groups); only the 14-bit address field of the lower word moves.  The issuing thread runs alone, one dependent
// instruction every few cycles, so an MMA is issued with two independent 32-bit adds and nothing else (building both
// 64-bit descriptors from an address cost ~75 cycles per MMA, 16 times per block).
constexpr uint32_t T16_DESC_HI = (uint32_t)(1024 >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t tc16_desc_lo(uint32_t smem_addr) { return ((smem_addr >> 4) & 0x3FFFu) | (1u << 16); }
template <bool ACC>
__device__ __forceinline__ void tc_mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .b64 db;\n\t"
        "mov.b64 db, {%2, %4};\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %3, {%6, %6, %6, %6}, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(idesc), "r"(T16_DESC_HI), "n"(ACC ? 1 : 0), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};\n"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
          "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
          "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
          "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
          "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}
__device__ __forceinline__ void tc_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *map, int x, int y, int z, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}

// ---- once per call: the activations as two fp16 planes ------------------------------------------------------------
// maxd[tok] = bits of the largest chunk scale of the token (non-negative floats order like their bit patterns);
// zeroed by the caller.  Block = 32 tokens x 8 chunk lanes, grid.y slices the chunks.
__global__ void __launch_bounds__(256) tc16_tokmax_kernel(const uint32_t *__restrict__ Xq, int n_chunks, int n_tok,
                                                          unsigned int *__restrict__ maxd) {
    const int tl = threadIdx.x & 31, grp = threadIdx.x >> 5;
    const int tok = blockIdx.x * 32 + tl;
    if (tok >= n_tok) return;
    const int per = (n_chunks + (int)gridDim.y - 1) / (int)gridDim.y;
    const int c0 = (int)blockIdx.y * per, c1 = min(n_chunks, c0 + per);
    unsigned int m = 0;
    for (int c = c0 + grp; c < c1; c += 8) m = max(m, __ldg(Xq + 9 * ((size_t)c * n_tok + tok)) & 0x7FFFu);
    if (m) atomicMax(maxd + tok, m);
}
// 2^S for the token: S = 8 - exponent(max_c da_c), so that every |da * a * 2^S| < 2^15 (da = f * 2^ex, 0.5 <= f < 1,
// times 128 is below 2^(ex + 7)).
__device__ __forceinline__ int tc16_shift(unsigned int maxd_bits) {
    const float m = f16_bits_to_f32(maxd_bits);
    int ex = 0;
    if (m > 0.0f) (void)frexpf(m, &ex);
    return m > 0.0f ? 8 - ex : 0;
}
// Thread = (chunk, token): 32 values -> 32 + 32 fp16, in the order the quantiser stored them (the order in which the
// code producers emit the codes).  planes: H at [tok][n_in], L at [n_tok + tok][n_in]; scale[tok] = 2^-S for the
// epilogue.  A warp takes 4 tokens x 8 consecutive chunks: its stores are four runs of 512 bytes per plane.
__global__ void __launch_bounds__(256) tc16_split_kernel(const uint32_t *__restrict__ Xq, int n_chunks, int n_tok,
                                                         const unsigned int *__restrict__ maxd, float *__restrict__ scale,
                                                         __half *__restrict__ planes) {
    const int lane = threadIdx.x & 31;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int cgroups = (n_chunks + 7) >> 3;
    const int tg = (int)(warp / cgroups), cgp = (int)(warp - (long long)tg * cgroups);
    const int tok = 4 * tg + (lane >> 3), c = 8 * cgp + (lane & 7);
    if (tok >= n_tok || c >= n_chunks) return;
    const int S = tc16_shift(maxd[tok]);
    if (c == 0) scale[tok] = ldexpf(1.0f, -S);
    const uint32_t *src = Xq + 9 * ((size_t)c * n_tok + tok);
    uint32_t w[9];
#pragma unroll
    for (int k = 0; k < 9; ++k) w[k] = __ldg(src + k);
    const float ds = __fmul_rn(f16_bits_to_f32(w[0] & 0xFFFFu), ldexpf(1.0f, S));        // da * 2^S: exact (a power of two)
    const size_t n_in = (size_t)n_chunks * 32;
    uint4 *hp = reinterpret_cast<uint4 *>(planes + (size_t)tok * n_in + (size_t)c * 32);
    uint4 *lp = reinterpret_cast<uint4 *>(planes + ((size_t)n_tok + tok) * n_in + (size_t)c * 32);
    const int8_t *ab = reinterpret_cast<const int8_t *>(w + 1);      // the chunk's 32 int8 in stored order
#pragma unroll
    for (int q = 0; q < 4; ++q) {                       // 8 values per 16-byte store, in the order of tc16_expand
        uint32_t h[4], l[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            constexpr unsigned char PERM[16] = {0, 8, 1, 9, 4, 12, 5, 13, 2, 10, 3, 11, 6, 14, 7, 15};
            const int j0 = 16 * (q >> 1) + PERM[8 * (q & 1) + 2 * e], j1 = 16 * (q >> 1) + PERM[8 * (q & 1) + 2 * e + 1];
            const int a0 = (int)ab[j0], a1 = (int)ab[j1];
            const float v0 = __fmul_rn(ds, (float)a0), v1 = __fmul_rn(ds, (float)a1);      // exact: 11 x 7 bits
            const __half h0 = __float2half_rn(v0), h1 = __float2half_rn(v1);
            const __half l0 = __float2half_rn(__fsub_rn(v0, __half2float(h0))), l1 = __float2half_rn(__fsub_rn(v1, __half2float(h1)));
            h[e] = (uint32_t)__half_as_ushort(h0) | ((uint32_t)__half_as_ushort(h1) << 16);
            l[e] = (uint32_t)__half_as_ushort(l0) | ((uint32_t)__half_as_ushort(l1) << 16);
        }
        hp[q] = make_uint4(h[0], h[1], h[2], h[3]);
        lp[q] = make_uint4(l[0], l[1], l[2], l[3]);
    }
}

// 16 two-bit codes of one word -> 16 fp16 (-1, 0, 1, 2) in eight words.  The four fp16 patterns 0xBC00, 0x0000, 0x3C00,
// 0x4000 have a zero low byte, so the high bytes are looked up four at a time by a byte permute whose selector nibbles
// ARE the codes (w & 0x3333 leaves a code in every nibble), and a second permute spreads them over two words.  19
// integer instructions per word: the expansion runs on the half-rate integer pipe, which this kernel keeps busiest.
// Order of the 16 values (the split kernel writes the activations in the same order): code (byte b, field k)
// of the word pairs with activation byte 4 k + b of the word's 16 (src/pq2_0.h:120-125, 158-166);
//   o[0..1] = (b0k0 b0k2 b1k0 b1k2)   o[2..3] = (b0k1 b0k3 b1k1 b1k3)   o[4..5], o[6..7]: the same for bytes 2, 3.
__device__ __forceinline__ void tc16_expand(uint32_t w, uint32_t *o) {
    constexpr uint32_t TB = 0x403C00BCu;
    const uint32_t wh = w >> 16;
    const uint32_t s0 = w & 0x3333u, s1 = (w >> 2) & 0x3333u, s2 = wh & 0x3333u, s3 = (wh >> 2) & 0x3333u;
    const uint32_t h0 = __byte_perm(TB, 0u, s0), h1 = __byte_perm(TB, 0u, s1), h2 = __byte_perm(TB, 0u, s2), h3 = __byte_perm(TB, 0u, s3);
    o[0] = __byte_perm(h0, 0u, 0x1404u);
    o[1] = __byte_perm(h0, 0u, 0x3424u);
    o[2] = __byte_perm(h1, 0u, 0x1404u);
    o[3] = __byte_perm(h1, 0u, 0x3424u);
    o[4] = __byte_perm(h2, 0u, 0x1404u);
    o[5] = __byte_perm(h2, 0u, 0x3424u);
    o[6] = __byte_perm(h3, 0u, 0x1404u);
    o[7] = __byte_perm(h3, 0u, 0x3424u);
}
struct Tc16Maps {
    CUtensorMap w;        // PQ2_0 matrix as [n_out][row words], box 68 x 128
    CUtensorMap x;        // fp16 planes as [2][n_tok][n_in], box 64 values x TN tokens x 2 planes, 128-byte swizzle
};

template <int TN>
__global__ void __launch_bounds__(T16C<TN>::THREADS, 1) gemm_tc16_kernel(float *Y, const TcParams P, const float *__restrict__ tokscale,
                                                                         const __grid_constant__ Tc16Maps maps) {
    using C = T16C<TN>;
    constexpr int T16_N = TN, T16_ACC = C::ACC, T16_NB = C::NB, T16_BUNIT = C::BUNIT, T16_EPI_WARPS = C::EPI_WARPS,
                  T16_PROD_WARPS = C::PROD_WARPS, T16_PROD_SETS = C::PROD_SETS, T16_EPI_THREADS = C::EPI_THREADS,
                  T16_PROD_THREADS = C::PROD_THREADS, T16_EPI_TOKS = 32;
    extern __shared__ __align__(128) uint8_t smem[];
    // unit u = 2 * block + K half lives in slot u % NA of the code ring and slot u % NB of the activation ring
    uint64_t *afull = reinterpret_cast<uint64_t *>(smem);              // [NA] code producers -> issuer
    uint64_t *afree = afull + T16_NA;                                   // [NA] tensor core -> code producers
    uint64_t *bfull = afree + T16_NA;                                   // [NB] loader (bytes landed) -> issuer
    uint64_t *bfree = bfull + T16_NB;                                   // [NB] tensor core -> loader
    uint64_t *mma_done = bfree + T16_NB;                                // [4] tensor core -> epilogue
    uint64_t *tmem_empty = mma_done + T16_ACC;                          // [4] epilogue -> issuer
    uint64_t *wfull = tmem_empty + T16_ACC;                             // [2] loader -> producers
    uint64_t *wfree = wfull + T16_WBUFS;                                // [2] producers -> loader
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(wfree + T16_WBUFS);
    uint8_t *stages = smem + 1024 + ((1024u - (smem_u32(smem) & 1023u)) & 1023u);
    uint8_t *bring = stages;
    float *dwring = reinterpret_cast<float *>(bring + T16_NB * 2 * T16_BUNIT);
    uint8_t *wraw = reinterpret_cast<uint8_t *>(dwring + T16_DWRING * T16_M);

    const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nblocks = P.nblocks, n_tok = P.n_tok, n_out = P.n_out;

    if (threadIdx.x == 0) {
        for (int s = 0; s < T16_NA; ++s) { mbar_init(&afull[s], T16_PROD_THREADS / (2 * T16_PROD_SETS)); mbar_init(&afree[s], 1); }
        for (int s = 0; s < T16_NB; ++s) { mbar_init(&bfull[s], 1); mbar_init(&bfree[s], 1); }
        for (int s = 0; s < T16_ACC; ++s) { mbar_init(&mma_done[s], 1); mbar_init(&tmem_empty[s], T16_EPI_WARPS); }
        for (int s = 0; s < T16_WBUFS; ++s) { mbar_init(&wfull[s], 1); mbar_init(&wfree[s], T16_PROD_THREADS); }
        mbar_fence_init();
    }
    constexpr int ISSUER = T16_EPI_WARPS + T16_PROD_WARPS, LOADER = ISSUER + T16_ISSUERS;
    if (threadIdx.x == LOADER * 32) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&maps.w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&maps.x) : "memory");
    }
    if (wid == ISSUER) {
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

    if (wid < T16_EPI_WARPS) {
        // ---------------- epilogue: one weight row per thread, 32 tokens ----------------
        const int q = wid & 3, cg = wid >> 2;
        const int row_l = 32 * q + lane;
        unsigned int *flags = g_gemm_flags[P.epoch & (TC_FLAG_SETS - 1)];
        bool ok = true;
        int n = 0;
        while (ok && walk.next(P, tile, kb0, kb1)) {
            const int rt = tile / P.tiles_tok, tt = tile - rt * P.tiles_tok;
            const int row = rt * T16_M + row_l, tokb = tt * T16_N + T16_EPI_TOKS * cg;
            float acc[T16_EPI_TOKS];
#pragma unroll
            for (int j = 0; j < T16_EPI_TOKS; ++j) acc[j] = 0.0f;
            const uint32_t tlane = tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(T16_EPI_TOKS * cg);
            for (int kb = kb0; kb < kb1; ++kb, ++n) {
                const int t = n & (T16_ACC - 1);
                if (!mbar_wait_bounded(&mma_done[t], (uint32_t)((n / T16_ACC) & 1), 20, 80)) { ok = false; break; }
                tc_fence_after();
                int v[16];
                tc_ld16(tlane + (uint32_t)(t * T16_N), v);
                const float dw = dwring[(n & (T16_DWRING - 1)) * T16_M + row_l];
                tc_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[j] = __fmaf_rn(dw, __int_as_float(v[j]), acc[j]);
                tc_ld16(tlane + (uint32_t)(t * T16_N + 16), v);
                tc_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&tmem_empty[t]);          // the block's sums are in registers
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[16 + j] = __fmaf_rn(dw, __int_as_float(v[j]), acc[16 + j]);
            }
            if (!ok) break;
            // ---- the tile (or this CTA's part of it) is done: undo the token's power-of-two scale
#pragma unroll
            for (int j = 0; j < T16_EPI_TOKS; ++j) acc[j] = __fmul_rn(acc[j], tokb + j < n_tok ? __ldg(tokscale + tokb + j) : 0.0f);
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
                        unsigned int fv;
                        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(fv) : "l"(f) : "memory");
                        if (fv != 0u) { there = true; break; }
                        __nanosleep(ns);
                        ns = min(ns * 2, 1024u);
                    }
                    if (!there) atomicExch(&g_device_status, STATUS_GRID_TIMEOUT);
                    *const_cast<volatile unsigned int *>(f) = 0u;     // lowered by its only reader (graph replays reuse the number)
                }
                asm volatile("bar.sync 1, %0;" ::"n"(T16_EPI_THREADS) : "memory");
                if (row < n_out) {
#pragma unroll
                    for (int j = 0; j < T16_EPI_TOKS; ++j)
                        if (tokb + j < n_tok) acc[j] = __fadd_rn(acc[j], __ldcg(yrow + j));
                }
            }
            if (row < n_out) {
                if (vec) {
#pragma unroll
                    for (int j = 0; j < T16_EPI_TOKS; j += 4)
                        if (tokb + j < n_tok) *reinterpret_cast<float4 *>(yrow + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
                } else {
#pragma unroll
                    for (int j = 0; j < T16_EPI_TOKS; ++j)
                        if (tokb + j < n_tok) yrow[j] = acc[j];
                }
            }
            if (late_part) {
                __threadfence();
                asm volatile("bar.sync 1, %0;" ::"n"(T16_EPI_THREADS) : "memory");
                if (threadIdx.x == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(flags + blockIdx.x), "r"(P.epoch) : "memory");
            }
        }
    } else if (wid < ISSUER) {
        // ---------------- code producers: thread (row p, K half g) of every second block: 64 codes -> 64 fp16 ----------------
        const int pi = threadIdx.x - T16_EPI_THREADS;
        // A warp reaches only the 32 tensor-memory lanes of its own quarter (warp index mod 4): producer warp pw takes
        // rows 32 (pw % 4) + lane, K half (pw / 4) % 2, and the blocks n with n % 2 == pw / 8.  Two sets on alternate
        // blocks because a warp's own chain per block -- raw loads, expansion, tcgen05.st, wait::st, fence, arrive -- is
        // ~1300 cycles long and was the kernel's period when every warp took every block.  The store of one block is
        // completed (wait::st, fence, arrive) only after the NEXT own block has been loaded and expanded.
        const int pw = pi >> 5, p = 32 * (pw & 3) + lane, g = (pw >> 2) & 1, set = pw >> 3;    // set: 0 when there is one set
        const uint32_t a_lane = tmem_base + ((uint32_t)(32 * (pw & 3)) << 16) + (uint32_t)T16_A_COL0;
        bool ok = true;
        int n = 0, oct = 0, pending = -1;           // pending: slot whose store is in flight
        while (ok && walk.next(P, tile, kb0, kb1)) {
            for (int kb = kb0; kb < kb1; ++kb, ++n) {
                if (kb == kb0 || (kb & 7) == 0) {
                    if (!mbar_wait_bounded(&wfull[oct % T16_WBUFS], (uint32_t)((oct / T16_WBUFS) & 1))) { ok = false; break; }
                    ++oct;
                }
                const int wbuf = (oct - 1) % T16_WBUFS;
                if ((n & (T16_PROD_SETS - 1)) == set) {
                    const int u = 2 * n + g, sa = u % T16_NA;
                    // The half's four code words sit at byte 34 j + 2 + 16 g of the row's 272-byte piece, 2-byte aligned:
                    // five aligned words and funnel shifts by 0 or 16 bits.  (Rows are 68 words apart: a warp's loads
                    // spread over eight banks, four passes each.)
                    const uint32_t off = (uint32_t)(kb & 7) * 34u + 2u + 16u * (uint32_t)g;
                    const uint8_t *rowp = wraw + (size_t)wbuf * TC_WRAW_BYTES + (size_t)p * 272;
                    const uint32_t *wa = reinterpret_cast<const uint32_t *>(rowp + (off & ~3u));
                    const uint32_t x0 = wa[0], x1 = wa[1], x2 = wa[2], x3 = wa[3], x4 = wa[4], sh = (off & 2u) * 8u;
                    const uint32_t dbits = g == 0 ? (uint32_t)*reinterpret_cast<const unsigned short *>(rowp + (kb & 7) * 34) : 0u;
                    uint32_t pc[32];
                    tc16_expand(__funnelshift_r(x0, x1, sh), pc);
                    tc16_expand(__funnelshift_r(x1, x2, sh), pc + 8);
                    tc16_expand(__funnelshift_r(x2, x3, sh), pc + 16);
                    tc16_expand(__funnelshift_r(x3, x4, sh), pc + 24);
                    if (pending >= 0) {
                        tc_st_wait();
                        tc_fence_before();
                        mbar_arrive(&afull[pending]);
                    }
                    if (!mbar_wait_bounded(&afree[sa], (uint32_t)(((u / T16_NA) & 1) ^ 1), 20, 80)) { ok = false; pending = -1; break; }
                    tc_fence_after();
                    if (g == 0) dwring[(n & (T16_DWRING - 1)) * T16_M + p] = f16_bits_to_f32(dbits);
                    tc_st32(a_lane + (uint32_t)(sa * T16_A_UNIT_COLS), pc);     // 64 fp16 = 32 columns of this thread's lane
                    pending = sa;
                }
                // every producer passes every block: at a piece's last block it has read all it needs of the piece
                if ((kb & 7) == 7 || kb == kb1 - 1) mbar_arrive(&wfree[wbuf]);
            }
        }
        if (pending >= 0) {
            tc_st_wait();
            tc_fence_before();
            mbar_arrive(&afull[pending]);
        }
    } else if (wid == LOADER) {
        // ---------------- weight loader: a piece (8 blocks x 128 rows, one tiled copy) as soon as its buffer is free ----------------
        int oct = 0;
        bool ok = true;
        while (ok && walk.next(P, tile, kb0, kb1)) {
            for (int kb = kb0; kb < kb1 && ok; kb = min(kb1, (kb | 7) + 1), ++oct) {
                const int wb = oct % T16_WBUFS;
                if (!mbar_wait_bounded(&wfree[wb], (uint32_t)(((oct / T16_WBUFS) & 1) ^ 1))) { ok = false; break; }
                if (elect_one()) {
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    mbar_expect_tx(&wfull[wb], (uint32_t)TC_WRAW_BYTES);
                    tma_load_2d(wraw + (size_t)wb * TC_WRAW_BYTES, &maps.w, (kb >> 3) * 68, (tile / P.tiles_tok) * T16_M, &wfull[wb]);
                }
                __syncwarp();
            }
        }
    } else if (wid == LOADER + 1) {
        // ---------------- activation loader: a block's boxes (two copies of 64 values x 64 tokens x {H, L}) ----------------
        int n = 0;
        bool ok = true;
        while (ok && walk.next(P, tile, kb0, kb1)) {
            const int tt = tile % P.tiles_tok;
            for (int kb = kb0; kb < kb1; ++kb, ++n) {
                const int sb = n % T16_NB;
                if (!mbar_wait_bounded(&bfree[sb], (uint32_t)(((n / T16_NB) & 1) ^ 1), 20, 80)) { ok = false; break; }
                if (elect_one()) {
                    uint8_t *b = bring + (size_t)sb * (2 * T16_BUNIT);
                    mbar_expect_tx(&bfull[sb], (uint32_t)(2 * T16_BUNIT));
                    tma_load_3d(b, &maps.x, kb * 128, tt * T16_N, 0, &bfull[sb]);
                    tma_load_3d(b + T16_BUNIT, &maps.x, kb * 128 + 64, tt * T16_N, 0, &bfull[sb]);
                }
                __syncwarp();
            }
        }
    } else {
        // ---------------- issuer: sixteen K = 16 MMAs per weight block, one accumulator ----------------
        // The whole warp walks the loop and waits; one elected lane issues.  Kept warp-uniform on purpose: the MMA takes
        // its operands from uniform registers, and inside a one-lane branch every operand had to be moved there first
        // (~70 cycles per MMA, measured).  Two such warps take alternate blocks: one warp's waits, fences and commits
        // are a serial chain of ~2000 cycles per block, more than the block's MMAs take; blocks use different
        // accumulators, so their MMAs may interleave, and a commit covers the issuing thread's own MMAs.
        const int me = wid - ISSUER;
        bool ok = true;
        int n = 0;
        while (ok && walk.next(P, tile, kb0, kb1)) {
            for (int kb = kb0; kb < kb1; ++kb, ++n) {
                if ((n & (T16_ISSUERS - 1)) != me) continue;
                const int t = n & (T16_ACC - 1);
                const uint32_t d = tmem_base + (uint32_t)(t * T16_N);
                // K half 0, then K half 1: each half's 8 MMAs (H and L planes x four K steps) go out as soon as its two
                // units are there, and the units are handed back as soon as the MMAs have read them.
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    const int u = 2 * n + g, sa = u % T16_NA, sb = n % T16_NB;
                    if (!mbar_wait_hot(&afull[sa], (uint32_t)((u / T16_NA) & 1))) { ok = false; break; }
                    if (g == 0 && (!mbar_wait_hot(&bfull[sb], (uint32_t)((n / T16_NB) & 1)) ||
                                   !mbar_wait_hot(&tmem_empty[t], (uint32_t)(((n / T16_ACC) & 1) ^ 1)))) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_t = tmem_base + (uint32_t)(T16_A_COL0 + sa * T16_A_UNIT_COLS);
                    const uint32_t b_lo = tc16_desc_lo(smem_u32(bring + (size_t)(2 * sb + g) * T16_BUNIT));
                    if (elect_one()) {
#pragma unroll
                        for (int m = 0; m < 8; ++m) {
                            const int pl = m >> 2, i = m & 3;
                            if (g == 0 && m == 0) tc_mma_f16_ts<false>(d, a_t, b_lo, C::IDESC);        // K step i: 16 fp16 = 8 columns of A
                            else tc_mma_f16_ts<true>(d, a_t + (uint32_t)(8 * i), b_lo + (uint32_t)(pl * ((T16_N * 128) >> 4) + 2 * i), C::IDESC);
                        }
                        tc_commit(&afree[sa]);
                        if (g == 1) {
                            tc_commit(&bfree[sb]);
                            tc_commit(&mma_done[t]);
                        }
                    }
                    __syncwarp();
                }
                if (!ok) break;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (wid == ISSUER) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

}  // namespace b200
