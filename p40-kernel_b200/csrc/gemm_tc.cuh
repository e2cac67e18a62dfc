// gemm_tc.cuh -- prefill mat-mul Y[n_out][n_tok] = W . X on the 5th-generation tensor cores.
//
// Replaces, for sm_100a, gemm_pq2_0_p40_kernel (src/kernels/gemm_p40.cu:44-139).  The contraction is
// a real dense one, so the integer dot products run as tcgen05.mma.kind::i8 with int32 accumulators
// in tensor memory.  Every 32-weight chunk has its own fp16 x fp16 scale, so chunks cannot be summed
// inside the tensor core: each K = 32 MMA writes its own TMEM columns (accumulate off), and the
// epilogue warps read the int32 tile back (tcgen05.ld), subtract the activation sum, convert, scale
// with (dw * da) and add into fp32 registers -- chunk by chunk, in the order of the reference's host
// loop (tests/test_p40.cpp:460-467), so Y is bit-identical to it.
//
// CTA tile: 128 weight rows x 64 tokens, K stepped one weight block (128 weights = 4 MMAs) at a time.
//   warps 0-7  : epilogue; warp w owns TMEM lanes 32 * (w & 3) .. (one weight row per thread) and
//                tokens 32 * (w >> 2) .. + 31 (32 fp32 accumulators per thread)
//   warps 8-11 : producers; expand the 2-bit codes of 128 rows x 1 block to int8 in the K-major
//                core-matrix layout the MMA reads (8 rows x 16 bytes per core matrix), copy the
//                int8 activations of 64 tokens x 4 chunks into the same layout, and set up the scale /
//                sum tables of the block
//   warp 12    : one thread issues the MMAs and commits them to an mbarrier; the warp owns the TMEM
//                allocation (512 columns = 2 stages x 4 chunks x 64 tokens)
// The byte order inside a chunk is the permuted one on both sides: extracting field k of a 16-code
// word gives the four codes that the activation quantiser stored as word k (src/pq2_0.h:120-125,
// 158-166), so no shuffle is needed on either operand.
// Every wait is bounded; on a time-out the CTA still reaches the common exit and frees its TMEM.
#pragma once

#include "common.cuh"

namespace b200 {

constexpr int TC_M = 128, TC_N = 64;
constexpr int TC_SMEM_STAGES = 4, TC_TMEM_STAGES = 2;
constexpr int TC_A_BYTES = 4 * TC_M * 32;                 // 4 chunks x 128 rows x 32 bytes
constexpr int TC_B_BYTES = 4 * TC_N * 32;
constexpr int TC_STAGE_BYTES = TC_A_BYTES + TC_B_BYTES + TC_M * 4 + 4 * TC_N * 4 + 4 * TC_N * 4;
constexpr int TC_EPI_THREADS = 256, TC_PROD_THREADS = 128, TC_THREADS = TC_EPI_THREADS + TC_PROD_THREADS + 32;
constexpr int TC_SMEM_BYTES = 1024 + TC_SMEM_STAGES * TC_STAGE_BYTES + 8192;   // > half an SM: one CTA (one TMEM owner) per SM

// Shared-memory matrix descriptor, K-major, no swizzle: core matrices of 8 rows x 16 bytes; the two
// core matrices along K are 128 bytes apart (leading offset), 8-row groups 256 bytes apart (stride).
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)(128 >> 4) << 16) | ((uint64_t)(256 >> 4) << 32) |
           (1ull << 46);
}
// Instruction descriptor: D = int32, A and B signed 8-bit (codes 0..3 are the same numbers signed),
// both K-major, N = 64, M = 128.
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
__device__ __forceinline__ void tc_ld32(uint32_t taddr, int (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

struct TcStage {
    uint8_t *a, *b;      // 4 x (128 x 32) and 4 x (64 x 32) int8, core-matrix layout
    float *dw;           // [128] weight scale of the block, per row
    float *da;           // [4][64] activation scale per chunk and token
    int *sn;             // [4][64] activation sum per chunk and token
};
__device__ __forceinline__ TcStage tc_stage(uint8_t *base, int s) {
    uint8_t *p = base + (size_t)s * TC_STAGE_BYTES;
    TcStage st;
    st.a = p;
    st.b = p + TC_A_BYTES;
    st.dw = reinterpret_cast<float *>(p + TC_A_BYTES + TC_B_BYTES);
    st.da = st.dw + TC_M;
    st.sn = reinterpret_cast<int *>(st.da + 4 * TC_N);
    return st;
}

__global__ void __launch_bounds__(TC_THREADS, 1) gemm_tc_kernel(const uint8_t *__restrict__ W, const uint32_t *__restrict__ Xq,
                                                                float *__restrict__ Y, int n_out, int nblocks, int n_tok) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);               // [4] producers -> issuer
    uint64_t *released = full + TC_SMEM_STAGES;                         // [4] epilogue -> producers
    uint64_t *mma_done = released + TC_SMEM_STAGES;                     // [2] tensor core -> epilogue
    uint64_t *tmem_empty = mma_done + TC_TMEM_STAGES;                   // [2] epilogue -> issuer
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tmem_empty + TC_TMEM_STAGES);
    uint8_t *stages = smem + 1024;

    const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.x * TC_M, tok0 = blockIdx.y * TC_N;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_SMEM_STAGES; ++s) { mbar_init(&full[s], TC_PROD_THREADS); mbar_init(&released[s], TC_EPI_THREADS); }
        for (int s = 0; s < TC_TMEM_STAGES; ++s) { mbar_init(&mma_done[s], 1); mbar_init(&tmem_empty[s], TC_EPI_THREADS); }
        mbar_fence_init();
    }
    if (wid == 12) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (wid < 8) {
        // ---------------- epilogue: one weight row per thread, 32 tokens ----------------
        const int q = wid & 3, hf = wid >> 2;
        const int row_l = 32 * q + lane;
        float acc[32];
#pragma unroll
        for (int t = 0; t < 32; ++t) acc[t] = 0.0f;
        for (int b = 0; b < nblocks; ++b) {
            const int s = b % TC_SMEM_STAGES, ts = b % TC_TMEM_STAGES;
            if (!mbar_wait_bounded(&mma_done[ts], (uint32_t)((b / TC_TMEM_STAGES) & 1))) break;
            tc_fence_after();
            const TcStage st = tc_stage(stages, s);
            const float dw = st.dw[row_l];
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                int v[32];
                tc_ld32(tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(ts * 256 + c * TC_N + 32 * hf), v);
                if (c == 3) {           // the tile of this stage is in registers: the tensor core may reuse it
                    tc_fence_before();
                    mbar_arrive(&tmem_empty[ts]);
                }
                const float4 *da4 = reinterpret_cast<const float4 *>(st.da + c * TC_N + 32 * hf);
                const int4 *sn4 = reinterpret_cast<const int4 *>(st.sn + c * TC_N + 32 * hf);
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    const float4 d = da4[g];
                    const int4 sm = sn4[g];
                    acc[4 * g + 0] = __fadd_rn(acc[4 * g + 0], __fmul_rn(__fmul_rn(dw, d.x), (float)(v[4 * g + 0] - sm.x)));
                    acc[4 * g + 1] = __fadd_rn(acc[4 * g + 1], __fmul_rn(__fmul_rn(dw, d.y), (float)(v[4 * g + 1] - sm.y)));
                    acc[4 * g + 2] = __fadd_rn(acc[4 * g + 2], __fmul_rn(__fmul_rn(dw, d.z), (float)(v[4 * g + 2] - sm.z)));
                    acc[4 * g + 3] = __fadd_rn(acc[4 * g + 3], __fmul_rn(__fmul_rn(dw, d.w), (float)(v[4 * g + 3] - sm.w)));
                }
            }
            mbar_arrive(&released[s]);          // the scale tables (and A/B) of this stage are free
        }
        const int row = row0 + row_l;
        if (row < n_out) {
#pragma unroll
            for (int t = 0; t < 32; ++t) {
                const int tok = tok0 + 32 * hf + t;
                if (tok < n_tok) Y[(size_t)row * n_tok + tok] = acc[t];
            }
        }
    } else if (wid < 12) {
        // ---------------- producers: expand codes, lay out activations ----------------
        const int p = threadIdx.x - TC_EPI_THREADS;            // 0..127 = weight row of the tile
        const int row = min(row0 + p, n_out - 1);               // rows past the end repeat the last one (never stored)
        const uint8_t *wrow = W + (size_t)row * nblocks * W_BLOCK_BYTES;
        const uint32_t a_off = (uint32_t)((p >> 3) * 256 + (p & 7) * 16);
        for (int b = 0; b < nblocks; ++b) {
            const int s = b % TC_SMEM_STAGES;
            if (!mbar_wait_bounded(&released[s], (uint32_t)(((b / TC_SMEM_STAGES) & 1) ^ 1))) break;
            const TcStage st = tc_stage(stages, s);
            const uint8_t *wb = wrow + (size_t)b * W_BLOCK_BYTES;
            // all 17 + 18 loads of this thread are issued before anything is stored: one memory round
            // trip per block instead of one per word
            uint32_t h[17];
#pragma unroll
            for (int i = 0; i < 17; ++i) h[i] = ldg_nc_u16(wb + 2 * i);
            constexpr int ACT_WORDS = 4 * TC_N * 9 / TC_PROD_THREADS;       // 18 words of Q8_1 per thread and block
            uint32_t av[ACT_WORDS];
#pragma unroll
            for (int j = 0; j < ACT_WORDS; ++j) {
                const int i = p + j * TC_PROD_THREADS;
                const int c = i / (TC_N * 9), rem = i - c * (TC_N * 9);
                const int t = rem / 9, w = rem - t * 9;
                av[j] = (tok0 + t < n_tok) ? __ldg(Xq + 9 * ((size_t)(4 * b + c) * n_tok + tok0 + t) + w) : 0u;
            }
            st.dw[p] = f16_bits_to_f32(h[0]);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint32_t w0 = h[1 + 4 * c] | (h[2 + 4 * c] << 16), w1 = h[3 + 4 * c] | (h[4 + 4 * c] << 16);
                uint4 lo, hi;
                lo.x = w0 & 0x03030303u; lo.y = (w0 >> 2) & 0x03030303u; lo.z = (w0 >> 4) & 0x03030303u; lo.w = (w0 >> 6) & 0x03030303u;
                hi.x = w1 & 0x03030303u; hi.y = (w1 >> 2) & 0x03030303u; hi.z = (w1 >> 4) & 0x03030303u; hi.w = (w1 >> 6) & 0x03030303u;
                uint8_t *ac = st.a + c * (TC_M * 32) + a_off;
                *reinterpret_cast<uint4 *>(ac) = lo;             // bytes 0..15 of the chunk: first K core matrix
                *reinterpret_cast<uint4 *>(ac + 128) = hi;       // bytes 16..31: second K core matrix
            }
#pragma unroll
            for (int j = 0; j < ACT_WORDS; ++j) {
                const int i = p + j * TC_PROD_THREADS;
                const int c = i / (TC_N * 9), rem = i - c * (TC_N * 9);
                const int t = rem / 9, w = rem - t * 9;
                const uint32_t v = av[j];
                if (w == 0) {
                    st.da[c * TC_N + t] = f16_bits_to_f32(v & 0xFFFFu);
                    st.sn[c * TC_N + t] = (int)(short)(v >> 16);
                } else {
                    const int k = w - 1;
                    *reinterpret_cast<uint32_t *>(st.b + c * (TC_N * 32) + (t >> 3) * 256 + (k >> 2) * 128 + (t & 7) * 16 +
                                                  (k & 3) * 4) = v;
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");    // the tensor core reads through the async proxy
            mbar_arrive(&full[s]);
        }
    } else if (lane == 0) {
        // ---------------- issuer: four K = 32 MMAs per weight block, one commit ----------------
        for (int b = 0; b < nblocks; ++b) {
            const int s = b % TC_SMEM_STAGES, ts = b % TC_TMEM_STAGES;
            if (!mbar_wait_bounded(&full[s], (uint32_t)((b / TC_SMEM_STAGES) & 1))) break;
            if (!mbar_wait_bounded(&tmem_empty[ts], (uint32_t)(((b / TC_TMEM_STAGES) & 1) ^ 1))) break;
            tc_fence_after();
            const TcStage st = tc_stage(stages, s);
#pragma unroll
            for (int c = 0; c < 4; ++c)
                tc_mma_i8(tmem_base + (uint32_t)(ts * 256 + c * TC_N), tc_smem_desc(smem_u32(st.a + c * (TC_M * 32))),
                          tc_smem_desc(smem_u32(st.b + c * (TC_N * 32))));
            tc_commit(&mma_done[ts]);
        }
    }
    // common exit: every role arrives here, also after a time-out, so the TMEM columns are always freed
    tc_fence_before();
    __syncthreads();
    if (wid == 12) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

}  // namespace b200
