// bonsai_b200.cu -- the C-ABI of the sm_100a build: argument checks, launch geometry, launches.
//
// One translation unit on purpose: every kernel shares the device status word of common.cuh.
// Host side mirrors the reference wrappers (src/kernels/gemv_p40.cu:200-219, gemm_p40.cu:143-154,
// gemv_repack_p40.cu:196-220, elementwise_p40.cu:75-80): validate, compute a grid, launch on the
// caller's stream, return cudaGetLastError().  No allocation, no synchronisation, no CPU fallback.
#include "../../include/bonsai_b200_ext.h"

#include "activation.cuh"
#include "gemm_simt.cuh"
#include "gemv.cuh"
#include "repack.cuh"
#include "synth.cuh"

#include <atomic>
#include <cstring>

using namespace b200;

namespace {

constexpr int SM_COUNT = 148;                 // B200
constexpr int SMEM_LIMIT = 227 * 1024;        // dynamic shared memory a CTA may opt into

std::atomic<int> g_opt_pdl{0};
std::atomic<int> g_opt_gemv_variant{-1};

inline cudaStream_t as_stream(bonsai_stream s) { return reinterpret_cast<cudaStream_t>(s); }
inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// cudaFuncSetAttribute is per device; remember which devices have been configured per kernel.
struct SmemOptIn {
    std::atomic<unsigned long long> done{0};
    template <typename K>
    cudaError_t ensure(K kernel) {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        const unsigned long long bit = 1ull << (dev & 63);
        if (done.load(std::memory_order_acquire) & bit) return cudaSuccess;
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT);
        if (e == cudaSuccess) done.fetch_or(bit, std::memory_order_release);
        return e;
    }
};

template <typename... KArgs, typename... Args>
cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl,
                   Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    if (pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Rows per CTA / per stage for the staged mat-vec kernels.  `row_bytes` is the row stride,
// `fixed` the shared memory that does not depend on the row count.
GemvPlan plan_rows(long long n_out, size_t row_bytes, size_t fixed, int variant) {
    // variant = rr_code * 100 + span_code * 10 + thread_code, or -1 for the tuned default
    int rr = 2, span_kb = 48, threads = 256;
    if (variant >= 0) {
        const int rr_code = variant / 100, span_code = (variant / 10) % 10, thr_code = variant % 10;
        rr = rr_code == 0 ? 1 : (rr_code == 1 ? 2 : 4);
        static const int spans[] = {16, 24, 32, 48, 64, 96, 128, 160};
        span_kb = spans[span_code & 7];
        threads = thr_code == 0 ? 128 : (thr_code == 1 ? 256 : (thr_code == 2 ? 192 : 64));
    }
    GemvPlan p;
    p.rr = rr;
    p.threads = threads;
    size_t budget = (size_t)span_kb * 1024;
    const size_t room = SMEM_LIMIT - 128 - fixed - 64;
    if (budget > room) budget = room;
    long long rows = (long long)(budget / row_bytes) & ~3ll;
    if (rows < 4) rows = 4;
    // do not leave SMs idle on small matrices: at most n_out / (2 * SM_COUNT) rows per CTA
    long long cap = ((n_out + 2 * SM_COUNT - 1) / (2 * SM_COUNT) + 3) & ~3ll;
    if (cap < 4) cap = 4;
    if (rows > cap) rows = cap;
    p.rows_per_cta = (int)rows;
    int rps = (int)((rows + GEMV_MAX_STAGES - 1) / GEMV_MAX_STAGES);
    // a stage of roughly 8 KB or more keeps the number of bulk copies low
    const int min_rows = (int)((8192 + row_bytes - 1) / row_bytes);
    if (rps < min_rows) rps = min_rows;
    rps = (rps + 3) & ~3;
    p.rows_per_stage = rps;
    p.smem_bytes = (int)(128 + fixed + (size_t)rows * row_bytes + 64);
    return p;
}

}  // namespace

extern "C" {

int bonsai_p40_quant_activations(const float *x, void *out, int64_t n, bonsai_stream stream) {
    if (n <= 0 || n % 32 != 0) return 1;
    if (!aligned16(x) || (reinterpret_cast<uintptr_t>(out) & 3u)) return 1;
    const long long threads = n / 4;
    const int blocks = (int)((threads + 255) / 256);
    quant_q8_1_kernel<<<blocks, 256, 0, as_stream(stream)>>>(x, static_cast<uint32_t *>(out), (int)n, 1);
    return (int)cudaGetLastError();
}

int bonsai_p40_fwht(float *x, const float *signs, int64_t n, bonsai_stream stream) {
    if (n <= 0 || n % FWHT_N != 0) return 1;
    if (!aligned16(x) || (signs && !aligned16(signs))) return 1;
    const int warps = (int)(n / FWHT_N);
    fwht_quant_kernel<<<(warps + 3) / 4, 128, 0, as_stream(stream)>>>(x, signs, x, nullptr, (int)n, 1);
    return (int)cudaGetLastError();
}

int bonsai_b200_fwht_quant(const float *x, const float *signs, void *xq, float *x_rot, int64_t n,
                           bonsai_stream stream) {
    if (n <= 0 || n % FWHT_N != 0) return 1;
    if (!aligned16(x) || (signs && !aligned16(signs)) || (x_rot && !aligned16(x_rot))) return 1;
    if (reinterpret_cast<uintptr_t>(xq) & 3u) return 1;
    const int warps = (int)(n / FWHT_N);
    fwht_quant_kernel<<<(warps + 3) / 4, 128, 0, as_stream(stream)>>>(x, signs, x_rot, static_cast<uint32_t *>(xq),
                                                                      (int)n, 1);
    return (int)cudaGetLastError();
}

int bonsai_b200_quant_batch(const float *X, const float *signs, void *Xq, int64_t n_in, int64_t n_tok, int rotate,
                            bonsai_stream stream) {
    if (n_in <= 0 || n_tok <= 0 || n_in % 32 != 0) return 1;
    if (rotate && n_in % FWHT_N != 0) return 1;
    if (!aligned16(X) || (signs && !aligned16(signs)) || (reinterpret_cast<uintptr_t>(Xq) & 3u)) return 1;
    if (n_in > INT32_MAX || n_tok > INT32_MAX) return 1;
    if (rotate) {
        const long long warps = (n_in / FWHT_N) * n_tok;
        fwht_quant_kernel<<<(unsigned)((warps + 3) / 4), 128, 0, as_stream(stream)>>>(
            X, signs, nullptr, static_cast<uint32_t *>(Xq), (int)n_in, (int)n_tok);
    } else {
        const long long threads = n_in / 4 * n_tok;
        long long blocks = (threads + 255) / 256;
        if (blocks > 8 * SM_COUNT * 4) blocks = 8 * SM_COUNT * 4;
        quant_q8_1_kernel<<<(unsigned)blocks, 256, 0, as_stream(stream)>>>(X, static_cast<uint32_t *>(Xq), (int)n_in,
                                                                           (int)n_tok);
    }
    return (int)cudaGetLastError();
}

int bonsai_p40_gemv(const void *W, const void *xq, float *y, int64_t n_out, int64_t n_in, bonsai_stream stream) {
    if (n_in <= 0 || n_in % 128 != 0) return 1;
    if (n_out <= 0) return 0;
    if (n_out > INT32_MAX || n_in / 128 > INT32_MAX / 64) return 1;
    const int nblocks = (int)(n_in / 128);
    const bool pdl = g_opt_pdl.load() != 0;
    const size_t row_bytes = (size_t)nblocks * W_BLOCK_BYTES;
    const size_t act_bytes = (size_t)(nblocks / 2) * ACT_REC_WORDS * 4;
    const bool staged = (nblocks % 2 == 0) && aligned16(W) && !(reinterpret_cast<uintptr_t>(xq) & 3u) &&
                        (128 + act_bytes + 4 * row_bytes + 64 <= (size_t)SMEM_LIMIT);
    if (!staged) {
        return (int)launch(gemv_pq2_generic_kernel, dim3((unsigned)((n_out + 7) / 8)), dim3(256), 0, as_stream(stream),
                           pdl, static_cast<const uint8_t *>(W), static_cast<const uint8_t *>(xq), y, (int)n_out,
                           nblocks);
    }
    const GemvPlan p = plan_rows(n_out, row_bytes, act_bytes, g_opt_gemv_variant.load());
    const dim3 grid((unsigned)((n_out + p.rows_per_cta - 1) / p.rows_per_cta));
    static SmemOptIn opt1, opt2, opt4;
    cudaError_t e;
    auto go = [&](auto kernel, SmemOptIn &opt) -> cudaError_t {
        cudaError_t err = opt.ensure(kernel);
        if (err != cudaSuccess) return err;
        return launch(kernel, grid, dim3(p.threads), (size_t)p.smem_bytes, as_stream(stream), pdl,
                      static_cast<const uint8_t *>(W), static_cast<const uint32_t *>(xq), y, (int)n_out, nblocks / 2,
                      p.rows_per_cta, p.rows_per_stage);
    };
    if (p.rr == 1) e = go(gemv_pq2_kernel<1>, opt1);
    else if (p.rr == 2) e = go(gemv_pq2_kernel<2>, opt2);
    else e = go(gemv_pq2_kernel<4>, opt4);
    return (int)e;
}

int bonsai_b200_gemv_chunk_sums(const void *W, const void *xq, int32_t *out, int64_t row0, int64_t n_rows,
                                int64_t n_in, bonsai_stream stream) {
    if (n_in <= 0 || n_in % 128 != 0 || row0 < 0) return 1;
    if (n_rows <= 0) return 0;
    if (n_rows > INT32_MAX || (reinterpret_cast<uintptr_t>(xq) & 3u)) return 1;
    const long long total = n_rows * (n_in / 32);
    long long blocks = (total + 255) / 256;
    if (blocks > 16 * SM_COUNT) blocks = 16 * SM_COUNT;
    gemv_chunk_sums_kernel<<<(unsigned)blocks, 256, 0, as_stream(stream)>>>(
        static_cast<const uint8_t *>(W), static_cast<const uint8_t *>(xq), out, row0, (int)n_rows, (int)(n_in / 128));
    return (int)cudaGetLastError();
}

int bonsai_p40_gemm(const void *W, const void *Xq, float *Y, int64_t n_out, int64_t n_in, int64_t n_tok,
                    bonsai_stream stream) {
    if (n_in <= 0 || n_in % 128 != 0) return 1;
    if (n_out <= 0 || n_tok <= 0) return 0;
    if (n_out > INT32_MAX || n_tok > INT32_MAX || (reinterpret_cast<uintptr_t>(Xq) & 3u)) return 1;
    const dim3 grid((unsigned)((n_out + GS_ROWS - 1) / GS_ROWS), (unsigned)((n_tok + GS_TOKS - 1) / GS_TOKS));
    if (grid.y > 65535) return 1;
    gemm_simt_kernel<<<grid, 256, 0, as_stream(stream)>>>(static_cast<const uint8_t *>(W),
                                                          static_cast<const uint32_t *>(Xq), Y, (int)n_out,
                                                          (int)(n_in / 128), (int)n_tok);
    return (int)cudaGetLastError();
}

int bonsai_p40_repack(const void *src, void *dst, int64_t n_out, int64_t n_in, bonsai_stream stream) {
    if (n_in % 128 != 0 || n_out <= 0) return 1;
    const int64_t nb = n_in / 128;
    if (nb <= 0 || nb % 8 != 0 || nb > INT32_MAX / 64) return 1;
    if (!aligned16(dst) || (reinterpret_cast<uintptr_t>(src) & 1u)) return 1;
    const long long total = n_out * 4 * nb;
    long long blocks = (total + 255) / 256;
    if (blocks > 32 * SM_COUNT) blocks = 32 * SM_COUNT;
    repack_kernel<<<(unsigned)blocks, 256, 0, as_stream(stream)>>>(static_cast<const uint8_t *>(src),
                                                                   static_cast<uint8_t *>(dst), n_out, (int)nb);
    return (int)cudaGetLastError();
}

int bonsai_p40_gemv_repack(const void *W, const float *x, float *y, int64_t n_out, int64_t n_in,
                           bonsai_stream stream) {
    if (n_in % 128 != 0 || n_out <= 0) return 1;
    const int64_t nb64 = n_in / 128;
    if (nb64 <= 0 || nb64 % 8 != 0 || n_out > INT32_MAX) return 1;
    const int nb = (int)nb64;
    const size_t row_bytes = (size_t)nb * W_BLOCK_BYTES;
    const size_t act_bytes = (size_t)4 * nb * RP_REC_WORDS * 4;
    // the reference refuses vectors whose Q8_1 image exceeds 48 KiB; this build takes anything that
    // leaves room for four rows beside the activation records
    if (128 + act_bytes + 4 * row_bytes + 64 > (size_t)SMEM_LIMIT) return 1;
    if (!aligned16(W) || !aligned16(x)) return 1;
    const bool pdl = g_opt_pdl.load() != 0;
    const GemvPlan p = plan_rows(n_out, row_bytes, act_bytes, g_opt_gemv_variant.load());
    const dim3 grid((unsigned)((n_out + p.rows_per_cta - 1) / p.rows_per_cta));
    static SmemOptIn opt1, opt2, opt4;
    auto go = [&](auto kernel, SmemOptIn &opt) -> cudaError_t {
        cudaError_t err = opt.ensure(kernel);
        if (err != cudaSuccess) return err;
        return launch(kernel, grid, dim3(p.threads), (size_t)p.smem_bytes, as_stream(stream), pdl,
                      static_cast<const uint8_t *>(W), x, y, (int)n_out, nb, p.rows_per_cta, p.rows_per_stage);
    };
    cudaError_t e;
    if (p.rr == 1) e = go(gemv_repack_kernel<1>, opt1);
    else if (p.rr == 2) e = go(gemv_repack_kernel<2>, opt2);
    else e = go(gemv_repack_kernel<4>, opt4);
    return (int)e;
}

int bonsai_b200_synth_pq2_0(void *W, int64_t first_block, int64_t n_blocks, uint64_t seed, bonsai_stream stream) {
    if (n_blocks <= 0) return n_blocks == 0 ? 0 : 1;
    if (reinterpret_cast<uintptr_t>(W) & 1u) return 1;
    long long blocks = (n_blocks * 17 + 255) / 256;
    if (blocks > 64 * SM_COUNT) blocks = 64 * SM_COUNT;
    synth_pq2_kernel<<<(unsigned)blocks, 256, 0, as_stream(stream)>>>(static_cast<unsigned short *>(W), first_block,
                                                                      n_blocks, seed);
    return (int)cudaGetLastError();
}

int bonsai_b200_set_option(const char *key, int64_t value) {
    if (!key) return 1;
    if (!std::strcmp(key, "pdl")) { g_opt_pdl.store(value != 0); return 0; }
    if (!std::strcmp(key, "gemv_variant")) { g_opt_gemv_variant.store((int)value); return 0; }
    return 1;
}

int bonsai_b200_device_status(void) {
    int v = -1;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return (int)e + 1000;
    e = cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int));
    if (e != cudaSuccess) return (int)e + 1000;
    return v;
}

int bonsai_b200_version(void) { return 100; }

// Not on the PQ2_0 mat-vec / mat-mul path: exported so that programs written against the reference
// link; each refuses without touching its arguments (reference: include/bonsai_p40.h:44-56).
int bonsai_p40_rmsnorm(const float *, const float *, float *, int64_t, int64_t, float, bonsai_stream) {
    return BONSAI_P40_ENOTIMPL;
}
int bonsai_p40_gdn_step(float *, const float *, const float *, const float *, const float *, const float *, float *,
                        int, int, int, int, bonsai_stream) {
    return BONSAI_P40_ENOTIMPL;
}
int bonsai_p40_attn(const float *, const float *, const float *, float *, int, int, int, int, float, bonsai_stream) {
    return BONSAI_P40_ENOTIMPL;
}

}  // extern "C"
