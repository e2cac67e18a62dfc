// bonsai_b200.cu -- the C-ABI of the sm_100a build: argument checks, launch geometry, launches.
//
// One translation unit on purpose: every kernel shares the device status word of common.cuh.
// Host side mirrors the reference wrappers (src/kernels/gemv_p40.cu:200-219, gemm_p40.cu:143-154,
// gemv_repack_p40.cu:196-220, elementwise_p40.cu:75-80): validate, compute a grid, launch on the
// caller's stream, return cudaGetLastError().  No allocation, no synchronisation, no CPU fallback.
#include "../../include/bonsai_b200_ext.h"
#include "../../include/bonsai_kv.h"

#include "activation.cuh"
#include "gemm_simt.cuh"
#include "gemm_tc.cuh"
#include "gemm_tc16.cuh"
#include "gemv.cuh"
#include "gemv_stream.cuh"
#include "gemv_chain.cuh"
#include "gemv_mma.cuh"
#include "kv.cuh"
#include "ops.cuh"
#include "probe.cuh"
#include "ptq.cuh"
#include "repack.cuh"
#include "synth.cuh"

#include <atomic>
#include <cstring>
#include <mutex>
#include <new>
#include <type_traits>
#include <vector>

using namespace b200;

namespace {

constexpr int SM_COUNT = 148;                 // B200
constexpr int SMEM_LIMIT = 227 * 1024;        // dynamic shared memory a CTA may opt into

std::atomic<int> g_opt_pdl{0};
std::atomic<int> g_opt_gemv_variant{-1};
std::atomic<int> g_opt_gemv_order{0};
std::atomic<int> g_opt_fuse_linear{0};         // 1: bonsai_b200_linear runs as one kernel when it can (measured slower)
std::atomic<int> g_opt_chain_threads{512};       // threads per CTA of the chain kernel: 512 (5 blocks per lane and task), 640 (4), 768 (3)
std::atomic<int> g_opt_chain_spread_nb{40};      // dependent ops with at least this many blocks per row rotate their input
                                                 // once for the grid instead of once per CTA; 0 = never
std::atomic<int> g_opt_chain_tile_kb{16};
std::atomic<int> g_opt_gemm_tile{0};              // fp16 tensor-core mat-mul: 0 by token count, 64 or 128 tokens per tile
std::atomic<int> g_opt_chain_seg{40};            // longest row segment of one task, in blocks: 8, 16, 24, 32 or 40        // target bytes of one ring slot
std::atomic<int> g_opt_gemm_path{-1};          // -1: by token count, 0: integer SIMT kernel, 1: tensor cores, 2: small-batch kernel, 3: integer tensor-core kernel          // 0: streaming kernel (fixed tree order), 1: the host's sequential order

inline cudaStream_t as_stream(bonsai_stream s) { return reinterpret_cast<cudaStream_t>(s); }
inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool aligned4(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 3u) == 0; }

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

// ceil(2^32 / d): __umulhi(n, magic) == n / d for every n with n * d < 2^32; 0 stands for d == 1.
inline uint32_t magic_u32(uint32_t d) {
    if (d <= 1) return 0u;
    return (uint32_t)(((1ull << 32) + d - 1) / d);
}

// Geometry of the streaming mat-vec (gemv_stream.cuh).
// variant = thr_code * 1000 + seg_code * 100 + tile_code * 10 + cap_code, -1 = default.
bool plan_stream(long long n_out, int nb, int variant, StreamParams &p, int &threads, int &smem_bytes) {
    if (nb % 2 != 0) return false;                  // rows must start on a word boundary
    int seg = 8 * STREAM_STEPS, tile_kb = 16, cap_kb = 108;
    threads = 512;
    if (variant >= 0) {
        static const int thr[] = {512, 384, 256, 128};
        static const int segs[] = {40, 32, 24, 16, 8, 40, 40, 40};
        static const int tiles[] = {16, 8, 12, 24, 32, 48, 6, 4};
        static const int caps[] = {108, 200, 72, 150};
        threads = thr[(variant / 1000) & 3];
        seg = segs[(variant / 100) % 10 & 7];
        tile_kb = tiles[(variant / 10) % 10 & 7];
        cap_kb = caps[variant % 10 & 3];
    }
    auto round_up = [](long long v, long long m) { return (v + m - 1) / m * m; };
    long long ctas = (n_out + 3) / 4;
    if (ctas > SM_COUNT) ctas = SM_COUNT;
    long long rows = round_up((n_out + ctas - 1) / ctas, 4);
    p.n_out = (int)n_out;
    p.nb = nb;
    const size_t row_bytes = (size_t)nb * W_BLOCK_BYTES;
    // segments: equal multiples of 8 blocks (every block lane of a task gets the same count), at most
    // what a task holds in registers
    p.nseg = (nb + seg - 1) / seg;
    p.seg_blocks = (int)round_up((nb + p.nseg - 1) / p.nseg, 8);
    if (p.seg_blocks > 8 * STREAM_STEPS) p.seg_blocks = 8 * STREAM_STEPS;
    p.nseg = (nb + p.seg_blocks - 1) / p.seg_blocks;
    for (int attempt = 0;; ++attempt) {
        const size_t fixed = 2 * RING_MAX_TILES * 8 + (size_t)nb * (STREAM_ACT_WORDS * 4 + 32) +
                             (size_t)rows * p.nseg * 4 + (size_t)((rows / 4 + 3) & ~3) * 4 + 16;
        if ((size_t)cap_kb * 1024 < fixed + 64) return false;
        const size_t room = (size_t)cap_kb * 1024 - fixed - 64;
        long long tr = ((long long)tile_kb * 1024 / (long long)row_bytes) & ~3ll;
        if (tr < 4) tr = 4;
        if (tr > rows) tr = rows;
        while (tr > 4 && 3 * ((size_t)tr * row_bytes + 16) > room) tr -= 4;
        if (2 * ((size_t)tr * row_bytes + 16) > room) return false;
        long long nslot = (long long)(room / ((size_t)tr * row_bytes + 16));
        if (nslot > RING_MAX_SLOTS) nslot = RING_MAX_SLOTS;
        const long long ntiles = (rows + tr - 1) / tr;
        if (ntiles > RING_MAX_TILES) {          // very tall matrix: more CTAs, each with fewer rows
            if (attempt > 64) return false;
            const long long k = attempt + 2;
            rows = round_up((n_out + SM_COUNT * k - 1) / (SM_COUNT * k), 4);
            continue;
        }
        p.rows_per_cta = (int)rows;
        p.tr = (int)tr;
        p.nslot = (int)nslot;
        p.tpt = (p.tr / 4) * p.nseg;
        p.magic_tpt = magic_u32((uint32_t)p.tpt);
        p.magic_nseg = magic_u32((uint32_t)p.nseg);
        p.magic_nslot = magic_u32((uint32_t)p.nslot);
        smem_bytes = (int)(fixed + (size_t)p.nslot * ((size_t)tr * row_bytes + 16) + 64);
        return true;
    }
}

// Geometry of the tensor-core mat-vec (gemv_mma.cuh): tiles of 16 rows x one row segment, a ring of slots as deep
// as `cap_kb` of shared memory allows.  Rows must start on a word (nb even); rows longer than one segment are cut at
// multiples of 8 blocks (16-byte aligned pieces), which needs nb % 8 == 0.
bool plan_mma(long long n_out, int nb, int cap_kb, MmaGeom &P, int &smem_bytes, int &grid) {
    if (nb <= 0 || nb % 2 != 0) return false;
    P = MmaGeom{};
    P.n_out = (int)n_out;
    P.nb = nb;
    P.ngroups = (int)((n_out + 15) / 16);
    int seg_max;
    if (nb % 8 == 0) {
        const int units = nb / 8;
        P.nseg = (nb + MMA_SEG_MAX - 1) / MMA_SEG_MAX;
        P.seg_q = units / P.nseg;
        P.seg_r = units % P.nseg;
        seg_max = 8 * (P.seg_q + (P.seg_r ? 1 : 0));
    } else {
        if (nb > MMA_SEG_MAX + 8) return false;
        P.nseg = 1;
        seg_max = nb;
    }
    P.pairs_max = seg_max / 2;
    const int row_bytes = nb * W_BLOCK_BYTES;
    if (nb % 8 == 0) {
        // rows of a tile 16 * (odd) bytes apart: the 8 rows a load instruction touches fall into 8 different bank groups
        int stride = seg_max * W_BLOCK_BYTES;
        if ((stride / 16) % 2 == 0) stride += 16;
        P.contiguous = (P.nseg == 1 && stride == row_bytes) ? 1 : 0;
        P.stride = stride;
    } else {
        P.contiguous = 1;
        P.stride = row_bytes;
    }
    P.slot_bytes = (16 * P.stride + 127) & ~127;
    auto fixed = [&](int n) { return mma_fixed_bytes(P, n); };
    int nslot = MMA_MAX_SLOTS;
    while (nslot >= 2 && fixed(nslot) + (size_t)nslot * P.slot_bytes > (size_t)cap_kb * 1024) --nslot;
    if (nslot < 2) return false;
    P.nslot = nslot;
    P.magic_pairs = magic_u32((uint32_t)P.pairs_max);
    P.magic_nseg = magic_u32((uint32_t)P.nseg);
    P.magic_nslot = magic_u32((uint32_t)P.nslot);
    smem_bytes = (int)(fixed(nslot) + (size_t)nslot * P.slot_bytes);
    grid = P.ngroups < SM_COUNT ? P.ngroups : SM_COUNT;
    return true;
}

// Geometry of the small-batch mat-mul (gemv_mma.cuh, gemm_mma_kernel): tiles of 16 rows x one segment of at most
// MMAB_SEG_UNITS * 8 blocks, brought by one tiled copy when rows are a multiple of 8 blocks (16-byte aligned segment
// starts, row pitch a multiple of 16), else whole rows by one bulk copy (rows of at most 48 blocks).
bool plan_mmab(long long n_out, int nb, int n_tok, int cap_kb, MmabGeom &P, int &smem_bytes, int &grid) {
    if (nb <= 0 || nb % 2 != 0 || n_tok < 1 || n_tok > 16) return false;
    P = MmabGeom{};
    P.ntg = n_tok > 8 ? 2 : 1;
    // The segments and the items fix the order in which a row's terms are added: they depend on the row's length and
    // the token count only, never on n_out, so that a row slice gives the bits of the whole matrix.
    const int seg_units = P.ntg == 2 ? 1 : (nb >= 64 ? MMAB_SEG_UNITS : 2);
    // Two row groups per tile (a chunk's activation and header loads serve two MMAs) pay when a CTA has enough groups
    // to keep its warps busy with tiles of twice the size, and when the ring stays deep (16-block segments): measured
    // 172 -> 160 us on 5120 x 248320; with 2 .. 3 groups per CTA (17408 x 5120) 23 -> 29 us.
    P.nrg = (P.ntg == 1 && seg_units == 2 && (n_out + 15) / 16 >= 6ll * SM_COUNT) ? 2 : 1;
    P.n_out = (int)n_out;
    P.nb = nb;
    P.ngroups = (int)((n_out + 15) / 16);
    int seg_max;
    if (nb % 8 == 0) {
        const int units = nb / 8;
        P.nseg = (units + seg_units - 1) / seg_units;
        P.seg_q = units / P.nseg;
        P.seg_r = units % P.nseg;
        seg_max = 8 * (P.seg_q + (P.seg_r ? 1 : 0));
        int s16 = seg_max * W_BLOCK_BYTES / 16;         // rows of a tile 16 * (odd) bytes apart
        if (s16 % 2 == 0) ++s16;
        P.stride = 16 * s16;
        P.tiled = 1;
    } else {
        if (nb > 48 || P.ntg > 1) return false;
        P.nseg = 1;
        seg_max = nb;
        P.stride = nb * W_BLOCK_BYTES;
        P.tiled = 0;
    }
    P.pairs_max = seg_max / 2;
    P.ppi = P.ntg == 2 ? 1 : 2;                         // an item is 16 MMAs
    P.items = (P.pairs_max + P.ppi - 1) / P.ppi;
    P.slot_bytes = (P.nrg * 16 * P.stride + 127) & ~127;
    P.act_bufs = P.nseg > 1 ? 3 : 1;
    P.act_tab_off = (seg_max * 4 * n_tok * 36 + 8 * P.ntg * 36 + 127) & ~127;       // + what lanes past n_tok read beyond the last block
    P.act_buf_bytes = P.act_tab_off + seg_max * 4 * 64 * P.ntg;
    int nslot = MMA_MAX_SLOTS;
    while (nslot >= 2 && mmab_fixed_bytes(P, nslot) + (size_t)nslot * P.slot_bytes > (size_t)cap_kb * 1024) --nslot;
    if (nslot < 2) return false;
    P.nslot = nslot;
    P.magic_nslot = magic_u32((uint32_t)nslot);
    P.magic_bt = magic_u32((uint32_t)(MMAB_GB / P.nrg * P.nseg));
    P.magic_items = magic_u32((uint32_t)P.items);
    // tile and step numbers stay small enough for the multiplicative divisions of the kernel
    const long long groups_per_cta = (P.ngroups + SM_COUNT - 1) / SM_COUNT;
    if (groups_per_cta * P.nseg * P.items >= (1 << 24) || (groups_per_cta / MMAB_GB + 1) * P.nseg >= 65536) return false;
    smem_bytes = (int)(mmab_fixed_bytes(P, nslot) + (size_t)nslot * P.slot_bytes);
    grid = P.ngroups < SM_COUNT ? P.ngroups : SM_COUNT;
    return true;
}

// Geometry of the ring mat-vec: one CTA per SM, tiles of about 16 rows by one row segment, a ring that
// keeps the CTA under half of an SM's shared memory.
// variant = thr_code * 100000 + rr_code * 10000 + seg_code * 1000 + rs_code * 100 + chain_code * 10 + cap_code,
// -1 = default.
bool plan_ring(long long n_out, int npairs, int variant, RingParams &p, int &threads, int &smem_bytes, int &rr) {
    rr = 2;
    int seg_pairs = 16, rs_target = 16, chain = 3, cap_kb = 108;
    threads = 1024;
    if (variant >= 0) {
        static const int rrs[] = {1, 2, 4, 2};
        static const int segs[] = {16, 12, 20, 24, 32, 8, 1 << 20, 16};
        static const int rst[] = {16, 8, 32, 12, 24, 4, 16, 16};
        static const int chains[] = {3, 5, 1, 7};    // odd: with the copy warp an even count of warps computes
        static const int caps[] = {108, 200, 72, 150};
        rr = rrs[(variant / 10000) & 3];
        seg_pairs = segs[(variant / 1000) % 10 & 7];
        rs_target = rst[(variant / 100) % 10 & 7];
        chain = chains[(variant / 10) % 10 & 3];
        cap_kb = caps[variant % 10 & 3];
        static const int thr[] = {1024, 512, 768, 256};
        threads = thr[(variant / 100000) & 3];
    }
    if (rr == 4 && threads > 512) threads = 512;        // register budget of the four-row variant
    auto round_up = [](long long v, long long m) { return (v + m - 1) / m * m; };
    const int granule = npairs % 4 == 0 ? 1 : (npairs % 2 == 0 ? 2 : 4);      // rows per 16-byte aligned run
    const int unit = granule > rr ? granule : rr;
    long long ctas = (n_out + unit - 1) / unit;
    if (ctas > SM_COUNT) ctas = SM_COUNT;
    long long rows = round_up((n_out + ctas - 1) / ctas, unit);
    // a CTA has RING_MAX_TILES single-use barrier pairs: very tall matrices take more CTAs per SM
    const long long nseg_est = (npairs % 4 == 0 && npairs >= 2 * seg_pairs) ? npairs / seg_pairs : 1;
    const long long max_rows = (RING_MAX_TILES / nseg_est) * unit;      // tiles hold at least `unit` rows
    if (rows > max_rows) {
        const long long k = (n_out + max_rows * SM_COUNT - 1) / (max_rows * SM_COUNT);
        rows = round_up((n_out + SM_COUNT * k - 1) / (SM_COUNT * k), unit);
    }
    p.n_out = (int)n_out;
    p.npairs = npairs;
    p.rows_per_cta = (int)rows;
    if (npairs % 4 == 0 && npairs >= 2 * seg_pairs) {
        p.seg_base = seg_pairs;
        p.nseg = npairs / seg_pairs;
        p.sp = npairs - (p.nseg - 1) * seg_pairs;
        p.sw = 17 * p.sp;
        if ((p.sw / 4) % 2 == 0) p.sw += 4;            // odd count of 16-byte units: rows spread over 8 bank groups
    } else {
        p.nseg = 1;
        p.seg_base = p.sp = npairs;
        p.sw = 17 * npairs;
    }
    const size_t fixed = RING_BAR_BYTES + (size_t)npairs * ACT_REC_WORDS * 4;
    const size_t room = (size_t)cap_kb * 1024 > fixed + 64 ? (size_t)cap_kb * 1024 - fixed - 64 : 0;
    p.ts = 8 * p.sp + 4;                                   // an odd count of 16-byte units per row
    p.ntb = 3;
    long long rs = rs_target < rows ? round_up((rows + (rows + rs_target - 1) / rs_target - 1) /
                                               ((rows + rs_target - 1) / rs_target), unit)
                                    : rows;
    if (rs > 32) rs = 32 / unit * unit;
    auto need = [&](long long r, int slots) { return (size_t)r * ((size_t)p.sw * 4 * slots + (size_t)p.ts * 4 * p.ntb); };
    while (rs > unit && need(rs, 3) > room) rs -= unit;                 // three weight slots at least
    if (need(rs, 2) > room || rs < unit) return false;
    p.rs = (int)rs;
    long long nslot = (long long)((room - (size_t)rs * p.ts * 4 * p.ntb) / ((size_t)rs * p.sw * 4));
    if (nslot > RING_MAX_SLOTS) nslot = RING_MAX_SLOTS;
    p.nslot = (int)nslot;
    p.chain_warps = chain;
    if (((rows + p.rs - 1) / p.rs) * p.nseg > RING_MAX_TILES) return false;
    p.ppt = (p.rs / rr) * p.sp;
    p.magic_ppt = magic_u32((uint32_t)p.ppt);
    p.magic_sp = magic_u32((uint32_t)p.sp);
    p.magic_nseg = magic_u32((uint32_t)p.nseg);
    p.magic_nslot = magic_u32((uint32_t)p.nslot);
    p.magic_ntb = magic_u32((uint32_t)p.ntb);
    smem_bytes = (int)(fixed + need(p.rs, p.nslot) + 64);
    return true;
}

// Geometry of the staged mat-vec kernels.  `row_bytes` is the row stride, `fixed` the shared
// memory that does not depend on the row count, `granule` the row multiple that keeps a run of
// rows 16-byte aligned.  CTA counts are multiples of the SM count, so every SM gets the same
// share, and a CTA stays under half of an SM's shared memory so that a second CTA -- of this launch
// or, with programmatic launches, of the next kernel in the stream -- can stream beside it.
GemvPlan plan_rows(long long n_out, size_t row_bytes, size_t fixed, int granule, int variant) {
    // variant = rr_code * 1000 + cap_code * 100 + stage_code * 10 + thread_code, or -1 = tuned default
    int rr = 2, cap_kb = 111, stage_kb = 8, threads = 512;
    if (variant >= 0) {
        static const int rrs[] = {1, 2, 4, 2};
        static const int caps[] = {111, 220, 72, 56};
        static const int stages[] = {4, 8, 12, 16, 24, 32, 48, 64};
        static const int thr[] = {256, 512, 1024, 384};
        rr = rrs[(variant / 1000) & 3];
        cap_kb = caps[(variant / 100) % 10 & 3];
        stage_kb = stages[(variant / 10) % 10 & 7];
        threads = thr[variant % 10 & 3];
    }
    if (rr == 4 && threads > 512) threads = 512;       // register budget of the four-row variant
    const int unit = granule > rr ? granule : rr;      // both are powers of two
    auto round_up = [](long long v, long long m) { return (v + m - 1) / m * m; };
    const size_t room = (size_t)cap_kb * 1024 - GEMV_BAR_BYTES - fixed - 64;
    long long rows = unit;
    for (int k = 1;; ++k) {
        const long long ctas = (long long)SM_COUNT * k;
        rows = round_up((n_out + ctas - 1) / ctas, unit);
        if ((size_t)rows * row_bytes <= room || rows == unit) break;
    }
    GemvPlan p;
    p.rr = rr;
    p.threads = threads;
    p.rows_per_cta = (int)rows;
    p.ctas = (int)((n_out + rows - 1) / rows);
    long long rps = round_up(((long long)stage_kb * 1024 + row_bytes - 1) / row_bytes, unit);
    const long long min_rps = round_up((rows + GEMV_MAX_STAGES - 1) / GEMV_MAX_STAGES, unit);
    if (rps < min_rps) rps = min_rps;
    p.rows_per_stage = (int)rps;
    // chain warps come in twos (compute warps must stay paired), at most a quarter of the CTA
    int chain = 2 * (int)((rows + 63) / 64);
    const int max_chain = threads / 32 / 4 >= 2 ? (threads / 32 / 4) & ~1 : 2;
    p.chain_warps = chain < max_chain ? chain : max_chain;
    p.smem_bytes = (int)(GEMV_BAR_BYTES + fixed + (size_t)rows * row_bytes + 64);
    return p;
}

}  // namespace

extern "C" {

int bonsai_p40_quant_activations(const float *x, void *out, int64_t n, bonsai_stream stream) {
    if (n <= 0 || n % 32 != 0) return 1;
    if (!aligned4(x) || !aligned4(out) || n > INT32_MAX) return 1;
    const long long threads = n / 4;
    const int blocks = (int)((threads + 255) / 256);
    // any float pointer is taken, as by the reference; 16-byte aligned ones get 16-byte loads
    if (aligned16(x)) quant_q8_1_kernel<true><<<blocks, 256, 0, as_stream(stream)>>>(x, static_cast<uint32_t *>(out), (int)n, 1);
    else quant_q8_1_kernel<false><<<blocks, 256, 0, as_stream(stream)>>>(x, static_cast<uint32_t *>(out), (int)n, 1);
    return (int)cudaGetLastError();
}

int bonsai_p40_fwht(float *x, const float *signs, int64_t n, bonsai_stream stream) {
    if (n <= 0 || n % FWHT_N != 0) return 1;
    if (!aligned4(x) || (signs && !aligned4(signs)) || n > INT32_MAX) return 1;
    const int warps = (int)(n / FWHT_N);
    if (aligned16(x) && (!signs || aligned16(signs)))
        fwht_quant_kernel<true><<<(warps + 3) / 4, 128, 0, as_stream(stream)>>>(x, signs, x, nullptr, (int)n, 1);
    else
        fwht_quant_kernel<false><<<(warps + 3) / 4, 128, 0, as_stream(stream)>>>(x, signs, x, nullptr, (int)n, 1);
    return (int)cudaGetLastError();
}

int bonsai_b200_fwht_quant(const float *x, const float *signs, void *xq, float *x_rot, int64_t n,
                           bonsai_stream stream) {
    if (n <= 0 || n % FWHT_N != 0 || n > INT32_MAX) return 1;
    if (!aligned4(x) || (signs && !aligned4(signs)) || (x_rot && !aligned4(x_rot)) || !aligned4(xq)) return 1;
    const int warps = (int)(n / FWHT_N);
    if (aligned16(x) && (!signs || aligned16(signs)) && (!x_rot || aligned16(x_rot)))
        fwht_quant_kernel<true><<<(warps + 3) / 4, 128, 0, as_stream(stream)>>>(x, signs, x_rot, static_cast<uint32_t *>(xq),
                                                                                (int)n, 1);
    else
        fwht_quant_kernel<false><<<(warps + 3) / 4, 128, 0, as_stream(stream)>>>(x, signs, x_rot, static_cast<uint32_t *>(xq),
                                                                                 (int)n, 1);
    return (int)cudaGetLastError();
}

int bonsai_b200_quant_batch(const float *X, const float *signs, void *Xq, int64_t n_in, int64_t n_tok, int rotate,
                            bonsai_stream stream) {
    if (n_in <= 0 || n_tok <= 0 || n_in % 32 != 0) return 1;
    if (rotate && n_in % FWHT_N != 0) return 1;
    if (!aligned4(X) || (signs && !aligned4(signs)) || !aligned4(Xq)) return 1;
    if (n_in > INT32_MAX || n_tok > INT32_MAX) return 1;
    const bool vec = aligned16(X) && (!signs || aligned16(signs));
    if (rotate) {
        const long long warps = (n_in / FWHT_N) * n_tok;
        const unsigned blocks = (unsigned)((warps + 3) / 4);
        if (vec) fwht_quant_kernel<true><<<blocks, 128, 0, as_stream(stream)>>>(X, signs, nullptr, static_cast<uint32_t *>(Xq), (int)n_in, (int)n_tok);
        else fwht_quant_kernel<false><<<blocks, 128, 0, as_stream(stream)>>>(X, signs, nullptr, static_cast<uint32_t *>(Xq), (int)n_in, (int)n_tok);
    } else {
        const long long threads = n_in / 4 * n_tok;
        long long blocks = (threads + 255) / 256;
        if (blocks > 8 * SM_COUNT * 4) blocks = 8 * SM_COUNT * 4;
        if (vec) quant_q8_1_kernel<true><<<(unsigned)blocks, 256, 0, as_stream(stream)>>>(X, static_cast<uint32_t *>(Xq), (int)n_in, (int)n_tok);
        else quant_q8_1_kernel<false><<<(unsigned)blocks, 256, 0, as_stream(stream)>>>(X, static_cast<uint32_t *>(Xq), (int)n_in, (int)n_tok);
    }
    return (int)cudaGetLastError();
}

int bonsai_p40_gemv(const void *W, const void *xq, float *y, int64_t n_out, int64_t n_in, bonsai_stream stream) {
    if (n_in <= 0 || n_in % 128 != 0) return 1;
    if (n_out <= 0) return 0;
    if (n_out > INT32_MAX || n_in / 128 > INT32_MAX / 64) return 1;
    const int nblocks = (int)(n_in / 128);
    const bool pdl = g_opt_pdl.load() != 0;
    const int variant = g_opt_gemv_variant.load();
    const bool base_ok = (nblocks % 2 == 0) && aligned16(W) && !(reinterpret_cast<uintptr_t>(xq) & 3u);
    int threads = 0, smem_bytes = 0, rr = 2;
    if (g_opt_gemv_order.load() == 2) {
        MmaGeom mp;
        int grid = 0;
        if (base_ok && plan_mma(n_out, nblocks, 200, mp, smem_bytes, grid)) {
            static SmemOptIn opt;
            cudaError_t err = opt.ensure(gemv_mma_kernel<false>);
            if (err != cudaSuccess) return (int)err;
            return (int)launch(gemv_mma_kernel<false>, dim3((unsigned)grid), dim3(MMA_THREADS), (size_t)smem_bytes,
                               as_stream(stream), pdl, static_cast<const uint8_t *>(W), static_cast<const uint32_t *>(xq), y,
                               mp, static_cast<int32_t *>(nullptr));
        }
    }
    if (g_opt_gemv_order.load() != 1) {
        StreamParams sp;
        if (base_ok && plan_stream(n_out, nblocks, variant, sp, threads, smem_bytes)) {
            static SmemOptIn opt;
            cudaError_t err = opt.ensure(gemv_stream_kernel<false>);
            if (err != cudaSuccess) return (int)err;
            return (int)launch(gemv_stream_kernel<false>, dim3((unsigned)((n_out + sp.rows_per_cta - 1) / sp.rows_per_cta)),
                               dim3(threads), (size_t)smem_bytes, as_stream(stream), pdl,
                               static_cast<const uint8_t *>(W), static_cast<const uint32_t *>(xq), y, sp,
                               static_cast<const float *>(nullptr), static_cast<const float *>(nullptr),
                               static_cast<uint32_t *>(nullptr));
        }
    }
    RingParams rp;
    const bool ring = base_ok && g_opt_gemv_order.load() == 1 &&
                      plan_ring(n_out, nblocks / 2, variant, rp, threads, smem_bytes, rr);
    if (!ring) {
        // odd block count, unaligned weights or a row too long for the rings: plain loads, host order
        return (int)launch(gemv_pq2_generic_kernel, dim3((unsigned)((n_out + 7) / 8)), dim3(256), 0, as_stream(stream),
                           pdl, static_cast<const uint8_t *>(W), static_cast<const uint8_t *>(xq), y, (int)n_out,
                           nblocks);
    }
    const dim3 grid((unsigned)((n_out + rp.rows_per_cta - 1) / rp.rows_per_cta));
    static SmemOptIn opt1, opt2, opt4;
    auto go = [&](auto kernel, SmemOptIn &opt) -> cudaError_t {
        cudaError_t err = opt.ensure(kernel);
        if (err != cudaSuccess) return err;
        return launch(kernel, grid, dim3(threads), (size_t)smem_bytes, as_stream(stream), pdl,
                      static_cast<const uint8_t *>(W), static_cast<const uint32_t *>(xq), y, rp);
    };
    cudaError_t e;
    if (rr == 1) e = go(gemv_ring_kernel<1>, opt1);
    else if (rr == 2) e = go(gemv_ring_kernel<2>, opt2);
    else e = go(gemv_ring_kernel<4>, opt4);
    return (int)e;
}

int bonsai_b200_linear(const void *W, const float *x, const float *signs, float *y, void *xq_scratch, int64_t n_out,
                       int64_t n_in, bonsai_stream stream) {
    if (n_out <= 0 || n_in <= 0 || n_in % FWHT_N != 0 || !xq_scratch) return 1;
    if (n_out > INT32_MAX || !aligned4(x) || (signs && !aligned4(signs)) || !aligned4(xq_scratch)) return 1;
    // one launch when the streaming mat-vec takes the shape: rotation and quantiser run in its prologue
    StreamParams sp;
    int threads = 0, smem_bytes = 0;
    if (g_opt_gemv_order.load() == 0 && g_opt_fuse_linear.load() != 0 && aligned16(W) && aligned16(x) &&
        (!signs || aligned16(signs)) &&
        plan_stream(n_out, (int)(n_in / 128), g_opt_gemv_variant.load(), sp, threads, smem_bytes)) {
        static SmemOptIn opt;
        cudaError_t err = opt.ensure(gemv_stream_kernel<true>);
        if (err != cudaSuccess) return (int)err;
        return (int)launch(gemv_stream_kernel<true>, dim3((unsigned)((n_out + sp.rows_per_cta - 1) / sp.rows_per_cta)),
                           dim3(threads), (size_t)smem_bytes, as_stream(stream), g_opt_pdl.load() != 0,
                           static_cast<const uint8_t *>(W), static_cast<const uint32_t *>(nullptr), y, sp, x, signs,
                           static_cast<uint32_t *>(xq_scratch));
    }
    const int rc = bonsai_b200_fwht_quant(x, signs, xq_scratch, nullptr, n_in, stream);
    if (rc != 0) return rc;
    return bonsai_p40_gemv(W, xq_scratch, y, n_out, n_in, stream);
}

// ---- projection without any allocation: the Q8_1 scratch is part of the library image -----------
// In host code the array's name is only a handle: the device address comes from
// cudaGetSymbolAddress, once per device, with that device current.
static __device__ __align__(256) unsigned char g_linear_static_xq[BONSAI_B200_LINEAR_STATIC_MAX_N_IN / 32 * A_BLOCK_BYTES];

int bonsai_b200_linear_static(const void *W, const float *x, const float *signs, float *y, int64_t n_out, int64_t n_in,
                              bonsai_stream stream) {
    if (n_in > BONSAI_B200_LINEAR_STATIC_MAX_N_IN) return BONSAI_B200_ETOOLARGE;
    if (n_out <= 0 || n_in <= 0 || n_in % FWHT_N != 0) return 1;
    constexpr int MAX_DEVICES = 64;
    static std::atomic<void *> scratch_of_device[MAX_DEVICES];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= MAX_DEVICES) return 1;
    void *scratch = scratch_of_device[dev].load(std::memory_order_acquire);
    if (!scratch) {     // first call on this device: resolve the device address of the array
        e = cudaGetSymbolAddress(&scratch, g_linear_static_xq);
        if (e != cudaSuccess) return (int)e;
        if (!scratch) return (int)cudaErrorInvalidSymbol;
        scratch_of_device[dev].store(scratch, std::memory_order_release);
    }
    const int rc = bonsai_b200_fwht_quant(x, signs, scratch, nullptr, n_in, stream);
    if (rc != 0) return rc;
    return bonsai_p40_gemv(W, scratch, y, n_out, n_in, stream);
}


// ---- a list of projections in one persistent launch ------------------------------------------------
struct bonsai_b200_chain {
    ChainOp *d_ops = nullptr;
    unsigned int *d_counter = nullptr;      // [0] arrivals of ops that others wait for, [1] rotated blocks in the image
    uint8_t *d_image = nullptr;             // activation tables of a spread op, shared through L2
    bool tp = false;                        // several ranks: counters live in the caller's peer-mapped buffer, never reset
    ChainPeers peers{};
    int n_ops = 0, threads = 0, grid = 0, device = 0;
    size_t smem = 0, counter_bytes = 0;
    ChainGeom G{};
};

static int chain_create_impl(const bonsai_b200_op *ops, int64_t n_ops, int tp_rank, int tp_world,
                             const void *const *peer_base, int64_t buffer_bytes, int64_t counter_offset,
                             int64_t wait_limit_us, bonsai_b200_chain **out) {
    if (!ops || !out || n_ops <= 0 || n_ops > (1 << 20)) return 1;
    *out = nullptr;
    const bool tp = tp_world > 1;
    if (tp) {
        if (tp_world > CHAIN_MAX_RANKS || tp_rank < 0 || tp_rank >= tp_world || !peer_base || counter_offset < 0 ||
            (counter_offset & 63) || wait_limit_us < 0)
            return 1;
        // the counter block lies inside the buffer, behind every output; every mapping is 16-byte aligned
        if (buffer_bytes < counter_offset + BONSAI_B200_TP_COUNTER_BYTES) return 1;
        for (int q = 0; q < tp_world; ++q)
            if (!peer_base[q] || !aligned16(peer_base[q])) return 1;
        // every output must lie inside [buffer, counters): the kernel stores it at the same offset of every
        // rank's mapping, so an output outside the buffer would be a store into memory that is not ours
        const char *lo = static_cast<const char *>(peer_base[tp_rank]);
        for (int64_t i = 0; i < n_ops; ++i) {
            const char *y = reinterpret_cast<const char *>(ops[i].y);
            if (!y || ops[i].n_out <= 0 || y < lo || y + ops[i].n_out * 4 > lo + counter_offset) return 1;
        }
    }
    int dev = 0, sms = 0, smem_limit = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
    if ((e = cudaDeviceGetAttribute(&smem_limit, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev)) != cudaSuccess) return (int)e;
    if (sms <= 0) return 1;
    auto round_up = [](long long v, long long m) { return (v + m - 1) / m * m; };
    const long long tile_target = (long long)g_opt_chain_tile_kb.load() * 1024;
    const int threads_opt = g_opt_chain_threads.load();
    const int steps_max = threads_opt == 768 ? 3 : threads_opt == 640 ? 4 : STREAM_STEPS;
    const int seg_max = g_opt_chain_seg.load() < 8 * steps_max ? g_opt_chain_seg.load() : 8 * steps_max;

    std::vector<ChainOp> rec((size_t)n_ops);
    ChainGeom G{};
    long long slot_payload = 0;
    // Table buffers: a third one lets the sequencer prepare two inputs ahead, which pays when most ops bring
    // their own Q8_1 vector; lists whose ops mostly share inputs keep the shared memory for the ring instead.
    int q8_ops = 0, q8_fills = 0;
    for (int64_t i = 0; i < n_ops; ++i) {
        if (ops[i].flags & BONSAI_B200_OP_ROTATE) continue;
        ++q8_ops;
        const bool shared = (ops[i].flags & BONSAI_B200_OP_SAME_INPUT) ||
                            (i > 0 && ops[i - 1].x == ops[i].x && ops[i - 1].n_in == ops[i].n_in &&
                             !(ops[i - 1].flags & BONSAI_B200_OP_ROTATE));
        if (!shared) ++q8_fills;
    }
    const int ntables = q8_ops == 0 ? 1 : (2 * q8_fills > q8_ops ? CHAIN_TABLES : 2);
    int shift = 0, buf = ntables - 1, last_user[CHAIN_TABLES], ready_uses[CHAIN_TABLES];
    for (int b = 0; b < CHAIN_TABLES; ++b) last_user[b] = -1, ready_uses[b] = 0;
    bool any_rotate = false, any_q8 = false, any_spread = false, any_rescale = false;
    unsigned int spread_total = 0;
    const int spread_nb = g_opt_chain_spread_nb.load();
    unsigned int signals = 0;
    for (int64_t i = 0; i < n_ops; ++i) {
        const bonsai_b200_op &o = ops[i];
        ChainOp &r = rec[(size_t)i];
        std::memset(&r, 0, sizeof(r));
        const bool rotate = o.flags & BONSAI_B200_OP_ROTATE, depends = o.flags & BONSAI_B200_OP_DEPENDS;
        bool same = o.flags & BONSAI_B200_OP_SAME_INPUT;
        const uint32_t producer = o.flags & (BONSAI_B200_OP_RMSNORM | BONSAI_B200_OP_SWIGLU | BONSAI_B200_OP_RESCALE);
        // two ops read the same prepared input: same vector, width, signs, kind and producer (with its arguments)
        auto same_input = [](const bonsai_b200_op &a, const bonsai_b200_op &b) {
            const uint32_t kind = BONSAI_B200_OP_ROTATE | BONSAI_B200_OP_RMSNORM | BONSAI_B200_OP_SWIGLU | BONSAI_B200_OP_RESCALE;
            return a.x == b.x && a.n_in == b.n_in && a.signs == b.signs && !((a.flags ^ b.flags) & kind) && a.aux == b.aux &&
                   a.eps == b.eps && a.src_len == b.src_len;
        };
        // the same vector as the op before, and no wait asked for: its tables are reused without being told
        // (nothing may write x during the launch unless a later reader says OP_DEPENDS)
        if (!same && i > 0 && !depends && same_input(ops[i - 1], o)) same = true;
        if ((o.flags & ~63u) || o.reserved) return 1;
        if (!o.W || !o.x || !o.y || o.n_out <= 0 || o.n_out > INT32_MAX || o.n_in <= 0) return 1;
        if (o.n_in % 256 != 0 || (rotate && o.n_in % FWHT_N != 0) || o.n_in / 128 > 1024) return 1;
        if (!aligned16(o.W) || !aligned16(o.x) || (o.signs && !aligned16(o.signs)) || (reinterpret_cast<uintptr_t>(o.y) & 3u))
            return 1;
        if (depends && !rotate) return 1;               // outputs are fp32: a dependent op must quantise
        if (o.signs && !rotate) return 1;
        // producers work on the fp32 vector, one at a time
        if (producer && (!rotate || (producer & (producer - 1)))) return 1;
        if ((producer & (BONSAI_B200_OP_RMSNORM | BONSAI_B200_OP_SWIGLU)) && (!o.aux || !aligned16(o.aux))) return 1;
        if (!(producer & (BONSAI_B200_OP_RMSNORM | BONSAI_B200_OP_SWIGLU)) && o.aux) return 1;
        if ((producer & BONSAI_B200_OP_RMSNORM) && o.n_in / FWHT_N > 7) return 1;      // the whole vector must fit one pass
        if (!(producer & BONSAI_B200_OP_RMSNORM) && o.eps != 0.0f) return 1;
        int src_op = -1;
        if (producer & BONSAI_B200_OP_RESCALE) {
            // x is the output of an earlier op of the list (all of it), whose largest magnitude the kernel records
            if (tp || o.src_len == 0 || o.src_len % 4 != 0 || o.src_len > INT32_MAX) return 1;
            for (int64_t pidx = i - 1; pidx >= 0 && src_op < 0; --pidx)
                if (ops[pidx].y == o.x && ops[pidx].n_out == (int64_t)o.src_len) src_op = (int)pidx;
            if (src_op < 0) return 1;
        } else if (o.src_len != 0) {
            return 1;
        }
        if (same) {
            if (i == 0 || depends) return 1;
            if (!same_input(ops[i - 1], o)) return 1;
        }
        r.W = static_cast<const uint8_t *>(o.W);
        r.x = o.x;
        r.signs = o.signs;
        r.y = o.y;
        r.nb = (int)(o.n_in / 128);
        r.n_out = (int)o.n_out;
        long long ctas = (o.n_out + 3) / 4;
        if (ctas > sms) ctas = sms;
        r.rows_per_cta = (int)round_up((o.n_out + ctas - 1) / ctas, 4);
        const long long used = (o.n_out + r.rows_per_cta - 1) / r.rows_per_cta;
        const long long row_bytes = (long long)r.nb * W_BLOCK_BYTES;
        long long tr = (tile_target / row_bytes) & ~3ll;
        if (tr < 4) tr = 4;
        if (tr > r.rows_per_cta) tr = r.rows_per_cta;
        r.tr = (int)tr;
        r.nseg = (r.nb + seg_max - 1) / seg_max;
        r.seg_blocks = (int)round_up((r.nb + r.nseg - 1) / r.nseg, 8);
        if (r.seg_blocks > seg_max) r.seg_blocks = seg_max;
        r.nseg = (r.nb + r.seg_blocks - 1) / r.seg_blocks;
        r.tpt = (r.tr / 4) * r.nseg;
        r.magic_tpt = magic_u32((uint32_t)r.tpt);
        r.magic_nseg = magic_u32((uint32_t)r.nseg);
        r.cta_shift = shift;
        shift = (int)((shift + used) % sms);            // the next op starts on the CTA after this one's last
        r.flags = (rotate ? CHAIN_ROTATE : 0) | (depends ? CHAIN_DEPENDS : 0) | (same ? CHAIN_SAME_INPUT : 0) |
                  ((producer & BONSAI_B200_OP_RMSNORM) ? CHAIN_RMSNORM : 0) | ((producer & BONSAI_B200_OP_SWIGLU) ? CHAIN_SWIGLU : 0) |
                  ((producer & BONSAI_B200_OP_RESCALE) ? CHAIN_RESCALE : 0);
        r.aux = o.aux;
        r.eps = o.eps;
        r.src_len = (int)o.src_len;
        r.src_op = src_op;
        if (src_op >= 0) {
            rec[(size_t)src_op].flags |= CHAIN_MAXSRC;
            any_rescale = true;
        }
        if (depends) rec[(size_t)i - 1].flags |= CHAIN_SIGNAL;     // i > 0: op 0 may not depend
        if (depends && i == 0) return 1;
        if (!same) buf = (buf + 1) % ntables;
        r.buf = buf;
        r.prev_user = same ? -1 : last_user[buf];
        last_user[buf] = (int)i;
        if (!same && !rotate) r.ready_parity = ready_uses[buf]++ & 1;
        if (rotate) any_rotate = true; else any_q8 = true;
        // (an RMSNorm producer needs the whole vector in every CTA for its sum of squares: such an op rotates for itself)
        if (rotate && depends && !same && !(r.flags & CHAIN_RMSNORM) && spread_nb > 0 && r.nb >= spread_nb && r.nb / 8 <= sms) {
            r.flags |= CHAIN_SPREAD;
            spread_total += (unsigned)(r.nb / 8);
            r.spread_blocks = spread_total;
            any_spread = true;
        }
        if (r.nb > G.nb_max) G.nb_max = r.nb;
        if (r.nseg > 1) {        // only rows in several segments are joined through shared memory
            if (r.rows_per_cta * r.nseg > G.partial_floats) G.partial_floats = r.rows_per_cta * r.nseg;
            if (r.rows_per_cta / 4 > G.quad_ints) G.quad_ints = r.rows_per_cta / 4;
        }
        if (tr * row_bytes > slot_payload) slot_payload = tr * row_bytes;
    }
    if (tp) rec[(size_t)n_ops - 1].flags |= CHAIN_SIGNAL;       // the closing arrival of a run
    // arrivals a dependent op must see: one per CTA for every signalling op before it
    for (int64_t i = 0; i < n_ops; ++i) {
        rec[(size_t)i].arrivals_needed = signals;
        if (rec[(size_t)i].flags & CHAIN_SIGNAL) ++signals;
    }
    G.stage_blocks = any_q8 ? G.nb_max : 0;
    G.ntables = ntables;
    G.rot_blocks = any_rotate ? (G.nb_max / 8 < 7 ? G.nb_max / 8 : 7) : 0;
    if (tp)
        for (const auto &r : rec)
            if (r.rows_per_cta > G.rows_stage) G.rows_stage = r.rows_per_cta;
    G.partial_floats = (int)round_up(G.partial_floats, 4);
    G.quad_ints = (int)round_up(G.quad_ints, 4);
    G.slot_bytes = (int)round_up(slot_payload + 16, 128);
    const size_t fixed = chain_fixed_bytes(G);
    if (fixed + 3 * (size_t)G.slot_bytes > (size_t)smem_limit) return 1;
    long long nslot = ((long long)smem_limit - (long long)fixed) / G.slot_bytes;
    if (nslot > CHAIN_MAX_SLOTS) nslot = CHAIN_MAX_SLOTS;
    G.nslot = (int)nslot;
    G.magic_nslot = magic_u32((uint32_t)G.nslot);

    bonsai_b200_chain *c = new (std::nothrow) bonsai_b200_chain;
    if (!c) return (int)cudaErrorMemoryAllocation;
    c->n_ops = (int)n_ops;
    c->threads = threads_opt;
    c->tp = tp;
    if (tp) {
        if (threads_opt != 512) { delete c; return 1; }             // the several-rank kernel is built for 512 threads
        c->peers.rank = tp_rank;
        c->peers.world = tp_world;
        c->peers.arrivals_per_run = signals;
        c->peers.spread_per_run = spread_total;
        c->peers.wait_limit_ns = (unsigned long long)(wait_limit_us > 0 ? wait_limit_us : 1000000) * 1000ull;
        for (int q = 0; q < tp_world; ++q) {
            c->peers.y_delta[q] = (long long)(static_cast<const char *>(peer_base[q]) - static_cast<const char *>(peer_base[tp_rank]));
            c->peers.counter[q] = reinterpret_cast<unsigned int *>(const_cast<char *>(static_cast<const char *>(peer_base[q])) + counter_offset);
        }
    }
    c->grid = sms;
    c->device = dev;
    c->G = G;
    c->smem = fixed + (size_t)G.nslot * G.slot_bytes;
    // the launch is cooperative: every CTA must be resident at once
    int per_sm = 0;
    auto prepare = [&](auto kernel) {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_limit);
        if (err == cudaSuccess) err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, c->threads, c->smem);
        return err;
    };
    if (tp) e = prepare(gemv_chain_kernel<512, 5, true>);
    else if (c->threads == 768) e = prepare(gemv_chain_kernel<768, 3, false>);
    else if (c->threads == 640) e = prepare(gemv_chain_kernel<640, 4, false>);
    else if (c->threads == 512) e = prepare(gemv_chain_kernel<512, 5, false>);
    else e = cudaErrorInvalidValue;
    if (e == cudaSuccess && per_sm < 1) e = cudaErrorLaunchOutOfResources;
    if (e == cudaSuccess) e = cudaMalloc(&c->d_ops, sizeof(ChainOp) * (size_t)n_ops);
    if (e == cudaSuccess && tp) c->d_counter = c->peers.counter[tp_rank];
    c->counter_bytes = 256 + (any_rescale ? 4 * (size_t)n_ops : 0);        // counters, then the largest |y| of every op
    if (e == cudaSuccess && !tp) e = cudaMalloc(&c->d_counter, c->counter_bytes);
    if (e == cudaSuccess && any_spread) e = cudaMalloc(&c->d_image, (size_t)G.nb_max * 176);
    if (e == cudaSuccess) e = cudaMemcpy(c->d_ops, rec.data(), sizeof(ChainOp) * (size_t)n_ops, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        bonsai_b200_chain_destroy(c);
        return (int)e;
    }
    *out = c;
    return 0;
}

int bonsai_b200_chain_create(const bonsai_b200_op *ops, int64_t n_ops, bonsai_b200_chain **out) {
    return chain_create_impl(ops, n_ops, 0, 1, nullptr, 0, 0, 0, out);
}

int bonsai_b200_chain_create_tp(const bonsai_b200_op *ops, int64_t n_ops, int rank, int world, const void *const *peer_base,
                                int64_t buffer_bytes, int64_t counter_offset, int64_t wait_limit_us,
                                bonsai_b200_chain **out) {
    if (world < 2) return 1;
    return chain_create_impl(ops, n_ops, rank, world, peer_base, buffer_bytes, counter_offset, wait_limit_us, out);
}

int bonsai_b200_chain_run(bonsai_b200_chain *c, bonsai_stream stream) {
    if (!c || !c->d_ops) return 1;
    cudaStream_t st = as_stream(stream);
    cudaError_t e = cudaSuccess;
    if (!c->tp) e = cudaMemsetAsync(c->d_counter, 0, c->counter_bytes > 256 ? c->counter_bytes : 2 * sizeof(unsigned int), st);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)c->grid);
    cfg.blockDim = dim3((unsigned)c->threads);
    cfg.dynamicSmemBytes = c->smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const ChainOp *ops = c->d_ops;
    auto go = [&](auto kernel) {
        return cudaLaunchKernelEx(&cfg, kernel, ops, c->n_ops, c->G, c->d_counter, c->d_image, c->peers);
    };
    if (c->tp) e = go(gemv_chain_kernel<512, 5, true>);
    else if (c->threads == 768) e = go(gemv_chain_kernel<768, 3, false>);
    else if (c->threads == 640) e = go(gemv_chain_kernel<640, 4, false>);
    else e = go(gemv_chain_kernel<512, 5, false>);
    return (int)e;
}

int bonsai_b200_chain_destroy(bonsai_b200_chain *c) {
    if (!c) return 0;
    cudaError_t e1 = c->d_ops ? cudaFree(c->d_ops) : cudaSuccess;
    cudaError_t e2 = (c->d_counter && !c->tp) ? cudaFree(c->d_counter) : cudaSuccess;
    if (c->d_image) cudaFree(c->d_image);
    delete c;
    return (int)(e1 != cudaSuccess ? e1 : e2);
}

int bonsai_b200_chain_info(const bonsai_b200_chain *c, int64_t out[4]) {
    if (!c || !out) return 1;
    out[0] = c->threads;
    out[1] = c->G.nslot;
    out[2] = c->G.slot_bytes;
    out[3] = c->grid;
    return 0;
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

int bonsai_b200_gemv_dump(const void *W, const void *xq, float *y, int32_t *sums, int64_t n_out, int64_t n_in,
                          bonsai_stream stream) {
    if (n_in <= 0 || n_in % 128 != 0 || n_out <= 0 || n_out > INT32_MAX || !sums) return 1;
    const int nblocks = (int)(n_in / 128);
    MmaGeom mp;
    int smem_bytes = 0, grid = 0;
    if (!aligned16(W) || !aligned4(xq) || !plan_mma(n_out, nblocks, 200, mp, smem_bytes, grid)) return 1;
    static SmemOptIn opt;
    cudaError_t err = opt.ensure(gemv_mma_kernel<true>);
    if (err != cudaSuccess) return (int)err;
    return (int)launch(gemv_mma_kernel<true>, dim3((unsigned)grid), dim3(MMA_THREADS), (size_t)smem_bytes, as_stream(stream),
                       false, static_cast<const uint8_t *>(W), static_cast<const uint32_t *>(xq), y, mp, sums);
}

// 2-D tensor map: dims {d0 (fastest), d1}, row stride in bytes, box {b0, b1}.  The encoder is a driver entry point; it is
// looked up through the runtime so that the library links against nothing but cudart.  false: not available (the
// caller takes a form that needs no map).
static bool tensor_map_2d(CUtensorMap *map, CUtensorMapDataType type, const void *base, uint64_t d0, uint64_t d1,
                          uint64_t stride_bytes, uint32_t b0, uint32_t b1, CUtensorMapSwizzle swizzle) {
    using Encode = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static Encode encode = [] {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            fn = nullptr;
        return reinterpret_cast<Encode>(fn);
    }();
    if (!encode) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)d0, (cuuint64_t)d1};
    const cuuint64_t strides[1] = {(cuuint64_t)stride_bytes};
    const cuuint32_t box[2] = {b0, b1};
    const cuuint32_t estr[2] = {1u, 1u};
    return encode(map, type, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
// The two fp16 planes of the split activations, [2][n_tok][n_in]: box = 64 values x one tile of tokens x both planes, landing with
// the 128-byte swizzle the MMA reads; tokens past the end arrive as zeros.
static bool tensor_map_planes(CUtensorMap *map, const void *planes, uint64_t n_in, uint64_t n_tok, uint32_t tile_tokens) {
    using Encode = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess || !fn)
        return false;
    const cuuint64_t dims[3] = {n_in, n_tok, 2};
    const cuuint64_t strides[2] = {n_in * 2, n_tok * n_in * 2};
    const cuuint32_t box[3] = {64u, (cuuint32_t)tile_tokens, 2u};
    const cuuint32_t estr[3] = {1u, 1u, 1u};
    return reinterpret_cast<Encode>(fn)(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void *>(planes), dims, strides, box, estr,
                                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
// A PQ2_0 matrix seen as [n_out][row_bytes / 4] 32-bit words, box = 68 words (8 blocks) x 128 rows.
static bool encode_w_map(CUtensorMap *map, const void *W, int64_t n_out, int64_t row_bytes) {
    return tensor_map_2d(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, W, (uint64_t)(row_bytes / 4), (uint64_t)n_out, (uint64_t)row_bytes,
                         68u, (uint32_t)TC_M, CU_TENSOR_MAP_SWIZZLE_NONE);
}

// Scratch of the fp16 tensor-core mat-mul (the activations as two fp16 planes + the per-token scales): one buffer per
// (device, stream), grown with cudaMalloc when a call needs more -- never while the stream is being captured (then,
// and when 16 buffers exist already, the caller takes the integer kernel, which needs no scratch).
struct GemmScratch { int dev; cudaStream_t st; void *ptr; size_t bytes; };
static std::mutex g_scratch_mu;
static std::vector<GemmScratch> g_scratch;
static void *gemm_scratch(size_t bytes, cudaStream_t st) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    std::lock_guard<std::mutex> lock(g_scratch_mu);
    GemmScratch *e = nullptr;
    for (auto &g : g_scratch)
        if (g.dev == dev && g.st == st) e = &g;
    if (e && e->bytes >= bytes) return e->ptr;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) return nullptr;
    if (!e) {
        if (g_scratch.size() >= 16) return nullptr;
        g_scratch.push_back(GemmScratch{dev, st, nullptr, 0});
        e = &g_scratch.back();
    }
    if (e->ptr) cudaFree(e->ptr);               // synchronises the device: nothing in flight reads the old buffer
    e->ptr = nullptr;
    e->bytes = 0;
    void *pnew = nullptr;
    if (cudaMalloc(&pnew, bytes) != cudaSuccess) { (void)cudaGetLastError(); return nullptr; }
    e->ptr = pnew;
    e->bytes = bytes;
    return pnew;
}

static std::atomic<unsigned int> g_gemm_epoch{0};       // launch number of the tensor-core mat-muls (tags partial-tile flags)

static void fill_tc_params(TcParams &P, int64_t n_out, int64_t n_in, int64_t n_tok, int tile_m, int tile_n) {
    P.n_out = (int)n_out;
    P.nblocks = (int)(n_in / 128);
    P.n_tok = (int)n_tok;
    P.tiles_tok = (int)((n_tok + tile_n - 1) / tile_n);
    P.n_tiles = (int)(((n_out + tile_m - 1) / tile_m) * P.tiles_tok);
    P.total_it = (long long)P.n_tiles * P.nblocks;
}

// The fp16 tensor-core mat-mul (gemm_tc16.cuh).  -1: not taken (shape, alignment, no scratch, no tensor-map encoder).
extern "C++" {
template <int TN>
static int launch_gemm_tc16_n(const void *W, const void *Xq, float *Y, int64_t n_out, int64_t n_in, int64_t n_tok, cudaStream_t st) {
    constexpr int T16_N = TN;
    const int64_t nblocks = n_in / 128;
    if (nblocks % 8 != 0 || !aligned16(W) || !aligned4(Xq) || n_tok > (1 << 28)) return -1;
    const long long tiles = (long long)((n_out + T16_M - 1) / T16_M) * ((n_tok + T16_N - 1) / T16_N);
    if (tiles > INT32_MAX) return -1;
    const size_t plane_bytes = (size_t)n_tok * (size_t)n_in * sizeof(__half);
    const size_t bytes = 2 * plane_bytes + 2 * (size_t)n_tok * sizeof(float);
    uint8_t *ws = static_cast<uint8_t *>(gemm_scratch(bytes, st));
    if (!ws) return -1;
    __half *planes = reinterpret_cast<__half *>(ws);
    float *scale = reinterpret_cast<float *>(ws + 2 * plane_bytes);
    alignas(64) Tc16Maps maps;
    std::memset(&maps, 0, sizeof(maps));
    if (!encode_w_map(&maps.w, W, n_out, nblocks * W_BLOCK_BYTES)) return -1;
    if (!tensor_map_planes(&maps.x, planes, (uint64_t)n_in, (uint64_t)n_tok, (uint32_t)TN)) return -1;
    TcParams P{};
    fill_tc_params(P, n_out, n_in, n_tok, T16_M, T16_N);
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return (int)e;
    if (sms > TC_MAX_CTAS - 1) sms = TC_MAX_CTAS - 1;
    // Tiles for at most half of the SMs (a short token batch over few rows): up to four CTAs share a tile's blocks, at least 16
    // blocks each.  A CTA whose whole range lies inside one tile is both a "late" and an "early" part: it waits for
    // the part behind it, adds, stores, and raises its own flag -- the sums reach the tile's first CTA along the chain.
    int grid = (int)(tiles < sms ? tiles : sms);
    if (2 * tiles <= sms) {
        long long g = P.total_it / 16;
        if (g > 4 * tiles) g = 4 * tiles;
        if (g > sms) g = sms;
        if (g > grid) grid = (int)g;
    }
    P.stream_k = (tiles % grid != 0 && (grid > tiles || P.total_it / grid >= P.nblocks)) ? 1 : 0;
    P.epoch = g_gemm_epoch.fetch_add(1) + 1u;
    const int n_chunks = (int)(n_in / 32);
    const uint32_t *x32 = static_cast<const uint32_t *>(Xq);
    unsigned int *maxd = reinterpret_cast<unsigned int *>(scale + n_tok);
    e = cudaMemsetAsync(maxd, 0, (size_t)n_tok * sizeof(unsigned int), st);
    if (e != cudaSuccess) return (int)e;
    const int slices = n_chunks >= 64 ? 16 : 1;
    tc16_tokmax_kernel<<<dim3((unsigned)((n_tok + 31) / 32), (unsigned)slices), 256, 0, st>>>(x32, n_chunks, (int)n_tok, maxd);
    const long long warps = ((n_tok + 3) / 4) * (long long)((n_chunks + 7) / 8);
    tc16_split_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, st>>>(x32, n_chunks, (int)n_tok, maxd, scale, planes);
    static SmemOptIn opt;
    e = opt.ensure(gemm_tc16_kernel<TN>);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(T16C<TN>::THREADS);
    cfg.dynamicSmemBytes = T16C<TN>::SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, gemm_tc16_kernel<TN>, Y, P, (const float *)scale, maps);
}
}  // extern "C++"
// Tiles of 128 tokens from 96 tokens on (the code expansion, the kernel's busiest part, is paid once per tile), of 64 below.
static int launch_gemm_tc16(const void *W, const void *Xq, float *Y, int64_t n_out, int64_t n_in, int64_t n_tok, cudaStream_t st) {
    const int tile = g_opt_gemm_tile.load();
    if (tile == 64 || (tile != 128 && n_tok < 96)) return launch_gemm_tc16_n<64>(W, Xq, Y, n_out, n_in, n_tok, st);
    return launch_gemm_tc16_n<128>(W, Xq, Y, n_out, n_in, n_tok, st);
}

// The tensor-core mat-mul: one CTA per SM walks its share of the (tile, weight block) iterations.
static int launch_gemm_tc(const void *W, const void *Xq, float *Y, int64_t n_out, int64_t n_in, int64_t n_tok,
                          int32_t *dump, cudaStream_t st) {
    TcParams P{};
    const long long tiles = (long long)((n_out + TC_M - 1) / TC_M) * ((n_tok + TC_N - 1) / TC_N);
    if (tiles > INT32_MAX) return 1;
    fill_tc_params(P, n_out, n_in, n_tok, TC_M, TC_N);
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return (int)e;
    if (sms > TC_MAX_CTAS - 1) sms = TC_MAX_CTAS - 1;
    const int grid = (int)(tiles < sms ? tiles : sms);
    // contiguous ranges when they are at least one tile long (then a tile is cut at most once); whole tiles otherwise
    P.stream_k = (tiles % grid != 0 && P.total_it / grid >= P.nblocks) ? 1 : 0;
    P.epoch = g_gemm_epoch.fetch_add(1) + 1u;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = TC_SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;        // a CTA may wait for its neighbour's partial tile: all must be resident
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const uint8_t *w8 = static_cast<const uint8_t *>(W);
    const uint32_t *x32 = static_cast<const uint32_t *>(Xq);
    // bulk-copy staging of the raw bytes needs 16-byte multiples everywhere; other shapes load from global memory
    alignas(64) CUtensorMap wmap;
    std::memset(&wmap, 0, sizeof(wmap));
    const bool tma = P.nblocks % 8 == 0 && n_tok % 4 == 0 && aligned16(W) && aligned16(Xq) &&
                     encode_w_map(&wmap, W, n_out, (int64_t)P.nblocks * W_BLOCK_BYTES);
    static SmemOptIn opt[4];
    auto go = [&](auto kernel, SmemOptIn &o, int smem) -> int {
        cudaError_t err = o.ensure(kernel);
        if (err != cudaSuccess) return (int)err;
        cfg.dynamicSmemBytes = (size_t)smem;
        return (int)cudaLaunchKernelEx(&cfg, kernel, w8, x32, Y, P, dump, wmap);
    };
    if (dump) return tma ? go(gemm_tc_kernel<true, true>, opt[0], TC_SMEM_BYTES_TMA) : go(gemm_tc_kernel<true, false>, opt[1], TC_SMEM_BYTES);
    return tma ? go(gemm_tc_kernel<false, true>, opt[2], TC_SMEM_BYTES_TMA) : go(gemm_tc_kernel<false, false>, opt[3], TC_SMEM_BYTES);
}

// The streaming small-batch mat-mul (gemv_mma.cuh).  -1: shape not taken (more than 8 tokens, odd block count, rows of
// more than 48 blocks that are not a multiple of 8 blocks, unaligned W, no tensor-map encoder in the driver).
static int launch_gemm_small(const void *W, const void *Xq, float *Y, int64_t n_out, int64_t n_in, int64_t n_tok,
                             int32_t *dump, cudaStream_t st) {
    if (n_tok < 1 || n_tok > 16 || (dump && n_tok > 8) || !aligned16(W) || n_out > INT32_MAX - 16) return -1;
    MmabGeom mp;
    int smem_bytes = 0, grid = 0;
    const int nb = (int)(n_in / 128);
    if (!plan_mmab(n_out, nb, (int)n_tok, 224, mp, smem_bytes, grid)) return -1;
    CUtensorMap wmap;
    std::memset(&wmap, 0, sizeof(wmap));
    if (mp.tiled && !tensor_map_2d(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, W, (uint64_t)nb * W_BLOCK_BYTES / 4, (uint64_t)n_out,
                                   (uint64_t)nb * W_BLOCK_BYTES, (uint32_t)(mp.stride / 4), 16u, CU_TENSOR_MAP_SWIZZLE_NONE))
        return -1;
    static SmemOptIn opt, opt2, opt_dump;
    const bool pdl = g_opt_pdl.load() != 0;
    if (mp.ntg == 2) {
        cudaError_t err = opt2.ensure(gemm_mma_kernel<false, 2, 1>);
        if (err != cudaSuccess) return (int)err;
        return (int)launch(gemm_mma_kernel<false, 2, 1>, dim3((unsigned)grid), dim3(MMAB_THREADS), (size_t)smem_bytes, st, pdl,
                           static_cast<const uint8_t *>(W), static_cast<const uint32_t *>(Xq), Y, mp, (int)n_tok, dump, wmap);
    }
    auto go = [&](auto kernel, SmemOptIn &o, bool with_pdl) -> int {
        cudaError_t err = o.ensure(kernel);
        if (err != cudaSuccess) return (int)err;
        return (int)launch(kernel, dim3((unsigned)grid), dim3(MMAB_THREADS), (size_t)smem_bytes, st, with_pdl,
                           static_cast<const uint8_t *>(W), static_cast<const uint32_t *>(Xq), Y, mp, (int)n_tok, dump, wmap);
    };
    static SmemOptIn opt_r2, opt_dump_r2;
    if (dump) return mp.nrg == 2 ? go(gemm_mma_kernel<true, 1, 2>, opt_dump_r2, false) : go(gemm_mma_kernel<true, 1, 1>, opt_dump, false);
    return mp.nrg == 2 ? go(gemm_mma_kernel<false, 1, 2>, opt_r2, pdl) : go(gemm_mma_kernel<false, 1, 1>, opt, pdl);
}

int bonsai_p40_gemm(const void *W, const void *Xq, float *Y, int64_t n_out, int64_t n_in, int64_t n_tok,
                    bonsai_stream stream) {
    if (n_in <= 0 || n_in % 128 != 0) return 1;
    if (n_out <= 0 || n_tok <= 0) return 0;
    if (n_out > INT32_MAX || n_tok > INT32_MAX || !aligned4(Xq)) return 1;
    const int path = g_opt_gemm_path.load();
    // One token is the mat-vec (chunk-major Xq of one token is the plain Q8_1 vector, Y[n_out][1] the output vector):
    // 8 us against 140 us of the integer SIMT kernel on 5120 -> 17408; same bits and options as bonsai_p40_gemv.
    if (n_tok == 1 && path < 0) return bonsai_p40_gemv(W, Xq, Y, n_out, n_in, stream);
    // From 9 tokens on the tensor cores win even with a 64-token tile mostly empty (5120 -> 17408 at 16 tokens:
    // 40 us against 140 us of the integer SIMT kernel); 2 .. 8 tokens stream the weights once through mma.sync.
    // 9 .. 16 tokens: the streaming kernel with two token groups per code extraction is ahead of the tensor cores
    // (31 against 40 us at 24 MB, 297 against 312 us at 338 MB); it needs rows of a multiple of 8 blocks.
    const bool small16 = n_tok >= 9 && n_tok <= 16 && (n_in / 128) % 8 == 0;
    if (path == 2 || (path < 0 && n_tok >= 2 && (n_tok <= 8 || small16))) {     // a handful of tokens: weights streamed once for all of them
        const int rc = launch_gemm_small(W, Xq, Y, n_out, n_in, n_tok, nullptr, as_stream(stream));
        if (rc >= 0) return rc;                                       // -1: the shape does not fit, a kernel below takes it
    }
    if (path == 1 || path == 3 || (path < 0 && n_tok >= 9)) {
        if (path != 3) {                                              // the fp16 form first; -1: it does not take the call
            const int rc = launch_gemm_tc16(W, Xq, Y, n_out, n_in, n_tok, as_stream(stream));
            if (rc >= 0) return rc;
        }
        return launch_gemm_tc(W, Xq, Y, n_out, n_in, n_tok, nullptr, as_stream(stream));
    }
    const dim3 grid((unsigned)((n_out + GS_ROWS - 1) / GS_ROWS), (unsigned)((n_tok + GS_TOKS - 1) / GS_TOKS));
    if (grid.y > 65535) return 1;
    gemm_simt_kernel<<<grid, 256, 0, as_stream(stream)>>>(static_cast<const uint8_t *>(W),
                                                          static_cast<const uint32_t *>(Xq), Y, (int)n_out,
                                                          (int)(n_in / 128), (int)n_tok);
    return (int)cudaGetLastError();
}

int bonsai_b200_gemm_release(void) {
    std::lock_guard<std::mutex> lock(g_scratch_mu);
    int dev = 0;
    const bool have = cudaGetDevice(&dev) == cudaSuccess;
    for (auto &g : g_scratch) {
        if (!g.ptr) continue;
        if (have) (void)cudaSetDevice(g.dev);
        (void)cudaFree(g.ptr);
    }
    g_scratch.clear();
    if (have) (void)cudaSetDevice(dev);
    return 0;
}

int bonsai_b200_gemm_reserve(int64_t n_in, int64_t n_tok, bonsai_stream stream) {
    if (n_in <= 0 || n_in % 128 != 0 || n_tok <= 0 || n_tok > (1 << 28)) return 1;
    const size_t bytes = 2 * (size_t)n_tok * (size_t)n_in * sizeof(__half) + 2 * (size_t)n_tok * sizeof(float);
    return gemm_scratch(bytes, as_stream(stream)) ? 0 : (int)cudaErrorMemoryAllocation;
}

int bonsai_b200_gemm_dump(const void *W, const void *Xq, float *Y, int32_t *sums, int64_t n_out, int64_t n_in,
                          int64_t n_tok, bonsai_stream stream) {
    if (n_in <= 0 || n_in % 128 != 0 || n_out <= 0 || n_tok <= 0 || !sums) return 1;
    if (n_out > INT32_MAX || n_tok > INT32_MAX || !aligned4(Xq)) return 1;
    if (n_tok <= 8) {           // the streaming small-batch kernel, when it takes the shape
        const int rc = launch_gemm_small(W, Xq, Y, n_out, n_in, n_tok, sums, as_stream(stream));
        if (rc >= 0) return rc;
    }
    return launch_gemm_tc(W, Xq, Y, n_out, n_in, n_tok, sums, as_stream(stream));
}

int bonsai_p40_repack(const void *src, void *dst, int64_t n_out, int64_t n_in, bonsai_stream stream) {
    if (n_in % 128 != 0 || n_out <= 0) return 1;
    const int64_t nb = n_in / 128;
    if (nb <= 0 || nb % 8 != 0 || nb > INT32_MAX / 64) return 1;
    if (!aligned16(dst) || (reinterpret_cast<uintptr_t>(src) & 1u)) return 1;
    const int64_t row_bytes = nb * W_BLOCK_BYTES;
    if (aligned16(src) && row_bytes <= RPK_SMEM_BYTES) {
        const int rows_per_pass = (int)(RPK_SMEM_BYTES / row_bytes);
        long long passes = (n_out + rows_per_pass - 1) / rows_per_pass;
        if (passes > 6 * SM_COUNT) passes = 6 * SM_COUNT;
        repack_staged_kernel<<<(unsigned)passes, 256, RPK_SMEM_BYTES, as_stream(stream)>>>(
            static_cast<const uint8_t *>(src), static_cast<uint8_t *>(dst), n_out, (int)nb, rows_per_pass);
        return (int)cudaGetLastError();
    }
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
    if (GEMV_BAR_BYTES + act_bytes + 4 * row_bytes + 64 > (size_t)111 * 1024) return 1;
    if (!aligned16(W) || !aligned4(x)) return 1;        // dst of bonsai_p40_repack is 16-byte aligned; x is any float pointer
    const bool pdl = g_opt_pdl.load() != 0;
    GemvPlan p = plan_rows(n_out, row_bytes, act_bytes, 1, g_opt_gemv_variant.load());
    if (p.threads > 256) p.threads = 256;
    const dim3 grid((unsigned)p.ctas);
    static SmemOptIn opt[12];
    auto go = [&](auto kernel, SmemOptIn &o) -> cudaError_t {
        cudaError_t err = o.ensure(kernel);
        if (err != cudaSuccess) return err;
        return launch(kernel, grid, dim3(p.threads), (size_t)p.smem_bytes, as_stream(stream), pdl,
                      static_cast<const uint8_t *>(W), x, y, (int)n_out, nb, p.rows_per_cta, p.rows_per_stage);
    };
    // gemv_order 1: the terms of a row added in unit order by one lane (the bits of repack_row_dot); otherwise by a warp
    const bool tree = g_opt_gemv_order.load() != 1;
    const bool vec = aligned16(x);
    // the streaming kernel (ring of tiles, quantiser in the prologue) when it takes the shape: the default
    {
        StreamParams sp;
        int threads = 0, smem_bytes = 0;
        if (tree && vec && n_in % FWHT_N == 0 && plan_stream(n_out, nb, g_opt_gemv_variant.load(), sp, threads, smem_bytes)) {
            static SmemOptIn sopt;
            cudaError_t err = sopt.ensure(gemv_stream_kernel<true, true>);
            if (err != cudaSuccess) return (int)err;
            return (int)launch(gemv_stream_kernel<true, true>, dim3((unsigned)((n_out + sp.rows_per_cta - 1) / sp.rows_per_cta)),
                               dim3(threads), (size_t)smem_bytes, as_stream(stream), pdl, static_cast<const uint8_t *>(W),
                               static_cast<const uint32_t *>(nullptr), y, sp, x, static_cast<const float *>(nullptr),
                               static_cast<uint32_t *>(nullptr));
        }
    }
    auto pick = [&](auto t, auto v, int base) -> cudaError_t {
        constexpr bool T = decltype(t)::value, V = decltype(v)::value;
        if (p.rr == 1) return go(gemv_repack_kernel<1, V, T>, opt[base]);
        if (p.rr == 2) return go(gemv_repack_kernel<2, V, T>, opt[base + 1]);
        return go(gemv_repack_kernel<4, V, T>, opt[base + 2]);
    };
    cudaError_t e;
    if (tree) e = vec ? pick(std::true_type{}, std::true_type{}, 0) : pick(std::true_type{}, std::false_type{}, 3);
    else e = vec ? pick(std::false_type{}, std::true_type{}, 6) : pick(std::false_type{}, std::false_type{}, 9);
    return (int)e;
}

int bonsai_b200_ptq1_pack(const void *src, void *dst, int64_t n_blocks, uint64_t *code3_count, bonsai_stream stream) {
    if (n_blocks <= 0) return n_blocks == 0 ? 0 : 1;
    if ((reinterpret_cast<uintptr_t>(src) & 1u) || (reinterpret_cast<uintptr_t>(dst) & 1u) || !code3_count ||
        (reinterpret_cast<uintptr_t>(code3_count) & 7u))
        return 1;
    long long blocks = (n_blocks + 255) / 256;
    if (blocks > 16 * SM_COUNT) blocks = 16 * SM_COUNT;
    ptq1_pack_kernel<<<(unsigned)blocks, 256, 0, as_stream(stream)>>>(static_cast<const uint8_t *>(src), static_cast<uint8_t *>(dst),
                                                                      n_blocks, reinterpret_cast<unsigned long long *>(code3_count));
    return (int)cudaGetLastError();
}

int bonsai_b200_ptq1_unpack(const void *src, void *dst, int64_t n_blocks, bonsai_stream stream) {
    if (n_blocks <= 0) return n_blocks == 0 ? 0 : 1;
    if ((reinterpret_cast<uintptr_t>(src) & 1u) || (reinterpret_cast<uintptr_t>(dst) & 1u)) return 1;
    long long blocks = (n_blocks + 255) / 256;
    if (blocks > 16 * SM_COUNT) blocks = 16 * SM_COUNT;
    ptq1_unpack_kernel<<<(unsigned)blocks, 256, 0, as_stream(stream)>>>(static_cast<const uint8_t *>(src), static_cast<uint8_t *>(dst),
                                                                        n_blocks);
    return (int)cudaGetLastError();
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

int bonsai_b200_stream_probe(const void *buf, int64_t bytes, int mode, void *sink, bonsai_stream stream) {
    if (bytes <= 0 || !aligned16(buf) || !sink) return 1;
    if (mode == 0) {
        probe_ldg_kernel<<<SM_COUNT * 8, 256, 0, as_stream(stream)>>>(static_cast<const uint4 *>(buf), bytes / 16,
                                                                     static_cast<unsigned *>(sink));
    } else if (mode == 1) {
        const int slot = 16384, stages = 6;
        if (bytes < slot) return 1;
        static SmemOptIn opt;
        cudaError_t e = opt.ensure(probe_bulk_kernel);
        if (e != cudaSuccess) return (int)e;
        probe_bulk_kernel<<<SM_COUNT * 2, 32, 128 + slot * stages, as_stream(stream)>>>(
            static_cast<const uint8_t *>(buf), bytes, slot, stages, static_cast<unsigned *>(sink));
    } else {
        return 1;
    }
    return (int)cudaGetLastError();
}

int bonsai_b200_set_option(const char *key, int64_t value) {
    if (!key) return 1;
    if (!std::strcmp(key, "pdl")) { g_opt_pdl.store(value != 0); return 0; }
    if (!std::strcmp(key, "gemv_order")) {
        if (value < 0 || value > 2) return 1;
        g_opt_gemv_order.store((int)value);
        return 0;
    }
    if (!std::strcmp(key, "gemm_path")) { g_opt_gemm_path.store((int)value); return 0; }
    if (!std::strcmp(key, "fuse_linear")) { g_opt_fuse_linear.store(value != 0); return 0; }
#ifdef BONSAI_B200_TUNING
    // Geometry knobs of the test build (build.py --tuning, the default of this repository's build script): they let the
    // parity tests force every tiling.  A build without the macro has no such keys and always uses the tuned defaults.
    if (!std::strcmp(key, "gemv_variant")) { g_opt_gemv_variant.store((int)value); return 0; }
    if (!std::strcmp(key, "chain_threads")) {
        if (value != 512 && value != 640 && value != 768) return 1;
        g_opt_chain_threads.store((int)value);
        return 0;
    }
    if (!std::strcmp(key, "chain_seg")) {
        if (value < 8 || value > 8 * STREAM_STEPS || value % 8 != 0) return 1;
        g_opt_chain_seg.store((int)value);
        return 0;
    }
    if (!std::strcmp(key, "chain_spread_nb")) {
        if (value < 0) return 1;
        g_opt_chain_spread_nb.store((int)value);
        return 0;
    }
    if (!std::strcmp(key, "gemm_tile")) {
        if (value != 0 && value != 64 && value != 128) return 1;
        g_opt_gemm_tile.store((int)value);
        return 0;
    }
    if (!std::strcmp(key, "chain_tile_kb")) {
        if (value < 4 || value > 48) return 1;
        g_opt_chain_tile_kb.store((int)value);
        return 0;
    }
#endif
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

int bonsai_b200_clear_status(void) {
    const int zero = 0;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return (int)e + 1000;
    e = cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
    return e == cudaSuccess ? 0 : (int)e + 1000;
}

int bonsai_b200_version(void) { return 200; }

// ---- the operators beside the mat-vec path (reference: include/bonsai_p40.h:44-56) ---------------------------
int bonsai_p40_rmsnorm(const float *x, const float *w, float *y, int64_t n_rows, int64_t n, float eps,
                       bonsai_stream stream) {
    // return convention of src/kernels/elementwise_p40.cu:82-88
    if (n <= 0 || n_rows <= 0) return (n <= 0) ? 1 : 0;
    if (n > INT32_MAX || n_rows > INT32_MAX || !aligned4(x) || !aligned4(w) || !aligned4(y)) return 1;
    if (n % 4 == 0 && aligned16(x)) rmsnorm_kernel<true><<<(unsigned)n_rows, 256, 0, as_stream(stream)>>>(x, w, y, (int)n, eps);
    else rmsnorm_kernel<false><<<(unsigned)n_rows, 256, 0, as_stream(stream)>>>(x, w, y, (int)n, eps);
    return (int)cudaGetLastError();
}

int bonsai_b200_swiglu(const float *gate, const float *up, float *y, int64_t n, bonsai_stream stream) {
    if (n <= 0 || n > INT32_MAX || !aligned4(gate) || !aligned4(up) || !aligned4(y)) return 1;
    swiglu_kernel<<<(unsigned)((n + 255) / 256), 256, 0, as_stream(stream)>>>(gate, up, y, (int)n);
    return (int)cudaGetLastError();
}

int bonsai_p40_gdn_step(float *state, const float *q, const float *k, const float *v, const float *g, const float *beta,
                        float *out, int n_k_heads, int n_v_heads, int K, int V, bonsai_stream stream) {
    // rejections of src/kernels/attn_p40.cu:121-124
    if (V <= 0 || V % 32 != 0 || K <= 0 || K > GDN_KMAX) return 1;
    if (n_v_heads <= 0 || n_k_heads <= 0 || n_v_heads % n_k_heads != 0) return 1;
    const int blocks = n_v_heads * (V / 32);
    gdn_step_kernel<<<blocks, GDN_WARPS * 32, 0, as_stream(stream)>>>(state, q, k, v, g, beta, out, n_k_heads, n_v_heads, K, V);
    return (int)cudaGetLastError();
}

int bonsai_p40_attn(const float *q, const float *k, const float *v, float *out, int n_tok, int n_head, int n_head_kv,
                    int head_dim, float scale, bonsai_stream stream) {
    // rejections of src/kernels/attn_p40.cu:134-136
    if (head_dim != ATT_D || n_head_kv == 0 || (n_head % n_head_kv) != 0) return 1;
    if (n_tok <= 0 || n_head <= 0 || n_head_kv <= 0) return (n_tok <= 0) ? 0 : 1;
    if (!aligned16(k) || !aligned16(v) || !aligned4(q) || !aligned4(out)) return 1;    // rows of 256 floats: 16-byte loads
    const long long blocks = (long long)n_head * ((n_tok + ATT_QPC - 1) / ATT_QPC);
    if (blocks > INT32_MAX) return 1;
    static SmemOptIn opt;
    cudaError_t err = opt.ensure(attn_kernel);
    if (err != cudaSuccess) return (int)err;
    attn_kernel<<<(unsigned)blocks, ATT_WARPS * 32, ATT_SMEM_BYTES, as_stream(stream)>>>(q, k, v, out, n_tok, n_head, n_head_kv, scale);
    return (int)cudaGetLastError();
}

// ---- K/V cache (reference: include/bonsai_kv.h, src/kernels/kv_p40.cu:247-367) ----------------------------------
// Geometry of the 27B model (include/bonsai_model.h:29-52): 16 full-attention layers, 24 query / 4 kv heads of 256;
// 48 linear-attention layers with 48 value heads of 128 x 128 state.
namespace {
constexpr int KVM_FULL = 16, KVM_HEADS = 24, KVM_KV_HEADS = 4, KVM_CONTEXT = 262144;
constexpr int KVM_LINEAR = 48, KVM_V_HEADS = 48, KVM_STATE = 128;
constexpr int KV_MAX_SPLIT = KV_COMBINE_MAX;
constexpr size_t KV_SPLIT_SMEM = KV_SPLIT_SMEM_BYTES;
inline int64_t kv_array_bytes(int capacity) { return (int64_t)KVM_FULL * KVM_KV_HEADS * capacity * KV_ROW; }
inline int64_t kv_gdn_bytes() { return (int64_t)KVM_LINEAR * KVM_V_HEADS * KVM_STATE * KVM_STATE * (int64_t)sizeof(float); }
}  // namespace

struct bonsai_kv_cache {
    int capacity = 0;
    uint8_t *d_k = nullptr, *d_v = nullptr;
    float *d_gdn = nullptr, *d_ws = nullptr;
};

int64_t bonsai_kv_bytes(int capacity) {
    if (capacity <= 0) return 0;
    if (capacity > KVM_CONTEXT) capacity = KVM_CONTEXT;
    return 2 * kv_array_bytes(capacity);
}
int64_t bonsai_kv_gdn_bytes(void) { return kv_gdn_bytes(); }

bonsai_kv_cache *bonsai_kv_create(int capacity, bonsai_stream stream) {
    if (capacity <= 0) return nullptr;
    if (capacity > KVM_CONTEXT) capacity = KVM_CONTEXT;
    bonsai_kv_cache *kv = new (std::nothrow) bonsai_kv_cache;
    if (!kv) return nullptr;
    kv->capacity = capacity;
    const size_t ws = (size_t)KVM_HEADS * KV_MAX_SPLIT * KV_WS * sizeof(float);
    if (cudaMalloc(&kv->d_k, (size_t)kv_array_bytes(capacity)) != cudaSuccess || cudaMalloc(&kv->d_v, (size_t)kv_array_bytes(capacity)) != cudaSuccess ||
        cudaMalloc(&kv->d_gdn, (size_t)kv_gdn_bytes()) != cudaSuccess || cudaMalloc(&kv->d_ws, ws) != cudaSuccess ||
        cudaFuncSetAttribute(kv_attn_split_kernel<KVM_HEADS / KVM_KV_HEADS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)KV_SPLIT_SMEM) != cudaSuccess) {
        bonsai_kv_free(kv);
        return nullptr;
    }
    (void)cudaMemsetAsync(kv->d_gdn, 0, (size_t)kv_gdn_bytes(), as_stream(stream));
    return kv;
}

void bonsai_kv_free(bonsai_kv_cache *kv) {
    if (!kv) return;
    cudaFree(kv->d_k);
    cudaFree(kv->d_v);
    cudaFree(kv->d_gdn);
    cudaFree(kv->d_ws);
    delete kv;
}

void bonsai_kv_reset(bonsai_kv_cache *kv, bonsai_stream stream) {
    if (kv) (void)cudaMemsetAsync(kv->d_gdn, 0, (size_t)kv_gdn_bytes(), as_stream(stream));
}

float *bonsai_kv_gdn_state(bonsai_kv_cache *kv, int layer) {
    if (!kv || layer < 0 || layer >= KVM_LINEAR) return nullptr;
    return kv->d_gdn + (size_t)layer * KVM_V_HEADS * KVM_STATE * KVM_STATE;
}

int bonsai_kv_append_batch(bonsai_kv_cache *kv, int layer, int pos0, int n_tok, const float *k, const float *v,
                           bonsai_stream stream) {
    if (!kv || !k || !v) return 1;
    if (layer < 0 || layer >= KVM_FULL) return 1;
    if (n_tok <= 0 || pos0 < 0 || (long long)pos0 + n_tok > kv->capacity) return 1;
    const int nrow = n_tok * KVM_KV_HEADS;
    kv_append_kernel<<<(nrow + 7) / 8, 256, 0, as_stream(stream)>>>(kv->d_k, kv->d_v, k, v, pos0, n_tok, KVM_KV_HEADS, kv->capacity, layer);
    return (int)cudaGetLastError();
}

int bonsai_kv_append(bonsai_kv_cache *kv, int layer, int pos, const float *k, const float *v, bonsai_stream stream) {
    return bonsai_kv_append_batch(kv, layer, pos, 1, k, v, stream);
}

int bonsai_kv_attn_decode(bonsai_kv_cache *kv, int layer, int pos, const float *q, float *out, bonsai_stream stream) {
    if (!kv || !q || !out) return 1;
    if (layer < 0 || layer >= KVM_FULL) return 1;
    if (pos < 0 || pos >= kv->capacity) return 1;
    // splits of at least 4 tiles each, and no more CTAs than are resident at once (one wave): at long context
    // 2 CTAs per SM x 148 SMs / 4 kv heads = 74 splits
    const int grp = KVM_HEADS / KVM_KV_HEADS;
    static int slots = 0;
    if (slots == 0) {
        int per_sm = 0, dev = 0, sms = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kv_attn_split_kernel<KVM_HEADS / KVM_KV_HEADS>, grp * 32, KV_SPLIT_SMEM) != cudaSuccess ||
            cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            return (int)cudaGetLastError();
        slots = per_sm * sms > 0 ? per_sm * sms : 1;
    }
    int n_split = (pos + 1 + 4 * KV_TILE - 1) / (4 * KV_TILE);
    if (n_split > slots / KVM_KV_HEADS) n_split = slots / KVM_KV_HEADS > 0 ? slots / KVM_KV_HEADS : 1;
    if (n_split > KV_MAX_SPLIT) n_split = KV_MAX_SPLIT;
    kv_attn_split_kernel<KVM_HEADS / KVM_KV_HEADS><<<dim3((unsigned)n_split, KVM_KV_HEADS), grp * 32, KV_SPLIT_SMEM, as_stream(stream)>>>(
        q, kv->d_k, kv->d_v, kv->d_ws, pos, n_split, KVM_KV_HEADS, kv->capacity, layer, 0.0625f);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    kv_attn_combine_kernel<<<KVM_HEADS, KV_D, 0, as_stream(stream)>>>(kv->d_ws, out, n_split);
    return (int)cudaGetLastError();
}

// Test access to the cache arrays (byte parity of the quantiser): device pointers of K and V.
int bonsai_b200_kv_arrays(bonsai_kv_cache *kv, void **k, void **v, int64_t *bytes_each) {
    if (!kv || !k || !v || !bytes_each) return 1;
    *k = kv->d_k;
    *v = kv->d_v;
    *bytes_each = kv_array_bytes(kv->capacity);
    return 0;
}

}  // extern "C"
