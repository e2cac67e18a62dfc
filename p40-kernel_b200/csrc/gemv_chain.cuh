// gemv_chain.cuh -- a list of decode projections in ONE persistent launch.
//
// The per-matrix entry point (bonsai_p40_gemv, src/kernels/gemv_p40.cu:210-219 in the reference) pays,
// for every matrix, a kernel start (barriers, activation vector, first-tile latency) and a tail (the
// last tiles are multiplied after the last byte has landed); at batch 1 a projection streams for
// 0.2 - 4 us, so start and tail cost as much as the stream.  Weights never depend on the previous
// projection, only activations do.  Here one CTA per SM walks the whole list: a copy warp streams
// the CTA's rows of op after op into one ring of shared-memory slots without ever stopping at an op
// boundary, compute warps take (row quad x row segment) tasks exactly as gemv_stream_kernel does --
// same lanes, same terms, same summation tree, so y is bit-identical to the per-matrix kernel -- and
// a projection that reads an earlier projection's output waits on a grid-wide arrival counter
// (bounded) while the ring keeps filling behind it.
//
// Warp roles (THREADS / 32 - 2 compute warps, 1 copy warp, 1 sequencer warp; the several-rank form
// gives one compute warp's place to a peer warp, described further down):
//   sequencer : copies op records into a shared ring of 8, and for ops whose activations arrive as
//               Q8_1 blocks stages them (one bulk copy) and re-lays them into one of up to three
//               table buffers while the compute warps are still on earlier ops;
//   copy      : tile g of the CTA (whole rows of one op, <= slot bytes, one contiguous bulk copy)
//               goes to slot g % nslot once every task of tile g - nslot has copied its blocks out;
//   compute   : tasks are handed out in order across ops; entering an op a warp waits for its
//               tables (Q8_1 ops), or -- ops that rotate and quantise an fp32 vector -- all compute
//               warps meet, wait for the producers of that vector, and rotate it together.
//
// Barrier discipline.  Shared-memory barriers are reused, so a waiter identifies a phase by parity;
// that is only sound when the barrier cannot complete a second phase before the waiter has seen the
// first.  Only three kinds of barrier are waited on by parity, and each has that property by
// construction: ready[buf] (its next phase needs every compute warp to have left an op that comes
// after the one being waited for), xs and dep (every waiter must arrive, or pass xs, before the next
// phase can complete), full[slot] (a task first sees `issued > g`, published after the barrier was
// armed for tile g, and the slot cannot be re-armed before that task has copied out).  Everything
// that a warp may fall arbitrarily far behind on is a monotonic counter instead: ops_done (every
// compute warp has left ops [0, ops_done)), ops_loaded, issued, copy_op.  Slot release is a plain
// counter too, because the number of tasks per tile changes from op to op.
// Every wait is bounded; a time-out sets the status word and the warp leaves.
#pragma once

#include "activation.cuh"
#include "common.cuh"
#include "gemv.cuh"
#include "gemv_stream.cuh"
#include "ops.cuh"

namespace b200 {

// Bits 0-5 are the caller's (bonsai_b200_ext.h); the others are set while the list is laid out.
enum : int {
    CHAIN_ROTATE = 1, CHAIN_DEPENDS = 2, CHAIN_SAME_INPUT = 4,
    CHAIN_RMSNORM = 8,        // input = RMSNorm(x; aux = weights, eps)   (src/ops.h:13-22), then signs, rotation, quantiser
    CHAIN_SWIGLU = 16,        // input = silu(x) * aux                     (src/ops.h:27-31)
    CHAIN_RESCALE = 32,       // input[j] = x[j mod src_len] * 2^-e, e = floor(log2(max |x|)): the exact glue of the synthetic decode step
    CHAIN_SIGNAL = 64, CHAIN_SPREAD = 128,
    CHAIN_MAXSRC = 256        // a later CHAIN_RESCALE op reads this op's output: its largest magnitude is recorded
};

constexpr int CHAIN_MAX_SLOTS = 16;
constexpr int CHAIN_OP_RING = 8;
constexpr int CHAIN_TABLES = 3;          // activation-table buffers: the sequencer prepares this many inputs ahead
constexpr uint32_t CHAIN_NS0 = 32, CHAIN_NSMAX = 256;             // first and longest sleep between two polls of a wait
constexpr uint32_t CHAIN_GATE_NS0 = 32, CHAIN_GATE_NSMAX = 256;   // ... of the waits that usually last microseconds
constexpr int CHAIN_GATES = 3;           // a warp may run this many ops ahead of the slowest one

struct __align__(16) ChainOp {                 // 128 bytes, one per projection, device table
    const uint8_t *W;
    const void *x;                             // fp32 vector (CHAIN_ROTATE) or permuted Q8_1 blocks
    const float *signs;
    float *y;
    int nb, n_out, rows_per_cta, tr;
    int nseg, seg_blocks, tpt, flags;
    uint32_t magic_tpt, magic_nseg;
    int cta_shift;                             // CTA c takes the rows of CTA (c + shift) % grid
    uint32_t arrivals_needed;                  // CHAIN_DEPENDS: signalling ops before this one
    int buf;                                   // table buffer this op reads
    int ready_parity;                          // phase parity of ready[buf] (Q8_1 ops that fill a buffer)
    int prev_user;                             // last op that read the previous contents of buf, or -1
    uint32_t spread_blocks;                    // CHAIN_SPREAD: 1024-blocks rotated by spread ops up to and including this one
    const float *aux;                          // CHAIN_RMSNORM: norm weights; CHAIN_SWIGLU: the second vector
    float eps;                                 // CHAIN_RMSNORM
    int src_len;                               // CHAIN_RESCALE: floats at x
    int src_op;                                // CHAIN_RESCALE: the op whose output x is
    int pad[3];
};
static_assert(sizeof(ChainOp) == 128, "op records are copied as 32 words");

struct ChainGeom {
    int nslot, slot_bytes;
    uint32_t magic_nslot;
    int nb_max;               // longest row, in blocks: sizes the tables
    int stage_blocks;         // nb_max if any op takes Q8_1 blocks (staging area of the sequencer), else 0
    int rot_blocks;           // 1024-blocks of rotation scratch (0 if no op rotates)
    int rows_stage;           // several ranks: max rows per CTA (finished rows are staged in shared memory for the peer warp), else 0
    int ntables;              // table buffers in use: CHAIN_TABLES, or 1 when every op rotates its own input (the
                              // compute warps fill the buffer themselves, after all of them have left the op before)
    int partial_floats;       // per buffer: max rows_per_cta * nseg, multiple of 4
    int quad_ints;            // per buffer: max rows_per_cta / 4, multiple of 4
};

// Shared-memory bytes before the ring (the host uses the same function).
__host__ __device__ inline size_t chain_fixed_bytes(const ChainGeom &G) {
    const size_t b = 640 + CHAIN_OP_RING * sizeof(ChainOp) + (size_t)G.ntables * G.nb_max * 176 + (size_t)G.stage_blocks * 144 +
                     (size_t)G.rot_blocks * 4096 +
                     CHAIN_GATES * (size_t)G.partial_floats * 4 + CHAIN_GATES * (size_t)G.quad_ints * 4 +
                     CHAIN_GATES * (size_t)G.rows_stage * 4;
    return (b + 127) & ~(size_t)127;
}

__device__ __forceinline__ bool spin_until_gt(volatile int *p, int v, uint32_t first_ns = CHAIN_NS0,
                                              uint32_t max_ns = CHAIN_NSMAX) {
    uint32_t ns = first_ns;
    for (uint32_t n = 0; n < (1u << 22); ++n) {
        if (*p > v) return true;
        __nanosleep(ns);
        ns = min(ns * 2, max_ns);
    }
    atomicExch(&g_device_status, STATUS_MBARRIER_TIMEOUT);
    return false;
}
__device__ __forceinline__ bool spin_until_eq(volatile int *p, int v) {
    uint32_t ns = CHAIN_NS0;
    for (uint32_t n = 0; n < (1u << 22); ++n) {
        if (*p == v) return true;
        __nanosleep(ns);
        ns = min(ns * 2, (uint32_t)CHAIN_NSMAX);
    }
    atomicExch(&g_device_status, STATUS_MBARRIER_TIMEOUT);
    return false;
}
// Arrival counter of this GPU's own CTAs, polled by one lane, bounded by an iteration count.  Counters only grow,
// so "reached" is a wrap-safe signed difference.
__device__ __forceinline__ bool grid_counter_wait(const unsigned int *counter, unsigned int target) {
    uint32_t ns = CHAIN_NS0;
    for (uint32_t n = 0; n < (1u << 22); ++n) {
        unsigned int v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
        if ((int)(v - target) >= 0) return true;
        __nanosleep(ns);
        ns = min(ns * 2, CHAIN_NSMAX);
    }
    atomicExch(&g_device_status, STATUS_GRID_TIMEOUT);
    return false;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Several ranks: flag word q of this rank's counter block is written by rank q (one store over NVLink per signal).
// Lane q < world polls flag q (acquire at system scope) until it has reached `target`; the wait ends for the whole
// warp when every flag is there, or when `limit_ns` nanoseconds have passed (status word, false).  Called by a
// whole warp.
__device__ __forceinline__ bool rank_flags_wait(const unsigned int *flags, int world, unsigned int target,
                                                unsigned long long limit_ns, int lane) {
    const unsigned long long t0 = global_timer_ns();
    uint32_t ns = CHAIN_NS0;
    for (uint32_t n = 1; n < (1u << 26); ++n) {
        bool here = true;
        if (lane < world) {
            unsigned int v;
            asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + lane) : "memory");
            here = (int)(v - target) >= 0;
        }
        if (__all_sync(0xffffffffu, here)) {
            __threadfence_system();         // acquire: what the other ranks wrote before their flags is visible from here on
            return true;
        }
        if ((n & 15u) == 0 && global_timer_ns() - t0 > limit_ns) break;      // the clock is read now and then, not per poll
        __nanosleep(ns);
        ns = min(ns * 2, CHAIN_NSMAX);
    }
    if (lane == 0) atomicExch(&g_device_status, STATUS_GRID_TIMEOUT);
    return false;
}

// Row-partitioned lists over several GPUs (one process and one launch per GPU, same list on every rank over its
// own row slices).  The rows a CTA writes are also copied into the same place of every peer's buffer when the CTA
// leaves the op (coalesced stores to peer-mapped memory over NVLink), so each rank ends up with the whole vector.
// "Every row of every earlier op is there" then means on every rank.  Signalling costs ONE store per peer and
// signal: after an op that others wait for, each CTA's peer warp fences at system scope and adds 1 to a counter in
// LOCAL memory; the CTA that completes the count (all CTAs of this GPU have sent their rows) writes the signal's
// sequence number into flag word `rank` of every rank's counter block, and a dependent op polls the `world` flag
// words of its own block.  Sequence numbers are never reset: a launch reads its run number from counter word 2 and
// the last CTA to leave adds 1 to it; every launch ends with one more signal + wait, so that no rank starts its
// next run (and writes into its peers' outputs) before every rank has finished this one.
// Counter block (16 words): [0] arrivals of dependent-op producers (one-rank form) [1] spread blocks [2] run
// [3] CTAs out [4] CTAs of this GPU that have sent their rows, all signals so far [8 + q] last signal of rank q.
constexpr int CHAIN_MAX_RANKS = 8;
struct ChainPeers {
    int rank, world;
    unsigned int arrivals_per_run;              // signalling ops (the closing one included) of one run
    unsigned int spread_per_run;                // 1024-blocks rotated by spread ops in one run
    unsigned long long wait_limit_ns;           // longest wait for the other ranks
    long long y_delta[CHAIN_MAX_RANKS];         // byte offset from this rank's buffer to rank p's mapping of its own
    unsigned int *counter[CHAIN_MAX_RANKS];     // rank p's counter block
};

template <int THREADS, int MAXSTEPS, bool TP>
__global__ void __launch_bounds__(THREADS, 1) gemv_chain_kernel(const ChainOp *__restrict__ ops, const int n_ops,
                                                                const ChainGeom G, unsigned int *grid_counter,
                                                                uint8_t *table_image, const ChainPeers PE) {
    constexpr int C = THREADS / 32 - 2 - (TP ? 1 : 0);      // compute warps (several ranks: one warp talks to the peers)
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);      // [16] tile landed in slot
    uint64_t *ready = full + CHAIN_MAX_SLOTS;                 // [2]  tables of a Q8_1 op are filled
    uint64_t *xs = ready + CHAIN_TABLES;                                  // [1]  rotate: every warp has written its blocks
    uint64_t *dep = xs + 1;                                   // [1]  rotate: the producers of x have arrived
    uint64_t *stage_full = dep + 1;                           // [1]  Q8_1 staging copy landed
    int *done_cnt = reinterpret_cast<int *>(smem + 192);      // [16] tasks of the slot's tile that have copied out
    int *expect_cnt = done_cnt + CHAIN_MAX_SLOTS;             // [16] ... of how many
    volatile int *ctrl = expect_cnt + CHAIN_MAX_SLOTS;        // [16] 0 issued, 1 ops_loaded, 2 next_task, 3 copy_op, 4-7 warps that
                                                              //      left op (index & 3), 8 ops_done: every compute warp has left ops [0, ops_done),
                                                              //      9 (several ranks) ops whose rows the peer warp has sent,
                                                              //      10-13 largest |y| of op (index & 3) so far, as float bits
    float *ssum = reinterpret_cast<float *>(smem + 384);     // [56] sums of squares of the slices of an RMSNorm input
    ChainOp *opring = reinterpret_cast<ChainOp *>(smem + 640);
    uint8_t *p = smem + 640 + CHAIN_OP_RING * sizeof(ChainOp);
    const size_t table_bytes = (size_t)G.nb_max * 176;
    uint8_t *tables = p;
    p += (size_t)G.ntables * table_bytes;
    uint32_t *stage = reinterpret_cast<uint32_t *>(p);
    p += (size_t)G.stage_blocks * 144;
    float4 *scratch = reinterpret_cast<float4 *>(p);
    p += (size_t)G.rot_blocks * FWHT_N * 4;
    float *partial_base = reinterpret_cast<float *>(p);
    p += CHAIN_GATES * (size_t)G.partial_floats * 4;
    int *quad_base = reinterpret_cast<int *>(p);
    p += CHAIN_GATES * (size_t)G.quad_ints * 4;
    float *ystage = reinterpret_cast<float *>(p);
    uint8_t *ring = smem + chain_fixed_bytes(G);

    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int ncta = (int)gridDim.x;

    if (threadIdx.x == 0) {
        for (int s = 0; s < CHAIN_MAX_SLOTS; ++s) mbar_init(&full[s], 1);
        for (int i = 0; i < CHAIN_TABLES; ++i) mbar_init(&ready[i], 1);
        mbar_init(xs, C);
        mbar_init(dep, 1);
        mbar_init(stage_full, 1);
        mbar_fence_init();
    }
    for (int i = threadIdx.x; i < 3 * CHAIN_MAX_SLOTS; i += THREADS) done_cnt[i] = 0;     // done, expect, ctrl
    for (int i = threadIdx.x; i < CHAIN_GATES * G.quad_ints; i += THREADS) quad_base[i] = 0;
    __syncthreads();

    // several ranks: counters are never reset, this launch's targets start at run * (what one run adds)
    unsigned int arrive_base = 0, spread_base = 0;
    if (TP) {
        const unsigned int run = __ldcg(grid_counter + 2);          // written by the previous launch on this stream
        arrive_base = run * PE.arrivals_per_run;                    // signals before this run
        spread_base = run * PE.spread_per_run;
    }
    // a finished y element (several ranks: the CTA's rows go to the peers in one piece when it leaves the op)
    float ymax = 0.0f;          // largest |y| this lane has stored in the current op (kept only for CHAIN_MAXSRC ops)
    auto store_y = [&](float *p, float v, int op_, int r_) {
        *p = v;
        ymax = fmaxf(ymax, fabsf(v));
        if (TP) ystage[(size_t)(op_ % CHAIN_GATES) * G.rows_stage + r_] = v;
    };
    unsigned int *opmax = grid_counter + 64;     // one word per op behind the counters (one-rank form)
    // this CTA's rows of every op so far are written: tell the grid
    auto arrive_all = [&]() {
        __threadfence();
        atomicAdd(grid_counter, 1u);
    };

    // rows of op R that this CTA owns
    auto cta_rows = [&](const ChainOp &R, int &row0, int &rows_here) {
        int c = (int)blockIdx.x + R.cta_shift;
        if (c >= ncta) c -= ncta;
        row0 = c * R.rows_per_cta;
        rows_here = max(0, min(R.rows_per_cta, R.n_out - row0));
    };

    if (wid < C) {
        // ================================ compute warps ================================
        const int rr = lane & 3, bl = lane >> 2;
        int op = -1, flags = 0;
        int issued_seen = 0;
        uint32_t xs_phase = 0, dep_phase = 0;     // every compute warp takes part in every meeting, so it counts them itself
        int task_base = 0, ntasks = 0, g_base = 0, ntiles = 0, row0 = 0, rows_here = 0;
        for (;;) {
            int task = 0;
            if (lane == 0) task = atomicAdd(const_cast<int *>(&ctrl[2]), 1);
            task = __shfl_sync(0xffffffffu, task, 0);
            bool alive = true;
            while (task >= task_base + ntasks) {
                // ---- leave op `op`
                if (op >= 0) {
                    // this warp's y rows are in memory (device scope) before it is counted out below: other CTAs read them
                    // once everybody has arrived (several ranks: the peer warp reads its copy in shared memory)
                    if (flags & CHAIN_SIGNAL) __threadfence();
                    if (!TP && (flags & CHAIN_MAXSRC)) {                // the warp's largest |y|, then the CTA's (float bits order as ints)
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) ymax = fmaxf(ymax, __shfl_xor_sync(0xffffffffu, ymax, o));
                        if (lane == 0) atomicMax(const_cast<int *>(&ctrl[10 + (op & 3)]), __float_as_int(ymax));
                    }
                    __syncwarp();
                    if (lane == 0) {
                        __threadfence_block();                          // this warp's reads of op's tables and partial sums
                        const int old = atomicAdd(const_cast<int *>(&ctrl[4 + (op & 3)]), 1);
                        if (old == C - 1) {                             // last warp out: the CTA's rows of every op so far are written
                            ctrl[4 + (op & 3)] = 0;
                            if (!TP && (flags & CHAIN_MAXSRC)) {        // ... and the largest of them is known: to the grid, before the arrival
                                atomicMax(opmax + op, (unsigned int)ctrl[10 + (op & 3)]);
                                ctrl[10 + (op & 3)] = 0;
                            }
                            if (!TP && (flags & CHAIN_SIGNAL)) arrive_all();
                            __threadfence_block();
                            ctrl[8] = op + 1;                           // monotonic: ops are left in order
                        }
                    }
                }
                task_base += ntasks;
                g_base += ntiles;
                ++op;
                if (op >= n_ops) { alive = false; break; }
                // ---- enter op `op`
                if (!spin_until_gt(&ctrl[1], op, CHAIN_GATE_NS0, CHAIN_GATE_NSMAX)) { alive = false; break; }
                if (op >= CHAIN_GATES && !spin_until_gt(&ctrl[8], op - CHAIN_GATES, CHAIN_GATE_NS0, CHAIN_GATE_NSMAX)) { alive = false; break; }
                // several ranks: the peer warp has sent the rows staged where this op will stage its own
                if (TP && op >= CHAIN_GATES && !spin_until_gt(&ctrl[9], op - CHAIN_GATES)) { alive = false; break; }
                const ChainOp &R = opring[op & (CHAIN_OP_RING - 1)];
                flags = R.flags;
                cta_rows(R, row0, rows_here);
                ntiles = (rows_here + R.tr - 1) / R.tr;
                ntasks = ntiles * R.tpt;
                ymax = 0.0f;
                if (!(flags & CHAIN_SAME_INPUT)) {
                    if (flags & CHAIN_ROTATE) {
                        // every compute warp has left op - 1: both table buffers' readers are gone
                        if (op >= 1 && !spin_until_gt(&ctrl[8], op - 1)) { alive = false; break; }
                        if (flags & CHAIN_DEPENDS) {
                            if (wid == 0) {
                                bool ok = true;
                                if (TP) ok = rank_flags_wait(grid_counter + 8, PE.world, arrive_base + R.arrivals_needed,
                                                             PE.wait_limit_ns, lane);
                                else if (lane == 0) ok = grid_counter_wait(grid_counter, R.arrivals_needed * (unsigned)ncta);
                                __syncwarp();
                                if (lane == 0 && ok) mbar_arrive(dep);
                            }
                            if (!mbar_wait_bounded(dep, dep_phase & 1u, CHAIN_NS0, CHAIN_NSMAX)) { alive = false; break; }
                            ++dep_phase;
                        }
                        // Wide inputs of dependent ops are rotated ONCE for the whole grid instead of once per CTA
                        // (every CTA repeating 17 blocks costs ~10 us): block fb is rotated by CTA fb, which writes
                        // its part of the tables to an image in global memory; a second arrival counter tells
                        // everybody when all blocks are there, and every CTA copies the image into its tables.
                        const bool spread = flags & CHAIN_SPREAD;
                        uint8_t *own = tables + (size_t)R.buf * table_bytes;
                        uint32_t *act_q = reinterpret_cast<uint32_t *>(spread ? table_image : own);
                        float *act_s = reinterpret_cast<float *>(act_q + (size_t)G.nb_max * STREAM_ACT_WORDS);
                        int *act_i = reinterpret_cast<int *>(act_s + (size_t)G.nb_max * 4);
                        const float *x = static_cast<const float *>(R.x);
                        const float *signs = R.signs;
                        const float *aux = R.aux;
                        const int nfb = R.nb >> 3;
                        const int fb_lo = spread ? min((int)blockIdx.x, nfb) : 0;
                        const int fb_hi = spread ? min((int)blockIdx.x + 1, nfb) : nfb;
                        // the exact power-of-two rescale of the synthetic decode step: the producer recorded max |x|
                        float rescale = 1.0f;
                        const int src_len = R.src_len;
                        if (flags & CHAIN_RESCALE) {
                            const unsigned int mb = __ldcg(opmax + R.src_op);
                            const int e8 = (int)(mb >> 23);                     // biased exponent of the largest magnitude
                            if (e8 >= 1) rescale = __int_as_float(max(1, 254 - e8) << 23);      // 2^-(e8 - 127); zero / subnormal: unscaled
                        }
                        // One warp per 128-element slice, G.rot_blocks 1024-blocks per round trip through
                        // the scratch area: front butterflies, meet, back butterflies + quantiser, meet.
                        bool ok = true;
                        for (int fb0 = fb_lo; fb0 < fb_hi && ok; fb0 += G.rot_blocks) {
                            const int units = min(G.rot_blocks, fb_hi - fb0) * 8;
                            // all of this warp's loads first (they come from L2: written by other SMs
                            // during this launch), then the butterflies
                            constexpr int UPW = (7 * 8 + C - 1) / C;           // units per warp and round trip
                            float4 f[UPW];
#pragma unroll
                            for (int k = 0; k < UPW; ++k) {
                                const int u = wid + k * C;
                                if (u < units) {
                                    int idx = fb0 * FWHT_N + u * 128 + 4 * lane;
                                    if (flags & CHAIN_RESCALE) idx %= src_len;
                                    f[k] = __ldcg(reinterpret_cast<const float4 *>(x + idx));
                                }
                            }
                            if (flags & (CHAIN_SWIGLU | CHAIN_RESCALE)) {
#pragma unroll
                                for (int k = 0; k < UPW; ++k) {
                                    const int u = wid + k * C;
                                    if (u < units) {
                                        if (flags & CHAIN_SWIGLU) {
                                            const float4 up = __ldcg(reinterpret_cast<const float4 *>(aux + (size_t)fb0 * FWHT_N + (size_t)u * 128 + 4 * lane));
                                            f[k] = make_float4(swiglu1(f[k].x, up.x), swiglu1(f[k].y, up.y), swiglu1(f[k].z, up.z), swiglu1(f[k].w, up.w));
                                        } else {
                                            f[k] = make_float4(__fmul_rn(f[k].x, rescale), __fmul_rn(f[k].y, rescale), __fmul_rn(f[k].z, rescale), __fmul_rn(f[k].w, rescale));
                                        }
                                    }
                                }
                            }
                            if (flags & CHAIN_RMSNORM) {
                                // the whole vector is in the registers of this pass (the host refuses longer ones): slice sums
                                // of squares, meet, every warp adds them in slice order, scales and applies the weights
#pragma unroll
                                for (int k = 0; k < UPW; ++k) {
                                    const int u = wid + k * C;
                                    if (u < units) {
                                        const float sq = slice_sumsq(f[k]);
                                        if (lane == 0) ssum[u] = sq;
                                    }
                                }
                                __syncwarp();
                                if (lane == 0) mbar_arrive(xs);
                                ok = mbar_wait_bounded(xs, xs_phase & 1u, CHAIN_NS0, CHAIN_NSMAX);
                                ++xs_phase;
                                if (!ok) break;
                                float ss = 0.0f;
                                for (int u = 0; u < units; ++u) ss = __fadd_rn(ss, ssum[u]);
                                const float sc = rms_scale(ss, R.nb * 128, R.eps);
#pragma unroll
                                for (int k = 0; k < UPW; ++k) {
                                    const int u = wid + k * C;
                                    if (u < units) {
                                        const float4 wv = __ldg(reinterpret_cast<const float4 *>(aux + (size_t)u * 128 + 4 * lane));
                                        f[k] = make_float4(__fmul_rn(__fmul_rn(f[k].x, sc), wv.x), __fmul_rn(__fmul_rn(f[k].y, sc), wv.y),
                                                           __fmul_rn(__fmul_rn(f[k].z, sc), wv.z), __fmul_rn(__fmul_rn(f[k].w, sc), wv.w));
                                    }
                                }
                            }
#pragma unroll
                            for (int k = 0; k < UPW; ++k) {
                                const int u = wid + k * C;
                                if (u < units) {
                                    float v[4] = {f[k].x, f[k].y, f[k].z, f[k].w};
                                    if (signs) {
                                        const float4 sg = __ldg(reinterpret_cast<const float4 *>(signs + (size_t)fb0 * FWHT_N + (size_t)u * 128 + 4 * lane));
                                        v[0] = __fmul_rn(v[0], sg.x); v[1] = __fmul_rn(v[1], sg.y);
                                        v[2] = __fmul_rn(v[2], sg.z); v[3] = __fmul_rn(v[3], sg.w);
                                    }
                                    fwht_slice_front(v, lane);
                                    scratch[u * 32 + lane] = make_float4(v[0], v[1], v[2], v[3]);
                                }
                            }
                            __syncwarp();
                            if (lane == 0) mbar_arrive(xs);
                            ok = mbar_wait_bounded(xs, xs_phase & 1u, CHAIN_NS0, CHAIN_NSMAX);
                            ++xs_phase;
                            if (!ok) break;
                            for (int u = wid; u < units; u += C) {
                                float v[4];
                                fwht_slice_back(scratch + (u >> 3) * 256, u & 7, lane, v);
                                uint32_t word, header;
                                quantise_chunk_8lanes(v, lane, word, header);
                                const int chunk = fb0 * 32 + u * 4 + (lane >> 3);
                                act_q[(chunk >> 2) * STREAM_ACT_WORDS + (chunk & 3) * 8 + (lane & 7)] = word;
                                if ((lane & 7) == 0) {
                                    act_s[chunk] = f16_bits_to_f32(header & 0xFFFFu);
                                    act_i[chunk] = -64 * (int)(short)(header >> 16);
                                }
                            }
                            if (spread) __threadfence();                // the image rows written above, before the arrival below
                            __syncwarp();
                            if (lane == 0) mbar_arrive(xs);
                            ok = mbar_wait_bounded(xs, xs_phase & 1u, CHAIN_NS0, CHAIN_NSMAX);
                            ++xs_phase;
                        }
                        if (!ok) { alive = false; break; }
                        if (spread) {
                            if (wid == 0) {
                                bool there = true;
                                if (lane == 0) {
                                    if (fb_lo < fb_hi) {                // this CTA's block is in the image (every warp has fenced)
                                        __threadfence();
                                        atomicAdd(grid_counter + 1, (unsigned)(fb_hi - fb_lo));
                                    }
                                    there = grid_counter_wait(grid_counter + 1, spread_base + R.spread_blocks);
                                }
                                __syncwarp();
                                if (lane == 0 && there) mbar_arrive(dep);
                            }
                            if (!mbar_wait_bounded(dep, dep_phase & 1u, CHAIN_NS0, CHAIN_NSMAX)) { alive = false; break; }
                            ++dep_phase;
                            // image -> this CTA's tables (written by other SMs during this launch: read at L2)
                            const uint4 *src16 = reinterpret_cast<const uint4 *>(table_image);
                            uint4 *dst16 = reinterpret_cast<uint4 *>(own);
                            const int n16 = (int)(table_bytes >> 4);
                            for (int i = wid * 32 + lane; i < n16; i += C * 32) dst16[i] = __ldcg(src16 + i);
                            __syncwarp();
                            if (lane == 0) mbar_arrive(xs);
                            if (!mbar_wait_bounded(xs, xs_phase & 1u, CHAIN_NS0, CHAIN_NSMAX)) { alive = false; break; }
                            ++xs_phase;
                        }
                    } else {
                        if (!mbar_wait_bounded(&ready[R.buf], (uint32_t)R.ready_parity, CHAIN_GATE_NS0, CHAIN_GATE_NSMAX)) { alive = false; break; }
                    }
                }
            }
            if (!alive) break;

            // ---- one task of op `op`: same lanes, terms and sums as gemv_stream_kernel
            const ChainOp &R = opring[op & (CHAIN_OP_RING - 1)];
            const int nb = R.nb, nseg = R.nseg;
            const int row_bytes = nb * W_BLOCK_BYTES;
            const int local_task = task - task_base;
            const int t = (int)fast_div((uint32_t)local_task, R.magic_tpt);
            const int local = local_task - t * R.tpt;
            const int quad = (int)fast_div((uint32_t)local, R.magic_nseg);
            const int j = local - quad * nseg;
            const int r_quad = t * R.tr + quad * 4;
            if (r_quad >= rows_here) continue;                      // padding quad of a ragged last tile
            const int g = g_base + t;
            const int lap = (int)fast_div((uint32_t)g, G.magic_nslot);
            const int slot = g - lap * G.nslot;
            if (g >= issued_seen) {                                 // tile g must be armed: then the parity below is unambiguous
                if (!spin_until_gt(&ctrl[0], g)) break;
                issued_seen = ctrl[0];
            }
            if (!mbar_wait_bounded(&full[slot], (uint32_t)(lap & 1), CHAIN_NS0, CHAIN_NSMAX)) break;
            const int b0 = j * R.seg_blocks;
            const int blocks = min(R.seg_blocks, nb - b0);
            const uint8_t *rowp = ring + (size_t)slot * G.slot_bytes + (size_t)(quad * 4 + rr) * row_bytes +
                                  (size_t)b0 * W_BLOCK_BYTES;
            const uint32_t *act_q = reinterpret_cast<const uint32_t *>(tables + (size_t)R.buf * table_bytes);
            const float *act_s = reinterpret_cast<const float *>(act_q + (size_t)G.nb_max * STREAM_ACT_WORDS);
            const int *act_i = reinterpret_cast<const int *>(act_s + (size_t)G.nb_max * 4);
            float acc = stream_task<MAXSTEPS>(rowp, bl, b0, blocks, act_q, act_s, act_i, [&]() {
                __syncwarp();
                if (lane == 0) {
                    __threadfence_block();                          // the loads above, before the slot is handed back
                    atomicAdd(&done_cnt[slot], 1);
                }
            });
            acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 4));
            acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 8));
            acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 16));
            const int r = r_quad + rr;
            float *y = R.y;
            if (nseg == 1) {
                if (bl == 0 && r < rows_here) store_y(&y[row0 + r], acc, op, r);
            } else {
                float *partial = partial_base + (size_t)(op % CHAIN_GATES) * G.partial_floats;
                int *quad_count = quad_base + (size_t)(op % CHAIN_GATES) * G.quad_ints;
                if (bl == 0) partial[r * nseg + j] = acc;
                __syncwarp();
                int last = 0;
                if (lane == 0) {
                    __threadfence_block();
                    last = atomicAdd(&quad_count[r_quad >> 2], 1) == nseg - 1;
                    if (last) quad_count[r_quad >> 2] = 0;           // left clean for the next op that uses this buffer
                }
                last = __shfl_sync(0xffffffffu, last, 0);
                if (last) {
                    __threadfence_block();
                    if (bl == 0 && r < rows_here) {
                        float total = partial[r * nseg];
                        for (int sgm = 1; sgm < nseg; ++sgm) total = __fadd_rn(total, partial[r * nseg + sgm]);
                        store_y(&y[row0 + r], total, op, r);
                    }
                }
            }
        }
    } else if (wid == C) {
        // ================================ copy warp (one lane) ================================
        if (lane != 0) return;
        const uint64_t pol = policy_evict_first();
        int g = 0, slot = 0;
        for (int op = 0; op < n_ops; ++op) {
            if (!spin_until_gt(&ctrl[1], op)) return;
            const ChainOp &R = opring[op & (CHAIN_OP_RING - 1)];
            int row0, rows_here;
            cta_rows(R, row0, rows_here);
            const int tr = R.tr, nseg = R.nseg;
            const size_t row_bytes = (size_t)R.nb * W_BLOCK_BYTES;
            const uint8_t *src = R.W + (size_t)row0 * row_bytes;
            const int ntiles = (rows_here + tr - 1) / tr;
            for (int t = 0; t < ntiles; ++t) {
                if (g >= G.nslot && !spin_until_eq(&done_cnt[slot], expect_cnt[slot])) return;
                const int r_cnt = min(tr, rows_here - t * tr);
                done_cnt[slot] = 0;
                expect_cnt[slot] = ((r_cnt + 3) >> 2) * nseg;
                __threadfence_block();
                // the slot was read through ordinary loads: order them before the asynchronous overwrite
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                uint8_t *dst = ring + (size_t)slot * G.slot_bytes;
                const uint32_t bytes = (uint32_t)(r_cnt * row_bytes);
                const uint32_t bulk = bytes & ~15u;
                const uint8_t *s = src + (size_t)t * tr * row_bytes;
                for (uint32_t o = bulk; o < bytes; o += 4) *reinterpret_cast<uint32_t *>(dst + o) = ldg_nc_u32(s + o);
                mbar_expect_tx(&full[slot], bulk);
                if (bulk) bulk_g2s(dst, s, bulk, &full[slot], pol);
                __threadfence_block();
                ctrl[0] = g + 1;                                    // tile g is armed
                ++g;
                if (++slot == G.nslot) slot = 0;
            }
            ctrl[3] = op + 1;                                       // this op's record is no longer read here
        }
    } else if (TP && wid == C + 2) {
        // ================================ peer warp (several ranks) ================================
        // Follows ops_done: when every compute warp has left op k, copies the CTA's rows of op k (contiguous in y)
        // into every peer's buffer, 128 bytes per store; after an op that others wait for it fences at system scope
        // and adds 1 to the arrival counter of every rank.  All traffic to the peers comes from this one warp, so
        // its own program order and fences cover it, and the compute warps never wait for NVLink.
        bool good = true;
        for (int k = 0; k < n_ops && good; ++k) {
            good = spin_until_gt(&ctrl[8], k);
            if (!good) break;
            const ChainOp *Rk = ops + k;                    // the device table: the shared ring may be past op k by now
            const int rpc = __ldg(&Rk->rows_per_cta), n_out = __ldg(&Rk->n_out), kflags = __ldg(&Rk->flags);
            int c = (int)blockIdx.x + __ldg(&Rk->cta_shift);
            if (c >= ncta) c -= ncta;
            const int r0 = c * rpc, rows = max(0, min(rpc, n_out - r0));
            if (rows > 0) {
                float *home = reinterpret_cast<float *>(__ldg(reinterpret_cast<const unsigned long long *>(&Rk->y))) + r0;
                const float *staged = ystage + (size_t)(k % CHAIN_GATES) * G.rows_stage;
#pragma unroll 1
                for (int q = 0; q < PE.world; ++q) {
                    if (q == PE.rank) continue;
                    float *dst = reinterpret_cast<float *>(reinterpret_cast<char *>(home) + PE.y_delta[q]);
                    for (int i = lane; i < rows; i += 32) dst[i] = staged[i];
                }
            }
            __syncwarp();
            if (lane == 0) {
                __threadfence_block();
                ctrl[9] = k + 1;                            // the staging rows of op k may be reused
            }
            if (kflags & CHAIN_SIGNAL) {
                // this CTA's rows are on their way to every rank: count it in local memory; whoever completes the
                // count for this signal tells every rank (one store each), ordered behind every CTA's stores
                // (the warp's stores are ordered before lane 0's fence by the warp barrier; one fence per CTA, then,
                // in the CTA that completes the count, one more behind the count and plain stores of the flags)
                __syncwarp();
                if (lane == 0) {
                    __threadfence_system();
                    const unsigned int seq = arrive_base + __ldg(&Rk->arrivals_needed) + 1u;    // this signal, counted from 1
                    const unsigned int old = atomicAdd(grid_counter + 4, 1u);
                    if (old + 1u == seq * (unsigned)ncta) {
                        __threadfence_system();
                        for (int q = 0; q < PE.world; ++q)
                            asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(PE.counter[q] + 8 + PE.rank), "r"(seq) : "memory");
                    }
                }
            }
        }
        // the closing wait: every rank has sent the rows of its last op (the host marks it as one that others wait
        // for), so nobody is still reading this run's vectors when a rank starts its next run
        if (good) good = rank_flags_wait(grid_counter + 8, PE.world, arrive_base + PE.arrivals_per_run, PE.wait_limit_ns, lane);
        if (good && lane == 0) {
            if (atomicAdd(grid_counter + 3, 1u) == (unsigned)ncta - 1u) {        // last CTA out: the next launch is run + 1
                grid_counter[3] = 0u;
                __threadfence();
                atomicAdd(grid_counter + 2, 1u);
            }
        }
    } else {
        // ================================ sequencer warp ================================
        int gate_seen = 0;                  // every compute warp has left ops [0, gate_seen)
        uint32_t stage_parity = 0;
        const uint64_t pol = policy_evict_first();
        auto see_gates = [&](int upto) {    // waits until every compute warp has left ops [0, upto]
            if (gate_seen > upto) return true;
            if (!spin_until_gt(&ctrl[8], upto, CHAIN_GATE_NS0, CHAIN_GATE_NSMAX)) return false;
            gate_seen = ctrl[8];
            return true;
        };
        int rec_next = 0;                   // records [0, rec_next) are in the shared ring
        // Record r goes where record r - 8 was: every compute warp and the copy lane must be past that
        // one.  Loads whatever is allowed without blocking, so that the copy lane can run ahead of the
        // table preparation below; blocks only when `must` is not there yet.
        auto load_records = [&](int must) {
            for (;;) {
                gate_seen = ctrl[8];
                while (rec_next < n_ops &&
                       (rec_next < CHAIN_OP_RING ||
                        (gate_seen > rec_next - CHAIN_OP_RING && ctrl[3] > rec_next - CHAIN_OP_RING))) {
                    reinterpret_cast<uint32_t *>(opring + (rec_next & (CHAIN_OP_RING - 1)))[lane] =
                        __ldg(reinterpret_cast<const uint32_t *>(ops + rec_next) + lane);
                    __syncwarp();
                    if (lane == 0) {
                        __threadfence_block();
                        ctrl[1] = rec_next + 1;
                    }
                    __syncwarp();
                    ++rec_next;
                }
                if (rec_next > must) return true;
                if (!see_gates(must - CHAIN_OP_RING)) return false;
                if (!spin_until_gt(&ctrl[3], must - CHAIN_OP_RING)) return false;
            }
        };
        for (int op = 0; op < n_ops; ++op) {
            if (!load_records(op)) return;
            const ChainOp &R = opring[op & (CHAIN_OP_RING - 1)];
            if (R.flags & (CHAIN_ROTATE | CHAIN_SAME_INPUT)) continue;
            // Q8_1 blocks: stage the raw bytes with one bulk copy (the staging area is this warp's own, so
            // the copy flies while the table buffer is still being read), then re-lay them into the tables
            const int nchunks = R.nb * 4;
            if (lane == 0) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_expect_tx(stage_full, (uint32_t)nchunks * A_BLOCK_BYTES);
                bulk_g2s(stage, R.x, (uint32_t)nchunks * A_BLOCK_BYTES, stage_full, pol);
            }
            if (!see_gates(R.prev_user)) return;
            if (!mbar_wait_bounded(stage_full, stage_parity, CHAIN_NS0, CHAIN_NSMAX)) return;
            stage_parity ^= 1u;
            uint32_t *act_q = reinterpret_cast<uint32_t *>(tables + (size_t)R.buf * table_bytes);
            float *act_s = reinterpret_cast<float *>(act_q + (size_t)G.nb_max * STREAM_ACT_WORDS);
            int *act_i = reinterpret_cast<int *>(act_s + (size_t)G.nb_max * 4);
            for (int chunk = lane; chunk < nchunks; chunk += 32) {
                const uint32_t *s = stage + 9 * chunk;
                uint32_t *q = act_q + (chunk >> 2) * STREAM_ACT_WORDS + (chunk & 3) * 8;
                const uint32_t h = s[0];
                *reinterpret_cast<uint4 *>(q) = make_uint4(s[1], s[2], s[3], s[4]);
                *reinterpret_cast<uint4 *>(q + 4) = make_uint4(s[5], s[6], s[7], s[8]);
                act_s[chunk] = f16_bits_to_f32(h & 0xFFFFu);
                act_i[chunk] = -64 * (int)(short)(h >> 16);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&ready[R.buf]);
        }
    }
}

}  // namespace b200
