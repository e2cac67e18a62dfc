// kv.cuh -- the growing Q8_0 K/V cache of the full-attention layers: append (quantise) and single-query decode
// attention over it.  Replaces, for sm_100a, src/kernels/kv_p40.cu:47-245 of the reference; the numeric core it
// follows is src/kv_cache.h:100-176 (Q8_0 rows: d = amax / 127, round to nearest with ties away, fp16 scale by the
// host's rule; score = int8 dot x both scales; split-K online softmax; merge of the splits).
//
// Layout (unchanged, it is the format, src/kv_cache.h:35-46): head-major, K and V separate,
// block[((layer * n_kv_head + kv_head) * capacity + pos) * 8 + blk], 34-byte blocks -- the 8 blocks of a position are
// 272 contiguous bytes, consecutive positions follow each other, so a run of positions of one (layer, kv head) is ONE
// contiguous, 16-byte aligned span.
//
// Decode on B200: one CTA per (kv head, split of the positions) serves the SIX query heads that share the kv head
// (grouped-query attention), so K and V cross HBM once per group, not once per query head.  Tiles of 32 positions
// (8.7 KB of K, 8.7 KB of V) arrive by bulk async copy into a two-deep ring; the CTA dequantises the V tile to fp32
// once for its six warps; warp w = query head w of the group: lane = position for the scores (64 dp4a per lane
// against the query's int8 words in registers), tile-wise online softmax, then lane = 8 output dimensions for the
// value sum.  The query heads are quantised in the kernel's prologue (no separate launch, no buffer).  Partial
// (m, l, acc) per (head, split) go to a workspace; a second kernel merges the splits (src/kv_cache.h:153-170).
#pragma once

#include "common.cuh"

namespace b200 {

constexpr int KV_D = 256, KV_NBLK = 8, KV_ROW = KV_NBLK * 34;      // 272 bytes per position and head
constexpr int KV_TILE = 32;                                          // positions per tile
constexpr int KV_WS = KV_D + 8;                                      // workspace floats per (head, split): acc, m, l, pad (16-byte rows)
constexpr int KV_MAX_GROUP = 8;                                      // query heads per kv head the kernel is built for

// ---- Q8_0 row quantiser: 4 lanes per 32-value block, 8 values per lane ---------------------------------------------
// Bytes equal kv_quantize_row_q8_0 (src/kv_cache.h:100-117).  (The reference's device kernels give a lane 4 values,
// which covers only half of every block, src/kernels/kv_p40.cu:47-51,72; the host function is the one followed.)
__device__ __forceinline__ void kv_quantise_8(const float (&x)[8], float &d_out, uint32_t (&word)[2]) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(x[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const float d = __fdiv_rn(amax, 127.0f);
    const float id = d > 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    word[0] = word[1] = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int v = round_ties_away(__fmul_rn(x[i], id));
        v = max(-127, min(127, v));
        word[i >> 2] |= ((uint32_t)v & 0xFFu) << (8 * (i & 3));
    }
    d_out = d;
}

// One warp per (token, kv head) row of K and of V: lane = (block lane / 4, eight dims).
__global__ void __launch_bounds__(256) kv_append_kernel(uint8_t *__restrict__ K, uint8_t *__restrict__ V,
                                                        const float *__restrict__ ksrc, const float *__restrict__ vsrc,
                                                        int pos0, int n_tok, int n_kv_head, int capacity, int layer) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);        // token * n_kv_head + head
    if (row >= n_tok * n_kv_head) return;
    const int tok = row / n_kv_head, h = row - tok * n_kv_head;
    const int blk = lane >> 2, sub = lane & 3;
    const size_t base = ((((size_t)layer * n_kv_head + h) * capacity + (size_t)(pos0 + tok)) * KV_NBLK + blk) * 34;
    const float *kr = ksrc + (size_t)row * KV_D + blk * 32 + sub * 8;
    const float *vr = vsrc + (size_t)row * KV_D + blk * 32 + sub * 8;
    float kx[8], vx[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { kx[i] = kr[i]; vx[i] = vr[i]; }
    float kd, vd;
    uint32_t kw[2], vw[2];
    kv_quantise_8(kx, kd, kw);
    kv_quantise_8(vx, vd, vw);
    // blocks start on 2-byte boundaries: halfword stores (scale, then this lane's 8 bytes)
    unsigned short *kp = reinterpret_cast<unsigned short *>(K + base), *vp = reinterpret_cast<unsigned short *>(V + base);
    if (sub == 0) {
        kp[0] = (unsigned short)f32_to_f16_bits_ties_away(kd);
        vp[0] = (unsigned short)f32_to_f16_bits_ties_away(vd);
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        kp[1 + 4 * sub + 2 * j] = (unsigned short)(kw[j] & 0xFFFFu); kp[2 + 4 * sub + 2 * j] = (unsigned short)(kw[j] >> 16);
        vp[1 + 4 * sub + 2 * j] = (unsigned short)(vw[j] & 0xFFFFu); vp[2 + 4 * sub + 2 * j] = (unsigned short)(vw[j] >> 16);
    }
}

__device__ __forceinline__ int dp4a_ss(int a, int b, int c) {
    int r;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}

// grid (n_split, n_kv_head), block grp * 32 threads (warp w = query head kvh * grp + w).
// Workspace per (head, split): [256 acc][m][l][6 pad].
__global__ void __launch_bounds__(KV_MAX_GROUP * 32) kv_attn_split_kernel(const float *__restrict__ q, const uint8_t *__restrict__ K,
                                                                          const uint8_t *__restrict__ V, float *__restrict__ ws,
                                                                          int pos, int n_split, int n_kv_head, int capacity,
                                                                          int layer, float scale, int grp) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);                         // [2]
    uint8_t *kraw = smem + 128;                                                  // [2][32 x 272]
    uint8_t *vraw = kraw + 2 * KV_TILE * KV_ROW;                                 // [2][32 x 272]
    float *vf = reinterpret_cast<float *>(vraw + 2 * KV_TILE * KV_ROW);          // [32][256] the current tile's values
    uint32_t *q8 = reinterpret_cast<uint32_t *>(vf + KV_TILE * KV_D);            // [grp][8 blocks][8 words]
    float *qd = reinterpret_cast<float *>(q8 + KV_MAX_GROUP * 64);               // [grp][8] scales x `scale`

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int split = blockIdx.x, kvh = blockIdx.y, head = kvh * grp + warp;
    const int n_pos = pos + 1;
    const int chunk = (((n_pos + n_split - 1) / n_split) + KV_TILE - 1) / KV_TILE * KV_TILE;   // whole tiles per split
    const int p_begin = split * chunk, p_end = min(p_begin + chunk, n_pos);
    const int ntiles = p_end > p_begin ? (p_end - p_begin + KV_TILE - 1) / KV_TILE : 0;
    const uint8_t *kbase = K + (((size_t)layer * n_kv_head + kvh) * capacity) * KV_ROW;
    const uint8_t *vbase = V + (((size_t)layer * n_kv_head + kvh) * capacity) * KV_ROW;
    const uint64_t pol = policy_evict_first();

    auto issue = [&](int t) {           // one thread
        const int p0 = p_begin + t * KV_TILE, n = min(KV_TILE, p_end - p0);
        const uint32_t bytes = (uint32_t)n * KV_ROW;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_expect_tx(&full[t & 1], 2 * bytes);
        bulk_g2s(kraw + (size_t)(t & 1) * KV_TILE * KV_ROW, kbase + (size_t)p0 * KV_ROW, bytes, &full[t & 1], pol);
        bulk_g2s(vraw + (size_t)(t & 1) * KV_TILE * KV_ROW, vbase + (size_t)p0 * KV_ROW, bytes, &full[t & 1], pol);
    };
    if (threadIdx.x == 0) {
        mbar_init(&full[0], 1);
        mbar_init(&full[1], 1);
        mbar_fence_init();
        if (ntiles > 0) issue(0);
    }
    // the group's query heads, quantised as the cache rows are (host rule, src/kv_cache.h:100-117)
    {
        const int blk = lane >> 2, sub = lane & 3;
        const float *qr = q + (size_t)head * KV_D + blk * 32 + sub * 8;
        float x[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = qr[i];
        float d;
        uint32_t w[2];
        kv_quantise_8(x, d, w);
        q8[(warp * 8 + blk) * 8 + 2 * sub] = w[0];
        q8[(warp * 8 + blk) * 8 + 2 * sub + 1] = w[1];
        if (sub == 0) qd[warp * 8 + blk] = __fmul_rn(f16_bits_to_f32(f32_to_f16_bits_ties_away(d)), scale);
    }
    __syncthreads();
    float m = -INFINITY, l = 0.0f;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.0f;

    for (int t = 0; t < ntiles; ++t) {
        if (threadIdx.x == 0 && t + 1 < ntiles) issue(t + 1);       // its buffer was released by the barrier that ended tile t - 1
        // (the outcome of the bounded wait is made uniform: a CTA either goes on as a whole or leaves as a whole)
        if (!__syncthreads_and(mbar_wait_bounded(&full[t & 1], (uint32_t)((t >> 1) & 1)) ? 1 : 0)) break;
        const uint8_t *kt = kraw + (size_t)(t & 1) * KV_TILE * KV_ROW;
        const uint8_t *vt = vraw + (size_t)(t & 1) * KV_TILE * KV_ROW;
        const int n = min(KV_TILE, p_end - (p_begin + t * KV_TILE));
        // the tile's values as fp32, once for all query heads: thread i takes (position, block) pairs
        for (int i = threadIdx.x; i < n * KV_NBLK; i += blockDim.x) {
            const int p = i >> 3, b = i & 7;
            const unsigned short *src = reinterpret_cast<const unsigned short *>(vt + (size_t)p * KV_ROW + b * 34);
            const float dv = f16_bits_to_f32(src[0]);
            float *dst = vf + p * KV_D + b * 32;
#pragma unroll
            for (int h2 = 0; h2 < 16; ++h2) {
                const unsigned short two = src[1 + h2];
                dst[2 * h2] = __fmul_rn((float)(int)(signed char)(two & 0xFF), dv);
                dst[2 * h2 + 1] = __fmul_rn((float)(int)(signed char)(two >> 8), dv);
            }
        }
        // scores: lane = position
        float s = -INFINITY;
        if (lane < n) {
            const unsigned short *kr = reinterpret_cast<const unsigned short *>(kt + (size_t)lane * KV_ROW);
            float sc = 0.0f;
#pragma unroll
            for (int b = 0; b < KV_NBLK; ++b) {
                const unsigned short *kb = kr + 17 * b;
                int sumi = 0;
#pragma unroll
                for (int w = 0; w < 8; ++w) {
                    const int kw = (int)((uint32_t)kb[1 + 2 * w] | ((uint32_t)kb[2 + 2 * w] << 16));
                    sumi = dp4a_ss((int)q8[(warp * 8 + b) * 8 + w], kw, sumi);
                }
                sc = __fadd_rn(sc, __fmul_rn(__fmul_rn(qd[warp * 8 + b], f16_bits_to_f32(kb[0])), (float)sumi));
            }
            s = sc;
        }
        // tile-wise online softmax
        float tmax = s;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
        const float m_new = fmaxf(m, tmax);
        const float alpha = expf(__fsub_rn(m, m_new));
        const float pw = lane < n ? expf(__fsub_rn(s, m_new)) : 0.0f;
        float psum = pw;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) psum = __fadd_rn(psum, __shfl_xor_sync(0xffffffffu, psum, o));
        l = __fadd_rn(__fmul_rn(l, alpha), psum);
        m = m_new;
        __syncthreads();                                            // the fp32 value tile is complete
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = __fmul_rn(acc[i], alpha);
        for (int p = 0; p < n; ++p) {
            const float wp = __shfl_sync(0xffffffffu, pw, p);
            const float4 a = *reinterpret_cast<const float4 *>(vf + p * KV_D + 8 * lane);
            const float4 b = *reinterpret_cast<const float4 *>(vf + p * KV_D + 8 * lane + 4);
            acc[0] = __fmaf_rn(wp, a.x, acc[0]); acc[1] = __fmaf_rn(wp, a.y, acc[1]);
            acc[2] = __fmaf_rn(wp, a.z, acc[2]); acc[3] = __fmaf_rn(wp, a.w, acc[3]);
            acc[4] = __fmaf_rn(wp, b.x, acc[4]); acc[5] = __fmaf_rn(wp, b.y, acc[5]);
            acc[6] = __fmaf_rn(wp, b.z, acc[6]); acc[7] = __fmaf_rn(wp, b.w, acc[7]);
        }
        __syncthreads();                                            // tile t's buffers (raw and fp32) may be overwritten
    }
    float *slot = ws + ((size_t)head * n_split + split) * KV_WS;
    *reinterpret_cast<float4 *>(slot + 8 * lane) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4 *>(slot + 8 * lane + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    if (lane == 0) { slot[KV_D] = m; slot[KV_D + 1] = l; }
}

// Merge of the splits and normalisation (src/kv_cache.h:153-176): one warp per query head, lane = 8 dims.
__global__ void __launch_bounds__(32) kv_attn_combine_kernel(const float *__restrict__ ws, float *__restrict__ out, int n_split) {
    const int lane = threadIdx.x & 31, head = blockIdx.x;
    float m = -INFINITY, l = 0.0f;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
    for (int s = 0; s < n_split; ++s) {
        const float *slot = ws + ((size_t)head * n_split + s) * KV_WS;
        const float sm = slot[KV_D], sl = slot[KV_D + 1];
        if (sl == 0.0f) continue;                                   // a split without positions
        const float mn = fmaxf(m, sm);
        const float wa = expf(__fsub_rn(m, mn)), wb = expf(__fsub_rn(sm, mn));
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = __fadd_rn(__fmul_rn(acc[i], wa), __fmul_rn(slot[8 * lane + i], wb));
        l = __fadd_rn(__fmul_rn(l, wa), __fmul_rn(sl, wb));
        m = mn;
    }
    const float inv = __fdiv_rn(1.0f, l);
#pragma unroll
    for (int i = 0; i < 8; ++i) out[(size_t)head * KV_D + 8 * lane + i] = __fmul_rn(acc[i], inv);
}

}  // namespace b200
