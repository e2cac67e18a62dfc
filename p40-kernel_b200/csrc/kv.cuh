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
// (8.7 KB of K, 8.7 KB of V) arrive by bulk async copy into a four-deep ring; warp w = query head w of the group for
// the scores (int8 dot products against the query's int8 words in registers, tile-wise online softmax) and = every
// sixth position for the value sum, where a dequantised V row is added into the accumulators of all six heads.  The
// query heads are quantised in the kernel's prologue (no separate launch, no buffer).  Partial (m, l, acc) per
// (head, split) go to a workspace; a second kernel merges the splits (src/kv_cache.h:153-170).
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

// grid (n_split, n_kv_head), block grp * 32 threads.  Workspace per (head, split): [256 acc][m][l][6 pad].
// Per tile of 32 positions:
//   scores   warp w = query head w of the group.  Four lanes share a position and each reads a 68-byte piece of the K
//            row (17 words: two blocks), eight positions per pass: a warp's loads are one contiguous run (a lane per
//            position at a row stride of 272 bytes met 4-way bank conflicts on every load).  Tile-wise online softmax;
//            the head's 32 weights and its rescale factor go to a small table in shared memory.
//   values   warp w takes the positions p = w, w + grp, ...: it dequantises the V row once (lane = 8 dims, straight from
//            the raw bytes) and adds it into the accumulators of ALL heads of the group, so the value tile is read from
//            shared memory once, not once per head, and no fp32 copy of it is made (a thread per (position, block)
//            writing that copy met a 32-way conflict on every store).  The warps' partial sums meet once, at the end.
constexpr int KV_BUFS = 4;                                           // raw tiles in flight per CTA
constexpr int KV_TILE_BYTES = 2 * KV_TILE * KV_ROW;                  // K tile, then V tile
constexpr int KV_SPLIT_SMEM_BYTES = 128 + KV_BUFS * KV_TILE_BYTES + KV_MAX_GROUP * 64 * 4 + KV_MAX_GROUP * 8 * 4 +
                                    KV_MAX_GROUP * (KV_TILE + 8) * 4;
static_assert(KV_BUFS * KV_TILE_BYTES >= KV_MAX_GROUP * KV_MAX_GROUP * KV_D * 4, "the final meeting reuses the raw buffers");
template <int GRP>
__global__ void __launch_bounds__(GRP * 32) kv_attn_split_kernel(const float *__restrict__ q, const uint8_t *__restrict__ K,
                                                                 const uint8_t *__restrict__ V, float *__restrict__ ws,
                                                                 int pos, int n_split, int n_kv_head, int capacity,
                                                                 int layer, float scale) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);                         // [KV_BUFS]
    uint8_t *raw = smem + 128;                                                   // [KV_BUFS][K tile | V tile]
    uint32_t *q8 = reinterpret_cast<uint32_t *>(raw + KV_BUFS * KV_TILE_BYTES);  // [grp][8 blocks][8 words]
    float *qd = reinterpret_cast<float *>(q8 + KV_MAX_GROUP * 64);               // [grp][8] scales x `scale`
    float *pwt = qd + KV_MAX_GROUP * 8;                                          // [grp][32 weights, rescale factor, 7 pad]

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int split = blockIdx.x, kvh = blockIdx.y, head = kvh * GRP + warp;
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
        uint8_t *dst = raw + (size_t)(t % KV_BUFS) * KV_TILE_BYTES;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_expect_tx(&full[t % KV_BUFS], 2 * bytes);
        bulk_g2s(dst, kbase + (size_t)p0 * KV_ROW, bytes, &full[t % KV_BUFS], pol);
        bulk_g2s(dst + KV_TILE * KV_ROW, vbase + (size_t)p0 * KV_ROW, bytes, &full[t % KV_BUFS], pol);
    };
    if (threadIdx.x == 0) {
        for (int b = 0; b < KV_BUFS; ++b) mbar_init(&full[b], 1);
        mbar_fence_init();
        for (int t = 0; t < min(ntiles, KV_BUFS - 1); ++t) issue(t);
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
    // scores: lane = (position of the pass, quarter of the row); the quarter's two query blocks stay in registers
    const int pp = lane >> 2, sub = lane & 3;
    uint32_t qw[2][8];
    float qs[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int w = 0; w < 8; ++w) qw[j][w] = q8[(warp * 8 + 2 * sub + j) * 8 + w];
        qs[j] = qd[warp * 8 + 2 * sub + j];
    }
    float m = -INFINITY, l = 0.0f;              // of this warp's head
    float acc[GRP][8];                          // of this warp's positions, every head of the group
#pragma unroll
    for (int h = 0; h < GRP; ++h)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[h][i] = 0.0f;

    for (int t = 0; t < ntiles; ++t) {
        // buffer (t - 1) % KV_BUFS was released by the barrier that ended tile t - 1
        if (threadIdx.x == 0 && t + KV_BUFS - 1 < ntiles) issue(t + KV_BUFS - 1);
        // (the outcome of the bounded wait is made uniform: a CTA either goes on as a whole or leaves as a whole)
        if (!__syncthreads_and(mbar_wait_bounded(&full[t % KV_BUFS], (uint32_t)((t / KV_BUFS) & 1)) ? 1 : 0)) break;
        const uint8_t *kt = raw + (size_t)(t % KV_BUFS) * KV_TILE_BYTES;
        const uint8_t *vt = kt + KV_TILE * KV_ROW;
        const int n = min(KV_TILE, p_end - (p_begin + t * KV_TILE));
        // scores of the tile's 32 positions in four passes of eight
        float s[4];
#pragma unroll
        for (int ps = 0; ps < 4; ++ps) {
            const int p = 8 * ps + pp;
            float part = 0.0f;
            if (p < n) {
                // the quarter's 68 bytes = 17 words: block 2 sub (scale in the low half of word 0, its int8 from byte 2)
                // and block 2 sub + 1 (scale in the high half of word 8, its int8 from word 9)
                const uint32_t *kw = reinterpret_cast<const uint32_t *>(kt + (size_t)p * KV_ROW + 68 * sub);
                uint32_t L[17];
#pragma unroll
                for (int i = 0; i < 17; ++i) L[i] = kw[i];
                int s0 = 0, s1 = 0;
#pragma unroll
                for (int w = 0; w < 8; ++w) {
                    s0 = dp4a_ss((int)qw[0][w], (int)__funnelshift_r(L[w], L[w + 1], 16), s0);
                    s1 = dp4a_ss((int)qw[1][w], (int)L[9 + w], s1);
                }
                part = __fmul_rn(__fmul_rn(qs[0], f16_bits_to_f32(L[0] & 0xFFFFu)), (float)s0);
                part = __fadd_rn(part, __fmul_rn(__fmul_rn(qs[1], f16_bits_to_f32(L[8] >> 16)), (float)s1));
            }
            part = __fadd_rn(part, __shfl_xor_sync(0xffffffffu, part, 1));
            part = __fadd_rn(part, __shfl_xor_sync(0xffffffffu, part, 2));
            s[ps] = p < n ? part : -INFINITY;
        }
        // tile-wise online softmax (every lane of a quad holds the same four scores)
        float tmax = fmaxf(fmaxf(s[0], s[1]), fmaxf(s[2], s[3]));
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
        const float m_new = fmaxf(m, tmax);
        const float alpha = expf(__fsub_rn(m, m_new));
        float psum = 0.0f;
#pragma unroll
        for (int ps = 0; ps < 4; ++ps) {
            const float w = 8 * ps + pp < n ? expf(__fsub_rn(s[ps], m_new)) : 0.0f;
            if (sub == 0) pwt[warp * (KV_TILE + 8) + 8 * ps + pp] = w;
            psum = __fadd_rn(psum, w);
        }
        if (lane == 0) pwt[warp * (KV_TILE + 8) + KV_TILE] = alpha;
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) psum = __fadd_rn(psum, __shfl_xor_sync(0xffffffffu, psum, o));
        l = __fadd_rn(__fmul_rn(l, alpha), psum);
        m = m_new;
        __syncthreads();                                            // every head's weights of this tile are in the table
#pragma unroll
        for (int h = 0; h < GRP; ++h) {
            const float al = pwt[h * (KV_TILE + 8) + KV_TILE];
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[h][i] = __fmul_rn(acc[h][i], al);
        }
        for (int p = warp; p < n; p += GRP) {
            const unsigned short *src = reinterpret_cast<const unsigned short *>(vt + (size_t)p * KV_ROW + (lane >> 2) * 34);
            const float dv = f16_bits_to_f32(src[0]);
            const unsigned short *b8 = src + 1 + 4 * (lane & 3);
            // int8 -> fp32 without the conversion unit: the byte, with its sign bit flipped (value + 128), is placed under
            // the exponent of 2^23 by a byte permute, and 2^23 + 128 is subtracted: exact
            float v[8];
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
                const uint32_t four = ((uint32_t)b8[2 * h2] | ((uint32_t)b8[2 * h2 + 1] << 16)) ^ 0x80808080u;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float f = __uint_as_float(__byte_perm(four, 0x4B000000u, 0x7440u + (uint32_t)e));
                    v[4 * h2 + e] = __fmul_rn(__fsub_rn(f, 8388736.0f), dv);
                }
            }
#pragma unroll
            for (int h = 0; h < GRP; ++h) {
                const float wp = pwt[h * (KV_TILE + 8) + p];
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[h][i] = __fmaf_rn(wp, v[i], acc[h][i]);
            }
        }
        __syncthreads();                                            // tile t's buffer and the table may be overwritten
    }
    // the warps' partial sums meet: red[warp][head][256] over the raw buffers (nothing is in flight any more)
    float *red = reinterpret_cast<float *>(raw);
#pragma unroll
    for (int h = 0; h < GRP; ++h) {
        float4 *dst = reinterpret_cast<float4 *>(red + ((size_t)warp * GRP + h) * KV_D + 8 * lane);
        dst[0] = make_float4(acc[h][0], acc[h][1], acc[h][2], acc[h][3]);
        dst[1] = make_float4(acc[h][4], acc[h][5], acc[h][6], acc[h][7]);
    }
    __syncthreads();
    float o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = 0.0f;
#pragma unroll
    for (int w = 0; w < GRP; ++w) {             // this warp's head, the warps in ascending order
        const float4 *srcp = reinterpret_cast<const float4 *>(red + ((size_t)w * GRP + warp) * KV_D + 8 * lane);
        const float4 a = srcp[0], b = srcp[1];
        o[0] = __fadd_rn(o[0], a.x); o[1] = __fadd_rn(o[1], a.y); o[2] = __fadd_rn(o[2], a.z); o[3] = __fadd_rn(o[3], a.w);
        o[4] = __fadd_rn(o[4], b.x); o[5] = __fadd_rn(o[5], b.y); o[6] = __fadd_rn(o[6], b.z); o[7] = __fadd_rn(o[7], b.w);
    }
    float *slot = ws + ((size_t)head * n_split + split) * KV_WS;
    *reinterpret_cast<float4 *>(slot + 8 * lane) = make_float4(o[0], o[1], o[2], o[3]);
    *reinterpret_cast<float4 *>(slot + 8 * lane + 4) = make_float4(o[4], o[5], o[6], o[7]);
    if (lane == 0) { slot[KV_D] = m; slot[KV_D + 1] = l; }
}

// Merge of the splits and normalisation (src/kv_cache.h:153-176): one CTA per query head, thread = output dimension.
// The weights exp(m_s - max) of the splits are formed once in shared memory; every thread then adds its dimension
// over the splits with independent, coalesced loads (a single warp walking the splits one dependent load after the
// other took 65 us at 64 splits).
constexpr int KV_COMBINE_MAX = 256;
__global__ void __launch_bounds__(KV_D) kv_attn_combine_kernel(const float *__restrict__ ws, float *__restrict__ out, int n_split) {
    __shared__ float wgt[KV_COMBINE_MAX];
    __shared__ float red[2];
    const int head = blockIdx.x, d = threadIdx.x;
    const float *base = ws + (size_t)head * n_split * KV_WS;
    if (d < 32) {                                                   // one warp: maximum, weights, denominator
        float mx = -INFINITY;
        for (int s = d; s < n_split; s += 32)
            if (base[(size_t)s * KV_WS + KV_D + 1] != 0.0f) mx = fmaxf(mx, base[(size_t)s * KV_WS + KV_D]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float lsum = 0.0f;
        for (int s = d; s < n_split; s += 32) {
            const float sl = base[(size_t)s * KV_WS + KV_D + 1];
            const float w = sl != 0.0f ? expf(__fsub_rn(base[(size_t)s * KV_WS + KV_D], mx)) : 0.0f;   // a split without positions: 0
            wgt[s] = w;
            lsum = __fadd_rn(lsum, __fmul_rn(sl, w));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) lsum = __fadd_rn(lsum, __shfl_xor_sync(0xffffffffu, lsum, o));
        if (d == 0) red[0] = lsum;
    }
    __syncthreads();
    float a = 0.0f;
#pragma unroll 8
    for (int s = 0; s < n_split; ++s) a = __fmaf_rn(base[(size_t)s * KV_WS + d], wgt[s], a);
    out[(size_t)head * KV_D + d] = __fmul_rn(a, __fdiv_rn(1.0f, red[0]));
}

}  // namespace b200
