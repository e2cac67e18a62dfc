// ops.cuh -- the three entry points of the reference ABI that sit beside the mat-vec path: RMSNorm, the gated
// delta-net recurrent step and causal attention (include/bonsai_p40.h:44-56 in the reference).
//
// Oracles: src/ops.h:13-22 (rmsnorm), :66-92 (gdn_step) and the online-softmax recurrence of
// src/kernels/attn_p40.cu:92-118 / tests/test_p40.cpp:240-262.  The host code adds long sums sequentially and calls
// the C library's expf; the kernels add in a fixed tree order and use the device's expf, so outputs are held to
// 1e-5 of the largest output (the reference's own tests use 1e-4), not to the bit.
#pragma once

#include "activation.cuh"
#include "common.cuh"

namespace b200 {

// ---- sum of squares in the library's canonical order ------------------------------------------------------------
// A vector is cut into slices of 128 floats; inside a slice lane l adds x[4l]^2 .. x[4l+3]^2 in that order and a
// 5-step butterfly joins the lanes; slices are added in ascending order.  The fused producer of the list kernel
// (gemv_chain.cuh) uses the same order, so a fused RMSNorm gives the bits of this kernel.
__device__ __forceinline__ float slice_sumsq(float4 f) {
    float s = __fmul_rn(f.x, f.x);
    s = __fadd_rn(s, __fmul_rn(f.y, f.y));
    s = __fadd_rn(s, __fmul_rn(f.z, f.z));
    s = __fadd_rn(s, __fmul_rn(f.w, f.w));
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, o));
    return s;
}
// 1 / sqrt(ss / n + eps), every step one IEEE operation (src/ops.h:13-17).
__device__ __forceinline__ float rms_scale(float ss, int n, float eps) {
    return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)n), eps)));
}
// silu(g) * u (src/ops.h:27-31); expf is the device's, not the host library's.
__device__ __forceinline__ float swiglu1(float g, float u) {
    return __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), u);
}

__global__ void __launch_bounds__(256) swiglu_kernel(const float *__restrict__ gate, const float *__restrict__ up,
                                                     float *__restrict__ y, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = swiglu1(gate[i], up[i]);
}

// One CTA per row, n % 128 == 0 handled by whole slices (VEC: 16-byte loads), any n by the scalar tail path.
template <bool VEC>
__global__ void __launch_bounds__(256) rmsnorm_kernel(const float *__restrict__ x, const float *__restrict__ w,
                                                      float *__restrict__ y, int n, float eps) {
    __shared__ float part[512];
    __shared__ float scale;
    const float *xr = x + (size_t)blockIdx.x * n;
    float *yr = y + (size_t)blockIdx.x * n;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int nslice = (n + 127) >> 7;
    float acc = 0.0f;                               // rows longer than 512 slices: a warp adds its slices in ascending order
    for (int s0 = 0; s0 < nslice; s0 += 512) {
        for (int sl = s0 + wid; sl < min(nslice, s0 + 512); sl += nw) {
            const int i = sl * 128 + 4 * lane;
            float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
            if (VEC) {
                if (i + 3 < n) f = *reinterpret_cast<const float4 *>(xr + i);
            } else {
                if (i < n) f.x = xr[i];
                if (i + 1 < n) f.y = xr[i + 1];
                if (i + 2 < n) f.z = xr[i + 2];
                if (i + 3 < n) f.w = xr[i + 3];
            }
            const float s = slice_sumsq(f);
            if (lane == 0) part[sl - s0] = s;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int k = 0; k < min(512, nslice - s0); ++k) acc = __fadd_rn(acc, part[k]);
            scale = rms_scale(acc, n, eps);
        }
        __syncthreads();
    }
    const float sc = scale;
    for (int i = threadIdx.x; i < n; i += blockDim.x) yr[i] = __fmul_rn(__fmul_rn(xr[i], sc), w[i]);
}

// ---- gated delta-net step ------------------------------------------------------------------------------------------
// state [n_v_heads][K][V]; one CTA per (value head, 32 state columns), 8 warps: lane = column, warp w holds rows
// w, w + 8, ... of the column in registers, so the state is read once and written once (2 * K * V * 4 bytes per head,
// the floor) and every access is a coalesced 128-byte row segment.  The column sums (k . S and q . S) are formed per
// warp over its rows in ascending order and joined across the warps in ascending warp order: a fixed order, not the
// host's strictly sequential one (src/ops.h:66-92) -- within the 1e-5 this operator is held to.  (A thread per whole
// column kept 128 values in registers and left 6144 threads for a 3 MB state: 45 us per call; this shape: see profiles.)
constexpr int GDN_KMAX = 128, GDN_WARPS = 8, GDN_RPW = GDN_KMAX / GDN_WARPS;
__global__ void __launch_bounds__(GDN_WARPS * 32) gdn_step_kernel(float *__restrict__ state, const float *__restrict__ q,
                                                                  const float *__restrict__ k, const float *__restrict__ v,
                                                                  const float *__restrict__ g, const float *__restrict__ beta,
                                                                  float *__restrict__ out, int n_k_heads, int n_v_heads, int K, int V) {
    __shared__ float ks[GDN_KMAX], qs[GDN_KMAX];
    __shared__ float part[GDN_WARPS][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tiles = V / 32;
    const int vh = blockIdx.x / tiles, vt = blockIdx.x - vh * tiles;
    const int j = vt * 32 + lane;
    const int kh = vh / (n_v_heads / n_k_heads);
    for (int i = threadIdx.x; i < K; i += blockDim.x) {
        ks[i] = k[(size_t)kh * K + i];
        qs[i] = q[(size_t)kh * K + i];
    }
    float *Sg = state + (size_t)vh * K * V + j;
    const float decay = expf(g[vh]);
    float col[GDN_RPW];
#pragma unroll
    for (int r = 0; r < GDN_RPW; ++r) {
        const int i = warp + GDN_WARPS * r;
        col[r] = i < K ? Sg[(size_t)i * V] : 0.0f;
    }
    __syncthreads();
    float kv = 0.0f;
#pragma unroll
    for (int r = 0; r < GDN_RPW; ++r) {
        const int i = warp + GDN_WARPS * r;
        if (i < K) {
            col[r] = __fmul_rn(col[r], decay);
            kv = __fadd_rn(kv, __fmul_rn(ks[i], col[r]));
        }
    }
    part[warp][lane] = kv;
    __syncthreads();
    kv = 0.0f;
#pragma unroll
    for (int w = 0; w < GDN_WARPS; ++w) kv = __fadd_rn(kv, part[w][lane]);
    __syncthreads();                                    // part is reused below
    const float b = beta[vh];
    const float d = __fsub_rn(v[(size_t)vh * V + j], kv);
    float o = 0.0f;
#pragma unroll
    for (int r = 0; r < GDN_RPW; ++r) {
        const int i = warp + GDN_WARPS * r;
        if (i < K) {
            col[r] = __fadd_rn(col[r], __fmul_rn(__fmul_rn(b, ks[i]), d));
            o = __fadd_rn(o, __fmul_rn(qs[i], col[r]));
            Sg[(size_t)i * V] = col[r];
        }
    }
    part[warp][lane] = o;
    __syncthreads();
    if (warp == 0) {
        o = 0.0f;
#pragma unroll
        for (int w = 0; w < GDN_WARPS; ++w) o = __fadd_rn(o, part[w][lane]);
        out[(size_t)vh * V + j] = o;
    }
}

// ---- causal attention, head_dim 256 ------------------------------------------------------------------------------
// One warp per (head, query); lane l owns dimensions 8l .. 8l+7.  The eight warps of a CTA take eight consecutive
// queries of ONE head, so they walk the same keys and values: a tile of 16 keys (K and V rows, 32 KB) is staged in
// shared memory once per CTA and read by all eight warps.  Online softmax in the order of the reference's kernel
// (src/kernels/attn_p40.cu:101-113): one key at a time, running maximum, rescale, accumulate.
constexpr int ATT_D = 256, ATT_TILE = 16, ATT_WARPS = 8;
__global__ void __launch_bounds__(ATT_WARPS * 32) attn_kernel(const float *__restrict__ q, const float *__restrict__ k,
                                                              const float *__restrict__ v, float *__restrict__ out,
                                                              int n_tok, int n_head, int n_head_kv, float scale) {
    __shared__ __align__(16) float kt[ATT_TILE][ATT_D];
    __shared__ __align__(16) float vt[ATT_TILE][ATT_D];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int qblocks = (n_tok + ATT_WARPS - 1) / ATT_WARPS;
    const int head = blockIdx.x / qblocks, qb = blockIdx.x - head * qblocks;
    const int qi = qb * ATT_WARPS + warp;
    const int kvh = head / (n_head / n_head_kv);
    const bool live = qi < n_tok;
    float qreg[8], oreg[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { qreg[i] = 0.0f; oreg[i] = 0.0f; }
    if (live) {
        const float *qp = q + ((size_t)qi * n_head + head) * ATT_D + 8 * lane;
#pragma unroll
        for (int i = 0; i < 8; ++i) qreg[i] = __fmul_rn(qp[i], scale);
    }
    float m = -INFINITY, l = 0.0f;
    const int last = min(n_tok - 1, qb * ATT_WARPS + ATT_WARPS - 1);        // keys 0 .. last serve the CTA's queries
    for (int j0 = 0; j0 <= last; j0 += ATT_TILE) {
        __syncthreads();
        const int nk = min(ATT_TILE, last + 1 - j0);
        for (int i = threadIdx.x; i < nk * (ATT_D / 4); i += blockDim.x) {
            const int r = i / (ATT_D / 4), c4 = i - r * (ATT_D / 4);
            const size_t src = ((size_t)(j0 + r) * n_head_kv + kvh) * ATT_D + 4 * c4;
            *reinterpret_cast<float4 *>(&kt[r][4 * c4]) = *reinterpret_cast<const float4 *>(k + src);
            *reinterpret_cast<float4 *>(&vt[r][4 * c4]) = *reinterpret_cast<const float4 *>(v + src);
        }
        __syncthreads();
        if (!live) continue;
        for (int r = 0; r < nk && j0 + r <= qi; ++r) {
            float part = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) part = __fadd_rn(part, __fmul_rn(qreg[i], kt[r][8 * lane + i]));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) part = __fadd_rn(part, __shfl_xor_sync(0xffffffffu, part, o));
            const float m_new = fmaxf(m, part);
            const float alpha = expf(__fsub_rn(m, m_new));
            const float p = expf(__fsub_rn(part, m_new));
            l = __fadd_rn(__fmul_rn(l, alpha), p);
#pragma unroll
            for (int i = 0; i < 8; ++i) oreg[i] = __fadd_rn(__fmul_rn(oreg[i], alpha), __fmul_rn(p, vt[r][8 * lane + i]));
            m = m_new;
        }
    }
    if (live) {
        const float inv = __fdiv_rn(1.0f, l);
        float *op = out + ((size_t)qi * n_head + head) * ATT_D + 8 * lane;
#pragma unroll
        for (int i = 0; i < 8; ++i) op[i] = __fmul_rn(oreg[i], inv);
    }
}

}  // namespace b200
