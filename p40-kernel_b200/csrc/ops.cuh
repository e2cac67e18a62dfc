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
// column kept 128 values in registers and left 6144 threads for a 3 MB state: 45 us per call against 4 us for this shape.)
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
// A warp owns FOUR consecutive queries of a head; lane l owns dimensions 8l .. 8l+7 of q and of the outputs.  The eight
// warps of a CTA take 32 consecutive queries of ONE head, so they walk the same keys and values: a tile of 32 keys (K
// and V rows, 64 KB) is staged in shared memory once per CTA, and every row a warp reads from it serves four queries
// (with one query per warp the kernel was bound by shared-memory bandwidth: 2 KB read per (query, key)).  Scores: for
// eight keys at a time the lanes' partial dot products of the 4 x 8 (query, key) pairs go through one transposing
// reduction (31 shuffles for 32 scores instead of 5 per score), which leaves lane (query, key) with its score.  The
// softmax step is taken a tile at a time -- one running maximum, one rescale and four exps per lane per 32 keys: the
// online softmax of the reference's kernel (src/kernels/attn_p40.cu:101-113) with 32 keys per step instead of one.
// fp32 on the CUDA cores throughout; outputs are held to 1e-5 of the largest output.
constexpr int ATT_D = 256, ATT_TILE = 32, ATT_WARPS = 8, ATT_QPW = 4, ATT_QPC = ATT_WARPS * ATT_QPW;
constexpr int ATT_SMEM_BYTES = 2 * ATT_TILE * ATT_D * 4;

// part[r] of every lane -> returned value of lane r = sum over the lanes of part[r] (r = 0 .. 31).
__device__ __forceinline__ float transpose_sum32(float (&part)[32], int lane) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const bool up = (lane & o) != 0;
#pragma unroll
        for (int i = 0; i < o; ++i) {
            // the lane keeps the half of the values whose index has bit `o` equal to its own, and takes the partner's
            const float keep = up ? part[i + o] : part[i], give = up ? part[i] : part[i + o];
            part[i] = __fadd_rn(keep, __shfl_xor_sync(0xffffffffu, give, o));
        }
    }
    return part[0];
}

__global__ void __launch_bounds__(ATT_WARPS * 32) attn_kernel(const float *__restrict__ q, const float *__restrict__ k,
                                                              const float *__restrict__ v, float *__restrict__ out,
                                                              int n_tok, int n_head, int n_head_kv, float scale) {
    extern __shared__ __align__(16) float att_smem[];
    float (*kt)[ATT_D] = reinterpret_cast<float (*)[ATT_D]>(att_smem);
    float (*vt)[ATT_D] = reinterpret_cast<float (*)[ATT_D]>(att_smem + ATT_TILE * ATT_D);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int qblocks = (n_tok + ATT_QPC - 1) / ATT_QPC;
    const int head = blockIdx.x / qblocks, qb = blockIdx.x - head * qblocks;
    const int q0 = qb * ATT_QPC + ATT_QPW * warp;           // the warp's first query
    const int kvh = head / (n_head / n_head_kv);
    const int myq = lane >> 3, mykk = lane & 7;             // after the reduction: lane = (query of the warp, key of the group of 8)
    float qreg[ATT_QPW][8], oreg[ATT_QPW][8];
#pragma unroll
    for (int a = 0; a < ATT_QPW; ++a) {
        const int qi = q0 + a;
#pragma unroll
        for (int i = 0; i < 8; ++i) { qreg[a][i] = 0.0f; oreg[a][i] = 0.0f; }
        if (qi < n_tok) {
            const float *qp = q + ((size_t)qi * n_head + head) * ATT_D + 8 * lane;
#pragma unroll
            for (int i = 0; i < 8; ++i) qreg[a][i] = __fmul_rn(qp[i], scale);
        }
    }
    float m = -INFINITY, l = 0.0f;                          // of query q0 + myq (the same in the 8 lanes of its group)
    const int last = min(n_tok - 1, qb * ATT_QPC + ATT_QPC - 1);            // keys 0 .. last serve the CTA's queries
    const int wlast = min(n_tok - 1, q0 + ATT_QPW - 1);                     // ... 0 .. wlast this warp's
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
        if (q0 >= n_tok || j0 > wlast) continue;
        const int wn = min(nk, wlast - j0 + 1);             // keys of this tile that any of the warp's queries may see
        float sc[4];
#pragma unroll
        for (int st = 0; st < 4; ++st) {
            sc[st] = -INFINITY;
            if (8 * st < wn) {                              // warp-uniform
                float part[32];
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const int r = 8 * st + kk;              // rows past wn hold stale data: masked below
                    const float4 ka = *reinterpret_cast<const float4 *>(&kt[r][8 * lane]);
                    const float4 kb = *reinterpret_cast<const float4 *>(&kt[r][8 * lane + 4]);
#pragma unroll
                    for (int a = 0; a < ATT_QPW; ++a) {
                        float pr = __fmul_rn(qreg[a][0], ka.x);
                        pr = __fmaf_rn(qreg[a][1], ka.y, pr); pr = __fmaf_rn(qreg[a][2], ka.z, pr); pr = __fmaf_rn(qreg[a][3], ka.w, pr);
                        pr = __fmaf_rn(qreg[a][4], kb.x, pr); pr = __fmaf_rn(qreg[a][5], kb.y, pr); pr = __fmaf_rn(qreg[a][6], kb.z, pr);
                        pr = __fmaf_rn(qreg[a][7], kb.w, pr);
                        part[8 * a + kk] = pr;
                    }
                }
                const float s = transpose_sum32(part, lane);            // lane (myq, mykk): score of key j0 + 8 st + mykk
                const int key = j0 + 8 * st + mykk;
                sc[st] = (key <= q0 + myq && key < n_tok && q0 + myq < n_tok) ? s : -INFINITY;
            }
        }
        // softmax step of the tile, per query (groups of 8 lanes)
        float tmax = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
        const float m_new = fmaxf(m, tmax);
        const float alpha = m_new == -INFINITY ? 1.0f : expf(__fsub_rn(m, m_new));      // a query with no key yet
        float p[4], psum = 0.0f;
#pragma unroll
        for (int st = 0; st < 4; ++st) {
            p[st] = sc[st] == -INFINITY ? 0.0f : expf(__fsub_rn(sc[st], m_new));
            psum = __fadd_rn(psum, p[st]);
        }
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) psum = __fadd_rn(psum, __shfl_xor_sync(0xffffffffu, psum, o));
        l = __fadd_rn(__fmul_rn(l, alpha), psum);
        m = m_new;
#pragma unroll
        for (int a = 0; a < ATT_QPW; ++a) {
            const float al = __shfl_sync(0xffffffffu, alpha, 8 * a);
#pragma unroll
            for (int i = 0; i < 8; ++i) oreg[a][i] = __fmul_rn(oreg[a][i], al);
        }
#pragma unroll
        for (int st = 0; st < 4; ++st) {
            if (8 * st < wn) {
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const int r = 8 * st + kk;
                    if (r < wn) {                           // warp-uniform
                        const float4 va = *reinterpret_cast<const float4 *>(&vt[r][8 * lane]);
                        const float4 vb = *reinterpret_cast<const float4 *>(&vt[r][8 * lane + 4]);
#pragma unroll
                        for (int a = 0; a < ATT_QPW; ++a) {
                            const float pr = __shfl_sync(0xffffffffu, p[st], 8 * a + kk);
                            oreg[a][0] = __fmaf_rn(pr, va.x, oreg[a][0]); oreg[a][1] = __fmaf_rn(pr, va.y, oreg[a][1]);
                            oreg[a][2] = __fmaf_rn(pr, va.z, oreg[a][2]); oreg[a][3] = __fmaf_rn(pr, va.w, oreg[a][3]);
                            oreg[a][4] = __fmaf_rn(pr, vb.x, oreg[a][4]); oreg[a][5] = __fmaf_rn(pr, vb.y, oreg[a][5]);
                            oreg[a][6] = __fmaf_rn(pr, vb.z, oreg[a][6]); oreg[a][7] = __fmaf_rn(pr, vb.w, oreg[a][7]);
                        }
                    }
                }
            }
        }
    }
#pragma unroll
    for (int a = 0; a < ATT_QPW; ++a) {
        const int qi = q0 + a;
        const float la = __shfl_sync(0xffffffffu, l, 8 * a);
        if (qi < n_tok) {
            const float inv = __fdiv_rn(1.0f, la);
            float *op = out + ((size_t)qi * n_head + head) * ATT_D + 8 * lane;
#pragma unroll
            for (int i = 0; i < 8; ++i) op[i] = __fmul_rn(oreg[a][i], inv);
        }
    }
}

}  // namespace b200
