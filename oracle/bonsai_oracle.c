/* bonsai_oracle.c -- CPU restatement of the Bonsai PQ2_0 hot path (TEST INFRASTRUCTURE).
 *
 * This file is a checker, not a product path.  It restates, in plain C99, the host
 * arithmetic of the reference (boetti-dev/p40-kernel) for the PQ2_0 x Q8_1 mat-vec /
 * mat-mul, the FWHT-1024 rotation and the Q8_1 activation quantiser.  Only the test
 * suite, the smoke check and the CPU-baseline leg of the benchmark may load it; the
 * CUDA library never links or calls it.
 *
 * Parity status: PINNED.  Every function below is compared bit for bit against the
 * reference's own headers compiled unmodified (oracle/ref_shim.cpp -> oracle/_ref/)
 * and against the committed vectors in tests/golden/ that were produced by that build.
 *
 * Build: gcc -O2 -std=c99 -ffp-contract=off -fPIC -shared (no -ffast-math, no
 * -march=native: the fp32 operations must stay separate IEEE mul / add / div).
 *
 * Each function cites the reference file:line whose behaviour it follows.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define BO_QK_W 128 /* weights per PQ2_0 block        (src/pq2_0.h:33) */
#define BO_QK_A 32  /* activations per Q8_1 block     (src/pq2_0.h:39) */
#define BO_W_BYTES 34
#define BO_A_BYTES 36
#define BO_FWHT_N 1024

/* ---- fp16 <-> fp32 ------------------------------------------------------------- */

/* Exact widening of an IEEE binary16 bit pattern (src/p40_common.h:57-80, host branch). */
float bo_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h >> 15) << 31;
    int e = (h >> 10) & 31;
    uint32_t m = h & 1023u;
    uint32_t bits;
    if (e == 31) {
        bits = sign | 0x7F800000u | (m << 13);
    } else if (e != 0) {
        bits = sign | ((uint32_t)(e + 112) << 23) | (m << 13);
    } else if (m == 0) {
        bits = sign;
    } else {
        int k = 113; /* exponent of the leading bit once normalised */
        while (!(m & 1024u)) { m <<= 1; --k; }
        bits = sign | ((uint32_t)k << 23) | ((m & 1023u) << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* Narrowing with the reference HOST rule: the first dropped mantissa bit alone decides
 * whether the magnitude is bumped, i.e. round to nearest with ties AWAY from zero.  The
 * hardware conversion (ties to even) differs on exact ties, so it is not used
 * (src/p40_common.h:82-114, non-CUDA branch). */
uint16_t bo_f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t e8 = (x >> 23) & 255u;
    uint32_t frac = x & 0x7FFFFFu;
    if (e8 == 255u) return (uint16_t)(sign | 0x7C00u | (frac ? 0x200u : 0u));
    int e = (int)e8 - 112; /* rebias 127 -> 15 */
    if (e >= 31) return (uint16_t)(sign | 0x7C00u);
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;
        uint32_t full = frac | 0x800000u;
        uint32_t sh = (uint32_t)(14 - e);
        uint32_t q = full >> sh;
        if ((full >> (sh - 1)) & 1u) q += 1;
        return (uint16_t)(sign | q);
    }
    uint32_t q = frac >> 13;
    if (frac & 0x1000u) {
        q += 1;
        if (q == 1024u) {
            q = 0;
            e += 1;
            if (e >= 31) return (uint16_t)(sign | 0x7C00u);
        }
    }
    return (uint16_t)(sign | ((uint32_t)e << 10) | q);
}

/* ---- byte-level views of the two block formats ---------------------------------- */
/* PQ2_0 block: [u16 d][32 code bytes]          (src/pq2_0.h:45-48)
 * Q8_1 block : [u16 d][u16 s][32 int8]         (src/pq2_0.h:50-54)                 */

static uint16_t rd16(const uint8_t *p) { uint16_t v; memcpy(&v, p, 2); return v; }
static void wr16(uint8_t *p, uint16_t v) { memcpy(p, &v, 2); }

/* Position j of a permuted Q8_1 block holds source element perm(j): a 4x4 transpose inside
 * each half of 16 (src/pq2_0.h:120-125). */
static int bo_perm(int j) { return 16 * (j >> 4) + 4 * (j & 3) + ((j >> 2) & 3); }

/* ---- activation quantiser (src/pq2_0.h:99-126) ----------------------------------- */
void bo_quantize_q8_1(const float *x, uint8_t *out, int64_t k, int permute) {
    int64_t nb = k / BO_QK_A;
    for (int64_t i = 0; i < nb; ++i) {
        const float *xi = x + i * BO_QK_A;
        uint8_t *blk = out + i * BO_A_BYTES;
        float amax = 0.0f;
        for (int j = 0; j < BO_QK_A; ++j) amax = fmaxf(amax, fabsf(xi[j]));
        float d = amax / 127.0f;
        float id = d > 0.0f ? 1.0f / d : 0.0f;
        int8_t q[BO_QK_A];
        int sum = 0;
        for (int j = 0; j < BO_QK_A; ++j) {
            int v = (int)lroundf(xi[j] * id);
            if (v < -127) v = -127;
            if (v > 127) v = 127;
            q[j] = (int8_t)v;
            sum += v;
        }
        wr16(blk, bo_f32_to_f16(d));
        wr16(blk + 2, (uint16_t)(int16_t)sum);
        for (int j = 0; j < BO_QK_A; ++j) blk[4 + j] = (uint8_t)q[permute ? bo_perm(j) : j];
    }
}

/* ---- weight quantiser / dequantiser (src/pq2_0.h:62-90) -------------------------- */
void bo_quantize_pq2_0(const float *x, uint8_t *out, int64_t k) {
    int64_t nb = k / BO_QK_W;
    for (int64_t i = 0; i < nb; ++i) {
        const float *xi = x + i * BO_QK_W;
        uint8_t *blk = out + i * BO_W_BYTES;
        float amax = 0.0f;
        for (int j = 0; j < BO_QK_W; ++j) amax = fmaxf(amax, fabsf(xi[j]));
        float id = amax > 0.0f ? 1.0f / amax : 0.0f;
        wr16(blk, bo_f32_to_f16(amax));
        memset(blk + 2, 0, 32);
        for (int j = 0; j < BO_QK_W; ++j) {
            int c = (int)lroundf(xi[j] * id) + 1;
            if (c < 0) c = 0;
            if (c > 3) c = 3;
            blk[2 + (j >> 2)] |= (uint8_t)(c << (2 * (j & 3)));
        }
    }
}

void bo_dequantize_pq2_0(const uint8_t *in, float *y, int64_t k) {
    int64_t nb = k / BO_QK_W;
    for (int64_t i = 0; i < nb; ++i) {
        const uint8_t *blk = in + i * BO_W_BYTES;
        float d = bo_f16_to_f32(rd16(blk));
        for (int j = 0; j < BO_QK_W; ++j) {
            int c = (blk[2 + (j >> 2)] >> (2 * (j & 3))) & 3;
            y[i * BO_QK_W + j] = (float)(c - 1) * d;
        }
    }
}

/* ---- FWHT-1024 (src/fwht.h:20-42) -------------------------------------------------- */
static void bo_fwht_1024(float *x, const float *signs) {
    if (signs)
        for (int i = 0; i < BO_FWHT_N; ++i) x[i] *= signs[i];
    for (int h = 1; h < BO_FWHT_N; h *= 2)
        for (int base = 0; base < BO_FWHT_N; base += 2 * h)
            for (int j = base; j < base + h; ++j) {
                float lo = x[j], hi = x[j + h];
                x[j] = lo + hi;
                x[j + h] = lo - hi;
            }
    for (int i = 0; i < BO_FWHT_N; ++i) x[i] *= (1.0f / 32.0f);
}

/* `signs` (nullable) has length n: block b uses signs + b (src/fwht.h:38-42). */
void bo_fwht_blocks(float *x, const float *signs, int64_t n) {
    for (int64_t b = 0; b < n; b += BO_FWHT_N) bo_fwht_1024(x + b, signs ? signs + b : NULL);
}

/* ---- per-chunk integer core (src/pq2_0.h:149-172, src/p40_common.h:119-141) -------- */

/* Sum over 32 weights of (code - 1) * activation for chunk `iqs` of one weight block against
 * one PERMUTED activation block: code field k of 16-code word w pairs with activation word
 * 4w + k byte for byte. */
int32_t bo_chunk_sumi(const uint8_t *wblk, const uint8_t *ablk, int iqs) {
    const uint8_t *codes = wblk + 2 + 8 * iqs;
    const int8_t *act = (const int8_t *)(ablk + 4);
    int32_t acc = 0;
    for (int w = 0; w < 2; ++w)
        for (int k = 0; k < 4; ++k)
            for (int i = 0; i < 4; ++i) {
                int c = (codes[4 * w + i] >> (2 * k)) & 3;
                acc += c * (int32_t)act[16 * w + 4 * k + i];
            }
    return acc - (int32_t)(int16_t)rd16(ablk + 2);
}

/* (f32(dw) * f32(da)) * (float)sumi, in that association (src/pq2_0.h:170-171). */
float bo_chunk_dot(const uint8_t *wblk, const uint8_t *ablk, int iqs) {
    float d = bo_f16_to_f32(rd16(wblk)) * bo_f16_to_f32(rd16(ablk));
    return d * (float)bo_chunk_sumi(wblk, ablk, iqs);
}

/* One output row: sequential fp32 sum over blocks, then chunks (src/pq2_0.h:183-191). */
float bo_row_dot(const uint8_t *wrow, const uint8_t *xq, int64_t n_in) {
    float acc = 0.0f;
    for (int64_t b = 0; b < n_in / BO_QK_W; ++b)
        for (int iqs = 0; iqs < 4; ++iqs)
            acc += bo_chunk_dot(wrow + b * BO_W_BYTES, xq + (4 * b + iqs) * BO_A_BYTES, iqs);
    return acc;
}

/* Per-chunk integer sums of one row (debug parity level: int32 exact). */
void bo_row_chunk_sums(const uint8_t *wrow, const uint8_t *xq, int64_t n_in, int32_t *out) {
    for (int64_t b = 0; b < n_in / BO_QK_W; ++b)
        for (int iqs = 0; iqs < 4; ++iqs)
            out[4 * b + iqs] = bo_chunk_sumi(wrow + b * BO_W_BYTES, xq + (4 * b + iqs) * BO_A_BYTES, iqs);
}

/* ---- mat-vec / mat-mul ----------------------------------------------------------------- */

/* y[r] = row_dot(W[r], xq); the value src/kernels/gemv_p40.cu:82-165 is defined by. */
void bo_gemv_rows(const uint8_t *W, const uint8_t *xq, float *y, int64_t r0, int64_t r1, int64_t n_in) {
    int64_t rb = n_in / BO_QK_W * BO_W_BYTES;
    for (int64_t r = r0; r < r1; ++r) y[r] = bo_row_dot(W + r * rb, xq, n_in);
}

void bo_gemv(const uint8_t *W, const uint8_t *xq, float *y, int64_t n_out, int64_t n_in) {
    bo_gemv_rows(W, xq, y, 0, n_out, n_in);
}

/* Y[r * n_tok + t] over chunk-major Xq[(chunk) * n_tok + t]; per (r, t) the same block-then-
 * chunk order as the row dot (src/kernels/gemm_p40.cu:68-136, tests/test_p40.cpp:460-467). */
void bo_gemm_rows(const uint8_t *W, const uint8_t *Xq, float *Y, int64_t r0, int64_t r1, int64_t n_in,
                  int64_t n_tok) {
    int64_t nb = n_in / BO_QK_W, rb = nb * BO_W_BYTES;
    for (int64_t r = r0; r < r1; ++r)
        for (int64_t t = 0; t < n_tok; ++t) {
            float acc = 0.0f;
            for (int64_t b = 0; b < nb; ++b)
                for (int iqs = 0; iqs < 4; ++iqs)
                    acc += bo_chunk_dot(W + r * rb + b * BO_W_BYTES, Xq + ((4 * b + iqs) * n_tok + t) * BO_A_BYTES,
                                        iqs);
            Y[r * n_tok + t] = acc;
        }
}

void bo_gemm(const uint8_t *W, const uint8_t *Xq, float *Y, int64_t n_out, int64_t n_in, int64_t n_tok) {
    bo_gemm_rows(W, Xq, Y, 0, n_out, n_in, n_tok);
}

/* ---- aligned repacked layout (src/pq2_0_repack.h:46-82) ----------------------------------- */
/* Row = nb fp16 scales, then 4 planes of nb 8-byte units; unit u = plane * nb + block.        */

void bo_repack_row(const uint8_t *src, int nb, uint8_t *dst) {
    for (int b = 0; b < nb; ++b) {
        memcpy(dst + 2 * b, src + b * BO_W_BYTES, 2);
        for (int p = 0; p < 4; ++p) memcpy(dst + 2 * nb + 8 * (p * nb + b), src + b * BO_W_BYTES + 2 + 8 * p, 8);
    }
}

void bo_unpack_row(const uint8_t *src, int nb, uint8_t *dst) {
    for (int b = 0; b < nb; ++b) {
        memcpy(dst + b * BO_W_BYTES, src + 2 * b, 2);
        for (int p = 0; p < 4; ++p) memcpy(dst + b * BO_W_BYTES + 2 + 8 * p, src + 2 * nb + 8 * (p * nb + b), 8);
    }
}

/* 1 on shapes the reference wrapper rejects (src/kernels/gemv_repack_p40.cu:198-200). */
int bo_repack(const uint8_t *src, uint8_t *dst, int64_t n_out, int64_t n_in) {
    if (n_in % 128 != 0 || n_out <= 0) return 1;
    int nb = (int)(n_in / 128);
    if (nb <= 0 || nb % 8 != 0) return 1;
    for (int64_t r = 0; r < n_out; ++r) bo_repack_row(src + r * 34 * nb, nb, dst + r * 34 * nb);
    return 0;
}

/* Integer sum of unit u against activation chunk 4 * block + plane (src/pq2_0_repack.h:97-119). */
int32_t bo_repack_unit_sumi(const uint8_t *row, const uint8_t *xq, int nb, int u) {
    int p = u / nb, b = u % nb;
    uint8_t blk[BO_W_BYTES];
    memset(blk, 0, sizeof blk);
    memcpy(blk + 2 + 8 * p, row + 2 * nb + 8 * u, 8);
    return bo_chunk_sumi(blk, xq + (4 * b + p) * BO_A_BYTES, p);
}

/* Sequential fp32 sum in UNIT order (plane-major), each term (dw * da) * sumi
 * (src/pq2_0_repack.h:122-138). */
float bo_repack_row_dot(const uint8_t *row, const uint8_t *xq, int nb) {
    float acc = 0.0f;
    for (int u = 0; u < 4 * nb; ++u) {
        int p = u / nb, b = u % nb;
        const uint8_t *a = xq + (4 * b + p) * BO_A_BYTES;
        float dw = bo_f16_to_f32(rd16(row + 2 * b));
        float da = bo_f16_to_f32(rd16(a));
        acc += dw * da * (float)bo_repack_unit_sumi(row, xq, nb, u);
    }
    return acc;
}

/* Fused entry: quantise fp32 x (NOT rotated) then repacked row dots
 * (src/kernels/gemv_repack_p40.cu:91-162, 209-220). */
int bo_gemv_repack(const uint8_t *W, const float *x, float *y, int64_t n_out, int64_t n_in) {
    if (n_in % 128 != 0 || n_out <= 0) return 1;
    int nb = (int)(n_in / 128);
    if (nb <= 0 || nb % 8 != 0) return 1;
    uint8_t *xq = (uint8_t *)malloc((size_t)(n_in / 32) * BO_A_BYTES);
    if (!xq) return 2;
    bo_quantize_q8_1(x, xq, n_in, 1);
    for (int64_t r = 0; r < n_out; ++r) y[r] = bo_repack_row_dot(W + r * 34 * nb, xq, nb);
    free(xq);
    return 0;
}

/* ---- row-parallel drivers for the timed CPU baseline ------------------------------------------ */
typedef struct {
    const uint8_t *W, *Xq;
    float *Y;
    int64_t r0, r1, n_in, n_tok;
} bo_job;

static void *bo_worker(void *p) {
    bo_job *j = (bo_job *)p;
    if (j->n_tok == 0) bo_gemv_rows(j->W, j->Xq, j->Y, j->r0, j->r1, j->n_in);
    else bo_gemm_rows(j->W, j->Xq, j->Y, j->r0, j->r1, j->n_in, j->n_tok);
    return NULL;
}

static int bo_run_mt(const uint8_t *W, const uint8_t *Xq, float *Y, int64_t n_out, int64_t n_in, int64_t n_tok,
                     int nthreads) {
    if (nthreads < 1) nthreads = 1;
    if (nthreads > 256) nthreads = 256;
    pthread_t th[256];
    bo_job jobs[256];
    int started = 0;
    for (int t = 0; t < nthreads; ++t) {
        jobs[t].W = W; jobs[t].Xq = Xq; jobs[t].Y = Y; jobs[t].n_in = n_in; jobs[t].n_tok = n_tok;
        jobs[t].r0 = n_out * t / nthreads;
        jobs[t].r1 = n_out * (t + 1) / nthreads;
        if (pthread_create(&th[t], NULL, bo_worker, &jobs[t]) != 0) break;
        ++started;
    }
    for (int t = 0; t < started; ++t) pthread_join(th[t], NULL);
    for (int t = started; t < nthreads; ++t) bo_worker(&jobs[t]);
    return 0;
}

/* Rows are independent, so a row split over threads returns the same bits as bo_gemv. */
int bo_gemv_mt(const uint8_t *W, const uint8_t *xq, float *y, int64_t n_out, int64_t n_in, int nthreads) {
    return bo_run_mt(W, xq, y, n_out, n_in, 0, nthreads);
}

int bo_gemm_mt(const uint8_t *W, const uint8_t *Xq, float *Y, int64_t n_out, int64_t n_in, int64_t n_tok,
               int nthreads) {
    return bo_run_mt(W, Xq, Y, n_out, n_in, n_tok, nthreads);
}

/* ---- the operators beside the mat-vec path ------------------------------------------------------
 * RMSNorm and SwiGLU follow src/ops.h:13-31, the gated delta-net step src/ops.h:66-92 with the head
 * mapping of src/kernels/attn_p40.cu:36-38; attention is the online-softmax recurrence of
 * tests/test_p40.cpp:240-262 applied to every (query, head) under the causal mask of
 * src/kernels/attn_p40.cu:101. */
void bo_rmsnorm(const float *x, const float *w, float *y, int64_t n_rows, int64_t n, float eps) {
    for (int64_t r = 0; r < n_rows; ++r) {
        const float *xr = x + r * n;
        float ss = 0.0f;
        for (int64_t i = 0; i < n; ++i) ss += xr[i] * xr[i];
        const float s = 1.0f / sqrtf(ss / (float)n + eps);
        for (int64_t i = 0; i < n; ++i) y[r * n + i] = xr[i] * s * w[i];
    }
}

void bo_swiglu(const float *gate, const float *up, float *y, int64_t n) {
    for (int64_t i = 0; i < n; ++i) y[i] = gate[i] / (1.0f + expf(-gate[i])) * up[i];
}

void bo_gdn_step(float *state, const float *q, const float *k, const float *v, const float *g, const float *beta,
                 float *out, int n_k_heads, int n_v_heads, int K, int V) {
    for (int vh = 0; vh < n_v_heads; ++vh) {
        const int kh = vh / (n_v_heads / n_k_heads);
        float *S = state + (size_t)vh * K * V;
        const float *kk = k + (size_t)kh * K, *qq = q + (size_t)kh * K, *vv = v + (size_t)vh * V;
        float *o = out + (size_t)vh * V;
        const float decay = expf(g[vh]);
        for (int i = 0; i < K; ++i)
            for (int j = 0; j < V; ++j) S[i * V + j] *= decay;
        for (int j = 0; j < V; ++j) {
            float acc = 0.0f;
            for (int i = 0; i < K; ++i) acc += kk[i] * S[i * V + j];
            o[j] = acc;
        }
        for (int i = 0; i < K; ++i) {
            const float bk = beta[vh] * kk[i];
            for (int j = 0; j < V; ++j) S[i * V + j] += bk * (vv[j] - o[j]);
        }
        for (int j = 0; j < V; ++j) {
            float acc = 0.0f;
            for (int i = 0; i < K; ++i) acc += qq[i] * S[i * V + j];
            o[j] = acc;
        }
    }
}

void bo_attn(const float *q, const float *k, const float *v, float *out, int n_tok, int n_head, int n_head_kv, int D,
             float scale) {
    float *acc = (float *)malloc(sizeof(float) * (size_t)D);
    for (int qi = 0; qi < n_tok; ++qi)
        for (int head = 0; head < n_head; ++head) {
            const int kvh = head / (n_head / n_head_kv);
            const float *qp = q + ((size_t)qi * n_head + head) * D;
            float m = -INFINITY, l = 0.0f;
            for (int d = 0; d < D; ++d) acc[d] = 0.0f;
            for (int j = 0; j <= qi; ++j) {
                const float *kp = k + ((size_t)j * n_head_kv + kvh) * D;
                const float *vp = v + ((size_t)j * n_head_kv + kvh) * D;
                float s = 0.0f;
                for (int d = 0; d < D; ++d) s += qp[d] * kp[d];
                s *= scale;
                const float m_new = fmaxf(m, s);
                const float alpha = expf(m - m_new), p = expf(s - m_new);
                l = l * alpha + p;
                for (int d = 0; d < D; ++d) acc[d] = acc[d] * alpha + p * vp[d];
                m = m_new;
            }
            for (int d = 0; d < D; ++d) out[((size_t)qi * n_head + head) * D + d] = acc[d] / l;
        }
    free(acc);
}

/* ---- K/V cache numeric core ---------------------------------------------------------------------
 * Q8_0 rows as src/kv_cache.h:100-117 (d = amax / 127, lroundf, clamp, fp16 scale by bo_f32_to_f16); block score as
 * src/kv_cache.h:129-145; attention of one query position over positions 0..pos of one layer, every query head, as the
 * recurrence of src/kernels/kv_p40.cu:178-199 (one position at a time, online softmax) on the cache layout of
 * src/kv_cache.h:81-84: block[((layer * n_kv + kvh) * capacity + pos) * 8 + blk], 34-byte blocks. */
void bo_kv_quantize_row_q8_0(const float *x, uint8_t *y, int n) {
    for (int b = 0; b < n / 32; ++b) {
        const float *src = x + b * 32;
        uint8_t *blk = y + b * 34;
        float amax = 0.0f;
        for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(src[i]));
        const float d = amax / 127.0f;
        const float id = d > 0.0f ? 1.0f / d : 0.0f;
        const uint16_t dh = bo_f32_to_f16(d);
        memcpy(blk, &dh, 2);
        for (int i = 0; i < 32; ++i) {
            int v = (int)lroundf(src[i] * id);
            if (v < -127) v = -127;
            if (v > 127) v = 127;
            blk[2 + i] = (uint8_t)(int8_t)v;
        }
    }
}

void bo_kv_dequantize_row_q8_0(const uint8_t *x, float *y, int n) {
    for (int b = 0; b < n / 32; ++b) {
        uint16_t dh;
        memcpy(&dh, x + b * 34, 2);
        const float d = bo_f16_to_f32(dh);
        for (int i = 0; i < 32; ++i) y[b * 32 + i] = (float)(int8_t)x[b * 34 + 2 + i] * d;
    }
}

float bo_kv_score(const uint8_t *q, const uint8_t *k, int nblocks) {
    float acc = 0.0f;
    for (int b = 0; b < nblocks; ++b) {
        int sumi = 0;
        for (int i = 0; i < 32; ++i) sumi += (int)(int8_t)q[b * 34 + 2 + i] * (int)(int8_t)k[b * 34 + 2 + i];
        uint16_t dq, dk;
        memcpy(&dq, q + b * 34, 2);
        memcpy(&dk, k + b * 34, 2);
        acc += bo_f16_to_f32(dq) * bo_f16_to_f32(dk) * (float)sumi;
    }
    return acc;
}

/* K, V: whole cache arrays; q, out: [n_head][256]. */
void bo_kv_attn_decode(const uint8_t *K, const uint8_t *V, const float *q, float *out, int capacity, int layer, int pos,
                       int n_head, int n_kv_head, float scale) {
    const int D = 256, nblk = 8;
    uint8_t q8[8 * 34];
    float vrow[256], acc[256];
    for (int head = 0; head < n_head; ++head) {
        const int kvh = head / (n_head / n_kv_head);
        bo_kv_quantize_row_q8_0(q + (size_t)head * D, q8, D);
        const size_t base = ((size_t)layer * n_kv_head + kvh) * (size_t)capacity;
        float m = -INFINITY, l = 0.0f;
        for (int d = 0; d < D; ++d) acc[d] = 0.0f;
        for (int p = 0; p <= pos; ++p) {
            const uint8_t *kb = K + (base + p) * nblk * 34, *vb = V + (base + p) * nblk * 34;
            const float s = bo_kv_score(q8, kb, nblk) * scale;
            const float m_new = fmaxf(m, s);
            const float alpha = expf(m - m_new), pw = expf(s - m_new);
            l = l * alpha + pw;
            bo_kv_dequantize_row_q8_0(vb, vrow, D);
            for (int d = 0; d < D; ++d) acc[d] = acc[d] * alpha + pw * vrow[d];
            m = m_new;
        }
        for (int d = 0; d < D; ++d) out[(size_t)head * D + d] = acc[d] / l;
    }
}

