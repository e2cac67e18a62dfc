// ref_shim.cpp -- C-ABI window onto the reference's OWN host headers (TEST INFRASTRUCTURE).
//
// Nothing here implements arithmetic.  Each export forwards to a function of the
// boetti-dev/p40-kernel headers, which are compiled where they lie (passed with -I by
// oracle/build_oracle.py; no reference source is copied into this repository).  The
// resulting oracle/_ref/libbonsai_ref.so pins oracle/bonsai_oracle.c, produces the vectors
// under tests/golden/, and can serve as the timed CPU baseline (kind "reference").
//
// Compiled with g++ (never nvcc), so the headers take their non-CUDA branches: software
// f32_to_f16 / f16_to_f32 and the dp4a emulation.
#include "fwht.h"
#include "kv_cache.h"
#include "ops.h"
#include "pq2_0.h"
#include "pq2_0_repack.h"

#include <cstdint>
#include <thread>
#include <vector>

using namespace bonsai;

static_assert(sizeof(block_pq2_0) == 34, "PQ2_0 block is 34 bytes");
static_assert(sizeof(block_q8_1) == 36, "Q8_1 block is 36 bytes");

extern "C" {

float ref_f16_to_f32(uint16_t h) { return f16_to_f32(h); }
uint16_t ref_f32_to_f16(float f) { return f32_to_f16(f); }

void ref_quantize_q8_1(const float *x, void *out, int64_t k, int permute) {
    quantize_row_q8_1(x, (block_q8_1 *)out, k, permute != 0);
}
void ref_quantize_pq2_0(const float *x, void *out, int64_t k) { quantize_row_pq2_0(x, (block_pq2_0 *)out, k); }
void ref_dequantize_pq2_0(const void *in, float *y, int64_t k) {
    dequantize_row_pq2_0((const block_pq2_0 *)in, y, k);
}
void ref_fwht_blocks(float *x, const float *signs, int64_t n) { fwht_blocks(x, signs, (int)n); }

float ref_chunk_dot(const void *wblk, const void *ablk, int iqs) {
    return pq2_0_dot_q8_1_block((const block_pq2_0 *)wblk, (const block_q8_1 *)ablk, iqs);
}
float ref_row_dot(const void *wrow, const void *xq, int64_t n_in) {
    return pq2_0_row_dot_perm((const block_pq2_0 *)wrow, (const block_q8_1 *)xq, (int)n_in);
}

static void gemv_rows(const block_pq2_0 *W, const block_q8_1 *xq, float *y, int64_t r0, int64_t r1, int64_t n_in) {
    const int64_t nb = n_in / BONSAI_QK_PQ2_0;
    for (int64_t r = r0; r < r1; ++r) y[r] = pq2_0_row_dot_perm(W + r * nb, xq, (int)n_in);
}
static void gemm_rows(const block_pq2_0 *W, const block_q8_1 *X, float *Y, int64_t r0, int64_t r1, int64_t n_in,
                      int64_t n_tok) {
    // The accumulation the reference's own GEMM test uses per (row, token): blocks, then chunks.
    const int64_t nb = n_in / BONSAI_QK_PQ2_0;
    for (int64_t r = r0; r < r1; ++r)
        for (int64_t t = 0; t < n_tok; ++t) {
            float acc = 0.0f;
            for (int64_t b = 0; b < nb; ++b)
                for (int iqs = 0; iqs < BONSAI_QI_PQ2_0; ++iqs)
                    acc += pq2_0_dot_q8_1_block(W + r * nb + b, X + (b * BONSAI_QI_PQ2_0 + iqs) * n_tok + t, iqs);
            Y[r * n_tok + t] = acc;
        }
}

void ref_gemv(const void *W, const void *xq, float *y, int64_t n_out, int64_t n_in) {
    gemv_rows((const block_pq2_0 *)W, (const block_q8_1 *)xq, y, 0, n_out, n_in);
}
void ref_gemm(const void *W, const void *Xq, float *Y, int64_t n_out, int64_t n_in, int64_t n_tok) {
    gemm_rows((const block_pq2_0 *)W, (const block_q8_1 *)Xq, Y, 0, n_out, n_in, n_tok);
}

// Row split over host threads; rows are independent so the bits equal the serial call.
int ref_gemv_mt(const void *W, const void *xq, float *y, int64_t n_out, int64_t n_in, int nthreads) {
    if (nthreads < 1) nthreads = 1;
    std::vector<std::thread> th;
    for (int t = 0; t < nthreads; ++t)
        th.emplace_back(gemv_rows, (const block_pq2_0 *)W, (const block_q8_1 *)xq, y, n_out * t / nthreads,
                        n_out * (t + 1) / nthreads, n_in);
    for (auto &t : th) t.join();
    return 0;
}
int ref_gemm_mt(const void *W, const void *Xq, float *Y, int64_t n_out, int64_t n_in, int64_t n_tok, int nthreads) {
    if (nthreads < 1) nthreads = 1;
    std::vector<std::thread> th;
    for (int t = 0; t < nthreads; ++t)
        th.emplace_back(gemm_rows, (const block_pq2_0 *)W, (const block_q8_1 *)Xq, Y, n_out * t / nthreads,
                        n_out * (t + 1) / nthreads, n_in, n_tok);
    for (auto &t : th) t.join();
    return 0;
}

void ref_repack_row(const void *src, int nb, uint8_t *dst) { repack_row_pq2_0((const block_pq2_0 *)src, nb, dst); }
void ref_unpack_row(const uint8_t *src, int nb, void *dst) { unpack_row_pq2_0(src, nb, (block_pq2_0 *)dst); }
int32_t ref_repack_unit_sumi(const uint8_t *row, const void *xq, int nb, int u) {
    return repack_unit_sumi(row, (const block_q8_1 *)xq, nb, u);
}
float ref_repack_row_dot(const uint8_t *row, const void *xq, int nb) {
    return repack_row_dot(row, (const block_q8_1 *)xq, nb);
}

// ---- the operators beside the mat-vec path (src/ops.h) ---------------------------------------------------------
void ref_rmsnorm(const float *x, const float *w, float *y, int64_t n_rows, int64_t n, float eps) {
    for (int64_t r = 0; r < n_rows; ++r) rmsnorm(x + r * n, w, y + r * n, (int)n, eps);
}
void ref_swiglu(const float *gate, const float *up, float *y, int64_t n) { swiglu(gate, up, y, (int)n); }
// One recurrent step for every value head, with the grouped-query mapping of the reference's wrapper
// (src/kernels/attn_p40.cu:36-38): value head vh reads key head vh / (n_v_heads / n_k_heads).
void ref_gdn_step(float *state, const float *q, const float *k, const float *v, const float *g, const float *beta,
                  float *out, int n_k_heads, int n_v_heads, int K, int V) {
    for (int vh = 0; vh < n_v_heads; ++vh) {
        const int kh = vh / (n_v_heads / n_k_heads);
        gdn_step(state + (size_t)vh * K * V, q + (size_t)kh * K, k + (size_t)kh * K, v + (size_t)vh * V, g[vh], beta[vh],
                 out + (size_t)vh * V, K, V);
    }
}

// ---- K/V cache numeric core (src/kv_cache.h) -------------------------------------------------------------------
static_assert(sizeof(block_q8_0) == 34, "Q8_0 block is 34 bytes");
void ref_kv_quantize_row_q8_0(const float *x, void *y, int n) { kv_quantize_row_q8_0(x, (block_q8_0 *)y, n); }
void ref_kv_dequantize_row_q8_0(const void *x, float *y, int n) { kv_dequantize_row_q8_0((const block_q8_0 *)x, y, n); }
float ref_kv_score(const void *q, const void *k, int nblocks) { return kv_score((const block_q8_0 *)q, (const block_q8_0 *)k, nblocks); }
int64_t ref_kv_block_index(int capacity, int layer, int kv_head, int pos, int blk) {
    return kv_geometry::for_27b(capacity).block_index(layer, kv_head, pos, blk);
}
int64_t ref_kv_total_bytes(int capacity) { return kv_geometry::for_27b(capacity).total_bytes(); }
int64_t ref_kv_gdn_bytes() { return gdn_state_bytes(); }

}  // extern "C"
