/* bonsai_p40.h -- compute entry points of the Bonsai PQ2_0 kernel library, sm_100a build.
 *
 * This header declares the same C ABI as the reference library (boetti-dev/p40-kernel,
 * include/bonsai_p40.h:16-56): same symbol names, same argument order and meaning, same
 * return convention, so a program linked against the reference's libbonsai_p40 can be
 * relinked against this library without source changes.  The implementation behind it is
 * written from scratch for NVIDIA B200 (sm_100a).
 *
 * Common contract (reference: src/kernels/gemv_p40.cu:200-219, gemm_p40.cu:143-154,
 * gemv_repack_p40.cu:196-220, elementwise_p40.cu:75-80):
 *   - every pointer is a DEVICE pointer owned by the caller; the library allocates nothing,
 *     frees nothing and never synchronises; each call enqueues work on `stream` and returns;
 *   - return 0 on success, 1 on a rejected shape, otherwise the CUDA error code of the launch;
 *   - a call with nothing to do (n_out <= 0 where noted) returns 0 without launching.
 *
 * Data formats (reference: src/pq2_0.h:45-54):
 *   PQ2_0 block, 34 bytes : uint16 d (fp16 bits) + 32 code bytes; weight j of the block is
 *                           ((qs[j/4] >> 2*(j%4)) & 3) - 1, times d.  A matrix is row-major,
 *                           n_in/128 consecutive blocks per row, rows contiguous.
 *   Q8_1 block, 36 bytes  : uint16 d (fp16 bits of amax/127) + uint16 s (int16 sum of the 32
 *                           quantised values, raw bits) + 32 int8 in the 4x4-transposed order
 *                           written by bonsai_p40_quant_activations.
 *
 * Numerics: the integer dot products equal the reference's host implementation bit for bit;
 * quantised activations, rotated activations and the fp32 outputs of the mat-vec / mat-mul
 * are bit-identical to the reference's HOST code (src/pq2_0.h, src/fwht.h).  The reference's own
 * device build differs from its host code (ties-to-even rounding, approximate division); the
 * host code is the one followed here.
 */
#ifndef BONSAI_P40_H
#define BONSAI_P40_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* A cudaStream_t passed as an opaque pointer (reference: include/bonsai_p40.h:16). */
typedef void *bonsai_stream;

/* Decode mat-vec: y[n_out] = W[n_out, n_in] . x, W in PQ2_0, xq = x already quantised by
 * bonsai_p40_quant_activations.  Returns 1 if n_in <= 0 or n_in % 128 != 0; 0 without a
 * launch if n_out <= 0.  Replaces include/bonsai_p40.h:21 / src/kernels/gemv_p40.cu:210. */
int bonsai_p40_gemv(const void *W, const void *xq, float *y, int64_t n_out, int64_t n_in, bonsai_stream stream);

/* Quantise n floats to n/32 permuted Q8_1 blocks.  Returns 1 if n <= 0 or n % 32 != 0.
 * Replaces include/bonsai_p40.h:25 / src/kernels/gemv_p40.cu:200. */
int bonsai_p40_quant_activations(const float *x, void *out, int64_t n, bonsai_stream stream);

/* Prefill mat-mul: Y[n_out][n_tok] (row-major fp32) = W . X, with Xq chunk-major
 * [n_in/32][n_tok] Q8_1 blocks.  Returns 1 on a bad n_in; 0 without a launch if n_out <= 0
 * or n_tok <= 0.  Replaces include/bonsai_p40.h:29 / src/kernels/gemm_p40.cu:143.
 * From 17 tokens on (from 9 when rows are not a multiple of 1024 weights) the call may allocate a scratch buffer
 * once per (device, stream) and size, outside graph capture (see "gemm_path" in bonsai_b200_ext.h). */
int bonsai_p40_gemm(const void *W, const void *Xq, float *Y, int64_t n_out, int64_t n_in, int64_t n_tok,
                    bonsai_stream stream);

/* Aligned repacked layout, same size as the source (row stride 34 * n_in/128): per row the
 * n_in/128 fp16 scales, then four planes of 8-byte code units.  Both calls return 1 unless
 * n_in % 128 == 0, n_out > 0 and (n_in/128) % 8 == 0.  bonsai_p40_gemv_repack takes the fp32
 * activation vector and quantises it itself (it does NOT rotate it); its y is within 1e-5 of the reference's
 * repack_row_dot (same terms, a fixed launch-independent order: for a 16-byte aligned x and n_in % 1024 == 0 the
 * order of bonsai_p40_gemv, to whose result on the un-repacked matrix it is then bit-identical);
 * bonsai_b200_set_option("gemv_order", 1) restores repack_row_dot's plane-major order to the bit.
 * Replace include/bonsai_p40.h:35-36 / src/kernels/gemv_repack_p40.cu:196,209. */
int bonsai_p40_repack(const void *src, void *dst, int64_t n_out, int64_t n_in, bonsai_stream stream);
int bonsai_p40_gemv_repack(const void *W, const float *x, float *y, int64_t n_out, int64_t n_in,
                           bonsai_stream stream);

/* In-place normalised Walsh-Hadamard rotation in blocks of 1024; `signs` is NULL or n values
 * of +-1 applied before the transform.  Returns 1 if n <= 0 or n % 1024 != 0.
 * Replaces include/bonsai_p40.h:41 / src/kernels/elementwise_p40.cu:75. */
int bonsai_p40_fwht(float *x, const float *signs, int64_t n, bonsai_stream stream);

/* RMSNorm over n_rows rows of length n: y = x * (1 / sqrt(mean(x^2) + eps)) * w.  Returns 1 if n <= 0, 0 without
 * a launch if n_rows <= 0.  Within 1e-5 of the host formula (src/ops.h:13-22): the sum of squares is added in a
 * fixed tree order, not sequentially.  Replaces include/bonsai_p40.h:44 / src/kernels/elementwise_p40.cu:82. */
int bonsai_p40_rmsnorm(const float *x, const float *w, float *y, int64_t n_rows, int64_t n, float eps,
                       bonsai_stream stream);

/* One gated delta-net step for n_v_heads value heads (state [n_v_heads][K][V], updated in place; q, k per key head,
 * value head vh reads key head vh / (n_v_heads / n_k_heads); v, out [n_v_heads][V]; g, beta [n_v_heads]).  Returns 1
 * unless V > 0, V % 32 == 0, 0 < K <= 128 and n_v_heads % n_k_heads == 0.  Arithmetic in the order of src/ops.h:66-92;
 * exp(g) is the device's.  Replaces include/bonsai_p40.h:49 / src/kernels/attn_p40.cu:119. */
int bonsai_p40_gdn_step(float *state, const float *q, const float *k, const float *v, const float *g,
                        const float *beta, float *out, int n_k_heads, int n_v_heads, int K, int V,
                        bonsai_stream stream);

/* Causal attention, head_dim 256, grouped-query heads: q, out [n_tok][n_head][256]; k, v [n_tok][n_head_kv][256]
 * (16-byte aligned).  Returns 1 if head_dim != 256 or n_head % n_head_kv != 0; 0 without a launch if n_tok <= 0.
 * Online softmax, one key at a time (src/kernels/attn_p40.cu:92-118).  Replaces include/bonsai_p40.h:54 /
 * src/kernels/attn_p40.cu:131. */
int bonsai_p40_attn(const float *q, const float *k, const float *v, float *out, int n_tok, int n_head,
                    int n_head_kv, int head_dim, float scale, bonsai_stream stream);

#ifdef __cplusplus
}
#endif
#endif /* BONSAI_P40_H */
