/* bonsai_kv.h -- the K/V cache of the full-attention layers and the recurrent state of the linear-attention layers,
 * sm_100a build.
 *
 * Same C ABI as the reference (boetti-dev/p40-kernel, include/bonsai_kv.h:24-57): same symbols, argument order and
 * meaning.  The model is hybrid: 16 full-attention layers own a growing Q8_0 cache (4 kv heads x 256 dims per
 * position), 48 gated delta-net layers own a constant fp32 state (48 value heads x 128 x 128 per layer).  Both are
 * allocated once by bonsai_kv_create; nothing is paged or evicted.
 *
 * Cache format (reference: src/kv_cache.h:35-46, 62-66): Q8_0 blocks of 34 bytes (fp16 scale + 32 int8), head-major,
 *   block[((layer * 4 + kv_head) * capacity + pos) * 8 + blk],  K and V in separate arrays.
 * Quantisation follows the reference's HOST function (src/kv_cache.h:100-117): d = amax / 127, values rounded to
 * nearest with ties away from zero, the scale stored as fp16 by the host's rounding rule; cache bytes are equal to it.
 * Attention outputs are held to 1e-5 of the largest output against the host arithmetic (int8 dot products are
 * exact; the softmax runs tile by tile, the host position by position).
 */
#ifndef BONSAI_KV_H
#define BONSAI_KV_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void *bonsai_stream;
typedef struct bonsai_kv_cache bonsai_kv_cache;

/* Bytes of the growing K + V cache at `capacity` positions (clamped to the model's 262144-token window), and of the
 * constant delta-net state.  Replace include/bonsai_kv.h:27-29 / src/kernels/kv_p40.cu:249-255. */
int64_t bonsai_kv_bytes(int capacity);
int64_t bonsai_kv_gdn_bytes(void);

/* Allocates cache, state and the decode workspace on the current device (the only calls of this library family that
 * allocate: as in the reference, src/kernels/kv_p40.cu:257-291); the state is zeroed on `stream`.  NULL on failure or
 * capacity <= 0.  bonsai_kv_reset zeroes the state again (position counters belong to the caller). */
bonsai_kv_cache *bonsai_kv_create(int capacity, bonsai_stream stream);
void bonsai_kv_free(bonsai_kv_cache *kv);
void bonsai_kv_reset(bonsai_kv_cache *kv, bonsai_stream stream);

/* Quantises and stores K and V of one full-attention layer (0..15) at position `pos`; k, v are [4][256] floats.  The
 * batch form stores n_tok positions from pos0 on; k, v are [n_tok][4][256].  Return 1 on a bad layer or range.
 * Replace include/bonsai_kv.h:40-46 / src/kernels/kv_p40.cu:317-339. */
int bonsai_kv_append(bonsai_kv_cache *kv, int layer, int pos, const float *k, const float *v, bonsai_stream stream);
int bonsai_kv_append_batch(bonsai_kv_cache *kv, int layer, int pos0, int n_tok, const float *k, const float *v,
                           bonsai_stream stream);

/* Attention of one query position over positions 0..pos of `layer`: q, out are [24][256] floats; scale 1/sqrt(256).
 * Replaces include/bonsai_kv.h:52-53 / src/kernels/kv_p40.cu:341-367. */
int bonsai_kv_attn_decode(bonsai_kv_cache *kv, int layer, int pos, const float *q, float *out, bonsai_stream stream);

/* Device pointer to the state of linear-attention layer 0..47 ([48][128][128] floats), NULL otherwise.
 * Replaces include/bonsai_kv.h:57 / src/kernels/kv_p40.cu:309-315. */
float *bonsai_kv_gdn_state(bonsai_kv_cache *kv, int layer);

#ifdef __cplusplus
}
#endif
#endif /* BONSAI_KV_H */
