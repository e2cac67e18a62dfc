/* bonsai_b200_ext.h -- additive entry points of the sm_100a build.
 *
 * None of these exists in the reference library; they do not change the meaning of any
 * symbol in bonsai_p40.h.  Same conventions: device pointers owned by the caller, work is
 * enqueued on `stream`, 0 = success, 1 = rejected shape, otherwise a CUDA error code.
 */
#ifndef BONSAI_B200_EXT_H
#define BONSAI_B200_EXT_H

#include "bonsai_p40.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Rotation and quantiser in one launch: xq = Q8_1(FWHT1024(signs * x)).  x is left untouched;
 * if x_rot is not NULL it receives the rotated fp32 vector.  No counterpart in the reference,
 * which launches src/kernels/elementwise_p40.cu:75 and src/kernels/gemv_p40.cu:200 in turn;
 * the bytes written equal those two calls. */
int bonsai_b200_fwht_quant(const float *x, const float *signs, void *xq, float *x_rot, int64_t n,
                           bonsai_stream stream);

/* One decode projection in one call: xq_scratch = Q8_1(FWHT1024(signs * x)), then y = W . xq_scratch.
 * xq_scratch is caller-provided device memory of n_in / 32 * 36 bytes (4-byte aligned) that the call
 * overwrites; x is left untouched.  Two launches by default; with the option "fuse_linear" = 1 and a shape
 * the streaming mat-vec takes, ONE launch (rotation and quantiser run in the mat-vec's prologue, once per
 * CTA).  Either way y and the scratch equal bonsai_b200_fwht_quant followed by bonsai_p40_gemv.  No counterpart in the reference, whose callers issue the steps themselves
 * (docs/INTEGRATION.md:260-263).  Returns 1 if n_in % 1024 != 0 or n_out <= 0. */
int bonsai_b200_linear(const void *W, const float *x, const float *signs, float *y, void *xq_scratch,
                       int64_t n_out, int64_t n_in, bonsai_stream stream);

/* The same projection for callers that must not allocate device memory and have no spare buffer to
 * lend: the quantised activation vector lives in an array compiled into the library instead of in
 * caller memory.  Typical callers: a plugin inside a host runtime that reserved the whole device for
 * its own pool up front and hands out no sub-allocations to plugins (the reference's fork hook
 * allocates its scratch lazily with cudaMalloc, integrations/prismml/bonsai-p40.diff:275-281, which
 * such a host forbids), and latency-critical loops where a cudaMalloc would synchronise the device.
 * This entry point has no counterpart in the reference.
 *   - limit: n_in <= BONSAI_B200_LINEAR_STATIC_MAX_N_IN (the array is 36 864 bytes per GPU that loads
 *     the library, held until the process exits); larger n_in returns BONSAI_B200_ETOOLARGE and
 *     launches nothing.  Other shape errors return 1 as in bonsai_b200_linear.
 *   - it calls no cudaMalloc / cudaFree nor any allocating library routine, on any call.
 *   - the first call on each device looks up the array's device address (cudaGetSymbolAddress) and
 *     remembers it for the life of the process; make that first call outside of any stream capture, and
 *     do not call cudaDeviceReset() afterwards (the remembered address would belong to the old context).
 *   - every call on a device uses the same array and leaves its Q8_1 bytes there.  Nothing has to be
 *     cleared between calls (each call overwrites the n_in / 32 blocks it then reads), but two calls
 *     whose kernels overlap on the GPU -- different streams, or concurrent host threads -- race on it:
 *     serialise them on one stream. */
#define BONSAI_B200_LINEAR_STATIC_MAX_N_IN 32768
#define BONSAI_B200_ETOOLARGE 2
int bonsai_b200_linear_static(const void *W, const float *x, const float *signs, float *y, int64_t n_out,
                              int64_t n_in, bonsai_stream stream);

/* y = silu(gate) * up, elementwise (src/ops.h:27-31; the reference has no entry point for it).  The unfused form of
 * BONSAI_B200_OP_SWIGLU below. */
int bonsai_b200_swiglu(const float *gate, const float *up, float *y, int64_t n, bonsai_stream stream);

/* Token batch for the mat-mul: X is fp32 [n_tok][n_in] (token-major); Xq receives the
 * chunk-major [n_in/32][n_tok] Q8_1 layout that bonsai_p40_gemm reads (the reference has no
 * entry point that produces it; its test builds it by hand, tests/test_p40.cpp:438-447).
 * With rotate != 0 every token is first rotated in blocks of 1024 (signs: NULL or n_in values
 * shared by all tokens).  Returns 1 if n_in % 32 != 0, or rotate and n_in % 1024 != 0. */
int bonsai_b200_quant_batch(const float *X, const float *signs, void *Xq, int64_t n_in, int64_t n_tok,
                            int rotate, bonsai_stream stream);

/* Parity probe: the int32 value (sum of code*activation) - (sum of activation) of every
 * 32-weight chunk of rows [row0, row0 + n_rows), written to out[n_rows][n_in/32].  These are
 * the integers the reference computes in src/pq2_0.h:149-169 before scaling. */
int bonsai_b200_gemv_chunk_sums(const void *W, const void *xq, int32_t *out, int64_t row0, int64_t n_rows,
                                int64_t n_in, bonsai_stream stream);

/* The tensor-core mat-vec with its integers written out: y as bonsai_p40_gemv computes it, and in sums[n_out][n_in/32]
 * the int32 chunk sums (sum of code * activation - sum of activation) that THIS kernel formed on the way -- the
 * parity probe of the production arithmetic (src/pq2_0.h:149-169).  Shapes: n_in / 128 even. */
int bonsai_b200_gemv_dump(const void *W, const void *xq, float *y, int32_t *sums, int64_t n_out, int64_t n_in,
                          bonsai_stream stream);

/* The tensor-core mat-mul with its integers written out: Y as bonsai_p40_gemm computes it on the tensor-core path,
 * and in sums[(row * n_tok + tok) * (n_in / 32) + chunk] the int32 value (sum of code * activation - sum of
 * activation) that the tensor core produced for that row, token and chunk -- the host loop's integers
 * (tests/test_p40.cpp:460-467).  For small cases: the dump is n_out * n_tok * n_in / 32 words. */
int bonsai_b200_gemm_dump(const void *W, const void *Xq, float *Y, int32_t *sums, int64_t n_out, int64_t n_in,
                          int64_t n_tok, bonsai_stream stream);

/* Makes sure that the scratch buffer which bonsai_p40_gemm keeps per (device, stream) for its tensor-core form is large
 * enough for n_tok tokens of n_in values (4 bytes each), allocating it now (cudaMalloc) if it is not.  Call it once,
 * outside stream capture, before capturing graphs that contain bonsai_p40_gemm on `stream`: a call that would have to
 * allocate during capture runs the integer tensor-core kernel instead, which needs no scratch and is slower.  Returns
 * 0, 1 for bad arguments, cudaErrorMemoryAllocation (2) when the buffer cannot be had.  No reference counterpart. */
int bonsai_b200_gemm_reserve(int64_t n_in, int64_t n_tok, bonsai_stream stream);

/* Frees every scratch buffer of bonsai_p40_gemm (all devices, all streams); they are otherwise kept for the life of the
 * process.  No mat-mul of this library may be in flight or captured in a graph that will still be replayed.  Returns 0. */
int bonsai_b200_gemm_release(void);

/* PTQ1_0: the denser packing of the same ternary weights, 28 bytes per 128 weights instead of 34 (described, not
 * implemented, by the reference: docs/NEXT_STEPS.md:76-83).  Block = qs[24] (five base-3 digits per byte, weights
 * 0..119), qh[2] (four digits per byte, weights 120..127), fp16 d; digit = PQ2_0 code 0, 1, 2; weight j < 120 is digit
 * j % 5 of byte j / 5, least significant first.  pack converts n_blocks PQ2_0 blocks (src, 34 bytes each) to PTQ1_0
 * (dst, 28 bytes each) and ADDS to *code3_count (device memory, 8-byte aligned, zeroed by the caller) the number of
 * weights whose code is 3 (+2, not representable; stored as +1): the conversion is lossless exactly when the count
 * stays 0.  unpack converts back to PQ2_0 blocks that the mat-vec / mat-mul entry points read.  Load-time steps. */
int bonsai_b200_ptq1_pack(const void *src, void *dst, int64_t n_blocks, uint64_t *code3_count, bonsai_stream stream);
int bonsai_b200_ptq1_unpack(const void *src, void *dst, int64_t n_blocks, bonsai_stream stream);

/* Synthetic PQ2_0 weights written on the device: n_blocks blocks whose codes are drawn per
 * element from {0,1,2} with p = {0.33,0.34,0.33} plus code 3 at p = 0.001, and whose fp16
 * scale is |z| * 0.02 with z approximately standard normal.  Counter-based: block i of a
 * call depends only on (seed, first_block + i). */
int bonsai_b200_synth_pq2_0(void *W, int64_t first_block, int64_t n_blocks, uint64_t seed, bonsai_stream stream);

/* Read-only streaming probe over `bytes` of device memory (16-byte aligned): mode 0 reads with
 * aligned 16-byte loads into registers, mode 1 with 1-D bulk async copies into a shared-memory ring
 * (the transport of the mat-vec, no arithmetic).  `sink` is 4 writable bytes.  Timed by the caller;
 * B200 counterpart of the reference's tools/bwtest.cu:37-90. */
int bonsai_b200_stream_probe(const void *buf, int64_t bytes, int mode, void *sink, bonsai_stream stream);

/* Launch options.  key "pdl": 1 = launch the mat-vec with programmatic stream serialisation,
 * so that its weight stream starts while the previous kernel of the stream drains (weights
 * must not be written by that previous kernel); 0 = plain launches (default).
 * key "gemv_order": 0 (default) = the streaming mat-vec, whose fp32 terms equal the host's bit for
 * bit and are added in a fixed tree order (outputs within 1e-5 of the host's, identical from launch
 * to launch); 1 = the mat-vec that also adds them in the host's sequential order (outputs
 * bit-identical to src/pq2_0.h:183-191, slower); 2 = the mat-vec whose integer products run on mma.sync
 * (csrc/gemv_mma.cuh: same terms, another fixed tree; measured slower than 0 at batch 1, kept as the measured
 * alternative and as the body of the 2 .. 16 token kernel).
 * key "gemm_path": -1 (default) = the mat-mul picks its kernel by token count (2 .. 8 tokens: the streaming
 * small-batch kernel, which also takes 9 .. 16 tokens when rows are a multiple of 8 blocks; otherwise 9 tokens and more: the
 * tensor cores; one token: the mat-vec of bonsai_p40_gemv), 0 = integer SIMT kernel (Y
 * bit-identical to the host loop), 1 = tensor cores (the fp16 form, csrc/gemm_tc16.cuh, where it takes the call,
 * else the integer form), 2 = the small-batch kernel where it takes the shape, 3 = the integer tensor-core kernel
 * (csrc/gemm_tc.cuh: forms the host's int32 chunk sums, needs no scratch).  1, 2 and 3 hold fp32 Y to 1e-5 of
 * max |Y|.  The fp16 form keeps one scratch buffer per (device, stream), 4 bytes per token and input value, allocated
 * with cudaMalloc on first use or growth -- never while the stream is being captured (then the integer form runs).
 * key "fuse_linear": 0 (default) = bonsai_b200_linear is two launches, 1 = one kernel when it can (saves a
 * launch, but every CTA then waits for its own rotation before its first multiply: measured ~6 % slower
 * on the 401-projection decode chain).
 * Options are process-wide: set them once at start-up, not from threads that call the library concurrently.
 * A library compiled with -DBONSAI_B200_TUNING (the test build) also takes geometry keys ("gemv_variant",
 * "chain_threads", "chain_seg", "chain_tile_kb", "chain_spread_nb", "gemm_tile") that force a tiling; they change no result bits
 * beyond what the documented options say and are not part of the interface.
 * Returns 0, or 1 for an unknown key. */
int bonsai_b200_set_option(const char *key, int64_t value);

/* Status word written by device-side bounded waits: 0 = no kernel of this library has given up on a
 * wait on the current device since the word was last cleared; 1 = a wait on a shared-memory barrier or
 * counter ran out; 2 = a wait for other CTAs or other ranks ran out (the launch still ends by itself and
 * the context stays usable; the outputs of that launch are incomplete).  Both calls synchronise the device
 * (cudaDeviceSynchronize), so neither may be made while a stream of the device is being captured.
 * Failures of the calls themselves come back as 1000 + the CUDA error code. */
int bonsai_b200_device_status(void);
int bonsai_b200_clear_status(void);

/* ---- a list of projections in one persistent launch (no counterpart in the reference) ---------
 * The reference launches one kernel per matrix (bonsai_p40_gemv, include/bonsai_p40.h:26-28).  On a
 * B200 a decode projection streams for 0.2 - 4 us, about as long as a kernel takes to start and drain,
 * so this entry point takes the whole list: weights of the next projection stream while the previous
 * one is multiplied, and only a projection that reads an earlier projection's output waits.
 *
 * Each op computes y = W . q(x): W as for bonsai_p40_gemv; x is either the permuted Q8_1 blocks of
 * the activation vector (as bonsai_p40_quant_activations / bonsai_b200_fwht_quant write them), or, with
 * BONSAI_B200_OP_ROTATE, the fp32 vector itself, which the kernel rotates (FWHT-1024, optional signs)
 * and quantises exactly as bonsai_b200_fwht_quant does.  y is bit-identical to bonsai_p40_gemv with
 * the default kernel.
 *   BONSAI_B200_OP_DEPENDS     x is written (as some y) by an earlier op of this list: the op starts
 *                              only when every row of every earlier op is in memory.  Needs OP_ROTATE
 *                              (ops write fp32).  Without this flag an op may start at any time, so x
 *                              must not be an output of the list.
 *   BONSAI_B200_OP_SAME_INPUT  same x (and kind) as the previous op: its quantised vector is reused.  An op that
 *                              names the same x, n_in, signs and kind as the op before it and does not say
 *                              OP_DEPENDS is treated this way without the flag.
 * Shapes: n_in a multiple of 256 (of 1024 with OP_ROTATE), W and x 16-byte aligned.
 * create() allocates a small device table (cudaMalloc) and copies the list; run() allocates nothing,
 * launches one cooperative kernel of one CTA per SM on `stream` (plus a 4-byte memset) and can be
 * captured in a CUDA graph; a chain object must not run on two streams at once.  Errors: 1 for a bad
 * argument, otherwise the CUDA error code. */
/* Producers (with OP_ROTATE, at most one per op): what turns the fp32 vector at x into the vector that is rotated and
 * quantised, fused into the op's prologue -- the step that precedes every projection of a decode step
 * (reference: src/ops.h:13-31; its device code runs them as kernels of their own, src/kernels/elementwise_p40.cu:48-88).
 *   BONSAI_B200_OP_RMSNORM     input = x * (1 / sqrt(mean(x^2) + eps)) * aux[0 .. n_in); n_in <= 7168.  Same bits as
 *                              bonsai_p40_rmsnorm followed by the op without the flag.
 *   BONSAI_B200_OP_SWIGLU      input = silu(x) * aux  (x = gate, aux = up, both n_in floats).  Same bits as
 *                              bonsai_b200_swiglu followed by the op without the flag.
 *   BONSAI_B200_OP_RESCALE     x is the whole output (src_len floats) of an earlier op of the list;
 *                              input[j] = x[j mod src_len] * 2^-e with e = floor(log2(max |x|)) (x unscaled if that
 *                              maximum is zero or subnormal): an exact, order-independent glue between the ops of a
 *                              synthetic decode step.  Needs OP_DEPENDS (or OP_SAME_INPUT after such an op); one-rank
 *                              lists only. */
#define BONSAI_B200_OP_ROTATE 1u
#define BONSAI_B200_OP_DEPENDS 2u
#define BONSAI_B200_OP_SAME_INPUT 4u
#define BONSAI_B200_OP_RMSNORM 8u
#define BONSAI_B200_OP_SWIGLU 16u
#define BONSAI_B200_OP_RESCALE 32u
typedef struct bonsai_b200_op {
    const void *W;
    const void *x;
    const float *signs;     /* OP_ROTATE only, may be NULL */
    float *y;
    int64_t n_out, n_in;
    uint32_t flags;
    uint32_t reserved;      /* 0 */
    const float *aux;       /* OP_RMSNORM: norm weights, OP_SWIGLU: the second vector; else NULL */
    float eps;              /* OP_RMSNORM; else 0 */
    uint32_t src_len;       /* OP_RESCALE: floats at x; else 0 */
} bonsai_b200_op;
typedef struct bonsai_b200_chain bonsai_b200_chain;
int bonsai_b200_chain_create(const bonsai_b200_op *ops, int64_t n_ops, bonsai_b200_chain **out);
int bonsai_b200_chain_run(bonsai_b200_chain *chain, bonsai_stream stream);
int bonsai_b200_chain_destroy(bonsai_b200_chain *chain);
/* The same list over the row slices of several GPUs (one process and one chain per GPU; no reference counterpart,
 * the reference is single-GPU).  Every rank passes the same list with ITS rows of every matrix (W, n_out of the
 * slice) and y pointing at its slice inside a buffer that every rank has allocated with the same layout and mapped
 * into every other rank (CUDA IPC or any other peer mapping): peer_base[q] is rank q's buffer as addressed from
 * this process (peer_base[rank] is the local one).  The kernel stores every y element it produces into all `world`
 * buffers, so each rank ends up with the whole vector without a collective, and OP_DEPENDS waits for every row of
 * every rank.  The buffer is buffer_bytes long on every rank; BONSAI_B200_TP_COUNTER_BYTES bytes at counter_offset
 * (a multiple of 64, behind every output) are the kernel's counters and flags: zero them once after allocation and
 * never touch them again.  Refused (1): an output that does not lie inside [buffer, buffer + counter_offset), a
 * counter block that does not fit in buffer_bytes, a mapping that is not 16-byte aligned.  Every rank must run on a
 * GPU with the same number of SMs.  All ranks must call run() the same number of times; the launches of different
 * ranks wait for each other, so each rank needs its own GPU.  The waits are bounded by wait_limit_us microseconds
 * (0 = one second): a rank that never comes makes the others give up, set the status word to 2 and return; a
 * chain that has given up must be destroyed and its counter block zeroed again before the buffer is reused.
 * Reading the outputs on the host needs the usual ordering between ranks: a peer's next run() overwrites them. */
#define BONSAI_B200_TP_COUNTER_BYTES 64
int bonsai_b200_chain_create_tp(const bonsai_b200_op *ops, int64_t n_ops, int rank, int world,
                                const void *const *peer_base, int64_t buffer_bytes, int64_t counter_offset,
                                int64_t wait_limit_us, bonsai_b200_chain **out);
/* kernels launched so far by run() on this chain's behalf, and its geometry (threads per CTA, ring
 * slots, bytes per slot, CTAs): for benchmarks and tests. */
int bonsai_b200_chain_info(const bonsai_b200_chain *chain, int64_t out[4]);

/* Device pointers of the K and V arrays of a cache made by bonsai_kv_create (include/bonsai_kv.h) and the size of
 * each: lets a test read the Q8_0 bytes back.  No counterpart in the reference, whose cache object is opaque. */
struct bonsai_kv_cache;
int bonsai_b200_kv_arrays(struct bonsai_kv_cache *kv, void **k, void **v, int64_t *bytes_each);

/* Version of this build as major * 100 + minor. */
int bonsai_b200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* BONSAI_B200_EXT_H */
