// common.cuh -- device helpers shared by every kernel of the sm_100a build.
//
// Arithmetic rules (they make the device output equal the reference's HOST code bit for bit):
//   * every fp32 operation that the host performs is issued as one explicit IEEE operation
//     (__fmul_rn / __fadd_rn / __fdiv_rn), so the compiler can neither fuse nor approximate it;
//   * fp32 -> fp16 uses the host's ties-away rule, not the hardware ties-to-even conversion;
//   * float -> int uses ties-away (lroundf semantics), not ties-to-even.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

constexpr int W_BLOCK_BYTES = 34;   // PQ2_0 block: fp16 scale + 32 code bytes (128 weights)
constexpr int A_BLOCK_BYTES = 36;   // Q8_1 block: fp16 scale + int16 sum + 32 int8
constexpr int FWHT_N = 1024;

// Sticky status word: bounded waits write a non-zero code here instead of spinning forever.
__device__ int g_device_status = 0;

enum : int { STATUS_OK = 0, STATUS_MBARRIER_TIMEOUT = 1, STATUS_GRID_TIMEOUT = 2 };

// ---- fp16 <-> fp32 -------------------------------------------------------------------------
__device__ __forceinline__ float f16_bits_to_f32(uint32_t h) {
    return __half2float(__ushort_as_half((unsigned short)h));   // exact widening
}

// Host rule of the reference (src/p40_common.h:91-112): the first dropped mantissa bit alone
// decides the bump, i.e. nearest with ties away from zero; subnormals and overflow included.
__device__ __forceinline__ uint32_t f32_to_f16_bits_ties_away(float f) {
    const uint32_t x = __float_as_uint(f);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const uint32_t e8 = (x >> 23) & 255u;
    const uint32_t frac = x & 0x7FFFFFu;
    if (e8 == 255u) return sign | 0x7C00u | (frac ? 0x200u : 0u);
    int e = (int)e8 - 112;
    if (e >= 31) return sign | 0x7C00u;
    if (e <= 0) {
        if (e < -10) return sign;
        const uint32_t full = frac | 0x800000u;
        const uint32_t sh = (uint32_t)(14 - e);
        return sign | ((full >> sh) + ((full >> (sh - 1)) & 1u));
    }
    uint32_t q = (frac >> 13) + ((frac >> 12) & 1u);
    if (q == 1024u) { q = 0; e += 1; if (e >= 31) return sign | 0x7C00u; }
    return sign | ((uint32_t)e << 10) | q;
}

// lroundf semantics for |t| < 2^23 (a NaN gives 0, as the host's conversion does on x86-64).
__device__ __forceinline__ int round_ties_away(float t) {
    const float r = truncf(t);
    const float frac = __fsub_rn(t, r);          // exact
    int q = (t == t) ? (int)r : 0;
    if (fabsf(frac) >= 0.5f) q += (t < 0.0f) ? -1 : 1;
    return q;
}

// ---- integer dot ------------------------------------------------------------------------------
// Four unsigned bytes of `w` times four signed bytes of `a`, plus c (reference: the host dp4a
// emulation, src/p40_common.h:131-140, applied to codes 0..3 which are non-negative either way).
__device__ __forceinline__ int dp4a_us(uint32_t w, int a, int c) {
    int r;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(r) : "r"(w), "r"(a), "r"(c));
    return r;
}

// Sum over one 32-weight chunk of code * activation.  w0 / w1 are the two 16-code words, a[0..7] the
// eight activation words of the permuted Q8_1 block: field k of word w pairs with activation word
// 4w + k (src/pq2_0.h:155-166).  Fields are masked in place, so the four field sums come out scaled
// by 64, 16, 4 and 1; they are four independent dp4a chains (the scheduler can overlap them), joined
// as (s3 + 4 s2 + 16 s1 + 64 s0) >> 6, which is exact because the sum is a multiple of 64.  Callers
// pass init64 = -64 * s so that the result is (sum code*a) - s.
__device__ __forceinline__ int chunk_sumi_scaled(uint32_t w0, uint32_t w1, const int (&a)[8], int init64) {
    int s3 = dp4a_us(w0 & 0xC0C0C0C0u, a[3], init64);
    int s2 = dp4a_us(w0 & 0x30303030u, a[2], 0);
    int s1 = dp4a_us(w0 & 0x0C0C0C0Cu, a[1], 0);
    int s0 = dp4a_us(w0 & 0x03030303u, a[0], 0);
    s3 = dp4a_us(w1 & 0xC0C0C0C0u, a[7], s3);
    s2 = dp4a_us(w1 & 0x30303030u, a[6], s2);
    s1 = dp4a_us(w1 & 0x0C0C0C0Cu, a[5], s1);
    s0 = dp4a_us(w1 & 0x03030303u, a[4], s0);
    return (s3 + (s2 << 2) + (s1 << 4) + (s0 << 6)) >> 6;
}

// ---- shared-memory barriers and bulk copies (sm_90+ PTX, every copy is local to its CTA) -------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait: returns false (and records the status word) instead of spinning forever.  The
// barrier is polled with the non-blocking test; between polls the thread sleeps first_ns, 2 first_ns, ... max_ns,
// which keeps a waiting warp off the issue ports (the blocking form of the wait expands to a
// software time-out loop of a couple of dozen instructions per poll).
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity, uint32_t first_ns = 32,
                                                  uint32_t max_ns = 256) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .u32 n, ns;\n\t"
        "mov.u32 n, %3;\n\t"
        "mov.u32 ns, %4;\n\t"
        "mov.u32 %0, 1;\n\t"
        "WAIT_LOOP:\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "@p bra WAIT_DONE;\n\t"
        "nanosleep.u32 ns;\n\t"
        "add.u32 ns, ns, ns;\n\t"
        "min.u32 ns, ns, %5;\n\t"
        "sub.u32 n, n, 1;\n\t"
        "setp.ne.u32 p, n, 0;\n\t"
        "@p bra WAIT_LOOP;\n\t"
        "mov.u32 %0, 0;\n\t"
        "WAIT_DONE:\n\t"
        "}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(1u << 22), "r"(first_ns), "r"(max_ns)
        : "memory");
    if (!ok) atomicExch(&g_device_status, STATUS_MBARRIER_TIMEOUT);
    return ok != 0;
}
// The same wait for a barrier that is expected within a fraction of a microsecond (a tensor-core result, a stage a
// neighbouring role is about to hand over): polls back to back first, and sleeps between polls only when that did
// not help.  Bounded like the one above.
__device__ __forceinline__ bool mbar_wait_hot(uint64_t *bar, uint32_t parity) {
    uint32_t ok = 0;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .u32 n;\n\t"
        "mov.u32 n, 512;\n\t"
        "mov.u32 %0, 1;\n\t"
        "HOT_LOOP:\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "@p bra HOT_DONE;\n\t"
        "sub.u32 n, n, 1;\n\t"
        "setp.ne.u32 p, n, 0;\n\t"
        "@p bra HOT_LOOP;\n\t"
        "mov.u32 %0, 0;\n\t"
        "HOT_DONE:\n\t"
        "}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    if (ok) return true;
    return mbar_wait_bounded(bar, parity, 32, 128);
}
// One non-blocking poll: has the phase with this parity completed?
__device__ __forceinline__ bool mbar_test(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// 1-D bulk copy global -> shared of `bytes` (multiple of 16, both addresses 16-byte aligned),
// completion counted on `bar`.
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
        ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}
__device__ __forceinline__ uint64_t policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t policy_evict_normal() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(p));
    return p;
}
// Cache policy for data that many CTAs re-read (activation blocks of a token tile): keep it in L2.
__device__ __forceinline__ uint64_t policy_evict_last_or_default() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
// Programmatic dependent launch: both are no-ops unless the launch carries the attribute.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait_prior_grid() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ uint32_t ldg_nc_u32(const void *p) {
    uint32_t v;
    asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ldg_nc_u16(const void *p) {
    unsigned short v;
    asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}

}  // namespace b200
