/*
 * sampler_device.cuh — small device helpers shared by the sampling kernels:
 * the reference generator (src/engine/sampler.c:27-48 of geistlib), ordered
 * keys, exact exponentials for the entries that decide a draw, warp sums and
 * the mbarrier / bulk-copy wrappers (every copy goes to the issuing CTA's own
 * shared memory).
 */
#pragma once
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "sampler_params.h"

namespace gb {

__device__ __forceinline__ unsigned order_key(float x) {
    /* monotone map float -> uint32 (larger float, larger key); -0 and +0 are one value, as the
     * comparison of floats has it (x + 0 turns -0 into +0 and leaves everything else alone) */
    unsigned b = __float_as_uint(x + 0.0f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ unsigned long long xorshift_next(unsigned long long &s) {
    s ^= s >> 12;
    s ^= s << 25;
    s ^= s >> 27;
    return s * 0x2545F4914F6CDD1DULL;
}

__device__ __forceinline__ float unit_from(unsigned long long r) {
    return (float) (unsigned) (r >> 40) * (1.0f / 16777216.0f);
}

/* expf of the reference, for the few entries that decide a draw: the double
 * exponential rounded once to binary32 (what a correctly rounded expf gives). */
__device__ __forceinline__ float exp_exact(float a) { return __double2float_rn(exp((double) a)); }

/* 2^y by the special-function unit (two ulp, flushes denormals, 2^-inf = 0): for the bulk sums of the
 * stream kernel only, where thirty-two exponentials per thread and slice are on the critical path and a
 * relative error of 1e-7 in a sum of 10^5 terms moves no draw that is not within 1e-7 of a step already. */
__device__ __forceinline__ float exp2_fast(float y) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(y));
    return r;
}

__device__ __forceinline__ float scaled_arg(float x, float m, float inv_t) {
    return __fmul_rn(__fsub_rn(x, m), inv_t); /* two roundings, never fused */
}

__device__ __forceinline__ bool pair_before(float av, int ai, float bv, int bi) {
    return av > bv || (av == bv && ai < bi);
}

__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        v += __shfl_xor_sync(0xffffffffu, v, o);
    }
    return v;
}

__device__ __forceinline__ long long warp_sum_ll(long long v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        v += __shfl_xor_sync(0xffffffffu, v, o);
    }
    return v;
}

/* mbarrier + bulk copy (global -> this CTA's shared memory only) */
__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned) __cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long *bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

/* Several barriers, then one pair of fences for all of them. */
__device__ __forceinline__ void mbar_init_only(unsigned long long *bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(unsigned long long *bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

/* One 32-bit word from global to shared memory without passing through a register of the caller;
 * complete for the issuing thread after async_copies_wait(). */
__device__ __forceinline__ void copy_word_async(void *dst_shared, const void *src_global) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned) __cvta_generic_to_shared(dst_shared)), "l"(src_global) : "memory");
}
__device__ __forceinline__ void async_copies_wait() {
    asm volatile("cp.async.wait_all;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(unsigned long long *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, unsigned bytes, unsigned long long *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

/* Asks for a run of global memory to be brought into L2 (nothing is read and there is no completion to wait
 * for; address and size on the 16-byte grid). */
__device__ __forceinline__ void bulk_prefetch_l2(const void *src, unsigned bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(unsigned long long *bar, unsigned parity) {
    unsigned ok;
    asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(smem_u32(bar)), "r"(parity)
            : "memory");
    return ok != 0;
}

/* Non-blocking test of a phase (try_wait may suspend the thread for a while). */
__device__ __forceinline__ bool mbar_test(unsigned long long *bar, unsigned parity) {
    unsigned ok;
    asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(smem_u32(bar)), "r"(parity)
            : "memory");
    return ok != 0;
}

/* Bounded wait: gives up kWaitLimitNs after it began (one second of %globaltimer; the count of rounds is a
 * second limit, should the timer not advance). Returns false when the copy never signalled; the caller then
 * stops asking for copies and reports the rows it touches as not loaded. */
constexpr unsigned long long kWaitLimitNs = 1000000000ull;
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool mbar_wait_bounded(unsigned long long *bar, unsigned parity) {
    if (mbar_try_wait(bar, parity)) {
        return true;
    }
    const unsigned long long t0 = global_ns();
    for (int round = 0; round < (1 << 22); round++) {
        for (int i = 0; i < 64; i++) {
            if (mbar_try_wait(bar, parity)) {
                return true;
            }
        }
        if (global_ns() - t0 > kWaitLimitNs) {
            return false;
        }
    }
    return false;
}


/* (key, id) packed so that a larger word comes earlier in (key desc, id asc). */
__device__ __forceinline__ unsigned long long composite(unsigned key, int gid, int idx_bits) {
    const unsigned long long mask = (1ull << idx_bits) - 1ull;
    return ((unsigned long long) key << idx_bits) | (mask - (unsigned long long) gid);
}

} /* namespace gb */
