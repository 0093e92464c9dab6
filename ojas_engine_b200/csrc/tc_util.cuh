// Pieces shared by the kernels that use tcgen05 and TMA: mbarrier operations with bounded waits, tensor-map copies,
// shared-memory operand descriptors, commit and fences, and the driver's tensor-map encoder.  Everything is in an
// unnamed namespace: each translation unit that includes this file gets its own copy.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr long long WAIT_CYCLES = 4000000000LL;   // about two seconds
// A waiting thread that polls takes issue slots from the warps that work; the hint lets the hardware park it instead.
#ifndef OJAS_TRY_WAIT_HINT_NS
#define OJAS_TRY_WAIT_HINT_NS 20000u
#endif

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint64_t *bar, uint32_t parity) {   // non-blocking probe
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_try(uint64_t *bar, uint32_t parity) {    // suspends the thread until the phase completes or the hinted time passes
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(OJAS_TRY_WAIT_HINT_NS) : "memory");
    return ok != 0;
}

// Bounded wait.  Returns false if the CTA is aborting (this wait or another one ran out).  `nap` > 0 puts the
// thread to sleep for that many nanoseconds between probes: roles that wait for a whole tile must not compete
// with the working warps for issue slots.
__device__ __noinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, unsigned *status, unsigned code, unsigned nap) {
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; i++) {
            if (mbar_try(bar, parity)) return true;
            if (nap) __nanosleep(nap);
        }
        if (*abort_flag) return false;
        if (clock64() - t0 > WAIT_CYCLES) {
            *abort_flag = 1;
            atomicOr(status, code);
            __threadfence_system();
            return false;
        }
    }
}

// Single-thread roles (MMA issue, TMA) and warp leaders: one probe, then probes `nap` nanoseconds apart.  A
// thread that spins on a barrier takes issue slots from the dequantizing warps on its scheduler, and there are
// half a dozen waiting threads at any time; the short sleeps cost less than that contention.
constexpr unsigned OJAS_GEMM_NAP = 32u;
__device__ __forceinline__ bool mbar_wait_spin(uint64_t *bar, uint32_t parity, volatile int *abort_flag, unsigned *status, unsigned code,
                                               unsigned nap = OJAS_GEMM_NAP) {
    if (mbar_test(bar, parity)) return true;
    return mbar_wait(bar, parity, abort_flag, status, code, nap);
}

// Warp form.  The common case (the phase is already complete) is one probe by all lanes and a vote; otherwise
// lane 0 waits and the result is broadcast.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t *bar, uint32_t parity, volatile int *abort_flag, unsigned *status, unsigned code) {
    if (__all_sync(0xffffffffu, mbar_test(bar, parity))) return true;
    int ok = 1;
    if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, abort_flag, status, code, OJAS_GEMM_NAP) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    return ok != 0;
}
// The same for waits that are known to be long (a whole tile): one probe, then sleep between probes.
__device__ __forceinline__ bool mbar_wait_warp_long(uint64_t *bar, uint32_t parity, volatile int *abort_flag, unsigned *status, unsigned code) {
    int ok = 1;
    if ((threadIdx.x & 31) == 0) ok = (mbar_test(bar, parity) || mbar_wait(bar, parity, abort_flag, status, code, 256u)) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    return ok != 0;
}

__device__ __forceinline__ void tma_load_2d(void *smem_dst, const CUtensorMap *tmap, int x, int y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(smem_dst)), "l"((uint64_t)tmap), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}

__device__ __forceinline__ void tma_load_4d(void *smem_dst, const CUtensorMap *tmap, int c0, int c1, int c2, int c3, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                 ::"r"(smem_u32(smem_dst)), "l"((uint64_t)tmap), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}

// K-major operand tile with the 128-byte swizzle: rows of 128 bytes, groups of eight rows 1024
// bytes apart (stride byte offset), descriptor version 1, layout type 2.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);        // start address
    d |= (uint64_t)1 << 16;                              // leading byte offset (unused with a swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;                    // stride byte offset
    d |= (uint64_t)1 << 46;                              // descriptor version
    d |= (uint64_t)2 << 61;                              // 128-byte swizzle
    return d;
}

__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }


// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

}  // namespace
