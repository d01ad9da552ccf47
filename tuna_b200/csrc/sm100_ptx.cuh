// mbarrier / TMA wrappers and the bounded-wait protocol shared by the sm_100a pipeline kernels.
#pragma once
#include <cuda.h>
#include "common.cuh"

namespace tuna {

constexpr long long kWaitCycles = 4000000000ll;  // ~2 s at 1.9 GHz

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Non-blocking poll (mbarrier.try_wait may suspend the thread for a system-dependent time before
// it answers false; test_wait answers at once).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait.  Returns false when the time limit ran out or another role raised the abort
// flag; the caller unwinds.
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                            DeviceStatus *status, int where, long long limit = kWaitCycles)
{
    const long long t0 = clock64();
    for (;;) {
        for (int i = 0; i < 64; ++i) {
            if (mbar_try_wait(bar, parity)) return true;
#ifdef TUNA_WAIT_BACKOFF
            __nanosleep(TUNA_WAIT_BACKOFF);  // leave the issue slots to the warps that have work
#endif
        }
        if (*abort_flag) return false;
        if (clock64() - t0 > limit) {
            *abort_flag = 1;
            if (atomicCAS(&status->code, 0, where) == 0) status->detail = (int)blockIdx.x;
            return false;
        }
    }
}

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                          DeviceStatus *status, int where)
{
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, abort_flag, status, where);
}

// The same wait executed by a whole converged warp, with one answer for all its lanes.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                               DeviceStatus *status, int where)
{
    return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, status, where)) != 0;
}

// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool elect_one_sync()
{
    uint32_t e;
    asm volatile("{\n .reg .pred P;\n elect.sync _|P, 0xffffffff;\n selp.u32 %0, 1, 0, P;\n}" : "=r"(e));
    return e != 0;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int c0, int c1, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, int c0, int c1, int c2, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap *map, int c0, int c1, int c2, int c3, int c4, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(bar)
        : "memory");
}

// Position in a ring of n mbarrier-guarded buffers: slot index and the parity of its current use.
struct Ring {
    int idx;
    uint32_t phase;
    __device__ Ring() : idx(0), phase(0) {}
    __device__ void advance(int n)
    {
        if (++idx == n) { idx = 0; phase ^= 1u; }
    }
};

// The CTA i whose contiguous range [floor(i*U/G), floor((i+1)*U/G)) holds unit u.
__device__ __forceinline__ int cta_of_unit(long long u, long long units, int ctas)
{
    return (int)(((u + 1) * ctas + units - 1) / units) - 1;
}

}  // namespace tuna
