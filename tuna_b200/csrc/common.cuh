// Shared device/host helpers for the sm_100a kernels of tuna_b200.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tuna {

constexpr int kCodeSize = 16;  // entries of the codebook (configs.cu:41 of the reference: codeSize = 16)

__host__ __device__ constexpr int div_up(int a, int b) { return (a + b - 1) / b; }
__host__ __device__ constexpr long long div_up_ll(long long a, long long b) { return (a + b - 1) / b; }

// Packed-weight strides in bytes (reference kernel.cu:3171): one 8x8 tile is 32
// bytes, one 8-row group is k/8 tiles = 4k bytes.
__host__ __device__ inline size_t row_group_bytes(int k) { return (size_t)k * 4; }

__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 128-bit streaming load: weights are read exactly once, keep them out of L1.
__device__ __forceinline__ uint4 ldg_stream_u4(const void *p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi)
{
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}

// The byte -> half2 dequantisation table: 256 entries (one per packed byte = two codes) at a
// 256-byte stride, 32 copies of an entry side by side (one per bank), at a 64-KB-aligned
// shared address.  ONE prmt then builds a lookup's whole address (table base | byte << 8 |
// lane * 4, `lane_key` holding the first and last part) and every lookup is conflict free.
constexpr int kLut64Bytes = 65536;

__device__ __forceinline__ uint32_t lut_lookup(uint32_t w, uint32_t lane_key, uint32_t selector)
{
    // result bytes: [0] = lane*4, [1] = the selected byte of w, [2..3] = upper address bytes
    uint32_t addr, v;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(addr) : "r"(w), "r"(lane_key), "r"(selector));
    // not volatile: the table is constant once built, so the compiler may schedule lookups freely
    asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

// 128-bit streaming load under a predicate (zeros when the predicate is false), without a branch.
__device__ __forceinline__ uint4 ldg_stream_pred(const void *p, unsigned pred)
{
    uint4 v;
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %5, 0;\n"
        " mov.b32 %0, 0;\n mov.b32 %1, 0;\n mov.b32 %2, 0;\n mov.b32 %3, 0;\n"
        " @p ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];\n}"
        : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
        : "l"(p), "r"(pred));
    return v;
}

// Error word shared by the kernels that contain bounded waits.
struct DeviceStatus {
    int code;      // 0 = ok, otherwise where a wait gave up
    int detail;
};

}  // namespace tuna
