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

// Error word shared by the kernels that contain bounded waits.
struct DeviceStatus {
    int code;      // 0 = ok, otherwise where a wait gave up
    int detail;
};

}  // namespace tuna
