// Standalone dequantisation kernel for sm_100a: packed 4-bit codes -> fp16.
//
// Replaces the reference's dequantize_4bit (kernel.cu:3158-3241) and is
// bit-exact to it: out = (half)(code[nibble] * absmax[row]) with the multiply
// in fp32 (kernel.cu:3223-3228).  HBM-bound: reads m*k/2 bytes, writes 2*m*k.
//
// Mapping: one warp owns one 8-row group and walks along K.  A lane reads 16
// packed bytes (half of an 8x8 tile: 4 rows x 8 columns) with one 128-bit
// load, looks every nibble up in a per-row 16-entry fp16 table held in shared
// memory (built once per warp with the fp32 multiply), and writes four 16-byte
// row segments.  Across a warp each of those stores covers 256 contiguous
// bytes per row.
#include "common.cuh"
#include "launchers.h"

namespace tuna {

constexpr int kDqWarps = 8;

__global__ void __launch_bounds__(kDqWarps * 32)
dequant_w4_kernel(const uint8_t *__restrict__ q, const float *__restrict__ absmax,
                  const float *__restrict__ code, __half *__restrict__ out, int m, int k,
                  int tiles_per_split)
{
    __shared__ __align__(16) __half lut[kDqWarps][8][kCodeSize];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rg = blockIdx.x * kDqWarps + warp;  // 8-row group
    const int n_rg = m >> 3, n_kt = k >> 3;
    if (rg < n_rg) {
        // 128 table entries per warp, 4 per lane: row = e / 16, nibble = e % 16
        for (int e = lane; e < 8 * kCodeSize; e += 32) {
            float v = code[e & 15] * absmax[rg * 8 + (e >> 4)];
            lut[warp][e >> 4][e & 15] = __float2half_rn(v);
        }
    }
    __syncwarp();
    if (rg >= n_rg) return;

    const int kt_begin = blockIdx.y * tiles_per_split;
    const int kt_end = min(n_kt, kt_begin + tiles_per_split);
    const int half_sel = lane & 1;  // which 4 rows of the tile this lane holds
    const uint8_t *src_rg = q + (size_t)rg * row_group_bytes(k);
    const __half *my_lut = &lut[warp][half_sel * 4][0];
    __half *dst_rows = out + (size_t)(rg * 8 + half_sel * 4) * k;

    for (int kt = kt_begin + (lane >> 1); kt < kt_end; kt += 16) {
        uint4 v = ldg_stream_u4(src_rg + (size_t)kt * 32 + half_sel * 16);
        const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {  // row 4*half_sel + i, columns 8kt .. 8kt+7
            const uint32_t w = words[i];
            const __half *l = my_lut + i * kCodeSize;
            uint32_t o[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const uint32_t byte = (w >> (8 * b)) & 0xffu;
                const __half hi = l[byte >> 4];  // even column: high nibble
                const __half lo = l[byte & 15];
                o[b] = (uint32_t)__half_as_ushort(hi) | ((uint32_t)__half_as_ushort(lo) << 16);
            }
            *reinterpret_cast<uint4 *>(dst_rows + (size_t)i * k + (size_t)kt * 8) =
                make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
}

cudaError_t launch_dequant(const void *q, const void *absmax, const void *code, void *o, int m,
                           int k, int sm_count, cudaStream_t stream)
{
    const int n_rg = m / 8, n_kt = k / 8;
    const int gx = div_up(n_rg, kDqWarps);
    // enough CTAs to fill the machine a few times over, at least 16 tiles (one warp pass) each
    int want_y = div_up(sm_count * 8, gx);
    int max_y = div_up(n_kt, 16);
    int gy = max(1, min(want_y, max_y));
    int tiles_per_split = div_up(div_up(n_kt, gy), 16) * 16;
    gy = div_up(n_kt, tiles_per_split);
    dequant_w4_kernel<<<dim3(gx, gy), kDqWarps * 32, 0, stream>>>(
        (const uint8_t *)q, (const float *)absmax, (const float *)code, (__half *)o, m, k,
        tiles_per_split);
    return cudaGetLastError();
}

}  // namespace tuna
