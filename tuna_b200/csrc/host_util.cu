// Host-side helpers shared by the pipeline kernels' launchers: the per-device status word that
// bounded waits report into, and TMA tensor-map construction through the driver entry point
// (resolved at run time, so the library does not link against libcuda).
#include <mutex>
#include "common.cuh"
#include "launchers.h"
#include "sm100_ptx.cuh"

namespace tuna {

DeviceStatus *device_status_word()
{
    static DeviceStatus *ptrs[64] = {nullptr};
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!ptrs[dev]) {
        DeviceStatus *p = nullptr;
        if (cudaMalloc(&p, sizeof(DeviceStatus)) != cudaSuccess) return nullptr;
        cudaMemset(p, 0, sizeof(DeviceStatus));
        ptrs[dev] = p;
    }
    return ptrs[dev];
}

int read_device_status(cudaStream_t stream)
{
    DeviceStatus *d = device_status_word();
    if (!d) return TUNA_ERR_NO_DEVICE;
    DeviceStatus h;
    if (cudaMemcpyAsync(&h, d, sizeof(h), cudaMemcpyDeviceToHost, stream) != cudaSuccess) return TUNA_ERR_LAUNCH;
    if (cudaStreamSynchronize(stream) != cudaSuccess) return TUNA_ERR_LAUNCH;
    if (h.code != 0) {
        cudaMemsetAsync(d, 0, sizeof(DeviceStatus), stream);
        return TUNA_ERR_DEVICE_TIMEOUT;
    }
    return TUNA_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)ptr;
    });
    return fn;
}

bool make_tensor_map_2d(CUtensorMap *map, CUtensorMapDataType dt, const void *base, uint64_t inner, uint64_t outer,
                        uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swizzle)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {row_stride_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, dt, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Three dimensions, innermost first: extents d0, d1, d2; byte strides of d1 and d2 (any order).
bool make_tensor_map_3d(CUtensorMap *map, CUtensorMapDataType dt, const void *base, uint64_t d0, uint64_t d1, uint64_t d2,
                        uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0, uint32_t box1, uint32_t box2,
                        CUtensorMapSwizzle swizzle)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[3] = {d0, d1, d2};
    cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
    cuuint32_t box[3] = {box0, box1, box2};
    cuuint32_t estr[3] = {1, 1, 1};
    return fn(map, dt, 3, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Any rank up to 5, innermost dimension first; `strides` are the byte strides of dimensions 1 .. rank-1.
bool make_tensor_map_nd(CUtensorMap *map, CUtensorMapDataType dt, const void *base, int rank, const uint64_t *dims,
                        const uint64_t *strides, const uint32_t *box, CUtensorMapSwizzle swizzle)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn || rank < 1 || rank > 5) return false;
    cuuint64_t d[5], s[4];
    cuuint32_t b[5], e[5];
    for (int i = 0; i < rank; ++i) { d[i] = dims[i]; b[i] = box[i]; e[i] = 1; }
    for (int i = 0; i + 1 < rank; ++i) s[i] = strides[i];
    return fn(map, dt, (cuuint32_t)rank, const_cast<void *>(base), d, s, b, e, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace tuna

// ------------------------------------------------------------------ self-test of the bounded waits
//
// Every mbarrier wait of the pipeline kernels gives up after a time limit, records where in the
// device status word and lets the kernel unwind (tuna_check_device_status then reports
// TUNA_ERR_DEVICE_TIMEOUT).  This entry point exercises exactly that path without a real failure:
// one warp waits, with a limit of about a millisecond, on a barrier that nothing ever arrives at.
namespace tuna {
__global__ void bounded_wait_selftest_kernel(DeviceStatus *status, long long limit_cycles)
{
    __shared__ __align__(8) uint64_t bar;
    __shared__ int s_abort;
    if (threadIdx.x == 0) {
        s_abort = 0;
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // phase 0 of a barrier that expects one arrival and never gets it
    if (!mbar_try_wait(smem_u32(&bar), 0)) mbar_wait_slow(smem_u32(&bar), 0, &s_abort, status, 99, limit_cycles);
}
}  // namespace tuna

extern "C" int tuna_selftest_bounded_wait(void *stream)
{
    tuna::DeviceStatus *d = tuna::device_status_word();
    if (!d) return TUNA_ERR_NO_DEVICE;
    tuna::bounded_wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(d, 2000000ll);  // ~1 ms
    return cudaGetLastError() == cudaSuccess ? TUNA_OK : TUNA_ERR_LAUNCH;
}
