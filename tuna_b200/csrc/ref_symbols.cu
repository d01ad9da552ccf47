// Link-compatible definitions of the two native symbols the reference's pybind module declares
// and calls (extension.cpp:22-24, 34-37, 46-48): `wrapper` (kernel.cu:3009) and
// `dequantize_wrapper` (kernel.cu:3243), C++ linkage, same parameter lists.  A build of the
// reference's extension.cpp that links this library instead of compiling kernel.cu/configs.cu
// gets the sm_100a kernels with no source change.
//
// The reference has no workspace argument (its split-K accumulates into `o` with fp16 atomics,
// kernel.cu:2739-2745) and reports no errors.  Here the workspace is one cached allocation per
// device, grown on demand and zero-filled once; the status of the last call of the calling
// thread can be read with tuna_last_wrapper_status().
#include <cuda_runtime.h>
#include <mutex>
#include "../../include/tuna_b200.h"

namespace {

struct DeviceScratch {
    void *ptr = nullptr;
    size_t bytes = 0;
};
DeviceScratch g_scratch[64];
std::mutex g_scratch_mutex;
thread_local int t_last_status = TUNA_OK;

// The cached workspace of the current device, at least `need` bytes.  Growing it waits for the
// device (the old buffer may be in use by an earlier call) - a rare, one-time cost per size.
void *scratch_for(size_t need, size_t *bytes)
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    DeviceScratch &s = g_scratch[dev];
    if (s.bytes < need) {
        if (cudaDeviceSynchronize() != cudaSuccess) return nullptr;
        if (s.ptr) cudaFree(s.ptr);
        s.ptr = nullptr;
        s.bytes = 0;
        size_t want = need < (size_t(32) << 20) ? (size_t(32) << 20) : need;
        if (cudaMalloc(&s.ptr, want) != cudaSuccess) { s.ptr = nullptr; return nullptr; }
        if (cudaMemset(s.ptr, 0, want) != cudaSuccess) { cudaFree(s.ptr); s.ptr = nullptr; return nullptr; }
        s.bytes = want;
    }
    *bytes = s.bytes;
    return s.ptr;
}

}  // namespace

// kernel.cu:3009 - note the native argument order (q, x, c, s, o), not the Python one
void wrapper(void *q, void *x, void *c, void *s, void *o, int m, int n, int k, cudaStream_t stream)
{
    const size_t need = tuna_matmul_workspace_bytes(m, n, k);
    if (need == 0) { t_last_status = TUNA_ERR_BAD_SHAPE; return; }
    size_t bytes = 0;
    void *ws = scratch_for(need, &bytes);
    if (!ws) { t_last_status = TUNA_ERR_WORKSPACE; return; }
    t_last_status = tuna_matmul(q, x, c, s, o, m, n, k, ws, bytes, (void *)stream);
}

// kernel.cu:3243
void dequantize_wrapper(void *q, void *a, void *c, void *o, const int m, const int k, cudaStream_t stream)
{
    t_last_status = tuna_dequant(q, a, c, o, m, k, (void *)stream);
}

extern "C" int tuna_last_wrapper_status(void) { return t_last_status; }
