// Link-compatible definitions of the two native symbols the reference's pybind module declares
// and calls (extension.cpp:22-24, 34-37, 46-48): `wrapper` (kernel.cu:3009) and
// `dequantize_wrapper` (kernel.cu:3243), C++ linkage, same parameter lists.  A build of the
// reference's extension.cpp that links this library instead of compiling kernel.cu/configs.cu
// gets the sm_100a kernels with no source change.
//
// The reference has no workspace argument (its split-K accumulates into `o` with fp16 atomics,
// kernel.cu:2739-2745) and reports no errors.  Here the workspace is a cached allocation per
// (device, stream) - the reference's wrapper may run concurrently on different streams, and two
// overlapping calls must not share arrival counters - zero-filled on that stream when it is
// created.  A buffer that has been handed to a launch is never freed (an earlier call or a
// captured graph may still refer to it): when a larger one is needed the old one is kept.
// Allocation is impossible while the stream is being captured; the call then fails with
// TUNA_ERR_WORKSPACE unless an earlier, uncaptured call on that stream already created a large
// enough buffer.  The status of the calling thread's last call can be read with
// tuna_last_wrapper_status().
#include <cuda_runtime.h>
#include <map>
#include <mutex>
#include <utility>
#include <vector>
#include "../../include/tuna_b200.h"

namespace {

struct StreamScratch {
    void *ptr = nullptr;
    size_t bytes = 0;
};
std::map<std::pair<int, cudaStream_t>, StreamScratch> g_scratch;
std::vector<void *> g_retired;  // outgrown buffers, kept alive on purpose
std::mutex g_scratch_mutex;
thread_local int t_last_status = TUNA_OK;

// The cached workspace of (current device, stream), at least `need` bytes.
void *scratch_for(size_t need, cudaStream_t stream, size_t *bytes)
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    StreamScratch &s = g_scratch[std::make_pair(dev, stream)];
    if (s.bytes < need) {
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) return nullptr;
        const size_t want = need < (size_t(32) << 20) ? (size_t(32) << 20) : need;
        void *p = nullptr;
        if (cudaMalloc(&p, want) != cudaSuccess) return nullptr;
        if (cudaMemsetAsync(p, 0, want, stream) != cudaSuccess) { cudaFree(p); return nullptr; }  // never launched on: safe to free
        if (s.ptr) g_retired.push_back(s.ptr);
        s.ptr = p;
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
    void *ws = scratch_for(need, stream, &bytes);
    if (!ws) { t_last_status = TUNA_ERR_WORKSPACE; return; }
    t_last_status = tuna_matmul(q, x, c, s, o, m, n, k, ws, bytes, (void *)stream);
}

// kernel.cu:3243
void dequantize_wrapper(void *q, void *a, void *c, void *o, const int m, const int k, cudaStream_t stream)
{
    t_last_status = tuna_dequant(q, a, c, o, m, k, (void *)stream);
}

extern "C" int tuna_last_wrapper_status(void) { return t_last_status; }
