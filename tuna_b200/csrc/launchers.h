// Internal launcher interface between the C ABI (tuna_api.cu) and the kernels.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>
#include "../../include/tuna_b200.h"

namespace tuna {

struct GemmArgs {
    const uint8_t *q;
    const void *x;       // fp16 [n, k]
    const float *code;   // [16]
    const float *absmax; // [m]
    void *o;             // fp16 [n, m]
    int m, n, k;
    void *workspace;
    size_t workspace_bytes;
    cudaStream_t stream;
    int sm_count;
    // strided batch of independent GEMMs of one shape (streaming kernel only); strides in bytes
    int batch = 1;
    size_t q_stride = 0, x_stride = 0, absmax_stride = 0, o_stride = 0;
};

// Workspace layout shared by both GEMM kernels: [split-K partial tiles: a region of fixed size]
// [arrival counters].  The partial region has the same size for every shape and configuration
// (two slots per CTA, a slot as large as the largest tile either kernel can be configured with),
// so the counters of any call lie beyond every byte an earlier call may have written partials
// to: one zero-initialised workspace can be shared by calls of any shapes, the counters being
// the only part that must be zero and every call leaving them zero.
constexpr size_t kMaxPartialSlotBytes = 192 * 1024;  // tcgen05 kernel: 128 rows x 384 accumulator columns x 4 bytes
inline size_t partial_region_bytes(int sm_count) { return 2 * (size_t)sm_count * kMaxPartialSlotBytes; }

struct DeviceStatus;
// One zero-initialised status word per device; bounded in-kernel waits report into it.
DeviceStatus *device_status_word();
int read_device_status(cudaStream_t stream);
bool make_tensor_map_2d(CUtensorMap *map, CUtensorMapDataType dt, const void *base, uint64_t inner, uint64_t outer,
                        uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swizzle);
bool make_tensor_map_3d(CUtensorMap *map, CUtensorMapDataType dt, const void *base, uint64_t d0, uint64_t d1, uint64_t d2,
                        uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0, uint32_t box1, uint32_t box2,
                        CUtensorMapSwizzle swizzle);
bool make_tensor_map_nd(CUtensorMap *map, CUtensorMapDataType dt, const void *base, int rank, const uint64_t *dims,
                        const uint64_t *strides, const uint32_t *box, CUtensorMapSwizzle swizzle);

cudaError_t launch_quantize(const void *w, const void *code, void *q, void *absmax, int m, int k, int sm_count,
                            cudaStream_t stream);
cudaError_t launch_dequant(const void *q, const void *absmax, const void *code, void *o, int m,
                           int k, int sm_count, cudaStream_t stream);

// mma.sync weight-streaming kernel.  Returns a tuna_status.
int launch_gemm_stream(const GemmArgs &a, const tuna_config &cfg);
size_t gemm_stream_workspace_bytes(int m, int n, int k, const tuna_config &cfg, int sm_count, int batch = 1);
int gemm_stream_normalize_config(int m, int n, int k, int sm_count, tuna_config *cfg);
// The same launches with a caller-provided scratch in a compact layout ([counters][partial tiles]).
size_t gemm_stream_compact_scratch_bytes(int m, int k, const tuna_config &cfg, size_t *counter_bytes);
int launch_gemm_stream_compact(const GemmArgs &a, const tuna_config &cfg, void *scratch, size_t counter_bytes, DeviceStatus *status);

// tcgen05/TMEM kernel.  Returns a tuna_status.
int launch_gemm_umma(const GemmArgs &a, const tuna_config &cfg);
size_t gemm_umma_workspace_bytes(int m, int n, int k, const tuna_config &cfg, int sm_count);
int gemm_umma_normalize_config(int m, int n, int k, int sm_count, tuna_config *cfg);

// tcgen05 weight-streaming kernel (small token counts).  Returns a tuna_status.
int launch_gemm_tstream(const GemmArgs &a, const tuna_config &cfg);
size_t gemm_tstream_workspace_bytes(int m, int n, int k, const tuna_config &cfg, int sm_count);
int gemm_tstream_normalize_config(int m, int n, int k, int sm_count, tuna_config *cfg);
// The same kernel walking a table of independent GEMMs in one persistent launch (up to 64 per launch).
bool gemm_tstream_sequence_supported(const tuna_gemm_desc *d, int count);
size_t gemm_tstream_sequence_workspace_bytes(const tuna_gemm_desc *d, int count, int sm_count);
// `ex` != nullptr: every GEMM is a K-split partial whose finished rows go to all ranks' exchange buffers,
// and each launch is followed by the kernel that sums them into o (exchange_sm100a.cu).
int launch_gemm_tstream_sequence(const tuna_gemm_desc *d, int count, const float *code, void *workspace, size_t workspace_bytes,
                                 int sm_count, cudaStream_t stream, const tuna_exchange *ex = nullptr);

// Exchange buffers (layout in exchange_sm100a.cu): header, then two parity regions.
constexpr int kExMaxPeers = TUNA_MAX_PEERS;
constexpr int kExMaxItems = 64;          // GEMMs per launch, as in the sequence kernel
constexpr int kExHeaderBytes = 4096;
constexpr int kExFlag0Words = 64;        // flag of source rank j: 32-bit word 64 + 32 j of the header
constexpr int kExFlagStrideWords = 32;
size_t exchange_region_bytes(const tuna_gemm_desc *d, int count, int world);
int launch_exchange_reduce(const tuna_exchange &ex, const tuna_gemm_desc *d, const long long *slab0_off, int count, int tile_tok,
                           long long region_bytes, cudaStream_t stream);

}  // namespace tuna
