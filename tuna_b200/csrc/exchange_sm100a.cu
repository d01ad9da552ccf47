// Row-parallel (K-split) GEMMs fused with the reduction of their partial outputs across GPUs.
//
// The reference has no multi-GPU path; a tensor-parallel user of it shards the K dimension of the
// down / output projections, runs one GEMM per rank and sums the fp16 partial outputs with an
// all-reduce.  Here the GEMM kernel's epilogue writes every finished row of its partial output, as
// it is produced, into a slab of the exchange buffer of EVERY rank (ordinary stores to peer memory:
// NVLink traffic overlaps the weight streaming), and one small kernel per launch then
//   1. tells every peer that this rank's slabs are complete (a release store of the exchange
//      number into the peer's flag word, after the GEMM kernel has finished),
//   2. waits - bounded, with an error status - until every rank's flag has reached that number,
//   3. adds the slabs in rank order in fp32 (the same result on every rank, independent of
//      arrival order) and stores fp16 outputs.
// No multicast, no TMA from peer memory, no collective library on the data path.
//
// Exchange buffer of a rank (one allocation, zero-filled at creation):
//   [0, 4096)   header: word 0 = exchanges completed on this rank, word 1 = arrival counter of the
//               reduce kernel's blocks, flag of source rank j at byte 256 + 128 j
//   two parity regions of equal size: exchange number e uses region e % 2.  A region holds, GEMM
//   after GEMM of the launch, `world` slabs of [m][tile_tok] fp16, slab j written by rank j.
// Two regions suffice: a rank can start writing exchange e + 2 only after its own reduce kernel
// of exchange e + 1 has seen every peer's flag e + 1, which a peer raises only after its reduce
// kernel of exchange e - the last reader of that region - has completed.
#include <cstring>
#include "common.cuh"
#include "launchers.h"

namespace tuna {

struct ReduceItem {
    __half *o;        // [n, m] fp16
    int m, n;
    long long off;    // of rank 0's slab inside a parity region
};

struct ReduceLaunch {
    unsigned char *local;                  // this rank's exchange buffer
    unsigned int *peer_header[kExMaxPeers];  // header of every rank's buffer (rank order)
    DeviceStatus *status;
    long long region0, region_bytes, wait_limit;
    int rank, world, count, tile_tok;
    ReduceItem item[kExMaxItems];
};

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int *p)
{
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned int *p, unsigned int v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// grid (blocks per item, items).  Block (0, 0) signals; every block waits for all the flags itself.
__global__ void __launch_bounds__(256) exchange_reduce_kernel(const __grid_constant__ ReduceLaunch R)
{
    unsigned int *hdr = reinterpret_cast<unsigned int *>(R.local);
    __shared__ unsigned int s_e;
    __shared__ int s_ok;
    if (threadIdx.x == 0) s_e = ld_acquire_sys(hdr) + 1u;  // the number of this exchange
    __syncthreads();
    const unsigned int e = s_e;
    if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x < R.world) {
        // the GEMM kernel before this one has completed: its stores to peer memory are ordered
        // before this release at system scope
        __threadfence_system();
        st_release_sys(R.peer_header[threadIdx.x] + kExFlag0Words + kExFlagStrideWords * R.rank, e);
    }
    if (threadIdx.x == 0) {
        int ok = 1;
        const long long t0 = clock64();
        for (int j = 0; j < R.world && ok; ++j) {
            const unsigned int *flag = hdr + kExFlag0Words + kExFlagStrideWords * j;
            while ((int)(ld_acquire_sys(flag) - e) < 0) {
                if (clock64() - t0 > R.wait_limit) {
                    ok = 0;
                    if (atomicCAS(&R.status->code, 0, 98) == 0) R.status->detail = j;
                    break;
                }
                __nanosleep(200);
            }
        }
        s_ok = ok;
    }
    __syncthreads();
    if (s_ok && (int)blockIdx.y < R.count) {
        const ReduceItem &it = R.item[blockIdx.y];
        const int groups = R.tile_tok / 8;  // 8 tokens = 16 bytes of a slab row
        const long long slab = (long long)it.m * R.tile_tok * 2;
        const unsigned char *base = R.local + R.region0 + (long long)(e & 1u) * R.region_bytes + it.off;
        for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < (long long)it.m * groups;
             idx += (long long)gridDim.x * blockDim.x) {
            const int g = (int)(idx / it.m), row = (int)(idx - (long long)g * it.m);
            if (g * 8 >= it.n) continue;
            float acc[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = 0.f;
            for (int j = 0; j < R.world; ++j) {  // rank order: the same sum on every rank
                const uint4 v = __ldcg(reinterpret_cast<const uint4 *>(base + j * slab + ((long long)row * R.tile_tok + g * 8) * 2));
                const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
                    acc[2 * i] += f.x;
                    acc[2 * i + 1] += f.y;
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int tok = g * 8 + i;
                if (tok < it.n) it.o[(size_t)tok * it.m + row] = __float2half_rn(acc[i]);
            }
        }
    }
    // the last block to finish completes the exchange: nothing reads the number before that
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned int blocks = gridDim.x * gridDim.y;
        if (atomicAdd(hdr + 1, 1u) == blocks - 1) {
            hdr[1] = 0;
            __threadfence();
            st_release_sys(hdr, e);
        }
    }
}

size_t exchange_region_bytes(const tuna_gemm_desc *d, int count, int world)
{
    // the largest launch (kExMaxItems GEMMs at most) decides
    size_t worst = 0;
    for (int first = 0; first < count; first += kExMaxItems) {
        const int cnt = count - first < kExMaxItems ? count - first : kExMaxItems;
        int max_n = 1;
        for (int i = 0; i < cnt; ++i) max_n = d[first + i].n > max_n ? d[first + i].n : max_n;
        const size_t tile_tok = max_n <= 16 ? 16 : (max_n <= 32 ? 32 : 64);
        size_t need = 0;
        for (int i = 0; i < cnt; ++i)
            if (d[first + i].flags & TUNA_GEMM_PARTIAL) need += (size_t)world * d[first + i].m * tile_tok * 2;
        worst = need > worst ? need : worst;
    }
    return (worst + 255) / 256 * 256;
}

int launch_exchange_reduce(const tuna_exchange &ex, const tuna_gemm_desc *d, const long long *slab0_off, int count, int tile_tok,
                           long long region_bytes, cudaStream_t stream)
{
    if (count < 1 || count > kExMaxItems) return TUNA_ERR_BAD_CONFIG;
    static thread_local ReduceLaunch R;
    std::memset(&R, 0, sizeof(R) - sizeof(R.item));
    R.local = (unsigned char *)ex.buffer[ex.rank];
    for (int j = 0; j < ex.world; ++j) R.peer_header[j] = (unsigned int *)ex.buffer[j];
    R.status = device_status_word();
    if (!R.status) return TUNA_ERR_NO_DEVICE;
    R.region0 = kExHeaderBytes;
    R.region_bytes = region_bytes;
    R.wait_limit = 2000000000ll;  // about a second
    R.rank = ex.rank;
    R.world = ex.world;
    R.count = count;
    R.tile_tok = tile_tok;
    int items = 0;
    for (int i = 0; i < count; ++i) {
        if (slab0_off[i] < 0) continue;  // an ordinary GEMM of the launch
        R.item[items].o = (__half *)d[i].o;
        R.item[items].m = d[i].m;
        R.item[items].n = d[i].n;
        R.item[items].off = slab0_off[i];
        ++items;
    }
    R.count = items;
    // A launch without partial GEMMs still runs the exchange (flags, number): every rank's launches stay in step.
    // one thread per (row, 8 tokens) where that still fills the GPU: the slabs are read once, at HBM speed
    int max_work = 1;
    for (int i = 0; i < items; ++i) {
        const int w = R.item[i].m * (tile_tok / 8);
        max_work = w > max_work ? w : max_work;
    }
    int blocks_x = (max_work + 255) / 256;
    if (blocks_x > 32) blocks_x = 32;
    const dim3 grid((unsigned)blocks_x, (unsigned)(items > 0 ? items : 1));
    // an ordinary launch: it starts when the GEMM kernel before it has completed (its stores, the remote
    // ones included, are then performed); launching it and its successor programmatically early was
    // measured and gained nothing
    exchange_reduce_kernel<<<grid, 256, 0, stream>>>(R);
    return cudaGetLastError() == cudaSuccess ? TUNA_OK : TUNA_ERR_LAUNCH;
}

}  // namespace tuna

// ------------------------------------------------------------------ C ABI: exchange buffers

extern "C" size_t tuna_exchange_bytes(const tuna_gemm_desc *gemms, int count, int world)
{
    if (!gemms || count < 1 || world < 1 || world > TUNA_MAX_PEERS) return 0;
    return tuna::kExHeaderBytes + 2 * tuna::exchange_region_bytes(gemms, count, world);
}

extern "C" int tuna_exchange_create(size_t bytes, void **buffer, void *ipc_handle)
{
    if (!buffer) return TUNA_ERR_NULL_POINTER;
    if (bytes < (size_t)tuna::kExHeaderBytes + 512) return TUNA_ERR_WORKSPACE;
    void *p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) return TUNA_ERR_NO_DEVICE;
    if (cudaMemset(p, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
        cudaFree(p);
        return TUNA_ERR_NO_DEVICE;
    }
    if (ipc_handle) {
        cudaIpcMemHandle_t h;
        if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
            cudaFree(p);
            return TUNA_ERR_NO_DEVICE;
        }
        static_assert(sizeof(h) == TUNA_IPC_HANDLE_BYTES, "handle size");
        std::memcpy(ipc_handle, &h, sizeof(h));
    }
    *buffer = p;
    return TUNA_OK;
}

extern "C" int tuna_exchange_open(const void *ipc_handle, void **buffer)
{
    if (!ipc_handle || !buffer) return TUNA_ERR_NULL_POINTER;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, ipc_handle, sizeof(h));
    void *p = nullptr;
    if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        cudaGetLastError();
        return TUNA_ERR_NO_DEVICE;
    }
    *buffer = p;
    return TUNA_OK;
}

extern "C" int tuna_exchange_close(void *peer_buffer)
{
    if (!peer_buffer) return TUNA_ERR_NULL_POINTER;
    return cudaIpcCloseMemHandle(peer_buffer) == cudaSuccess ? TUNA_OK : TUNA_ERR_NO_DEVICE;
}

extern "C" int tuna_exchange_destroy(void *buffer)
{
    if (!buffer) return TUNA_ERR_NULL_POINTER;
    return cudaFree(buffer) == cudaSuccess ? TUNA_OK : TUNA_ERR_NO_DEVICE;
}
