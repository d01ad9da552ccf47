// Microbenchmarks behind the design decisions of the streaming GEMM (sm_100a).  Stand-alone
// program: `python -m tuna_b200.build --microbench && ./tuna_b200/microbench_sm100a`.
//   1. mma.sync.m16n8k16 issue rate
//   2. tcgen05.mma cost per instruction against M, N and the A-operand source
//   3. byte -> half2 table lookups (prmt-built address + ld.shared), conflict-free table
//   4. the GEMM's weight access pattern: 128-bit loads into a register ring against cp.async rings
//   5. the GEMM's compute path alone (table lookups + MMAs + shared loads, operands resident)
// Every wait is bounded by a clock64() limit.
#include <cstdint>
#include <cstdio>
#include <cuda_runtime.h>

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { printf("CUDA error %s at line %d\n", cudaGetErrorString(e_), __LINE__); return 1; } } while (0)

static __device__ __forceinline__ uint32_t s32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
static __device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
static __device__ __forceinline__ uint32_t lut_lookup(uint32_t w, uint32_t key, uint32_t sel)
{
    uint32_t a, v;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(a) : "r"(w), "r"(key), "r"(sel));
    asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
static __device__ __forceinline__ uint4 lds128(uint32_t a)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
static __device__ __forceinline__ uint4 ldg_stream(const void *p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// ---- 1. mma.sync rate: 8 independent accumulators per warp
__global__ void k_mma_sync(float *out, int iters)
{
    float d[8][4] = {};
    uint32_t a0 = threadIdx.x, a1 = a0 * 3, a2 = a0 * 5, a3 = a0 * 7, b0 = a0 * 11, b1 = a0 * 13;
    for (int it = 0; it < iters; ++it)
#pragma unroll
        for (int i = 0; i < 8; ++i) mma16816(d[i], a0, a1, a2, a3, b0, b1);
    float s = 0;
    for (int i = 0; i < 8; ++i) for (int j = 0; j < 4; ++j) s += d[i][j];
    if (s == 123.456f) out[0] = s;
}

// ---- 2. tcgen05.mma cost: warp 1, converged, issues `iters` MMAs (elect.sync picks the lane), four per
// loop trip with compile-time operand offsets, then commits.  `accumulators` = 1: every MMA accumulates
// into the same tile (a dependent chain); 2: consecutive groups of four alternate between two tiles.  PER_GROUP adds what a
// pipeline stage costs the issuing warp: two waits on barriers that are already complete and two commits.
static __device__ __forceinline__ uint32_t elect_one()
{
    uint32_t e;
    asm volatile("{ .reg .pred P; elect.sync _|P, 0xffffffff; selp.u32 %0, 1, 0, P; }" : "=r"(e));
    return e;
}
static __device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
template <int N_TILE, int A_FROM_TMEM, int PER_GROUP>
__global__ void __launch_bounds__(256, 1) k_umma(int groups, int accumulators, long long *out, int *err)
{
    extern __shared__ __align__(1024) uint8_t sm[];
    __shared__ __align__(8) uint64_t bar, bar_stage, bar_ready;
    __shared__ uint32_t tbase;
    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < 40960; i += blockDim.x) ((uint32_t *)sm)[i] = 0x3c003c00u;
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s32(&bar)));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s32(&bar_stage)));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s32(&bar_ready)));
        asm volatile("fence.mbarrier_init.release.cluster;");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(s32(&tbase)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tm = tbase;
    if (warp == 1) {
        constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(N_TILE >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
        auto desc = [](uint32_t a) { return (uint64_t)((a & 0x3FFFFu) >> 4) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61); };
        const uint32_t sbase = s32(sm);
        const long long t0 = clock64();
        for (int g = 0; g < groups; ++g) {
            const uint32_t a_t = tm + 256 + (g & 7) * 32, b_s = sbase + (g & 3) * 32768, a_s = sbase + 131072 + (g & 1) * 16384;
            const uint32_t d_t = tm + (uint32_t)(g & (accumulators - 1)) * N_TILE;  // consecutive groups on different accumulators (power of two)
            if (PER_GROUP) {
                for (int w = 0; w < 2; ++w) {
                    uint32_t ok = 0;  // parity 1 of a fresh barrier: the wait returns at once
                    while (!ok) asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 1; selp.u32 %0,1,0,p; }" : "=r"(ok) : "r"(s32(&bar_ready)) : "memory");
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            }
            if (elect_one()) {
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    const uint32_t acc = (g >= accumulators || kk != 0);
                    if (A_FROM_TMEM)
                        asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}" ::"r"(d_t), "r"(a_t + kk * 8), "l"(desc(b_s + kk * 32)), "r"(idesc), "r"(acc) : "memory");
                    else
                        asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(d_t), "l"(desc(a_s + kk * 32)), "l"(desc(b_s + kk * 32)), "r"(idesc), "r"(acc) : "memory");
                }
                if (PER_GROUP) { umma_commit(s32(&bar_stage)); umma_commit(s32(&bar_stage)); }
            }
            __syncwarp();
        }
        if (elect_one()) umma_commit(s32(&bar));
        uint32_t ok = 0;
        while (!ok) {
            asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0; selp.u32 %0,1,0,p; }" : "=r"(ok) : "r"(s32(&bar)) : "memory");
            if (clock64() - t0 > 4000000000ll) { *err = 1; break; }
        }
        if (blockIdx.x == 0 && lane == 0) out[0] = clock64() - t0;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tm) : "memory");
    }
}

// ---- 3 and 5. table lookups and the whole compute path.  MODE bit 0: lookups, bit 1: MMAs, bit 2: stage loads
template <int NT, int MODE>
__global__ void k_compute(float *out, int iters)
{
    extern __shared__ __align__(1024) uint8_t sm[];
    const uint32_t lut = (s32(sm) + 0xFFFFu) & ~0xFFFFu;
    for (int i = threadIdx.x; i < 16384; i += blockDim.x) asm volatile("st.shared.u32 [%0], %1;" ::"r"(lut + i * 4), "r"(0x3c003c00u));
    for (int i = threadIdx.x; i < 8192; i += blockDim.x) asm volatile("st.shared.u32 [%0], %1;" ::"r"(lut + 65536 + i * 4), "r"(i * 2654435761u));
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t key = (lut & 0xFFFF0000u) | (lane * 4), st = lut + 65536 + warp * 1536;
    float acc[2][NT][4] = {};
    uint4 wv = lds128(st + lane * 16), xv[NT];
    for (int n = 0; n < NT; ++n) xv[n] = lds128(st + 512 + n * 512 + lane * 16);
    for (int it = 0; it < iters; ++it) {
        if (MODE & 4) {
            wv = lds128(st + ((lane * 16 + it * 16) & 511));
            for (int n = 0; n < NT; ++n) xv[n] = lds128(st + 512 + n * 512 + ((lane * 16 + it * 16) & 511));
        }
        const uint32_t w[4] = {wv.x, wv.y, wv.z, wv.w};
        uint32_t a[2][8];
#pragma unroll
        for (int P = 0; P < 2; ++P) {
            const uint32_t wa = w[2 * P], wb = w[2 * P + 1];
            if (MODE & 1) {
                a[P][0] = lut_lookup(wa, key, 0x7604); a[P][1] = lut_lookup(wb, key, 0x7604);
                a[P][2] = lut_lookup(wa, key, 0x7614); a[P][3] = lut_lookup(wb, key, 0x7614);
                a[P][4] = lut_lookup(wa, key, 0x7624); a[P][5] = lut_lookup(wb, key, 0x7624);
                a[P][6] = lut_lookup(wa, key, 0x7634); a[P][7] = lut_lookup(wb, key, 0x7634);
            } else {
                for (int j = 0; j < 8; ++j) a[P][j] = wa + j * wb;
            }
        }
        if (MODE & 2) {
#pragma unroll
            for (int P = 0; P < 2; ++P)
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    mma16816(acc[P][n], a[P][0], a[P][1], a[P][2], a[P][3], xv[n].x, xv[n].y);
                    mma16816(acc[P][n], a[P][4], a[P][5], a[P][6], a[P][7], xv[n].z, xv[n].w);
                }
        } else {
            for (int P = 0; P < 2; ++P) for (int j = 0; j < 8; ++j) acc[P][0][j & 3] += __uint_as_float(a[P][j]);
        }
        if (!(MODE & 4)) { wv.x += 0x01010101u; wv.y += 0x03030303u; wv.z += 0x05050505u; wv.w += 0x07070707u; }
    }
    float s = 0;
    for (int P = 0; P < 2; ++P) for (int n = 0; n < NT; ++n) for (int c = 0; c < 4; ++c) s += acc[P][n][c];
    if (s == 123.456f) out[0] = s;
}

// ---- 4. weight stream in the GEMM's access pattern: each warp owns 4 row groups (pitch 4k bytes)
// and reads 128 bytes of each per step; lane (g,t) reads row group g/2, bytes t*32 + (g&1)*16.
template <int USE_CP_ASYNC, int D>
__global__ void k_stream(const uint8_t *__restrict__ q, int kcols, int rows_total, uint32_t *out)
{
    extern __shared__ __align__(1024) uint8_t sm[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const long long gw = (long long)blockIdx.x * (blockDim.x >> 5) + warp, nwarps = (long long)gridDim.x * (blockDim.x >> 5);
    const size_t rgb = (size_t)kcols * 4;
    const int steps = kcols / 32, nblocks = rows_total / 32;
    uint32_t acc = 0;
    const uint32_t ring = s32(sm) + warp * D * 512 + lane * 16;
    for (long long blk = gw; blk < nblocks; blk += nwarps) {
        const uint8_t *src = q + (size_t)(blk * 4 + (g >> 1)) * rgb + t * 32 + (g & 1) * 16;
        if (!USE_CP_ASYNC) {
            uint4 buf[D];
#pragma unroll
            for (int j = 0; j < D; ++j) buf[j] = ldg_stream(src + (size_t)j * 128);
            for (int s = 0; s < steps; s += D)
#pragma unroll
                for (int j = 0; j < D; ++j) {
                    const uint4 v = buf[j];
                    if (s + j + D < steps) buf[j] = ldg_stream(src + (size_t)(s + j + D) * 128);
                    acc += v.x ^ v.y ^ v.z ^ v.w;
                }
        } else {
            for (int j = 0; j < D - 1; ++j) {
                asm volatile("cp.async.cg.shared.global.L2::128B [%0], [%1], 16;" ::"r"(ring + j * 512), "l"(src + (size_t)j * 128) : "memory");
                asm volatile("cp.async.commit_group;" ::: "memory");
            }
            int ps = D - 1, pslot = D - 1, cslot = 0;
            for (int s = 0; s < steps; ++s) {
                if (ps < steps) asm volatile("cp.async.cg.shared.global.L2::128B [%0], [%1], 16;" ::"r"(ring + pslot * 512), "l"(src + (size_t)ps * 128) : "memory");
                asm volatile("cp.async.commit_group;" ::: "memory");
                ++ps;
                if (++pslot == D) pslot = 0;
                asm volatile("cp.async.wait_group %0;" ::"n"(D - 1) : "memory");
                const uint4 v = lds128(ring + cslot * 512);
                if (++cslot == D) cslot = 0;
                acc += v.x ^ v.y ^ v.z ^ v.w;
            }
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
    }
    if (acc == 0x12345) out[0] = acc;
}

int main()
{
    cudaDeviceProp prop;
    CK(cudaGetDeviceProperties(&prop, 0));
    const int sms = prop.multiProcessorCount;
    printf("device %s, %d SMs; rates below assume 1.9 GHz where given per clock\n", prop.name, sms);
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    float ms, *fout;
    CK(cudaMalloc(&fout, 1024));
    long long *lout;
    int *derr;
    CK(cudaMalloc(&lout, 64));
    CK(cudaMalloc(&derr, 4));
    CK(cudaMemset(derr, 0, 4));

    {   // 1
        const int iters = 20000, warps = 16;
        k_mma_sync<<<sms, warps * 32>>>(fout, 100);
        CK(cudaDeviceSynchronize());
        cudaEventRecord(e0); k_mma_sync<<<sms, warps * 32>>>(fout, iters); cudaEventRecord(e1);
        CK(cudaDeviceSynchronize());
        cudaEventElapsedTime(&ms, e0, e1);
        const double macs = (double)sms * warps * iters * 8 * 16 * 8 * 16;
        printf("[1] mma.sync m16n8k16 f16->f32, 16 warps/SM: %.0f TFLOP/s, %.0f MAC/clk/SM\n", 2 * macs / ms / 1e9, macs / (ms * 1e-3) / sms / 1.9e9);
    }
    {   // 2
        auto run = [&](auto kern, int n, int a_tmem, int per_group, int accs) {
            CK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 170 * 1024));
            const int groups = 1000;
            kern<<<sms, 256, 170 * 1024>>>(groups, accs, lout, derr);
            CK(cudaDeviceSynchronize());
            long long h;
            int he;
            cudaMemcpy(&h, lout, 8, cudaMemcpyDeviceToHost);
            cudaMemcpy(&he, derr, 4, cudaMemcpyDeviceToHost);
            printf("[2] tcgen05.mma kind::f16 M=128 N=%3d K=16, A from %s, %d accumulator%s%s: %.1f clk per MMA (ideal %d; timeout flag %d)\n", n,
                   a_tmem ? "TMEM" : "smem", accs, accs > 1 ? "s" : "", per_group ? ", +2 waits +2 commits per 4 MMAs" : "",
                   (double)h / (groups * 4), n / 2, he);
            return 0;
        };
        run(k_umma<16, 1, 0>, 16, 1, 0, 1);   run(k_umma<32, 1, 0>, 32, 1, 0, 1);   run(k_umma<64, 1, 0>, 64, 1, 0, 1);
        run(k_umma<128, 1, 0>, 128, 1, 0, 1); run(k_umma<256, 1, 0>, 256, 1, 0, 1);
        run(k_umma<16, 1, 0>, 16, 1, 0, 2);   run(k_umma<32, 1, 0>, 32, 1, 0, 2);   run(k_umma<64, 1, 0>, 64, 1, 0, 2);
        run(k_umma<16, 0, 0>, 16, 0, 0, 1);   run(k_umma<64, 0, 0>, 64, 0, 0, 1);   run(k_umma<256, 0, 0>, 256, 0, 0, 1);
        run(k_umma<16, 1, 1>, 16, 1, 1, 1);   run(k_umma<64, 1, 1>, 64, 1, 1, 1);   run(k_umma<256, 1, 1>, 256, 1, 1, 1);
        run(k_umma<16, 1, 1>, 16, 1, 1, 2);   run(k_umma<64, 1, 1>, 64, 1, 1, 2);
    }
    {   // 3, 5
        const int iters = 20000;
        const size_t smem = 200 * 1024;
        auto run = [&](auto kern, const char *name, int warps) {
            CK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            kern<<<sms, warps * 32, smem>>>(fout, 100);
            CK(cudaDeviceSynchronize());
            cudaEventRecord(e0); kern<<<sms, warps * 32, smem>>>(fout, iters); cudaEventRecord(e1);
            CK(cudaDeviceSynchronize());
            cudaEventElapsedTime(&ms, e0, e1);
            printf("%s, %d warps/SM: %.1f weights/clk/SM (HBM needs %.0f)\n", name, warps, (double)sms * warps * iters * 1024 / (ms * 1e-3) / sms / 1.9e9, 6556e9 * 2 / sms / 1.9e9);
            return 0;
        };
        run(k_compute<2, 1>, "[3] table lookups only (prmt + ld.shared, 16 tokens)", 16);
        run(k_compute<2, 2>, "[5] MMAs only (16 tokens)", 16);
        run(k_compute<2, 3>, "[5] lookups + MMAs, operands in registers", 16);
        run(k_compute<2, 7>, "[5] lookups + MMAs + shared-memory operand loads (16 tokens)", 16);
        run(k_compute<2, 7>, "[5] lookups + MMAs + shared-memory operand loads (16 tokens)", 24);
        run(k_compute<2, 7>, "[5] lookups + MMAs + shared-memory operand loads (16 tokens)", 32);
        run(k_compute<1, 7>, "[5] lookups + MMAs + shared-memory operand loads (8 tokens)", 16);
        run(k_compute<1, 7>, "[5] lookups + MMAs + shared-memory operand loads (8 tokens)", 32);
    }
    {   // 4
        const int kcols = 8192, rows = 57344;
        const size_t bytes = (size_t)rows * kcols / 2;
        uint8_t *buf[3];
        uint32_t *uout = (uint32_t *)fout;
        for (int i = 0; i < 3; ++i) { CK(cudaMalloc(&buf[i], bytes)); CK(cudaMemset(buf[i], i + 1, bytes)); }
        auto run = [&](auto kern, const char *name, size_t smem) {
            CK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            kern<<<sms, 512, smem>>>(buf[0], kcols, rows, uout);
            CK(cudaDeviceSynchronize());
            cudaEventRecord(e0);
            for (int r = 0; r < 6; ++r) kern<<<sms, 512, smem>>>(buf[r % 3], kcols, rows, uout);
            cudaEventRecord(e1);
            CK(cudaDeviceSynchronize());
            cudaEventElapsedTime(&ms, e0, e1);
            printf("[4] 57344x8192 packed weights, GEMM access pattern, %s: %.0f GB/s\n", name, bytes * 6 / ms / 1e6);
            return 0;
        };
        run(k_stream<0, 4>, "ld.global.v4 register ring depth 4", 1024);
        run(k_stream<0, 8>, "ld.global.v4 register ring depth 8", 1024);
        run(k_stream<0, 16>, "ld.global.v4 register ring depth 16", 1024);
        run(k_stream<1, 8>, "cp.async 16B ring depth 8", 16 * 8 * 512);
        run(k_stream<1, 16>, "cp.async 16B ring depth 16", 16 * 16 * 512);
    }
    return 0;
}
