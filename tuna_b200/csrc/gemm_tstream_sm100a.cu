// Weight-streaming FP16 x 4-bit(codebook) GEMM on tcgen05 for small token counts (one pass
// covers 16, 32 or 64 tokens) on sm_100a: the memory-bound regime every row of the
// reference's README table is measured in.  Counterpart of the reference's Tuna<> kernel and its
// cp.async / ldmatrix / mma.sync main loop (kernel.cu:1043-2505, 2816-2960); the orientation
// is kept (weights are MMA operand A, tokens operand B, the accumulator is an o^T tile,
// kernel.cu:2182-2192) and nothing else.
//
// The idea.  The packed layout stores an 8x8 weight tile as 32 bytes in mma A-fragment order
// (test.py:58-65: byte j = row j/4, column pair j%4).  A 16-byte piece of it is 4 rows x 8
// columns, and that is exactly what one thread supplies to two tcgen05.st of shape 16x256b:
// lane (g, t) of a warp (g = lane/4, t = lane%4) loads the 16 bytes of row group g/2, rows
// 4(g%2)..+3, 8-column tile t of a 32-column step with ONE 128-bit ld.global (a warp load =
// four fully used 128-byte lines), turns its 16 bytes into 16 half2 by 16 table lookups and
// stores them into tensor memory with two instructions.  No shared-memory staging of the
// weights, no shuffles, no transposition: the dequantised weights exist only in registers and
// tensor memory.  The price is a permutation that costs nothing:
//   * rows: tensor-memory lane l of a 32-lane quarter holds weight row 4*(l%8) + l/8 of the
//     quarter's 32 rows (undone by the epilogue, which owns one lane per thread);
//   * K: column c of a step's 16 tensor-memory columns holds the column pair
//     k = 8*((c%8)/2) + 2*(c%2) + 4*(c/8) (+0, +1) of the step's 32, so the two 16-wide MMAs of
//     a step see K positions kappa <-> k = 8*(kappa/4) + 4*u + kappa%4 (u = MMA index).  The
//     activation producer writes x into shared memory in the same order (8-byte pieces), which
//     is free because it has to re-tile x into 8x16-byte core matrices anyway.
//
// One persistent CTA per SM, warp-specialised (24 warps, warps 2-3 idle; 80 registers per
// thread.  Re-balancing registers between warpgroups with setmaxnreg made ptxas spill more,
// not less, in this kernel):
//   warp 0       MMA issue: tcgen05.mma (M=128, N=tile_tok, K=16, fp32 accumulate), A from
//                tensor memory, B through a no-swizzle shared-memory descriptor, D in tensor memory
//   warp 1       activation producer: x (fp16 [n,k], L2 resident) -> shared memory in
//                core-matrix order with 8-byte cp.async, 128-column chunks, 6-deep ring
//   warps 4-7    epilogue: tcgen05.ld of the accumulator, fp32 scale by absmax, fp16 store,
//                split-K partials and fix-up
//   warps 8-23   dequant: 128-bit ld.global.nc into an 8-deep register ring -> prmt + ld.shared
//                table lookups -> tcgen05.st into the A slots.  Warp (quarter q, group j)
//                handles rows 32q..+31 of the 128x128 slots j, j+4, j+8, ... of the CTA.
// The scale is constant along K (one block per row, test.py:81, kernel.cu:2178-2180) and is
// applied once, in fp32, to the accumulated sum.
//
// Work decomposition ("stream-K"): a unit is (tile of 128*row_blocks rows, 128-column chunk) =
// row_blocks slots; the units, tile-major, are cut into one contiguous range per CTA so that
// every SM streams the same number of bytes whatever the shape.  A tile cut across CTAs is
// finished by whichever CTA arrives last at the tile's counter (per 32-row quarter): it adds
// the fp32 partials from the workspace in range order, so the result does not depend on
// arrival order (the reference adds fp16 partials with atomicAdd, kernel.cu:2739-2745).  No
// floating-point atomics, no zero-filled output.
//
// Programmatic dependent launch: the kernel lets its successor start as SMs free up and itself
// waits for its predecessors only before it touches what they may have written (activations,
// workspace, output); the weights and the codebook are constants and are requested before.
//
// Every wait is bounded: when one runs out the CTA records where in the device status word,
// raises a CTA-wide abort flag and unwinds to the common exit, where tensor memory is released.
#include <cstring>
#include <mutex>
#include "common.cuh"
#include "launchers.h"
#include "sm100_ptx.cuh"
#include "tcgen05.cuh"

// Optional per-warp timing (debug builds with -DTUNA_TS_PROFILE only): absolute times of the
// warp's milestones and the clocks it spent in each kind of wait.
#ifdef TUNA_TS_PROFILE
__device__ long long g_ts_prof[160 * 24 * 8];
__device__ __forceinline__ long long ts_gtime()
{
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define TS_PROF_DECL long long pw_[4] = {0, 0, 0, 0}, pt_ = 0, pg_[4] = {ts_gtime(), 0, 0, 0}; (void)pt_;
#define TS_PROF_MARK(i) pg_[i] = ts_gtime();
#define TS_PROF_BEGIN pt_ = clock64();
#define TS_PROF_END(i) pw_[i] += clock64() - pt_;
#define TS_PROF_STORE                                                                     \
    if ((threadIdx.x & 31) == 0) {                                                        \
        long long *d_ = g_ts_prof + ((size_t)blockIdx.x * 24 + (threadIdx.x >> 5)) * 8;   \
        for (int i_ = 0; i_ < 4; ++i_) { d_[i_] = pg_[i_]; d_[4 + i_] = pw_[i_]; }        \
    }
#else
#define TS_PROF_DECL
#define TS_PROF_MARK(i)
#define TS_PROF_BEGIN
#define TS_PROF_END(i)
#define TS_PROF_STORE
#endif

namespace tuna {

constexpr int kTsChunkK = 128;        // K extent of a unit / an A slot
constexpr int kTsSlotCols = 64;       // tensor-memory columns of one A slot (128 rows x 128 fp16)
constexpr int kTsMaxASlots = 8;       // A-slot ring: as many as the accumulators leave room for (6 or 7)
constexpr int kTsAccCols = 64;        // columns of one accumulator buffer (row_blocks * tile_tok <= 64)
constexpr int kTsTmemCols = 512;
constexpr int kTsMaxXStages = 6;
constexpr int kTsLoads = 8;           // 128-bit weight loads in flight per lane
constexpr int kTsEpilogueWarp0 = 4;   // warps 2-3 idle: the epilogue warps' quarters are 0..3 in order
constexpr int kTsDequantWarp0 = 8;
constexpr int kTsDequantWarps = 16;
constexpr int kTsThreads = 32 * (kTsDequantWarp0 + kTsDequantWarps);

struct TsParams {
    const uint8_t *q;
    const __half *x;
    const float *code;
    const float *absmax;
    __half *o;
    float *partials;
    unsigned int *counters;
    DeviceStatus *status;
    int m, n, k;
    int tok0;         // first token of this pass
    int row_blocks;   // RB: 128-row blocks per tile
    int a_slots;      // A-slot ring depth
    int a_base;       // first tensor-memory column of the A slots (behind the two accumulator buffers)
    int acc_cols;     // columns of one accumulator buffer
    int chunks;       // ceil(k / 128)
    int row_tiles;    // ceil(m / (128 RB))
    int units;        // row_tiles * chunks
    int units_q, units_r;  // units = units_q * CTAs + units_r: the first units_r CTAs take units_q + 1
};

// The CTA whose range holds unit u.
__device__ __forceinline__ int ts_cta_of_unit(const TsParams &p, int u)
{
    const int big = p.units_r * (p.units_q + 1);
    return u < big ? u / (p.units_q + 1) : p.units_r + (u - big) / p.units_q;
}

template <int N_TILE>
__global__ void __launch_bounds__(kTsThreads, 1) gemm_w4a16_tstream_kernel(const TsParams p)
{
    constexpr uint32_t kBTileBytes = N_TILE * 32;           // one 16-wide MMA's activations
    constexpr uint32_t kXStageBytes = 8 * kBTileBytes;      // 4 steps x 2 MMAs
    constexpr uint32_t kLbo = N_TILE * 16, kSbo = 128;
    extern __shared__ __align__(1024) uint8_t smem[];
    constexpr int kXS = N_TILE == 64 ? 3 : 6;   // activation stages (48 KB at most)
    constexpr int kLag = N_TILE == 64 ? 1 : 3;  // units between issuing a stage's copies and handing it over
    __shared__ __align__(8) uint64_t bars[2 * kTsMaxASlots + 2 * kTsMaxXStages + 4];
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;

    TS_PROF_DECL
    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;
    const int cta = blockIdx.x;
    const int RB = p.row_blocks;

    // Let the next kernel in the stream become resident as SMs free up.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // shared memory: the activation ring at the start of the dynamic window, the table at the
    // first 64-KB boundary of the shared address space
    const uint32_t xring = smem_u32(smem);
    const uint32_t lut_addr = (xring + kXS * kXStageBytes + 0xFFFFu) & ~0xFFFFu;

    const uint32_t bar0 = smem_u32(&bars[0]);
    const uint32_t a_full = bar0, a_empty = a_full + 8 * kTsMaxASlots;
    const uint32_t x_full = a_empty + 8 * kTsMaxASlots, x_empty = x_full + 8 * kXS;
    const uint32_t d_full = x_empty + 8 * kXS, d_empty = d_full + 16;
    volatile int *abort_flag = &s_abort;

    // this CTA's contiguous range of units
    const int u_begin = cta * p.units_q + min(cta, p.units_r);
    const int n_units = p.units_q + (cta < p.units_r ? 1 : 0);
    const int tile0 = u_begin / p.chunks, chunk0 = u_begin - tile0 * p.chunks;

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int i = 0; i < kTsMaxASlots; ++i) { mbar_init(a_full + 8 * i, 4); mbar_init(a_empty + 8 * i, 1); }
        for (int i = 0; i < kXS; ++i) { mbar_init(x_full + 8 * i, 1); mbar_init(x_empty + 8 * i, 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(d_full + 8 * i, 1); mbar_init(d_empty + 8 * i, 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)),
                     "r"(kTsTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }

    const int quarter = warp & 3;          // the 32 tensor-memory lanes this warp may access
    const int total_slots = n_units * RB;

    // Rest of the prologue, run by every warp inside its own role's branch (so that the dequant
    // warps can have their first weight loads in flight across it without those registers being
    // live in the other roles): the byte -> half2 table (even column = high nibble in the low
    // half), one copy per bank - the codebook is a constant, so this runs before the
    // dependency wait - then the wait, then the CTA barrier that publishes table, barriers and
    // the tensor-memory base.
    auto finish_prologue = [&]() -> uint32_t {
        const float cv = p.code[lane & 15];
        const uint32_t ch = (uint32_t)__half_as_ushort(__float2half_rn(cv));
        for (int e = warp; e < 256; e += kTsThreads / 32) {
            const uint32_t v = __shfl_sync(0xffffffffu, ch, e >> 4) | (__shfl_sync(0xffffffffu, ch, e & 15) << 16);
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(lut_addr + (uint32_t)e * 256 + lane * 4), "r"(v) : "memory");
        }
        asm volatile("griddepcontrol.wait;" ::: "memory");
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
        TS_PROF_MARK(1)
        return s_tmem_base;
    };
    uint32_t tmem = 0;

    if (warp == 0) {
        // ------------------------------------------------------------------ MMA issue
        // The warp stays converged: every lane runs the loop and the waits, one elected lane
        // issues the MMAs and the commits.
        tmem = finish_prologue();
        constexpr uint32_t idesc = make_idesc(N_TILE);
        Ring ra, rx, rd;
        int tile = tile0, chunk = chunk0;
        bool seg_first = true;  // first unit of a segment (the units of one tile inside the range)
        for (int u = 0; u < n_units; ++u) {
            const bool seg_last = (chunk + 1 == p.chunks) || (u + 1 == n_units);
            bool ok = true;
            TS_PROF_BEGIN
            if (seg_first) ok = mbar_wait(d_empty + 8 * rd.idx, rd.phase ^ 1, abort_flag, p.status, 3);
            TS_PROF_END(0)
            TS_PROF_BEGIN
            ok = ok && mbar_wait(x_full + 8 * rx.idx, rx.phase, abort_flag, p.status, 4);
            if (!__all_sync(0xffffffffu, ok)) break;
            TS_PROF_END(1)
            const uint32_t xbase = xring + (uint32_t)rx.idx * kXStageBytes;
            const uint32_t dbase = tmem + (uint32_t)(rd.idx * p.acc_cols);
            for (int rb = 0; rb < RB; ++rb) {
                TS_PROF_BEGIN
                if (!mbar_wait_warp(a_full + 8 * ra.idx, ra.phase, abort_flag, p.status, 5)) { ok = false; break; }
                TS_PROF_END(2)
                tc_fence_after();
                TS_PROF_BEGIN
                if (elect_one_sync()) {
                    const uint32_t abase = tmem + (uint32_t)p.a_base + (uint32_t)ra.idx * kTsSlotCols;
#pragma unroll
#ifdef TS_ABL_NOMMA  // timing experiment: commits only
                    for (int mm = 0; mm < 0; ++mm) {
#else
                    for (int mm = 0; mm < 8; ++mm) {  // step mm/2, 16-wide MMA mm%2
#endif
                        const uint64_t bdesc = make_desc_noswizzle(xbase + mm * kBTileBytes, kLbo, kSbo);
                        tc_mma_ts(dbase + (uint32_t)rb * N_TILE, abase + mm * 8, bdesc, idesc, (seg_first && mm == 0) ? 0u : 1u);
                    }
                    tc_commit(a_empty + 8 * ra.idx);
                    if (rb + 1 == RB) {
                        tc_commit(x_empty + 8 * rx.idx);
                        if (seg_last) tc_commit(d_full + 8 * rd.idx);
                    }
                }
                __syncwarp();
                TS_PROF_END(3)
                ra.advance(p.a_slots);
            }
            if (!ok) break;
            rx.advance(kXS);
            if (seg_last) rd.advance(2);
            seg_first = seg_last;
            if (++chunk == p.chunks) { chunk = 0; ++tile; }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ activation producer
        // 8-byte cp.async copies (no registers, many in flight), issued kLag units ahead of the
        // unit that is handed to the MMA warp.  Lane (tok%8 = lane%8, t%2 = (lane/8)%2, lane/16)
        // so that a half-warp writes one 128-byte core matrix (8 tokens x 16 bytes), conflict
        // free; copy i of a unit covers rest = 2*(i/2) + lane/16 over (t/2 [2], step [4],
        // tok/8 [N_TILE/8]) and MMA u = i%2.
        tmem = finish_prologue();
        Ring rx, rdone;
        int chunk = chunk0;
        const int tok_lo = lane & 7, t_lo = (lane >> 3) & 1, rest_lo = lane >> 4;
        // per copy i: source offset in halfs relative to x[tok0][k0] (-1: token past n), its
        // column inside the chunk, and the destination offset inside a stage - all independent of
        // the unit.  Kept in registers for the 16-token tile (whose units are the shortest).
        const __half *x_pass = p.x + (size_t)p.tok0 * p.k;
        auto copy_params = [&](int i, int &src_off, int &col, uint32_t &dst) {
            const int rest = (i & ~1) + rest_lo, uu = i & 1;
            const int t_hi = rest & 1, step = (rest >> 1) & 3, ng = rest >> 3;
            const int tok = ng * 8 + tok_lo;
            col = 32 * step + 8 * (2 * t_hi + t_lo);
            src_off = p.tok0 + tok < p.n ? tok * p.k + col + 4 * uu : -1;
            // B tile (step, u): [t/2][tok/8][tok%8][16 bytes]; columns col + 4u .. +3 of the
            // 8-column weight tile go to MMA u, at byte 8*(t%2) of the token's row
            dst = (uint32_t)(2 * step + uu) * kBTileBytes + (uint32_t)t_hi * kLbo + (uint32_t)ng * kSbo + (uint32_t)tok_lo * 16 + (uint32_t)t_lo * 8;
        };
        constexpr bool kHoist = N_TILE == 16;
        int src_off[kHoist ? N_TILE : 1], col_off[kHoist ? N_TILE : 1];
        uint32_t dst_off[kHoist ? N_TILE : 1];
        if (kHoist) {
#pragma unroll
            for (int i = 0; i < N_TILE; ++i) copy_params(i, src_off[i], col_off[i], dst_off[i]);
        }
        auto hand_over = [&]() {
            // this lane's copies of the oldest unit have landed; generic-proxy writes -> visible
            // to the tensor core's (async proxy) reads; then one arrival for the warp
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(x_full + 8 * rdone.idx);
            rdone.advance(kXS);
        };
        bool ok = true;
        for (int u = 0; u < n_units; ++u) {
            TS_PROF_BEGIN
            if (!mbar_wait_warp(x_empty + 8 * rx.idx, rx.phase ^ 1, abort_flag, p.status, 2)) { ok = false; break; }
            TS_PROF_END(0)
            const uint32_t stage = xring + (uint32_t)rx.idx * kXStageBytes;
            const int k0 = chunk * kTsChunkK;
            const __half *xk = x_pass + k0;
            auto copy_one = [&](int so, int co, uint32_t dd) {
                const bool in = so >= 0 && k0 + co < p.k;
                const __half *src = in ? xk + so : p.x;
                asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(stage + dd), "l"(src), "r"(in ? 8u : 0u) : "memory");
            };
            if constexpr (kHoist) {
#pragma unroll
                for (int i = 0; i < N_TILE; ++i) copy_one(src_off[i], col_off[i], dst_off[i]);
            } else {
#pragma unroll 8
                for (int i = 0; i < N_TILE; ++i) {
                    int so, co;
                    uint32_t dd;
                    copy_params(i, so, co, dd);
                    copy_one(so, co, dd);
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            if (u >= kLag) {
                TS_PROF_BEGIN
                asm volatile("cp.async.wait_group %0;" ::"n"(kLag) : "memory");
                TS_PROF_END(1)
                hand_over();
            }
            rx.advance(kXS);
            if (++chunk == p.chunks) chunk = 0;
        }
        if (ok) {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            for (int u = max(n_units - kLag, 0); u < n_units; ++u) hand_over();
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
    } else if (warp < kTsEpilogueWarp0) {
        tmem = finish_prologue();  // idle warps
    } else if (warp < kTsDequantWarp0) {
        // ------------------------------------------------------------------ epilogue
        tmem = finish_prologue();
        const int row_in_block = 32 * quarter + 4 * (lane & 7) + (lane >> 3);
        const int tmem_lane = 32 * quarter + lane;
        const size_t slot_floats = (size_t)RB * kBlockRows * N_TILE;
        Ring rd;
        int u = 0, tile = tile0, chunk = chunk0;
        while (u < n_units) {
            // the segment: chunks [c0, c1) of `tile`
            const int c0 = chunk;
            const int c1 = min(p.chunks, c0 + (n_units - u));
            const bool full = (c0 == 0 && c1 == p.chunks);
            TS_PROF_BEGIN
            if (!mbar_wait_warp(d_full + 8 * rd.idx, rd.phase, abort_flag, p.status, 6)) break;
            TS_PROF_END(0)
            tc_fence_after();
            TS_PROF_BEGIN
            float *my_partial = p.partials + (size_t)(2 * cta + (c0 == 0 ? 1 : 0)) * slot_floats;
            for (int rb = 0; rb < RB; ++rb) {
                const int row = (tile * RB + rb) * kBlockRows + row_in_block;
                const float sc = (full && row < p.m) ? p.absmax[row] : 0.f;
#pragma unroll 1
                for (int piece = 0; piece < N_TILE / 16; ++piece) {
                    float v[16];
                    tc_ld_x16(tmem + ((uint32_t)(32 * quarter) << 16) + (uint32_t)(rd.idx * p.acc_cols) + (uint32_t)rb * N_TILE + piece * 16, v);
                    if (full) {
                        if (row < p.m) {
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                const int tok = p.tok0 + piece * 16 + i;
                                if (tok < p.n) p.o[(size_t)tok * p.m + row] = __float2half_rn(v[i] * sc);
                            }
                        }
                    } else {
                        // [rb][4-token group][128 lanes] float4: a warp store is 512 contiguous bytes
                        float4 *dst = reinterpret_cast<float4 *>(my_partial) + ((size_t)rb * (N_TILE / 4) + piece * 4) * kBlockRows + tmem_lane;
#pragma unroll
                        for (int i = 0; i < 4; ++i) dst[i * kBlockRows] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(d_empty + 8 * rd.idx);
            if (!full) {
                // Each epilogue warp finishes its own 32 lanes of the tile alone: it arrives at the
                // counter of (tile, quarter); the last warp to arrive adds that quarter's partials in
                // range order and stores the rows.
                __threadfence();
                __syncwarp();
                const int cta_first = ts_cta_of_unit(p, tile * p.chunks);
                const int cta_last = ts_cta_of_unit(p, (tile + 1) * p.chunks - 1);
                const int nseg = cta_last - cta_first + 1;
                unsigned int *counter = p.counters + (size_t)tile * 4 + quarter;
                unsigned int old = 0;
                if (lane == 0) old = atomicAdd(counter, 1u);
                old = __shfl_sync(0xffffffffu, old, 0);
                if (old == (unsigned)nseg - 1) {
                    if (lane == 0) *counter = 0;  // leave the counter clean for the next call
                    __threadfence();
                    for (int rb = 0; rb < RB; ++rb) {
                        const int row = (tile * RB + rb) * kBlockRows + row_in_block;
                        if (row >= p.m) continue;
                        const float sc = p.absmax[row];
#pragma unroll 1
                        for (int piece = 0; piece < N_TILE / 16; ++piece) {
                            float acc[16];
#pragma unroll
                            for (int i = 0; i < 16; ++i) acc[i] = 0.f;
                            auto seg_ptr = [&](int sgm) {
                                return reinterpret_cast<const float4 *>(p.partials + (size_t)(2 * (cta_first + sgm) + (sgm == 0 ? 1 : 0)) * slot_floats) +
                                       ((size_t)rb * (N_TILE / 4) + piece * 4) * kBlockRows + tmem_lane;
                            };
                            // the loads of two segments in flight; the adds keep the range order
                            int sgm = 0;
                            for (; sgm + 2 <= nseg; sgm += 2) {
                                float4 a[4], b[4];
                                const float4 *s0 = seg_ptr(sgm), *s1 = seg_ptr(sgm + 1);
#pragma unroll
                                for (int i = 0; i < 4; ++i) { a[i] = __ldcg(s0 + i * kBlockRows); b[i] = __ldcg(s1 + i * kBlockRows); }
#pragma unroll
                                for (int i = 0; i < 4; ++i) { acc[4 * i] += a[i].x; acc[4 * i + 1] += a[i].y; acc[4 * i + 2] += a[i].z; acc[4 * i + 3] += a[i].w; }
#pragma unroll
                                for (int i = 0; i < 4; ++i) { acc[4 * i] += b[i].x; acc[4 * i + 1] += b[i].y; acc[4 * i + 2] += b[i].z; acc[4 * i + 3] += b[i].w; }
                            }
                            if (sgm < nseg) {
                                const float4 *s0 = seg_ptr(sgm);
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    const float4 a = __ldcg(s0 + i * kBlockRows);
                                    acc[4 * i] += a.x; acc[4 * i + 1] += a.y; acc[4 * i + 2] += a.z; acc[4 * i + 3] += a.w;
                                }
                            }
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                const int tok = p.tok0 + piece * 16 + i;
                                if (tok < p.n) p.o[(size_t)tok * p.m + row] = __float2half_rn(acc[i] * sc);
                            }
                        }
                    }
                }
            }
            TS_PROF_END(1)
            u += c1 - c0;
            chunk = 0;
            ++tile;
            rd.advance(2);
        }
    } else {
        // ------------------------------------------------------------------ dequant
        // Group j (4 warps, one per 32-lane quarter) converts the slots j, j+4, j+8, ... of this CTA
        // whole: 4 steps = 4 loads per lane per slot, one wait / fence / arrival per slot.  The four
        // groups work on four different slots at once, so the latency of a slot's chain (lookups ->
        // tcgen05.st -> wait::st -> arrive) is overlapped four times.
        // Position and first loads before anything else (the weights are constants; nothing another
        // kernel writes is touched before griddepcontrol.wait).
        const int group = (warp - kTsDequantWarp0) >> 2;
        const int g = lane >> 2, t = lane & 3;
        const int n_rg = p.m >> 3;
        const size_t rg_bytes = row_group_bytes(p.k);
        const int A = p.a_slots;
        // Cursor of the next slot to prefetch.  The group's slots are 4 apart in the CTA's slot
        // sequence: with RB in {1, 2, 4} that is always the same row block of the tile
        // (rb = group % RB) and 4 / RB units further on - no division in the loop.
        const int rb = group % RB, ustep = 4 / RB;
        int pf_unit = group / RB;
        int pf_tile = (u_begin + pf_unit) / p.chunks, pf_chunk = (u_begin + pf_unit) - pf_tile * p.chunks;
        const int lane_rg = 4 * quarter + (g >> 1);
        const uint32_t lane_off = (uint32_t)(8 * t) * 4 + (g & 1) * 16;
        // source and predicate mask (bit st = step st) of this lane's 4 loads of the slot at the
        // cursor; advances the cursor
        auto prefetch_prepare = [&](unsigned &mask) -> const uint8_t * {
            const int rg = (pf_tile * RB + rb) * 16 + lane_rg;
            const int col = pf_chunk * kTsChunkK + 8 * t;
            const int steps_in = min((p.k - col + 31) >> 5, 4);  // steps whose 8-column tile starts before k
            const bool in = pf_unit < n_units && rg < n_rg;
            mask = in ? (1u << steps_in) - 1u : 0u;
            const uint8_t *src = p.q + (in ? (size_t)rg * rg_bytes + (size_t)pf_chunk * (kTsChunkK * 4) + lane_off : 0);
            pf_unit += ustep;
            pf_chunk += ustep;
            while (pf_chunk >= p.chunks) { pf_chunk -= p.chunks; ++pf_tile; }
            return src;
        };
        uint4 ring[2][4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            unsigned mask;
            const uint8_t *src = prefetch_prepare(mask);
#pragma unroll
            for (int st = 0; st < 4; ++st) ring[h][st] = ldg_stream_pred(src + (mask ? st * 128 : 0), (mask >> st) & 1u);
        }
        tmem = finish_prologue();
        const uint32_t lane_key = (lut_addr & 0xFFFF0000u) | (uint32_t)(lane * 4);
        const uint32_t a_lane0 = tmem + ((uint32_t)(32 * quarter) << 16) + (uint32_t)p.a_base;
        int a_idx = group;      // ring position of slot `sl`: sl % A, parity of its use (sl / A) & 1
        uint32_t a_phase = 0;
        bool ok = true;
#ifdef TUNA_TS_PROFILE
        const long long loop_c0 = clock64();
#endif
        for (int sl = group; ok && sl < total_slots; sl += 8) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                if (sl + 4 * h >= total_slots) break;
                TS_PROF_BEGIN
                if (!mbar_wait_warp(a_empty + 8 * a_idx, a_phase ^ 1, abort_flag, p.status, 7)) { ok = false; break; }
                TS_PROF_END(0)
                tc_fence_after();
                TS_PROF_BEGIN
                const uint32_t ta = a_lane0 + (uint32_t)a_idx * kTsSlotCols;
                unsigned pf_mask;
                const uint8_t *pf_src = prefetch_prepare(pf_mask);  // the slot two ahead of this one
#pragma unroll
                for (int st = 0; st < 4; ++st) {
                    const uint4 wv = ring[h][st];
#ifndef TS_ABL_NOLDG
                    ring[h][st] = ldg_stream_pred(pf_src + (pf_mask ? st * 128 : 0), (pf_mask >> st) & 1u);
#else
                    ring[h][st].x += (uint32_t)(size_t)pf_src;  // timing experiment: no global loads
#endif
                    const uint32_t w[4] = {wv.x, wv.y, wv.z, wv.w};  // word r = row 4(g%2)+r, byte c = column pair c
                    uint32_t v[4][4];  // the step's 16 lookups in flight together
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
#ifdef TS_ABL_NOLUT  // timing experiment: no table lookups
                        v[r][0] = w[r]; v[r][1] = w[r] + lane_key; v[r][2] = w[r] ^ lane_key; v[r][3] = w[r] >> 1;
#else
                        v[r][0] = lut_lookup(w[r], lane_key, 0x7604);
                        v[r][1] = lut_lookup(w[r], lane_key, 0x7614);
                        v[r][2] = lut_lookup(w[r], lane_key, 0x7624);
                        v[r][3] = lut_lookup(w[r], lane_key, 0x7634);
#endif
                    }
                    // rows 0, 1 -> lanes g, g+8; rows 2, 3 -> lanes g+16, g+24
#ifdef TS_ABL_NOST  // timing experiment: keep the lookups alive, skip the stores
                    asm volatile("" ::"r"(v[0][0] ^ v[0][1] ^ v[0][2] ^ v[0][3] ^ v[1][0] ^ v[1][1] ^ v[1][2] ^ v[1][3] ^ v[2][0] ^ v[2][1] ^ v[2][2] ^ v[2][3] ^ v[3][0] ^ v[3][1] ^ v[3][2] ^ v[3][3]), "r"(ta));
#else
                    tc_st_16x256b_x2(ta + 16u * st, v[0][0], v[0][1], v[1][0], v[1][1], v[0][2], v[0][3], v[1][2], v[1][3]);
                    tc_st_16x256b_x2(ta + (16u << 16) + 16u * st, v[2][0], v[2][1], v[3][0], v[3][1], v[2][2], v[2][3], v[3][2], v[3][3]);
#endif
                }
                TS_PROF_END(1)
                TS_PROF_BEGIN
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                TS_PROF_END(2)
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(a_full + 8 * a_idx);
                a_idx += 4;
                if (a_idx >= A) { a_idx -= A; a_phase ^= 1u; }
            }
        }
#ifdef TUNA_TS_PROFILE
        pw_[3] = clock64() - loop_c0;
#endif
    }

    // ------------------------------------------------------------------ common exit
    TS_PROF_MARK(2)
    tc_fence_before();
    __syncthreads();
    TS_PROF_MARK(3)
    TS_PROF_STORE
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTsTmemCols) : "memory");
    }
}

// ------------------------------------------------------------------ host side

// Dynamic shared memory: the activation ring, slack up to the next 64-KB boundary of the shared
// window, the table.  The static part (barriers) sits in front of the dynamic window, so the
// ring ends below 64 KB as long as it is smaller than 64 KB minus the static part.
static size_t ts_smem_bytes() { return 65536 + kLut64Bytes; }

int gemm_tstream_normalize_config(int m, int n, int k, int sm_count, tuna_config *c)
{
    (void)m; (void)k;
    if (c->tile_tok == 0) c->tile_tok = (n <= 16) ? 16 : (n <= 32 ? 32 : 64);
    if (c->tile_tok != 16 && c->tile_tok != 32 && c->tile_tok != 64) return TUNA_ERR_BAD_CONFIG;
    if (c->row_blocks == 0) c->row_blocks = 1;
    if ((c->row_blocks != 1 && c->row_blocks != 2 && c->row_blocks != 4) || c->row_blocks * c->tile_tok > kTsAccCols)
        return TUNA_ERR_BAD_CONFIG;
    if (c->ctas < 0) return TUNA_ERR_BAD_CONFIG;
    if (c->ctas == 0 || c->ctas > sm_count) c->ctas = sm_count;
    return TUNA_OK;
}

size_t gemm_tstream_workspace_bytes(int m, int n, int k, const tuna_config &c, int sm_count)
{
    (void)n; (void)k;
    const size_t tiles = (size_t)div_up(m, kBlockRows * c.row_blocks);
    const size_t counters = (tiles * 16 + 255) / 256 * 256;  // one counter per tile and 32-row quarter
    return partial_region_bytes(sm_count) + counters;
}

template <int N_TILE>
static int launch_ts(const TsParams &p, int ctas, cudaStream_t stream)
{
    static bool attr_set[64] = {false};  // one-time, per device, opt-in to large dynamic shared memory
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return TUNA_ERR_NO_DEVICE;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!attr_set[dev]) {
            if (cudaFuncSetAttribute(gemm_w4a16_tstream_kernel<N_TILE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)ts_smem_bytes()) != cudaSuccess)
                return TUNA_ERR_NO_DEVICE;
            attr_set[dev] = true;
        }
    }
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3((unsigned)ctas);
    lc.blockDim = dim3(kTsThreads);
    lc.dynamicSmemBytes = ts_smem_bytes();
    lc.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr;
    lc.numAttrs = 1;
    return cudaLaunchKernelEx(&lc, gemm_w4a16_tstream_kernel<N_TILE>, p) == cudaSuccess ? TUNA_OK : TUNA_ERR_LAUNCH;
}

int launch_gemm_tstream(const GemmArgs &a, const tuna_config &c)
{
    TsParams p;
    std::memset(&p, 0, sizeof(p));
    p.q = a.q; p.x = (const __half *)a.x; p.code = a.code; p.absmax = a.absmax; p.o = (__half *)a.o;
    p.m = a.m; p.n = a.n; p.k = a.k;
    p.row_blocks = c.row_blocks;
    p.acc_cols = c.row_blocks * c.tile_tok < 32 ? 32 : c.row_blocks * c.tile_tok;  // 32-column allocation granule
    p.a_base = 2 * p.acc_cols;
    p.a_slots = (kTsTmemCols - p.a_base) / kTsSlotCols;
    if (p.a_slots > kTsMaxASlots) p.a_slots = kTsMaxASlots;
    p.chunks = div_up(a.k, kTsChunkK);
    p.row_tiles = div_up(a.m, kBlockRows * c.row_blocks);
    const long long units = (long long)p.row_tiles * p.chunks;
    if (units >= (1ll << 30)) return TUNA_ERR_TOO_LARGE;
    p.units = (int)units;
    p.status = device_status_word();
    if (!p.status) return TUNA_ERR_NO_DEVICE;
    if (a.workspace == nullptr || a.workspace_bytes < gemm_tstream_workspace_bytes(a.m, a.n, a.k, c, a.sm_count))
        return TUNA_ERR_WORKSPACE;
    p.partials = (float *)a.workspace;
    p.counters = (unsigned int *)((uint8_t *)a.workspace + partial_region_bytes(a.sm_count));
    int ctas = c.ctas;
    if (ctas > p.units) ctas = p.units;
    p.units_q = p.units / ctas;
    p.units_r = p.units % ctas;
    for (int tok0 = 0; tok0 < a.n; tok0 += c.tile_tok) {
        p.tok0 = tok0;
        int st;
        switch (c.tile_tok) {
            case 16: st = launch_ts<16>(p, ctas, a.stream); break;
            case 32: st = launch_ts<32>(p, ctas, a.stream); break;
            case 64: st = launch_ts<64>(p, ctas, a.stream); break;
            default: return TUNA_ERR_BAD_CONFIG;
        }
        if (st != TUNA_OK) return st;
    }
    return TUNA_OK;
}

}  // namespace tuna

#ifdef TUNA_TS_PROFILE
extern "C" int tuna_debug_ts_profile(void *host_out, size_t bytes)
{
    if (bytes > sizeof(long long) * 160 * 24 * 8) bytes = sizeof(long long) * 160 * 24 * 8;
    return (int)cudaMemcpyFromSymbol(host_out, g_ts_prof, bytes);
}
#endif
