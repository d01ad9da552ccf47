// Weight-streaming FP16 x 4-bit(codebook) GEMM for small token counts (n <= 32
// per pass) on sm_100a: the memory-bound regime every row of the reference's
// README table is measured in.  Counterpart of the reference's Tuna<> kernel and
// its Deq4GemmIterator main loop (kernel.cu:1043-2505, 2816-2960); it keeps the
// mma orientation (weights are the m16 "A" operand, tokens the n8 "B" operand,
// kernel.cu:2182-2192) and nothing else.
//
// Why mma.sync here: measured on B200, mma.sync.m16n8k16 on 16 warps sustains 45.6 weights per
// clock per SM at 16 tokens with no serial issuer and no cross-role synchronisation, against the
// 47 that HBM delivers.  The tensor pipe is far faster through tcgen05 (a 128x16x16 MMA takes
// 11.6 clocks from a tight issuing loop), but each wait, commit or stray instruction of the
// issuing warp shows up directly and the tensor-memory kernel's dequant pipeline is not yet
// fast enough at small token tiles; it takes over for large token counts.
//
// Data movement, also chosen by measurement on B200 in this kernel's access pattern (a warp
// load = four 128-byte runs, one per row group): 128-bit ld.global straight into a register
// ring, eight loads in flight per lane, reaches 5.8 TB/s; cp.async into shared memory stops at
// 2.7 TB/s and TMA boxes of short strided rows at ~3 TB/s.  So every warp streams its own
// weights into registers.  The activations of a unit (tile_tok tokens x the unit's columns, a
// few KB, L2 resident) are staged in shared memory by all warps with cp.async, one unit ahead,
// double buffered; the warps meet once per unit.
//
// Mapping.  A lane's 16 packed bytes are half an 8x8 tile (4 rows x 8 columns): lane (g,t)
// (g = lane/4, t = lane%4) takes row group g/2, rows 4(g%2)..+3, tile t of the four tiles of a
// 32-column step.  Each 32-bit word is 8 consecutive columns of one row and becomes the A
// fragments of two m16n8k16 (the k index of an mma is a label: slots 2t,2t+1 <-> columns 0,1
// of tile t, slots 2t+8,+9 <-> columns 2,3; the B fragment is the matching 16 contiguous
// bytes of x).  Rows 4g, 4g+1 feed accumulator tile P0, rows 4g+2, 4g+3 tile P1.
//
// Dequantisation: a byte holds two codes; a 256-entry byte -> half2(fp16(code[hi]),
// fp16(code[lo])) table is replicated once per bank (entry stride 256 bytes) at a
// 64-KB-aligned shared address, so that ONE prmt builds the whole address
// (0x10000*j | byte << 8 | lane*4) and every lookup is conflict free.  The per-row scale
// is constant along K (one block per row, test.py:81, kernel.cu:2178-2180) and is applied
// once, in fp32, to the accumulated sum.
//
// Work decomposition.  One persistent CTA per SM, 16 warps arranged warps_m x warps_k.  A
// "unit" is (row tile of 32*R*warps_m rows, K chunk of 32*S*warps_k columns) and consists of S
// steps (a step = every warp's next 32 columns).  The steps of all units, tile-major, are cut
// into one contiguous range per CTA ("stream-K" at step granularity), so every SM streams the
// same number of bytes whatever the shape; a range may begin and end inside a unit.  Warps
// that share rows reduce through shared memory in a fixed tree.  A tile cut across CTAs is
// finished per warp slice: each warp writes its fp32 partial to the workspace and arrives at
// its slice's counter; the last warp to arrive adds the slice's partials in segment order and
// stores the rows.  Results are bit-identical from run to run, the output needs no zero fill,
// and there are no floating-point atomics (the reference atomically adds fp16 partials,
// kernel.cu:2739-2745).
//
// Launch.  Programmatic dependent launch: the kernel lets its successor in the stream start
// at once (griddepcontrol.launch_dependents) and itself waits for its predecessors
// (griddepcontrol.wait) only after it has requested its first weights; everything another
// kernel may have produced (activations, workspace, output) is touched after that wait.
// Reading the packed weights before the wait is safe even when the preceding kernel of the
// stream wrote them (a quantizer): a kernel can only start early behind a predecessor that
// triggers early, the only kernels that do are this one (which never writes weights), and a
// predecessor that does not trigger has completed - with its writes performed - before a
// dependent grid starts.
//
// The kernel waits on nothing but its own CTA barrier and the stream's kernel order: no
// spinning on other CTAs, no asynchronous engine.
#include <cstring>
#include <mutex>
#include "common.cuh"
#include "launchers.h"
#include "sm100_ptx.cuh"

namespace tuna {

constexpr int kStreamWarps = 16;
constexpr int kStreamThreads = 32 * kStreamWarps;
constexpr int kLoadsInFlight = 8;   // 128-bit weight loads in flight per lane

struct StreamParams {
    const uint8_t *q;
    const __half *x;
    const float *code;
    const float *absmax;
    __half *o;
    float *partials;
    unsigned int *counters;
    DeviceStatus *status;
    int m, n, k;
    int tok0;  // first token of this pass
    int warps_m, warps_k;
    int ksteps;  // S: 32-column steps per warp per unit, a multiple of the prefetch distance
    int row_tiles, chunks;  // row tiles of ONE matrix; the tile index runs over batch * row_tiles
    int batch;              // independent GEMMs of the same shape in this launch (strides below, in bytes)
    long long q_stride, x_stride, absmax_stride, o_stride;
    long long units;
    int steps_q, steps_r;  // units * ksteps = steps_q * CTAs + steps_r: the first steps_r CTAs take steps_q + 1 steps
    int red_bytes;    // shared-memory scratch of the in-CTA reduction
    int x_buf_bytes;  // one activation buffer
};

__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                             uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 16-byte asynchronous global -> shared copy; src_bytes = 0 fills the destination with zeros.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, uint32_t src_bytes)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}

__device__ __forceinline__ uint4 lds128(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

// BATCHED: the tile index runs over several matrices (tuna_matmul_batched); without it the
// matrix index is the constant 0 and its bookkeeping compiles away.
template <int R, int NT, bool BATCHED>
__global__ void __launch_bounds__(kStreamThreads, 1) gemm_stream_kernel(const StreamParams p)
{
    constexpr int PF = kLoadsInFlight / R;  // steps of weights in flight per warp
    extern __shared__ __align__(1024) uint8_t smem[];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cta = blockIdx.x, ctas = gridDim.x;
    const int WM = p.warps_m, WK = p.warps_k, S = p.ksteps;

    // Shared memory: the table at the first 64-KB boundary of the shared window, the reduction
    // scratch right behind it.
    const uint32_t lut_addr = (smem_u32(smem) + 0xFFFFu) & ~0xFFFFu;
    const uint32_t red_addr = lut_addr + kLut64Bytes;
    // two activation buffers behind it: [tile_tok rows] x [unit columns] fp16, rows padded by 64
    // bytes so that the two token rows a quarter-warp reads fall into different bank halves
    const uint32_t x_pitch = (uint32_t)(64 * S * WK + 64);
    const uint32_t x_buf_bytes = (uint32_t)(NT * 8) * x_pitch;
    const uint32_t xbuf_addr = red_addr + (uint32_t)p.red_bytes;

    // Let the next kernel in the stream start as soon as SMs free up (it waits for this grid to
    // complete before it touches anything this grid writes, see below).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // This CTA's contiguous range of STEPS (one step = every warp's 32 columns; a unit is S of
    // them): the split is as even as one step allows, whatever the shape.  A range may begin
    // and end inside a unit; the loads and the math of the steps outside it are masked off.
    // (32-bit arithmetic throughout: the 64-bit divisions of a general formula cost a microsecond.)
    const int g_begin = cta * p.steps_q + min(cta, p.steps_r);
    const int n_steps = p.steps_q + (cta < p.steps_r ? 1 : 0);  // steps of this CTA
    const int tile_steps = p.chunks * S;                        // steps of one row tile
    // the CTA whose range holds step g
    auto cta_of_step = [&](int gstep) {
        const int big = p.steps_r * (p.steps_q + 1);
        return gstep < big ? gstep / (p.steps_q + 1) : p.steps_r + (gstep - big) / p.steps_q;
    };
    int tile = g_begin / tile_steps;  // over all matrices of the batch
    int tile_b = BATCHED ? tile / p.row_tiles : 0;  // matrix, row tile inside it
    int tile_rt = tile - tile_b * p.row_tiles;
    const int first_in_tile = g_begin - tile * tile_steps;
    int chunk = first_in_tile / S;
    // positions below are relative to the first step of the first unit this CTA touches
    const int r_begin = first_in_tile - chunk * S;  // where in that unit the range begins
    const int r_end = r_begin + n_steps;

    const int wm = warp % WM, wk = warp / WM;
    const int g = lane >> 2, t = lane & 3;
    const bool active = wk < WK;  // warps beyond warps_m * warps_k only take part in the rendezvous
    const uint32_t lane_key = (lut_addr & 0xFFFF0000u) | (uint32_t)(lane * 4);
    const int n_rg = p.m >> 3;
    const size_t rg_bytes = row_group_bytes(p.k);

    float acc[R][2][NT][4];
    auto zero_acc = [&]() {
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int P = 0; P < 2; ++P)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int c = 0; c < 4; ++c) acc[r][P][nt][c] = 0.f;
    };
    constexpr int kAccRegs = R * 2 * NT * 4;
    float *accf = &acc[0][0][0][0];
    // Rendezvous of the 16 warps.  A plain CTA barrier: every warp runs the same unit loop, nothing
    // in this kernel waits on another CTA or on an asynchronous engine, so it cannot stall.  (An
    // mbarrier-based rendezvous cost about a microsecond per use here.)
    auto warps_sync = [&]() -> bool {
        __syncthreads();
        return true;
    };

    // ---- weight prefetch cursor: one block of PF steps ahead of the math, across unit and tile
    // boundaries.  next_block() describes the block at the cursor (per row block: this lane's
    // source address and how many of the PF steps are inside the matrix) and advances the cursor.
    int pb = tile_b, prt = tile_rt, pchunk = chunk, ps0 = (r_begin / PF) * PF;
    int ppos = ps0;  // relative position of the cursor's block
    // next_block() also returns, per row block, the mask of the block's PF steps that are
    // inside the CTA's range and the matrix (bit j = step j).
    auto next_block = [&](const uint8_t *(&src)[R], unsigned (&vmask)[R]) {
        const int col = (pchunk * WK + wk) * 32 * S + ps0 * 32 + t * 8;  // this lane's first column
        const int nv = (p.k - col + 31) / 32;                            // steps whose tile starts before k
        const int lo = max(r_begin - ppos, 0);
        const int hi = active ? min(min(r_end - ppos, PF), nv) : 0;
        const unsigned window = hi > lo ? ((1u << hi) - 1u) & ~((1u << lo) - 1u) : 0u;
#pragma unroll
        for (int rr = 0; rr < R; ++rr) {
            const int rg = prt * (4 * R * WM) + 4 * (wm * R + rr) + (g >> 1);
            const bool in = rg < n_rg && window != 0u;
            vmask[rr] = in ? window : 0u;
            src[rr] = p.q + (in ? (size_t)pb * (size_t)p.q_stride + (size_t)rg * rg_bytes + (size_t)col * 4 + (g & 1) * 16 : 0);
        }
        ps0 += PF;
        ppos += PF;
        if (ps0 == S) {
            ps0 = 0;
            if (++pchunk == p.chunks) {
                pchunk = 0;
                ++prt;
                if (BATCHED && prt == p.row_tiles) { prt = 0; ++pb; }
            }
        }
    };

    auto compute = [&](const uint4 (&wv)[R], const uint4 (&xv)[NT]) {
#pragma unroll
        for (int rr = 0; rr < R; ++rr) {
            const uint32_t w[4] = {wv[rr].x, wv[rr].y, wv[rr].z, wv[rr].w};
            uint32_t a[2][8];
#pragma unroll
            for (int P = 0; P < 2; ++P) {
                const uint32_t wa = w[2 * P], wb = w[2 * P + 1];
                a[P][0] = lut_lookup(wa, lane_key, 0x7604); a[P][1] = lut_lookup(wb, lane_key, 0x7604);
                a[P][2] = lut_lookup(wa, lane_key, 0x7614); a[P][3] = lut_lookup(wb, lane_key, 0x7614);
                a[P][4] = lut_lookup(wa, lane_key, 0x7624); a[P][5] = lut_lookup(wb, lane_key, 0x7624);
                a[P][6] = lut_lookup(wa, lane_key, 0x7634); a[P][7] = lut_lookup(wb, lane_key, 0x7634);
            }
            // k-half-major order: the two MMAs into one accumulator are never back to back, so the
            // accumulate dependency is hidden behind the other accumulators' MMAs
#pragma unroll
            for (int P = 0; P < 2; ++P)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) mma_m16n8k16(acc[rr][P][nt], a[P][0], a[P][1], a[P][2], a[P][3], xv[nt].x, xv[nt].y);
#pragma unroll
            for (int P = 0; P < 2; ++P)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) mma_m16n8k16(acc[rr][P][nt], a[P][4], a[P][5], a[P][6], a[P][7], xv[nt].z, xv[nt].w);
        }
    };

    // Everything that follows the last unit of a segment (the units of one tile inside this
    // CTA's range: chunks [c0, c1) of tile seg_tile).
    auto finish_segment = [&](const int seg_tile, const int t0, const int t1) -> bool {  // steps [t0, t1) of the tile
        // ---- reduce the warps that share rows: fixed binary tree over wk
        if (WK > 1) {
            for (int half = 1; half < WK; half <<= 1) {
                const bool sender = active && (wk & (2 * half - 1)) == half;
                const bool receiver = active && (wk & (2 * half - 1)) == 0 && wk + half < WK;
                const uint32_t slot = red_addr + (uint32_t)(((wk >> 1) / half) * WM + wm) * (uint32_t)(kAccRegs * 128) + lane * 4;
                if (sender) {
#pragma unroll
                    for (int i = 0; i < kAccRegs; ++i)
                        asm volatile("st.shared.f32 [%0], %1;" ::"r"(slot + i * 128), "f"(accf[i]) : "memory");
                }
                if (!warps_sync()) return false;
                if (receiver) {
#pragma unroll
                    for (int i = 0; i < kAccRegs; ++i) {
                        float v;
                        asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(slot + i * 128));
                        accf[i] += v;
                    }
                }
                if (!warps_sync()) return false;
            }
        }

        // ---- a tile cut across CTAs: partials through the workspace.  Every warp that holds
        // sums (wk == 0) handles its own rows alone: it writes its partial, arrives at the counter
        // of its slice of the tile, and the last warp to arrive there adds the slice's partials in
        // segment order and stores the rows.  No CTA-wide rendezvous; the other warps go on.
        const bool full_tile = (t0 == 0 && t1 == tile_steps);
        bool do_store = full_tile;
        if (!full_tile && active && wk == 0) {
            const size_t tile_floats = (size_t)WM * kAccRegs * 32;
            float *dst = p.partials + (size_t)(2 * cta + (t0 == 0 ? 1 : 0)) * tile_floats + (size_t)wm * kAccRegs * 32 + lane;
#pragma unroll
            for (int i = 0; i < kAccRegs; ++i) dst[i * 32] = accf[i];
            __threadfence();
            __syncwarp();
            const int cta_first = cta_of_step(seg_tile * tile_steps);
            const int cta_last = cta_of_step((seg_tile + 1) * tile_steps - 1);
            const int nseg = cta_last - cta_first + 1;
            unsigned int *counter = p.counters + (size_t)seg_tile * kStreamWarps + wm;
            unsigned int old = 0;
            if (lane == 0) old = atomicAdd(counter, 1u);
            old = __shfl_sync(0xffffffffu, old, 0);
            if (old == (unsigned)nseg - 1) {
                if (lane == 0) *counter = 0;  // leave the counter clean for the next call
                __threadfence();
#pragma unroll
                for (int i = 0; i < kAccRegs; ++i) accf[i] = 0.f;
                // segments in unit order (the sum does not depend on arrival order); the loads of
                // several segments are issued before their adds so that L2 latency is paid once per group
                auto seg_ptr = [&](int s) {
                    return p.partials + (size_t)(2 * (cta_first + s) + (s == 0 ? 1 : 0)) * tile_floats +
                           (size_t)wm * kAccRegs * 32 + lane;
                };
                constexpr int kFix = kAccRegs >= 16 ? 2 : 4;  // segments in flight (register budget)
                int s = 0;
                for (; s + kFix <= nseg; s += kFix) {
                    float v[kFix][kAccRegs];
#pragma unroll
                    for (int q = 0; q < kFix; ++q) {
                        const float *src = seg_ptr(s + q);
#pragma unroll
                        for (int i = 0; i < kAccRegs; ++i) v[q][i] = __ldcg(src + i * 32);
                    }
#pragma unroll
                    for (int q = 0; q < kFix; ++q)
#pragma unroll
                        for (int i = 0; i < kAccRegs; ++i) accf[i] += v[q][i];
                }
                for (; s < nseg; ++s) {
                    const float *src = seg_ptr(s);
#pragma unroll
                    for (int i = 0; i < kAccRegs; ++i) accf[i] += __ldcg(src + i * 32);
                }
                do_store = true;
            }
        }

        // ---- epilogue: fp32 scale by absmax, one rounding to fp16, 8-byte stores of 4 rows
        if (do_store && active && wk == 0) {
#pragma unroll
            for (int rr = 0; rr < R; ++rr) {
                const int row = tile_rt * 32 * R * WM + (wm * R + rr) * 32 + 4 * g;  // in matrix tile_b
                if (row >= p.m) continue;  // m % 8 == 0 and the 4 rows sit inside one 8-row group
                // four scalar loads: absmax only has to be 4-byte aligned (a slice of a larger scale buffer)
                const float *scp = reinterpret_cast<const float *>(
                    reinterpret_cast<const uint8_t *>(p.absmax) + (size_t)tile_b * (size_t)p.absmax_stride + (size_t)row * 4);
                const float4 sc = make_float4(__ldg(scp), __ldg(scp + 1), __ldg(scp + 2), __ldg(scp + 3));
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {  // token 2t + e
                        const int tok = p.tok0 + nt * 8 + 2 * t + e;
                        if (tok >= p.n) continue;
                        uint2 v;
                        v.x = pack_half2(acc[rr][0][nt][e] * sc.x, acc[rr][0][nt][2 + e] * sc.y);
                        v.y = pack_half2(acc[rr][1][nt][e] * sc.z, acc[rr][1][nt][2 + e] * sc.w);
                        *reinterpret_cast<uint2 *>(reinterpret_cast<uint8_t *>(p.o) + (size_t)tile_b * (size_t)p.o_stride +
                                                   ((size_t)tok * p.m + row) * 2) = v;
                    }
                }
            }
        }
        zero_acc();
        return true;
    };

    // ---- main loop: units of this CTA; inside a unit S steps in blocks of PF, so that the
    // register ring is indexed statically and the prefetch addresses are immediates
    uint4 ring[PF][R];
    {
        const uint8_t *src[R];
        unsigned vmask[R];
        next_block(src, vmask);
#pragma unroll
        for (int j = 0; j < PF; ++j)
#pragma unroll
            for (int rr = 0; rr < R; ++rr) ring[j][rr] = ldg_stream_pred(src[rr] + j * 128, (vmask[rr] >> j) & 1u);
    }
    int seg_t0 = first_in_tile;  // where in its tile the current segment began
    zero_acc();
    // Stages the activations of unit (`xchunk`) into buffer `b`: every thread copies 16-byte
    // pieces; tokens >= n and columns >= k are filled with zeros.
    const int pieces_per_row = 4 * S * WK;  // 16-byte pieces of one token row of a unit
    auto stage_x = [&](int xbatch, int xchunk, int b) {
        const __half *xbase = reinterpret_cast<const __half *>(reinterpret_cast<const uint8_t *>(p.x) + (size_t)xbatch * (size_t)p.x_stride);
        const int c0 = xchunk * 32 * S * WK;
        for (int i = threadIdx.x; i < NT * 8 * pieces_per_row; i += kStreamThreads) {
            const int row = i / pieces_per_row, pc = i - row * pieces_per_row;
            const int tok = p.tok0 + row, c = c0 + pc * 8;
            const bool in = tok < p.n && c < p.k;
            cp_async16(xbuf_addr + (uint32_t)b * x_buf_bytes + (uint32_t)row * x_pitch + (uint32_t)pc * 16,
                       in ? (const void *)(xbase + (size_t)tok * p.k + c) : (const void *)p.x, in ? 16u : 0u);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // this lane's 16 bytes of a step inside a buffer: token row g (+8 per token group), piece t
    const uint32_t x_lane = (uint32_t)g * x_pitch + (uint32_t)wk * 64u * (uint32_t)S + (uint32_t)t * 16;

    int xb = 0;
    bool ok = true;
    // Start-up order: the first weights are already on their way (above; weights and the codebook
    // are constants).  Everything another kernel may have written - activations, the workspace,
    // the output - is touched only after the grids this one depends on have completed.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (n_steps > 0) stage_x(tile_b, chunk, 0);
    // byte -> half2 table: even column = high nibble in the low half; 32 copies, one per bank.
    // Built while the first activations and weights are in flight.  Warp w writes the entries
    // w, w + 16, ...: their low nibble is w, their high nibble counts up.
    {
        const float cv = p.code[lane & 15];
        const uint32_t ch = (uint32_t)__half_as_ushort(__float2half_rn(cv));
        const uint32_t lo16 = __shfl_sync(0xffffffffu, ch, warp & 15) << 16;
        for (int e = warp; e < 256; e += kStreamWarps) {
            const uint32_t v = __shfl_sync(0xffffffffu, ch, e >> 4) | lo16;
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(lut_addr + (uint32_t)e * 256 + lane * 4), "r"(v) : "memory");
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    ok = warps_sync();

    // `pos` is the relative position of the current unit's first step
    for (int pos = 0; ok && n_steps > 0 && pos < r_end; pos += S) {
        const int s_lo = max(r_begin - pos, 0), s_hi = min(r_end - pos, S);  // this unit's steps in range
        const bool last_unit = pos + S >= r_end;
        if (!last_unit) {  // next unit, other buffer
            const bool wrap = chunk + 1 == p.chunks;
            stage_x((BATCHED && wrap && tile_rt + 1 == p.row_tiles) ? tile_b + 1 : tile_b, wrap ? 0 : chunk + 1, xb ^ 1);
        }
        if (active) {
            const int s_first = (s_lo / PF) * PF;
            uint32_t xsrc = xbuf_addr + (uint32_t)xb * x_buf_bytes + x_lane + (uint32_t)s_first * 64u;
            for (int s0 = s_first; s0 < s_hi; s0 += PF, xsrc += PF * 64) {
                const uint8_t *src[R];
                unsigned vmask[R];
                next_block(src, vmask);  // the block PF steps ahead of this one
                const int jlo = max(s_lo - s0, 0), jhi = min(s_hi - s0, PF);
                const unsigned cmask = ((1u << jhi) - 1u) & ~((1u << jlo) - 1u);  // this block's steps inside the range
#pragma unroll
                for (int j = 0; j < PF; ++j) {
                    uint4 wv[R], xv[NT];
#pragma unroll
                    for (int rr = 0; rr < R; ++rr) {
                        wv[rr] = ring[j][rr];
                        ring[j][rr] = ldg_stream_pred(src[rr] + j * 128, (vmask[rr] >> j) & 1u);
                    }
                    if ((cmask >> j) & 1u) {
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) xv[nt] = lds128(xsrc + j * 64 + (uint32_t)nt * 8u * x_pitch);
                        compute(wv, xv);
                    }
                }
            }
        }
        // the next unit's activations have landed and everybody is done with this unit's
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        if (!warps_sync()) break;
        xb ^= 1;
        const bool seg_end = (chunk + 1 == p.chunks) || last_unit;
        if (seg_end && !finish_segment(tile, seg_t0, chunk * S + s_hi)) break;
        if (++chunk == p.chunks) {
            chunk = 0;
            ++tile;
            ++tile_rt;
            if (BATCHED && tile_rt == p.row_tiles) { tile_rt = 0; ++tile_b; }
        }
        if (seg_end) seg_t0 = 0;  // a later segment of this CTA starts a tile
    }
}

// ------------------------------------------------------------------ host side

// one arrival counter per (row tile, warp slice of the tile)
static size_t stream_counter_bytes(int row_tiles) { return ((size_t)row_tiles * kStreamWarps * 4 + 255) / 256 * 256; }

// The even split of the steps over the CTAs; false when the step count leaves 32-bit range.
static bool stream_split_steps(StreamParams *p, int ctas)
{
    const long long steps = p->units * p->ksteps;
    if (steps >= (1ll << 31) || ctas < 1) return false;
    p->steps_q = (int)(steps / ctas);
    p->steps_r = (int)(steps % ctas);
    return true;
}

static void stream_geometry(int m, int k, const tuna_config &c, int nt, int batch, StreamParams *p)
{
    p->batch = batch;
    p->warps_m = c.warps_m; p->warps_k = c.warps_k; p->ksteps = c.k_steps;
    const int tile_rows = 32 * c.rows_per_warp * c.warps_m;
    const int chunk_cols = 32 * c.k_steps * c.warps_k;
    p->row_tiles = div_up(m, tile_rows);
    p->chunks = div_up(k, chunk_cols);
    p->units = (long long)batch * p->row_tiles * p->chunks;
    const int acc_regs = c.rows_per_warp * 2 * nt * 4;
    p->red_bytes = c.warps_k > 1 ? (c.warps_k / 2) * c.warps_m * acc_regs * 128 : 0;
    p->x_buf_bytes = nt * 8 * (chunk_cols * 2 + 64);
}

// Dynamic shared memory: up to 64 KB of slack in front of the table (it must sit on a 64-KB
// boundary of the shared window), the table, the reduction scratch.
static size_t stream_smem_bytes(const StreamParams &p) { return 65536 + kLut64Bytes + (size_t)p.red_bytes + 2 * (size_t)p.x_buf_bytes; }
constexpr size_t kStreamSmemLimit = 227 * 1024 - 1024;

int gemm_stream_normalize_config(int m, int n, int k, int sm_count, tuna_config *c)
{
    if (c->tile_tok == 0) c->tile_tok = (n <= 8) ? 8 : (n <= 16 ? 16 : 32);
    if (c->tile_tok != 8 && c->tile_tok != 16 && c->tile_tok != 32) return TUNA_ERR_BAD_CONFIG;
    const int nt = c->tile_tok / 8;
    if (c->ctas < 0) return TUNA_ERR_BAD_CONFIG;
    if (c->ctas == 0 || c->ctas > sm_count) c->ctas = sm_count;
    StreamParams p;
    if (c->rows_per_warp == 0 || c->warps_m == 0 || c->warps_k == 0 || c->k_steps == 0) {
        // No table entry: pick the geometry with the least estimated overhead.  Weights are read
        // once whatever the geometry; what differs is the per-unit bookkeeping, the split-K
        // partials (written and read back once per cut tile) and the in-CTA reduction.
        double best = 1e300;
        tuna_config bc = *c;
        for (int r = 1; r <= 2; ++r)
            for (int wm = 1; wm <= 16; wm <<= 1)
                for (int ks = kLoadsInFlight; ks <= 32; ks <<= 1) {
                    tuna_config t = *c;
                    t.rows_per_warp = c->rows_per_warp ? c->rows_per_warp : r;
                    t.warps_m = c->warps_m ? c->warps_m : wm;
                    t.warps_k = c->warps_k ? c->warps_k : 16 / t.warps_m;
                    t.k_steps = c->k_steps ? c->k_steps : ks;
                    if (!c->warps_k)
                        while (t.warps_k > 1 && 32 * t.k_steps * (t.warps_k / 2) >= k) t.warps_k >>= 1;
                    if (t.rows_per_warp * nt > 4 || t.warps_m * t.warps_k > kStreamWarps) continue;
                    stream_geometry(m, k, t, nt, 1, &p);
                    if (stream_smem_bytes(p) > kStreamSmemLimit) continue;
                    const double tile_bytes = (double)t.warps_m * t.rows_per_warp * 32 * nt * 8 * 4;
                    const double cuts = (p.units % c->ctas == 0 && p.chunks % (p.units / c->ctas) == 0) ? 0 : 2.0 * c->ctas;
                    const double pad = ((double)p.row_tiles * 32 * t.rows_per_warp * t.warps_m / m) *
                                       ((double)p.chunks * 32 * t.k_steps * t.warps_k / k);  // work on padding
                    double cost = (double)m * k / 2 * pad + 3.0 * cuts * tile_bytes + (double)p.units * kStreamWarps * 512 +
                                  2e5 * t.warps_k + (t.rows_per_warp == 2 ? 1e5 : 0);
                    if (cost < best) { best = cost; bc = t; }
                }
        if (best >= 1e300) return TUNA_ERR_BAD_CONFIG;
        *c = bc;
    }
    auto pow2 = [](int v) { return v > 0 && (v & (v - 1)) == 0; };
    if (c->rows_per_warp != 1 && c->rows_per_warp != 2) return TUNA_ERR_BAD_CONFIG;
    if (c->rows_per_warp * nt > 4) return TUNA_ERR_BAD_CONFIG;  // accumulator registers
    if (!pow2(c->k_steps) || c->k_steps > 64 || c->k_steps % (kLoadsInFlight / c->rows_per_warp)) return TUNA_ERR_BAD_CONFIG;
    if (!pow2(c->warps_m) || !pow2(c->warps_k) || c->warps_m * c->warps_k > kStreamWarps) return TUNA_ERR_BAD_CONFIG;
    stream_geometry(m, k, *c, nt, 1, &p);
    if (stream_smem_bytes(p) > kStreamSmemLimit) return TUNA_ERR_BAD_CONFIG;
    (void)n;
    return TUNA_OK;
}

size_t gemm_stream_workspace_bytes(int m, int n, int k, const tuna_config &c, int sm_count, int batch)
{
    (void)n;
    StreamParams p;
    const int nt = c.tile_tok / 8;
    stream_geometry(m, k, c, nt, batch, &p);
    const size_t counters = stream_counter_bytes(batch * p.row_tiles);
    return partial_region_bytes(sm_count) + counters;
}

template <int R, int NT, bool BATCHED>
static int launch_one_b(const StreamParams &p, int ctas, size_t smem, cudaStream_t stream)
{
    static bool attr_set[64] = {false};  // one-time, per device, opt-in to large dynamic shared memory
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return TUNA_ERR_NO_DEVICE;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!attr_set[dev]) {
            if (cudaFuncSetAttribute(gemm_stream_kernel<R, NT, BATCHED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)kStreamSmemLimit) != cudaSuccess)
                return TUNA_ERR_NO_DEVICE;
            attr_set[dev] = true;
        }
    }
    // Programmatic dependent launch: this grid may become resident while the previous kernel of
    // the stream is still draining; the kernel orders itself with griddepcontrol.wait.
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3((unsigned)ctas);
    lc.blockDim = dim3(kStreamThreads);
    lc.dynamicSmemBytes = smem;
    lc.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr;
    lc.numAttrs = 1;
    return cudaLaunchKernelEx(&lc, gemm_stream_kernel<R, NT, BATCHED>, p) == cudaSuccess ? TUNA_OK : TUNA_ERR_LAUNCH;
}

template <int R, int NT>
static int launch_one(const StreamParams &p, int ctas, size_t smem, cudaStream_t stream)
{
    return p.batch > 1 ? launch_one_b<R, NT, true>(p, ctas, smem, stream) : launch_one_b<R, NT, false>(p, ctas, smem, stream);
}

// The launches of one GEMM (one per pass of tile_tok tokens) with the given scratch: `partials`
// holds two partial tiles per CTA, `counters` one zeroed word per (row tile, warp slice).
static int stream_launch_passes(const GemmArgs &a, const tuna_config &cfg, float *partials, unsigned int *counters,
                                DeviceStatus *status)
{
    const int nt = cfg.tile_tok / 8;
    StreamParams p;
    std::memset(&p, 0, sizeof(p));
    p.q = a.q; p.x = (const __half *)a.x; p.code = a.code; p.absmax = a.absmax; p.o = (__half *)a.o;
    p.m = a.m; p.n = a.n; p.k = a.k;
    stream_geometry(a.m, a.k, cfg, nt, a.batch, &p);
    p.q_stride = (long long)a.q_stride; p.x_stride = (long long)a.x_stride;
    p.absmax_stride = (long long)a.absmax_stride; p.o_stride = (long long)a.o_stride;
    p.status = status;
    p.partials = partials;
    p.counters = counters;
    int ctas = cfg.ctas;
    {   // no CTA with less than one block of prefetched steps
        const long long blocks = p.units * (cfg.k_steps / (kLoadsInFlight / cfg.rows_per_warp));
        if ((long long)ctas > blocks) ctas = (int)blocks;
    }
    if (!stream_split_steps(&p, ctas)) return TUNA_ERR_TOO_LARGE;
    const size_t smem = stream_smem_bytes(p);

    for (int tok0 = 0; tok0 < a.n; tok0 += cfg.tile_tok) {
        p.tok0 = tok0;
        int st;
        switch (cfg.rows_per_warp * 10 + nt) {
            case 11: st = launch_one<1, 1>(p, ctas, smem, a.stream); break;
            case 12: st = launch_one<1, 2>(p, ctas, smem, a.stream); break;
            case 14: st = launch_one<1, 4>(p, ctas, smem, a.stream); break;
            case 21: st = launch_one<2, 1>(p, ctas, smem, a.stream); break;
            case 22: st = launch_one<2, 2>(p, ctas, smem, a.stream); break;
            default: return TUNA_ERR_BAD_CONFIG;
        }
        if (st != TUNA_OK) return st;
    }
    return TUNA_OK;
}

int launch_gemm_stream(const GemmArgs &a, const tuna_config &cfg)
{
    DeviceStatus *status = device_status_word();
    if (!status) return TUNA_ERR_NO_DEVICE;
    if (a.workspace == nullptr || a.workspace_bytes < gemm_stream_workspace_bytes(a.m, a.n, a.k, cfg, a.sm_count, a.batch))
        return TUNA_ERR_WORKSPACE;
    return stream_launch_passes(a, cfg, (float *)a.workspace,
                                (unsigned int *)((uint8_t *)a.workspace + partial_region_bytes(a.sm_count)), status);
}

// Scratch of the entry point that allocates nothing (below): its own compact layout,
// [counters of this shape][two partial tiles per CTA of this configuration].
size_t gemm_stream_compact_scratch_bytes(int m, int k, const tuna_config &c, size_t *counter_bytes)
{
    StreamParams geo;
    const int nt = c.tile_tok / 8;
    stream_geometry(m, k, c, nt, 1, &geo);
    const size_t tile_floats = (size_t)c.warps_m * (c.rows_per_warp * 2 * nt * 4) * 32;
    *counter_bytes = stream_counter_bytes(geo.row_tiles);
    return *counter_bytes + 2 * (size_t)c.ctas * tile_floats * 4;
}

int launch_gemm_stream_compact(const GemmArgs &a, const tuna_config &cfg, void *scratch, size_t counter_bytes, DeviceStatus *status)
{
    return stream_launch_passes(a, cfg, (float *)((uint8_t *)scratch + counter_bytes), (unsigned int *)scratch, status);
}

}  // namespace tuna

// ------------------------------------------------------------------ entry point that allocates nothing
//
// Scratch of the streaming kernel (tile counters + split-K partial tiles) and its status word live
// in file-scope device arrays, so that a caller that must not allocate device memory while it runs
// can still use the GEMM.  In host code the array names are only handles: the device addresses come
// from cudaGetSymbolAddress, looked up once per device with that device current.
static __device__ __align__(256) unsigned char g_noalloc_scratch[TUNA_NOALLOC_SCRATCH_BYTES];
static __device__ __align__(256) tuna::DeviceStatus g_noalloc_status;

namespace {
struct NoAllocDevice {
    bool ready = false;
    void *scratch = nullptr;
    tuna::DeviceStatus *status = nullptr;
};
NoAllocDevice g_noalloc_devices[64];
std::mutex g_noalloc_mutex;
}  // namespace

extern "C" int tuna_matmul_noalloc(const void *q, const void *x, const void *code, const void *absmax, void *o,
                                   int m, int n, int k, void *stream)
{
    using namespace tuna;
    if (!q || !x || !code || !absmax || !o) return TUNA_ERR_NULL_POINTER;
    if (m <= 0 || k <= 0 || n <= 0 || (m % 8) || (k % 8)) return TUNA_ERR_BAD_SHAPE;
    if ((long long)m * k / 2 > (1ll << 40)) return TUNA_ERR_TOO_LARGE;  // the same limit as tuna_matmul
    auto misaligned = [](const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) != 0; };
    if (misaligned(q, 16) || misaligned(x, 16) || misaligned(o, 16) || misaligned(absmax, 4) || misaligned(code, 4))
        return TUNA_ERR_MISALIGNED;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return TUNA_ERR_NO_DEVICE;
    NoAllocDevice &d = g_noalloc_devices[dev];
    {
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        if (!d.ready) {  // first call on this device: resolve the device addresses of the two arrays
            void *p = nullptr, *s = nullptr;
            if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess) return TUNA_ERR_NO_DEVICE;
            if (cudaGetSymbolAddress(&s, g_noalloc_status) != cudaSuccess) return TUNA_ERR_NO_DEVICE;
            d.scratch = p;
            d.status = (DeviceStatus *)s;
            d.ready = true;
        }
    }
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return TUNA_ERR_NO_DEVICE;
    tuna_config c;
    std::memset(&c, 0, sizeof(c));
    c.path = TUNA_PATH_STREAM;
    int st = tuna_lookup_config(m, n, k, &c);  // the table's choice when it is a streaming one
    if (st != TUNA_OK || c.path != TUNA_PATH_STREAM) {
        std::memset(&c, 0, sizeof(c));
        c.path = TUNA_PATH_STREAM;
        st = gemm_stream_normalize_config(m, n, k, sms, &c);
        if (st != TUNA_OK) return st;
    }
    size_t counters = 0;
    const size_t need = gemm_stream_compact_scratch_bytes(m, k, c, &counters);
    if (need > (size_t)TUNA_NOALLOC_SCRATCH_BYTES) return TUNA_ERR_TOO_LARGE;
    // the counters must start at zero; the array keeps whatever the last call (or an aborted one) left
    if (cudaMemsetAsync(d.scratch, 0, counters, (cudaStream_t)stream) != cudaSuccess) return TUNA_ERR_LAUNCH;
    GemmArgs a;
    a.q = (const uint8_t *)q; a.x = x; a.code = (const float *)code; a.absmax = (const float *)absmax; a.o = o;
    a.m = m; a.n = n; a.k = k; a.workspace = nullptr; a.workspace_bytes = 0;
    a.stream = (cudaStream_t)stream; a.sm_count = sms;
    return launch_gemm_stream_compact(a, c, d.scratch, counters, d.status);
}
