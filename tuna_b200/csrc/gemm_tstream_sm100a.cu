// Weight-streaming FP16 x 4-bit(codebook) GEMM on tcgen05 for small token counts (one pass
// covers 16, 32 or 64 tokens) on sm_100a: the memory-bound regime every row of the
// reference's README table is measured in.  Counterpart of the reference's Tuna<> kernel and its
// cp.async / ldmatrix / mma.sync main loop (kernel.cu:1043-2505, 2816-2960); the orientation
// is kept (weights are MMA operand A, tokens operand B, the accumulator is an o^T tile,
// kernel.cu:2182-2192) and nothing else.
//
// The idea.  The packed layout stores an 8x8 weight tile as 32 bytes (test.py:58-65: byte j =
// row j/4, column pair j%4), so the 8 columns of one row are one 32-bit word of the tile.  A
// dequant thread owns one weight row = one tensor-memory lane: per 32-column step it reads the
// row's four words (one per tile), turns their 16 bytes into 16 half2 by 16 table lookups and
// writes them to 16 consecutive tensor-memory columns with one tcgen05.st (shape 32x32b).  K
// stays in natural order, so the activations need no re-ordering at all: TMA writes x straight
// into the 128-byte-swizzled K-major tiles the MMA's shared-memory descriptor reads.  The
// dequantised weights exist only in registers and tensor memory.  (An earlier version used the
// 16x256b store shape, whose fragment is exactly a 16-byte piece of the packed layout: no
// row permutation to undo, but a K permutation that two extra warps had to apply to x through
// shared memory, and a store shape that costs the tensor-memory write path a third more.)
// Which row a lane holds is chosen for the shared-memory reads: lane 32q + l holds row
// 8*rg + l%8 with rg = 8*(q/2) + q%2 + 2*(l/8), so the four row groups a warp reads at once
// differ in bits 1-2 of rg - the bits the 128-byte swizzle XORs into the 16-byte chunk index -
// and the warp's 32-bit reads are bank-conflict free.  The epilogue undoes it (one lane per thread).
//
// The packed weights are staged by TMA: per slot (16 row groups x 512 or 1024 bytes = 128 rows
// x 128 or 256 columns) one 3-D box, or one 2-D box per step where the 3-D view does not exist
// (k not a multiple of 32), into an mbarrier-tracked ring of [step][row group][128 bytes]
// stages, 128-byte swizzled, that takes all the shared memory left; out-of-range rows and
// columns are zero-filled by the copy engine.  (A first version streamed the weights with
// ld.global into a per-lane register ring: 64 KB per SM at best, less whenever a warp was busy
// converting, and the loaded HBM latency of ~2 us capped it near 3.3 TB/s.)
//
// One persistent CTA per SM, warp-specialised (24 warps; 80 registers per
// thread.  Re-balancing registers between warpgroups with setmaxnreg made ptxas spill more,
// not less, in this kernel):
//   warp 0       MMA issue: tcgen05.mma (M=128, N=tile_tok, K=16, fp32 accumulate), A from tensor
//                memory, B through a 128-byte-swizzle shared-memory descriptor, D in tensor memory.
//                The warp stays converged and one elected lane issues (a lone diverged thread
//                running this loop needed ~80 clocks per MMA instead of ~12); a slot is 8 or 16
//                MMAs per wait and commit, because that fixed cost per slot is what limits it
//   warps 1, 3   idle (they only help to build the lookup table)
//   warp 2       copy producer: TMA boxes of packed weights into the weight ring and of x (fp16
//                [n,k], L2 resident; one box per 64 columns) into the activation ring
//   warps 4-7    epilogue: tcgen05.ld of the accumulator, fp32 scale by absmax, fp16 store,
//                split-K partials and fix-up
//   warps 8-23   dequant: ld.shared.u32 -> prmt + ld.shared table lookups -> tcgen05.st into the A
//                slots.  A warp handles rows 32q..+31 (q = its 32-lane quarter) and four
//                32-column steps of a slot; with 128-column slots four groups of four warps
//                convert four slots at once, with 256-column slots two groups of eight warps two.
// The scale is constant along K (one block per row, test.py:81, kernel.cu:2178-2180) and is
// applied once, in fp32, to the accumulated sum.
//
// Work decomposition ("stream-K"): a unit is (tile of 128*row_blocks rows, 128- or 256-column chunk) =
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

constexpr int kTsMaxASlots = 8;       // A-slot ring: as many slots as the accumulators leave room for
constexpr int kTsTmemCols = 512;
constexpr int kTsMaxXStages = 6;
constexpr int kTsMaxWStages = 16;     // weight ring: as many stages as shared memory holds
constexpr int kTsLutBytes = 256 * 128;    // byte -> half2 table: 256 entries, 32 copies (one per bank) of 4 bytes
constexpr int kTsSmemTotal = 227 * 1024;             // static + dynamic shared memory of a CTA on sm_100
constexpr int kTsSmemDynamic = kTsSmemTotal - 1024;  // the static part (barriers) stays below 1 KB
constexpr int kTsDequantWarp0 = 8;
#ifndef TS_DEQUANT_WARPS
#define TS_DEQUANT_WARPS 16
#endif
constexpr int kTsDequantWarps = TS_DEQUANT_WARPS;
constexpr int kTsThreads = 32 * (kTsDequantWarp0 + kTsDequantWarps);

constexpr int kTsMaxSeq = 64;  // GEMMs of one launch (tuna_matmul_sequence)
constexpr int kMaxPeers = TUNA_MAX_PEERS;

// One GEMM of a launch.  The two tensor maps are what the copy producer hands to TMA; everything
// else is read by the epilogue warps and the cursors.
struct __align__(64) TsGemm {
    CUtensorMap map_q;   // packed weights: the 5-D view (w_mode 1), else the 3-D view if q3d, else [m/8 row groups] x [k 32-bit words]
    CUtensorMap map_x;   // activations as [n] x [k] fp16
    const float *absmax;
    __half *o;
    int m, n, k;
    int chunks;       // ceil(k / chunk columns)
    int row_tiles;    // ceil(m / (128 RB))
    int unit0;        // index of its first unit in the launch's unit sequence
    int tile0;        // index of its first tile among the launch's tiles (arrival counters)
    int q3d;          // map_q is the 3-D view (one copy per slot) rather than the 2-D one (one copy per step)
    long long slab_off;  // exchange launches: offset of this rank's slab for this GEMM inside a parity region, -1: none (o is written)
};

struct TsParams {
    const float *code;
    float *partials;
    unsigned int *counters;
    DeviceStatus *status;
    int count;        // GEMMs of this launch
    int tok0;         // first token of this pass (0 unless a single GEMM runs as several passes)
    int row_blocks;   // RB: 128-row blocks per tile
    int a_slots;      // A-slot ring depth
    int a_base;       // first tensor-memory column of the A slots (behind the two accumulator buffers)
    int acc_cols;     // columns of one accumulator buffer
    int units;        // units of all the GEMMs
    int units_q, units_r;  // units = units_q * CTAs + units_r: the first units_r CTAs take units_q + 1
    int w_mode;       // layout of the weight stages (the kernel's WMODE)
    // Exchange launches (K-split GEMMs whose partial outputs every rank sums): instead of o, a
    // finished row goes to this rank's slab ([row][tile_tok] fp16) in the exchange buffer of every
    // rank, with ordinary stores to peer memory; the reduce kernel that follows sums the slabs.
    int n_peers;                 // 0: an ordinary launch
    unsigned char *peer[kMaxPeers];
    const unsigned int *epoch;   // exchanges completed so far on this rank (device counter): its parity selects the region
    long long region0, region_bytes;  // offset of parity region 0 inside an exchange buffer, and the size of a region
};

template <int MAXG>
struct __align__(64) TsLaunch {
    TsParams c;
    TsGemm g[MAXG];
};

// Table lookup: the selected byte of w (two 4-bit codes) -> half2 of the two code values.  Entry e
// of the table lies at 128 * e, one copy per bank: conflict free.
__device__ __forceinline__ uint32_t ts_lookup(uint32_t w, uint32_t lane_base, uint32_t selector)
{
    uint32_t b, v;
    asm("prmt.b32 %0, %1, 0, %2;" : "=r"(b) : "r"(w), "r"(selector));
    // not volatile: the table is constant once built, so the compiler may schedule lookups freely
    asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(lane_base + (b << 7)));
    return v;
}

// The same lookup when the table lies at shared address 0x10000 with 256 bytes per entry: the
// address 0x10000 + 256 * byte + 4 * lane is assembled by ONE prmt from `key` = 0x00010000 | 4 * lane
// (bytes 0, 2, 3) and the selected byte of w (byte 1); `selector` = 0x7604 | (byte index << 4).
__device__ __forceinline__ uint32_t ts_lookup256(uint32_t w, uint32_t key, uint32_t selector)
{
    uint32_t a, v;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(a) : "r"(w), "r"(key), "r"(selector));
    asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}

// The CTA whose range holds unit u.
__device__ __forceinline__ int ts_cta_of_unit(const TsParams &p, int u)
{
    const int big = p.units_r * (p.units_q + 1);
    return u < big ? u / (p.units_q + 1) : p.units_r + (u - big) / p.units_q;
}

// Position in a CTA's contiguous range of the launch's unit sequence (GEMM after GEMM, each
// tile-major): which GEMM, which row tile, which K chunk.
struct TsCursor {
    int g, tile, chunk;
    int chunks, row_tiles;  // of GEMM g
    int left;               // units of the range still ahead, including the current one
    bool seg_first;         // the current unit starts a segment (the units of one tile inside the range)
    template <class Launch>
    __device__ void init(const Launch &L, int u_begin, int n_units)
    {
        g = 0;
        while (g + 1 < L.c.count && L.g[g + 1].unit0 <= u_begin) ++g;
        chunks = L.g[g].chunks;
        row_tiles = L.g[g].row_tiles;
        const int r = u_begin - L.g[g].unit0;
        tile = r / chunks;
        chunk = r - tile * chunks;
        left = n_units;
        seg_first = true;
    }
    __device__ bool seg_last() const { return chunk + 1 == chunks || left == 1; }
    template <class Launch>
    __device__ void next(const Launch &L)
    {
        seg_first = seg_last();
        --left;
        if (++chunk == chunks) {
            chunk = 0;
            if (++tile == row_tiles && left > 0) {
                tile = 0;
                ++g;
                chunks = L.g[g].chunks;
                row_tiles = L.g[g].row_tiles;
            }
        }
    }
};

// STEPS: 32-column steps per slot (4 or 8).  MAXG: capacity of the launch's GEMM table (1 for a
// single GEMM, kTsMaxSeq for a sequence).  WMODE: layout of a weight stage (128-byte rows, 128-byte
// swizzle), the same for all GEMMs of a launch:
//   1  [32-row block][step pair][row group of the block][step of the pair]: one 5-D box per slot
//      that reads global memory in runs of 256 contiguous bytes (m % 32 == 0 and k % 64 == 0);
//      a warp's four row groups are consecutive and the swizzle separates them, so tensor-memory
//      lane l holds row l of the 128;
//   0  [step][row group]: one 3-D box per slot (k % 32 == 0; 128-byte runs, measured 8 % slower in
//      the copy alone) or one 2-D box per step (any k); rows assigned to lanes by lane_row_group().
template <int N_TILE, int STEPS, int MAXG, int WMODE>
__global__ void __launch_bounds__(kTsThreads, 1) gemm_w4a16_tstream_kernel(const __grid_constant__ TsLaunch<MAXG> L)
{
    const TsParams &p = L.c;
    constexpr int kChunkK = 32 * STEPS;                     // columns of a unit / slot
    constexpr int kSlotCols = 16 * STEPS;                   // tensor-memory columns of one A slot
    constexpr int kSlotBytes = 16 * kChunkK * 4;            // packed bytes of a slot: 16 row groups x 4 bytes per column
    constexpr int kHalves = STEPS / 4;                      // warps that share a quarter of a slot
    constexpr int kGroups = kTsDequantWarps / (4 * kHalves);  // slots converted at once
    // Activations of a unit: one tile of [token][64 columns] fp16 (128-byte rows, 128-byte swizzle,
    // 8-token groups 1024 bytes apart) per 64 columns, as TMA writes it and the MMA descriptor reads it.
    constexpr int kXTiles = kChunkK / 64;
    constexpr uint32_t kXTileBytes = N_TILE * 128;
    constexpr uint32_t kXStageBytes = kXTiles * kXTileBytes;
    // activation stages (TMA -> MMA); up to 32 tokens the ring has to fit below the lookup table (shared address 0x10000)
    constexpr int kXS = (N_TILE >= 64 || 4 * kXStageBytes + 4096 > 0x10000) ? 3 : 4;
    constexpr uint32_t kStepBytes = 16 * 128;                         // one step of a weight stage: 16 row groups x 128 bytes
    static_assert(kXS <= kTsMaxXStages, "barrier arrays too small");
    static_assert(N_TILE > 32 || kXS * kXStageBytes + 4096 <= 0x10000, "the activation ring must end below the lookup table");
    static_assert(kXStageBytes % 1024 == 0 && kSlotBytes % 1024 == 0, "swizzle atoms are 1024 bytes");
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ __align__(8) uint64_t bars[2 * kTsMaxASlots + 2 * kTsMaxXStages + 4 + 2 * kTsMaxWStages];
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;

    TS_PROF_DECL
    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;
    const int cta = blockIdx.x;
    const int RB = p.row_blocks;

    // Let the next kernel in the stream become resident as SMs free up.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // Shared memory (everything 1024-byte aligned): the byte -> half2 table (256 entries, one copy per
    // bank), the activation ring, and weight stages in everything that is left.
    //   kLut256 (token tiles up to 32): the table occupies shared addresses [0x10000, 0x20000) with 256
    //   bytes per entry (half of them unused), which lets one prmt build a lookup's address; the
    //   activation ring and the first weight stages lie below it, the other weight stages above.
    //   Otherwise (64-token tiles need the room): 128 bytes per entry at the start of dynamic shared memory.
    constexpr bool kLut256 = N_TILE <= 32;
    const uint32_t dyn0 = smem_u32(smem);
    const uint32_t smem_end = dyn0 + kTsSmemDynamic;
    const uint32_t lut_addr = kLut256 ? 0x10000u : dyn0;
    const uint32_t xring = kLut256 ? dyn0 : dyn0 + kTsLutBytes;
    const uint32_t w_low = xring + kXS * kXStageBytes;                       // first weight stage
    const int n_low = (kLut256 && w_low < 0x10000u) ? (int)((0x10000u - w_low) / kSlotBytes) : 0;   // weight stages below the table
    const uint32_t w_high = kLut256 ? 0x20000u : w_low;
#ifdef TS_WS_LIMIT  // timing experiment: fewer weight stages in flight
    const int WS = min(TS_WS_LIMIT, n_low + (int)((smem_end - w_high) / kSlotBytes));
#else
    const int WS = min(kTsMaxWStages, n_low + (int)((smem_end - w_high) / kSlotBytes));
#endif
    auto w_stage = [&](int i) -> uint32_t { return i < n_low ? w_low + (uint32_t)i * kSlotBytes : w_high + (uint32_t)(i - n_low) * kSlotBytes; };
    if (kLut256 && dyn0 > 4096u) {  // the layout above assumes that dynamic shared memory starts within the first 4 KB
        if (threadIdx.x == 0 && atomicCAS(&p.status->code, 0, 97) == 0) p.status->detail = (int)dyn0;
        return;
    }

    const uint32_t bar0 = smem_u32(&bars[0]);
    const uint32_t a_full = bar0, a_empty = a_full + 8 * kTsMaxASlots;
    const uint32_t x_full = a_empty + 8 * kTsMaxASlots, x_empty = x_full + 8 * kTsMaxXStages;
    const uint32_t d_full = x_empty + 8 * kTsMaxXStages, d_empty = d_full + 16;
    const uint32_t w_full = d_empty + 16, w_empty = w_full + 8 * kTsMaxWStages;
    volatile int *abort_flag = &s_abort;

    // this CTA's contiguous range of units
    const int u_begin = cta * p.units_q + min(cta, p.units_r);
    const int n_units = p.units_q + (cta < p.units_r ? 1 : 0);

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int i = 0; i < kTsMaxASlots; ++i) { mbar_init(a_full + 8 * i, 4 * kHalves); mbar_init(a_empty + 8 * i, 1); }
        for (int i = 0; i < kTsMaxXStages; ++i) { mbar_init(x_full + 8 * i, 1); mbar_init(x_empty + 8 * i, 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(d_full + 8 * i, 1); mbar_init(d_empty + 8 * i, 4); }
        for (int i = 0; i < kTsMaxWStages; ++i) { mbar_init(w_full + 8 * i, 1); mbar_init(w_empty + 8 * i, 4 * kHalves); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)),
                     "r"(kTsTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    __syncthreads();  // barriers initialised: the weight producer may start

    const int quarter = warp & 3;          // the 32 tensor-memory lanes this warp may access
    const int total_slots = n_units * RB;

    // Rest of the prologue, run by every warp inside its own role's branch: the byte -> half2
    // table (even column = high nibble in the low half), one copy per bank - the codebook is a
    // constant, so this runs before the dependency wait - then the wait, then the CTA barrier
    // that publishes the table and the tensor-memory base.
    auto finish_prologue = [&]() -> uint32_t {
        const float cv = p.code[lane & 15];
        const uint32_t ch = (uint32_t)__half_as_ushort(__float2half_rn(cv));
        for (int e = warp; e < 256; e += kTsThreads / 32) {
            const uint32_t v = __shfl_sync(0xffffffffu, ch, e >> 4) | (__shfl_sync(0xffffffffu, ch, e & 15) << 16);
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(lut_addr + (uint32_t)e * (kLut256 ? 256 : 128) + lane * 4), "r"(v) : "memory");
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
        // issues the MMAs and the commits.  Descriptors (K-major, 128-byte swizzle): the high word
        // is constant (8-token groups 1024 bytes apart, version 1, layout type 2), the low word is the
        // start address; 16 columns further along K is 32 bytes further inside the 128-byte row.
        tmem = finish_prologue();
        constexpr uint32_t idesc = make_idesc(N_TILE);
        constexpr uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);
        Ring ra, rx, rd;
        TsCursor cur;
        cur.init(L, u_begin, n_units);
        bool ok = true;
        for (int u = 0; ok && u < n_units; ++u, cur.next(L)) {
            const bool seg_first = cur.seg_first, seg_last = cur.seg_last();
            TS_PROF_BEGIN
            if (seg_first) ok = mbar_wait(d_empty + 8 * rd.idx, rd.phase ^ 1, abort_flag, p.status, 3);
            TS_PROF_END(0)
            TS_PROF_BEGIN
            ok = ok && mbar_wait(x_full + 8 * rx.idx, rx.phase, abort_flag, p.status, 4);
            ok = __all_sync(0xffffffffu, ok) != 0;
            TS_PROF_END(1)
            if (!ok) break;
            const uint32_t desc_lo0 = ((xring + (uint32_t)rx.idx * kXStageBytes) & 0x3FFFFu) >> 4;
            const uint32_t dbase = tmem + (uint32_t)(rd.idx * p.acc_cols);
            for (int rb = 0; rb < RB; ++rb) {
                TS_PROF_BEGIN
                ok = mbar_wait_warp(a_full + 8 * ra.idx, ra.phase, abort_flag, p.status, 5);
                TS_PROF_END(2)
                if (!ok) break;
                tc_fence_after();
                TS_PROF_BEGIN
                if (elect_one_sync()) {
                    const uint32_t abase = tmem + (uint32_t)p.a_base + (uint32_t)ra.idx * kSlotCols;
#pragma unroll
#ifdef TS_ABL_NOMMA  // timing experiment: commits only
                    for (int mm = 0; mm < 0; ++mm) {
#else
                    for (int mm = 0; mm < 2 * STEPS; ++mm) {  // columns 16 mm .. 16 mm + 15 of the slot: 64-column tile mm/4
#endif
                        const uint64_t bdesc = ((uint64_t)desc_hi << 32) | (uint64_t)(desc_lo0 + (mm >> 2) * (kXTileBytes >> 4) + (mm & 3) * 2);
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
            rx.advance(kXS);
            if (seg_last) rd.advance(2);
        }
    } else if (warp == 1 || warp == 3) {
        // ------------------------------------------------------------------ no role after the prologue
        tmem = finish_prologue();
    } else if (warp == 2) {
        // ------------------------------------------------------------------ copy producer
        // One elected lane of the converged warp issues every TMA copy of the CTA: per slot the
        // packed weights (16 row groups x kChunkK 32-bit words; one 3-D box, or one 2-D box per
        // step) into the weight ring, and per unit kChunkK/64 boxes of x (tile_tok tokens x 64
        // columns, L2 resident; tokens past n and columns past k zero-filled) into the activation
        // ring, released by the MMAs' commit.  The weights are constants:
        // the first ring-full of their copies is issued before the dependency wait (and before
        // this warp joins the rest of the prologue); x may come from the kernel before this one.
        Ring rw, rn;
        int sl = 0, w_rb = 0, xu = 0;
        TsCursor wc, xc;
        wc.init(L, u_begin, n_units);
        xc.init(L, u_begin, n_units);
        bool ok = true;
        auto issue_x = [&](bool blocking) {
            // as many activation copies as have a free stage (all the outstanding ones if `blocking`)
            while (ok && xu < n_units) {
                if (blocking) ok = mbar_wait_warp(x_empty + 8 * rn.idx, rn.phase ^ 1, abort_flag, p.status, 9);
                else if (!(__all_sync(0xffffffffu, mbar_test_wait(x_empty + 8 * rn.idx, rn.phase ^ 1)) != 0)) break;
                if (!ok) break;
                if (elect_one_sync()) {
                    mbar_expect_tx(x_full + 8 * rn.idx, kXStageBytes);
#pragma unroll
                    for (int t = 0; t < kXTiles; ++t)
                        tma_load_2d(xring + (uint32_t)rn.idx * kXStageBytes + (uint32_t)t * kXTileBytes, &L.g[xc.g].map_x,
                                    xc.chunk * kChunkK + 64 * t, p.tok0, x_full + 8 * rn.idx);
                }
                __syncwarp();
                rn.advance(kXS);
                ++xu;
                xc.next(L);
            }
        };
        auto issue_w_until = [&](int end, bool with_x) {
            for (; ok && sl < end; ++sl) {
                if (with_x) issue_x(false);
                TS_PROF_BEGIN
                ok = mbar_wait_warp(w_empty + 8 * rw.idx, rw.phase ^ 1, abort_flag, p.status, 1);
                TS_PROF_END(0)
                if (!ok) break;
                if (elect_one_sync()) {
                    const TsGemm &G = L.g[wc.g];
                    mbar_expect_tx(w_full + 8 * rw.idx, kSlotBytes);
                    if (WMODE == 1) {
                        tma_load_5d(w_stage(rw.idx), &G.map_q, 0, 0, 0, wc.chunk * (STEPS / 2), (wc.tile * RB + w_rb) * 4, w_full + 8 * rw.idx);
                    } else if (G.q3d) {
                        tma_load_3d(w_stage(rw.idx), &G.map_q, 0, (wc.tile * RB + w_rb) * 16, wc.chunk * STEPS, w_full + 8 * rw.idx);
                    } else {
#pragma unroll
                        for (int st = 0; st < STEPS; ++st)
                            tma_load_2d(w_stage(rw.idx) + (uint32_t)st * kStepBytes, &G.map_q, wc.chunk * kChunkK + 32 * st,
                                        (wc.tile * RB + w_rb) * 16, w_full + 8 * rw.idx);
                    }
                }
                __syncwarp();
                rw.advance(WS);
                if (++w_rb == RB) {
                    w_rb = 0;
                    wc.next(L);
                }
            }
        };
        issue_w_until(min(WS, total_slots), false);
        tmem = finish_prologue();
        issue_w_until(total_slots, true);
        issue_x(true);
    } else if (warp < kTsDequantWarp0) {
        // ------------------------------------------------------------------ epilogue
        tmem = finish_prologue();
        // the row this thread's lane holds
        const int row_in_block = WMODE == 1 ? 32 * quarter + lane : 8 * lane_row_group(quarter, lane) + (lane & 7);
        const int tmem_lane = 32 * quarter + lane;
        const size_t slot_floats = (size_t)RB * kBlockRows * N_TILE;
        // exchange launches: where this launch's slabs start (the counter is read after the dependency wait)
        long long region = 0;
        if (p.n_peers > 0) region = p.region0 + (long long)((__ldcg(p.epoch) + 1u) & 1u) * p.region_bytes;
        // 16 tokens (one accumulator piece) of one finished row, scaled: to o, or to every rank's slab
        auto store_row = [&](const TsGemm &G, int row, int piece, const float (&v)[16], float sc) {
            if (p.n_peers > 0 && G.slab_off >= 0) {
                uint32_t h[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const __half2 t = __floats2half2_rn(v[2 * i] * sc, v[2 * i + 1] * sc);
                    h[i] = *reinterpret_cast<const uint32_t *>(&t);
                }
                const long long off = region + G.slab_off + ((long long)row * N_TILE + piece * 16) * 2;
                for (int pr = 0; pr < p.n_peers; ++pr) {
                    uint4 *dst = reinterpret_cast<uint4 *>(p.peer[pr] + off);
                    dst[0] = make_uint4(h[0], h[1], h[2], h[3]);
                    dst[1] = make_uint4(h[4], h[5], h[6], h[7]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int tok = p.tok0 + piece * 16 + i;
                    if (tok < G.n) G.o[(size_t)tok * G.m + row] = __float2half_rn(v[i] * sc);
                }
            }
        };
        Ring rd;
        TsCursor cur;
        cur.init(L, u_begin, n_units);
        int u = 0;
        while (u < n_units) {
            // the segment: chunks [c0, c1) of tile `tile` of GEMM `cur.g`
            const TsGemm &G = L.g[cur.g];
            const int tile = cur.tile, c0 = cur.chunk;
            const int c1 = min(G.chunks, c0 + cur.left);
            const bool full = (c0 == 0 && c1 == G.chunks);
            TS_PROF_BEGIN
            if (!mbar_wait_warp(d_full + 8 * rd.idx, rd.phase, abort_flag, p.status, 6)) break;
            TS_PROF_END(0)
            tc_fence_after();
            TS_PROF_BEGIN
            float *my_partial = p.partials + (size_t)(2 * cta + (c0 == 0 ? 1 : 0)) * slot_floats;
            for (int rb = 0; rb < RB; ++rb) {
                const int row = (tile * RB + rb) * kBlockRows + row_in_block;
                const float sc = (full && row < G.m) ? G.absmax[row] : 0.f;
#pragma unroll 1
                for (int piece = 0; piece < N_TILE / 16; ++piece) {
                    float v[16];
                    tc_ld_x16(tmem + ((uint32_t)(32 * quarter) << 16) + (uint32_t)(rd.idx * p.acc_cols) + (uint32_t)rb * N_TILE + piece * 16, v);
                    if (full) {
                        if (row < G.m) store_row(G, row, piece, v, sc);
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
                const int cta_first = ts_cta_of_unit(p, G.unit0 + tile * G.chunks);
                const int cta_last = ts_cta_of_unit(p, G.unit0 + (tile + 1) * G.chunks - 1);
                const int nseg = cta_last - cta_first + 1;
                unsigned int *counter = p.counters + (size_t)(G.tile0 + tile) * 4 + quarter;
                unsigned int old = 0;
                if (lane == 0) old = atomicAdd(counter, 1u);
                old = __shfl_sync(0xffffffffu, old, 0);
                if (old == (unsigned)nseg - 1) {
                    if (lane == 0) *counter = 0;  // leave the counter clean for the next call
                    __threadfence();
                    for (int rb = 0; rb < RB; ++rb) {
                        const int row = (tile * RB + rb) * kBlockRows + row_in_block;
                        if (row >= G.m) continue;
                        const float sc = G.absmax[row];
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
                            store_row(G, row, piece, acc, sc);
                        }
                    }
                }
            }
            TS_PROF_END(1)
            for (int i = c0; i < c1; ++i) cur.next(L);
            u += c1 - c0;
            rd.advance(2);
        }
    } else {
        // ------------------------------------------------------------------ dequant
        // A group (4 * kHalves warps: one per 32-lane quarter and per four steps of a slot) converts
        // the slots j, j + kGroups, ... of this CTA: one wait / fence / arrival per slot and warp.
        // The groups work on different slots at once, so the latency of a slot's chain (shared
        // loads -> lookups -> tcgen05.st -> wait::st -> arrive) is overlapped kGroups times.
        const int dq = warp - kTsDequantWarp0;
        const int half = (dq >> 2) % kHalves;      // which four steps of the slot
        const int group = dq / (4 * kHalves);
        tmem = finish_prologue();
        const uint32_t lane_key = lut_addr + (uint32_t)(lane * 4);  // this lane's copy of the table (kLut256: also the prmt's second operand)
        const uint32_t a_lane0 = tmem + ((uint32_t)(32 * quarter) << 16) + (uint32_t)p.a_base + 64u * (uint32_t)half;
        // This thread's row inside a stage: word r%4 of 16-byte chunk 2 kt + r/4 of the 128-byte row
        // of (row group, step), the chunk index XORed with (index of that 128-byte row in the stage) % 8.
        //   WMODE 0: row index = 16 step + row group: offsets lane_soff[kt] + step * 2048;
        //   WMODE 1: row index = ((quarter * STEPS/2 + step/2) * 4 + l/8) * 2 + step%2, whose low three
        //            bits are 2 (l/8) + step%2: an odd step flips bit 0 of the chunk index (^ 16 bytes).
        const int r = lane & 7;
        const int rg = WMODE == 1 ? (lane >> 3) : lane_row_group(quarter, lane);
        const uint32_t row0 = WMODE == 1 ? (uint32_t)((quarter * (STEPS / 2) + 2 * half) * 8 + 2 * rg) : (uint32_t)(64 * half + rg);
        const uint32_t xor0 = WMODE == 1 ? (uint32_t)(2 * rg) : (uint32_t)(rg & 7);
        uint32_t lane_soff[4];
#pragma unroll
        for (int kt = 0; kt < 4; ++kt)
            lane_soff[kt] = row0 * 128u + (((uint32_t)(2 * kt + (r >> 2)) ^ xor0) << 4) + (uint32_t)(r & 3) * 4u;
        auto w_addr = [&](uint32_t stage, int st, int kt) -> uint32_t {
            if (WMODE == 1) return stage + (lane_soff[kt] ^ ((st & 1) ? 16u : 0u)) + (uint32_t)((st >> 1) * 1024 + (st & 1) * 128);
            return stage + lane_soff[kt] + (uint32_t)st * kStepBytes;
        };
        const int A = p.a_slots;
        int a_idx = group % A, w_idx = group % WS;  // ring positions of slot `sl`: sl % A, sl % WS
        uint32_t a_phase = (uint32_t)(group / A) & 1u, w_phase = (uint32_t)(group / WS) & 1u;
        bool ok = true;
#ifdef TUNA_TS_PROFILE
        const long long loop_c0 = clock64();
#endif
        for (int sl = group; ok && sl < total_slots; sl += kGroups) {
            TS_PROF_BEGIN
            ok = mbar_wait_warp(w_full + 8 * w_idx, w_phase, abort_flag, p.status, 8);
            TS_PROF_END(3)
            if (!ok) break;
            uint32_t wv[4][4];  // [step][tile]: the row's 8 columns of that tile
            {
                const uint32_t src = w_stage(w_idx);
#pragma unroll
                for (int st = 0; st < 4; ++st)
#pragma unroll
                    for (int kt = 0; kt < 4; ++kt)
#ifdef TS_ABL_LDS4  // timing experiment: a quarter of the weight loads
                        if (kt > 0) wv[st][kt] = wv[st][0] + kt; else
#endif
                        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(wv[st][kt]) : "r"(w_addr(src, st, kt)));
            }
            // software pipeline: the 16 lookups of step st + 1 are in flight while step st is stored
            uint32_t v[2][16];
            auto lookups = [&](const uint32_t (&w)[4], uint32_t (&o)[16]) {
#pragma unroll
                for (int kt = 0; kt < 4; ++kt) {  // byte c of word kt = column pair c of tile kt
#ifdef TS_ABL_NOLUT  // timing experiment: no table lookups
                    o[4 * kt] = w[kt]; o[4 * kt + 1] = w[kt] + lane_key; o[4 * kt + 2] = w[kt] ^ lane_key; o[4 * kt + 3] = w[kt] >> 1;
#else
                    if (kLut256) {
                        o[4 * kt] = ts_lookup256(w[kt], lane_key, 0x7604);
                        o[4 * kt + 1] = ts_lookup256(w[kt], lane_key, 0x7614);
                        o[4 * kt + 2] = ts_lookup256(w[kt], lane_key, 0x7624);
                        o[4 * kt + 3] = ts_lookup256(w[kt], lane_key, 0x7634);
                    } else {
                        o[4 * kt] = ts_lookup(w[kt], lane_key, 0x4440);
                        o[4 * kt + 1] = ts_lookup(w[kt], lane_key, 0x4441);
                        o[4 * kt + 2] = ts_lookup(w[kt], lane_key, 0x4442);
                        o[4 * kt + 3] = ts_lookup(w[kt], lane_key, 0x4443);
                    }
#endif
                }
            };
            lookups(wv[0], v[0]);
            // All sixteen shared loads of the stage have been issued and the first have returned
            // (their data fed the lookups; they return in order): hand the stage back to the
            // producer.  The arrival is a release: it is ordered after this warp's loads.
            __syncwarp();
            if (lane == 0) mbar_arrive(w_empty + 8 * w_idx);
            TS_PROF_BEGIN
            ok = mbar_wait_warp(a_empty + 8 * a_idx, a_phase ^ 1, abort_flag, p.status, 7);
            TS_PROF_END(0)
            if (!ok) break;
            tc_fence_after();
            TS_PROF_BEGIN
            const uint32_t ta = a_lane0 + (uint32_t)a_idx * kSlotCols;
#pragma unroll
            for (int st = 0; st < 4; ++st) {
                if (st < 3) lookups(wv[st + 1], v[(st + 1) & 1]);
                uint32_t (&c)[16] = v[st & 1];
#ifdef TS_ABL_NOST  // timing experiment: keep the lookups alive, skip the stores
                asm volatile("" ::"r"(c[0] ^ c[1] ^ c[2] ^ c[3] ^ c[4] ^ c[5] ^ c[6] ^ c[7] ^ c[8] ^ c[9] ^ c[10] ^ c[11] ^ c[12] ^ c[13] ^ c[14] ^ c[15]), "r"(ta));
#else
                tc_st_x16(ta + 16u * st, c);  // columns 16 st .. + 15 of this warp's half slot = the step's 32 columns of K
#endif
            }
            TS_PROF_END(1)
            TS_PROF_BEGIN
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            TS_PROF_END(2)
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(a_full + 8 * a_idx);
            a_idx += kGroups;
            while (a_idx >= A) { a_idx -= A; a_phase ^= 1u; }
            w_idx += kGroups;
            while (w_idx >= WS) { w_idx -= WS; w_phase ^= 1u; }
        }
#ifdef TUNA_TS_PROFILE
        pg_[3] = clock64() - loop_c0;
#endif
    }

    // ------------------------------------------------------------------ common exit
    TS_PROF_MARK(2)
    tc_fence_before();
    __syncthreads();
    if (warp < kTsDequantWarp0) { TS_PROF_MARK(3) }
    TS_PROF_STORE
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTsTmemCols) : "memory");
    }
}

// ------------------------------------------------------------------ host side

// Columns of a slot: 256 (16 MMAs per wait and commit of the issuing warp) when the matrix is
// large enough for 16-KB units to balance across the SMs, else 128.
static int ts_steps(const tuna_config &c) { return c.k_steps == 4 ? 4 : 8; }

int gemm_tstream_normalize_config(int m, int n, int k, int sm_count, tuna_config *c)
{
    if (c->tile_tok == 0) c->tile_tok = (n <= 16) ? 16 : (n <= 32 ? 32 : (n <= 64 ? 64 : 128));
    if (c->tile_tok != 16 && c->tile_tok != 32 && c->tile_tok != 64 && c->tile_tok != 128) return TUNA_ERR_BAD_CONFIG;
    if (c->tile_tok == 128) {
        // 128-token tiles (token counts above 64 run as passes of 128): the tensor pipe needs 64 clocks
        // per MMA there, as long as the dequantisation of 16 columns, so a slot is 128 columns (8 MMAs per
        // wait and commit are enough) and a tile one row block (the accumulators take 2 x 128 columns)
        if (c->row_blocks == 0) c->row_blocks = 1;
        if (c->k_steps == 0) c->k_steps = 4;
        if (c->row_blocks != 1 || c->k_steps != 4) return TUNA_ERR_BAD_CONFIG;
    }
    // two row blocks share an activation stage when the matrix is tall enough for 32-KB units to balance
    if (c->row_blocks == 0) c->row_blocks = (m >= 8192 && c->tile_tok <= 32) ? 2 : 1;
    if ((c->row_blocks != 1 && c->row_blocks != 2 && c->row_blocks != 4) || (c->tile_tok <= 64 && c->row_blocks * c->tile_tok > 64))
        return TUNA_ERR_BAD_CONFIG;
    if (c->ctas < 0) return TUNA_ERR_BAD_CONFIG;
    if (c->ctas == 0 || c->ctas > sm_count) c->ctas = sm_count;
    if (c->k_steps == 0) {
        // 256-column slots unless they leave fewer than ~12 units per CTA to balance with
        const long long units256 = (long long)div_up(m, kBlockRows * c->row_blocks) * div_up(k, 256);
        c->k_steps = units256 >= 12ll * c->ctas ? 8 : 4;
    }
    if (c->k_steps != 4 && c->k_steps != 8) return TUNA_ERR_BAD_CONFIG;
    return TUNA_OK;
}

size_t gemm_tstream_workspace_bytes(int m, int n, int k, const tuna_config &c, int sm_count)
{
    (void)n; (void)k;
    const size_t tiles = (size_t)div_up(m, kBlockRows * c.row_blocks);
    const size_t counters = (tiles * 16 + 255) / 256 * 256;  // one counter per tile and 32-row quarter
    return partial_region_bytes(sm_count) + counters;
}

template <int N_TILE, int STEPS, int MAXG, int WMODE>
static int launch_ts(const TsLaunch<MAXG> &L, int ctas, cudaStream_t stream)
{
    static bool attr_set[64] = {false};  // one-time, per device, opt-in to large dynamic shared memory
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return TUNA_ERR_NO_DEVICE;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!attr_set[dev]) {
            if (cudaFuncSetAttribute(gemm_w4a16_tstream_kernel<N_TILE, STEPS, MAXG, WMODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     kTsSmemDynamic) != cudaSuccess)
                return TUNA_ERR_NO_DEVICE;
            // The kernel places its lookup table at shared address 0x10000 and what lies below it right
            // after the start of dynamic shared memory, which must therefore begin within the first 4 KB
            // (static shared memory of the kernel + what the system reserves per block; the kernel checks too).
            cudaFuncAttributes fa;
            int reserved = 0;
            if (cudaFuncGetAttributes(&fa, gemm_w4a16_tstream_kernel<N_TILE, STEPS, MAXG, WMODE>) != cudaSuccess ||
                cudaDeviceGetAttribute(&reserved, cudaDevAttrReservedSharedMemoryPerBlock, dev) != cudaSuccess)
                return TUNA_ERR_NO_DEVICE;
            if ((fa.sharedSizeBytes + (size_t)reserved + 1023) / 1024 * 1024 > 4096) return TUNA_ERR_NO_DEVICE;
            attr_set[dev] = true;
        }
    }
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3((unsigned)ctas);
    lc.blockDim = dim3(kTsThreads);
    lc.dynamicSmemBytes = kTsSmemDynamic;
    lc.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = attr;
    lc.numAttrs = 1;
    return cudaLaunchKernelEx(&lc, gemm_w4a16_tstream_kernel<N_TILE, STEPS, MAXG, WMODE>, L) == cudaSuccess ? TUNA_OK : TUNA_ERR_LAUNCH;
}

template <int MAXG>
static int launch_ts_dispatch(const TsLaunch<MAXG> &L, int tile_tok, int steps, int ctas, cudaStream_t stream)
{
    switch (tile_tok * 100 + steps * 10 + L.c.w_mode) {
        case 1640: return launch_ts<16, 4, MAXG, 0>(L, ctas, stream);
        case 1641: return launch_ts<16, 4, MAXG, 1>(L, ctas, stream);
        case 1680: return launch_ts<16, 8, MAXG, 0>(L, ctas, stream);
        case 1681: return launch_ts<16, 8, MAXG, 1>(L, ctas, stream);
        case 3240: return launch_ts<32, 4, MAXG, 0>(L, ctas, stream);
        case 3241: return launch_ts<32, 4, MAXG, 1>(L, ctas, stream);
        case 3280: return launch_ts<32, 8, MAXG, 0>(L, ctas, stream);
        case 3281: return launch_ts<32, 8, MAXG, 1>(L, ctas, stream);
        case 6440: return launch_ts<64, 4, MAXG, 0>(L, ctas, stream);
        case 6441: return launch_ts<64, 4, MAXG, 1>(L, ctas, stream);
        case 6480: return launch_ts<64, 8, MAXG, 0>(L, ctas, stream);
        case 6481: return launch_ts<64, 8, MAXG, 1>(L, ctas, stream);
        case 12840: return launch_ts<128, 4, MAXG, 0>(L, ctas, stream);
        case 12841: return launch_ts<128, 4, MAXG, 1>(L, ctas, stream);
        default: return TUNA_ERR_BAD_CONFIG;
    }
}

// Fills the table entry of one GEMM (tensor maps, geometry); `unit0` / `tile0` are where its units
// and tiles start in the launch.  Returns its unit count, or a negative status.
static bool ts_wmode1_shape(int m, int k) { return m % 32 == 0 && k % 64 == 0; }

static long long ts_fill_gemm(TsGemm *g, const void *q, const void *x, const float *absmax, void *o, int m, int n, int k,
                              int row_blocks, int steps, int tile_tok, int unit0, int tile0, int w_mode)
{
    const int chunk_k = 32 * steps;
    std::memset(g, 0, sizeof(*g));
    g->absmax = absmax; g->o = (__half *)o;
    g->m = m; g->n = n; g->k = k;
    g->chunks = div_up(k, chunk_k);
    g->row_tiles = div_up(m, kBlockRows * row_blocks);
    g->unit0 = unit0;
    g->tile0 = tile0;
    // Packed weights (a row group is 4k bytes = k 32-bit words; word index = column index).  One
    // step of a slot is a box of 16 row groups x 32 words (128 bytes), 128-byte swizzled.  Where k
    // is a multiple of 32 the matrix also has the 3-D view [k/32 steps][m/8 row groups][32 words]
    // (strides 128 bytes and 4k bytes) and a slot is one box of `steps` x 16 x 32; otherwise, or if
    // the driver refuses that view, the 2-D view and one box per step.  Rows, columns and steps
    // past the matrix are zero-filled by the copy.
    // w_mode 1: 32-row blocks x pairs of steps, [m/32][k/64][4 row groups][2 steps][32 words] with
    // strides 16k, 256, 4k and 128 bytes; a slot is one box of 4 x steps/2 x 4 x 2 x 32 words.
    g->q3d = 0;
    if (w_mode == 1) {
        const uint64_t dims[5] = {32, 2, 4, (uint64_t)k / 64, (uint64_t)m / 32};
        const uint64_t strides[4] = {128, (uint64_t)k * 4, 256, (uint64_t)k * 16};
        const uint32_t box[5] = {32, 2, 4, (uint32_t)steps / 2, 4};
        if (!ts_wmode1_shape(m, k) || !make_tensor_map_nd(&g->map_q, CU_TENSOR_MAP_DATA_TYPE_UINT32, q, 5, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
            return TUNA_ERR_BAD_CONFIG;
    } else
#ifdef TS_FORCE_Q2D  // timing experiment: one 2-D box per step even where the 3-D view exists
    if (false &&
#else
    if (k % 32 == 0 &&
#endif
        make_tensor_map_3d(&g->map_q, CU_TENSOR_MAP_DATA_TYPE_UINT32, q, 32, (uint64_t)m / 8, (uint64_t)k / 32, (uint64_t)k * 4, 128,
                           32, 16, (uint32_t)steps, CU_TENSOR_MAP_SWIZZLE_128B))
        g->q3d = 1;
    else if (!make_tensor_map_2d(&g->map_q, CU_TENSOR_MAP_DATA_TYPE_UINT32, q, (uint64_t)k, (uint64_t)m / 8, (uint64_t)k * 4, 32, 16,
                                 CU_TENSOR_MAP_SWIZZLE_128B))
        return TUNA_ERR_NO_DEVICE;
    // activations as [n tokens] x [k] fp16; box = tile_tok tokens x 64 columns (128-byte rows, swizzled)
    if (!make_tensor_map_2d(&g->map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, x, (uint64_t)k, (uint64_t)n, (uint64_t)k * 2, 64,
                            (uint32_t)tile_tok, CU_TENSOR_MAP_SWIZZLE_128B))
        return TUNA_ERR_NO_DEVICE;
    return (long long)g->row_tiles * g->chunks;
}

static void ts_fill_common(TsParams *p, const tuna_config &c, int steps, void *workspace, int sm_count)
{
    p->row_blocks = c.row_blocks;
    p->acc_cols = c.row_blocks * c.tile_tok < 32 ? 32 : c.row_blocks * c.tile_tok;  // 32-column allocation granule
    p->a_base = 2 * p->acc_cols;
    p->a_slots = (kTsTmemCols - p->a_base) / (16 * steps);
    if (p->a_slots > kTsMaxASlots) p->a_slots = kTsMaxASlots;
    p->partials = (float *)workspace;
    p->counters = (unsigned int *)((uint8_t *)workspace + partial_region_bytes(sm_count));
}

int launch_gemm_tstream(const GemmArgs &a, const tuna_config &c)
{
    const int steps = ts_steps(c);
    TsLaunch<1> L;
    std::memset(&L.c, 0, sizeof(L.c));
    L.c.code = a.code;
    L.c.count = 1;
    L.c.status = device_status_word();
    if (!L.c.status) return TUNA_ERR_NO_DEVICE;
    if (a.workspace == nullptr || a.workspace_bytes < gemm_tstream_workspace_bytes(a.m, a.n, a.k, c, a.sm_count))
        return TUNA_ERR_WORKSPACE;
    ts_fill_common(&L.c, c, steps, a.workspace, a.sm_count);
    L.c.w_mode = ts_wmode1_shape(a.m, a.k) ? 1 : 0;
    long long units = ts_fill_gemm(&L.g[0], a.q, a.x, a.absmax, a.o, a.m, a.n, a.k, c.row_blocks, steps, c.tile_tok, 0, 0, L.c.w_mode);
    if (units == TUNA_ERR_BAD_CONFIG && L.c.w_mode == 1) {  // the driver refused the 5-D view
        L.c.w_mode = 0;
        units = ts_fill_gemm(&L.g[0], a.q, a.x, a.absmax, a.o, a.m, a.n, a.k, c.row_blocks, steps, c.tile_tok, 0, 0, 0);
    }
    if (units < 0) return (int)units;
    if (units >= (1ll << 30)) return TUNA_ERR_TOO_LARGE;
    L.c.units = (int)units;
    int ctas = c.ctas;
    if (ctas > L.c.units) ctas = L.c.units;
    L.c.units_q = L.c.units / ctas;
    L.c.units_r = L.c.units % ctas;
    for (int tok0 = 0; tok0 < a.n; tok0 += c.tile_tok) {
        L.c.tok0 = tok0;
        const int st = launch_ts_dispatch(L, c.tile_tok, steps, ctas, a.stream);
        if (st != TUNA_OK) return st;
    }
    return TUNA_OK;
}

// ---- a sequence of independent GEMMs in one persistent launch

size_t gemm_tstream_sequence_workspace_bytes(const tuna_gemm_desc *d, int count, int sm_count)
{
    size_t tiles = 0;  // an upper bound: one 128-row block per tile
    for (int i = 0; i < count; ++i) tiles += (size_t)div_up(d[i].m, kBlockRows);
    return partial_region_bytes(sm_count) + (tiles * 16 + 255) / 256 * 256;
}

// Whether the sequence kernel can take these GEMMs (token counts of one pass; the rest is checked by the caller).
bool gemm_tstream_sequence_supported(const tuna_gemm_desc *d, int count)
{
    if (count < 1) return false;
    for (int i = 0; i < count; ++i)
        if (d[i].n > 64) return false;
    return true;
}

int launch_gemm_tstream_sequence(const tuna_gemm_desc *d, int count, const float *code, void *workspace, size_t workspace_bytes,
                                 int sm_count, cudaStream_t stream, const tuna_exchange *ex)
{
    if (workspace == nullptr || workspace_bytes < gemm_tstream_sequence_workspace_bytes(d, count, sm_count)) return TUNA_ERR_WORKSPACE;
    DeviceStatus *status = device_status_word();
    if (!status) return TUNA_ERR_NO_DEVICE;
    int tile0 = 0;  // tiles of the GEMMs launched so far: every launch has its own counters
    for (int first = 0; first < count; first += kTsMaxSeq) {
        const int cnt = count - first < kTsMaxSeq ? count - first : kTsMaxSeq;
        int max_n = 1;
        for (int i = 0; i < cnt; ++i) max_n = d[first + i].n > max_n ? d[first + i].n : max_n;
        tuna_config c;
        std::memset(&c, 0, sizeof(c));
        c.path = TUNA_PATH_TSTREAM;
        c.tile_tok = max_n <= 16 ? 16 : (max_n <= 32 ? 32 : 64);
        // as many row blocks per tile as the accumulator columns allow: they share one activation stage
        // (measured on the Mistral MLP sweep: 3.53 / 4.00 / 4.27 TB/s with 1 / 2 / 4 row blocks); the
        // sequence as a whole is still balanced at unit granularity (64 KB)
        c.row_blocks = 64 / c.tile_tok;
        c.k_steps = 8;
        c.ctas = sm_count;
        static thread_local TsLaunch<kTsMaxSeq> L;  // ~20 KB: not on the stack
        std::memset(&L.c, 0, sizeof(L.c));
        L.c.code = code;
        L.c.count = cnt;
        L.c.status = status;
        ts_fill_common(&L.c, c, 8, workspace, sm_count);
        long long slab0[kTsMaxSeq];  // exchange launches: rank 0's slab of each GEMM inside a parity region
        long long region_bytes = 0;
        if (ex) {
            region_bytes = (long long)((ex->bytes - kExHeaderBytes) / 2 / 256 * 256);
            L.c.n_peers = ex->world;
            for (int j = 0; j < ex->world; ++j) L.c.peer[j] = (unsigned char *)ex->buffer[j];
            L.c.epoch = (const unsigned int *)ex->buffer[ex->rank];
            L.c.region0 = kExHeaderBytes;
            L.c.region_bytes = region_bytes;
            long long off = 0;
            for (int i = 0; i < cnt; ++i) {
                slab0[i] = -1;
                if (!(d[first + i].flags & TUNA_GEMM_PARTIAL)) continue;
                slab0[i] = off;
                off += (long long)ex->world * d[first + i].m * c.tile_tok * 2;
            }
            if (off > region_bytes) return TUNA_ERR_WORKSPACE;
        }
        // one stage layout per launch: the 256-byte-run one if every GEMM has it
        L.c.w_mode = 1;
        for (int i = 0; i < cnt; ++i)
            if (!ts_wmode1_shape(d[first + i].m, d[first + i].k)) L.c.w_mode = 0;
        long long units = 0;
        const int tile0_launch = tile0;
        for (int attempt = 0; attempt < 2; ++attempt) {
            units = 0;
            tile0 = tile0_launch;
            bool refused = false;
            for (int i = 0; i < cnt; ++i) {
                const tuna_gemm_desc &g = d[first + i];
                const long long u = ts_fill_gemm(&L.g[i], g.q, g.x, (const float *)g.absmax, g.o, g.m, g.n, g.k, c.row_blocks, 8, c.tile_tok,
                                                 (int)units, tile0, L.c.w_mode);
                if (u == TUNA_ERR_BAD_CONFIG && L.c.w_mode == 1) { refused = true; break; }  // the driver refused the 5-D view
                if (u < 0) return (int)u;
                if (ex) L.g[i].slab_off = slab0[i] < 0 ? -1 : slab0[i] + (long long)ex->rank * g.m * c.tile_tok * 2;
                units += u;
                tile0 += L.g[i].row_tiles;
                if (units >= (1ll << 30)) return TUNA_ERR_TOO_LARGE;
            }
            if (!refused) break;
            L.c.w_mode = 0;
        }
        L.c.units = (int)units;
        int ctas = c.ctas;
        if (ctas > L.c.units) ctas = L.c.units;
        L.c.units_q = L.c.units / ctas;
        L.c.units_r = L.c.units % ctas;
        int st = launch_ts_dispatch(L, c.tile_tok, 8, ctas, stream);
        if (st == TUNA_OK && ex) st = launch_exchange_reduce(*ex, d + first, slab0, cnt, c.tile_tok, region_bytes, stream);
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
