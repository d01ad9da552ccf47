// Weight-streaming FP16 x 4-bit(codebook) GEMM for small token counts (n <= 32
// per pass) on sm_100a: the memory-bound regime every row of the reference's
// README table is measured in.  Counterpart of the reference's Tuna<> kernel and
// its Deq4GemmIterator main loop (kernel.cu:1043-2505, 2816-2960); it keeps the
// mma orientation (weights are the m16 "A" operand, tokens the n8 "B" operand,
// kernel.cu:2182-2192) and nothing else.
//
// Why mma.sync here and not tcgen05: on B200 a tcgen05.mma with M=128, K=16 takes
// ~128 clocks whatever N is, i.e. at most 16 weights per clock per SM, a third of
// what HBM delivers; mma.sync.m16n8k16 sustains ~990 MAC/clk/SM = 62 weights per
// clock at 16 tokens.  The tensor-memory kernel takes over for large token counts.
//
// Structure.  One persistent CTA per SM: warp 0 is a TMA producer, 16 consumer warps
// arranged warps_m x warps_k.  A "unit" is (row tile of 32*R*warps_m rows, K chunk of
// 32*S*warps_k columns).  Per unit the producer brings in, through an mbarrier ring,
//   * the packed weights: warps_k boxes of [4*R*warps_m row groups] x [128*S bytes] from the
//     [m/8] x [4k] byte view of q (one row group = 8 rows = 4k contiguous bytes, test.py:58-65);
//   * the activations: warps_k boxes of [tile_tok tokens] x [32*S columns] fp16.
// A consumer lane reads 16 packed bytes (half an 8x8 tile: 4 rows x 8 columns) with one
// 128-bit shared load; lane (g,t) takes row group g/2, rows 4(g%2)..+3, tile t of the four
// tiles of a 32-column step.  Each 32-bit word is 8 consecutive columns of one row and
// becomes the A fragments of two m16n8k16 (the k index of an mma is a label: slots 2t,2t+1
// <-> columns 0,1 of tile t, slots 2t+8,+9 <-> columns 2,3; the B fragment is the matching
// 16 contiguous bytes of x).  Rows 4g, 4g+1 feed accumulator tile P0, rows 4g+2, 4g+3 tile P1.
//
// Dequantisation: a byte holds two codes; a 256-entry byte -> half2(fp16(code[hi]),
// fp16(code[lo])) table is replicated once per bank (entry stride 256 bytes) at a
// 64-KB-aligned shared address, so that ONE prmt builds the whole address
// (0x10000*j | byte << 8 | lane*4) and every lookup is conflict free.  The per-row scale
// is constant along K (one block per row, test.py:81, kernel.cu:2178-2180) and is applied
// once, in fp32, to the accumulated sum.
//
// Split-K: units are numbered tile-major and cut into one contiguous range per CTA
// ("stream-K"), so every SM streams the same number of bytes.  Warps that share rows
// reduce through shared memory in a fixed tree; a tile cut across CTAs is finished by the
// CTA that arrives last at the tile's counter, which adds the fp32 partials from the
// workspace in unit order.  Results are bit-identical from run to run, the output needs no
// zero fill, and there are no floating-point atomics (the reference atomically adds fp16
// partials, kernel.cu:2739-2745).
//
// Every wait is bounded (see sm100_ptx.cuh): a wait that runs out records where, raises
// the CTA's abort flag and everybody unwinds to the common exit.
#include <cstring>
#include <mutex>
#include "common.cuh"
#include "launchers.h"
#include "sm100_ptx.cuh"

namespace tuna {

constexpr int kConsumerWarps = 16;
constexpr int kStreamThreads = 32 * (1 + kConsumerWarps);
constexpr int kLut64Bytes = 65536;           // 256 entries x 256-byte stride (32 lanes x 4 bytes used)
constexpr int kStreamSmemLimit = 227 * 1024 - 2048;  // dynamic request; static barriers take the rest
constexpr int S_MAX = 2;                     // 32-column steps per warp per unit, at most

struct StreamParams {
    const float *code;
    const float *absmax;
    __half *o;
    float *partials;
    unsigned int *counters;
    DeviceStatus *status;
    int m, n, k;
    int tok0;          // first token of this pass
    int warps_m, warps_k;
    int ksteps;        // S: 32-column steps per warp per unit
    int stages;
    int row_tiles, chunks;
    long long units;
    int stage_w_bytes, stage_x_bytes;
    int red_bytes;     // shared-memory scratch of the in-CTA reduction
};

__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                             uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t lut_lookup(uint32_t w, uint32_t lane_key, uint32_t selector)
{
    // result bytes: [0] = lane*4, [1] = the selected byte of w, [2..3] = upper address bytes
    uint32_t addr, v;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(addr) : "r"(w), "r"(lane_key), "r"(selector));
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

__device__ __forceinline__ uint4 lds128(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

template <int R, int NT>
__global__ void __launch_bounds__(kStreamThreads, 1)
gemm_stream_kernel(const StreamParams p, const __grid_constant__ CUtensorMap tmap_q,
                   const __grid_constant__ CUtensorMap tmap_x)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ __align__(8) uint64_t bars[40];
    __shared__ int s_abort;
    __shared__ int s_last;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cta = blockIdx.x, ctas = gridDim.x;
    const int WM = p.warps_m, WK = p.warps_k, S = p.ksteps;
    volatile int *abort_flag = &s_abort;

    // Shared-memory map: the table sits at the first 64-KB boundary; stage buffers fill the
    // space before it (if a whole stage fits) and after it; reduction scratch last.
    const uint32_t base = smem_u32(smem);
    const uint32_t lut_addr = (base + 0xFFFFu) & ~0xFFFFu;
    const uint32_t stage_bytes = (uint32_t)(p.stage_w_bytes + p.stage_x_bytes);
    uint32_t dyn_bytes;
    asm("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_bytes));
    const int stages_before = (int)((lut_addr - base) / stage_bytes);
    // the ring is as deep as asked for, or as deep as the space around the table allows
    const int room_after = (int)(((long long)base + dyn_bytes - (long long)lut_addr - kLut64Bytes - p.red_bytes) / (long long)stage_bytes);
    const int NS = min(p.stages, stages_before + max(room_after, 0));
    auto stage_addr = [&](int s) -> uint32_t {
        return s < stages_before ? base + (uint32_t)s * stage_bytes
                                 : lut_addr + kLut64Bytes + (uint32_t)(s - stages_before) * stage_bytes;
    };
    const int stages_after = NS > stages_before ? NS - stages_before : 0;
    const uint32_t red_addr = lut_addr + kLut64Bytes + (uint32_t)stages_after * stage_bytes;

    const uint32_t bar0 = smem_u32(&bars[0]);
    const uint32_t full = bar0, empty = bar0 + 8 * NS, sync_bar = bar0 + 16 * NS;

    if (NS < 2 || room_after < 0) {  // cannot happen with the launcher's request; never run without a ring
        if (threadIdx.x == 0 && atomicCAS(&p.status->code, 0, 20) == 0) p.status->detail = NS;
        return;
    }
    if (threadIdx.x == 0) {
        s_abort = 0;
        s_last = 0;
        for (int i = 0; i < NS; ++i) { mbar_init(full + 8 * i, 1); mbar_init(empty + 8 * i, kConsumerWarps); }
        mbar_init(sync_bar, kConsumerWarps);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // byte -> half2 table: even column = high nibble in the low half; 32 copies, one per bank
    for (int e = warp; e < 256; e += kStreamThreads / 32) {
        const __half hi = __float2half_rn(p.code[e >> 4]);
        const __half lo = __float2half_rn(p.code[e & 15]);
        const uint32_t v = (uint32_t)__half_as_ushort(hi) | ((uint32_t)__half_as_ushort(lo) << 16);
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(lut_addr + (uint32_t)e * 256 + lane * 4), "r"(v) : "memory");
    }
    __syncthreads();

    // this CTA's contiguous range of units
    long long u = (p.units * cta) / ctas;
    const long long u_end = (p.units * (cta + 1)) / ctas;
    int tile = (int)(u / p.chunks);
    int chunk = (int)(u - (long long)tile * p.chunks);
    PROF_ROLE_BEGIN();

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            Ring r;
            const int rg_per_tile = 4 * R * WM;
            for (; u < u_end; ++u, r.advance(NS)) {
                if (!mbar_wait(empty + 8 * r.idx, r.phase ^ 1, abort_flag, p.status, 1)) break;
                const uint32_t dst = stage_addr(r.idx);
                mbar_expect_tx(full + 8 * r.idx, stage_bytes);
                const int k0 = chunk * 32 * S * WK;  // first column of the unit
                for (int wk = 0; wk < WK; ++wk) {
                    // byte coordinate inside a row group: 4 bytes per column
                    tma_load_2d(dst + (uint32_t)wk * (uint32_t)(rg_per_tile * 128 * S), &tmap_q, (k0 + wk * 32 * S) * 4,
                                tile * rg_per_tile, full + 8 * r.idx);
                    tma_load_2d(dst + (uint32_t)p.stage_w_bytes + (uint32_t)wk * (uint32_t)(NT * 8 * 64 * S), &tmap_x,
                                k0 + wk * 32 * S, p.tok0, full + 8 * r.idx);
                }
                if (++chunk == p.chunks) { chunk = 0; ++tile; }
            }
        }
    } else {
        // ------------------------------------------------------------------ consumers
        const int cw = warp - 1;
        const int wm = cw % WM, wk = cw / WM;
        const int g = lane >> 2, t = lane & 3;
        const bool active = wk < WK;  // warps beyond warps_m * warps_k only take part in the barriers
        const uint32_t lane_key = (lut_addr & 0xFFFF0000u) | (uint32_t)(lane * 4);
        // offsets of this lane's 16 bytes inside a stage
        const uint32_t w_box_bytes = (uint32_t)(4 * R * WM * 128 * S);
        const uint32_t w_off = (uint32_t)wk * w_box_bytes + (uint32_t)(4 * wm * R + (g >> 1)) * (uint32_t)(128 * S) +
                               (uint32_t)t * 32 + (uint32_t)(g & 1) * 16;
        const uint32_t x_off = (uint32_t)p.stage_w_bytes + (uint32_t)wk * (uint32_t)(NT * 8 * 64 * S) +
                               (uint32_t)g * (uint32_t)(64 * S) + (uint32_t)t * 16;

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
        uint32_t sync_phase = 0;
        // bounded rendezvous of the 16 consumer warps
        auto consumers_sync = [&]() -> bool {
            __syncwarp();
            if (lane == 0) mbar_arrive(sync_bar);
            const bool ok = mbar_wait(sync_bar, sync_phase & 1, abort_flag, p.status, 3);
            ++sync_phase;
            return ok;
        };

        Ring r;
        bool ok = true;
        while (ok && u < u_end) {
            // ---- one segment: the units of one tile inside this CTA's range
            const int seg_tile = tile, c0 = chunk;
            const long long left = u_end - u;
            const int c1 = (int)((long long)(p.chunks - c0) <= left ? p.chunks : c0 + left);
            zero_acc();
            for (int c = c0; c < c1; ++c, r.advance(NS)) {
                if (!mbar_wait(full + 8 * r.idx, r.phase, abort_flag, p.status, 2)) { ok = false; break; }
                const uint32_t st = stage_addr(r.idx);
                uint4 wv[S_MAX][R];
                uint4 xv[S_MAX][NT];
#pragma unroll
                for (int s = 0; s < S_MAX; ++s) {
                    if (s < S && active) {
#pragma unroll
                        for (int rr = 0; rr < R; ++rr) wv[s][rr] = lds128(st + w_off + (uint32_t)rr * (uint32_t)(4 * 128 * S) + s * 128);
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) xv[s][nt] = lds128(st + x_off + (uint32_t)nt * (uint32_t)(8 * 64 * S) + s * 64);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty + 8 * r.idx);  // the stage is in registers
                if (active) {
#pragma unroll
                    for (int s = 0; s < S_MAX; ++s) {
                        if (s < S) {
#pragma unroll
                            for (int rr = 0; rr < R; ++rr) {
                                const uint32_t w[4] = {wv[s][rr].x, wv[s][rr].y, wv[s][rr].z, wv[s][rr].w};
#pragma unroll
                                for (int P = 0; P < 2; ++P) {
                                    const uint32_t wa = w[2 * P], wb = w[2 * P + 1];
                                    const uint32_t a0 = lut_lookup(wa, lane_key, 0x7604), a1 = lut_lookup(wb, lane_key, 0x7604);
                                    const uint32_t a2 = lut_lookup(wa, lane_key, 0x7614), a3 = lut_lookup(wb, lane_key, 0x7614);
                                    const uint32_t a4 = lut_lookup(wa, lane_key, 0x7624), a5 = lut_lookup(wb, lane_key, 0x7624);
                                    const uint32_t a6 = lut_lookup(wa, lane_key, 0x7634), a7 = lut_lookup(wb, lane_key, 0x7634);
#pragma unroll
                                    for (int nt = 0; nt < NT; ++nt) {
                                        mma_m16n8k16(acc[rr][P][nt], a0, a1, a2, a3, xv[s][nt].x, xv[s][nt].y);
                                        mma_m16n8k16(acc[rr][P][nt], a4, a5, a6, a7, xv[s][nt].z, xv[s][nt].w);
                                    }
                                }
                            }
                        }
                    }
                }
            }
            if (!ok) break;
            // advance the cursor past this segment
            u += c1 - c0;
            chunk = c1;
            if (chunk == p.chunks) { chunk = 0; ++tile; }

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
                    if (!consumers_sync()) { ok = false; break; }
                    if (receiver) {
#pragma unroll
                        for (int i = 0; i < kAccRegs; ++i) {
                            float v;
                            asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(slot + i * 128));
                            accf[i] += v;
                        }
                    }
                    if (!consumers_sync()) { ok = false; break; }
                }
                if (!ok) break;
            }

            // ---- a tile cut across CTAs: partials through the workspace, last arriver sums
            const bool full_tile = (c0 == 0 && c1 == p.chunks);
            bool do_store = full_tile;
            if (!full_tile) {
                const size_t tile_floats = (size_t)WM * kAccRegs * 32;
                if (active && wk == 0) {
                    float *dst = p.partials + (size_t)(2 * cta + (c0 == 0 ? 1 : 0)) * tile_floats + (size_t)wm * kAccRegs * 32 + lane;
#pragma unroll
                    for (int i = 0; i < kAccRegs; ++i) dst[i * 32] = accf[i];
                }
                __threadfence();
                if (!consumers_sync()) break;
                const int cta_first = cta_of_unit((long long)seg_tile * p.chunks, p.units, ctas);
                const int cta_last = cta_of_unit((long long)(seg_tile + 1) * p.chunks - 1, p.units, ctas);
                const int nseg = cta_last - cta_first + 1;
                if (cw == 0 && lane == 0) {
                    const unsigned int old = atomicAdd(&p.counters[seg_tile], 1u);
                    const int is_last = (old == (unsigned)nseg - 1);
                    if (is_last) p.counters[seg_tile] = 0;  // leave the counter clean for the next call
                    s_last = is_last;
                }
                if (!consumers_sync()) break;
                const int is_last = s_last;
                if (!consumers_sync()) break;  // s_last may be rewritten by the next segment
                if (is_last) {
                    __threadfence();
                    if (active && wk == 0) {
#pragma unroll
                        for (int i = 0; i < kAccRegs; ++i) accf[i] = 0.f;
                        for (int s = 0; s < nseg; ++s) {
                            const float *src = p.partials + (size_t)(2 * (cta_first + s) + (s == 0 ? 1 : 0)) * tile_floats +
                                               (size_t)wm * kAccRegs * 32 + lane;
#pragma unroll
                            for (int i = 0; i < kAccRegs; ++i) accf[i] += __ldcg(src + i * 32);
                        }
                    }
                    do_store = true;
                }
            }

            // ---- epilogue: fp32 scale by absmax, one rounding to fp16, 8-byte stores of 4 rows
            if (do_store && active && wk == 0) {
#pragma unroll
                for (int rr = 0; rr < R; ++rr) {
                    const int row = seg_tile * 32 * R * WM + (wm * R + rr) * 32 + 4 * g;
                    if (row >= p.m) continue;  // m % 8 == 0 and the 4 rows sit inside one 8-row group
                    const float4 sc = *reinterpret_cast<const float4 *>(p.absmax + row);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                        for (int e = 0; e < 2; ++e) {  // token 2t + e
                            const int tok = p.tok0 + nt * 8 + 2 * t + e;
                            if (tok >= p.n) continue;
                            uint2 v;
                            v.x = pack_half2(acc[rr][0][nt][e] * sc.x, acc[rr][0][nt][2 + e] * sc.y);
                            v.y = pack_half2(acc[rr][1][nt][e] * sc.z, acc[rr][1][nt][2 + e] * sc.w);
                            *reinterpret_cast<uint2 *>(p.o + (size_t)tok * p.m + row) = v;
                        }
                    }
                }
            }
        }
    }
    PROF_ROLE_END(warp == 0 ? 0 : 1);
}

// ------------------------------------------------------------------ host side

static void stream_geometry(int m, int k, const tuna_config &c, int nt, StreamParams *p)
{
    p->warps_m = c.warps_m; p->warps_k = c.warps_k; p->ksteps = c.k_steps; p->stages = c.stages_w;
    const int tile_rows = 32 * c.rows_per_warp * c.warps_m;
    const int chunk_cols = 32 * c.k_steps * c.warps_k;
    p->row_tiles = div_up(m, tile_rows);
    p->chunks = div_up(k, chunk_cols);
    p->units = (long long)p->row_tiles * p->chunks;
    p->stage_w_bytes = tile_rows * chunk_cols / 2;
    p->stage_x_bytes = nt * 8 * chunk_cols * 2;
    const int acc_regs = c.rows_per_warp * 2 * nt * 4;
    p->red_bytes = c.warps_k > 1 ? (c.warps_k / 2) * c.warps_m * acc_regs * 128 : 0;
}

// The kernel lays its buffers out around the first 64-KB boundary of its own shared window and
// takes as many stages as fit (at most `stages_w`); the launcher always asks for the whole SM.
// This is the lower bound that guarantees two stages wherever that boundary falls.
static size_t stream_min_smem_bytes(const StreamParams &p)
{
    const size_t stage = (size_t)p.stage_w_bytes + p.stage_x_bytes;
    return 4096 + kLut64Bytes + 2 * stage + p.red_bytes + (65536 - 4096) % stage;
}

int gemm_stream_normalize_config(int m, int n, int k, int sm_count, tuna_config *c)
{
    if (c->tile_tok == 0) c->tile_tok = (n <= 8) ? 8 : (n <= 16 ? 16 : 32);
    if (c->tile_tok != 8 && c->tile_tok != 16 && c->tile_tok != 32) return TUNA_ERR_BAD_CONFIG;
    const int nt = c->tile_tok / 8;
    if (c->stages_w == 0) c->stages_w = 12;  // an upper bound: the kernel takes what fits
    if (c->ctas < 0) return TUNA_ERR_BAD_CONFIG;
    if (c->ctas == 0 || c->ctas > sm_count) c->ctas = sm_count;
    StreamParams p;
    if (c->rows_per_warp == 0 || c->warps_m == 0 || c->warps_k == 0 || c->k_steps == 0) {
        // No table entry: pick the geometry with the least estimated traffic.  Weights are read
        // once whatever the geometry; what differs is the activation re-reads (one x box per
        // unit, from L2) and the split-K partials (written and read back once per cut tile).
        double best = 1e300;
        tuna_config bc = *c;
        for (int r = 1; r <= 2; ++r)
            for (int wm = 1; wm <= 16; wm <<= 1)
                for (int ks = 1; ks <= 2; ++ks) {
                    tuna_config t = *c;
                    t.rows_per_warp = c->rows_per_warp ? c->rows_per_warp : r;
                    t.warps_m = c->warps_m ? c->warps_m : wm;
                    t.warps_k = c->warps_k ? c->warps_k : 16 / t.warps_m;
                    t.k_steps = c->k_steps ? c->k_steps : ks;
                    while (t.warps_k > 1 && 32 * t.k_steps * (t.warps_k / 2) >= k) t.warps_k >>= 1;
                    if (t.rows_per_warp * nt > 4 || t.warps_m * t.warps_k > kConsumerWarps) continue;
                    stream_geometry(m, k, t, nt, &p);
                    if (stream_min_smem_bytes(p) > (size_t)kStreamSmemLimit) continue;
                    const double x_bytes = (double)p.units * p.stage_x_bytes;
                    const double tile_bytes = (double)t.warps_m * t.rows_per_warp * 32 * nt * 8 * 4;
                    const double cuts = (p.units % c->ctas == 0 && p.chunks % (p.units / c->ctas) == 0) ? 0 : 2.0 * c->ctas;
                    const double ring = (double)(kStreamSmemLimit - 70000 - p.red_bytes) / (p.stage_w_bytes + p.stage_x_bytes);
                    double cost = 0.5 * x_bytes + 3.0 * cuts * tile_bytes + (ring < 3 ? 1e12 : 0) +
                                  (t.warps_k > 1 ? 2e5 * t.warps_k : 0);
                    if (cost < best) { best = cost; bc = t; }
                }
        if (best >= 1e300) return TUNA_ERR_BAD_CONFIG;
        *c = bc;
    }
    auto pow2 = [](int v) { return v > 0 && (v & (v - 1)) == 0; };
    if (c->rows_per_warp != 1 && c->rows_per_warp != 2) return TUNA_ERR_BAD_CONFIG;
    if (c->rows_per_warp * nt > 4) return TUNA_ERR_BAD_CONFIG;  // accumulator registers
    if (c->k_steps != 1 && c->k_steps != 2) return TUNA_ERR_BAD_CONFIG;
    if (!pow2(c->warps_m) || !pow2(c->warps_k) || c->warps_m * c->warps_k > kConsumerWarps) return TUNA_ERR_BAD_CONFIG;
    if (4 * c->rows_per_warp * c->warps_m > 256) return TUNA_ERR_BAD_CONFIG;
    if (c->stages_w < 2 || c->stages_w > 16) return TUNA_ERR_BAD_CONFIG;
    stream_geometry(m, k, *c, nt, &p);
    if (stream_min_smem_bytes(p) > (size_t)kStreamSmemLimit) return TUNA_ERR_BAD_CONFIG;
    (void)n;
    return TUNA_OK;
}

size_t gemm_stream_workspace_bytes(int m, int n, int k, const tuna_config &c)
{
    (void)n;
    StreamParams p;
    const int nt = c.tile_tok / 8;
    stream_geometry(m, k, c, nt, &p);
    const size_t counters = ((size_t)p.row_tiles * 4 + 255) / 256 * 256;
    const size_t tile_floats = (size_t)c.warps_m * (c.rows_per_warp * 2 * nt * 4) * 32;
    return counters + 2 * (size_t)c.ctas * tile_floats * 4;
}

template <int R, int NT>
static int launch_one(const StreamParams &p, const CUtensorMap &mq, const CUtensorMap &mx, int ctas, size_t smem,
                      cudaStream_t stream)
{
    static bool attr_set = false;  // one-time opt-in to large dynamic shared memory
    if (!attr_set) {
        if (cudaFuncSetAttribute(gemm_stream_kernel<R, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kStreamSmemLimit) != cudaSuccess)
            return TUNA_ERR_NO_DEVICE;
        attr_set = true;
    }
    gemm_stream_kernel<R, NT><<<ctas, kStreamThreads, smem, stream>>>(p, mq, mx);
    return cudaGetLastError() == cudaSuccess ? TUNA_OK : TUNA_ERR_LAUNCH;
}

int launch_gemm_stream(const GemmArgs &a, const tuna_config &cfg)
{
    const int nt = cfg.tile_tok / 8;
    StreamParams p;
    std::memset(&p, 0, sizeof(p));
    p.code = a.code; p.absmax = a.absmax; p.o = (__half *)a.o;
    p.m = a.m; p.n = a.n; p.k = a.k;
    stream_geometry(a.m, a.k, cfg, nt, &p);
    p.status = device_status_word();
    if (!p.status) return TUNA_ERR_NO_DEVICE;
    const size_t counters = ((size_t)p.row_tiles * 4 + 255) / 256 * 256;
    if (a.workspace == nullptr || a.workspace_bytes < gemm_stream_workspace_bytes(a.m, a.n, a.k, cfg))
        return TUNA_ERR_WORKSPACE;
    p.counters = (unsigned int *)a.workspace;
    p.partials = (float *)((uint8_t *)a.workspace + counters);
    int ctas = cfg.ctas;
    if ((long long)ctas > p.units) ctas = (int)p.units;

    CUtensorMap mq, mx;
    // packed weights as [m/8 row groups][4k bytes]; box = tile's row groups x (128 * S) bytes
    if (!make_tensor_map_2d(&mq, CU_TENSOR_MAP_DATA_TYPE_UINT8, a.q, (uint64_t)a.k * 4, (uint64_t)a.m / 8,
                            (uint64_t)a.k * 4, 128u * cfg.k_steps, 4u * cfg.rows_per_warp * cfg.warps_m,
                            CU_TENSOR_MAP_SWIZZLE_NONE))
        return TUNA_ERR_NO_DEVICE;
    // activations as [n][k] fp16; box = tile_tok tokens x (32 * S) columns
    if (!make_tensor_map_2d(&mx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, a.x, (uint64_t)a.k, (uint64_t)a.n, (uint64_t)a.k * 2,
                            32u * cfg.k_steps, (uint32_t)cfg.tile_tok, CU_TENSOR_MAP_SWIZZLE_NONE))
        return TUNA_ERR_NO_DEVICE;
    const size_t smem = kStreamSmemLimit;

    for (int tok0 = 0; tok0 < a.n; tok0 += cfg.tile_tok) {
        p.tok0 = tok0;
        int st;
        switch (cfg.rows_per_warp * 10 + nt) {
            case 11: st = launch_one<1, 1>(p, mq, mx, ctas, smem, a.stream); break;
            case 12: st = launch_one<1, 2>(p, mq, mx, ctas, smem, a.stream); break;
            case 14: st = launch_one<1, 4>(p, mq, mx, ctas, smem, a.stream); break;
            case 21: st = launch_one<2, 1>(p, mq, mx, ctas, smem, a.stream); break;
            case 22: st = launch_one<2, 2>(p, mq, mx, ctas, smem, a.stream); break;
            default: return TUNA_ERR_BAD_CONFIG;
        }
        if (st != TUNA_OK) return st;
    }
    return TUNA_OK;
}

}  // namespace tuna
