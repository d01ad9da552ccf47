// Weight-streaming FP16 x 4-bit(codebook) GEMM for small token counts (n <= 16
// per pass), sm_100a.  Counterpart of the reference's Tuna<> kernel and its
// Deq4GemmIterator main loop (kernel.cu:1043-2505, 2816-2960) for the
// memory-bound regime; same mma orientation (weights are the m16 "A" operand,
// tokens the n8 "B" operand, kernel.cu:2182-2192), nothing else in common.
//
// Data path.  A lane reads 16 packed bytes with one streaming 128-bit load:
// half of an 8x8 tile = 4 rows x 8 columns of one row group.  Lane (g,t)
// (g = lane/4, t = lane%4) takes row group g/2, rows 4(g%2)..+3, tile 4*step+t,
// so a warp load covers four 128-byte runs (4 row groups x 4 tiles) = 32 rows x
// 32 columns.  Each 32-bit word is one row's 8 consecutive columns and becomes
// the A fragments of two m16n8k16 mma.sync (the k index of an mma is only a
// label: slot 2t,2t+1 <-> columns 0,1 of tile t, slot 2t+8,+9 <-> columns 2,3;
// the B fragment is gathered with the same labelling, 16 contiguous bytes of x
// per lane).  Rows 4g, 4g+1 feed tile "P0", rows 4g+2, 4g+3 tile "P1".
//
// Dequantisation.  A byte holds two codes; a 256-entry byte -> half2 table of
// fp16(code[hi]), fp16(code[lo]) is replicated once per lane (bank) in shared
// memory so every lookup is conflict free.  The per-row scale is applied once,
// in fp32, to the accumulated sum in the epilogue (absmax is constant along K:
// one block per row, test.py:81, kernel.cu:2178-2180).
//
// Split-K.  Warps of a CTA that share rows reduce through shared memory in a
// fixed order.  CTAs along K write fp32 partials to the workspace; the CTA that
// arrives last at the tile's counter adds them in split order, so the result
// does not depend on arrival order, the output needs no zero fill and there
// are no floating-point atomics (the reference atomically adds fp16 partials,
// kernel.cu:2739-2745).
#include "common.cuh"
#include "launchers.h"

namespace tuna {

constexpr int kLutBytes = 256 * 32 * 4;  // 256 entries x 32 lane copies x half2
constexpr int kStreamMaxSmem = 200 * 1024;
constexpr int kPrefetch = 2;  // k-steps of weight loads in flight per warp

struct StreamParams {
    const uint8_t *q;
    const __half *x;
    const float *code;
    const float *absmax;
    __half *o;
    float *partials;        // workspace: split-K partial tiles
    unsigned int *counters; // workspace: one per row tile, zero between calls
    int m, n, k;
    int tok0;               // first token of this pass
    int warps_m, warps_k, split_k;
    int steps_total;        // ceil(k / 32)
    int x_stride_bytes;     // shared-memory row pitch of the x slice
    int max_cta_steps;
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

// Even split of `total` items over `parts`: [begin, end) of part `i`.
__host__ __device__ inline void even_split(int total, int parts, int i, int &begin, int &end)
{
    begin = (int)(((long long)total * i) / parts);
    end = (int)(((long long)total * (i + 1)) / parts);
}

template <int R, int NT>
__global__ void __launch_bounds__(512, 1) gemm_stream_kernel(const StreamParams p)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    uint32_t *lut = reinterpret_cast<uint32_t *>(smem);
    uint8_t *xs = smem + kLutBytes;
    __shared__ unsigned int s_ticket;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int wm = warp % p.warps_m, wk = warp / p.warps_m;
    const int tile_rows = 32 * R * p.warps_m;
    const int row_tile = blockIdx.x;
    const int split = blockIdx.y;

    int cta_s0, cta_s1;
    even_split(p.steps_total, p.split_k, split, cta_s0, cta_s1);

    // ---- byte -> half2 table, one copy per bank
    for (int e = warp; e < 256; e += blockDim.x >> 5) {
        const __half hi = __float2half_rn(p.code[e >> 4]);
        const __half lo = __float2half_rn(p.code[e & 15]);
        lut[e * 32 + lane] = (uint32_t)__half_as_ushort(hi) | ((uint32_t)__half_as_ushort(lo) << 16);
    }
    // ---- x slice [NT*8 tokens][32*(s1-s0) columns], zero where token >= n or column >= k
    {
        const int cols = (cta_s1 - cta_s0) * 32;
        const int chunks_per_row = cols / 8;  // 16-byte chunks
        const int total = NT * 8 * chunks_per_row;
        for (int i = tid; i < total; i += blockDim.x) {
            const int row = i / chunks_per_row, c = i - row * chunks_per_row;
            const int tok = p.tok0 + row, col = cta_s0 * 32 + c * 8;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (tok < p.n && col < p.k)  // k % 8 == 0: a chunk is all in or all out
                v = *reinterpret_cast<const uint4 *>(p.x + (size_t)tok * p.k + col);
            *reinterpret_cast<uint4 *>(xs + (size_t)row * p.x_stride_bytes + c * 16) = v;
        }
    }
    __syncthreads();

    // ---- this warp's rows and k-steps
    int s0, s1;
    even_split(cta_s1 - cta_s0, p.warps_k, wk, s0, s1);
    s0 += cta_s0;
    s1 += cta_s0;
    const int warp_row0 = row_tile * tile_rows + wm * 32 * R;
    const int n_rg = p.m >> 3, n_kt = p.k >> 3;

    const uint8_t *src[R];
    bool row_ok[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int rg = (warp_row0 + 32 * r) / 8 + (g >> 1);
        row_ok[r] = rg < n_rg;
        src[r] = p.q + (size_t)(row_ok[r] ? rg : 0) * row_group_bytes(p.k) + (size_t)t * 32 + (g & 1) * 16;
    }

    float acc[R][2][NT][4];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int P = 0; P < 2; ++P)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[r][P][nt][c] = 0.f;

    auto load_step = [&](int s, uint4 (&dst)[R]) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (s < s1 && row_ok[r] && (4 * s + t) < n_kt)
                dst[r] = ldg_stream_u4(src[r] + (size_t)s * 128);
            else
                dst[r] = make_uint4(0, 0, 0, 0);
        }
    };

    uint4 buf[kPrefetch][R];
#pragma unroll
    for (int j = 0; j < kPrefetch; ++j) load_step(s0 + j, buf[j]);

    const uint32_t *lut_lane = lut + lane;
    const uint8_t *xs_lane = xs + (size_t)g * p.x_stride_bytes + t * 16;

    for (int sb = s0; sb < s1; sb += kPrefetch) {
#pragma unroll
        for (int j = 0; j < kPrefetch; ++j) {
            const int s = sb + j;
            if (s < s1) {
                uint4 cur[R];
#pragma unroll
                for (int r = 0; r < R; ++r) cur[r] = buf[j][r];
                load_step(s + kPrefetch, buf[j]);

                uint4 xb[NT];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
                    xb[nt] = *reinterpret_cast<const uint4 *>(
                        xs_lane + (size_t)(8 * nt) * p.x_stride_bytes + (size_t)(s - cta_s0) * 64);

#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const uint32_t w[4] = {cur[r].x, cur[r].y, cur[r].z, cur[r].w};
#pragma unroll
                    for (int P = 0; P < 2; ++P) {
                        const uint32_t wa = w[2 * P], wb = w[2 * P + 1];
                        uint32_t a[8];
#pragma unroll
                        for (int b = 0; b < 4; ++b) {
                            a[2 * b] = lut_lane[((wa >> (8 * b)) & 0xffu) * 32];
                            a[2 * b + 1] = lut_lane[((wb >> (8 * b)) & 0xffu) * 32];
                        }
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
                            mma_m16n8k16(acc[r][P][nt], a[0], a[1], a[2], a[3], xb[nt].x, xb[nt].y);
                            mma_m16n8k16(acc[r][P][nt], a[4], a[5], a[6], a[7], xb[nt].z, xb[nt].w);
                        }
                    }
                }
            }
        }
    }

    // ---- reduce the warps that share rows (fixed order: wk = 0, 1, 2, ...)
    constexpr int kAccRegs = R * 2 * NT * 4;
    if (p.warps_k > 1) {
        __syncthreads();  // everyone is done with the x slice; reuse it
        float *red = reinterpret_cast<float *>(xs);
        if (wk > 0) {
            float *dst = red + ((size_t)((wk - 1) * p.warps_m + wm) * kAccRegs) * 32 + lane;
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int P = 0; P < 2; ++P)
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            dst[(((r * 2 + P) * NT + nt) * 4 + c) * 32] = acc[r][P][nt][c];
        }
        __syncthreads();
        if (wk == 0) {
            for (int j = 1; j < p.warps_k; ++j) {
                const float *srcp = red + ((size_t)((j - 1) * p.warps_m + wm) * kAccRegs) * 32 + lane;
#pragma unroll
                for (int r = 0; r < R; ++r)
#pragma unroll
                    for (int P = 0; P < 2; ++P)
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                            for (int c = 0; c < 4; ++c)
                                acc[r][P][nt][c] += srcp[(((r * 2 + P) * NT + nt) * 4 + c) * 32];
            }
        }
    }

    // ---- reduce the CTAs along K through the workspace (last arriver sums in split order)
    if (p.split_k > 1) {
        const size_t tile_floats = (size_t)p.warps_m * kAccRegs * 32;
        float *tile_base = p.partials + (size_t)row_tile * p.split_k * tile_floats;
        if (wk == 0) {
            float *dst = tile_base + (size_t)split * tile_floats + (size_t)wm * kAccRegs * 32 + lane;
#pragma unroll
            for (int i = 0; i < kAccRegs; ++i)
                dst[i * 32] = (&acc[0][0][0][0])[i];
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const unsigned int old = atomicAdd(&p.counters[row_tile], 1u);
            s_ticket = old;
            if (old == (unsigned)p.split_k - 1) p.counters[row_tile] = 0;  // leave it clean
        }
        __syncthreads();
        if (s_ticket != (unsigned)p.split_k - 1) return;
        __threadfence();
        if (wk == 0) {
#pragma unroll
            for (int i = 0; i < kAccRegs; ++i) (&acc[0][0][0][0])[i] = 0.f;
            for (int s = 0; s < p.split_k; ++s) {
                const float *srcp = tile_base + (size_t)s * tile_floats + (size_t)wm * kAccRegs * 32 + lane;
#pragma unroll
                for (int i = 0; i < kAccRegs; ++i)
                    (&acc[0][0][0][0])[i] += __ldcg(srcp + i * 32);
            }
        }
    }
    if (wk != 0) return;

    // ---- epilogue: scale by absmax (fp32), round once to fp16, 8-byte stores of 4 rows
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int row = warp_row0 + 32 * r + 4 * g;
        if (row >= p.m) continue;  // m % 8 == 0 and 4 rows sit inside one 8-row group
        const float4 sc = *reinterpret_cast<const float4 *>(p.absmax + row);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {  // token 2t + e
                const int tok = p.tok0 + nt * 8 + 2 * t + e;
                if (tok >= p.n) continue;
                uint2 v;
                v.x = pack_half2(acc[r][0][nt][e] * sc.x, acc[r][0][nt][2 + e] * sc.y);
                v.y = pack_half2(acc[r][1][nt][e] * sc.z, acc[r][1][nt][2 + e] * sc.w);
                *reinterpret_cast<uint2 *>(p.o + (size_t)tok * p.m + row) = v;
            }
        }
    }
}

// ------------------------------------------------------------------ host side

static int stream_x_stride_bytes(int cta_steps)
{
    int b = cta_steps * 64;
    if (b % 128 == 0) b += 64;  // rows g and g+1 must land in different bank halves
    return b;
}

static size_t stream_smem_bytes(const tuna_config &c, int steps_total, int nt)
{
    const int max_cta_steps = div_up(steps_total, c.split_k);
    const size_t xbytes = (size_t)nt * 8 * stream_x_stride_bytes(max_cta_steps);
    const size_t red = (size_t)(c.warps_k - 1) * c.warps_m * (c.rows_per_warp * 2 * nt * 4) * 32 * 4;
    return kLutBytes + (xbytes > red ? xbytes : red);
}

int gemm_stream_normalize_config(int m, int n, int k, int sm_count, tuna_config *c)
{
    if (c->tile_tok == 0) c->tile_tok = (n <= 8) ? 8 : 16;
    if (c->tile_tok != 8 && c->tile_tok != 16) return TUNA_ERR_BAD_CONFIG;
    const int nt = c->tile_tok / 8;
    const int steps_total = div_up(k, 32);
    const bool heuristic = c->rows_per_warp == 0 || c->warps_m == 0 || c->warps_k == 0 || c->split_k == 0;
    if (heuristic) {
        // One CTA of 16 warps per SM.  Pick the row tile so that tiles x split_k lands just
        // under a multiple of the SM count, and keep >= ~8 k-steps per warp.
        const int blocks = div_up(m, 32);
        int best_r = 1, best_wm = 1, best_wk = 16, best_sk = 1;
        double best_cost = 1e30;
        for (int r : {1, 2, 4})
            for (int wmv : {1, 2, 4, 8, 16})
                for (int sk = 1; sk <= 32; ++sk) {
                    const int wkv = 16 / wmv;
                    if (steps_total / sk < 1) continue;
                    tuna_config t = *c;
                    t.rows_per_warp = r; t.warps_m = wmv; t.warps_k = wkv; t.split_k = sk;
                    if (stream_smem_bytes(t, steps_total, nt) > (size_t)kStreamMaxSmem) continue;
                    const int tiles = div_up(blocks, r * wmv);
                    const long long ctas = (long long)tiles * sk;
                    const int waves = (int)div_up_ll(ctas, sm_count);
                    // time ~ waves x (work per CTA) + fixed costs; work per CTA ~ r*wmv*steps/sk
                    const double steps_per_warp = (double)steps_total / sk / wkv;
                    double cost = waves * ((double)r * wmv * steps_total / sk + 400.0)
                                  + (sk > 1 ? 300.0 : 0.0) + 8.0 * wkv
                                  + (steps_per_warp < 4 ? 400.0 : 0.0)
                                  + 64.0 / r;  // B-fragment re-reads
                    if (cost < best_cost) { best_cost = cost; best_r = r; best_wm = wmv; best_wk = wkv; best_sk = sk; }
                }
        c->rows_per_warp = best_r; c->warps_m = best_wm; c->warps_k = best_wk; c->split_k = best_sk;
    }
    if (c->rows_per_warp != 1 && c->rows_per_warp != 2 && c->rows_per_warp != 4) return TUNA_ERR_BAD_CONFIG;
    if (c->warps_m < 1 || c->warps_k < 1 || c->warps_m * c->warps_k > 16) return TUNA_ERR_BAD_CONFIG;
    if (c->split_k < 1 || c->split_k > steps_total) return TUNA_ERR_BAD_CONFIG;
    if (stream_smem_bytes(*c, steps_total, nt) > (size_t)kStreamMaxSmem) return TUNA_ERR_BAD_CONFIG;
    (void)n;
    return TUNA_OK;
}

size_t gemm_stream_workspace_bytes(int m, int n, int k, const tuna_config &c)
{
    (void)n; (void)k;
    const int nt = c.tile_tok / 8;
    const int tiles = div_up(m, 32 * c.rows_per_warp * c.warps_m);
    const size_t counters = ((size_t)tiles * 4 + 255) / 256 * 256;
    if (c.split_k <= 1) return counters;
    const size_t tile_floats = (size_t)c.warps_m * (c.rows_per_warp * 2 * nt * 4) * 32;
    return counters + (size_t)tiles * c.split_k * tile_floats * 4;
}

template <int R, int NT>
static int launch_one(const StreamParams &p, dim3 grid, int threads, size_t smem, cudaStream_t stream)
{
    static bool attr_set = false;  // one-time opt-in to large dynamic shared memory
    if (!attr_set) {
        if (cudaFuncSetAttribute(gemm_stream_kernel<R, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kStreamMaxSmem) != cudaSuccess)
            return TUNA_ERR_NO_DEVICE;
        attr_set = true;
    }
    gemm_stream_kernel<R, NT><<<grid, threads, smem, stream>>>(p);
    return cudaGetLastError() == cudaSuccess ? TUNA_OK : TUNA_ERR_LAUNCH;
}

int launch_gemm_stream(const GemmArgs &a, const tuna_config &cfg)
{
    const int nt = cfg.tile_tok / 8;
    StreamParams p;
    p.q = a.q; p.x = (const __half *)a.x; p.code = a.code; p.absmax = a.absmax; p.o = (__half *)a.o;
    p.m = a.m; p.n = a.n; p.k = a.k;
    p.warps_m = cfg.warps_m; p.warps_k = cfg.warps_k; p.split_k = cfg.split_k;
    p.steps_total = div_up(a.k, 32);
    p.max_cta_steps = div_up(p.steps_total, cfg.split_k);
    p.x_stride_bytes = stream_x_stride_bytes(p.max_cta_steps);
    const int tiles = div_up(a.m, 32 * cfg.rows_per_warp * cfg.warps_m);
    const size_t counters = ((size_t)tiles * 4 + 255) / 256 * 256;
    const size_t need = gemm_stream_workspace_bytes(a.m, a.n, a.k, cfg);
    if (cfg.split_k > 1 && (a.workspace == nullptr || a.workspace_bytes < need)) return TUNA_ERR_WORKSPACE;
    p.counters = (unsigned int *)a.workspace;
    p.partials = a.workspace ? (float *)((uint8_t *)a.workspace + counters) : nullptr;
    const size_t smem = stream_smem_bytes(cfg, p.steps_total, nt);
    const dim3 grid(tiles, cfg.split_k);
    const int threads = 32 * cfg.warps_m * cfg.warps_k;

    for (int tok0 = 0; tok0 < a.n; tok0 += cfg.tile_tok) {
        p.tok0 = tok0;
        int st;
        const int key = cfg.rows_per_warp * 10 + nt;
        switch (key) {
            case 11: st = launch_one<1, 1>(p, grid, threads, smem, a.stream); break;
            case 12: st = launch_one<1, 2>(p, grid, threads, smem, a.stream); break;
            case 21: st = launch_one<2, 1>(p, grid, threads, smem, a.stream); break;
            case 22: st = launch_one<2, 2>(p, grid, threads, smem, a.stream); break;
            case 41: st = launch_one<4, 1>(p, grid, threads, smem, a.stream); break;
            case 42: st = launch_one<4, 2>(p, grid, threads, smem, a.stream); break;
            default: return TUNA_ERR_BAD_CONFIG;
        }
        if (st != TUNA_OK) return st;
    }
    return TUNA_OK;
}

}  // namespace tuna
