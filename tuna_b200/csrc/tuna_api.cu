// C ABI of tuna_b200: argument validation, shape -> config lookup, dispatch.
// Host-side counterpart of the reference's `wrapper` / `dequantize_wrapper`
// (kernel.cu:3009-3156, 3243-3253).  The reference resolves a shape with a
// compile-time if-chain and silently launches nothing for an unknown one; here
// the table is data (generated from param_map.json), lookup happens at run
// time and every failure is a status code.
#include <cstring>
#include <mutex>
#include <vector>
#include "common.cuh"
#include "launchers.h"

namespace tuna {

struct TableEntry {
    int m, n_bucket, k;
    tuna_config cfg;
};

static const TableEntry kTable[] = {
#include "config_table.inc"
    {0, 0, 0, {}}  // sentinel
};
static const int kTableSize = (int)(sizeof(kTable) / sizeof(kTable[0])) - 1;

// Token buckets of the table: the smallest listed bound >= n.
static int token_bucket(int n)
{
    static const int bounds[] = {8, 16, 32, 64, 128, 256, 512, 1024};
    for (int b : bounds)
        if (n <= b) return b;
    return 2048;
}

static int device_sm_count()
{
    static int cached[64];
    static std::once_flag once;
    std::call_once(once, [] { std::memset(cached, 0, sizeof(cached)); });
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        cached[dev] = v;
    }
    return cached[dev];
}

static int resolve_config(int m, int n, int k, int sm_count, const tuna_config *user, tuna_config *out)
{
    tuna_config c;
    std::memset(&c, 0, sizeof(c));
    if (user) {
        c = *user;
    } else {
        const int b = token_bucket(n);
        for (int i = 0; i < kTableSize; ++i)
            if (kTable[i].m == m && kTable[i].k == k && kTable[i].n_bucket == b) { c = kTable[i].cfg; break; }
    }
    // No table entry: the tcgen05 weight-streaming kernel up to one 64-token pass (the regime
    // bound by HBM), the TMA-staged tcgen05 kernel above it.
    if (c.path == TUNA_PATH_AUTO) c.path = (n <= 64) ? TUNA_PATH_TSTREAM : TUNA_PATH_UMMA;
    int st;
    if (c.path == TUNA_PATH_STREAM) st = gemm_stream_normalize_config(m, n, k, sm_count, &c);
    else if (c.path == TUNA_PATH_UMMA) st = gemm_umma_normalize_config(m, n, k, sm_count, &c);
    else if (c.path == TUNA_PATH_TSTREAM) st = gemm_tstream_normalize_config(m, n, k, sm_count, &c);
    else st = TUNA_ERR_BAD_CONFIG;
    if (st != TUNA_OK) return st;
    *out = c;
    return TUNA_OK;
}

static int check_shape(int m, int n, int k)
{
    if (m <= 0 || k <= 0 || n <= 0 || (m % 8) || (k % 8)) return TUNA_ERR_BAD_SHAPE;
    if ((long long)m * k / 2 > (1ll << 40)) return TUNA_ERR_TOO_LARGE;
    return TUNA_OK;
}

static bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

static size_t workspace_for(int m, int n, int k, const tuna_config &c, int sm_count)
{
    if (c.path == TUNA_PATH_STREAM) return gemm_stream_workspace_bytes(m, n, k, c, sm_count);
    if (c.path == TUNA_PATH_TSTREAM) return gemm_tstream_workspace_bytes(m, n, k, c, sm_count);
    return gemm_umma_workspace_bytes(m, n, k, c, sm_count);
}

static int launch_gemm(const GemmArgs &a, const tuna_config &c)
{
    if (c.path == TUNA_PATH_STREAM) return launch_gemm_stream(a, c);
    if (c.path == TUNA_PATH_TSTREAM) return launch_gemm_tstream(a, c);
    return launch_gemm_umma(a, c);
}

}  // namespace tuna

using namespace tuna;

extern "C" int tuna_matmul_cfg(const void *q, const void *x, const void *code, const void *absmax, void *o,
                               int m, int n, int k, void *workspace, size_t workspace_bytes, void *stream,
                               const tuna_config *cfg)
{
    if (!q || !x || !code || !absmax || !o) return TUNA_ERR_NULL_POINTER;
    int st = check_shape(m, n, k);
    if (st != TUNA_OK) return st;
    if (!aligned(q, 16) || !aligned(x, 16) || !aligned(o, 16) || !aligned(absmax, 4) || !aligned(code, 4) ||
        !aligned(workspace, 16))
        return TUNA_ERR_MISALIGNED;
    const int sms = device_sm_count();
    tuna_config c;
    st = resolve_config(m, n, k, sms, cfg, &c);
    if (st != TUNA_OK) return st;
    const size_t need = workspace_for(m, n, k, c, sms);
    if (need > 0 && (workspace == nullptr || workspace_bytes < need)) return TUNA_ERR_WORKSPACE;
    GemmArgs a;
    a.q = (const uint8_t *)q; a.x = x; a.code = (const float *)code; a.absmax = (const float *)absmax; a.o = o;
    a.m = m; a.n = n; a.k = k; a.workspace = workspace; a.workspace_bytes = workspace_bytes;
    a.stream = (cudaStream_t)stream; a.sm_count = sms;
    return launch_gemm(a, c);
}

extern "C" int tuna_matmul_batched(const void *q, const void *x, const void *code, const void *absmax, void *o,
                                   int m, int n, int k, int batch, size_t q_stride, size_t x_stride, size_t absmax_stride,
                                   size_t o_stride, void *workspace, size_t workspace_bytes, void *stream)
{
    if (!q || !x || !code || !absmax || !o) return TUNA_ERR_NULL_POINTER;
    int st = check_shape(m, n, k);
    if (st != TUNA_OK) return st;
    if (batch < 1 || batch > 65536) return TUNA_ERR_BAD_SHAPE;
    if (!aligned(q, 16) || !aligned(x, 16) || !aligned(o, 16) || !aligned(absmax, 16) || !aligned(code, 4) ||
        !aligned(workspace, 16) || (q_stride % 16) || (x_stride % 16) || (absmax_stride % 16) || (o_stride % 16))
        return TUNA_ERR_MISALIGNED;
    const int sms = device_sm_count();
    tuna_config c;
    st = resolve_config(m, n, k, sms, nullptr, &c);
    if (st != TUNA_OK) return st;
    GemmArgs a;
    a.code = (const float *)code;
    a.m = m; a.n = n; a.k = k; a.workspace = workspace; a.workspace_bytes = workspace_bytes;
    a.stream = (cudaStream_t)stream; a.sm_count = sms;
    if (c.path == TUNA_PATH_STREAM) {
        // one launch over all matrices: the step range of every CTA runs across them
        const size_t need = gemm_stream_workspace_bytes(m, n, k, c, sms, batch);
        if (workspace == nullptr || workspace_bytes < need) return TUNA_ERR_WORKSPACE;
        a.q = (const uint8_t *)q; a.x = x; a.absmax = (const float *)absmax; a.o = o;
        a.batch = batch; a.q_stride = q_stride; a.x_stride = x_stride; a.absmax_stride = absmax_stride; a.o_stride = o_stride;
        return launch_gemm_stream(a, c);
    }
    // the tcgen05 kernels: one launch per matrix
    const size_t need = workspace_for(m, n, k, c, sms);
    if (workspace == nullptr || workspace_bytes < need) return TUNA_ERR_WORKSPACE;
    for (int b = 0; b < batch; ++b) {
        a.q = (const uint8_t *)q + (size_t)b * q_stride;
        a.x = (const uint8_t *)x + (size_t)b * x_stride;
        a.absmax = (const float *)((const uint8_t *)absmax + (size_t)b * absmax_stride);
        a.o = (uint8_t *)o + (size_t)b * o_stride;
        st = launch_gemm(a, c);
        if (st != TUNA_OK) return st;
    }
    return TUNA_OK;
}

extern "C" size_t tuna_matmul_batched_workspace_bytes(int m, int n, int k, int batch)
{
    if (check_shape(m, n, k) != TUNA_OK || batch < 1) return 0;
    const int sms = device_sm_count();
    tuna_config c;
    if (resolve_config(m, n, k, sms, nullptr, &c) != TUNA_OK) return 0;
    return c.path == TUNA_PATH_STREAM ? gemm_stream_workspace_bytes(m, n, k, c, sms, batch) : workspace_for(m, n, k, c, sms);
}

// The GEMMs of a sequence that have tokens (n = 0 is an expert nobody was routed to: nothing to do).
static int sequence_compact(const tuna_gemm_desc *g, int count, std::vector<tuna_gemm_desc> *out)
{
    out->clear();
    for (int i = 0; i < count; ++i) {
        if (g[i].n == 0 && g[i].m > 0 && g[i].k > 0 && !(g[i].m % 8) && !(g[i].k % 8)) continue;
        if (!g[i].q || !g[i].x || !g[i].absmax || !g[i].o) return TUNA_ERR_NULL_POINTER;
        const int st = check_shape(g[i].m, g[i].n, g[i].k);
        if (st != TUNA_OK) return st;
        if (!aligned(g[i].q, 16) || !aligned(g[i].x, 16) || !aligned(g[i].o, 16) || !aligned(g[i].absmax, 4)) return TUNA_ERR_MISALIGNED;
        out->push_back(g[i]);
    }
    return TUNA_OK;
}

extern "C" size_t tuna_matmul_sequence_workspace_bytes(const tuna_gemm_desc *g, int count)
{
    if (!g || count < 1) return 0;
    const int sms = device_sm_count();
    size_t need = gemm_tstream_sequence_workspace_bytes(g, count, sms);  // an upper bound whatever the token counts
    for (int i = 0; i < count; ++i) {  // the fallback issues them one by one on the same workspace
        if (g[i].n == 0) continue;
        const size_t w = tuna_matmul_workspace_bytes(g[i].m, g[i].n, g[i].k);
        if (w == 0) return 0;
        need = w > need ? w : need;
    }
    return need;
}

extern "C" int tuna_matmul_sequence(const tuna_gemm_desc *g, int count, const void *code, void *workspace, size_t workspace_bytes,
                                    void *stream)
{
    if (!g || !code) return TUNA_ERR_NULL_POINTER;
    if (count < 1) return TUNA_ERR_BAD_SHAPE;
    if (!aligned(code, 4) || !aligned(workspace, 16)) return TUNA_ERR_MISALIGNED;
    std::vector<tuna_gemm_desc> live;
    int st = sequence_compact(g, count, &live);
    if (st != TUNA_OK) return st;
    if (live.empty()) return TUNA_OK;
    const int sms = device_sm_count();
    if (gemm_tstream_sequence_supported(live.data(), (int)live.size()))
        return launch_gemm_tstream_sequence(live.data(), (int)live.size(), (const float *)code, workspace, workspace_bytes, sms,
                                            (cudaStream_t)stream);
    for (const tuna_gemm_desc &d : live) {
        st = tuna_matmul(d.q, d.x, code, d.absmax, d.o, d.m, d.n, d.k, workspace, workspace_bytes, stream);
        if (st != TUNA_OK) return st;
    }
    return TUNA_OK;
}

extern "C" int tuna_matmul_sequence_reduce(const tuna_gemm_desc *g, int count, const void *code, void *workspace,
                                           size_t workspace_bytes, const tuna_exchange *ex, void *stream)
{
    if (!g || !code || !ex) return TUNA_ERR_NULL_POINTER;
    if (count < 1) return TUNA_ERR_BAD_SHAPE;
    if (ex->world < 1 || ex->world > TUNA_MAX_PEERS || ex->rank < 0 || ex->rank >= ex->world) return TUNA_ERR_BAD_CONFIG;
    for (int j = 0; j < ex->world; ++j) {
        if (!ex->buffer[j]) return TUNA_ERR_NULL_POINTER;
        if (!aligned(ex->buffer[j], 256)) return TUNA_ERR_MISALIGNED;
    }
    if (!aligned(code, 4) || !aligned(workspace, 16)) return TUNA_ERR_MISALIGNED;
    // every rank must run the same launches: no entry is skipped here, so n = 0 is refused
    for (int i = 0; i < count; ++i) {
        const tuna_gemm_desc &d = g[i];
        if (!d.q || !d.x || !d.absmax || !d.o) return TUNA_ERR_NULL_POINTER;
        const int st = check_shape(d.m, d.n, d.k);
        if (st != TUNA_OK) return st;
        if (d.n > 64) return TUNA_ERR_TOO_LARGE;
        if (!aligned(d.q, 16) || !aligned(d.x, 16) || !aligned(d.o, 16) || !aligned(d.absmax, 4)) return TUNA_ERR_MISALIGNED;
    }
    if (ex->bytes < tuna_exchange_bytes(g, count, ex->world)) return TUNA_ERR_WORKSPACE;
    return launch_gemm_tstream_sequence(g, count, (const float *)code, workspace, workspace_bytes, device_sm_count(),
                                        (cudaStream_t)stream, ex);
}

extern "C" int tuna_matmul(const void *q, const void *x, const void *code, const void *absmax, void *o,
                           int m, int n, int k, void *workspace, size_t workspace_bytes, void *stream)
{
    return tuna_matmul_cfg(q, x, code, absmax, o, m, n, k, workspace, workspace_bytes, stream, nullptr);
}

extern "C" size_t tuna_matmul_workspace_bytes(int m, int n, int k)
{
    if (check_shape(m, n, k) != TUNA_OK) return 0;
    const int sms = device_sm_count();
    tuna_config c;
    if (resolve_config(m, n, k, sms, nullptr, &c) != TUNA_OK) return 0;
    return workspace_for(m, n, k, c, sms);
}

extern "C" int tuna_lookup_config(int m, int n, int k, tuna_config *out)
{
    if (!out) return TUNA_ERR_NULL_POINTER;
    int st = check_shape(m, n, k);
    if (st != TUNA_OK) return st;
    return resolve_config(m, n, k, device_sm_count(), nullptr, out);
}

extern "C" int tuna_dequant(const void *q, const void *absmax, const void *code, void *o, int m, int k,
                            void *stream)
{
    if (!q || !absmax || !code || !o) return TUNA_ERR_NULL_POINTER;
    int st = check_shape(m, 1, k);
    if (st != TUNA_OK) return st;
    if (!aligned(q, 16) || !aligned(o, 16) || !aligned(absmax, 4) || !aligned(code, 4)) return TUNA_ERR_MISALIGNED;
    cudaError_t e = launch_dequant(q, absmax, code, o, m, k, device_sm_count(), (cudaStream_t)stream);
    return e == cudaSuccess ? TUNA_OK : TUNA_ERR_LAUNCH;
}

extern "C" int tuna_quantize(const void *w, const void *code, void *q, void *absmax, int m, int k, void *stream)
{
    if (!w || !code || !q || !absmax) return TUNA_ERR_NULL_POINTER;
    int st = check_shape(m, 1, k);
    if (st != TUNA_OK) return st;
    if (!aligned(w, 16) || !aligned(q, 16) || !aligned(absmax, 4) || !aligned(code, 4)) return TUNA_ERR_MISALIGNED;
    cudaError_t e = launch_quantize(w, code, q, absmax, m, k, device_sm_count(), (cudaStream_t)stream);
    return e == cudaSuccess ? TUNA_OK : TUNA_ERR_LAUNCH;
}

extern "C" int tuna_check_device_status(void *stream) { return read_device_status((cudaStream_t)stream); }

extern "C" const char *tuna_status_string(int s)
{
    switch (s) {
        case TUNA_OK: return "ok";
        case TUNA_ERR_NULL_POINTER: return "null pointer";
        case TUNA_ERR_BAD_SHAPE: return "bad shape: m and k must be positive multiples of 8, n >= 1";
        case TUNA_ERR_MISALIGNED: return "misaligned pointer";
        case TUNA_ERR_WORKSPACE: return "workspace missing or too small";
        case TUNA_ERR_BAD_CONFIG: return "inconsistent launch configuration";
        case TUNA_ERR_LAUNCH: return "CUDA launch failed";
        case TUNA_ERR_NO_DEVICE: return "no usable sm_100 device";
        case TUNA_ERR_DEVICE_TIMEOUT: return "a bounded in-kernel wait ran out";
        case TUNA_ERR_TOO_LARGE: return "size beyond a documented limit";
        default: return "unknown status";
    }
}

extern "C" int tuna_abi_version(void) { return 1; }
extern "C" int tuna_config_table_size(void) { return tuna::kTableSize; }
